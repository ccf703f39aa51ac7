"""CPU: the `experts.layout` text parser (bsx_layout_parse, basalt_b200/layout_file.py) accepts and refuses what the
reference's expert_layout_load_text does - against tests/golden/layout_tables.json, which holds the reference parser's own
verdicts and fields (the real models' tables of its test data, the cases of its tests/core/expert_layout_test.cpp:83-137, a
sweep over every type triple), and against the compiled reference itself on mutated texts when oracle/_ref is built - and
the section reader finds each blob where the table puts it."""
import json
import random
from pathlib import Path

import numpy as np
import pytest

GOLDEN = json.loads((Path(__file__).parent / "golden" / "layout_tables.json").read_text())


def fields(t):
    return [t.version, t.n_expert, t.max_blob, t.total, t.n_layers], [[r.gu_type, r.d_type, r.up_type, r.offset, r.blob_bytes] for r in t.rows]


@pytest.mark.parametrize("case", GOLDEN["cases"], ids=[c["name"] for c in GOLDEN["cases"]])
def test_golden_case_parses_as_the_reference_parser_did(lib, case):
    args = (case["text"], case["n_layers"], case["n_expert"], case["n_embd"], case["n_ff"])
    if not case["ok"]:
        with pytest.raises(ValueError):
            lf.parse_layout_text(*args)
        return
    head, rows = fields(lf.parse_layout_text(*args))
    assert head == case["head"]
    assert rows == [r[:5] for r in case["rows"]]


def test_golden_type_sweep(lib):
    """Every (gate, down, up) triple at three geometries: accepted or refused as the reference's loader did, and the up rows'
    type and offset as it placed them."""
    n_ok = 0
    for h, i, gt, dt, ut, blob, ok, up_type, up_off in GOLDEN["sweep"]:
        text = "# experts v7: x (n_expert 1, total %d)\n0 %d %d 0 %d %d\n" % (blob, gt, dt, blob, ut)
        try:
            t = lf.parse_layout_text(text, 1, 1, h, i)
        except ValueError:
            assert not ok, (h, i, gt, dt, ut)
            continue
        assert ok, (h, i, gt, dt, ut)
        n_ok += 1
        assert t.rows[0].up_type == up_type
        if t.rows[0].kernels:
            assert t.layout(0).up_off == up_off and t.layout(0).bytes == blob
    assert n_ok == sum(r[6] for r in GOLDEN["sweep"]) > 500


def test_mutated_texts_against_the_compiled_reference(lib):
    from oracle import oracle as O
    if O.ref_cpu() is None or not hasattr(O.ref_cpu(), "ref_layout_load_text"):
        pytest.skip("oracle/_ref is not built here")
    rnd = random.Random(7)
    base = [c for c in GOLDEN["cases"] if c["ok"]]
    accepted = 0
    for _ in range(1500):
        c = rnd.choice(base)
        t = c["text"]
        pos = rnd.randrange(len(t))
        kind = rnd.randrange(5)
        if kind == 0:
            t = t[:pos] + rnd.choice("0123456789 -+#\n\t x") + t[pos + 1:]
        elif kind == 1:
            t = t[:pos] + t[pos + 1:]
        elif kind == 2:
            t = t[:pos] + rnd.choice("0123456789 \n") + t[pos:]
        elif kind == 3:
            lines = t.split("\n")
            del lines[rnd.randrange(len(lines))]
            t = "\n".join(lines)
        else:
            t = t.replace("v5", "v" + str(rnd.randrange(10)), 1)
        ok, head, rows = O.ref_layout_load_text(t.encode(), c["n_layers"], c["n_expert"], c["n_embd"], c["n_ff"])
        try:
            mine = lf.parse_layout_text(t, c["n_layers"], c["n_expert"], c["n_embd"], c["n_ff"])
        except ValueError:
            assert not ok, t
            continue
        assert ok, t
        accepted += 1
        assert fields(mine) == (head, [r[:5] for r in rows]), t
    assert accepted > 200

from basalt_b200 import layout_file as lf

Q6_K, IQ1_M, NVFP4 = 14, 29, 40
H, I = 2560, 768          # n_embd % 256 == 0, n_ff % 256 == 0


def blob_bytes(gt, dt, ut=-1):
    t = lf.parse_layout_text(lf.layout_text([(gt, dt, ut)], 1, H, I), 1, 1, H, I)
    return t.blob_bytes(0)


def layout(version, blob, extra="", n_expert=2, types="14 14"):
    s = f"# experts v{version}: layer gu_type d_type offset blob_bytes (n_expert {n_expert}, total {2 * blob * n_expert})\n"
    s += f"0 {types} 0 {blob}{extra}\n"
    s += f"1 {types} {blob * n_expert} {blob}{extra}\n"
    return s


def load(text, n_layers=2, n_expert=512):
    return lf.parse_layout_text(text, n_layers, n_expert, H, I)


def test_blob_sizes_follow_the_formats():
    assert blob_bytes(Q6_K, Q6_K) == 3 * I * H // 256 * 210
    assert blob_bytes(IQ1_M, IQ1_M) == 3 * I * H // 256 * 56
    # NVFP4: the blob carries a 16-byte fp32 scale tail after down, counted in the blob size
    assert blob_bytes(NVFP4, NVFP4) == 2 * I * (H // 64 * 36) + H * (I // 64 * 36) + 16
    assert blob_bytes(IQ1_M, Q6_K) == 2 * I * H // 256 * 56 + H * I // 256 * 210


def test_versions_and_columns():
    b = blob_bytes(Q6_K, Q6_K)
    t = load(layout(5, b))
    assert (t.version, t.n_expert, t.total, t.max_blob) == (5, 2, 4 * b, b)      # the header's expert count wins
    assert [(r.offset, r.blob_bytes, r.gu_type, r.d_type, r.up_type) for r in t.rows] == [(0, b, 14, 14, 14), (2 * b, b, 14, 14, 14)]
    assert t.blob_offset(1, 1) == 3 * b
    load(layout(3, b, " 100 200 300 shard.gguf"))                                  # columns past the fifth are ignored
    with pytest.raises(ValueError, match="v8"):
        load(layout(8, b))
    nv = blob_bytes(NVFP4, NVFP4)
    assert load(layout(6, nv, types="40 40")).rows[1].gu_type == NVFP4
    with pytest.raises(ValueError, match="formats make"):
        load(layout(6, nv - 16, types="40 40"))                                    # an NVFP4 blob without its tail
    no_header = "0 14 14 0 %d\n1 14 14 %d %d\n" % (b, 512 * b, b)
    t = load(no_header)
    assert (t.version, t.n_expert, t.total) == (0, 512, 1024 * b)                 # no header: the caller's count stands


def test_refusals():
    b = blob_bytes(Q6_K, Q6_K)
    with pytest.raises(ValueError, match="empty"):
        load("")
    good = layout(5, b)
    with pytest.raises(ValueError, match="missing or not contiguous"):
        load(good[:good.rfind("1 14 14")])
    with pytest.raises(ValueError, match="formats make"):
        load(layout(5, b + 8))
    with pytest.raises(ValueError, match="malformed"):
        load("# experts v5: x\n0 14 seven 0 1\n", n_layers=1)
    with pytest.raises(ValueError, match="malformed"):
        load("# experts v5: x\n5 14 14 0 %d\n" % b, n_layers=1)                    # a layer id past the model's layers
    with pytest.raises(ValueError, match="come together"):
        load(layout(6, b, types="40 14"))                                          # NVFP4's scale tail covers all three matrices
    with pytest.raises(ValueError, match="no dot product"):
        load(layout(5, b, types="9 14"))                                           # Q8_1 is an activation format, not a weight's
    # every format the table knows has kernels: the low-bit ones too
    q23 = 2 * I * (H // 256 * 84) + H * (I // 256 * 110)                           # Q2_K gate/up, Q3_K down
    t = load(layout(5, q23, types="10 11"))
    assert t.rows[0].kernels and load(layout(5, b)).rows[0].kernels
    assert t.layout(0).bytes == q23


def test_v7_up_type_column():
    mixed = blob_bytes(IQ1_M, Q6_K, Q6_K)
    assert mixed == I * (H // 256 * 56) + I * (H // 256 * 210) + H * (I // 256 * 210)
    t = load(layout(7, mixed, " 14", types="29 14"))
    assert t.rows[1].up_type == Q6_K and t.total == 4 * mixed
    L = t.layout(1)
    assert (L.up_off, L.down_off, L.bytes) == (I * (H // 256 * 56), I * (H // 256 * 56) + I * (H // 256 * 210), mixed)
    uniform = blob_bytes(IQ1_M, Q6_K)
    assert load(layout(7, uniform, " 29", types="29 14")).rows[0].up_type == IQ1_M
    with pytest.raises(ValueError, match="malformed"):
        load(layout(7, mixed, "", types="29 14"))                                  # a v7 line without its up type
    with pytest.raises(ValueError, match="formats make"):
        load(layout(5, mixed, " 14", types="29 14"))                               # a v5 layout never reads a sixth column


def test_writer_and_reader_agree():
    layers = [(NVFP4, NVFP4, -1), (IQ1_M, Q6_K, -1), (Q6_K, Q6_K, -1)]
    for v in (6, 7):
        text = lf.layout_text(layers, 8, H, I, version=v)
        t = lf.parse_layout_text(text, 3, 999, H, I)
        assert t.version == v and t.n_expert == 8
        assert [r.blob_bytes for r in t.rows] == [blob_bytes(*x) for x in layers]
        assert t.total == 8 * sum(r.blob_bytes for r in t.rows)
        assert str(t.total) in text.splitlines()[0]


def test_section_reader_finds_each_blob(tmp_path):
    h, i, E = 256, 256, 3
    layers = [(NVFP4, NVFP4, -1), (Q6_K, Q6_K, -1)]
    t = lf.parse_layout_text(lf.layout_text(layers, E, h, i), 2, E, h, i)
    rng = np.random.default_rng(0)
    raw = rng.integers(0, 256, size=64 + t.total, dtype=np.uint8)
    path = tmp_path / "model.bin"
    raw.tofile(path)
    for src in (str(path), raw):
        sec = lf.ExpertsSection(src, t, base_offset=64)
        for l in range(2):
            for e in range(E):
                o = 64 + t.rows[l].offset + e * t.rows[l].blob_bytes
                assert np.array_equal(sec.blob(l, e), raw[o:o + t.rows[l].blob_bytes])
    with pytest.raises(ValueError, match="needs"):
        lf.ExpertsSection(raw[:100], t)
    with pytest.raises(IndexError):
        sec.blob(0, E)
