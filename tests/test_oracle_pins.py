"""CPU: pins the oracle (oracle/moe_oracle.c) against golden vectors generated from the reference's own code
(tests/golden/ref_vectors.npz, made by tests/golden/make_golden.py) and, where oracle/_ref was built, against the reference
live; and checks the oracle's router / dispatch / combine restatements against independent numpy definitions."""
import ctypes as C
from pathlib import Path

import numpy as np
import pytest

from oracle import oracle as O
from tests.helpers import make_expert_blobs, rel_l2

G = np.load(Path(__file__).parent / "golden" / "ref_vectors.npz")


@pytest.mark.parametrize("name,t,nv", [("nvfp4", 40, 64), ("q6k", 14, 256), ("iq1m", 29, 256), ("q8_0", 8, 32), ("q4k", 12, 256), ("q5k", 13, 256), ("q5_0", 6, 32), ("q5_1", 7, 32), ("iq4nl", 20, 32), ("iq4xs", 23, 256), ("q2_0", 42, 64), ("q2k", 10, 256), ("q3k", 11, 256), ("iq2xxs", 16, 256), ("iq2xs", 17, 256),
                                    ("iq2s", 22, 256), ("iq3xxs", 18, 256), ("iq3s", 21, 256), ("iq1s", 19, 256)])
def test_decoders_match_reference_golden(name, t, nv):
    raw, want = G[f"dec_{name}_raw"], G[f"dec_{name}_f32"]
    got = O.dequantize(t, raw, 1, want.size).reshape(-1)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("name,t", [("nvfp4", 40), ("q6k", 14)])
def test_quantisers_match_reference_golden(name, t):
    assert np.array_equal(O.quantize(t, G[f"quant_{name}_in"]), G[f"quant_{name}_out"])


def test_blob_geometry_matches_reference():
    for row in G["geometry"]:
        gt, dt, H, I, gu_row, d_row, up_off, down_off, nbytes, tail = [int(v) for v in row]
        if gt != dt:
            continue   # oracle.Layout describes same-type gate/up + any down: covered below through the C ABI test
        L = O.Layout(gt, dt, H, I)
        assert (L.gu_row, L.d_row, L.up_off, L.down_off, L.bytes, L.tail) == (gu_row, d_row, up_off, down_off, nbytes, tail)


@pytest.mark.parametrize("name,gt,dt", [("q6k", 14, 14), ("nvfp4", 40, 40)])
def test_dequantised_expert_vs_reference_cpu_pool(name, gt, dt):
    """The reference's CPU offload path rounds activations to int8 (Q8_K / Q8_0); its rows must sit within the
    reference's own tolerance (relative L1 < 3e-2, tests/kernels/native_expert_parity.cpp:372-373) of the dequantised fp32
    expert that is this build's parity bar."""
    H, I, E, T, k = 512, 256, 4, 6, 2
    r2 = np.random.default_rng(7)
    L, blobs = make_expert_blobs(r2, E, gt, dt, H, I)
    assert O.fnv1a(*blobs) == int(G[f"pool_{name}_blobhash"][0]), "seeded blobs differ from the ones the golden run used"
    x, ids, want = G[f"pool_{name}_x"], G[f"pool_{name}_ids"], G[f"pool_{name}_rows"]
    cnt, off, slot, src, _ = O.dispatch(ids, k, E)
    rows = np.zeros_like(want)
    for e in range(E):
        if cnt[e]:
            rows[off[e]:off[e + 1]] = O.expert_forward(L, blobs[e], x[src[off[e]:off[e + 1]]])
    l1 = np.abs(rows - want).sum() / np.abs(want).sum()
    assert l1 < 3e-2, l1
    f64 = np.zeros_like(want)
    for e in range(E):
        if cnt[e]:
            f64[off[e]:off[e + 1]] = O.expert_forward(L, blobs[e], x[src[off[e]:off[e + 1]]], dtype=np.float64)
    assert rel_l2(rows, f64) < 1e-5


@pytest.mark.skipif(O.ref_cpu() is None, reason="oracle/_ref/libref_cpu.so not built (no reference checkout)")
def test_formats_live_against_reference():
    R = O.ref_cpu()
    rng = np.random.default_rng(11)
    for t in (40, 14):
        w = (rng.standard_normal((8, 1024)) * 0.02).astype(np.float32)
        if t == 40:
            w = (w / (np.abs(w).max() / (6 * 448))).astype(np.float32)
        ref = np.zeros(8 * O.row_bytes(t, 1024), np.uint8)
        assert R.ref_quantize(t, w, ref, 8, 1024) == ref.size
        assert np.array_equal(O.quantize(t, w), ref)
    for t, bs in ((40, 36), (14, 210), (29, 56)):
        raw = rng.integers(0, 256, size=64 * bs, dtype=np.uint8)
        if t == 14:
            raw.reshape(-1, 210)[:, 209] &= 0x7B
        if t == 29:
            raw = O.random_iq1m_rows(rng, 1, 64 * 256)
        n = raw.size // bs * (64 if t == 40 else 256)
        want = np.empty(n, np.float32)
        R.ref_dequantize(t, raw.ctypes.data, want, n)
        assert np.array_equal(O.dequantize(t, raw, 1, n).reshape(-1).view(np.uint32), want.view(np.uint32))


def test_router_logits_close_to_double():
    rng = np.random.default_rng(3)
    x = rng.standard_normal((5, 2048)).astype(np.float32)
    g = (rng.standard_normal((64, 2048)) * 0.02).astype(np.float32)
    lg = O.router_logits(x, g)
    assert np.abs(lg - x.astype(np.float64) @ g.astype(np.float64).T).max() < 1e-5


def _select_numpy(logits, bias, k, kind, scale):
    """double-precision restatement with a stable sort (src/models/deepseek41/kernels/router_parity.cpp:26-47)"""
    lg = logits.astype(np.float64)
    s = np.sqrt(np.log1p(np.exp(lg))) if kind == 0 else 1 / (1 + np.exp(-lg))
    b = s + bias
    ids = np.argsort(-b, axis=1, kind="stable")[:, :k]
    sel = np.take_along_axis(s, ids, 1)
    return ids, sel / (sel.sum(1, keepdims=True) + 1e-20) * scale


@pytest.mark.parametrize("kind", [0, 1])
def test_router_select_vs_double(kind):
    rng = np.random.default_rng(4)
    lg = rng.standard_normal((32, 384)).astype(np.float32)
    bias = (rng.standard_normal(384) * 0.05).astype(np.float32)
    ids, w = O.router_select(lg, bias, 6, kind, 1.5)
    rid, rw = _select_numpy(lg, bias, 6, kind, 1.5)
    assert np.array_equal(ids, rid)
    assert np.abs(w - rw).max() < 1e-5


def test_router_select_ties_to_lower_index_and_groups():
    lg = np.zeros((1, 64), np.float32)
    bias = np.zeros(64, np.float32)
    ids, w = O.router_select(lg, bias, 4, 1, 1.0)
    assert ids.tolist() == [[0, 1, 2, 3]]
    assert np.allclose(w, 0.25)
    # groups: 4 groups of 16, keep 2; the winners must come from the two best groups by top-2 sum
    rng = np.random.default_rng(5)
    lg = rng.standard_normal((16, 64)).astype(np.float32)
    ids, w = O.router_select(lg, bias, 4, 1, 2.5, n_group=4, topk_group=2)
    s = 1 / (1 + np.exp(-lg.astype(np.float64)))
    for t in range(16):
        gsc = np.sort(s[t].reshape(4, 16), axis=1)[:, -2:].sum(1)
        keep = set(np.argsort(-gsc, kind="stable")[:2].tolist())
        assert set((ids[t] // 16).tolist()) <= keep
        live = np.isin(np.arange(64) // 16, list(keep))
        want = np.argsort(-np.where(live, s[t], -np.inf), kind="stable")[:4]
        assert ids[t].tolist() == want.tolist()
    # n_group = 1 is the plain selection bit for bit
    a = O.router_select(lg, bias, 4, 1, 2.5)
    b = O.router_select(lg, bias, 4, 1, 2.5, n_group=1, topk_group=1)
    assert np.array_equal(a[0], b[0]) and np.array_equal(a[1].view(np.uint32), b[1].view(np.uint32))


def test_router_softmax_forms():
    rng = np.random.default_rng(6)
    lg = (rng.standard_normal((16, 512)) * 2).astype(np.float32)
    ids, w = O.router_select(lg, None, 10, O.GATE_SOFTMAX)
    ids64, w64 = O.router_top10(lg, 10)
    assert np.array_equal(ids, ids64)
    assert np.abs(w - w64).max() < 1e-5
    assert np.allclose(w.sum(1), 1, atol=1e-5)
    # all-equal logits: lowest indices win (tests/models/qwen4exp/kernels/router_top10_parity.cpp:125-140)
    ids, w = O.router_select(np.zeros((1, 256), np.float32), None, 10, O.GATE_SOFTMAX)
    assert ids.tolist() == [list(range(10))]


def test_dispatch_and_plan_against_numpy():
    rng = np.random.default_rng(8)
    E, k, T = 64, 8, 37
    ids = np.stack([rng.permutation(E)[:k] for _ in range(T)]).astype(np.int32)
    ids[3, 2] = -1
    cnt, off, slot, src, tiles = O.dispatch(ids, k, E, tile_rows=4)
    flat = ids.reshape(-1)
    valid = flat >= 0
    assert np.array_equal(cnt, np.bincount(flat[valid], minlength=E))
    assert np.array_equal(off, np.concatenate([[0], np.cumsum(cnt)]))
    order = np.argsort(np.where(valid, flat, E), kind="stable")[:valid.sum()]   # stable counting sort
    assert np.array_equal(src[:valid.sum()], order // k)
    assert np.array_equal(slot[order], np.arange(valid.sum()))
    assert slot[3 * k + 2] == -1
    want_tiles = [(e, off[e] + r) for e in range(E) for r in range(0, cnt[e], 4)]
    assert tiles.tolist() == [list(t) for t in want_tiles]
    blobs = (np.arange(E, dtype=np.uint64) + 1) * 4096
    blobs[5] = 0
    ptr, start, ng, dst, tok = O.moe_plan(ids, k, E, blobs)
    used = [e for e in range(E) if blobs[e] and (flat == e).any()]
    assert ng == len(used)
    assert ptr[:ng].tolist() == [int(blobs[e]) for e in used]
    at = 0
    for g, e in enumerate(used):
        pairs = np.nonzero(flat == e)[0]
        assert start[g] == at
        assert dst[at:at + len(pairs)].tolist() == pairs.tolist()
        assert tok[at:at + len(pairs)].tolist() == (pairs // k).tolist()
        at += len(pairs)
    assert start[ng] == at and start[ng + 1] == at


def test_tail_skip_rule():
    ids = np.array([[1, 2, 3], [2, 4, 5]], np.int32)
    w = np.array([[0.5, 0.3, 0.2], [0.6, 0.3, 0.1]], np.float32)
    held = np.full(8, -1, np.int32)
    held[[1, 2]] = 0
    nid, nw, counts = O.route_tail_skip(ids, w, held, 3, 2, 8)
    # experts 3 and 5 are unheld and rank 2 (tail) everywhere -> dropped; 4 is unheld but ranks 1 -> kept
    assert nid.tolist() == [[1, 2, -1], [2, 4, -1]]
    assert nw[0, 2] == 0 and nw[1, 2] == 0 and nw[1, 1] == np.float32(0.3)
    assert counts.tolist() == [6, 3, 2]


def test_combine_order():
    rng = np.random.default_rng(9)
    rows = rng.standard_normal((12, 8)).astype(np.float32)
    w = rng.random((3, 4)).astype(np.float32)
    slot = rng.permutation(12).astype(np.int32).reshape(3, 4)
    shared = rng.standard_normal((3, 8)).astype(np.float32)
    y = O.combine(rows, slot, w, shared)
    want = np.zeros((3, 8), np.float32)
    for t in range(3):
        s = np.zeros(8, np.float64)
        for j in range(4):
            s = np.float32(np.float64(w[t, j]) * rows[slot[t, j]].astype(np.float64) + s.astype(np.float64)).astype(np.float32)
        want[t] = s + shared[t]
    assert np.array_equal(y.view(np.uint32), want.view(np.uint32))


def test_q8_1_blocks():
    rng = np.random.default_rng(10)
    x = rng.standard_normal(64).astype(np.float32)
    y = O.quantize_q8_1(x).reshape(2, 36)
    for b in range(2):
        d = y[b, :2].view(np.float16)[0]
        q = y[b, 4:].view(np.int8)
        assert abs(float(d) - np.abs(x[32 * b:32 * b + 32]).max() / 127) < 1e-3
        assert np.abs(q * np.float32(d) - x[32 * b:32 * b + 32]).max() <= float(d) * 0.51 + 1e-3
