"""Writes tests/golden/layout_tables.json: `experts.layout` texts with what the REFERENCE's own parser makes of them
(expert_layout_load_text compiled from the reference checkout into oracle/_ref/libref_cpu.so; run `make -C oracle` first).

Cases: the layouts of real models the reference ships as test data (tests/data/native_experts/*.txt, read from the reference
checkout given as argv[1]; 48 layers, n_embd 2560, n_ff 640, as tests/core/expert_layout_test.cpp:27-30,41-47 loads them), the
accept / refuse cases of that test (:83-137), and a sweep of every (gate, down, up) type triple at two geometries.

    python tests/golden/make_layout_golden.py <reference checkout>
"""
import json
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent.parent
sys.path.insert(0, str(ROOT))
from oracle import oracle as O  # noqa: E402

TYPES = [6, 7, 8, 9, 10, 11, 12, 13, 14, 15, 16, 17, 18, 19, 20, 21, 22, 23, 29, 30, 40, 41, 42]


def row(t, n):
    return int(O.ref_cpu().ref_row_bytes(t, n))


def blob(gt, dt, ut, H, I):
    ut = gt if ut < 0 else ut
    return I * (row(gt, H) + row(ut, H)) + H * row(dt, I) + (16 if gt == 40 else 0)


def case(name, text, n_layers, n_expert, H, I):
    ok, a, b = O.ref_layout_load_text(text.encode(), n_layers, n_expert, H, I)
    c = {"name": name, "text": text, "n_layers": n_layers, "n_expert": n_expert, "n_embd": H, "n_ff": I, "ok": bool(ok)}
    if ok:
        c["head"], c["rows"] = a, b
    else:
        c["err"] = a
    return c


def two(version, b, extra="", n_expert=2, types="12 7"):
    s = f"# experts v{version}: layer gu_type d_type offset blob_bytes (n_expert {n_expert}, total {2 * b * n_expert})\n"
    return s + f"0 {types} 0 {b}{extra}\n1 {types} {b * n_expert} {b}{extra}\n"


def main():
    ref = Path(sys.argv[1])
    cases = []
    for f in sorted((ref / "tests" / "data" / "native_experts").glob("*.txt")):
        cases.append(case("real:" + f.stem, f.read_text(), 48, 512, 2560, 640))
    H, I = 2560, 640
    b = blob(12, 7, -1, H, I)
    nv = blob(40, 40, -1, H, I)
    mx = blob(22, 42, 16, H, I)
    un = blob(22, 42, -1, H, I)
    good = two(5, b)
    for name, text, nl in [
        ("v5", good, 2), ("v3 extra columns", two(3, b, " 100 200 300 shard.gguf"), 2), ("v8 refused", two(8, b), 2),
        ("v6 nvfp4", two(6, nv, types="40 40"), 2), ("nvfp4 without tail", two(6, nv - 16, types="40 40"), 2),
        ("empty", "", 2), ("missing layer", good[:good.rfind("1 12 7")], 2), ("size mismatch", two(5, b + 8), 2),
        ("malformed", "# experts v5: x\n0 12 seven 0 1\n", 1), ("layer id past the end", "# experts v5: x\n3 12 7 0 %d\n" % b, 1),
        ("v7 mixed", two(7, mx, " 16", types="22 42"), 2), ("v7 uniform", two(7, un, " 22", types="22 42"), 2),
        ("v7 without up", two(7, mx, "", types="22 42"), 2), ("v5 never reads a sixth column", two(5, mx, " 16", types="22 42"), 2),
        ("no header", "0 12 7 0 %d\n1 12 7 %d %d\n" % (b, 512 * b, b), 2),
        ("blank lines, comments, CRLF", "# a comment\n\n" + good.replace("\n", "\r\n") + "\n# end\n", 2),
        ("negative offset", "# experts v5: x\n0 12 7 -0 %d\n" % b, 1), ("plus signs", "# experts v5: x\n+0 +12 +7 +0 +%d\n" % b, 1),
        ("layers out of order", "\n".join(reversed(good.strip().split("\n")[1:])) + "\n", 2),
        ("header after the rows", "0 12 7 0 %d 16\n# experts v7: x (n_expert 3, total 0)\n" % b, 1),
    ]:
        cases.append(case(name, text, nl, 512, H, I))
    sweep = []
    for (h, i) in ((2560, 640), (2048, 512), (2560, 608)):
        for gt in TYPES:
            for dt in TYPES:
                for ut in [-1] + ([6, 8, 14, 16, 20, 40, 42] if gt in (8, 22, 40, 42) else []):
                    bb = blob(gt, dt, ut, h, i)
                    text = "# experts v7: x (n_expert 1, total %d)\n0 %d %d 0 %d %d\n" % (bb, gt, dt, bb, ut)
                    ok, a, r = O.ref_layout_load_text(text.encode(), 1, 1, h, i)
                    sweep.append([h, i, gt, dt, ut, bb, int(ok), (r[0][2] if ok else -1), (r[0][5] if ok else -1)])
    out = Path(__file__).with_name("layout_tables.json")
    out.write_text(json.dumps({"cases": cases, "sweep": sweep,
                               "sweep_columns": ["n_embd", "n_ff", "gu_type", "d_type", "up_type column", "blob_bytes", "accepted",
                                                 "up_type", "up_off"]}, indent=None, separators=(",", ":")))
    print(len(cases), "cases,", len(sweep), "sweep rows,", sum(s[6] for s in sweep), "accepted ->", out, out.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
