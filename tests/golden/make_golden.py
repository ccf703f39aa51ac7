"""Generates tests/golden/ref_vectors.npz from the reference engine's own code (oracle/_ref/libref_cpu.so, built from a
reference checkout by oracle/Makefile).  Run in a container that has the reference; the .npz travels with the repository
so the CPU tests can pin the oracle where the reference is absent.

Contents: raw blocks of each format (NVFP4, Q6_K, IQ1_M, Q8_0, Q4_K, Q5_K, Q5_0, Q5_1, IQ4_NL, IQ4_XS, Q2_0, Q2_K, Q3_K, IQ2_XXS, IQ2_XS,
IQ2_S, IQ3_XXS, IQ3_S, IQ1_S) with the reference's to_float output; seeded fp32 rows with the reference quantiser's
bytes (NVFP4, Q6_K); the reference's blob geometry for the benchmark shapes; and the reference CPU expert pool's output
rows for a small Q6_K and a small NVFP4 layer (inputs are regenerated from the seeds stored alongside).
"""
import ctypes as C
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle import oracle as O   # noqa: E402
from tests.helpers import make_expert_blobs   # noqa: E402


def main():
    R = O.ref_cpu()
    assert R is not None, "build oracle/_ref first (make -C oracle ref_cpu)"
    out = {}
    rng = np.random.default_rng(2024)
    # decoders: random blocks (finite super-scales) and the reference's floats
    for name, t, bs, nv, nblk in (("nvfp4", 40, 36, 64, 8), ("q6k", 14, 210, 256, 3), ("iq1m", 29, 56, 256, 3)):
        raw = rng.integers(0, 256, size=nblk * bs, dtype=np.uint8)
        if t == 14:
            raw.reshape(-1, 210)[:, 209] &= 0x7B
        if t == 29:
            raw = O.random_iq1m_rows(rng, 1, nblk * 256)
        y = np.empty(nblk * nv, np.float32)
        assert R.ref_dequantize(t, raw.ctypes.data, y, y.size) == 0
        out[f"dec_{name}_raw"], out[f"dec_{name}_f32"] = raw, y
    # quantisers
    for name, t in (("nvfp4", 40), ("q6k", 14)):
        w = (rng.standard_normal((2, 512)) * 0.02).astype(np.float32)
        if t == 40:
            w = (w / (np.abs(w).max() / (6 * 448))).astype(np.float32)
        w[0, :16] = 0
        q = np.zeros(2 * O.row_bytes(t, 512), np.uint8)
        assert R.ref_quantize(t, w, q, 2, 512) == q.size
        out[f"quant_{name}_in"], out[f"quant_{name}_out"] = w, q
    # geometry
    geo = []
    for cfg in ((14, 14, 2048, 512), (40, 40, 2048, 512), (29, 29, 5120, 2304), (40, 40, 2560, 640), (29, 14, 2048, 512)):
        o = (C.c_int64 * 7)()
        err = C.create_string_buffer(256)
        rc = R.ref_native_fmt(*cfg, 0.0, o, err, 256)
        geo.append(list(cfg) + ([int(v) for v in o][:6] if rc == 0 else [-1] * 6))
    out["geometry"] = np.array(geo, np.int64)
    # the reference's CPU expert pool on a small layer (rows in expert-sorted order)
    pool = R.ref_pool_create(3)
    for name, gt, dt in (("q6k", 14, 14), ("nvfp4", 40, 40)):
        H, I, E, T, k = 512, 256, 4, 6, 2
        r2 = np.random.default_rng(7)
        L, blobs = make_expert_blobs(r2, E, gt, dt, H, I)
        x = r2.standard_normal((T, H)).astype(np.float32)
        ids = np.stack([r2.permutation(E)[:k] for _ in range(T)]).astype(np.int32)
        cnt, off, slot, src, _ = O.dispatch(ids, k, E)
        ptrs = (C.c_void_p * E)(*[b.ctypes.data for b in blobs])
        rows = np.zeros((T * k, H), np.float32)
        assert R.ref_pool_layer(pool, gt, dt, H, I, 0.0, ptrs, E, off, src, x, T, rows) == 0
        out[f"pool_{name}_x"], out[f"pool_{name}_ids"], out[f"pool_{name}_rows"] = x, ids, rows
        out[f"pool_{name}_blobhash"] = np.array([O.fnv1a(*blobs)], np.uint64)
    R.ref_pool_destroy(pool)
    # decoders of the formats added later (their own generator, so the vectors above keep their bytes)
    rng2 = np.random.default_rng(2025)
    for name, t, nv, nblk in (("q8_0", 8, 32, 16), ("q4k", 12, 256, 3), ("q5k", 13, 256, 3), ("q5_0", 6, 32, 16), ("q5_1", 7, 32, 16),
                              ("iq4nl", 20, 32, 16), ("iq4xs", 23, 256, 3)):
        raw = O.random_rows(t, rng2, 1, nblk * nv)
        y = np.empty(nblk * nv, np.float32)
        assert R.ref_dequantize(t, raw.ctypes.data, y, y.size) == 0
        out[f"dec_{name}_raw"], out[f"dec_{name}_f32"] = raw, y
    # the low-bit formats (again their own generator)
    rng3 = np.random.default_rng(2026)
    for name, t, nv, nblk in (("q2_0", 42, 64, 8), ("q2k", 10, 256, 3), ("q3k", 11, 256, 3), ("iq2xxs", 16, 256, 3), ("iq2xs", 17, 256, 3),
                              ("iq2s", 22, 256, 3), ("iq3xxs", 18, 256, 3), ("iq3s", 21, 256, 3), ("iq1s", 19, 256, 3)):
        raw = O.random_rows(t, rng3, 1, nblk * nv)
        y = np.empty(nblk * nv, np.float32)
        assert R.ref_dequantize(t, raw.ctypes.data, y, y.size) == 0
        out[f"dec_{name}_raw"], out[f"dec_{name}_f32"] = raw, y
    np.savez_compressed(Path(__file__).with_name("ref_vectors.npz"), **out)
    print("wrote ref_vectors.npz:", {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
