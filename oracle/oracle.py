"""TEST INFRASTRUCTURE, NOT PRODUCT: ctypes bindings of the CPU oracle (liboracle.so, built from moe_oracle.c) and, when
they have been built from a checkout of the reference engine, of the reference's own code for the path
(oracle/_ref/libref_cpu.so, oracle/_ref/libref_gpu.so).  Imported only by tests/, by the smoke check and by bench.py's CPU
baseline legs; the product package never imports it.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
T_Q6_K, T_IQ1_M, T_NVFP4 = 14, 29, 40
T_Q8_0, T_Q4_K, T_Q5_K = 8, 12, 13
T_Q5_0, T_Q5_1, T_IQ4_NL, T_IQ4_XS = 6, 7, 20, 23
T_Q2_K, T_Q3_K, T_IQ2_XXS, T_IQ2_XS, T_IQ3_XXS, T_IQ1_S, T_IQ3_S, T_IQ2_S, T_Q2_0 = 10, 11, 16, 17, 18, 19, 21, 22, 42
LOW_BIT = (T_Q2_K, T_Q3_K, T_IQ2_XXS, T_IQ2_XS, T_IQ3_XXS, T_IQ1_S, T_IQ3_S, T_IQ2_S, T_Q2_0)
UNQUANTISED = (T_IQ1_M, T_Q8_0, T_Q4_K, T_Q5_K, T_Q5_0, T_Q5_1, T_IQ4_NL, T_IQ4_XS) + LOW_BIT   # formats the oracle has no quantiser for
GATE_SQRT_SOFTPLUS, GATE_SIGMOID, GATE_SOFTMAX = 0, 1, 2

_f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
_i32p = np.ctypeslib.ndpointer(np.int32, flags="C_CONTIGUOUS")
_u8p = np.ctypeslib.ndpointer(np.uint8, flags="C_CONTIGUOUS")
_u64p = np.ctypeslib.ndpointer(np.uint64, flags="C_CONTIGUOUS")


def build(force: bool = False) -> None:
    """Compiles liboracle.so (always possible: gcc only) and, if a reference checkout is present, oracle/_ref/*."""
    so = HERE / "liboracle.so"
    src = HERE / "moe_oracle.c"
    if force or not so.exists() or so.stat().st_mtime < src.stat().st_mtime or not (HERE / "libstdrandn.so").exists():
        subprocess.check_call(["make", "-C", str(HERE), "oracle"], stdout=subprocess.DEVNULL)
    ref = reference_checkout()
    if ref.is_dir() and (force or not (HERE / "_ref" / "libref_cpu.so").exists() or not (HERE / "_ref" / "libref_gpu.so").exists()):
        subprocess.check_call(["make", "-C", str(HERE), "-j8", "ref", f"REF={ref}"], stdout=subprocess.DEVNULL)


def reference_checkout() -> Path:
    """Where the reference engine's sources lie: $BASALT_REFERENCE, else a directory named `reference` beside this repository."""
    env = os.environ.get("BASALT_REFERENCE")
    return Path(env) if env else HERE.parent.parent / "reference"


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(str(HERE / "liboracle.so"))
        L.orc_row_bytes.restype = C.c_int64
        L.orc_row_bytes.argtypes = [C.c_int, C.c_int64]
        L.orc_dequant_row.argtypes = [C.c_int, C.c_void_p, _f32p, C.c_int64]
        L.orc_quantize_rows.restype = C.c_int64
        L.orc_quantize_rows.argtypes = [C.c_int, _f32p, _u8p, C.c_int64, C.c_int64]
        L.orc_quantize_q8_1.argtypes = [_f32p, C.c_int64, _u8p]
        L.orc_router_logits.argtypes = [_f32p, _f32p, C.c_int, C.c_int, C.c_int, _f32p]
        L.orc_router_select.argtypes = [_f32p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float, C.c_int, C.c_int,
                                        C.c_float, C.c_void_p, _i32p, _f32p]
        L.orc_router_select_scores.argtypes = [_f32p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_float, C.c_int, C.c_int, C.c_float,
                                               C.c_void_p, _i32p, _f32p]
        L.orc_router_softmax.argtypes = [_f32p, C.c_int, C.c_int, C.c_int, C.c_int, _i32p, _f32p]
        L.orc_router_top10.argtypes = [_f32p, C.c_int, C.c_int, C.c_int, _i32p, _f32p]
        L.orc_route_tail_skip.argtypes = [_i32p, _f32p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]
        L.orc_dispatch.restype = C.c_int
        L.orc_dispatch.argtypes = [_i32p, C.c_int64, C.c_int, C.c_int, _i32p, _i32p, _i32p, _i32p, C.c_int, C.c_void_p]
        L.orc_moe_plan.argtypes = [_i32p, C.c_int, C.c_int, C.c_int, _u64p, _u64p, _i32p, _i32p, _i32p, _i32p]
        L.orc_combine.argtypes = [_f32p, C.c_void_p, _f32p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, _f32p]
        L.orc_expert_dense.argtypes = [_f32p, _f32p, _f32p, _f32p, _f32p, C.c_int, C.c_int, C.c_int, C.c_float, C.c_int, _f32p]
        L.orc_fnv1a.restype = C.c_uint64
        L.orc_fnv1a.argtypes = [C.c_uint64, C.c_void_p, C.c_size_t]
        L.orc_ue4m3_half.restype = C.c_float
        L.orc_ue4m3_half.argtypes = [C.c_uint8]
        _lib = L
    return _lib


def std_randn(n: int, seed: int, sigma: float = 1.0, mean: float = 0.0) -> np.ndarray:
    """n floats from std::mt19937(seed) + std::normal_distribution<float>(mean, sigma) (libstdc++), the generator of the
    reference's own tests."""
    build()
    L = C.CDLL(str(HERE / "libstdrandn.so"))
    L.std_randn.argtypes = [_f32p, C.c_size_t, C.c_uint32, C.c_float, C.c_float]
    out = np.empty(n, np.float32)
    L.std_randn(out, n, seed, sigma, mean)
    return out


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


# ---------------------------------------------------------------------------------------------- formats
def row_bytes(t: int, n: int) -> int:
    return int(lib().orc_row_bytes(t, n))


def dequantize(t: int, raw: np.ndarray, rows: int, cols: int) -> np.ndarray:
    """rows x cols fp32 from `raw` (uint8, rows * row_bytes)."""
    rb = row_bytes(t, cols)
    raw = np.ascontiguousarray(raw, dtype=np.uint8)
    assert raw.size >= rows * rb
    out = np.empty((rows, cols), np.float32)
    for r in range(rows):
        lib().orc_dequant_row(t, raw.ctypes.data + r * rb, out[r], cols)
    return out


def quantize(t: int, w: np.ndarray) -> np.ndarray:
    w = np.ascontiguousarray(w, dtype=np.float32)
    rows, cols = w.shape
    out = np.zeros(rows * row_bytes(t, cols), np.uint8)
    n = lib().orc_quantize_rows(t, w, out, rows, cols)
    assert n == out.size, "type has no quantiser"
    return out


def quantize_q8_1(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.zeros(x.size // 32 * 36, np.uint8)
    lib().orc_quantize_q8_1(x.reshape(-1), x.size, out)
    return out


def fnv1a(*arrays, h: int = 1469598103934665603) -> int:
    for a in arrays:
        a = np.ascontiguousarray(a)
        h = lib().orc_fnv1a(h, a.ctypes.data, a.nbytes)
    return int(h)


class Layout:
    """One expert blob [gate rows | up rows | down rows | NVFP4: fp32 {s_gate, s_up, s_down, 0}] - the reference's
    NativeExpertLayout (include/basalt/kernels/iq_kernels.hpp:51-66, src/kernels/cuda/iq_kernels.cu:3221-3238)."""

    def __init__(self, gu_type: int, d_type: int, H: int, I: int):
        self.gu_type, self.d_type, self.H, self.I = gu_type, d_type, H, I
        self.gu_row = row_bytes(gu_type, H)
        self.d_row = row_bytes(d_type, I)
        assert self.gu_row and self.d_row
        self.up_off = I * self.gu_row
        self.down_off = 2 * I * self.gu_row
        self.tail = 16 if gu_type == T_NVFP4 else 0
        self.bytes = self.down_off + H * self.d_row + self.tail


def make_blob(L: Layout, G: np.ndarray, U: np.ndarray, D: np.ndarray) -> np.ndarray:
    """Quantises fp32 matrices into one blob.  NVFP4 follows the reference's recipe for synthetic packs
    (tests/kernels/native_expert_parity.cpp:411-432): each matrix is divided by a per-matrix fp32 scale
    s = amax / (6 * 448) before block quantisation and s is stored in the tail."""
    blob = np.zeros(L.bytes, np.uint8)
    tail = np.ones(4, np.float32)
    mats = ((G, L.gu_type, 0), (U, L.gu_type, L.up_off), (D, L.d_type, L.down_off))
    for i, (w, t, off) in enumerate(mats):
        w = np.ascontiguousarray(w, np.float32)
        if t == T_NVFP4:
            s = np.float32(np.abs(w).max() / (6.0 * 448.0))
            s = s if s > 0 else np.float32(1)
            tail[i] = s
            w = (w / s).astype(np.float32)
        q = quantize(t, w)
        blob[off:off + q.size] = q
    if L.tail:
        tail[3] = 0
        blob[L.bytes - 16:] = tail.view(np.uint8)
    return blob


def random_iq1m_rows(rng: np.random.Generator, rows: int, cols: int) -> np.ndarray:
    """Random valid IQ1_M rows: uniform bytes with a finite fp16 super-scale near 2^-6 patched into the top nibbles of
    the four scale words (the reference's own tests do the same, having no IQ1_M quantiser:
    tests/kernels/iq1s_parity.cpp:65-93)."""
    nb = rows * cols // 256
    raw = rng.integers(0, 256, size=(nb, 56), dtype=np.uint8)
    d = (0x2000 + rng.integers(0, 0x400, size=nb)).astype(np.uint16)   # fp16 in [2^-7, 2^-6)
    sc = raw[:, 48:56].copy().view(np.uint16)
    sc[:, 0] = (sc[:, 0] & 0x0FFF) | ((d & 0x000F) << 12)
    sc[:, 1] = (sc[:, 1] & 0x0FFF) | ((d & 0x00F0) << 8)
    sc[:, 2] = (sc[:, 2] & 0x0FFF) | ((d & 0x0F00) << 4)
    sc[:, 3] = (sc[:, 3] & 0x0FFF) | (d & 0xF000)
    raw[:, 48:56] = sc.view(np.uint8)
    return raw.reshape(-1)


def random_rows(t: int, rng: np.random.Generator, rows: int, cols: int) -> np.ndarray:
    """Random valid rows of a format the oracle has no quantiser for: uniform bytes with finite fp16 scales near 2^-9 (so
    values are of order 0.02, like the quantised N(0, 0.02^2) weights of the other formats)."""
    if t == T_IQ1_M:
        return random_iq1m_rows(rng, rows, cols)
    if t in LOW_BIT:
        # (block bytes, values, {offset of an fp16 scale: its exponent bits}); the scales put values near 0.02 as above
        bs, nv, scales = {T_Q2_0: (18, 64, {0: 0x2400}), T_Q2_K: (84, 256, {80: 0x1000, 82: 0x1800}), T_Q3_K: (110, 256, {108: 0x0C00}),
                          T_IQ2_XXS: (66, 256, {0: 0x0800}), T_IQ2_XS: (74, 256, {0: 0x0800}), T_IQ2_S: (82, 256, {0: 0x0800}),
                          T_IQ3_XXS: (98, 256, {0: 0x0400}), T_IQ3_S: (110, 256, {0: 0x0400}), T_IQ1_S: (50, 256, {0: 0x1800})}[t]
        nb = rows * cols // nv
        raw = rng.integers(0, 256, size=(nb, bs), dtype=np.uint8)
        for at, base in scales.items():
            h = (base + rng.integers(0, 0x400, size=nb)).astype(np.uint16)
            raw[:, at:at + 2] = h.view(np.uint8).reshape(nb, 2)
        return raw.reshape(-1)
    bs, nv, scale_at = {T_Q8_0: (34, 32, (0,)), T_Q4_K: (144, 256, (0, 2)), T_Q5_K: (176, 256, (0, 2)), T_Q5_0: (22, 32, (0,)),
                        T_Q5_1: (24, 32, (0, 2)), T_IQ4_NL: (18, 32, (0,)), T_IQ4_XS: (136, 256, (0,))}[t]
    nb = rows * cols // nv
    raw = rng.integers(0, 256, size=(nb, bs), dtype=np.uint8)
    for at in scale_at:
        # fp16 scales: Q8_0 / IQ4_NL 2^-12 (x 8-bit level), Q5_0 2^-9 (x 5-bit code), Q5_1 2^-9 and m 2^-6 (negated below: codes are
        # unsigned), IQ4_XS 2^-15 (x 6-bit scale x level), Q4_K / Q5_K d 2^-13 (x 6-bit scale x code) and dmin 2^-10 (x 6-bit min)
        base = {T_Q8_0: 0x0C00, T_IQ4_NL: 0x0C00, T_Q5_0: 0x1800, T_IQ4_XS: 0x0200}.get(t, 0x0800 if at == 0 else 0x1400)
        if t == T_Q5_1:
            base = 0x1800 if at == 0 else 0xA400
        h = (base + rng.integers(0, 0x400, size=nb)).astype(np.uint16)
        raw[:, at:at + 2] = h.view(np.uint8).reshape(nb, 2)
    return raw.reshape(-1)


def blob_matrices(L: Layout, blob: np.ndarray):
    """(G, U, D, tail) decoded to fp32."""
    G = dequantize(L.gu_type, blob[0:], L.I, L.H)
    U = dequantize(L.gu_type, blob[L.up_off:], L.I, L.H)
    D = dequantize(L.d_type, blob[L.down_off:], L.H, L.I)
    tail = np.ones(3, np.float32)
    if L.tail:
        tail = blob[L.bytes - 16:L.bytes - 4].view(np.float32).copy()
    return G, U, D, tail


def expert_forward(L: Layout, blob: np.ndarray, x: np.ndarray, limit: float = 0.0, dtype=np.float32) -> np.ndarray:
    """The dequantised reference expert (tests/kernels/native_expert_parity.cpp:58-84): out = s_d D (silu(s_g G x) * (s_u U x))
    with matrix products accumulated in `dtype` (fp32 = the parity bar, fp64 = the second opinion)."""
    G, U, D, tail = blob_matrices(L, blob)
    x = np.asarray(x, np.float32).astype(dtype)
    g = (x @ G.astype(dtype).T) * dtype(tail[0])
    u = (x @ U.astype(dtype).T) * dtype(tail[1])
    if limit > 0:
        g = np.minimum(g, limit)
        u = np.clip(u, -limit, limit)
    h = (g / (1 + np.exp(-g)) * u).astype(dtype)
    return ((h @ D.astype(dtype).T) * dtype(tail[2])).astype(np.float32)


# ---------------------------------------------------------------------------------------------- router / dispatch / combine
def router_logits(x: np.ndarray, gate: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, np.float32)
    gate = np.ascontiguousarray(gate, np.float32)
    T, H = x.shape
    E = gate.shape[0]
    out = np.empty((T, E), np.float32)
    lib().orc_router_logits(x, gate, T, E, H, out)
    return out


def router_select(logits, bias, k, kind, scale=1.0, n_group=1, topk_group=1, prior=0.0, held=None):
    logits = np.ascontiguousarray(logits, np.float32)
    T, E = logits.shape
    ids = np.zeros((T, k), np.int32)
    w = np.zeros((T, k), np.float32)
    if kind == GATE_SOFTMAX:
        lib().orc_router_softmax(logits, T, E, k, 0, ids, w)
    else:
        bias = None if bias is None else np.ascontiguousarray(bias, np.float32)
        held = None if held is None else np.ascontiguousarray(held, np.int32)
        lib().orc_router_select(logits, _ptr(bias), T, E, k, kind, scale, n_group, topk_group, prior, _ptr(held), ids, w)
    return ids, w


def router_select_scores(scores, bias, k, scale=1.0, n_group=1, topk_group=1, prior=0.0, held=None):
    """router_select from gate scores already computed (e.g. by the device, so that no libm / device expf difference enters):
    the group-limited step, the ranks and the weights in fp32, bit for bit what the device kernels must give."""
    scores = np.ascontiguousarray(scores, np.float32)
    T, E = scores.shape
    ids = np.zeros((T, k), np.int32)
    w = np.zeros((T, k), np.float32)
    bias = None if bias is None else np.ascontiguousarray(bias, np.float32)
    held = None if held is None else np.ascontiguousarray(held, np.int32)
    lib().orc_router_select_scores(scores, _ptr(bias), T, E, k, scale, n_group, topk_group, prior, _ptr(held), ids, w)
    return ids, w


def router_softmax_fast(logits, k):
    logits = np.ascontiguousarray(logits, np.float32)
    T, E = logits.shape
    ids = np.zeros((T, k), np.int32)
    w = np.zeros((T, k), np.float32)
    lib().orc_router_softmax(logits, T, E, k, 1, ids, w)
    return ids, w


def router_top10(logits, k):
    logits = np.ascontiguousarray(logits, np.float32)
    T, E = logits.shape
    ids = np.zeros((T, k), np.int32)
    w = np.zeros((T, k), np.float32)
    lib().orc_router_top10(logits, T, E, k, ids, w)
    return ids, w


def route_tail_skip(ids, w, held, k, rank, E):
    ids = np.ascontiguousarray(ids, np.int32).copy()
    w = np.ascontiguousarray(w, np.float32).copy()
    counts = np.zeros(3, np.uint64)
    held = None if held is None else np.ascontiguousarray(held, np.int32)
    lib().orc_route_tail_skip(ids.reshape(-1), w.reshape(-1), _ptr(held), ids.size, k, rank, E, _ptr(counts))
    return ids, w, counts


def dispatch(ids, k, E, tile_rows=0):
    ids = np.ascontiguousarray(ids, np.int32).reshape(-1)
    n = ids.size
    cnt = np.zeros(E, np.int32)
    off = np.zeros(E + 1, np.int32)
    slot = np.zeros(n, np.int32)
    src = np.full(n, -1, np.int32)
    tiles = np.zeros(2 * (n + E), np.int32) if tile_rows else None
    nt = lib().orc_dispatch(ids, n, k, E, cnt, off, slot, src, tile_rows, _ptr(tiles))
    return cnt, off, slot, src, (tiles[:2 * nt].reshape(-1, 2) if tile_rows else None)


def moe_plan(ids, k, E, blobs):
    ids = np.ascontiguousarray(ids, np.int32).reshape(-1)
    n = ids.size
    blobs = np.ascontiguousarray(blobs, np.uint64)
    ptr = np.zeros(max(n, 1), np.uint64)
    start = np.zeros(n + 2, np.int32)
    ng = np.zeros(1, np.int32)
    dst = np.zeros(max(n, 1), np.int32)
    tok = np.zeros(max(n, 1), np.int32)
    lib().orc_moe_plan(ids, n, k, E, blobs, ptr, start, ng, dst, tok)
    return ptr, start, int(ng[0]), dst, tok


def combine(rows, slot, w, shared=None, sg=None):
    rows = np.ascontiguousarray(rows, np.float32)
    w = np.ascontiguousarray(w, np.float32)
    T, k = w.shape
    H = rows.shape[1]
    slot = None if slot is None else np.ascontiguousarray(slot, np.int32)
    shared = None if shared is None else np.ascontiguousarray(shared, np.float32)
    sg = None if sg is None else np.ascontiguousarray(sg, np.float32)
    y = np.empty((T, H), np.float32)
    lib().orc_combine(rows, _ptr(slot), w, _ptr(shared), _ptr(sg), T, k, H, y)
    return y


def moe_layer(x, gate_w, bias, blobs, L: Layout, k, kind, scale=1.0, n_group=1, topk_group=1, shared_blob=None,
              shared_layout=None, limit=0.0, dtype=np.float32):
    """The whole layer on the CPU: router -> dispatch -> dequantised experts -> combine (+ shared expert).  Returns
    (y, ids, weights, cnt, off, slot, src).  `blobs` is a sequence of per-expert uint8 arrays."""
    x = np.ascontiguousarray(x, np.float32)
    T, H = x.shape
    E = len(blobs)
    logits = router_logits(x, gate_w)
    ids, w = router_select(logits, bias, k, kind, scale, n_group, topk_group)
    cnt, off, slot, src, _ = dispatch(ids, k, E)
    rows = np.zeros((T * k, H), np.float32)
    for e in range(E):
        if cnt[e]:
            toks = src[off[e]:off[e + 1]]
            rows[off[e]:off[e + 1]] = expert_forward(L, blobs[e], x[toks], limit, dtype)
    shared = None
    if shared_blob is not None:
        shared = expert_forward(shared_layout or L, shared_blob, x, limit, dtype)
    y = combine(rows, slot, w, shared)
    return y, ids, w, cnt, off, slot, src


# ---------------------------------------------------------------------------------------------- the reference itself
_ref_cpu = None


def norm_pack(x: np.ndarray, w: np.ndarray, eps: float):
    """The RMS norm of each row, restating wgemm::norm_pack (src/kernels/cuda/window_gemm.cu:40-112): thread i of 512 sums the
    squares of columns i, i + 512, ... as one fma chain, a warp's 32 chains are added by xor butterfly, the 16 warp sums in
    warp order; inv = 1 / sqrt(sum / K + eps); value = (x * inv) * w.  fp32 throughout (an fma as a product and a sum in
    fp64 rounded once to fp32); the device's rsqrtf is an approximation, so the GPU rows sit within 4 ulp of these, not on
    them.  Returns (xn fp32, act = xn rounded to bf16 bits as uint16)."""
    x = np.ascontiguousarray(x, np.float32)
    T, K = x.shape
    n_chain = 512
    pad = (-K) % n_chain
    xp = np.pad(x, ((0, 0), (0, pad))).reshape(T, -1, n_chain)          # [T][j][thread]
    ss = np.zeros((T, n_chain), np.float32)
    for j in range(xp.shape[1]):
        v = xp[:, j, :].astype(np.float64)
        ss = (v * v + ss.astype(np.float64)).astype(np.float32)
    s = ss.reshape(T, 16, 32)
    for m in (16, 8, 4, 2, 1):
        s = (s + s[:, :, np.arange(32) ^ m]).astype(np.float32)
    t = np.zeros(T, np.float32)
    for wp in range(16):
        t = (t + s[:, wp, 0]).astype(np.float32)
    inv = (np.float32(1.0) / np.sqrt((t / np.float32(K) + np.float32(eps)).astype(np.float32))).astype(np.float32)
    xn = ((x * inv[:, None]).astype(np.float32) * w.astype(np.float32)[None, :]).astype(np.float32)
    u = xn.view(np.uint32)
    act = ((u + (0x7FFF + ((u >> 16) & 1))) >> 16).astype(np.uint16)      # round to nearest even (finite values)
    return xn, act


def ref_cpu():
    """oracle/_ref/libref_cpu.so (the reference's ggml quantisers and CPU expert pool), or None if it was never built."""
    global _ref_cpu
    p = HERE / "_ref" / "libref_cpu.so"
    if _ref_cpu is None and p.exists():
        L = C.CDLL(str(p))
        L.ref_row_bytes.restype = C.c_int64
        L.ref_row_bytes.argtypes = [C.c_int, C.c_int64]
        L.ref_quantize.restype = C.c_int64
        L.ref_quantize.argtypes = [C.c_int, _f32p, _u8p, C.c_int64, C.c_int64]
        L.ref_dequantize.argtypes = [C.c_int, C.c_void_p, _f32p, C.c_int64]
        L.ref_native_fmt.argtypes = [C.c_int, C.c_int, C.c_int64, C.c_int64, C.c_float, C.c_void_p, C.c_char_p, C.c_int]
        L.ref_pool_create.restype = C.c_void_p
        L.ref_pool_create.argtypes = [C.c_int]
        L.ref_pool_destroy.argtypes = [C.c_void_p]
        L.ref_pool_workers.argtypes = [C.c_void_p]
        L.ref_pool_layer.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int64, C.c_int64, C.c_float, C.c_void_p, C.c_int,
                                     _i32p, _i32p, _f32p, C.c_int, _f32p]
        if hasattr(L, "ref_avx2_layer"):
            L.ref_avx2_layer.argtypes = [C.c_int, C.c_int64, C.c_int64, C.c_void_p, C.c_int, _i32p, _i32p, _f32p, C.c_int, _f32p]
            L.ref_cpu_info.argtypes = [C.c_char_p, C.c_int]
        if hasattr(L, "ref_layout_load_text"):
            L.ref_layout_load_text.argtypes = [C.c_char_p, C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_float,
                                               C.c_void_p, C.c_void_p, C.c_char_p, C.c_int]
        _ref_cpu = L
    return _ref_cpu


def ref_layout_load_text(text: bytes, n_layers: int, n_expert: int, n_embd: int, n_ff: int, swiglu_limit: float = 0.0):
    """The reference's own parse of an `experts.layout` text (expert_layout_load_text, src/kernels/cpu/expert_layout.cpp:133-203)
    through oracle/_ref: (True, head, rows) with head = [version, n_expert, max_blob, total, n_layers] and one
    [gu_type, d_type, up_type, offset, blob_bytes, up_off] per layer, or (False, reason, None)."""
    L = ref_cpu()
    head = np.zeros(5, np.int64)
    rows = np.zeros((max(n_layers, 1), 6), np.int64)
    err = C.create_string_buffer(512)
    ok = L.ref_layout_load_text(text, len(text), n_layers, n_expert, n_embd, n_ff, swiglu_limit, head.ctypes.data, rows.ctypes.data,
                                err, len(err))
    if not ok:
        return False, err.value.decode("utf-8", "replace"), None
    return True, head.tolist(), rows[:n_layers].tolist()


def ref_gpu():
    """oracle/_ref/libref_gpu.so (the reference's portable CUDA kernels built for sm_100a), or None.  Needs a GPU."""
    p = HERE / "_ref" / "libref_gpu.so"
    if not p.exists():
        return None
    L = C.CDLL(str(p))
    L.refg_expert_blob_bytes.restype = C.c_int64
    L.refg_expert_scratch_bytes.restype = C.c_int64
    if hasattr(L, "refg_norm_pack"):
        L.refg_norm_pack.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_float, C.c_int64, C.c_int, C.c_void_p, C.c_void_p]
    return L
