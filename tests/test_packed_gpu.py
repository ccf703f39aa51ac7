"""GPU parity of the block-scaled FP4 tensor-core expert path (bsx_expert_pack + bsx_experts_grouped_packed): the plane
layout against a numpy re-ordering of the ggml blob (bit-exact), the grouped experts against the dequantised fp32-accumulated
oracle expert (bar: relative L2 <= 2e-3; four FP4 activation terms give ~1e-4), ragged passes, every activation kind, and the
whole layer against the fp16-image kernels."""
import ctypes as C

import numpy as np
import pytest
import torch

from basalt_b200 import capi, moe
from oracle import oracle as O
from tests.helpers import make_expert_blobs, rel_l2, stack_blobs

pytestmark = pytest.mark.gpu
TOL = 2e-3


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def planes_from_ggml(blob, H, I):
    """The packed layout restated on the host.  A matrix of R rows x K columns = (R / 128) x (K / 256) blocks of 18,432 bytes,
    row tile major; a block = its 128 rows x 128 code bytes with the 16-byte pieces of row r at piece index p ^ (r % 8), then
    four K-steps x (32 x 4) scale words, word (l, j) = row 32 j + l, scale bytes with bit 7 cleared and 0x7F -> 0."""
    def matrix(off, R, K):
        rows = blob[off:off + R * (K // 64) * 36].reshape(R, K // 64, 36)
        codes = np.ascontiguousarray(rows[:, :, 4:]).reshape(R // 128, 128, K // 256, 8, 16)      # [tile][r][chunk][piece][16]
        sc = rows[:, :, :4] & 0x7F
        sc = np.where(sc == 0x7F, 0, sc).astype(np.uint8)
        words = np.ascontiguousarray(sc).view(np.uint32).reshape(R // 128, 128, K // 256, 4)          # [tile][r][chunk][step]
        out = np.zeros((R // 128, K // 256, 18432), np.uint8)
        r = np.arange(128)
        for p in range(8):
            dst = (r // 8) * 1024 + (r % 8) * 128 + ((p ^ (r % 8)) << 4)
            for t in range(R // 128):
                for c in range(K // 256):
                    img = out[t, c]
                    idx = dst[:, None] + np.arange(16)[None, :]
                    img[idx] = codes[t, :, c, p, :]
        for t in range(R // 128):
            for c in range(K // 256):
                sf = np.zeros((4, 32, 4), np.uint32)
                sf[:, r % 32, r // 32] = words[t, :, c, :].T
                out[t, c, 16384:] = sf.reshape(-1).view(np.uint8)
        return out.reshape(-1)
    gu = I * (H // 64) * 36
    tail = blob[2 * gu + H * (I // 64) * 36:][:16]
    return np.concatenate([matrix(0, I, H), matrix(gu, I, H), matrix(2 * gu, H, I), tail])


@pytest.mark.parametrize("H,I", [(512, 256), (2048, 512)])
def test_pack_is_the_ggml_bytes_in_plane_order(lib, cuda, H, I):
    rng = np.random.default_rng(H)
    Lo, blobs = make_expert_blobs(rng, 2, O.T_NVFP4, O.T_NVFP4, H, I)
    blobs[1] = blobs[1].copy()
    blobs[1][0] = 0x7F                 # a scale byte the decoder reads as zero
    blobs[1][36 + 1] |= 0x80           # and one with the ignored top bit set
    L = moe.native_expert_layout(40, 40, H, I)
    packed = moe.pack_experts(L, dev(stack_blobs(blobs)))
    torch.cuda.synchronize()
    for e in range(2):
        want = planes_from_ggml(np.asarray(blobs[e]), H, I)
        got = packed[e].cpu().numpy()[:want.size]
        assert np.array_equal(got, want)


def run_packed(L, packed, group_experts, group_tokens, x_dev, n_x_rows=0, out_dtype=torch.float32):
    stride = packed.shape[1]
    ptr = torch.tensor([packed.data_ptr() + e * stride for e in group_experts] + [0], dtype=torch.int64).cuda()
    starts = np.concatenate([[0], np.cumsum([len(t) for t in group_tokens])]).astype(np.int32)
    n = int(starts[-1])
    start = dev(np.concatenate([starts, [starts[-1]]]).astype(np.int32))
    tok = dev(np.concatenate([np.asarray(t, np.int32) for t in group_tokens] + [np.zeros(1, np.int32)])[:max(n, 1)].astype(np.int32))
    dst = dev(np.arange(max(n, 1), dtype=np.int32))
    ng = dev(np.array([len(group_experts)], np.int32))
    out = torch.full((max(n, 1), L.n_embd), float("nan"), dtype=out_dtype, device="cuda")
    scratch = torch.empty(capi.lib().bsx_experts_packed_scratch_bytes(C.byref(L), max(n, 1)), dtype=torch.uint8, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    moe.native_expert_grouped_packed(L, ptr, start, ng, dst, tok, len(group_experts), n, x_dev, scratch, out, status, n_x_rows=n_x_rows)
    torch.cuda.synchronize()
    assert int(status.item()) == 0, "a bounded wait inside the kernel gave up"
    return out.float().cpu().numpy()


@pytest.mark.parametrize("kind", ["q8_1", "bf16_out", "limit"])
def test_packed_activation_output_and_swiglu_kinds(lib, cuda, kind):
    """The packed path with the reference's q8_1 activation rows (decoded as d * q), bf16 output rows, and the limited SwiGLU."""
    rng = np.random.default_rng(98)
    H, I, E, T = 2048, 512, 4, 9
    Lo, blobs = make_expert_blobs(rng, E, 40, 40, H, I, sigma=0.2 if kind == "limit" else 0.02)
    L = moe.native_expert_layout(40, 40, H, I, swiglu_limit=3.0 if kind == "limit" else 0.0)
    packed = moe.pack_experts(L, dev(stack_blobs(blobs)))
    x = rng.standard_normal((T, H)).astype(np.float32)
    group_tokens = [[0, 3], [1], [2, 4, 5, 6, 7, 8, 0, 1, 2], []]
    xt = torch.from_numpy(x).cuda()
    if kind == "q8_1":
        xd = moe.quantize_q8_1_rows(xt)
        q = xd.cpu().numpy().reshape(-1, 36)
        x_eff = (q[:, 4:].view(np.int8).astype(np.float32) * q[:, :2].copy().view(np.float16).astype(np.float32)).reshape(T, H)
    else:
        xd = xt.bfloat16()
        x_eff = xd.float().cpu().numpy()
    out = run_packed(L, packed, list(range(E)), group_tokens, xd, out_dtype=torch.bfloat16 if kind == "bf16_out" else torch.float32)
    at = 0
    for e, toks in enumerate(group_tokens):
        if toks:
            want = O.expert_forward(Lo, blobs[e], x_eff[toks], limit=3.0 if kind == "limit" else 0.0)
            tol = 4e-3 if kind == "bf16_out" else TOL                      # bf16 output rounding alone is ~1.7e-3
            assert rel_l2(out[at:at + len(toks)], want) < tol, (kind, e, rel_l2(out[at:at + len(toks)], want))
            if kind == "limit":
                assert rel_l2(out[at:at + len(toks)], O.expert_forward(Lo, blobs[e], x_eff[toks])) > 1e-2   # the limit bites
        at += len(toks)


@pytest.mark.parametrize("H,I,sizes", [(2048, 512, [37, 16, 1, 52]), (1024, 1024, [33, 47])])
def test_packed_deep_groups_take_the_wide_passes(lib, cuda, H, I, sizes):
    """Groups of tens of entries (what an expert-parallel rank sees): with 12+ entries a group on average the call takes passes of
    16 entries (MMA N = 64).  Every row against the dequantised reference, and against the same rows computed with shallow groups
    (passes of 8): the two widths sum the same products, so they agree to fp32 rounding."""
    rng = np.random.default_rng(H + I + len(sizes))
    E, T = len(sizes), 40
    Lo, blobs = make_expert_blobs(rng, E, 40, 40, H, I)
    L = moe.native_expert_layout(40, 40, H, I)
    packed = moe.pack_experts(L, dev(stack_blobs(blobs)))
    x = rng.standard_normal((T, H)).astype(np.float32)
    xd = torch.from_numpy(x).cuda().bfloat16()
    x_eff = xd.float().cpu().numpy()
    group_tokens = [rng.integers(0, T, n).tolist() for n in sizes]
    assert sum(sizes) >= 12 * E
    out = run_packed(L, packed, list(range(E)), group_tokens, xd, n_x_rows=T)
    at = 0
    for e, toks in enumerate(group_tokens):
        want = O.expert_forward(Lo, blobs[e], x_eff[toks])
        for r in range(len(toks)):
            assert rel_l2(out[at + r], want[r]) < TOL, (e, r, rel_l2(out[at + r], want[r]))
        # the same entries as groups of at most 5 (capacity below 12 a group: passes of 8)
        for lo in range(0, len(toks), 5):
            part = toks[lo:lo + 5]
            narrow = run_packed(L, packed, [e] * 2, [part, []], xd, n_x_rows=T)
            assert rel_l2(narrow[:len(part)], out[at + lo:at + lo + len(part)]) < 1e-6
        at += len(toks)
    del packed


def test_packed_call_with_no_groups_returns_cleanly(lib, cuda):
    """A plan without groups (every expert held elsewhere): the kernels start, find no work and return; nothing is written."""
    rng = np.random.default_rng(97)
    H, I = 512, 256
    Lo, blobs = make_expert_blobs(rng, 1, 40, 40, H, I)
    L = moe.native_expert_layout(40, 40, H, I)
    packed = moe.pack_experts(L, dev(stack_blobs(blobs)))
    ptr = torch.zeros(4, dtype=torch.int64, device="cuda")
    start = torch.zeros(4, dtype=torch.int32, device="cuda")
    ng = torch.zeros(1, dtype=torch.int32, device="cuda")
    idx = torch.zeros(8, dtype=torch.int32, device="cuda")
    x = torch.randn((4, H), device="cuda")
    out = torch.full((8, H), 7.0, dtype=torch.float32, device="cuda")
    scratch = torch.empty(capi.lib().bsx_experts_packed_scratch_bytes(C.byref(L), 8), dtype=torch.uint8, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    moe.native_expert_grouped_packed(L, ptr, start, ng, idx, idx, 2, 8, x, scratch, out, status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0 and bool((out == 7.0).all())
    del packed


@pytest.mark.parametrize("H,I,xdt,rows_known", [(512, 256, "f32", False), (2048, 512, "bf16", True), (2048, 512, "f32", False), (7168, 2048, "bf16", True)])
def test_packed_experts_vs_dequantised_reference(lib, cuda, H, I, xdt, rows_known):
    rng = np.random.default_rng(H + I)
    E = 3 if H > 4096 else 6
    Lo, blobs = make_expert_blobs(rng, E, O.T_NVFP4, O.T_NVFP4, H, I)
    L = moe.native_expert_layout(40, 40, H, I)
    packed = moe.pack_experts(L, dev(stack_blobs(blobs)))
    T = 24
    x = rng.standard_normal((T, H)).astype(np.float32)
    x[3] *= 1e-3
    x[5] *= 200.0
    xd = dev(x)
    if xdt == "bf16":
        xd = xd.bfloat16()
        x = xd.float().cpu().numpy()
    sizes = ([1, 0, 3, 11, 8, 20] if E == 6 else [2, 9, 1])
    group_tokens = [rng.integers(0, T, s).tolist() for s in sizes]
    out = run_packed(L, packed, list(range(E)), group_tokens, xd, n_x_rows=T if rows_known else 0)
    at, worst = 0, 0.0
    for e, toks in enumerate(group_tokens):
        if toks:
            want = O.expert_forward(Lo, blobs[e], x[toks])
            got = out[at:at + len(toks)]
            assert np.isfinite(got).all()
            worst = max(worst, rel_l2(got, want))
            for r in range(len(toks)):
                assert rel_l2(got[r], want[r]) < TOL, (e, r, rel_l2(got[r], want[r]))
        at += len(toks)
    print("worst relative L2 over experts:", worst)
    assert worst < TOL


def test_packed_layer_matches_the_fp16_image_layer(lib, cuda):
    rng = np.random.default_rng(11)
    E, H, I, K, T = 64, 2048, 512, 10, 64
    Lo, blobs = make_expert_blobs(rng, E + 1, O.T_NVFP4, O.T_NVFP4, H, I)
    L = moe.native_expert_layout(40, 40, H, I)
    bd = dev(stack_blobs(blobs))
    packed = moe.pack_experts(L, bd)
    gate = dev((rng.standard_normal((E, H)) * 0.02).astype(np.float32))
    args = moe.RouterArgs(n_expert=E, n_embd=H, k=K, weight_scale=1.0, gate=capi.GATE_SOFTMAX)
    x = torch.randn((T, H), device="cuda", generator=torch.Generator(device="cuda").manual_seed(5)).bfloat16()
    plain = moe.MoELayer(gate, None, bd[:E], L, args, shared_blob=bd[E], max_tokens=T)
    fast = moe.MoELayer(gate, None, packed[:E], L, args, shared_blob=packed[E], max_tokens=T, packed=True)
    want = plain.forward(x).clone()
    got = fast.forward(x).clone()
    got2 = fast.forward(x).clone()
    torch.cuda.synchronize()
    assert int(fast.status.item()) == 0
    rel = float((got - want).norm() / want.norm())
    print("packed layer vs fp16-image layer, relative L2:", rel)
    assert rel < 1e-3
    assert torch.equal(got.view(torch.int32), got2.view(torch.int32)), "not bit-stable from run to run"


def test_layer_step_replays_as_a_cuda_graph(lib, cuda):
    """The whole step (router, plan, images, experts, combine) is stream-ordered and allocation-free, so it records into a
    CUDA graph; the replay gives the bits of the launch-by-launch step."""
    rng = np.random.default_rng(12)
    E, H, I, K, T = 32, 512, 256, 4, 16
    Lo, blobs = make_expert_blobs(rng, E + 1, O.T_NVFP4, O.T_NVFP4, H, I)
    L = moe.native_expert_layout(40, 40, H, I)
    bd = dev(stack_blobs(blobs))
    packed = moe.pack_experts(L, bd)
    gate = dev((rng.standard_normal((E, H)) * 0.02).astype(np.float32))
    args = moe.RouterArgs(n_expert=E, n_embd=H, k=K, weight_scale=1.0, gate=capi.GATE_SOFTMAX)
    g = torch.Generator(device="cuda").manual_seed(6)
    xs = [torch.randn((T, H), device="cuda", generator=g).bfloat16() for _ in range(3)]
    for pk, b in ((True, packed), (False, bd)):
        layer = moe.MoELayer(gate, None, b[:E], L, args, shared_blob=b[E], max_tokens=T, packed=pk)
        want = [layer.forward(x).clone() for x in xs]
        layer.capture(xs[0])
        got = [layer.forward_graphed(x).clone() for x in xs]
        torch.cuda.synchronize()
        for w, gt in zip(want, got):
            assert torch.equal(w.view(torch.int32), gt.view(torch.int32))
