"""GPU parity of the prompt-sized grouped experts (tcgen05 path): dispatch -> bsx_experts_prefill -> rows, against the
dequantised fp32-accumulated oracle expert on the same gathered rows (bar: relative L2 <= 2e-3), with ragged expert loads
(Zipf 1.1), empty experts, experts held elsewhere, and the decode kernels as a second implementation of the same rows."""
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


def zipf_ids(rng, T, k, E):
    p = 1.0 / np.arange(1, E + 1) ** 1.1
    lg = np.log(p)[None, :] + rng.gumbel(size=(T, E))
    return np.argsort(-lg, axis=1)[:, :k].astype(np.int32)


def run_prefill(L, bd, ids, k, E, x, held=None):
    stride = bd.shape[1]
    table = bd.data_ptr() + np.arange(E, dtype=np.int64) * stride
    if held is not None:
        table = np.where(held, table, 0)
    cnt, off, slot, src, tiles, n_tiles = moe.dispatch(dev(ids.reshape(-1)), k, E, tile_rows=128)
    dm, status = moe.experts_prefill(L, dev(table), off, src, tiles, n_tiles, x, ids.size)
    torch.cuda.synchronize()
    assert int(status.item()) == 0, "a bounded wait inside the kernel gave up"
    return dm.cpu().numpy(), cnt.cpu().numpy(), off.cpu().numpy(), src.cpu().numpy(), slot.cpu().numpy()


@pytest.mark.parametrize("E,H,I,T,k,xdt", [(8, 512, 256, 300, 2, "f32"), (8, 512, 256, 5, 2, "bf16"), (16, 2048, 512, 1000, 4, "bf16"),
                                           (4, 7168, 2048, 200, 2, "bf16")])
def test_prefill_vs_dequantised_reference(lib, cuda, E, H, I, T, k, xdt):
    rng = np.random.default_rng(E + H + T)
    Lo, blobs = make_expert_blobs(rng, E, O.T_NVFP4, O.T_NVFP4, H, I)
    L = moe.native_expert_layout(40, 40, H, I)
    ids = zipf_ids(rng, T, k, E)
    ids[ids == E - 1] = 0 if k == 1 else ids[ids == E - 1]      # keep ids valid; the last expert may simply be cold
    x = rng.standard_normal((T, H)).astype(np.float32)
    xd = torch.from_numpy(x).cuda()
    if xdt == "bf16":
        xd = xd.bfloat16()
        x = xd.float().cpu().numpy()
    dm, cnt, off, src, slot = run_prefill(L, dev(stack_blobs(blobs)), ids, k, E, xd)
    worst = 0.0
    for e in range(E):
        if cnt[e]:
            want = O.expert_forward(Lo, blobs[e], x[src[off[e]:off[e + 1]]])
            got = dm[off[e]:off[e + 1]]
            assert np.isfinite(got).all()
            worst = max(worst, rel_l2(got, want))
    print("worst relative L2 over experts:", worst)
    assert worst < TOL, worst


@pytest.mark.parametrize("name,gt,dt,E,H,I,T,k", [("q6k", 14, 14, 8, 2048, 512, 1100, 2), ("iq1m", 29, 29, 8, 2048, 512, 1100, 2),
                                                   ("iq1m_q6k_down", 29, 14, 4, 1024, 512, 300, 2), ("iq1m_big", 29, 29, 3, 7168, 2048, 260, 1)])
def test_prefill_k_and_i_quant_blobs_vs_dequantised_reference(lib, cuda, name, gt, dt, E, H, I, T, k):
    """Prompt-sized experts over K- and I-quant blobs in place (the reference runs these through its int8 MMQ path,
    include/basalt/prefill/moe_mmq.hpp:37-125): the decoder warps of the tcgen05 kernel read Q6_K / IQ1_M rows."""
    rng = np.random.default_rng(E + H + T + gt)
    Lo, blobs = make_expert_blobs(rng, E, gt, dt, H, I)
    L = moe.native_expert_layout(gt, dt, H, I)
    ids = zipf_ids(rng, T, k, E)
    xd = torch.from_numpy(rng.standard_normal((T, H)).astype(np.float32)).cuda().bfloat16()
    x = xd.float().cpu().numpy()
    dm, cnt, off, src, slot = run_prefill(L, dev(stack_blobs(blobs)), ids, k, E, xd)
    worst = 0.0
    for e in range(E):
        if cnt[e]:
            want = O.expert_forward(Lo, blobs[e], x[src[off[e]:off[e + 1]]])
            got = dm[off[e]:off[e + 1]]
            assert np.isfinite(got).all()
            worst = max(worst, rel_l2(got, want))
    print("worst relative L2 over experts:", worst)
    assert worst < TOL, worst


def test_prefill_skips_experts_held_elsewhere_and_matches_decode_kernels(lib, cuda):
    rng = np.random.default_rng(77)
    E, H, I, T, k = 8, 2048, 512, 64, 4
    Lo, blobs = make_expert_blobs(rng, E, O.T_NVFP4, O.T_NVFP4, H, I)
    L = moe.native_expert_layout(40, 40, H, I)
    ids = np.stack([rng.permutation(E)[:k] for _ in range(T)]).astype(np.int32)
    xd = torch.from_numpy(rng.standard_normal((T, H)).astype(np.float32)).cuda().bfloat16()
    bd = dev(stack_blobs(blobs))
    held = np.arange(E) < 4
    dm, cnt, off, src, slot = run_prefill(L, bd, ids, k, E, xd, held=held)
    # the decode kernels on the same dispatch, local experts only
    stride = bd.shape[1]
    table = np.where(held, bd.data_ptr() + np.arange(E, dtype=np.int64) * stride, 0)
    n = ids.size
    ptr = torch.zeros(E + 2, dtype=torch.int64, device="cuda"); start = torch.zeros(E + 2, dtype=torch.int32, device="cuda")
    ng = torch.zeros(1, dtype=torch.int32, device="cuda"); ed = torch.zeros(n, dtype=torch.int32, device="cuda"); et = torch.zeros(n, dtype=torch.int32, device="cuda")
    st = torch.cuda.current_stream().cuda_stream or 1
    dcnt, doff, dsrc, dtab = dev(cnt), dev(off), dev(src), dev(table)     # kept alive until the kernels have run
    capi.check("plan", lib.bsx_plan_groups(dcnt.data_ptr(), doff.data_ptr(), dsrc.data_ptr(), E, dtab.data_ptr(), ptr.data_ptr(),
                                           start.data_ptr(), ng.data_ptr(), ed.data_ptr(), et.data_ptr(), st))
    rows = torch.zeros((n, H), dtype=torch.float32, device="cuda")
    scr = torch.empty(moe.native_expert_scratch_bytes(L, n), dtype=torch.uint8, device="cuda")
    moe.native_expert_grouped(L, ptr, start, ng, ed, et, E, n, xd, scr, rows, n_x_rows=T)
    torch.cuda.synchronize()
    assert int(ng.item()) == 4
    rows = rows.cpu().numpy()
    lo, hi = int(off[0]), int(off[4])
    assert rel_l2(dm[lo:hi], rows[lo:hi]) < 1e-3          # two implementations of the same rows (fp16 h vs fp32 h)
    assert np.all(rows[hi:] == 0)                          # rows of experts held elsewhere are not touched by the decode path


@pytest.mark.parametrize("T,E,H,xdt", [(300, 64, 512, "bf16"), (1000, 512, 2048, "bf16"), (130, 256, 7168, "bf16"), (257, 96, 1024, "f32")])
def test_router_logits_prefill_matches_the_fp32_chain(lib, cuda, T, E, H, xdt):
    """The tensor-core gate product against the fixed-order fp32 chain (bsx_router_logits): every logit within 4e-6 of
    |x_t| |gate_e| (both sums carry fp32 rounding of that order), and the top-k ids equal except where scores tie to it."""
    g = torch.Generator(device="cuda").manual_seed(T + E)
    x = torch.randn((T, H), generator=g, device="cuda")
    x[1] *= 1e-3                       # rows of very different scale: each row has its own power-of-two scale
    x[2] *= 300.0
    x = x.bfloat16() if xdt == "bf16" else x
    gate = torch.randn((E, H), generator=g, device="cuda") * 0.02
    gate[3] *= 50.0
    want = torch.empty((T, E), dtype=torch.float32, device="cuda")
    capi.check("logits", lib.bsx_router_logits_x(x.data_ptr(), moe._x_kind(x), gate.data_ptr(), T, E, H, want.data_ptr(), moe._stream(None)))
    got, status = moe.router_logits_prefill(x, gate)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    bound = x.float().norm(dim=1)[:, None] * gate.norm(dim=1)[None, :]
    err = ((got - want).abs() / bound).max().item()
    print("worst |logit difference| / (|x| |gate|):", err)
    assert err < 4e-6
    a = moe.RouterArgs(n_expert=E, n_embd=H, k=8, weight_scale=1.0, gate=capi.GATE_SOFTMAX)
    ids_w, _ = moe.router_select(want, None, a)
    ids_g, _ = moe.router_select(got, None, a)
    torch.cuda.synchronize()
    same = (ids_w == ids_g).all(dim=1).float().mean().item()
    assert same > 0.99


def run_prefill_packed(L, packed, ids, k, E, x):
    stride = packed.shape[1]
    table = packed.data_ptr() + np.arange(E, dtype=np.int64) * stride
    cnt, off, slot, src, tiles, n_tiles = moe.dispatch(dev(ids.reshape(-1)), k, E, tile_rows=128)
    T, n = x.shape[0], ids.size
    dm = torch.empty((n, L.n_embd), dtype=torch.float32, device="cuda")
    scratch = torch.empty(capi.lib().bsx_experts_prefill_packed_scratch_bytes(C.byref(L), T, n), dtype=torch.uint8, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    tab = dev(table)
    capi.check("prefill packed", capi.lib().bsx_experts_prefill_packed(C.byref(L), tab.data_ptr(), off.data_ptr(), src.data_ptr(), tiles.data_ptr(),
                                                                       n_tiles.data_ptr(), tiles.shape[0], n, x.data_ptr(), moe._x_kind(x), T, E,
                                                                       scratch.data_ptr(), dm.data_ptr(), status.data_ptr(), moe._stream(None)))
    torch.cuda.synchronize()
    assert int(status.item()) == 0, "a bounded wait inside the kernel gave up"
    return dm.cpu().numpy(), cnt.cpu().numpy(), off.cpu().numpy(), src.cpu().numpy()


@pytest.mark.parametrize("E,H,I,T,k,xdt", [(8, 512, 256, 300, 2, "f32"), (16, 2048, 512, 1000, 4, "bf16"), (4, 7168, 2048, 200, 2, "bf16")])
def test_packed_prefill_vs_dequantised_reference(lib, cuda, E, H, I, T, k, xdt):
    """The block-scaled FP4 prompt kernels (packed blobs, four FP4 activation terms) against the dequantised fp32 oracle."""
    rng = np.random.default_rng(E + H + T + 1)
    Lo, blobs = make_expert_blobs(rng, E, O.T_NVFP4, O.T_NVFP4, H, I)
    L = moe.native_expert_layout(40, 40, H, I)
    ids = zipf_ids(rng, T, k, E)
    x = rng.standard_normal((T, H)).astype(np.float32)
    xd = dev(x)
    if xdt == "bf16":
        xd = xd.bfloat16()
        x = xd.float().cpu().numpy()
    packed = moe.pack_experts(L, dev(stack_blobs(blobs)))
    dm, cnt, off, src = run_prefill_packed(L, packed, ids, k, E, xd)
    worst = 0.0
    for e in range(E):
        if cnt[e]:
            want = O.expert_forward(Lo, blobs[e], x[src[off[e]:off[e + 1]]])
            got = dm[off[e]:off[e + 1]]
            assert np.isfinite(got).all()
            worst = max(worst, rel_l2(got, want))
    print("worst relative L2 over experts:", worst)
    assert worst < TOL
