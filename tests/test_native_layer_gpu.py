"""GPU: the one-call layer step (bsx_moe_layer), the fused selection + plan launch (bsx_route_plan), the staged router-logits
kernel and the combine with a residual row - each against the separate calls it replaces, bit for bit, and the whole step
against the CPU oracle."""
import ctypes as C

import numpy as np
import pytest
import torch

from basalt_b200 import capi, moe
from oracle import oracle as O
from tests.helpers import make_expert_blobs, rel_l2, stack_blobs

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def bits(t):
    return t.contiguous().view(torch.int32)


@pytest.mark.parametrize("E,k,kind,T,shared", [(512, 10, capi.GATE_SOFTMAX, 64, True), (256, 8, capi.GATE_SIGMOID, 64, True), (64, 8, capi.GATE_SOFTMAX, 5, False),
                                               (384, 6, capi.GATE_SQRT_SOFTPLUS, 33, False), (1024, 1, capi.GATE_SOFTMAX, 64, True)])
def test_route_plan_equals_select_then_plan(lib, cuda, E, k, kind, T, shared):
    rng = np.random.default_rng(E + k)
    lg = (rng.standard_normal((T, E)) * 1.5).astype(np.float32)
    lg[0] = 0.25                                   # every expert ties
    lg[min(3, T - 1), :12] = 2.0
    bias = None if kind == capi.GATE_SOFTMAX else dev((rng.standard_normal(E) * 0.01).astype(np.float32))
    grouped = kind == capi.GATE_SIGMOID
    a = moe.RouterArgs(n_expert=E, k=k, weight_scale=2.5 if grouped else 1.0, gate=kind, n_group=8 if grouped else 1, topk_group=4 if grouped else 1)
    table = np.arange(1, E + 1, dtype=np.int64) * 4096
    table[5] = 0                                   # an expert this device does not hold: its pairs get no entry
    tab = dev(table)
    dl = dev(lg)
    ids, w = moe.router_select(dl, bias, a)
    n = T * k
    ptr = torch.zeros(n + 3, dtype=torch.int64, device="cuda"); start = torch.zeros(n + 3, dtype=torch.int32, device="cuda")
    ng = torch.zeros(1, dtype=torch.int32, device="cuda")
    dst = torch.zeros(n + T, dtype=torch.int32, device="cuda"); tok = torch.zeros(n + T, dtype=torch.int32, device="cuda")
    sb = 77 * 4096 if shared else 0
    moe.check("plan", lib.bsx_moe_plan_shared(ids.data_ptr(), T, k, E, tab.data_ptr(), sb, ptr.data_ptr(), start.data_ptr(), ng.data_ptr(), dst.data_ptr(),
                                               tok.data_ptr(), torch.cuda.current_stream().cuda_stream or 1))
    fi, fw, fptr, fstart, fng, fdst, ftok = moe.route_plan(dl, bias, a, tab, sb)
    torch.cuda.synchronize()
    assert torch.equal(fi, ids) and torch.equal(bits(fw), bits(w))
    g = int(ng.item())
    assert int(fng.item()) == g
    assert torch.equal(fptr[:g], ptr[:g]) and torch.equal(fstart[:g + 2], start[:g + 2])
    rows = int(start[g].item())
    assert torch.equal(fdst[:rows], dst[:rows]) and torch.equal(ftok[:rows], tok[:rows])


@pytest.mark.parametrize("T,E,H,dt", [(64, 512, 2048, "bf16"), (64, 512, 2048, "f32"), (17, 64, 1024, "bf16"), (40, 256, 4096, "bf16"), (100, 96, 512, "f32")])
def test_staged_logits_are_the_same_bits_whatever_the_window(lib, cuda, T, E, H, dt):
    rng = np.random.default_rng(T + H)
    x = torch.from_numpy(rng.standard_normal((T, H)).astype(np.float32)).cuda()
    if dt == "bf16":
        x = x.bfloat16()
    g = dev((rng.standard_normal((E, H)) * 0.02).astype(np.float32))
    a = moe.RouterArgs(n_expert=E, n_embd=H, k=4, gate=capi.GATE_SOFTMAX)
    full, _, _ = moe.router_x(x, g, None, a)          # T >= 16: the staged kernel
    want = O.router_logits(x.float().cpu().numpy(), g.cpu().numpy())
    assert np.array_equal(full.cpu().numpy().view(np.uint32), want.view(np.uint32))
    for t0, n in ((0, 1), (5, 3), (T - 8, 8)):             # short windows take the plain kernel: same bits
        part, _, _ = moe.router_x(x[t0:t0 + n].contiguous(), g, None, a)
        assert torch.equal(bits(part), bits(full[t0:t0 + n]))


def test_combine_with_residual(lib, cuda):
    rng = np.random.default_rng(3)
    T, k, H = 9, 6, 512
    rows = dev(rng.standard_normal((T * k, H)).astype(np.float32))
    w = dev(rng.random((T, k)).astype(np.float32))
    sh = dev(rng.standard_normal((T, H)).astype(np.float32))
    res = dev(rng.standard_normal((T, H)).astype(np.float32))
    y0 = moe.moe_combine(rows, None, w, sh)
    y1 = moe.moe_combine(rows, None, w, sh, residual=res)
    assert torch.equal(bits(y1), bits(y0 + res))
    y2 = res.clone()
    moe.moe_combine(rows, None, w, sh, y=y2, residual=y2)      # in place on the residual stream
    assert torch.equal(bits(y2), bits(y1))


def _layers(rng, E, H, I, k, kind, gt, dt, shared, packed, T, grouped, sgt=None):
    Lo, blobs = make_expert_blobs(rng, E + (1 if shared and sgt is None else 0), gt, dt, H, I)
    gate_w = dev((rng.standard_normal((E, H)) * 0.02).astype(np.float32))
    bias = dev((rng.standard_normal(E) * 0.01).astype(np.float32)) if grouped else None
    args = moe.RouterArgs(n_expert=E, n_embd=H, k=k, weight_scale=2.5 if grouped else 1.0, gate=kind, n_group=8 if grouped else 1, topk_group=4 if grouped else 1)
    L = moe.native_expert_layout(gt, dt, H, I)
    bd = dev(stack_blobs(blobs))
    sL = sblob = None
    if shared and sgt is not None:
        _, sb = make_expert_blobs(rng, 1, sgt, sgt, H, I)
        sblob = dev(stack_blobs(sb))[0]
        sL = moe.native_expert_layout(sgt, sgt, H, I)
    if packed:
        bd = moe.pack_experts(L, bd)
    if shared and sgt is None:
        sblob = bd[E]
    kw = dict(shared_blob=sblob, shared_layout=sL, max_tokens=T, packed=packed)
    return moe.MoELayer(gate_w, bias, bd[:E], L, args, **kw), moe.NativeMoELayer(gate_w, bias, bd[:E], L, args, **kw)


@pytest.mark.parametrize("name,E,H,I,k,kind,gt,dt,shared,packed,T,sgt", [
    ("flash_next_packed", 128, 2048, 512, 10, capi.GATE_SOFTMAX, 40, 40, True, True, 64, None),
    ("flash_next_packed_1", 128, 2048, 512, 10, capi.GATE_SOFTMAX, 40, 40, True, True, 1, None),
    ("deepseek_packed", 64, 1024, 512, 8, capi.GATE_SIGMOID, 40, 40, True, True, 19, None),
    ("nvfp4_in_place", 64, 2048, 512, 8, capi.GATE_SOFTMAX, 40, 40, True, False, 16, None),
    ("q6k_no_shared", 64, 2048, 512, 8, capi.GATE_SOFTMAX, 14, 14, False, False, 16, None),
    ("iq1m_q6k_shared", 32, 1024, 512, 4, capi.GATE_SIGMOID, 29, 29, True, False, 7, 14),
])
def test_one_call_layer_equals_the_call_by_call_layer(lib, cuda, name, E, H, I, k, kind, gt, dt, shared, packed, T, sgt):
    rng = np.random.default_rng(len(name))
    ref, nat = _layers(rng, E, H, I, k, kind, gt, dt, shared, packed, T, kind == capi.GATE_SIGMOID, sgt)
    x = torch.from_numpy(rng.standard_normal((T, H)).astype(np.float32)).cuda().bfloat16()
    res = torch.from_numpy(rng.standard_normal((T, H)).astype(np.float32)).cuda()
    y0 = ref.forward(x).clone()
    y1 = nat.forward(x).clone()
    nat.check_status()
    assert torch.equal(nat.ids[:T], ref.ids[:T]) and torch.equal(bits(nat.w[:T]), bits(ref.w[:T]))
    assert torch.equal(bits(nat.logits[:T]), bits(ref.logits[:T]))
    assert torch.equal(bits(y1), bits(y0))                       # the same kernels in the same order: the same bits
    y2 = nat.forward(x, residual=res).clone()
    assert torch.equal(bits(y2), bits(y0 + res))
    # plain launches and programmatic dependent launches give the same result; so does a captured graph of the call
    flat = moe.NativeMoELayer(nat.gate_w, nat.bias, nat.blobs, nat.L, nat.args, shared_blob=nat.shared_blob,
                              shared_layout=ref.shared_L if sgt is not None else None, max_tokens=T, packed=packed, pdl=False)
    assert torch.equal(bits(flat.forward(x)), bits(y0))
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        nat.capture(x)
        yg = nat.forward_graphed(x).clone()
        yg2 = nat.forward_graphed(x).clone()
    st.synchronize()
    nat.check_status()
    assert torch.equal(bits(yg[:T]), bits(y0)) and torch.equal(bits(yg2[:T]), bits(y0))


def test_one_call_layer_with_input_norm_vs_oracle(lib, cuda):
    rng = np.random.default_rng(11)
    E, H, I, k, T = 64, 2048, 512, 10, 24
    Lo, blobs = make_expert_blobs(rng, E + 1, 40, 40, H, I)
    gate_w = (rng.standard_normal((E, H)) * 0.02).astype(np.float32)
    nw = (1.0 + 0.1 * rng.standard_normal(H)).astype(np.float32)
    L = moe.native_expert_layout(40, 40, H, I)
    packed = moe.pack_experts(L, dev(stack_blobs(blobs)))
    args = moe.RouterArgs(n_expert=E, n_embd=H, k=k, weight_scale=1.0, gate=capi.GATE_SOFTMAX)
    nat = moe.NativeMoELayer(dev(gate_w), None, packed[:E], L, args, shared_blob=packed[E], max_tokens=T, packed=True, norm_w=dev(nw), norm_eps=1e-6)
    x = rng.standard_normal((T, H)).astype(np.float32) * 3.0
    y = nat.forward(dev(x)).cpu().numpy()
    nat.check_status()
    xn, _ = O.norm_pack(x, nw, 1e-6)
    ids, w = nat.ids[:T].cpu().numpy(), nat.w[:T].cpu().numpy()
    cnt, off, slot, src, _ = O.dispatch(ids, k, E)
    rows = np.zeros((T * k, H), np.float32)
    for e in range(E):
        if cnt[e]:
            rows[off[e]:off[e + 1]] = O.expert_forward(Lo, blobs[e], xn[src[off[e]:off[e + 1]]])
    want = O.combine(rows, slot, w, O.expert_forward(Lo, blobs[E], xn))
    assert rel_l2(y, want) < 2e-3, rel_l2(y, want)


def test_one_call_layer_wide_window_with_a_shared_expert_of_its_own_format(lib, cuda):
    """24 tokens, IQ1_M routed experts, a Q6_K shared expert with a layout of its own, through the one-call step: the rows sit
    on the call-by-call layer's (same kernels)."""
    rng = np.random.default_rng(8)
    E, H, I, k, T = 32, 1024, 512, 4, 24
    ref, nat = _layers(rng, E, H, I, k, capi.GATE_SIGMOID, 29, 29, True, False, T, True, 14)
    x = torch.from_numpy(rng.standard_normal((T, H)).astype(np.float32)).cuda().bfloat16()
    y0 = ref.forward(x).clone()
    y1 = nat.forward(x).clone()
    nat.check_status()
    assert torch.equal(nat.ids[:T], ref.ids[:T])
    assert rel_l2(y1.cpu().numpy(), y0.cpu().numpy()) < 1e-3


@pytest.mark.parametrize("packed", [False, True])
def test_expert_parallel_step_emulated_on_one_gpu(lib, cuda, packed):
    """The expert-parallel decode step's device side (bsx_ep_plan -> grouped experts -> bsx_combine_partial_ep) with the ranks
    emulated one after the other on one GPU: W = 4 ranks' gathered rows and routing in the layout the all-gathers leave, each
    rank holding a quarter of the experts; the sum of the ranks' partial rows (what the reduce-scatter forms) must equal the
    single-GPU layer's rows to fp32 rounding."""
    rng = np.random.default_rng(31)
    E, H, I, k, T, W = 64, 2048, 512, 10, 8, 4
    Lo, blobs = make_expert_blobs(rng, E + 1, 40, 40, H, I)
    L = moe.native_expert_layout(40, 40, H, I)
    bd = dev(stack_blobs(blobs))
    if packed:
        bd = moe.pack_experts(L, bd)
    gate_w = dev((rng.standard_normal((E, H)) * 0.02).astype(np.float32))
    args = moe.RouterArgs(n_expert=E, n_embd=H, k=k, weight_scale=1.0, gate=capi.GATE_SOFTMAX)
    x_all = torch.from_numpy(rng.standard_normal((W * T, H)).astype(np.float32)).cuda().bfloat16()
    single = moe.MoELayer(gate_w, None, bd[:E], L, args, shared_blob=bd[E], max_tokens=W * T, packed=packed)
    want = single.forward(x_all).clone()
    ids_all, w_all = single.ids[:W * T].clone(), single.w[:W * T].clone()
    # the all-gather's layout: per rank [ids T x k | weight bits T x k]
    route_all = torch.empty(W * 2 * T * k, dtype=torch.int32, device="cuda")
    for r in range(W):
        route_all[r * 2 * T * k:r * 2 * T * k + T * k] = ids_all[r * T:(r + 1) * T].reshape(-1)
        route_all[r * 2 * T * k + T * k:(r + 1) * 2 * T * k] = w_all[r * T:(r + 1) * T].reshape(-1).view(torch.int32)
    n = W * T * k
    st = torch.cuda.current_stream().cuda_stream or 1
    stride = bd.shape[1]
    total = torch.zeros((W * T, H), dtype=torch.float32, device="cuda")
    for r in range(W):
        lo, hi = r * E // W, (r + 1) * E // W
        table = np.zeros(E, np.int64)
        table[lo:hi] = bd.data_ptr() + np.arange(lo, hi, dtype=np.int64) * stride
        tab = dev(table)
        ptr = torch.zeros(E + 3, dtype=torch.int64, device="cuda"); start = torch.zeros(E + 3, dtype=torch.int32, device="cuda")
        ng = torch.zeros(1, dtype=torch.int32, device="cuda")
        ed = torch.zeros(n + T, dtype=torch.int32, device="cuda"); et = torch.zeros(n + T, dtype=torch.int32, device="cuda")
        moe.check("bsx_ep_plan", lib.bsx_ep_plan(route_all.data_ptr(), n, k, T * k, 2 * T * k, E, tab.data_ptr(), bd[E].data_ptr(), r * T, T, None, ptr.data_ptr(),
                                                  start.data_ptr(), ng.data_ptr(), ed.data_ptr(), et.data_ptr(), st))
        rows = torch.full((n + T, H), float("nan"), dtype=torch.float32, device="cuda")
        if packed:
            scratch = torch.empty(lib.bsx_experts_packed_scratch_bytes(C.byref(L), n + T), dtype=torch.uint8, device="cuda")
            status = torch.zeros(1, dtype=torch.int32, device="cuda")
            moe.native_expert_grouped_packed(L, ptr, start, ng, ed, et, hi - lo + 1, n + T, x_all, scratch, rows, status, n_x_rows=W * T)
            assert int(status.item()) == 0
        else:
            scratch = torch.empty(moe.native_expert_scratch_bytes(L, n + T), dtype=torch.uint8, device="cuda")
            moe.native_expert_grouped(L, ptr, start, ng, ed, et, hi - lo + 1, n + T, x_all, scratch, rows, n_x_rows=W * T)
        y_part = torch.empty((W * T, H), dtype=torch.float32, device="cuda")
        moe.check("bsx_combine_partial_ep", lib.bsx_combine_partial_ep(rows.data_ptr(), route_all.data_ptr() + 4 * T * k, route_all.data_ptr(), T, 2 * T * k, lo, hi,
                                                                        W * T, k, H, rows[n:].data_ptr(), r * T, T, None, y_part.data_ptr(), st))
        torch.cuda.synchronize()
        g = int(ng.item())
        # the groups are this rank's experts with pairs, ascending, plus the shared group; every local pair has exactly one entry
        local = ((ids_all >= lo) & (ids_all < hi)).reshape(-1)
        rows_used = int(start[g].item())
        assert rows_used == int(local.sum().item()) + T
        assert sorted(ed[:rows_used - T].tolist()) == torch.nonzero(local).reshape(-1).tolist()
        assert torch.equal(et[:rows_used - T], ed[:rows_used - T] // k)
        assert torch.isfinite(y_part).all()
        total += y_part
    assert rel_l2(total.cpu().numpy(), want.cpu().numpy()) < 2e-6
