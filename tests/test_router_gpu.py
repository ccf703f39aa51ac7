"""GPU parity of the router: logits bit-exact with the oracle's restatement of the reference summation order; selection
bit-exact with the reference's own CUDA kernels (oracle/_ref/libref_gpu.so, when built) and with the frozen hash of the
reference's router test; the CPU oracle agrees up to near-ties (its libm exp is not the GPU's)."""
import ctypes as C

import numpy as np
import pytest
import torch

from basalt_b200 import capi, moe
from oracle import oracle as O
from tests.helpers import group_near_tie_ok, near_tie_ok

pytestmark = pytest.mark.gpu
REFG = O.ref_gpu() if torch.cuda.is_available() else None
needs_ref = pytest.mark.skipif(REFG is None, reason="oracle/_ref/libref_gpu.so not built")


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def bits(a):
    return np.ascontiguousarray(a).view(np.uint32)


@pytest.mark.parametrize("T,E,H", [(1, 64, 2048), (11, 384, 5120), (64, 512, 2048), (9, 256, 7168), (70, 512, 2560), (300, 64, 128)])
def test_logits_bit_exact(lib, cuda, T, E, H):
    rng = np.random.default_rng(T + E)
    x = rng.standard_normal((T, H)).astype(np.float32)
    g = (rng.standard_normal((E, H)) * 0.02).astype(np.float32)
    got = moe.router_logits(dev(x), dev(g)).cpu().numpy()
    want = O.router_logits(x, g)
    assert np.array_equal(bits(got), bits(want))


@pytest.mark.parametrize("kind", [capi.GATE_SQRT_SOFTPLUS, capi.GATE_SIGMOID])
@pytest.mark.parametrize("E,k", [(384, 6), (256, 8), (64, 8), (512, 16)])
def test_select_vs_oracle_and_reference_kernel(lib, cuda, kind, E, k):
    rng = np.random.default_rng(E + k + kind)
    T = 33
    lg = (rng.standard_normal((T, E)) * 1.5).astype(np.float32)
    lg[5, 7] = lg[5, 3]              # an exact tie
    lg[6, :] = 0.25                  # everything ties
    bias = (rng.standard_normal(E) * 0.05).astype(np.float32)
    bias[7] = bias[3]
    a = moe.RouterArgs(n_expert=E, k=k, weight_scale=2.5, gate=kind)
    ids, w = moe.router_select(dev(lg), dev(bias), a)
    ids, w = ids.cpu().numpy(), w.cpu().numpy()
    oid, ow = O.router_select(lg, bias, k, kind, 2.5)
    lg64 = lg.astype(np.float64)
    s = np.sqrt(np.log1p(np.exp(lg64))) if kind == 0 else 1 / (1 + np.exp(-lg64))
    near_tie_ok(ids, oid, s + bias)       # every row that differs from the libm-based oracle is a near-tie, nothing else
    same = (ids == oid).all(1)
    assert same.any() and np.abs(w[same] - ow[same]).max() < 1e-5
    # with the device's own gate scores the CPU restatement must give the device's bits (no libm in between)
    if REFG is not None:
        sc = torch.zeros((T, E), dtype=torch.float32, device="cuda")
        dl = dev(lg)
        assert REFG.refg_gate_scores(C.c_void_p(dl.data_ptr()), C.c_int64(T * E), kind, C.c_void_p(sc.data_ptr())) == 0
        xid, xw = O.router_select_scores(sc.cpu().numpy(), bias, k, 2.5)
        assert np.array_equal(ids, xid) and np.array_equal(bits(w), bits(xw))
    # all logits and biases equal: the lowest indices win, in order
    zi, _ = moe.router_select(dev(np.full((1, E), 0.25, np.float32)), dev(np.zeros(E, np.float32)), a)
    assert zi.cpu().numpy().tolist() == [list(range(k))]
    if REFG is not None:
        rid = torch.zeros((T, k), dtype=torch.int32, device="cuda")
        rw = torch.zeros((T, k), dtype=torch.float32, device="cuda")
        dlg, dbias = dev(lg), dev(bias)    # keep the device copies alive until the reference kernel has run
        rc = REFG.refg_router_select(C.c_void_p(dlg.data_ptr()), C.c_void_p(dbias.data_ptr()), T, E, k, C.c_float(2.5), kind,
                                     C.c_float(0.0), None, C.c_void_p(rid.data_ptr()), C.c_void_p(rw.data_ptr()))
        assert rc == 0
        assert np.array_equal(ids, rid.cpu().numpy())
        assert np.array_equal(bits(w), bits(rw.cpu().numpy()))


def test_frozen_hash_of_reference_router_test(lib, cuda):
    """src/models/deepseek41/kernels/router_parity.cpp:179-203: 64 tokens at 384 x 5120, k = 6, sqrt-softplus, scale 1.5, plain and
    with every expert twinned; FNV-1a over ids then weights must equal the reference's frozen constant."""
    NE, ND, K = 384, 5120, 6
    gate = O.std_randn(NE * ND, 1, 0.02).reshape(NE, ND)
    bias = O.std_randn(NE, 2, 0.05)
    gate[201] = gate[77]
    bias[201] = bias[77]
    tg, tb = gate.copy(), bias.copy()
    tg[NE // 2:] = tg[:NE // 2]
    tb[NE // 2:] = tb[:NE // 2]
    xs = O.std_randn(64 * ND, 9).reshape(64, ND)
    a = moe.RouterArgs(n_expert=NE, n_embd=ND, k=K, weight_scale=1.5, gate=capi.GATE_SQRT_SOFTPLUS)
    h = 1469598103934665603
    for g_, b_ in ((gate, bias), (tg, tb)):
        _, ids, w = moe.router(dev(xs), dev(g_), dev(b_), a)
        h = O.fnv1a(ids.cpu().numpy(), h=h)
        h = O.fnv1a(w.cpu().numpy(), h=h)
    assert h == 0x3634b0999cf64e2a, hex(h)


@needs_ref
def test_router_whole_call_vs_reference_kernel(lib, cuda):
    rng = np.random.default_rng(77)
    for (T, E, H, k, kind) in ((11, 384, 5120, 6, 0), (64, 256, 7168, 8, 1), (3, 512, 2048, 10, 1)):
        x = dev(rng.standard_normal((T, H)).astype(np.float32))
        g = dev((rng.standard_normal((E, H)) * 0.02).astype(np.float32))
        b = dev((rng.standard_normal(E) * 0.01).astype(np.float32))
        a = moe.RouterArgs(n_expert=E, n_embd=H, k=k, weight_scale=2.5, gate=kind)
        lg, ids, w = moe.router(x, g, b, a)
        rl = torch.zeros_like(lg); rid = torch.zeros_like(ids); rw = torch.zeros_like(w)
        rc = REFG.refg_router(C.c_void_p(x.data_ptr()), C.c_void_p(g.data_ptr()), C.c_void_p(b.data_ptr()), T, E, H, k,
                              C.c_float(2.5), kind, C.c_void_p(rl.data_ptr()), C.c_void_p(rid.data_ptr()), C.c_void_p(rw.data_ptr()))
        assert rc == 0
        assert torch.equal(lg.view(torch.int32), rl.view(torch.int32))
        assert torch.equal(ids, rid)
        assert torch.equal(w.view(torch.int32), rw.view(torch.int32))


def test_window_and_position_independence(lib, cuda):
    rng = np.random.default_rng(5)
    E, H, k = 256, 7168, 8
    x = dev(rng.standard_normal((11, H)).astype(np.float32))
    g = dev((rng.standard_normal((E, H)) * 0.02).astype(np.float32))
    b = dev((rng.standard_normal(E) * 0.01).astype(np.float32))
    a = moe.RouterArgs(n_expert=E, n_embd=H, k=k, weight_scale=2.5, gate=capi.GATE_SIGMOID, n_group=8, topk_group=4)
    lg, ids, w = moe.router(x, g, b, a)
    for T in (1, 2, 3, 4):
        for s0 in (0, 3, 7):
            l2, i2, w2 = moe.router(x[s0:s0 + T].contiguous(), g, b, a)
            assert torch.equal(l2.view(torch.int32), lg[s0:s0 + T].view(torch.int32))
            assert torch.equal(i2, ids[s0:s0 + T]) and torch.equal(w2.view(torch.int32), w[s0:s0 + T].view(torch.int32))


def test_group_limited_selection(lib, cuda):
    rng = np.random.default_rng(6)
    E, k, T = 256, 8, 64
    lg = (rng.standard_normal((T, E)) * 1.5).astype(np.float32)
    bias = (rng.standard_normal(E) * 0.01).astype(np.float32)
    a = moe.RouterArgs(n_expert=E, k=k, weight_scale=2.5, gate=capi.GATE_SIGMOID, n_group=8, topk_group=4)
    ids, w = moe.router_select(dev(lg), dev(bias), a)
    oid, ow = O.router_select(lg, bias, k, 1, 2.5, n_group=8, topk_group=4)
    ids, w = ids.cpu().numpy(), w.cpu().numpy()
    # against the libm-based oracle: a row may differ only through a near-tie of expert scores or of group scores
    s64 = 1 / (1 + np.exp(-lg.astype(np.float64))) + bias
    group_near_tie_ok(ids, oid, s64, 8, 4)
    same = (ids == oid).all(1)
    assert same.any() and np.abs(w[same] - ow[same]).max() < 1e-5
    # with the device's own sigmoid values the CPU restatement of the group step, the ranks and the weights is exact
    if REFG is not None:
        for (ng, tg, kk) in ((8, 4, 8), (8, 1, 8), (4, 2, 6), (32, 3, 8), (8, 7, 16)):
            a2 = moe.RouterArgs(n_expert=E, k=kk, weight_scale=2.5, gate=capi.GATE_SIGMOID, n_group=ng, topk_group=tg)
            lg2 = lg.copy()
            lg2[7, :] = 0.5                       # every expert and every group ties
            lg2[9, 32:64] = lg2[9, 0:32]          # two identical groups
            dl = dev(lg2)
            i2, w2 = moe.router_select(dl, dev(bias * 0 if ng == 32 else bias), a2)
            sc = torch.zeros((T, E), dtype=torch.float32, device="cuda")
            assert REFG.refg_gate_scores(C.c_void_p(dl.data_ptr()), C.c_int64(T * E), 1, C.c_void_p(sc.data_ptr())) == 0
            xid, xw = O.router_select_scores(sc.cpu().numpy(), bias * 0 if ng == 32 else bias, kk, 2.5, n_group=ng, topk_group=tg)
            assert np.array_equal(i2.cpu().numpy(), xid), (ng, tg)
            assert np.array_equal(bits(w2.cpu().numpy()), bits(xw)), (ng, tg)
    # n_group = 1 (and topk_group = n_group) is the plain selection bit for bit
    p = moe.router_select(dev(lg), dev(bias), moe.RouterArgs(n_expert=E, k=k, weight_scale=2.5, gate=capi.GATE_SIGMOID))
    for ng, tg in ((1, 1), (8, 8)):
        q = moe.router_select(dev(lg), dev(bias), moe.RouterArgs(n_expert=E, k=k, weight_scale=2.5, gate=capi.GATE_SIGMOID, n_group=ng, topk_group=tg))
        assert torch.equal(p[0], q[0]) and torch.equal(p[1].view(torch.int32), q[1].view(torch.int32))
    # a group-tie: two identical groups, the lower one wins
    lg2 = np.full((1, 64), -3.0, np.float32)
    lg2[0, 16:32] = 1.0
    lg2[0, 48:64] = 1.0
    i2, _ = moe.router_select(dev(lg2), dev(np.zeros(64, np.float32)), moe.RouterArgs(n_expert=64, k=4, gate=capi.GATE_SIGMOID, n_group=4, topk_group=1))
    assert i2.cpu().numpy().tolist() == [[16, 17, 18, 19]]


@pytest.mark.parametrize("E,k", [(512, 10), (256, 10), (64, 8), (96, 4), (1024, 32)])
def test_softmax_routers(lib, cuda, E, k):
    rng = np.random.default_rng(E)
    T = 37
    lg = (rng.standard_normal((T, E)) * 2).astype(np.float32)
    lg[3] = 0.0
    lg[4, 10:20] = 50.0
    # the tie cases of the reference's own router test (tests/models/qwen4exp/kernels/router_top10_parity.cpp:125-140): every
    # expert equal, a 12-way exact tie among otherwise distinct values, one dominant expert
    lg[5] = 0.5
    lg[6, :12] = 2.0
    lg[7] = 0.0
    lg[7, 21] = 20.0
    lg[8, 32:44] = lg[8, 0:12]        # equal values on different lanes' second registers
    outs = {}
    for kind in (capi.GATE_SOFTMAX, capi.GATE_SOFTMAX_FAST, capi.GATE_SOFTMAX_F64):
        ids, w = moe.router_select(dev(lg), None, moe.RouterArgs(n_expert=E, k=k, gate=kind))
        outs[kind] = (ids.cpu().numpy(), w.cpu().numpy())
    oid, ow = O.router_select(lg, None, k, O.GATE_SOFTMAX)
    lg64 = lg.astype(np.float64)
    p64 = np.exp(lg64 - lg64.max(1, keepdims=True))
    p64 /= p64.sum(1, keepdims=True)
    for kind, (ids, w) in outs.items():
        near_tie_ok(ids, oid, p64)      # rows that differ from the libm-based oracle: probabilities within 1e-5 of the k-th only
        same = (ids == oid).all(1)
        assert same.any(), kind
        assert np.abs(w[same] - ow[same]).max() < (1e-3 if kind == capi.GATE_SOFTMAX_FAST else 1e-5)
        assert ids[3].tolist() == list(range(k))
        assert sorted(ids[4][:10].tolist()) == list(range(10, 20)) if k >= 10 else True
    if REFG is not None:
        rid = torch.zeros((T, k), dtype=torch.int32, device="cuda"); rw = torch.zeros((T, k), dtype=torch.float32, device="cuda")
        dlg = dev(lg)
        # the gate kind the layer runs by default: ids and weight bits of the prompt path's route_kernel (512 / 256 experts with
        # k = 10 are its own instantiations; the other sizes run the same sequence)
        if E != 96 or hasattr(REFG, "refg_route_softmax"):
            assert REFG.refg_route_softmax(C.c_void_p(dlg.data_ptr()), C.c_int64(T), E, k, C.c_void_p(rid.data_ptr()), C.c_void_p(rw.data_ptr())) == 0
            ids, w = outs[capi.GATE_SOFTMAX]
            assert np.array_equal(ids, rid.cpu().numpy())
            assert np.array_equal(bits(w), bits(rw.cpu().numpy()))
        assert REFG.refg_router_top10(C.c_void_p(dlg.data_ptr()), T, E, k, C.c_void_p(rid.data_ptr()), C.c_void_p(rw.data_ptr())) == 0
        ids, w = outs[capi.GATE_SOFTMAX_F64]
        assert np.array_equal(ids, rid.cpu().numpy())
        assert np.array_equal(bits(w), bits(rw.cpu().numpy()))
        if E == 512 and k == 10:
            assert REFG.refg_native_router_top10(C.c_void_p(dlg.data_ptr()), T, C.c_void_p(rid.data_ptr()), C.c_void_p(rw.data_ptr())) == 0
            ids, w = outs[capi.GATE_SOFTMAX_FAST]
            assert np.array_equal(ids, rid.cpu().numpy())
            assert np.array_equal(bits(w), bits(rw.cpu().numpy()))


def test_tail_skip(lib, cuda):
    rng = np.random.default_rng(12)
    E, k, T = 64, 8, 16
    ids = np.stack([rng.permutation(E)[:k] for _ in range(T)]).astype(np.int32)
    w = rng.random((T, k)).astype(np.float32)
    w /= w.sum(1, keepdims=True)
    held = np.where(rng.random(E) < 0.5, 0, -1).astype(np.int32)
    for rank in (0, 1, 3, 7, 8):
        di, dw, dh = dev(ids.copy()), dev(w.copy()), dev(held)
        counts = torch.zeros(3, dtype=torch.int64, device="cuda")
        moe.route_tail_skip(di, dw, [dh], k, rank, E, counts)
        oi, ow, oc = O.route_tail_skip(ids, w, held, k, rank, E)
        assert np.array_equal(di.cpu().numpy(), oi) and np.array_equal(bits(dw.cpu().numpy()), bits(ow))
        assert counts.cpu().numpy().tolist() == oc.astype(np.int64).tolist()
        if REFG is not None:
            ri, rw = dev(ids.copy()), dev(w.copy())
            rcnt = torch.zeros(3, dtype=torch.int64, device="cuda")
            assert REFG.refg_route_tail_skip(C.c_void_p(ri.data_ptr()), C.c_void_p(rw.data_ptr()), C.c_void_p(dh.data_ptr()), T * k, k, rank, E,
                                             C.c_void_p(rcnt.data_ptr())) == 0
            assert torch.equal(ri, di) and torch.equal(rw, dw) and torch.equal(rcnt, counts)
