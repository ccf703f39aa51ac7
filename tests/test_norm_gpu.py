"""GPU: the step before the layer, the RMS norm of the input rows (bsx_norm_pack) - bit-exact with the reference's own
norm_pack kernel (oracle/_ref/libref_gpu.so, compiled from the reference's window_gemm.cu), within 4 ulp of the numpy
restatement (the device's rsqrtf is an approximation) - and its fusion with the FP4 activation images of the packed expert
path: a layer given un-normed rows and the norm weights returns the bits of the norm followed by the plain layer."""
import numpy as np
import pytest
import torch

from basalt_b200 import capi, moe
from oracle import oracle as O
from tests.helpers import make_expert_blobs, stack_blobs

pytestmark = pytest.mark.gpu
REFG = O.ref_gpu() if torch.cuda.is_available() else None
needs_ref = pytest.mark.skipif(REFG is None or not hasattr(REFG, "refg_norm_pack"), reason="oracle/_ref/libref_gpu.so not built")


def inputs(T, K, seed, bf16):
    rng = np.random.default_rng(seed)
    x = (rng.standard_normal((T, K)) * rng.uniform(0.05, 30.0, size=(T, 1))).astype(np.float32)
    w = (1.0 + 0.2 * rng.standard_normal(K)).astype(np.float32)
    xd = torch.from_numpy(x).cuda()
    if bf16:
        xd = xd.bfloat16()
    return xd, torch.from_numpy(w).cuda()


@needs_ref
@pytest.mark.parametrize("bf16", [False, True])
@pytest.mark.parametrize("T,K", [(5, 2048), (64, 7168), (3, 8192), (2, 12288), (7, 96), (1, 2560)])
def test_norm_pack_has_the_reference_kernels_bits(lib, cuda, T, K, bf16):
    x, w = inputs(T, K, 100 + K, bf16)
    act, xn = moe.norm_pack(x, w, 1e-6)
    act_r = torch.empty_like(act)
    xn_r = torch.empty_like(xn)
    assert REFG.refg_norm_pack(x.data_ptr(), int(bf16), w.data_ptr(), 1e-6, K, T, act_r.data_ptr(), xn_r.data_ptr()) == 0
    torch.cuda.synchronize()
    assert torch.equal(xn.view(torch.int32), xn_r.view(torch.int32))
    assert torch.equal(act.view(torch.int16), act_r.view(torch.int16))
    only_act, none = moe.norm_pack(x, w, 1e-6, xn=False)
    assert none is None and torch.equal(only_act.view(torch.int16), act_r.view(torch.int16))


@pytest.mark.parametrize("T,K", [(4, 2048), (3, 7168), (2, 12288)])
def test_norm_pack_vs_numpy_restatement(lib, cuda, T, K):
    x, w = inputs(T, K, 7 + K, False)
    act, xn = moe.norm_pack(x, w, 1e-5)
    want_xn, want_act = O.norm_pack(x.cpu().numpy(), w.cpu().numpy(), 1e-5)
    got = xn.cpu().numpy()
    ulp = np.abs(got.view(np.int32).astype(np.int64) - want_xn.view(np.int32).astype(np.int64))
    assert ulp.max() <= 4, ulp.max()                       # tolerance: 4 units in the last place of fp32 (rsqrtf: 2, two products: 1 each)
    off = act.view(torch.int16).cpu().numpy().view(np.uint16).astype(np.int64) - want_act.astype(np.int64)
    assert np.abs(off).max() <= 1 and (off != 0).mean() < 0.01


@pytest.mark.parametrize("packed", [True, False])
def test_layer_with_its_input_norm_equals_norm_then_layer(lib, cuda, packed):
    rng = np.random.default_rng(21)
    E, H, I, K, T = 64, 2048, 512, 6, 40
    _, blobs = make_expert_blobs(rng, E + 1, O.T_NVFP4, O.T_NVFP4, H, I)
    L = moe.native_expert_layout(40, 40, H, I)
    bd = torch.from_numpy(stack_blobs(blobs)).cuda()
    if packed:
        bd = moe.pack_experts(L, bd)
    gate = torch.from_numpy((rng.standard_normal((E, H)) * 0.02).astype(np.float32)).cuda()
    args = moe.RouterArgs(n_expert=E, n_embd=H, k=K, weight_scale=1.0, gate=capi.GATE_SOFTMAX)
    x, w = inputs(T, H, 5, True)
    plain = moe.MoELayer(gate, None, bd[:E], L, args, shared_blob=bd[E], max_tokens=64, packed=packed)
    fused = moe.MoELayer(gate, None, bd[:E], L, args, shared_blob=bd[E], max_tokens=64, packed=packed, norm_w=w, norm_eps=1e-6)
    _, xn = moe.norm_pack(x, w, 1e-6, act=False)
    want = plain.forward(xn).clone()
    got = fused.forward(x).clone()
    torch.cuda.synchronize()
    assert torch.isfinite(got).all()
    assert torch.equal(got.view(torch.int32), want.view(torch.int32))
    assert torch.equal(fused.ids[:T], plain.ids[:T])
    if packed:
        assert int(fused.status.item()) == 0
        x64, _ = inputs(64, H, 6, True)
        eager = fused.forward(x64).clone()
        fused.capture(x64)
        again = fused.forward_graphed(x64).clone()
        torch.cuda.synchronize()
        assert torch.equal(eager.view(torch.int32), again.view(torch.int32))
