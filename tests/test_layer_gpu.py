"""GPU: the whole layer through the host-side mirror (router -> plan -> grouped experts -> combine, plus the shared
expert) against the oracle's CPU layer on the same seeded inputs: routing ids, counts and offsets bit-exact, layer output
within relative L2 2e-3 of the fp32-accumulated dequantised reference."""
import numpy as np
import pytest
import torch

from basalt_b200 import capi, moe
from oracle import oracle as O
from tests.helpers import group_near_tie_ok, make_expert_blobs, near_tie_ok, rel_l2, stack_blobs

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def build_layer(rng, E, H, I, k, gate_kind, gt, dt, shared, n_group=1, topk_group=1, scale=1.0, bias_sigma=0.0):
    Lo, blobs = make_expert_blobs(rng, E + (1 if shared else 0), gt, dt, H, I)
    gate_w = (rng.standard_normal((E, H)) * 0.02).astype(np.float32)
    bias = (rng.standard_normal(E) * bias_sigma).astype(np.float32) if bias_sigma else None
    args = moe.RouterArgs(n_expert=E, n_embd=H, k=k, weight_scale=scale, gate=gate_kind, n_group=n_group, topk_group=topk_group)
    L = moe.native_expert_layout(gt, dt, H, I)
    bd = dev(stack_blobs(blobs))
    layer = moe.MoELayer(dev(gate_w), None if bias is None else dev(bias), bd[:E], L, args, shared_blob=bd[E] if shared else None)
    return layer, Lo, blobs, gate_w, bias


@pytest.mark.parametrize("name,E,H,I,k,kind,gt,dt,shared,T", [
    ("cpu_reference_config", 64, 2048, 512, 8, capi.GATE_SOFTMAX, 14, 14, False, 16),       # the CPU offload path's layer: Q6_K, 64 experts
    ("flash_next_decode_small", 64, 2048, 512, 10, capi.GATE_SOFTMAX, 40, 40, True, 8),      # the flash-next-style layer with fewer experts
    ("deepseek_shape_small", 32, 1024, 512, 8, capi.GATE_SIGMOID, 40, 40, True, 11),
    ("iq1m_routed", 32, 1024, 512, 4, capi.GATE_SIGMOID, 29, 29, False, 5),
])
def test_layer_vs_oracle(lib, cuda, name, E, H, I, k, kind, gt, dt, shared, T):
    rng = np.random.default_rng(0)
    grouped = kind == capi.GATE_SIGMOID
    layer, Lo, blobs, gate_w, bias = build_layer(rng, E, H, I, k, kind, gt, dt, shared, n_group=8 if grouped else 1,
                                                 topk_group=4 if grouped else 1, scale=2.5 if grouped else 1.0,
                                                 bias_sigma=0.01 if grouped else 0.0)
    x = rng.standard_normal((T, H)).astype(np.float32)
    y = layer.forward(dev(x)).cpu().numpy()
    ids = layer.ids[:T].cpu().numpy()
    oy, oids, ow, ocnt, ooff, oslot, osrc = O.moe_layer(x, gate_w, bias, blobs[:E], Lo, k, O.GATE_SOFTMAX if kind == capi.GATE_SOFTMAX else kind,
                                                       scale=layer.args.weight_scale, n_group=layer.args.n_group,
                                                       topk_group=layer.args.topk_group, shared_blob=blobs[E] if shared else None)
    # logits carry the oracle's bits; a row whose ids differ from the libm-based oracle may differ only through a near-tie
    lg = O.router_logits(x, gate_w)
    assert np.array_equal(lg.view(np.uint32), layer.logits[:T].cpu().numpy().view(np.uint32))
    lg64 = lg.astype(np.float64)
    if kind == capi.GATE_SOFTMAX:
        p64 = np.exp(lg64 - lg64.max(1, keepdims=True))
        near_tie_ok(ids, oids, p64 / p64.sum(1, keepdims=True))
    else:
        group_near_tie_ok(ids, oids, 1 / (1 + np.exp(-lg64)) + (bias if bias is not None else 0.0), layer.args.n_group, layer.args.topk_group)
    w = layer.w[:T].cpu().numpy()
    cnt, off, slot, src, _ = O.dispatch(ids, k, E)
    rows = np.zeros((T * k, H), np.float32)
    for e in range(E):
        if cnt[e]:
            rows[off[e]:off[e + 1]] = O.expert_forward(Lo, blobs[e], x[src[off[e]:off[e + 1]]])
    sh = O.expert_forward(Lo, blobs[E], x) if shared else None
    want = O.combine(rows, slot, w, sh)
    assert rel_l2(y, want) < 2e-3, rel_l2(y, want)
    # device-side dispatch of the same ids: counts and offsets bit-exact
    dcnt, doff, dslot, dsrc, _, _ = moe.dispatch(layer.ids[:T].reshape(-1).contiguous(), k, E)
    assert np.array_equal(dcnt.cpu().numpy(), cnt) and np.array_equal(doff.cpu().numpy(), off) and np.array_equal(dslot.cpu().numpy(), slot)


def test_layer_bf16_activations_and_repeatability(lib, cuda):
    rng = np.random.default_rng(1)
    E, H, I, k, T = 64, 2048, 512, 10, 64
    layer, Lo, blobs, gate_w, _ = build_layer(rng, E, H, I, k, capi.GATE_SOFTMAX, 40, 40, True)
    x = torch.from_numpy(rng.standard_normal((T, H)).astype(np.float32)).cuda().bfloat16()
    y1 = layer.forward(x).clone()
    y2 = layer.forward(x).clone()
    assert torch.equal(y1.view(torch.int32), y2.view(torch.int32))      # gather combine: bit-stable run to run
    xe = x.float().cpu().numpy()
    ids, w = layer.ids[:T].cpu().numpy(), layer.w[:T].cpu().numpy()
    cnt, off, slot, src, _ = O.dispatch(ids, k, E)
    rows = np.zeros((T * k, H), np.float32)
    for e in range(E):
        if cnt[e]:
            rows[off[e]:off[e + 1]] = O.expert_forward(Lo, blobs[e], xe[src[off[e]:off[e + 1]]])
    want = O.combine(rows, slot, w, O.expert_forward(Lo, blobs[E], xe))
    assert rel_l2(y1.cpu().numpy(), want) < 2e-3
