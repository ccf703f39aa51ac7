"""GPU: the MoE layer at the full shapes of the benchmark's workloads, checked against the CPU oracle on a seeded sample.

  * flash-next-style decode layer: hidden 2048, 512 routed + 1 shared NVFP4 experts of 512, softmax top-10, bf16 rows,
    1 / 8 / 64 tokens, blobs packed into planes (the block-scaled FP4 tensor-core path);
  * v4-flash / DeepSeek-style decode layer: hidden 7168, 256 + 1 NVFP4 experts of 2048, sigmoid + bias, 8 groups keep 4,
    top-8, scale 2.5, 64 tokens, packed;
  * the same shape with IQ1_M routed experts and a Q6_K shared expert, 8 tokens, ggml blobs in place;
  * flash-next-style prefill: 4096 tokens whose expert popularity follows Zipf(1.1), packed, ragged tiles.

Routing is compared in full (logit bits; ids up to near-ties of the libm-based oracle; counts / offsets / slots bit-exact from
the device's ids); layer rows are compared for a seeded sample of tokens so the CPU oracle stays affordable: every routed row
and the shared row of a sampled token is recomputed by the dequantised fp32 expert, then combined.  Bar: relative L2 2e-3.
"""
import numpy as np
import pytest
import torch

from basalt_b200 import capi, moe, pack
from oracle import oracle as O
from tests.helpers import group_near_tie_ok, near_tie_ok, rel_l2

pytestmark = pytest.mark.gpu
TOL = 2e-3


def nvfp4_blobs(n, H, I, seed, dev):
    """n NVFP4 expert blobs quantised on the device from N(0, 0.02^2) (ggml layout, 16-byte aligned stride)."""
    blob_bytes = 3 * I * (H // 64 * 36) + 16
    out = torch.zeros((n, (blob_bytes + 15) // 16 * 16), dtype=torch.uint8, device=dev)
    g = torch.Generator(device=dev).manual_seed(seed)
    for e in range(n):
        G = torch.randn((I, H), generator=g, device=dev) * 0.02
        U = torch.randn((I, H), generator=g, device=dev) * 0.02
        D = torch.randn((H, I), generator=g, device=dev) * 0.02
        out[e, :blob_bytes] = pack.pack_nvfp4_expert(G, U, D)
    return out, blob_bytes


def codebook_blobs(type_id, n, H, I, seed, dev):
    """Random valid blocks of IQ1_M (29) or Q6_K (14), as the reference's own tests make IQ1_M weights
    (tests/kernels/iq1s_parity.cpp:65-93): finite fp16 super-scales, every code uniform."""
    g = torch.Generator(device=dev).manual_seed(seed)
    bb = 56 if type_id == 29 else 210
    nb = 3 * I * H // 256
    raw = torch.randint(0, 256, (n, nb, bb), generator=g, device=dev, dtype=torch.int16)
    if type_id == 29:
        d = 0x2000 + torch.randint(0, 0x400, (n, nb), generator=g, device=dev, dtype=torch.int32)
        for j in range(4):
            raw[:, :, 49 + 2 * j] = (raw[:, :, 49 + 2 * j] & 0x0F) | ((((d >> (4 * j)) & 0xF) << 4).to(torch.int16))
    else:
        raw[:, :, 192:208] = ((raw[:, :, 192:208] & 0x3F) - 32) & 0xFF
        raw[:, :, 208] = 0x00
        raw[:, :, 209] = 0x0C
    out = torch.zeros((n, (nb * bb + 15) // 16 * 16), dtype=torch.uint8, device=dev)
    out[:, :nb * bb] = raw.to(torch.uint8).reshape(n, -1)
    return out, nb * bb


def check_routing(layer, x32, gate_w, bias, T):
    """logit bits, ids (near-ties of the libm oracle only), and the dispatch of the device's ids bit for bit"""
    a = layer.args
    lg = O.router_logits(x32, gate_w)
    assert np.array_equal(lg.view(np.uint32), layer.logits[:T].cpu().numpy().view(np.uint32))
    ids, w = layer.ids[:T].cpu().numpy(), layer.w[:T].cpu().numpy()
    lg64 = lg.astype(np.float64)
    if a.gate == capi.GATE_SOFTMAX:
        oid, ow = O.router_select(lg, None, a.k, O.GATE_SOFTMAX)
        p = np.exp(lg64 - lg64.max(1, keepdims=True))
        near_tie_ok(ids, oid, p / p.sum(1, keepdims=True))
    else:
        oid, ow = O.router_select(lg, bias, a.k, a.gate, a.weight_scale, n_group=a.n_group, topk_group=a.topk_group)
        group_near_tie_ok(ids, oid, 1 / (1 + np.exp(-lg64)) + (bias if bias is not None else 0.0), a.n_group, a.topk_group)
    same = (ids == oid).all(1)
    assert same.any() and np.abs(w[same] - ow[same]).max() < 1e-5
    return ids, w


def expected_rows(Lo, blobs_ggml, x32, ids, w, tokens, shared):
    """y[t] for the sampled tokens: each routed row and the shared row by the dequantised fp32 expert, combined in k order"""
    k = ids.shape[1]
    by_expert = {}
    for t in tokens:
        for j in range(k):
            by_expert.setdefault(int(ids[t, j]), []).append((t, j))
    rows = np.zeros((len(tokens), k, x32.shape[1]), np.float32)
    pos = {t: i for i, t in enumerate(tokens)}
    for e, lst in by_expert.items():
        out = O.expert_forward(Lo, blobs_ggml[e].cpu().numpy()[:Lo.bytes], x32[[t for t, _ in lst]])
        for (t, j), r in zip(lst, out):
            rows[pos[t], j] = r
    sh = None
    if shared is not None:
        sLo, sblob = shared
        sh = O.expert_forward(sLo, sblob.cpu().numpy()[:sLo.bytes], x32[tokens])
    slot = np.arange(len(tokens) * k, dtype=np.int32)
    return O.combine(rows.reshape(len(tokens) * k, -1), slot, np.ascontiguousarray(w[tokens]), sh)


@pytest.mark.parametrize("T", [1, 8, 64])
def test_flash_next_decode_full_shape_packed(lib, cuda, T):
    dev = cuda
    E, H, I, k = 512, 2048, 512, 10
    blobs, nb = nvfp4_blobs(E + 1, H, I, 0, dev)
    L = moe.native_expert_layout(40, 40, H, I)
    assert L.bytes == nb
    packed = moe.pack_experts(L, blobs)
    gate_w = (torch.randn((E, H), generator=torch.Generator(device=dev).manual_seed(5), device=dev) * 0.02).float()
    args = moe.RouterArgs(n_expert=E, n_embd=H, k=k, weight_scale=1.0, gate=capi.GATE_SOFTMAX)
    layer = moe.MoELayer(gate_w, None, packed[:E], L, args, shared_blob=packed[E], max_tokens=T, packed=True)
    x = torch.randn((T, H), generator=torch.Generator(device=dev).manual_seed(T), device=dev).bfloat16()
    y = layer.forward(x).cpu().numpy()
    assert int(layer.status.item()) == 0
    x32 = x.float().cpu().numpy()
    ids, w = check_routing(layer, x32, gate_w.cpu().numpy(), None, T)
    tokens = list(range(T)) if T <= 8 else [0, 7, 19, 31, 42, 63]
    want = expected_rows(O.Layout(40, 40, H, I), blobs, x32, ids, w, tokens, (O.Layout(40, 40, H, I), blobs[E]))
    assert rel_l2(y[tokens], want) < TOL, rel_l2(y[tokens], want)
    # the in-place fp16-image kernels on the same ggml blobs agree on every token
    plain = moe.MoELayer(gate_w, None, blobs[:E], L, args, shared_blob=blobs[E], max_tokens=T)
    y2 = plain.forward(x).cpu().numpy()
    assert np.array_equal(plain.ids[:T].cpu().numpy(), ids)
    assert rel_l2(y, y2) < 1e-3, rel_l2(y, y2)


def test_deepseek_decode_full_shape_packed(lib, cuda):
    dev = cuda
    E, H, I, k, T = 256, 7168, 2048, 8, 64
    blobs, nb = nvfp4_blobs(E + 1, H, I, 1, dev)
    L = moe.native_expert_layout(40, 40, H, I)
    assert L.bytes == nb
    packed = moe.pack_experts(L, blobs)
    gate_w = (torch.randn((E, H), generator=torch.Generator(device=dev).manual_seed(6), device=dev) * 0.02).float()
    bias = (torch.randn(E, generator=torch.Generator(device=dev).manual_seed(7), device=dev) * 0.01).float()
    args = moe.RouterArgs(n_expert=E, n_embd=H, k=k, weight_scale=2.5, gate=capi.GATE_SIGMOID, n_group=8, topk_group=4)
    layer = moe.MoELayer(gate_w, bias, packed[:E], L, args, shared_blob=packed[E], max_tokens=T, packed=True)
    x = torch.randn((T, H), generator=torch.Generator(device=dev).manual_seed(2), device=dev).bfloat16()
    y = layer.forward(x).cpu().numpy()
    assert int(layer.status.item()) == 0
    x32 = x.float().cpu().numpy()
    ids, w = check_routing(layer, x32, gate_w.cpu().numpy(), bias.cpu().numpy(), T)
    tokens = [3, 28, 50]
    Lo = O.Layout(40, 40, H, I)
    want = expected_rows(Lo, blobs, x32, ids, w, tokens, (Lo, blobs[E]))
    assert rel_l2(y[tokens], want) < TOL, rel_l2(y[tokens], want)


def test_deepseek_decode_iq1m_routed_q6k_shared_full_shape(lib, cuda):
    dev = cuda
    E, H, I, k, T = 256, 7168, 2048, 8, 8
    blobs, rb = codebook_blobs(29, E, H, I, 11, dev)
    sblob, sb = codebook_blobs(14, 1, H, I, 12, dev)
    L, Ls = moe.native_expert_layout(29, 29, H, I), moe.native_expert_layout(14, 14, H, I)
    assert L.bytes == rb and Ls.bytes == sb
    gate_w = (torch.randn((E, H), generator=torch.Generator(device=dev).manual_seed(6), device=dev) * 0.02).float()
    bias = (torch.randn(E, generator=torch.Generator(device=dev).manual_seed(7), device=dev) * 0.01).float()
    args = moe.RouterArgs(n_expert=E, n_embd=H, k=k, weight_scale=2.5, gate=capi.GATE_SIGMOID, n_group=8, topk_group=4)
    layer = moe.MoELayer(gate_w, bias, blobs, L, args, shared_blob=sblob[0], shared_layout=Ls, max_tokens=T)
    x = torch.randn((T, H), generator=torch.Generator(device=dev).manual_seed(3), device=dev).bfloat16()
    y = layer.forward(x).cpu().numpy()
    x32 = x.float().cpu().numpy()
    ids, w = check_routing(layer, x32, gate_w.cpu().numpy(), bias.cpu().numpy(), T)
    tokens = [1, 6]
    want = expected_rows(O.Layout(29, 29, H, I), blobs, x32, ids, w, tokens, (O.Layout(14, 14, H, I), sblob[0]))
    assert rel_l2(y[tokens], want) < TOL, rel_l2(y[tokens], want)


def test_flash_next_prefill_4096_tokens_zipf_packed(lib, cuda):
    dev = cuda
    E, H, I, k, T = 512, 2048, 512, 10, 4096
    blobs, nb = nvfp4_blobs(E + 1, H, I, 0, dev)
    L = moe.native_expert_layout(40, 40, H, I)
    packed = moe.pack_experts(L, blobs)
    g = torch.Generator(device=dev).manual_seed(9)
    gate_w = (torch.randn((E, H), generator=g, device=dev) * 0.02).float()
    args = moe.RouterArgs(n_expert=E, n_embd=H, k=k, weight_scale=1.0, gate=capi.GATE_SOFTMAX)
    layer = moe.PrefillMoELayer(gate_w, None, packed[:E], L, args, shared_blob=packed[E], max_tokens=T, packed=True)
    x = torch.randn((T, H), generator=g, device=dev).bfloat16()
    # scores drawn so that expert popularity follows Zipf(1.1): log p_e + Gumbel noise, ranks dealt by a seeded permutation
    p = torch.arange(1, E + 1, device=dev, dtype=torch.float64) ** (-1.1)
    logp = torch.log(p / p.sum()).float()[torch.randperm(E, generator=g, device=dev)]
    u = torch.rand((T, E), generator=g, device=dev).clamp_(1e-20, 1.0 - 1e-7)
    scores = (logp[None, :] - torch.log(-torch.log(u))).contiguous()
    y = layer.forward(x, scores).cpu().numpy()
    assert int(layer.status.item()) == 0
    ids, w = layer.ids.cpu().numpy(), layer.w.cpu().numpy()
    lg = scores.cpu().numpy()
    oid, ow = O.router_select(lg, None, k, O.GATE_SOFTMAX)
    lg64 = lg.astype(np.float64)
    pr = np.exp(lg64 - lg64.max(1, keepdims=True))
    near_tie_ok(ids, oid, pr / pr.sum(1, keepdims=True))
    # the dispatch of the device's ids (with the shared expert as id E on every token): counts, offsets, slots, sources bit-exact
    ids_all = np.concatenate([ids, np.full((T, 1), E, np.int32)], axis=1)
    cnt, off, slot, src, _ = O.dispatch(ids_all, k + 1, E + 1)
    assert np.array_equal(layer.cnt.cpu().numpy(), cnt) and np.array_equal(layer.off.cpu().numpy(), off)
    assert np.array_equal(layer.slot.cpu().numpy(), slot) and np.array_equal(layer.src.cpu().numpy()[:off[-1]], src[:off[-1]])
    assert cnt[:E].max() > 4 * np.median(cnt[:E]) and (cnt[:E] < 64).sum() > 50      # ragged: hot experts and many short tiles
    # 26 sampled tokens = 260 routed rows + 26 shared rows through the dequantised fp32 expert, combined
    rng = np.random.default_rng(4)
    tokens = sorted(rng.choice(T, 26, replace=False).tolist())
    x32 = x.float().cpu().numpy()
    Lo = O.Layout(40, 40, H, I)
    want = expected_rows(Lo, blobs, x32, ids, w, tokens, (Lo, blobs[E]))
    assert rel_l2(y[tokens], want) < TOL, rel_l2(y[tokens], want)
    # and the rows themselves where the dispatch put them
    dm = layer.dm
    for t in tokens[:4]:
        for j in range(k):
            e = int(ids[t, j])
            r = O.expert_forward(Lo, blobs[e].cpu().numpy()[:Lo.bytes], x32[t:t + 1])[0]
            assert rel_l2(dm[slot[t * (k + 1) + j]].cpu().numpy(), r) < TOL
