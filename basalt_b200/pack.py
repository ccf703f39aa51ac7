"""Packing fp32 expert matrices into the ggml-layout blobs the kernels read ([gate rows | up rows | down rows | tail]).

NVFP4 only (the format a B200 deployment packs itself); K- and I-quant blobs come from GGUF files as they are.  The
rounding rule is ggml's reference quantiser for NVFP4 (Basalt: src/kernels/cpu/ggml/ggml_quants.c:1447-1476): per 16 values the
UE4M3 scale nearest amax / 6, then per value the nearest E2M1 code under that scale, the first candidate winning ties.
Runs on whatever device the input tensor is on (torch ops: this is load-time tooling, not the hot path).
"""
from __future__ import annotations

import torch

_E2M1_X2 = [0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12]


def _ue4m3_table(device) -> torch.Tensor:
    """value of UE4M3 code c (not halved), c in 0..126, ascending."""
    c = torch.arange(127, device=device)
    e, m = (c >> 3).float(), (c & 7).float()
    v = torch.where(c < 8, m * 2.0 ** -9, (1.0 + m / 8.0) * torch.exp2(e - 7.0))
    return v.float()


def quantize_nvfp4(w: torch.Tensor) -> torch.Tensor:
    """[rows][cols] fp32 (cols % 64 == 0) -> uint8 [rows][cols / 64 * 36] in ggml's block_nvfp4 layout
    (4 scale bytes, then per 16-value sub-block 8 bytes: byte j = value j in the low nibble, value j + 8 in the high)."""
    assert w.dtype == torch.float32 and w.dim() == 2 and w.shape[1] % 64 == 0
    rows, cols = w.shape
    dev = w.device
    sub = w.reshape(-1, 16)                                   # [n_sub][16]
    amax = sub.abs().amax(dim=1)
    target = amax / 6.0
    tab = _ue4m3_table(dev)
    hi = torch.searchsorted(tab, target.contiguous()).clamp_(0, 126)
    lo = (hi - 1).clamp_(0, 126)
    err_lo, err_hi = (tab[lo] - target).abs(), (tab[hi] - target).abs()
    code = torch.where(err_lo <= err_hi, lo, hi)              # the lower code wins a tie, as the ascending scan does
    d = tab[code] * 0.5                                        # ggml's decoded scale (the E2M1 table is doubled)
    kv = torch.tensor(_E2M1_X2, dtype=torch.float32, device=dev)
    q = torch.empty(sub.shape, dtype=torch.uint8, device=dev)
    step = 1 << 18
    for s in range(0, sub.shape[0], step):                    # bounded temporary: [step][16][16] floats
        cand = kv.view(1, 1, 16) * d[s:s + step].view(-1, 1, 1)
        err = (cand - sub[s:s + step].unsqueeze(-1)).abs()
        q[s:s + step] = err.argmin(dim=-1).to(torch.uint8)    # first minimum = lowest code
    qs = (q[:, :8] | (q[:, 8:] << 4)).reshape(-1, 4, 8)        # [n_blk][4 sub][8 bytes]
    blocks = torch.empty((qs.shape[0], 36), dtype=torch.uint8, device=dev)
    blocks[:, :4] = code.to(torch.uint8).reshape(-1, 4)
    blocks[:, 4:] = qs.reshape(-1, 32)
    return blocks.reshape(rows, cols // 64 * 36)


def pack_nvfp4_expert(G: torch.Tensor, U: torch.Tensor, D: torch.Tensor) -> torch.Tensor:
    """One expert blob from gate [I][H], up [I][H], down [H][I] fp32: each matrix is divided by its own fp32 scale
    s = amax / (6 * 448) before block quantisation and {s_gate, s_up, s_down, 0} closes the blob (the recipe of the
    reference's synthetic packs, tests/kernels/native_expert_parity.cpp:411-432, docs/model-file.md:176-178)."""
    parts, tail = [], []
    for w in (G, U, D):
        s = (w.abs().amax() / (6.0 * 448.0)).float()
        s = torch.where(s > 0, s, torch.ones_like(s))
        parts.append(quantize_nvfp4((w / s).float()).reshape(-1))
        tail.append(s)
    tail.append(torch.zeros((), device=G.device))
    return torch.cat(parts + [torch.stack(tail).float().contiguous().view(torch.uint8).reshape(-1)])
