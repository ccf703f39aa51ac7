"""Host-side mirror of the Basalt engine's MoE operator interface over the B200 C ABI (include/basalt_b200.h).

Function names and argument meanings follow the reference's `basalt::kernels` operators (router, router_select,
route_tail_skip, native_expert_layout, native_expert_grouped, native_moe_combine, ...; see each docstring), so a parity
test reads like the reference's own.  torch supplies device memory and streams only: every computation is a hand-written
CUDA kernel behind the C ABI, and a missing library or GPU raises instead of falling back.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import Optional, Sequence

import torch

from . import capi
from .capi import (GATE_SIGMOID, GATE_SOFTMAX, GATE_SOFTMAX_F64, GATE_SOFTMAX_FAST, GATE_SQRT_SOFTPLUS, OUT_BF16, OUT_F32,
                   TYPE_IQ1_M, TYPE_NVFP4, TYPE_Q6_K, X_BF16, X_F32, X_Q8_1, ExpertLayout, check)


def _stream(stream=None) -> int:
    if stream is None:
        stream = torch.cuda.current_stream()
    h = int(stream.cuda_stream) if hasattr(stream, "cuda_stream") else int(stream)
    # torch's default stream is the null handle, which the expert / dispatch / combine family refuses (as the reference
    # does); cudaStreamLegacy (1) names the same stream explicitly
    return h if h != 0 else 1


def _p(t: Optional[torch.Tensor]) -> Optional[int]:
    if t is None:
        return None
    assert t.is_cuda and t.is_contiguous(), "device, contiguous tensors only"
    return t.data_ptr()


@dataclass
class RouterArgs:
    """basalt::kernels::RouterArgs (include/basalt/kernels/router.hpp:16-27) plus the group-limited step and the softmax
    gate kinds this library adds."""
    n_expert: int = 384
    n_embd: int = 5120
    k: int = 6
    weight_scale: float = 1.5
    gate: int = GATE_SQRT_SOFTPLUS
    prior: float = 0.0
    held: Sequence[torch.Tensor] = field(default_factory=tuple)   # ResidentTabs: up to 4 int32 [n_expert] device tables
    n_group: int = 1
    topk_group: int = 1


def _held(args: RouterArgs):
    tabs = [t for t in args.held if t is not None]
    if not tabs:
        return None, 0, None
    arr = (C.c_void_p * len(tabs))(*[t.data_ptr() for t in tabs])
    return C.cast(arr, C.c_void_p), len(tabs), arr


def router(x, gate, bias, a: RouterArgs, logits=None, ids=None, weights=None, stream=None):
    """basalt::kernels::router (router.hpp:30-32): logits = gate . x, selection, weights.  Returns (logits, ids, weights)."""
    T = x.shape[0]
    dev = x.device
    logits = torch.empty((T, a.n_expert), dtype=torch.float32, device=dev) if logits is None else logits
    ids = torch.empty((T, a.k), dtype=torch.int32, device=dev) if ids is None else ids
    weights = torch.empty((T, a.k), dtype=torch.float32, device=dev) if weights is None else weights
    hp, hn, keep = _held(a)
    check("bsx_router", capi.lib().bsx_router(_p(x), _p(gate), _p(bias), T, a.n_expert, a.n_embd, a.k, a.gate, a.weight_scale,
                                               a.n_group, a.topk_group, a.prior, hp, hn, _p(logits), _p(ids), _p(weights),
                                               _stream(stream)))
    return logits, ids, weights


def router_x(x, gate, bias, a: RouterArgs, logits=None, ids=None, weights=None, stream=None):
    """router() on fp32 or bf16 activation rows (bf16 is widened exactly inside the kernel)."""
    T = x.shape[0]
    dev = x.device
    logits = torch.empty((T, a.n_expert), dtype=torch.float32, device=dev) if logits is None else logits
    ids = torch.empty((T, a.k), dtype=torch.int32, device=dev) if ids is None else ids
    weights = torch.empty((T, a.k), dtype=torch.float32, device=dev) if weights is None else weights
    hp, hn, keep = _held(a)
    check("bsx_router_x", capi.lib().bsx_router_x(_p(x), X_BF16 if x.dtype == torch.bfloat16 else X_F32, _p(gate), _p(bias), T, a.n_expert,
                                                   a.n_embd, a.k, a.gate, a.weight_scale, a.n_group, a.topk_group, a.prior, hp, hn,
                                                   _p(logits), _p(ids), _p(weights), _stream(stream)))
    return logits, ids, weights


def gather_rows(x, src, out=None, stream=None):
    """out[r] = x[src[r]] (the prompt path's gather_rows16, src/models/qwen4exp/prefill/kernels.cu:694-699)."""
    n = src.numel()
    out = torch.empty((n, x.shape[1]), dtype=x.dtype, device=x.device) if out is None else out
    check("bsx_gather_rows", capi.lib().bsx_gather_rows(_p(x), x.shape[1] * x.element_size(), _p(src), n, _p(out), _stream(stream)))
    return out


def router_logits(x, gate, logits=None, stream=None):
    T, H = x.shape
    E = gate.shape[0]
    logits = torch.empty((T, E), dtype=torch.float32, device=x.device) if logits is None else logits
    check("bsx_router_logits", capi.lib().bsx_router_logits(_p(x), _p(gate), T, E, H, _p(logits), _stream(stream)))
    return logits


def router_logits_prefill(x, gate, logits=None, scratch=None, status=None, stream=None):
    """The prompt path's router product (qwen4exp prefill routing.cpp:26) as a tensor-core GEMM; returns (logits, status)."""
    T, H = x.shape
    E = gate.shape[0]
    dev = x.device
    logits = torch.empty((T, E), dtype=torch.float32, device=dev) if logits is None else logits
    if scratch is None:
        scratch = torch.empty(capi.lib().bsx_router_logits_prefill_scratch_bytes(T, E, H), dtype=torch.uint8, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev) if status is None else status
    check("bsx_router_logits_prefill", capi.lib().bsx_router_logits_prefill(_p(x), _x_kind(x), _p(gate), T, E, H, _p(logits), _p(scratch), _p(status),
                                                                             _stream(stream)))
    return logits, status


def router_select(logits, bias, a: RouterArgs, ids=None, weights=None, stream=None):
    """basalt::kernels::router_select (router.hpp:36-37); with a softmax gate kind, qwen4exp's route / native_router_top10 /
    router_top10."""
    T, E = logits.shape
    ids = torch.empty((T, a.k), dtype=torch.int32, device=logits.device) if ids is None else ids
    weights = torch.empty((T, a.k), dtype=torch.float32, device=logits.device) if weights is None else weights
    hp, hn, keep = _held(a)
    check("bsx_router_select", capi.lib().bsx_router_select(_p(logits), _p(bias), T, E, a.k, a.gate, a.weight_scale, a.n_group,
                                                             a.topk_group, a.prior, hp, hn, _p(ids), _p(weights), _stream(stream)))
    return ids, weights


def route_tail_skip(ids, weights, held: Sequence[torch.Tensor], k: int, rank: int, n_expert: int, counts=None, stream=None):
    """basalt::kernels::route_tail_skip (include/basalt/kernels/route_lossy.hpp:58-59); edits ids / weights in place."""
    a = RouterArgs(held=tuple(held))
    hp, hn, keep = _held(a)
    check("bsx_route_tail_skip", capi.lib().bsx_route_tail_skip(_p(ids), _p(weights), hp, hn, ids.numel(), k, rank, n_expert,
                                                                 _p(counts), _stream(stream)))


def dispatch(ids, k: int, n_expert: int, tile_rows: int = 0, stream=None):
    """The prompt path's grouping (qwen4exp Group::group, routing.cpp:67-108; fused::group, moe_fused.hpp:46-50): returns
    (cnt, off, slot, src, tiles, n_tiles); tiles / n_tiles are None without tile_rows."""
    n = ids.numel()
    dev = ids.device
    cnt = torch.empty(n_expert, dtype=torch.int32, device=dev)
    off = torch.empty(n_expert + 1, dtype=torch.int32, device=dev)
    slot = torch.empty(max(n, 1), dtype=torch.int32, device=dev)
    src = torch.full((max(n, 1),), -1, dtype=torch.int32, device=dev)
    tiles = n_tiles = None
    if tile_rows > 0:
        tiles = torch.zeros((n // tile_rows + n_expert, 2), dtype=torch.int32, device=dev)
        n_tiles = torch.zeros(1, dtype=torch.int32, device=dev)
    scratch = torch.empty(capi.lib().bsx_dispatch_scratch_bytes(n, n_expert), dtype=torch.uint8, device=dev)
    check("bsx_dispatch", capi.lib().bsx_dispatch(_p(ids), n, k, n_expert, _p(cnt), _p(off), _p(slot), _p(src), tile_rows,
                                                   _p(tiles), _p(n_tiles), _p(scratch), _stream(stream)))
    return cnt, off, slot[:n], src[:n], tiles, n_tiles


def moe_plan(ids, k: int, n_expert: int, blob_table, stream=None):
    """inkling2 moe_plan (src/models/inkling2/kernels/ops.cu:488-498): (ptr, start, n_groups, dst, tok) device tensors."""
    n = ids.numel()
    T = n // k
    dev = ids.device
    ptr = torch.zeros(max(n, 1), dtype=torch.int64, device=dev)
    start = torch.zeros(n + 2, dtype=torch.int32, device=dev)
    n_groups = torch.zeros(1, dtype=torch.int32, device=dev)
    dst = torch.zeros(max(n, 1), dtype=torch.int32, device=dev)
    tok = torch.zeros(max(n, 1), dtype=torch.int32, device=dev)
    check("bsx_moe_plan", capi.lib().bsx_moe_plan(_p(ids), T, k, n_expert, _p(blob_table), _p(ptr), _p(start), _p(n_groups),
                                                   _p(dst), _p(tok), _stream(stream)))
    return ptr, start, n_groups, dst, tok


def native_expert_layout(gu_type: int, d_type: int, n_embd: int, n_ff: int, swiglu_limit: float = 0.0, up_type: int = -1,
                         gate_softcap: float = 0.0, up_softcap: float = 0.0) -> ExpertLayout:
    """basalt::kernels::native_expert_layout (include/basalt/kernels/iq_kernels.hpp:68-69)."""
    L = ExpertLayout()
    check("bsx_expert_layout_init", capi.lib().bsx_expert_layout_init(gu_type, d_type, up_type, n_embd, n_ff, swiglu_limit,
                                                                       gate_softcap, up_softcap, C.byref(L)))
    return L


def native_expert_supported(gu_type, d_type, n_embd, n_ff, up_type=-1) -> bool:
    return bool(capi.lib().bsx_expert_supported(gu_type, d_type, up_type, n_embd, n_ff))


def native_expert_scratch_bytes(L: ExpertLayout, cap_entries: int) -> int:
    """basalt::kernels::native_expert_scratch_bytes (iq_kernels.hpp:75), from the layout (the tensor-core path keeps fp16
    images of the activations in scratch, so the width n_embd matters too)."""
    return int(capi.lib().bsx_expert_scratch_bytes(C.byref(L), cap_entries))


def quantize_q8_1_rows(x, stream=None):
    """basalt::kernels::quantize_q8_1_rows (iq_kernels.hpp:23): [rows][cols] fp32 -> uint8 [rows * cols / 32 * 36]."""
    rows, cols = x.shape
    y = torch.empty(rows * cols // 32 * 36, dtype=torch.uint8, device=x.device)
    check("bsx_quantize_q8_1_rows", capi.lib().bsx_quantize_q8_1_rows(_p(x), rows, cols, _p(y), _stream(stream)))
    return y


def _x_kind(x) -> int:
    if x.dtype == torch.float32:
        return X_F32
    if x.dtype == torch.bfloat16:
        return X_BF16
    if x.dtype == torch.uint8:
        return X_Q8_1
    raise TypeError("activations must be fp32, bf16 or q8_1 bytes")


def native_expert_grouped(L: ExpertLayout, grp_ptr, grp_start, n_groups, ent_dst, ent_tok, cap_groups: int, cap_entries: int,
                          x, scratch, out, stream=None, n_x_rows: int = 0):
    """basalt::kernels::native_expert_grouped (iq_kernels.hpp:84-87).  `x` may be fp32, bf16 or q8_1 bytes; `out` fp32 or bf16.
    n_x_rows: the number of rows of x when known (activation images are then built once per row)."""
    out_kind = OUT_BF16 if out.dtype == torch.bfloat16 else OUT_F32
    check("bsx_experts_grouped", capi.lib().bsx_experts_grouped_rows(C.byref(L), _p(grp_ptr), _p(grp_start), _p(n_groups), _p(ent_dst),
                                                                      _p(ent_tok), cap_groups, cap_entries, _p(x), _x_kind(x), n_x_rows,
                                                                      _p(scratch), _p(out), out_kind, _stream(stream)))
    return out


def norm_pack(x, w, eps: float, act: bool = True, xn: bool = True, stream=None):
    """basalt::kernels::wgemm::norm_pack (include/basalt/kernels/window_gemm.hpp:36-40): the RMS norm of the rows of x (fp32 or
    bf16) as (bf16 rows or None, fp32 rows or None)."""
    T, K = x.shape
    a = torch.empty((T, K), dtype=torch.bfloat16, device=x.device) if act else None
    n = torch.empty((T, K), dtype=torch.float32, device=x.device) if xn else None
    check("bsx_norm_pack", capi.lib().bsx_norm_pack(_p(x), _x_kind(x), _p(w), eps, K, T, _p(a), _p(n), _stream(stream)))
    return a, n


def pack_experts(L: ExpertLayout, blobs: torch.Tensor, stream=None) -> torch.Tensor:
    """blobs [E][stride] (ggml NVFP4 expert blobs) -> [E][packed stride] in the plane layout bsx_experts_grouped_packed streams
    (a load-time step, like Basalt's nvfp4_planes: include/basalt/kernels/nvfp4_planes.hpp:6-20)."""
    nb = capi.lib().bsx_expert_packed_bytes(C.byref(L))
    if not nb:
        raise ValueError("layout not covered by the packed path (all-NVFP4, n_embd % 256 == 0, n_ff % 256 == 0)")
    out = torch.empty((blobs.shape[0], nb), dtype=torch.uint8, device=blobs.device)
    for e in range(blobs.shape[0]):
        check("bsx_expert_pack", capi.lib().bsx_expert_pack(C.byref(L), blobs[e].data_ptr(), out[e].data_ptr(), _stream(stream)))
    return out


def native_expert_grouped_packed(L: ExpertLayout, grp_ptr, grp_start, n_groups, ent_dst, ent_tok, cap_groups: int, cap_entries: int,
                                 x, scratch, out, status, stream=None, n_x_rows: int = 0):
    """native_expert_grouped over packed blobs on the block-scaled FP4 tensor cores (bsx_experts_grouped_packed)."""
    out_kind = OUT_BF16 if out.dtype == torch.bfloat16 else OUT_F32
    check("bsx_experts_grouped_packed", capi.lib().bsx_experts_grouped_packed(C.byref(L), _p(grp_ptr), _p(grp_start), _p(n_groups), _p(ent_dst),
                                                                               _p(ent_tok), cap_groups, cap_entries, _p(x), _x_kind(x), n_x_rows,
                                                                               _p(scratch), _p(out), out_kind, _p(status), _stream(stream)))
    return out


def experts_prefill(L: ExpertLayout, blob_table, off, src, tiles, n_tiles, x, n_rows: int, dm=None, scratch=None, status=None, stream=None):
    """The prompt path's grouped experts (Basalt: fp4::run_group, include/basalt/prefill/moe_fp4.hpp:104-113) over a dispatch's
    expert-sorted rows; returns (dm [n_rows][n_embd] fp32, status int32[1])."""
    T = x.shape[0]
    dev = x.device
    dm = torch.empty((max(n_rows, 1), L.n_embd), dtype=torch.float32, device=dev) if dm is None else dm
    if scratch is None:
        scratch = torch.empty(capi.lib().bsx_experts_prefill_scratch_bytes(C.byref(L), T, n_rows), dtype=torch.uint8, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev) if status is None else status
    check("bsx_experts_prefill", capi.lib().bsx_experts_prefill(C.byref(L), _p(blob_table), _p(off), _p(src), _p(tiles), _p(n_tiles), tiles.shape[0],
                                                                 n_rows, _p(x), _x_kind(x), T, _p(scratch), _p(dm), _p(status), _stream(stream)))
    return dm, status


def gated_mlp(L: ExpertLayout, blob, x, cap_tok: Optional[int] = None, out=None, scratch=None, stream=None):
    """basalt::kernels::gated_mlp_clamped (iq_kernels.hpp:93-98): a dense gated MLP (a shared expert) over the rows of x; the
    SwiGLU limit is the layout's."""
    n = x.shape[0]
    cap = cap_tok or n
    out = torch.empty((n, L.n_embd), dtype=torch.float32, device=x.device) if out is None else out
    if scratch is None:
        scratch = torch.empty(capi.lib().bsx_gated_mlp_scratch_bytes(C.byref(L), cap), dtype=torch.uint8, device=x.device)
    check("bsx_gated_mlp", capi.lib().bsx_gated_mlp(C.byref(L), _p(blob), n, cap, _p(x), _x_kind(x), _p(scratch), _p(out),
                                                     OUT_BF16 if out.dtype == torch.bfloat16 else OUT_F32, _stream(stream)))
    return out


def moe_combine(rows, slot, weights, shared=None, shared_gate=None, y=None, stream=None, residual=None):
    """native_moe_combine_multi (native_moe.hpp:10-15) / prompt-path moe_combine (prefill/kernels.cu:705-709); residual: the
    residual stream's rows, added last (the step after the layer, fused into the same pass)."""
    T, k = weights.shape
    H = rows.shape[-1]
    y = torch.empty((T, H), dtype=torch.float32, device=rows.device) if y is None else y
    check("bsx_combine", capi.lib().bsx_combine_residual(_p(rows), _p(slot), _p(weights), _p(shared), _p(shared_gate), _p(residual), T, k, H, _p(y),
                                                          _stream(stream)))
    return y


def route_plan(logits, bias, a: RouterArgs, blob_table, shared_blob: int = 0, stream=None):
    """bsx_route_plan: router_select and moe_plan[_shared] as one launch; returns (ids, weights, ptr, start, n_groups, dst, tok)."""
    T, E = logits.shape
    dev, n = logits.device, T * a.k
    rows = n + (T if shared_blob else 0)
    ids = torch.empty((T, a.k), dtype=torch.int32, device=dev)
    w = torch.empty((T, a.k), dtype=torch.float32, device=dev)
    ptr = torch.zeros(n + 3, dtype=torch.int64, device=dev)
    start = torch.zeros(n + 3, dtype=torch.int32, device=dev)
    n_groups = torch.zeros(1, dtype=torch.int32, device=dev)
    dst = torch.zeros(rows, dtype=torch.int32, device=dev)
    tok = torch.zeros(rows, dtype=torch.int32, device=dev)
    check("bsx_route_plan", capi.lib().bsx_route_plan(_p(logits), _p(bias), T, E, a.k, a.gate, a.weight_scale, a.n_group, a.topk_group, _p(blob_table),
                                                       shared_blob, _p(ids), _p(w), _p(ptr), _p(start), _p(n_groups), _p(dst), _p(tok), _stream(stream)))
    return ids, w, ptr, start, n_groups, dst, tok


class KernelWaitTimeout(RuntimeError):
    """A bounded wait inside a tcgen05 kernel ran out (the kernel returned early instead of hanging): the step's output is
    not complete."""


def read_status(status: Optional[torch.Tensor], what: str) -> None:
    """Reads a layer's device status word and clears it; raises KernelWaitTimeout when a kernel reported a wait that ran out.
    This is a device-to-host read (it synchronises the current stream), so call it where the caller synchronises anyway:
    after reading a step's output, or every so many graph replays."""
    if status is None:
        return
    v = int(status.item())
    if v != 0:
        status.zero_()
        raise KernelWaitTimeout(f"{what}: kernel status word {v:#x}: a bounded wait inside a kernel gave up; the output of the steps since the "
                                "last check is not valid")


class MoELayer:
    """One resident MoE layer: router gate, routed expert blobs, optional shared expert, run as the reference's decode
    window does (inkling2/session.cpp:680-716): router -> moe_plan -> native_expert_grouped -> combine.  A shared expert
    with the routed experts' layout rides in the same grouped call as one more group (bsx_moe_plan_shared); one with
    another layout (a Q6_K shared expert beside IQ1_M routed ones) gets its own call."""

    def __init__(self, gate_w: torch.Tensor, bias: Optional[torch.Tensor], blobs: torch.Tensor, layout: ExpertLayout,
                 args: RouterArgs, shared_blob: Optional[torch.Tensor] = None, shared_layout: Optional[ExpertLayout] = None,
                 max_tokens: int = 64, packed: bool = False, norm_w: Optional[torch.Tensor] = None, norm_eps: float = 1e-6,
                 norm_fused: bool = True, fork_images: Optional[bool] = None):
        """packed: blobs (and the shared blob) are already in the plane layout of pack_experts; the experts then run on the
        block-scaled FP4 tensor cores (needs a shared expert of the routed experts' layout, or none).
        norm_w: the layer's input norm weights [n_embd] fp32; forward() then takes the un-normed rows and applies the RMS norm
        itself (the reference's norm_pack step, fused with the FP4 activation images on the packed path; norm_fused=False keeps
        the two as separate launches, for comparison).
        fork_images: the packed path's activation images run on a side stream beside router and plan (True), ahead of them on
        the step's stream (False), or whichever measured faster for the step's token count (None)."""
        assert blobs.dtype == torch.uint8 and blobs.dim() == 2 and blobs.is_cuda
        self.gate_w, self.bias, self.blobs, self.L, self.args = gate_w, bias, blobs, layout, args
        self.shared_blob, self.shared_L = shared_blob, shared_layout or layout
        dev = blobs.device
        E, stride = blobs.shape
        assert stride % 16 == 0 and (packed or stride >= layout.bytes)
        self.packed = packed
        self.blob_table = (blobs.data_ptr() + torch.arange(E, dtype=torch.int64) * stride).to(dev)
        self.max_tokens = max_tokens
        n = max_tokens * args.k
        assert n <= 1024, "the decode-window plan takes at most 1024 (token, expert) pairs"
        self.fused_shared = shared_blob is not None and bytes(self.shared_L) == bytes(layout)
        rows = n + (max_tokens if self.fused_shared else 0)
        f32, i32 = torch.float32, torch.int32
        self.logits = torch.empty((max_tokens, E), dtype=f32, device=dev)
        self.ids = torch.empty((max_tokens, args.k), dtype=i32, device=dev)
        self.w = torch.empty((max_tokens, args.k), dtype=f32, device=dev)
        self.ptr = torch.zeros(n + 3, dtype=torch.int64, device=dev)
        self.start = torch.zeros(n + 3, dtype=i32, device=dev)
        self.n_groups = torch.zeros(1, dtype=i32, device=dev)
        self.dst = torch.zeros(rows, dtype=i32, device=dev)
        self.tok = torch.zeros(rows, dtype=i32, device=dev)
        self.rows = torch.empty((rows, layout.n_embd), dtype=f32, device=dev)
        if packed:
            assert shared_blob is None or self.fused_shared, "the packed path takes the shared expert as one more group"
            self.scratch = torch.empty(capi.lib().bsx_experts_packed_scratch_bytes(C.byref(layout), rows), dtype=torch.uint8, device=dev)
            self.status = torch.zeros(1, dtype=i32, device=dev)
            self.cap_rows = rows
            self.side = torch.cuda.Stream(device=dev)      # the FP4 images of x need no routing: they run beside router and plan
        else:
            self.scratch = torch.empty(native_expert_scratch_bytes(layout, rows), dtype=torch.uint8, device=dev)
        self.y = torch.empty((max_tokens, layout.n_embd), dtype=f32, device=dev)
        self.norm_w, self.norm_eps, self.norm_fused, self.fork_images = norm_w, float(norm_eps), norm_fused, fork_images
        if norm_w is not None:
            assert norm_w.dtype == f32 and norm_w.numel() == layout.n_embd and norm_w.is_cuda
            self.xn = torch.empty((max_tokens, layout.n_embd), dtype=f32, device=dev)
        if shared_blob is not None and not self.fused_shared:
            self.s_ptr = torch.tensor([shared_blob.data_ptr()], dtype=torch.int64, device=dev)
            self.s_iota = torch.arange(max_tokens, dtype=i32, device=dev)
            self.s_one = torch.ones(1, dtype=i32, device=dev)
            self.s_start = torch.zeros(3, dtype=i32, device=dev)
            self.s_out = torch.empty((max_tokens, layout.n_embd), dtype=f32, device=dev)
            self.s_scratch = torch.empty(native_expert_scratch_bytes(self.shared_L, max_tokens), dtype=torch.uint8, device=dev)
            self._s_T = -1

    def check_status(self) -> None:
        """Raises KernelWaitTimeout if any step since the last check hit a bounded wait that ran out (the tcgen05 kernels give up
        after 200 ms instead of hanging and set a status word); clears the word.  Synchronises: call it where the output is
        read on the host."""
        read_status(getattr(self, "status", None), "MoELayer")

    def capture(self, x_example: torch.Tensor):
        """Records forward() for max_tokens rows of x_example's dtype into a CUDA graph (every call of the step is
        stream-ordered and allocates nothing, as the reference requires of its own: iq_kernels.hpp:95); forward_graphed
        then costs one launch."""
        return _capture(self, x_example)

    def forward_graphed(self, x: Optional[torch.Tensor] = None) -> torch.Tensor:
        """x [max_tokens][n_embd] of the captured dtype -> y (a view of an internal buffer), by replaying the graph.  x may be
        a pinned host tensor (it is copied straight into the graph's input buffer); None: the caller has already written
        self.x_static."""
        if x is not None:
            self.x_static.copy_(x, non_blocking=True)
        self.graph.replay()
        return self.y

    def forward(self, x: torch.Tensor, x_router: Optional[torch.Tensor] = None, stream=None) -> torch.Tensor:
        """x: [T][n_embd] fp32 or bf16 activations; x_router: other rows for the router to read (defaults to x).
        Returns y [T][n_embd] fp32 (a view of an internal buffer)."""
        T = x.shape[0]
        a, lib, st = self.args, capi.lib(), _stream(stream)
        assert T <= self.max_tokens
        xr = x_router if x_router is not None else x     # fp32 or bf16 rows; bf16 is widened exactly inside the kernel
        hp, hn, keep = _held(a)
        images_ahead = self.packed and self.fused_shared
        fuse = images_ahead and self.norm_fused
        forked = images_ahead and (self.norm_w is None or not fuse)
        if self.norm_w is not None:
            # the step before the layer: RMS norm of the input rows (fp32 rows for the router and the experts), on the packed path
            # together with the FP4 images of the normed rows
            if fuse:
                check("bsx_norm_pack_images", lib.bsx_norm_pack_images(C.byref(self.L), _p(x), _x_kind(x), _p(self.norm_w), self.norm_eps, T,
                                                                       T * a.k + T, _p(self.scratch), _p(self.xn), None, st))
            else:
                check("bsx_norm_pack", lib.bsx_norm_pack(_p(x), _x_kind(x), _p(self.norm_w), self.norm_eps, a.n_embd, T, None, _p(self.xn), st))
            x = xr = self.xn[:T]
        # measured on a B200 (512 experts, top-10): beside the router the images save ~0.4 us a step at 1 - 8 tokens and cost
        # ~2.5 us at 64 (the join delays the gate/up launch more than the 5 us image kernel it hides)
        if forked and not (self.fork_images if self.fork_images is not None else T <= 16):
            # the images first on this stream, no fork
            check("bsx_experts_packed_x_images", lib.bsx_experts_packed_x_images(C.byref(self.L), _p(x), _x_kind(x), T, T * a.k + T, _p(self.scratch), st))
            forked = False
        if forked:
            # fork: the activation images on the side stream while the router and the plan run on this one (joined before the experts)
            cur = stream if stream is not None else torch.cuda.current_stream()
            self.side.wait_stream(cur)
            check("bsx_experts_packed_x_images", lib.bsx_experts_packed_x_images(C.byref(self.L), _p(x), _x_kind(x), T, T * a.k + T, _p(self.scratch),
                                                                                 _stream(self.side)))
        check("bsx_router", lib.bsx_router_x(_p(xr), X_BF16 if xr.dtype == torch.bfloat16 else X_F32, _p(self.gate_w), _p(self.bias), T,
                                              a.n_expert, a.n_embd, a.k, a.gate, a.weight_scale, a.n_group, a.topk_group, a.prior, hp, hn,
                                              _p(self.logits), _p(self.ids), _p(self.w), st))
        n = T * a.k
        kind = _x_kind(x)
        shared = None
        if self.fused_shared:
            check("bsx_moe_plan_shared", lib.bsx_moe_plan_shared(_p(self.ids), T, a.k, a.n_expert, _p(self.blob_table), self.shared_blob.data_ptr(),
                                                                 _p(self.ptr), _p(self.start), _p(self.n_groups), _p(self.dst), _p(self.tok), st))
            if forked:
                cur.wait_stream(self.side)       # join
            if self.packed:
                check("bsx_experts_grouped_packed", lib.bsx_experts_grouped_packed(C.byref(self.L), _p(self.ptr), _p(self.start), _p(self.n_groups),
                                                                                   _p(self.dst), _p(self.tok), min(n, a.n_expert) + 1, n + T, _p(x), kind,
                                                                                   -T if images_ahead else T, _p(self.scratch), _p(self.rows), OUT_F32,
                                                                                   _p(self.status), st))
            else:
                check("bsx_experts_grouped", lib.bsx_experts_grouped_rows(C.byref(self.L), _p(self.ptr), _p(self.start), _p(self.n_groups),
                                                                          _p(self.dst), _p(self.tok), min(n, a.n_expert) + 1, n + T, _p(x), kind, T,
                                                                          _p(self.scratch), _p(self.rows), OUT_F32, st))
            shared = self.rows[n:n + T]
        else:
            check("bsx_moe_plan", lib.bsx_moe_plan(_p(self.ids), T, a.k, a.n_expert, _p(self.blob_table), _p(self.ptr), _p(self.start),
                                                    _p(self.n_groups), _p(self.dst), _p(self.tok), st))
            if self.packed:
                check("bsx_experts_grouped_packed", lib.bsx_experts_grouped_packed(C.byref(self.L), _p(self.ptr), _p(self.start), _p(self.n_groups),
                                                                                   _p(self.dst), _p(self.tok), min(n, a.n_expert), n, _p(x), kind, T,
                                                                                   _p(self.scratch), _p(self.rows), OUT_F32, _p(self.status), st))
            else:
                check("bsx_experts_grouped", lib.bsx_experts_grouped_rows(C.byref(self.L), _p(self.ptr), _p(self.start), _p(self.n_groups),
                                                                          _p(self.dst), _p(self.tok), min(n, a.n_expert), n, _p(x), kind, T,
                                                                          _p(self.scratch), _p(self.rows), OUT_F32, st))
            if self.shared_blob is not None:
                if self._s_T != T:
                    self.s_start.copy_(torch.tensor([0, T, T], dtype=torch.int32))
                    self._s_T = T
                check("bsx_experts_grouped", lib.bsx_experts_grouped(C.byref(self.shared_L), _p(self.s_ptr), _p(self.s_start), _p(self.s_one),
                                                                     _p(self.s_iota), _p(self.s_iota), 1, T, _p(x), kind, _p(self.s_scratch),
                                                                     _p(self.s_out), OUT_F32, st))
                shared = self.s_out
        check("bsx_combine", lib.bsx_combine(_p(self.rows), None, _p(self.w), _p(shared), None, T, a.k, self.L.n_embd, _p(self.y), st))
        return self.y[:T]


class NativeMoELayer:
    """The same resident layer run by ONE C ABI call per step (bsx_moe_layer): the input norm, router logits, selection + plan,
    grouped experts with the shared expert, combine and the residual add are issued inside the library, every kernel after the
    first as a programmatic dependent launch.  What a C++ engine would call from its layer loop (the reference's sequence at
    src/models/inkling2/session.cpp:680-716); this class only owns the buffers.  Routing results (logits, ids, w) are views into
    the call's workspace."""

    def __init__(self, gate_w: torch.Tensor, bias: Optional[torch.Tensor], blobs: torch.Tensor, layout: ExpertLayout, args: RouterArgs,
                 shared_blob: Optional[torch.Tensor] = None, shared_layout: Optional[ExpertLayout] = None, max_tokens: int = 64,
                 packed: bool = False, norm_w: Optional[torch.Tensor] = None, norm_eps: float = 1e-6, pdl: bool = True):
        assert blobs.dtype == torch.uint8 and blobs.dim() == 2 and blobs.is_cuda
        dev = blobs.device
        E, stride = blobs.shape
        self.gate_w, self.bias, self.blobs, self.L, self.args, self.shared_blob, self.norm_w = gate_w, bias, blobs, layout, args, shared_blob, norm_w
        self.packed, self.max_tokens = packed, max_tokens
        self.blob_table = (blobs.data_ptr() + torch.arange(E, dtype=torch.int64) * stride).to(dev)
        d = capi.MoELayerDesc()
        d.layout = layout
        if shared_layout is not None:
            d.shared_layout = shared_layout
        d.n_expert, d.top_k, d.gate_kind, d.n_group, d.topk_group = E, args.k, args.gate, args.n_group, args.topk_group
        d.packed, d.flags, d.weight_scale, d.norm_eps = int(packed), 0 if pdl else capi.LAYER_NO_PDL, args.weight_scale, float(norm_eps)
        d.gate, d.bias, d.blob_table = gate_w.data_ptr(), (bias.data_ptr() if bias is not None else None), self.blob_table.data_ptr()
        d.shared_blob = shared_blob.data_ptr() if shared_blob is not None else 0
        d.norm_w = norm_w.data_ptr() if norm_w is not None else None
        self.desc = d
        nbytes = capi.lib().bsx_moe_layer_workspace_bytes(C.byref(d), max_tokens)
        if not nbytes:
            raise ValueError("bsx_moe_layer does not take this layer (experts, top-k, window size or block formats)")
        self.workspace = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        self.y = torch.empty((max_tokens, layout.n_embd), dtype=torch.float32, device=dev)
        v = capi.MoELayerViews()
        check("bsx_moe_layer_views", capi.lib().bsx_moe_layer_views(C.byref(d), max_tokens, self.workspace.data_ptr(), C.byref(v)))
        base = self.workspace.data_ptr()

        def view(ptr, shape, dtype):
            n = int(torch.tensor(shape).prod().item()) * torch.empty((), dtype=dtype).element_size()
            return self.workspace[ptr - base:ptr - base + n].view(dtype).view(shape)
        self.logits = view(v.logits, (max_tokens, E), torch.float32)
        self.ids = view(v.ids, (max_tokens, args.k), torch.int32)
        self.w = view(v.weights, (max_tokens, args.k), torch.float32)
        self.n_groups = view(v.n_groups, (1,), torch.int32)

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None, stream=None) -> torch.Tensor:
        T = x.shape[0]
        check("bsx_moe_layer", capi.lib().bsx_moe_layer(C.byref(self.desc), _p(x), _x_kind(x), T, self.max_tokens, _p(residual), self.workspace.data_ptr(),
                                                         _p(self.y), _p(self.status), _stream(stream)))
        return self.y[:T]

    def check_status(self) -> None:
        """See MoELayer.check_status."""
        read_status(self.status, "NativeMoELayer")

    def capture(self, x_example: torch.Tensor):
        return _capture(self, x_example)

    def forward_graphed(self, x: Optional[torch.Tensor] = None) -> torch.Tensor:
        if x is not None:
            self.x_static.copy_(x, non_blocking=True)
        self.graph.replay()
        return self.y


def _capture(layer, x_example: torch.Tensor):
    """Shared by the layer classes: run forward() twice outside a capture (one-time attribute calls, allocations), then
    record it into a CUDA graph over a static input buffer."""
    T, H = layer.max_tokens, layer.L.n_embd
    layer.x_static = torch.zeros((T, H), dtype=x_example.dtype, device=x_example.device)
    side = torch.cuda.Stream(device=x_example.device)
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):
            layer.forward(layer.x_static)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    layer.graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(layer.graph):
        layer.forward(layer.x_static)
    return layer


class PrefillMoELayer:
    """One resident MoE layer on a prompt-sized batch, as the reference's prompt path runs it (qwen4exp prefill: route ->
    Group::group -> fp4::run_group -> moe_combine; src/models/qwen4exp/prefill/routing.cpp:26-122, expert_fp4.cpp:26-46,
    kernels.cu:705-709): router -> bsx_dispatch (with the 128-row tile list) -> bsx_experts_prefill -> bsx_combine.  NVFP4
    blobs.  A shared expert of the same layout is expert id E of the same dispatch: every token gets one more (id, weight)
    pair (E, 1.0), so its rows go through the same grouped launch and the combine's last term adds them unweighted."""

    def __init__(self, gate_w: torch.Tensor, bias: Optional[torch.Tensor], blobs: torch.Tensor, layout: ExpertLayout, args: RouterArgs,
                 shared_blob: Optional[torch.Tensor] = None, max_tokens: int = 4096, packed: bool = False):
        """packed: blobs (and the shared blob) are in the plane layout of pack_experts; the experts then run on the
        block-scaled FP4 tensor cores (bsx_experts_prefill_packed)."""
        assert blobs.dtype == torch.uint8 and blobs.dim() == 2 and blobs.is_cuda
        self.gate_w, self.bias, self.blobs, self.L, self.args, self.shared_blob = gate_w, bias, blobs, layout, args, shared_blob
        self.packed = packed
        dev = blobs.device
        E, stride = blobs.shape
        table = blobs.data_ptr() + torch.arange(E, dtype=torch.int64) * stride
        self.kk = args.k + (1 if shared_blob is not None else 0)
        self.EE = E + (1 if shared_blob is not None else 0)
        if shared_blob is not None:
            table = torch.cat([table, torch.tensor([shared_blob.data_ptr()], dtype=torch.int64)])
        self.blob_table = table.to(dev)
        T, n = max_tokens, max_tokens * self.kk
        self.max_tokens = T
        f32, i32 = torch.float32, torch.int32
        self.logits = torch.empty((T, E), dtype=f32, device=dev)
        self.ids = torch.empty((T, args.k), dtype=i32, device=dev)
        self.w = torch.empty((T, args.k), dtype=f32, device=dev)
        self.ids_all = torch.full((T, self.kk), E, dtype=i32, device=dev)     # the last column stays (E, 1.0): the shared expert
        self.w_all = torch.ones((T, self.kk), dtype=f32, device=dev)
        self.cnt = torch.empty(self.EE, dtype=i32, device=dev)
        self.off = torch.empty(self.EE + 1, dtype=i32, device=dev)
        self.slot = torch.empty(n, dtype=i32, device=dev)
        self.src = torch.empty(n, dtype=i32, device=dev)
        self.tiles = torch.zeros((n // 128 + self.EE, 2), dtype=i32, device=dev)
        self.n_tiles = torch.zeros(1, dtype=i32, device=dev)
        self.dscratch = torch.empty(capi.lib().bsx_dispatch_scratch_bytes(n, self.EE), dtype=torch.uint8, device=dev)
        nscr = (capi.lib().bsx_experts_prefill_packed_scratch_bytes if packed else capi.lib().bsx_experts_prefill_scratch_bytes)(C.byref(layout), T, n)
        self.scratch = torch.empty(nscr, dtype=torch.uint8, device=dev)
        self.dm = torch.empty((n, layout.n_embd), dtype=f32, device=dev)
        self.status = torch.zeros(1, dtype=i32, device=dev)
        self.rscratch = torch.empty(capi.lib().bsx_router_logits_prefill_scratch_bytes(T, E, layout.n_embd), dtype=torch.uint8, device=dev)
        self.y = torch.empty((T, layout.n_embd), dtype=f32, device=dev)
        self.events = None      # set to a list to collect (name, event) marks between the stages

    def check_status(self) -> None:
        """See MoELayer.check_status."""
        read_status(self.status, "PrefillMoELayer")

    def _mark(self, name, stream):
        if self.events is not None:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record(stream if stream is not None else torch.cuda.current_stream())
            self.events.append((name, ev))

    def forward(self, x: torch.Tensor, logits: Optional[torch.Tensor] = None, stream=None) -> torch.Tensor:
        """x [T][n_embd] fp32 or bf16.  logits: when given, the selection reads these [T][E] fp32 scores instead of the ones
        just computed from x (a bench draws them to set the experts' popularity); the gate product still runs."""
        T = x.shape[0]
        a, lib, st, L = self.args, capi.lib(), _stream(stream), self.L
        assert T == self.max_tokens, "buffers are sized for max_tokens rows"
        self._mark("start", stream)
        check("bsx_router_logits_prefill", lib.bsx_router_logits_prefill(_p(x), _x_kind(x), _p(self.gate_w), T, a.n_expert, a.n_embd, _p(self.logits),
                                                                         _p(self.rscratch), _p(self.status), st))
        self._mark("router_logits", stream)
        router_select(self.logits if logits is None else logits, self.bias, a, self.ids, self.w, stream)
        if self.kk != a.k:
            self.ids_all[:, :a.k].copy_(self.ids)
            self.w_all[:, :a.k].copy_(self.w)
            ids, w = self.ids_all, self.w_all
        else:
            ids, w = self.ids, self.w
        self._mark("router_select", stream)
        n = T * self.kk
        check("bsx_dispatch", lib.bsx_dispatch(_p(ids), n, self.kk, self.EE, _p(self.cnt), _p(self.off), _p(self.slot), _p(self.src), 128,
                                               _p(self.tiles), _p(self.n_tiles), _p(self.dscratch), st))
        self._mark("dispatch", stream)
        if self.packed:
            check("bsx_experts_prefill_packed", lib.bsx_experts_prefill_packed(C.byref(L), _p(self.blob_table), _p(self.off), _p(self.src), _p(self.tiles),
                                                                               _p(self.n_tiles), self.tiles.shape[0], n, _p(x), _x_kind(x), T, self.EE,
                                                                               _p(self.scratch), _p(self.dm), _p(self.status), st))
        else:
            check("bsx_experts_prefill", lib.bsx_experts_prefill(C.byref(L), _p(self.blob_table), _p(self.off), _p(self.src), _p(self.tiles), _p(self.n_tiles),
                                                                 self.tiles.shape[0], n, _p(x), _x_kind(x), T, _p(self.scratch), _p(self.dm), _p(self.status), st))
        self._mark("experts", stream)
        check("bsx_combine", lib.bsx_combine(_p(self.dm), _p(self.slot), _p(w), None, None, T, self.kk, L.n_embd, _p(self.y), st))
        self._mark("combine", stream)
        return self.y
