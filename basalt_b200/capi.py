"""ctypes bindings of libbasalt_b200.so, the C ABI declared in include/basalt_b200.h.

Pointers are passed as integers (torch `tensor.data_ptr()` or any device address).  Loading fails loudly when the library
has not been built: there is no Python or CPU fallback behind these calls.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

PKG = Path(__file__).resolve().parent
LIB_PATH = PKG / "lib" / "libbasalt_b200.so"

OK, E_GEOMETRY, E_STREAM, E_TYPE, E_POINTER, E_LIMIT, E_UNAVAILABLE = 0, -1, -2, -3, -4, -5, -6
GATE_SQRT_SOFTPLUS, GATE_SIGMOID, GATE_SOFTMAX, GATE_SOFTMAX_FAST, GATE_SOFTMAX_F64 = 0, 1, 2, 3, 4
TYPE_Q6_K, TYPE_IQ1_M, TYPE_NVFP4 = 14, 29, 40
X_F32, X_BF16, X_Q8_1 = 0, 1, 2
OUT_F32, OUT_BF16 = 0, 1
EXPERT_STAGE_ALL, EXPERT_STAGE_GU, EXPERT_STAGE_DOWN, EXPERT_PLAIN = 0, 1, 2, 4   # bsx_expert_layout.options


class ExpertLayout(C.Structure):
    _fields_ = [("gu_type", C.c_int32), ("d_type", C.c_int32), ("up_type", C.c_int32), ("options", C.c_int32),
                ("n_embd", C.c_int64), ("n_ff", C.c_int64),
                ("gu_row", C.c_uint64), ("d_row", C.c_uint64), ("up_row", C.c_uint64),
                ("up_off", C.c_uint64), ("down_off", C.c_uint64), ("bytes", C.c_uint64),
                ("swiglu_limit", C.c_float), ("gate_softcap", C.c_float), ("up_softcap", C.c_float), ("reserved_f", C.c_float)]


class LayoutRow(C.Structure):
    _fields_ = [("gu_type", C.c_int32), ("d_type", C.c_int32), ("up_type", C.c_int32), ("kernels", C.c_int32),
                ("offset", C.c_uint64), ("blob_bytes", C.c_uint64)]


class LayoutInfo(C.Structure):
    _fields_ = [("version", C.c_int32), ("reserved", C.c_int32), ("n_layers", C.c_int64), ("n_expert", C.c_int64),
                ("max_blob", C.c_uint64), ("total", C.c_uint64)]


class MoELayerDesc(C.Structure):
    _fields_ = [("layout", ExpertLayout), ("shared_layout", ExpertLayout),
                ("n_expert", C.c_int32), ("top_k", C.c_int32), ("gate_kind", C.c_int32), ("n_group", C.c_int32), ("topk_group", C.c_int32),
                ("packed", C.c_int32), ("flags", C.c_int32), ("weight_scale", C.c_float), ("norm_eps", C.c_float),
                ("gate", C.c_void_p), ("bias", C.c_void_p), ("blob_table", C.c_void_p), ("shared_blob", C.c_uint64), ("norm_w", C.c_void_p)]


class EPLayerDesc(C.Structure):
    _fields_ = [("layout", ExpertLayout),
                ("n_expert", C.c_int32), ("top_k", C.c_int32), ("gate_kind", C.c_int32), ("n_group", C.c_int32), ("topk_group", C.c_int32),
                ("packed", C.c_int32), ("e_lo", C.c_int32), ("n_local", C.c_int32), ("n_replicas", C.c_int32), ("reserved", C.c_int32),
                ("weight_scale", C.c_float), ("reserved_f", C.c_float),
                ("gate", C.c_void_p), ("bias", C.c_void_p), ("blob_table", C.c_void_p), ("shared_blob", C.c_uint64), ("replicated", C.c_void_p)]


class MoELayerViews(C.Structure):
    _fields_ = [("logits", C.c_void_p), ("ids", C.c_void_p), ("weights", C.c_void_p), ("n_groups", C.c_void_p), ("grp_start", C.c_void_p),
                ("ent_dst", C.c_void_p), ("ent_tok", C.c_void_p), ("rows", C.c_void_p)]


LAYER_NO_PDL = 1

P = C.c_void_p
_SIGNATURES = {
    "bsx_experts_prefill_group_scratch_bytes": (C.c_size_t, [C.POINTER(ExpertLayout), C.c_int64, C.c_int64]),
    "bsx_experts_prefill_group": (C.c_int32, [C.POINTER(ExpertLayout), P, C.c_int32, P, P, C.c_int64, P, C.c_int32, C.c_int64, P, P, P, P]),
    "bsx_unit_offsets": (C.c_int32, [P, C.c_int32, C.c_int32, P, P]),
    "bsx_rebase_bounds": (C.c_int32, [P, C.c_int32, P, P]),
    "bsx_ep_available": (C.c_int32, []),
    "bsx_ep_layer_workspace_bytes": (C.c_size_t, [P, C.c_int32, C.c_int32]),
    "bsx_ep_layer_views": (C.c_int32, [P, C.c_int32, C.c_int32, P, P]),
    "bsx_ep_layer": (C.c_int32, [P, P, P, C.c_int32, C.c_int32, P, P, P, P, P, P, P]),
    "bsx_ep_plan": (C.c_int32, [P, C.c_int64, C.c_int32, C.c_int32, C.c_int32, C.c_int32, P, C.c_uint64, C.c_int32, C.c_int32, P, P, P, P, P, P, P]),
    "bsx_combine_partial_ep": (C.c_int32, [P, P, P, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, P, C.c_int32, C.c_int32, P, P, P]),
    "bsx_combine_residual": (C.c_int32, [P, P, P, P, P, P, C.c_int32, C.c_int32, C.c_int32, P, P]),
    "bsx_route_plan": (C.c_int32, [P, P, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_float, C.c_int32, C.c_int32, P, C.c_uint64, P, P, P, P, P, P, P, P]),
    "bsx_moe_layer_workspace_bytes": (C.c_size_t, [C.POINTER(MoELayerDesc), C.c_int32]),
    "bsx_moe_layer_views": (C.c_int32, [C.POINTER(MoELayerDesc), C.c_int32, P, C.POINTER(MoELayerViews)]),
    "bsx_moe_layer": (C.c_int32, [C.POINTER(MoELayerDesc), P, C.c_int32, C.c_int32, C.c_int32, P, P, P, P, P]),
    "bsx_router_logits": (C.c_int32, [P, P, C.c_int32, C.c_int32, C.c_int32, P, P]),
    "bsx_router_select": (C.c_int32, [P, P, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_float, C.c_int32, C.c_int32,
                                      C.c_float, P, C.c_int32, P, P, P]),
    "bsx_router": (C.c_int32, [P, P, P, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_float, C.c_int32,
                               C.c_int32, C.c_float, P, C.c_int32, P, P, P, P]),
    "bsx_experts_prefill_packed_scratch_bytes": (C.c_size_t, [C.POINTER(ExpertLayout), C.c_int64, C.c_int64]),
    "bsx_experts_prefill_packed": (C.c_int32, [C.POINTER(ExpertLayout), P, P, P, P, P, C.c_int64, C.c_int64, P, C.c_int32, C.c_int64, C.c_int32, P, P, P, P]),
    "bsx_expert_packed_bytes": (C.c_size_t, [C.POINTER(ExpertLayout)]),
    "bsx_expert_pack": (C.c_int32, [C.POINTER(ExpertLayout), P, P, P]),
    "bsx_experts_packed_scratch_bytes": (C.c_size_t, [C.POINTER(ExpertLayout), C.c_int64]),
    "bsx_experts_packed_x_images": (C.c_int32, [C.POINTER(ExpertLayout), P, C.c_int32, C.c_int32, C.c_int64, P, P]),
    "bsx_experts_grouped_packed": (C.c_int32, [C.POINTER(ExpertLayout), P, P, P, P, P, C.c_int64, C.c_int64, P, C.c_int32, C.c_int32, P, P, C.c_int32, P, P]),
    "bsx_router_logits_prefill_scratch_bytes": (C.c_size_t, [C.c_int64, C.c_int32, C.c_int32]),
    "bsx_router_logits_prefill": (C.c_int32, [P, C.c_int32, P, C.c_int64, C.c_int32, C.c_int32, P, P, P, P]),
    "bsx_router_logits_x": (C.c_int32, [P, C.c_int32, P, C.c_int32, C.c_int32, C.c_int32, P, P]),
    "bsx_router_x": (C.c_int32, [P, C.c_int32, P, P, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_float, C.c_int32,
                                 C.c_int32, C.c_float, P, C.c_int32, P, P, P, P]),
    "bsx_route_tail_skip": (C.c_int32, [P, P, P, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, P, P]),
    "bsx_dispatch_scratch_bytes": (C.c_size_t, [C.c_int64, C.c_int32]),
    "bsx_dispatch": (C.c_int32, [P, C.c_int64, C.c_int32, C.c_int32, P, P, P, P, C.c_int32, P, P, P, P]),
    "bsx_dispatch_static": (C.c_int32, [P, C.c_int64, C.c_int32, C.c_int32, P, P, P, P, P]),
    "bsx_gather_rows": (C.c_int32, [P, C.c_int64, P, C.c_int64, P, P]),
    "bsx_moe_plan": (C.c_int32, [P, C.c_int32, C.c_int32, C.c_int32, P, P, P, P, P, P, P]),
    "bsx_moe_plan_shared": (C.c_int32, [P, C.c_int32, C.c_int32, C.c_int32, P, C.c_uint64, P, P, P, P, P, P]),
    "bsx_expert_layout_init": (C.c_int32, [C.c_int32, C.c_int32, C.c_int32, C.c_int64, C.c_int64, C.c_float, C.c_float,
                                           C.c_float, C.POINTER(ExpertLayout)]),
    "bsx_expert_supported": (C.c_int32, [C.c_int32, C.c_int32, C.c_int32, C.c_int64, C.c_int64]),
    "bsx_expert_scratch_bytes": (C.c_size_t, [C.POINTER(ExpertLayout), C.c_int64]),
    "bsx_quantize_q8_1_rows": (C.c_int32, [P, C.c_int64, C.c_int64, P, P]),
    "bsx_experts_grouped": (C.c_int32, [C.POINTER(ExpertLayout), P, P, P, P, P, C.c_int64, C.c_int64, P, C.c_int32, P, P,
                                        C.c_int32, P]),
    "bsx_experts_grouped_rows": (C.c_int32, [C.POINTER(ExpertLayout), P, P, P, P, P, C.c_int64, C.c_int64, P, C.c_int32, C.c_int32, P, P,
                                             C.c_int32, P]),
    "bsx_gated_mlp_scratch_bytes": (C.c_size_t, [C.POINTER(ExpertLayout), C.c_int64]),
    "bsx_gated_mlp": (C.c_int32, [C.POINTER(ExpertLayout), P, C.c_int32, C.c_int64, P, C.c_int32, P, P, C.c_int32, P]),
    "bsx_experts_prefill_scratch_bytes": (C.c_size_t, [C.POINTER(ExpertLayout), C.c_int64, C.c_int64]),
    "bsx_experts_prefill": (C.c_int32, [C.POINTER(ExpertLayout), P, P, P, P, P, C.c_int64, C.c_int64, P, C.c_int32, C.c_int64, P, P, P, P]),
    "bsx_plan_groups": (C.c_int32, [P, P, P, C.c_int32, P, P, P, P, P, P, P]),
    "bsx_tiles_from_bounds": (C.c_int32, [P, C.c_int32, C.c_int32, P, P, P]),
    "bsx_plan_groups_shared": (C.c_int32, [P, P, P, C.c_int32, P, C.c_uint64, C.c_int32, C.c_int32, P, P, P, P, P, P]),
    "bsx_combine_partial": (C.c_int32, [P, P, P, P, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, P, P]),
    "bsx_combine": (C.c_int32, [P, P, P, P, P, C.c_int32, C.c_int32, C.c_int32, P, P]),
    "bsx_norm_pack": (C.c_int32, [P, C.c_int32, P, C.c_float, C.c_int64, C.c_int32, P, P, P]),
    "bsx_norm_pack_images": (C.c_int32, [C.POINTER(ExpertLayout), P, C.c_int32, P, C.c_float, C.c_int32, C.c_int64, P, P, P, P]),
    "bsx_layout_parse": (C.c_int32, [C.c_char_p, C.c_size_t, C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_float, P, P, C.c_char_p, C.c_size_t]),
    "bsx_host_decode_row": (C.c_int32, [C.c_int32, P, P, C.c_int64]),
    "bsx_row_bytes": (C.c_size_t, [C.c_int32, C.c_int64]),
    "bsx_version": (C.c_char_p, []),
}

_lib = None


def lib() -> C.CDLL:
    """The loaded library; raises if it is missing (build it with `python -m basalt_b200.build`)."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(f"{LIB_PATH} is missing: the CUDA library was not built (python basalt_b200/build.py); "
                               "there is no fallback implementation")
        L = C.CDLL(str(LIB_PATH))
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def exported_symbols():
    return list(_SIGNATURES)


class BsxError(RuntimeError):
    def __init__(self, fn: str, code: int):
        names = {-1: "unsupported geometry", -2: "null stream", -3: "unsupported block format", -4: "bad pointer",
                 -5: "size beyond a fixed limit", -6: "no NCCL library in the process, or NCCL refused the call"}
        super().__init__(f"{fn}: " + (names.get(code, f"CUDA error {code}") if code < 0 else f"CUDA error {code}"))
        self.code = code


def check(fn: str, code: int) -> None:
    if code != 0:
        raise BsxError(fn, code)
