"""CPU: the C ABI library loads, exports every symbol include/basalt_b200.h declares, and its host-side logic (block
decoders compiled for the host, blob geometry, argument checks) agrees with the oracle.  No compute call needs a GPU here."""
import ctypes as C
import re
from pathlib import Path

import numpy as np
import pytest

from basalt_b200 import capi
from oracle import oracle as O

ROOT = Path(__file__).resolve().parent.parent
G = np.load(Path(__file__).parent / "golden" / "ref_vectors.npz")


def test_every_declared_symbol_is_exported(lib):
    header = (ROOT / "include" / "basalt_b200.h").read_text()
    declared = set(re.findall(r"BSX_API\s+[\w\s\*]+?\b(bsx_\w+)\s*\(", header))
    assert declared, "no declarations parsed"
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared but not exported"
    assert declared == set(capi.exported_symbols()), declared ^ set(capi.exported_symbols())


@pytest.mark.parametrize("name,t", [("nvfp4", 40), ("q6k", 14), ("iq1m", 29), ("q8_0", 8), ("q4k", 12), ("q5k", 13), ("q5_0", 6), ("q5_1", 7), ("iq4nl", 20), ("iq4xs", 23), ("q2_0", 42), ("q2k", 10), ("q3k", 11), ("iq2xxs", 16), ("iq2xs", 17), ("iq2s", 22), ("iq3xxs", 18), ("iq3s", 21), ("iq1s", 19)])
def test_host_decoders_match_reference_golden(lib, name, t):
    raw, want = np.ascontiguousarray(G[f"dec_{name}_raw"]), G[f"dec_{name}_f32"]
    got = np.empty(want.size, np.float32)
    assert lib.bsx_host_decode_row(t, raw.ctypes.data, got.ctypes.data, want.size) == 0
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_layout_matches_reference_geometry(lib):
    for row in G["geometry"]:
        gt, dt, H, I, gu_row, d_row, up_off, down_off, nbytes, tail = [int(v) for v in row]
        L = capi.ExpertLayout()
        assert lib.bsx_expert_layout_init(gt, dt, -1, H, I, 0.0, 0.0, 0.0, C.byref(L)) == 0
        assert (L.gu_row, L.d_row, L.up_off, L.down_off, L.bytes) == (gu_row, d_row, up_off, down_off, nbytes)
    # the benchmark shapes the reference's CPU pool refuses but its GPU layout accepts (probed blob sizes)
    for cfg, nbytes in (((40, 40, 7168, 2048), 24772624), ((29, 29, 7168, 2048), 9633792), ((14, 14, 2048, 512), 2580480),
                        ((40, 40, 2048, 512), 1769488)):
        L = capi.ExpertLayout()
        assert lib.bsx_expert_layout_init(cfg[0], cfg[1], -1, cfg[2], cfg[3], 0.0, 0.0, 0.0, C.byref(L)) == 0
        assert L.bytes == nbytes


def test_argument_errors(lib):
    L = capi.ExpertLayout()
    assert lib.bsx_expert_layout_init(9, 40, -1, 2048, 512, 0.0, 0.0, 0.0, C.byref(L)) == capi.E_TYPE
    assert lib.bsx_expert_layout_init(40, 40, -1, 2000, 512, 0.0, 0.0, 0.0, C.byref(L)) == capi.E_TYPE
    assert lib.bsx_expert_supported(40, 40, -1, 2048, 512) == 1
    assert lib.bsx_expert_supported(40, 40, 14, 2048, 512) == 0
    assert lib.bsx_router_logits(None, None, 4, 100, 2048, None, None) == capi.E_GEOMETRY     # E % 32
    assert lib.bsx_router_logits(None, None, 4, 64, 2000, None, None) == capi.E_GEOMETRY      # H % 128
    assert lib.bsx_router_select(1, None, 4, 64, 17, capi.GATE_SIGMOID, 1.0, 1, 1, 0.0, None, 0, 1, 1, None) == capi.E_GEOMETRY
    assert lib.bsx_router_select(1, None, 4, 64, 8, capi.GATE_SIGMOID, 1.0, 16, 1, 0.0, None, 0, 1, 1, None) == capi.E_GEOMETRY
    assert lib.bsx_dispatch(None, 16, 2, 8, 1, 1, 1, 1, 0, None, None, 1, None) == capi.E_STREAM
    assert lib.bsx_moe_plan(None, 1025, 1, 8, None, None, None, None, None, None, 1) == capi.E_LIMIT
    assert lib.bsx_combine(None, None, None, None, None, 4, 2, 8, None, None) == capi.E_STREAM
    assert lib.bsx_experts_grouped(C.byref(L), None, None, None, None, None, 1, 1, None, 0, None, None, 0, None) == capi.E_STREAM
    assert lib.bsx_route_tail_skip(None, None, None, 0, 200, 4, 1, 8, None, None) == capi.OK   # out of range: a no-op
    assert lib.bsx_row_bytes(40, 2048) == 1152 and lib.bsx_row_bytes(14, 512) == 420 and lib.bsx_row_bytes(29, 100) == 0
    assert lib.bsx_dispatch_scratch_bytes(163840, 512) >= 163840 // 256 * 512 * 4
    assert lib.bsx_expert_layout_init(40, 40, -1, 2048, 512, 0.0, 0.0, 0.0, C.byref(L)) == 0
    assert lib.bsx_expert_scratch_bytes(C.byref(L), 640) >= 640 * 512 * 4 * 2 + 640 * 2048 * 4


def test_nvfp4_packer_matches_oracle():
    import torch
    from basalt_b200 import pack
    g = torch.Generator().manual_seed(0)
    w = torch.randn(16, 1024, generator=g) * 0.02
    w = (w / (w.abs().max() / (6 * 448))).float()
    w[0, :16] = 0
    assert np.array_equal(pack.quantize_nvfp4(w).numpy().reshape(-1), O.quantize(40, w.numpy()))
    L = O.Layout(40, 40, 256, 128)
    Gm, U, D = torch.randn(128, 256, generator=g) * 0.02, torch.randn(128, 256, generator=g) * 0.02, torch.randn(256, 128, generator=g) * 0.02
    assert np.array_equal(pack.pack_nvfp4_expert(Gm, U, D).numpy(), O.make_blob(L, Gm.numpy(), U.numpy(), D.numpy()))


def test_expert_parallel_entry_host_side(lib):
    """bsx_ep_layer's host logic without a GPU: NCCL is found in the process (torch loads it), the workspace size follows the
    descriptor, bad descriptors are refused, and a null stream or communicator is an argument error before anything is launched."""
    from basalt_b200 import moe
    assert lib.bsx_ep_available() in (0, 1)
    d = capi.EPLayerDesc()
    d.layout = moe.native_expert_layout(capi.TYPE_NVFP4, capi.TYPE_NVFP4, 2048, 512)
    d.n_expert, d.top_k, d.gate_kind, d.n_group, d.topk_group, d.packed = 512, 10, capi.GATE_SOFTMAX, 1, 1, 1
    d.e_lo, d.n_local, d.n_replicas, d.weight_scale = 128, 128, 0, 1.0
    d.shared_blob = 4096
    w4, w8 = lib.bsx_ep_layer_workspace_bytes(C.byref(d), 64, 4), lib.bsx_ep_layer_workspace_bytes(C.byref(d), 64, 8)
    assert 0 < w4 < w8
    assert lib.bsx_ep_layer_workspace_bytes(C.byref(d), 64, 16) == 0          # 16 x 64 x 10 pairs: beyond the plan's limit
    d.e_lo = 448                                                               # the block would end past the last expert
    assert lib.bsx_ep_layer_workspace_bytes(C.byref(d), 64, 4) == 0
    d.e_lo = 128
    assert lib.bsx_ep_layer(C.byref(d), None, None, capi.X_BF16, 64, None, None, None, None, None, None, None) == capi.E_STREAM
    if lib.bsx_ep_available():
        assert lib.bsx_ep_layer(C.byref(d), None, None, capi.X_BF16, 64, None, None, None, 1, None, None, None) == capi.E_POINTER
    else:
        assert lib.bsx_ep_layer(C.byref(d), None, None, capi.X_BF16, 64, None, None, None, 1, None, None, None) == capi.E_UNAVAILABLE
