"""GPU: a C++ program that includes only the reference-signature shim (include/basalt_shim.hpp) and the CUDA runtime runs a
decode-window step and the prompt path's group call on the device; its outputs equal, bit for bit, the same calls made through
ctypes - the drop-in claim exercised from the language the reference's callers are written in.  Also: the dense gated MLP
entry (bsx_gated_mlp) on one GPU."""
import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np
import pytest
import torch

from basalt_b200 import capi, moe
from oracle import oracle as O
from tests.helpers import make_expert_blobs, rel_l2, stack_blobs

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def test_cpp_caller_through_the_shim_on_the_gpu(lib, cuda, tmp_path):
    cuda_home = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))
    exe = tmp_path / "shim_gpu"
    libdir = ROOT / "basalt_b200" / "lib"
    subprocess.check_call(["g++", "-std=c++17", "-O1", "-I", str(ROOT / "include"), "-I", str(cuda_home / "include"), str(ROOT / "tests" / "cpp" / "shim_gpu.cpp"),
                           "-L", str(libdir), "-lbasalt_b200", "-L", str(cuda_home / "lib64"), "-lcudart", f"-Wl,-rpath,{libdir}", f"-Wl,-rpath,{cuda_home / 'lib64'}",
                           "-o", str(exe)])
    rng = np.random.default_rng(21)
    E, H, I, k, T = 64, 1024, 512, 4, 24
    Lo, blobs = make_expert_blobs(rng, E, 40, 40, H, I)
    sb = stack_blobs(blobs)
    gate = (rng.standard_normal((E, H)) * 0.02).astype(np.float32)
    x = rng.standard_normal((T, H)).astype(np.float32)
    with open(tmp_path / "in.bin", "wb") as f:
        f.write(np.array([E, H, I, k, T, sb.shape[1]], np.int32).tobytes())
        f.write(gate.tobytes()); f.write(x.tobytes()); f.write(sb.tobytes())
    out = subprocess.run([str(exe), str(tmp_path / "in.bin"), str(tmp_path / "out.bin")], capture_output=True, text=True)
    assert out.returncode == 0, out.stdout + out.stderr
    raw = np.fromfile(tmp_path / "out.bin", np.uint8)
    n = T * k
    sizes = [T * E * 4, n * 4, n * 4, T * H * 4, n * H * 4, n * 4, T * H * 4]
    parts = np.split(raw, np.cumsum(sizes)[:-1])
    c_logits, c_ids, c_w = parts[0].view(np.float32).reshape(T, E), parts[1].view(np.int32).reshape(T, k), parts[2].view(np.float32).reshape(T, k)
    c_y, c_dm = parts[3].view(np.float32).reshape(T, H), parts[4].view(np.float32).reshape(n, H)
    # the one-call layer from C++ (bsx_moe_layer): the routing of the call-by-call sequence to the bit, and the bits of the same
    # call made through ctypes; its rows sit within the q8_1 rounding (1e-2) of the call-by-call sequence's
    c_ids1, c_y1 = parts[5].view(np.int32).reshape(T, k), parts[6].view(np.float32).reshape(T, H)
    assert np.array_equal(c_ids1, c_ids)
    assert rel_l2(c_y1, c_y) < 3e-2
    # the same calls through ctypes
    a = moe.RouterArgs(n_expert=E, n_embd=H, k=k, weight_scale=2.5, gate=capi.GATE_SIGMOID)
    dx, bd = dev(x), dev(sb)
    lg, ids, w = moe.router(dx, dev(gate), None, a)
    table = (bd.data_ptr() + torch.arange(E, dtype=torch.int64) * sb.shape[1]).cuda()
    ptr, start, ng, dst, tok = moe.moe_plan(ids.reshape(-1), k, E, table)
    L = moe.native_expert_layout(40, 40, H, I)
    q8 = moe.quantize_q8_1_rows(dx)
    rows = torch.zeros((n, H), dtype=torch.float32, device="cuda")
    scratch = torch.empty(moe.native_expert_scratch_bytes(L, n), dtype=torch.uint8, device="cuda")
    moe.native_expert_grouped(L, ptr, start, ng, dst, tok, min(n, E), n, q8, scratch, rows)
    y = moe.moe_combine(rows, None, w)
    torch.cuda.synchronize()
    assert np.array_equal(c_logits.view(np.uint32), lg.cpu().numpy().view(np.uint32))
    assert np.array_equal(c_ids, ids.cpu().numpy()) and np.array_equal(c_w.view(np.uint32), w.cpu().numpy().view(np.uint32))
    assert np.array_equal(c_y.view(np.uint32), y.cpu().numpy().view(np.uint32))
    one = moe.NativeMoELayer(dev(gate), None, bd, L, a, max_tokens=T)
    y_one = one.forward(dx).cpu().numpy()
    assert np.array_equal(c_y1.view(np.uint32), y_one.view(np.uint32))
    # the prompt path's rows: the dispatch + bsx_experts_prefill through ctypes give the same bits, and the oracle agrees
    cnt, off, slot, src, tiles, n_tiles = moe.dispatch(ids.reshape(-1), k, E, tile_rows=128)
    dm, status = moe.experts_prefill(L, table, off, src, tiles, n_tiles, dx, n)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert np.array_equal(c_dm.view(np.uint32), dm.cpu().numpy().view(np.uint32))
    offh, srch = off.cpu().numpy(), src.cpu().numpy()
    for e in range(0, E, 7):
        if offh[e + 1] > offh[e]:
            want = O.expert_forward(Lo, blobs[e], x[srch[offh[e]:offh[e + 1]]])
            assert rel_l2(c_dm[offh[e]:offh[e + 1]], want) < 2e-3


@pytest.mark.parametrize("gt,H,I,T", [(40, 2048, 512, 9), (14, 2048, 512, 5)])
def test_gated_mlp_is_the_one_group_grouped_call(lib, cuda, gt, H, I, T):
    """bsx_gated_mlp (Basalt: gated_mlp_clamped, include/basalt/kernels/iq_kernels.hpp:93-98): a shared expert as a dense gated MLP."""
    rng = np.random.default_rng(gt + T)
    Lo, blobs = make_expert_blobs(rng, 1, gt, gt, H, I)
    L = moe.native_expert_layout(gt, gt, H, I)
    bd = dev(stack_blobs(blobs))
    x = rng.standard_normal((T, H)).astype(np.float32)
    out = moe.gated_mlp(L, bd[0], dev(x), cap_tok=16).cpu().numpy()
    want = O.expert_forward(Lo, blobs[0], x)
    assert rel_l2(out, want) < 2e-3
    # a clamp in the layout is honoured
    Lc = moe.native_expert_layout(gt, gt, H, I, swiglu_limit=0.05)
    outc = moe.gated_mlp(Lc, bd[0], dev(x), cap_tok=16).cpu().numpy()
    wantc = O.expert_forward(Lo, blobs[0], x, limit=0.05)
    assert rel_l2(outc, wantc) < 2e-3
