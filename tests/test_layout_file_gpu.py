"""GPU: a synthetic `experts` section written to disk with its `experts.layout` table comes back through
ExpertsSection.load_layer as the very bytes a direct upload gives (raw and packed, whole layers and one rank's block), and a
layer built from the loaded blobs gives the bits of a layer built from the blobs in memory."""
import numpy as np
import pytest
import torch

from basalt_b200 import capi, layout_file as lf, moe
from oracle import oracle as O
from tests.helpers import make_expert_blobs, stack_blobs

pytestmark = pytest.mark.gpu


def test_layers_load_from_a_file_as_direct_uploads(lib, cuda, tmp_path):
    rng = np.random.default_rng(3)
    E, H, I, K, T = 32, 512, 256, 4, 16
    _, nv = make_expert_blobs(rng, E, O.T_NVFP4, O.T_NVFP4, H, I)
    _, q6 = make_expert_blobs(rng, E, O.T_Q6_K, O.T_Q6_K, H, I)
    text = lf.layout_text([(40, 40, -1), (14, 14, -1)], E, H, I)
    table = lf.parse_layout_text(text, 2, E, H, I)
    assert table.total == sum(b.size for b in nv) + sum(b.size for b in q6)
    path = tmp_path / "experts.bin"
    with open(path, "wb") as f:
        f.write(b"\x5a" * 4096)                        # the sections before `experts` in a model file
        for b in nv + q6:
            f.write(b.tobytes())
    sec = lf.ExpertsSection(str(path), table, base_offset=4096)

    for layer, blobs in ((0, nv), (1, q6)):
        got, L = sec.load_layer(layer, cuda, chunk_experts=5)   # 5 does not divide 32: a ragged last chunk, buffers reused
        want = torch.from_numpy(stack_blobs(blobs)).to(cuda)
        assert got.shape == want.shape and torch.equal(got, want)
        assert L.bytes == blobs[0].size
    part, L = sec.load_layer(0, cuda, experts=range(8, 16))
    assert torch.equal(part, torch.from_numpy(stack_blobs(nv[8:16])).to(cuda))

    L = moe.native_expert_layout(40, 40, H, I)
    want_packed = moe.pack_experts(L, torch.from_numpy(stack_blobs(nv)).to(cuda))
    got_packed, _ = sec.load_layer(0, cuda, pack=True, chunk_experts=7)
    torch.cuda.synchronize()
    used = (2 * (I // 128) * (H // 256) + (H // 128) * (I // 256)) * 18432 + 16      # blocks + the fp32 tail; the rest is padding
    assert got_packed.shape == want_packed.shape and torch.equal(got_packed[:, :used], want_packed[:, :used])
    with pytest.raises(ValueError, match="packed path"):
        sec.load_layer(1, cuda, pack=True)

    gate = torch.from_numpy((rng.standard_normal((E, H)) * 0.02).astype(np.float32)).to(cuda)
    args = moe.RouterArgs(n_expert=E, n_embd=H, k=K, weight_scale=1.0, gate=capi.GATE_SOFTMAX)
    x = torch.randn((T, H), device=cuda, generator=torch.Generator(device=cuda).manual_seed(1)).bfloat16()
    a = moe.MoELayer(gate, None, got_packed, L, args, max_tokens=T, packed=True).forward(x).clone()
    b = moe.MoELayer(gate, None, want_packed, L, args, max_tokens=T, packed=True).forward(x).clone()
    torch.cuda.synchronize()
    assert torch.isfinite(a).all() and torch.equal(a.view(torch.int32), b.view(torch.int32))
