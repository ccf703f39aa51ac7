"""GPU: the dispatch entry point that brings its own scratch (bsx_dispatch_static).

It exists for hosts that cannot give the library scratch memory - an engine that carved all device memory into its own
arenas at start-up, or a caller on a path where the CUDA allocator is off limits - so the test allocates nothing between
its two calls and checks each against bsx_dispatch (caller-provided scratch) on the same ids: cnt, off, slot and src must
be identical, call after call, although both calls share the library's one resident table.  Collected last on purpose."""
import numpy as np
import pytest
import torch

from basalt_b200 import capi, moe

pytestmark = pytest.mark.gpu


def _ids(rng, T, k, E):
    p = 1.0 / np.arange(1, E + 1) ** 1.1
    lg = np.log(p)[None, :] + rng.gumbel(size=(T, E))
    ids = np.argsort(-lg, axis=1)[:, :k].astype(np.int32)
    ids[1, 0] = -1     # a dropped pair gets no row
    return ids.reshape(-1)


def test_static_scratch_dispatch_matches_dispatch_twice(lib, cuda):
    rng = np.random.default_rng(2026)
    E, k = 512, 10
    st = torch.cuda.Stream()
    calls = [(4096, _ids(rng, 4096, k, E)), (77, _ids(rng, 77, k, E))]      # a large call, then a small one over the stale table
    dev_ids = [torch.from_numpy(i).cuda() for _, i in calls]
    outs = [[torch.empty(n, dtype=torch.int32, device="cuda") for n in (E, E + 1, ids.size, ids.size)] for _, ids in calls]
    for o in outs:
        o[3].fill_(-1)
    torch.cuda.synchronize()
    for d, o in zip(dev_ids, outs):                                          # two calls in a row, nothing allocated in between
        rc = lib.bsx_dispatch_static(d.data_ptr(), d.numel(), k, E, o[0].data_ptr(), o[1].data_ptr(), o[2].data_ptr(), o[3].data_ptr(),
                                     st.cuda_stream)
        assert rc == 0, rc
    st.synchronize()
    for d, o in zip(dev_ids, outs):
        with torch.cuda.stream(st):
            cnt, off, slot, src, _, _ = moe.dispatch(d, k, E, stream=st)
        st.synchronize()
        rows = int(off[-1].item())
        assert torch.equal(o[0], cnt) and torch.equal(o[1], off) and torch.equal(o[2], slot)
        assert torch.equal(o[3][:rows], src[:rows])


def test_static_scratch_dispatch_refuses_what_does_not_fit(lib, cuda):
    st = torch.cuda.Stream()
    assert lib.bsx_dispatch_static(1, 65537, 10, 512, 1, 1, 1, 1, st.cuda_stream) == capi.E_LIMIT
    assert lib.bsx_dispatch_static(1, 64, 10, 2048, 1, 1, 1, 1, st.cuda_stream) == capi.E_LIMIT      # more experts than the resident table covers
    assert lib.bsx_dispatch_static(1, 64, 10, 512, 1, 1, 1, 1, None) == capi.E_STREAM
