"""GPU parity of dispatch: counts, offsets, the stable permutation, the tile list and the decode-window plan, all bit-exact
with the oracle's restatement of the reference's host counting sort."""
import numpy as np
import pytest
import torch

from basalt_b200 import moe
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("T,k,E", [(0, 8, 64), (1, 1, 8), (7, 3, 32), (64, 10, 512), (625, 8, 256), (4096, 10, 512), (16384, 10, 512),
                                   (999, 4, 1024), (300, 6, 384)])
def test_dispatch_bit_exact(lib, cuda, T, k, E):
    rng = np.random.default_rng(T + E)
    if T:
        p = 1.0 / np.arange(1, E + 1) ** 1.1                      # Zipf(1.1) expert popularity -> ragged tiles
        lg = np.log(p)[None, :] + rng.gumbel(size=(T, E))
        ids = np.argsort(-lg, axis=1)[:, :k].astype(np.int32)
        if T > 5:
            ids[3, 0] = -1                                         # a tail-skipped pair
            ids[5, k - 1] = E + 3                                  # an out-of-range id is treated the same way
    else:
        ids = np.zeros((0, k), np.int32)
    cnt, off, slot, src, tiles, nt = moe.dispatch(dev(ids.reshape(-1)) if T else torch.zeros(0, dtype=torch.int32, device="cuda"), k, E, tile_rows=64)
    ocnt, ooff, oslot, osrc, otiles = O.dispatch(ids, k, E, tile_rows=64)
    assert np.array_equal(cnt.cpu().numpy(), ocnt)
    assert np.array_equal(off.cpu().numpy(), ooff)
    assert np.array_equal(slot.cpu().numpy(), oslot)
    n_rows = int(ooff[-1])
    assert np.array_equal(src.cpu().numpy()[:n_rows], osrc[:n_rows])
    n = int(nt.item())
    assert n == len(otiles)
    assert np.array_equal(tiles.cpu().numpy()[:n], otiles.reshape(-1, 2))
    # size-independent properties: slot is a bijection of the valid pairs onto [0, rows), expert-sorted and stable
    flat = ids.reshape(-1)
    valid = (flat >= 0) & (flat < E)
    s = slot.cpu().numpy()
    assert sorted(s[valid].tolist()) == list(range(n_rows))
    order = np.argsort(s[valid], kind="stable")
    e_sorted = flat[valid][order]
    assert (np.diff(e_sorted) >= 0).all()
    pair_idx = np.nonzero(valid)[0][order]
    same = np.diff(e_sorted) == 0
    assert (np.diff(pair_idx)[same] > 0).all()


@pytest.mark.parametrize("T,k,E", [(1, 10, 512), (8, 10, 512), (64, 10, 512), (64, 8, 256), (3, 6, 384), (102, 10, 64)])
def test_moe_plan_bit_exact(lib, cuda, T, k, E):
    rng = np.random.default_rng(T * 7 + E)
    ids = np.stack([rng.permutation(E)[:k] for _ in range(T)]).astype(np.int32)
    blobs = (np.arange(E, dtype=np.uint64) + 1) * 65536
    blobs[rng.integers(0, E, 3)] = 0          # experts this card does not hold
    ptr, start, ng, dst, tok = moe.moe_plan(dev(ids.reshape(-1)), k, E, dev(blobs.view(np.int64)))
    optr, ostart, ong, odst, otok = O.moe_plan(ids, k, E, blobs)
    g = int(ng.item())
    assert g == ong
    assert np.array_equal(ptr.cpu().numpy()[:g].view(np.uint64), optr[:g])
    assert np.array_equal(start.cpu().numpy()[:g + 2], ostart[:g + 2])
    n = int(ostart[g])
    assert np.array_equal(dst.cpu().numpy()[:n], odst[:n]) and np.array_equal(tok.cpu().numpy()[:n], otok[:n])


def test_tiles_from_bounds_equals_the_dispatch_tile_list(lib, cuda):
    """bsx_tiles_from_bounds on a dispatch's row bounds gives the tile list bsx_dispatch itself made."""
    from basalt_b200 import capi, moe
    rng = np.random.default_rng(3)
    E, k, T = 40, 4, 700
    ids = rng.integers(0, E, (T, k)).astype(np.int32)
    ids[:, 0] = 7                                  # one hot expert: several tiles
    ids[ids == 11] = 12                            # and an empty one
    d = torch.from_numpy(ids.reshape(-1)).cuda()
    cnt, off, slot, src, tiles, n_tiles = moe.dispatch(d, k, E, tile_rows=128)
    tiles2 = torch.full_like(tiles, -1)
    n2 = torch.zeros(1, dtype=torch.int32, device="cuda")
    capi.check("tiles", lib.bsx_tiles_from_bounds(off.data_ptr(), E, 128, tiles2.data_ptr(), n2.data_ptr(), moe._stream(None)))
    torch.cuda.synchronize()
    n = int(n_tiles.item())
    assert int(n2.item()) == n and n > E - 2
    assert torch.equal(tiles[:n], tiles2[:n])
