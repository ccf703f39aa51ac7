"""CPU, two gloo ranks: the expert-parallel exchange logic (basalt_b200/ep.py: split sizes, the receive-side group plan, the
two all-to-alls) with the oracle standing in for the kernels.  Every rank's output must equal the single-process oracle
layer on its own tokens (to 1e-6: the oracle's BLAS products round differently for different batch shapes; on the GPU an
expert gives bit-identical rows whichever rank holds it)."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

E, H, I, K, WORLD = 32, 256, 256, 2, 2
TOKENS = [5, 3]     # ragged: the ranks hold different numbers of tokens


def _layer(seed=0):
    from oracle import oracle as O
    from tests.helpers import make_expert_blobs
    rng = np.random.default_rng(seed)
    L, blobs = make_expert_blobs(rng, E + 1, O.T_NVFP4, O.T_NVFP4, H, I)
    gate = (rng.standard_normal((E, H)) * 0.02).astype(np.float32)
    xs = [rng.standard_normal((t, H)).astype(np.float32) for t in TOKENS]
    return L, blobs, gate, xs


def _rank(rank, world, port, q):
    import torch
    import torch.distributed as dist
    from basalt_b200 import ep
    from oracle import oracle as O
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    L, blobs, gate, xs = _layer()
    x = xs[rank]
    T = x.shape[0]
    first = ep.ep_partition(E, world)
    ids, w = O.router_select(O.router_logits(x, gate), None, K, O.GATE_SOFTMAX)
    cnt, off, slot, src, _ = O.dispatch(ids, K, E)
    cnt_all = [torch.zeros(E, dtype=torch.int32) for _ in range(world)]
    dist.all_gather(cnt_all, torch.from_numpy(cnt))
    cnt_all = torch.stack(cnt_all).numpy()
    send, recv = ep.ep_splits(cnt_all, rank)
    experts, start, rows = ep.ep_recv_plan(cnt_all, rank)
    n = T * K
    xs_send = torch.from_numpy(x[src[:n]])
    xr = torch.zeros((int(recv.sum()), H))
    dist.all_to_all_single(xr, xs_send, recv.tolist(), send.tolist())
    out = torch.zeros_like(xr)
    for g, e in enumerate(experts):
        assert first[rank] <= e < first[rank + 1]
        r = rows[start[g]:start[g + 1]]
        out[r] = torch.from_numpy(O.expert_forward(L, blobs[e], xr.numpy()[r]))
    back = torch.zeros((n, H))
    dist.all_to_all_single(back, out, send.tolist(), recv.tolist())
    y = O.combine(back.numpy(), slot.reshape(T, K), w, O.expert_forward(L, blobs[E], x))
    want = O.moe_layer(x, gate, None, blobs[:E], L, K, O.GATE_SOFTMAX, shared_blob=blobs[E])[0]
    err = float(np.linalg.norm(y.astype(np.float64) - want) / np.linalg.norm(want))
    q.put((rank, err < 1e-6, int(recv.sum()), int(send.sum())))
    dist.destroy_process_group()


def test_ep_two_ranks_gloo():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 400
    procs = [ctx.Process(target=_rank, args=(r, WORLD, port, q)) for r in range(WORLD)]
    for p in procs:
        p.start()
    res = [q.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(r[0] for r in res) == [0, 1]
    assert all(r[1] for r in res), res
    assert sum(r[2] for r in res) == sum(r[3] for r in res) == sum(TOKENS) * K


def test_ep_plan_properties():
    from basalt_b200 import ep
    rng = np.random.default_rng(1)
    world, Et = 4, 32
    cnt_all = rng.integers(0, 5, size=(world, Et)).astype(np.int32)
    cnt_all[:, 3] = 0          # an expert nobody chose
    tot_send = np.zeros((world, world), np.int64)
    for r in range(world):
        send, recv = ep.ep_splits(cnt_all, r)
        tot_send[r] = send
        experts, start, rows = ep.ep_recv_plan(cnt_all, r)
        assert sorted(rows.tolist()) == list(range(int(recv.sum())))          # every received row is used exactly once
        assert 3 not in experts.tolist()
        lo = r * (Et // world)
        for g, e in enumerate(experts):
            assert start[g + 1] - start[g] == cnt_all[:, e].sum() and lo <= e < lo + Et // world
            seg = rows[start[g]:start[g + 1]]
            assert (np.diff(seg) > 0).all()                                    # source-rank order, then pair order
    for r in range(world):
        assert np.array_equal(ep.ep_splits(cnt_all, r)[1], tot_send[:, r])     # what r receives is what the others send it


def test_replica_choice_balances_a_skewed_load():
    """Hot-expert replication: with Zipf-like routing the owner of the popular experts gets most rows; holding the few most
    loaded experts on every rank moves their pairs to the tokens' own ranks and evens the rows out."""
    from basalt_b200 import ep
    rng = np.random.default_rng(0)
    E, W, T, k = 64, 4, 128, 4
    p = 1.0 / np.arange(1, E + 1) ** 1.1
    ids = np.stack([rng.choice(E, k, replace=False, p=p / p.sum()) for _ in range(W * T)]).astype(np.int32)
    load = np.bincount(ids.reshape(-1), minlength=E)
    plain = ep.ep_rank_rows(ids, T, E, W)
    assert plain.sum() == ids.size and plain[0] > 1.8 * plain.mean()          # rank 0 owns the popular experts
    reps = ep.choose_replicas(load, W, 6)
    assert reps.tolist() == sorted(np.argsort(-load, kind="stable")[:6].tolist())
    bal = ep.ep_rank_rows(ids, T, E, W, reps)
    assert bal.sum() == ids.size
    assert bal.max() / bal.mean() < 0.75 * plain.max() / plain.mean()
    assert ep.choose_replicas(load, W, 0).size == 0
