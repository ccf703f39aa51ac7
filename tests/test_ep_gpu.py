"""GPU, two ranks over NCCL: the expert-parallel layer (basalt_b200/ep.py) against the single-GPU layer on the same tokens.
Each rank's rows must be bit-identical to what one GPU computes for its tokens: routing is replicated and an expert gives
the same rows whichever rank holds it.  Needs two devices (skipped otherwise); NVLS is switched off for the test processes."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
E, H, I, K, T = 64, 2048, 512, 10, 24


def _weights():
    from oracle import oracle as O
    from tests.helpers import make_expert_blobs, stack_blobs
    rng = np.random.default_rng(3)
    L, blobs = make_expert_blobs(rng, E + 1, O.T_NVFP4, O.T_NVFP4, H, I)
    gate = (rng.standard_normal((E, H)) * 0.02).astype(np.float32)
    return stack_blobs(blobs), gate


def _rank(rank, world, port, q):
    try:
        _rank_body(rank, world, port, q)
    except BaseException:       # the parent shows the child's traceback instead of waiting for a result that never comes
        import traceback
        q.put(("error", rank, traceback.format_exc()))
        raise


def _rank_body(rank, world, port, q):
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    from basalt_b200 import capi, ep, moe
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    blobs, gate = _weights()
    bd = torch.from_numpy(blobs).to(dev)
    gw = torch.from_numpy(gate).to(dev)
    L = moe.native_expert_layout(capi.TYPE_NVFP4, capi.TYPE_NVFP4, H, I)
    args = moe.RouterArgs(n_expert=E, n_embd=H, k=K, weight_scale=1.0, gate=capi.GATE_SOFTMAX)
    g = torch.Generator(device=dev).manual_seed(10 + rank)
    x = torch.randn((T - 5 * rank, H), generator=g, device=dev).bfloat16()      # ragged token counts across ranks
    El = E // world
    own = bd[rank * El:(rank + 1) * El].contiguous()
    layer = ep.EPMoELayerA2A(gw, None, own, L, args, E, shared_blob=bd[E], max_tokens=T)
    y = layer.forward(x).clone()
    y2 = layer.forward(x).clone()
    single = moe.MoELayer(gw, None, bd[:E], L, args, shared_blob=bd[E], max_tokens=T)
    want = single.forward(x).clone()
    # the collective form (fixed sizes: every rank passes T rows): equal to rounding, and stable from run to run
    xf = torch.randn((T, H), generator=g, device=dev).bfloat16()
    coll = ep.EPMoELayer(gw, None, own, L, args, E, shared_blob=bd[E], max_tokens=T)
    yc = coll.forward(xf).clone()
    yc2 = coll.forward(xf).clone()
    wantc = single.forward(xf).clone()
    # hot experts held on every rank (one from each rank's block): a replicated expert's pairs run where their token lives
    reps = {e: bd[e] for e in (3, E // 2 + 5)}
    rep = ep.EPMoELayer(gw, None, own, L, args, E, shared_blob=bd[E], max_tokens=T, replicas=reps)
    yr = rep.forward(xf).clone()
    relr = float((yr - wantc).norm() / wantc.norm())
    assert relr < 1e-5, f"collective form with replicated experts differs from the single-GPU layer (relative L2 {relr})"
    # the collective form over packed blobs (block-scaled FP4 tensor cores), launched kernel by kernel and as a CUDA graph
    mine = moe.pack_experts(L, torch.cat([own, bd[E:E + 1]]))
    pk = ep.EPMoELayer(gw, None, mine[:El], L, args, E, shared_blob=mine[El], max_tokens=T, packed=True)
    ypk = pk.forward(xf).clone()
    pk.capture(xf)
    ypg = pk.forward_graphed(xf).clone()
    # the same step as one C ABI call on a communicator of the caller's own (bsx_ep_layer): the bits of the Python-driven form,
    # in place and over packed blobs, launched and replayed as a graph; with replicated experts too
    comm = ep.NcclComm()
    nat = ep.EPMoELayerNative(gw, None, own, L, args, E, comm, shared_blob=bd[E], max_tokens=T)
    yn = nat.forward(xf).clone()
    assert torch.equal(yn.view(torch.int32), yc.view(torch.int32)), "bsx_ep_layer differs from the Python-driven collective form"
    natp = ep.EPMoELayerNative(gw, None, mine[:El], L, args, E, comm, shared_blob=mine[El], max_tokens=T, packed=True)
    ynp = natp.forward(xf).clone()
    assert torch.equal(ynp.view(torch.int32), ypk.view(torch.int32)), "bsx_ep_layer (packed) differs from the Python-driven collective form"
    natp.capture(xf)
    yng = natp.forward_graphed(xf).clone()
    assert torch.equal(yng.view(torch.int32), ypk.view(torch.int32)), "bsx_ep_layer graph replay differs from the launched step"
    natp.check_status()
    natr = ep.EPMoELayerNative(gw, None, own, L, args, E, comm, shared_blob=bd[E], max_tokens=T, replicas=reps)
    ynr = natr.forward(xf).clone()
    assert torch.equal(ynr.view(torch.int32), yr.view(torch.int32)), "bsx_ep_layer with replicated experts differs from the Python-driven form"
    torch.cuda.synchronize()
    natp.graph.reset()
    del natp
    # the prompt-sized form (tensor-core experts): against the single-GPU prompt layer, and that layer against the decode one
    pre = ep.EPPrefillMoELayer(gw, None, own, L, args, E, shared_blob=bd[E], max_tokens=T)
    yp = pre.forward(xf).clone()
    prep = ep.EPPrefillMoELayer(gw, None, mine[:El], L, args, E, shared_blob=mine[El], max_tokens=T, packed=True)
    ypp = prep.forward(xf).clone()
    single_p = moe.PrefillMoELayer(gw, None, bd[:E], L, args, shared_blob=bd[E], max_tokens=T)
    wantp = single_p.forward(xf).clone()
    torch.cuda.synchronize()
    relc = float((yc - wantc).norm() / wantc.norm())
    relp = float((yp - wantp).norm() / wantp.norm())
    relpd = float((wantp - wantc).norm() / wantc.norm())
    st = int(pre.status.item()) | int(single_p.status.item()) | int(pk.status.item())
    relk = float((ypk - wantc).norm() / wantc.norm())
    relpp = float((ypp - wantc).norm() / wantc.norm())
    st |= int(prep.status.item())
    assert relpp < 2e-3, f"packed expert-parallel prompt layer differs from the single-GPU layer (relative L2 {relpp})"
    assert torch.equal(ypk.view(torch.int32), ypg.view(torch.int32)), "graph replay differs from the launched step"
    assert relk < 1e-3, f"packed collective form differs from the single-GPU layer (relative L2 {relk})"
    q.put((rank, bool(torch.equal(y.view(torch.int32), want.view(torch.int32))), bool(torch.equal(y.view(torch.int32), y2.view(torch.int32))),
           float((y - want).abs().max()), relc, bool(torch.equal(yc.view(torch.int32), yc2.view(torch.int32))), relp, relpd, st))
    torch.cuda.synchronize()
    pk.graph.reset()            # a recorded graph holds the communicator's resources: release it before the group goes away
    del pk
    dist.barrier()
    torch.cuda.synchronize()
    comm.destroy()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_ep_two_gpus_matches_single_gpu(lib):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29900 + os.getpid() % 90
    procs = [ctx.Process(target=_rank, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=140) for _ in procs]
    errs = [r for r in res if r[0] == "error"]
    if errs:
        for p in procs:
            p.join(timeout=20)
            if p.is_alive():
                p.terminate()
        raise AssertionError("rank %d failed:\n%s" % (errs[0][1], errs[0][2]))
    for p in procs:
        p.join(timeout=45)
        if p.is_alive():        # results are in; a rank stuck in its own teardown is not what this test is about
            p.terminate()
            p.join(timeout=10)
    for rank, same, stable, err, relc, stablec, relp, relpd, st in res:
        assert st == 0, f"rank {rank}: a bounded wait inside a prefill kernel gave up"
        assert relp < 1e-5, f"rank {rank}: expert-parallel prompt layer differs from the single-GPU prompt layer (relative L2 {relp})"
        assert relpd < 2e-3, f"rank {rank}: prompt layer differs from the decode layer (relative L2 {relpd})"
        assert stable, f"rank {rank}: all-to-all form not bit-stable from run to run"
        assert same, f"rank {rank}: all-to-all form differs from the single-GPU layer (max abs {err})"
        assert relc < 1e-5, f"rank {rank}: collective form differs from the single-GPU layer (relative L2 {relc})"
        assert stablec, f"rank {rank}: collective form not bit-stable from run to run"


def _single_rank(port, q):
    """one rank, one GPU: the expert-parallel entry with a communicator of size 1 must give the single-GPU layer's rows"""
    try:
        sys.path.insert(0, str(ROOT))
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
        import torch.distributed as dist
        from basalt_b200 import capi, ep, moe
        torch.cuda.set_device(0)
        dev = torch.device("cuda", 0)
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=dev)
        blobs, gate = _weights()
        bd = torch.from_numpy(blobs).to(dev)
        gw = torch.from_numpy(gate).to(dev)
        L = moe.native_expert_layout(capi.TYPE_NVFP4, capi.TYPE_NVFP4, H, I)
        args = moe.RouterArgs(n_expert=E, n_embd=H, k=K, weight_scale=1.0, gate=capi.GATE_SOFTMAX)
        x = torch.randn((T, H), generator=torch.Generator(device=dev).manual_seed(5), device=dev).bfloat16()
        comm = ep.NcclComm()
        packed = moe.pack_experts(L, bd)
        out = []
        for pk, src in ((False, bd), (True, packed)):
            single = moe.MoELayer(gw, None, src[:E], L, args, shared_blob=src[E], max_tokens=T, packed=pk)
            want = single.forward(x).clone()
            nat = ep.EPMoELayerNative(gw, None, src[:E], L, args, E, comm, shared_blob=src[E], max_tokens=T, packed=pk)
            got = nat.forward(x).clone()
            nat.check_status()
            nat.capture(x)
            rep = nat.forward_graphed(x).clone()
            torch.cuda.synchronize()
            out.append((float((got - want).norm() / want.norm()), bool(torch.equal(got.view(torch.int32), rep.view(torch.int32))),
                        bool(torch.equal(nat_ids(nat, capi), single.ids[:T]))))
            nat.graph.reset()
            del nat
        q.put(("ok", out))
        comm.destroy()
        dist.destroy_process_group()
    except BaseException:
        import traceback
        q.put(("error", traceback.format_exc()))
        raise


def nat_ids(nat, capi):
    """the ids the one-call step left in its workspace (bsx_ep_layer_views)"""
    import ctypes as C
    v = capi.MoELayerViews()
    capi.check("bsx_ep_layer_views", capi.lib().bsx_ep_layer_views(C.byref(nat.desc), nat.max_tokens, nat.world, nat.workspace.data_ptr(), C.byref(v)))
    n = nat.max_tokens * nat.args.k
    off = (v.ids - nat.workspace.data_ptr()) // 4
    return nat.workspace.view(torch.int32)[off:off + n].view(nat.max_tokens, nat.args.k)


def test_ep_entry_with_one_rank_is_the_single_gpu_layer(lib, cuda):
    """bsx_ep_layer on a communicator of one rank (every expert local, collectives of size one): the rows of the single-GPU layer
    to fp32 rounding, the same routing, and a graph replay with the launched step's bits.  Runs on one GPU."""
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    p = ctx.Process(target=_single_rank, args=(29990 - os.getpid() % 80, q))
    p.start()
    res = q.get(timeout=180)
    p.join(timeout=45)
    if p.is_alive():
        p.terminate()
    assert res[0] == "ok", res[1]
    for rel, same_graph, same_ids in res[1]:
        assert rel < 1e-5 and same_graph and same_ids, res[1]
