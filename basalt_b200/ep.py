"""Expert parallelism for the MoE layer: one process per GPU, experts sharded in contiguous blocks, tokens data-parallel,
rows exchanged by an all-to-all over NCCL (NVLink / NVSwitch) before and after the local grouped experts.

The reference shards experts across cards too ("expert tiers"), but moves rows through mapped host memory and doorbells
(Basalt: include/basalt/models/qwen4exp/kernels/dec_moe.hpp:1-11, src/core/peer_experts.cpp:420-548); this replaces that
transport with collectives and keeps its correctness argument - an expert gives the same rows on whichever card holds it
(include/basalt/core/peer_experts.hpp:11-12).

Step on rank r of N (router weights replicated, experts [r E/N, (r+1) E/N) local):
  1. route the rank's own tokens; stable dispatch by expert id (rows come out grouped by destination rank);
  2. all-gather the per-expert counts, from which every rank derives both directions' split sizes and its receive-side
     group plan (entries ordered by source rank, then pair order: deterministic);
  3. gather the activation rows in send order and all-to-all them;
  4. run the local grouped experts over the received rows (they sit in local HBM: no peer-memory loads in any kernel);
  5. all-to-all the result rows back (the mirror of 3) and combine them, with the locally computed shared expert.
That is EPMoELayerA2A.  EPMoELayer is the low-latency form for decode-sized steps, with fixed-size collectives and no host
round trip: all-gather the activations and the routing (a few MB), dispatch ALL pairs on every rank, run only the local
experts' groups (bsx_plan_groups skips experts held elsewhere), sum each token's local pairs (bsx_combine_partial) and
reduce-scatter the partial sums to the tokens' owners.  The cross-rank sum is NCCL's, so results match the single-GPU
layer to rounding, not bit for bit.

The planning functions are pure numpy so that the same code is exercised by the CPU tests (gloo, world_size 2) and the
GPU path.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple

import numpy as np


def ep_partition(n_expert: int, world: int) -> np.ndarray:
    """first expert of each rank's block (world + 1 entries); blocks are contiguous and equal."""
    assert n_expert % world == 0, "experts must divide evenly over the ranks"
    return np.arange(world + 1, dtype=np.int64) * (n_expert // world)


def choose_replicas(load: np.ndarray, world: int, n_replicas: int) -> np.ndarray:
    """Which experts to hold on every rank: the n_replicas most loaded ones (load[e] = pairs per step, e.g. a running count of
    the router's choices), ties to the lower id - the experts whose rows would otherwise all land on their one owner.  Returns
    their ids, ascending.  Basalt decides residency from the same kind of counts (include/basalt/core/tier_policy.hpp)."""
    load = np.asarray(load, np.float64)
    n = int(min(max(n_replicas, 0), load.size))
    order = np.lexsort((np.arange(load.size), -load))[:n]
    return np.sort(order).astype(np.int64)


def ep_rank_rows(ids_all: np.ndarray, tokens_per_rank: int, n_expert: int, world: int, replicated=()) -> np.ndarray:
    """rows each rank computes for gathered routing ids_all [world * tokens_per_rank][k]: an expert's pairs go to its owner, a
    replicated expert's pairs to the rank that owns the token.  The balance check of a replica choice."""
    first = ep_partition(n_expert, world)
    rep = np.zeros(n_expert, bool)
    rep[list(replicated)] = True
    ids = np.asarray(ids_all)
    tok_rank = np.repeat(np.arange(world), tokens_per_rank)[:, None] * np.ones_like(ids)
    owner = np.searchsorted(first, ids, side="right") - 1
    where = np.where(rep[np.clip(ids, 0, n_expert - 1)], tok_rank, owner)
    valid = (ids >= 0) & (ids < n_expert)
    return np.bincount(where[valid].reshape(-1), minlength=world)


def ep_splits(cnt_all: np.ndarray, rank: int) -> Tuple[np.ndarray, np.ndarray]:
    """cnt_all [N][E] = every rank's per-expert pair counts.  Returns (send_splits, recv_splits): rows this rank sends to /
    receives from each rank."""
    world, E = cnt_all.shape
    first = ep_partition(E, world)
    send = np.array([cnt_all[rank, first[d]:first[d + 1]].sum() for d in range(world)], np.int64)
    recv = np.array([cnt_all[s, first[rank]:first[rank + 1]].sum() for s in range(world)], np.int64)
    return send, recv


def ep_recv_plan(cnt_all: np.ndarray, rank: int):
    """The receive-side group plan.  Rows arrive ordered by (source rank, expert, pair order).  Returns
    (experts, start, rows): the local experts that received rows (ascending), start[g] = first entry of group g
    (len(experts) + 1 entries), rows[entry] = index of the entry's row in the receive buffer.  Inside a group the entries
    run by source rank, then in the source's pair order."""
    world, E = cnt_all.shape
    first = ep_partition(E, world)
    lo, hi = int(first[rank]), int(first[rank + 1])
    c = cnt_all[:, lo:hi].astype(np.int64)                       # [src][local expert]
    src_base = np.concatenate([[0], np.cumsum(c.sum(1))])[:-1]   # first receive row of each source
    within = np.cumsum(c, axis=1) - c                            # offset of expert e inside source s's rows
    tot = c.sum(0)
    experts = np.nonzero(tot)[0]
    start = np.concatenate([[0], np.cumsum(tot[experts])]).astype(np.int32)
    rows = np.empty(int(start[-1]), np.int32)
    at = 0
    for e in experts:
        for s in range(world):
            n = int(c[s, e])
            if n:
                b = int(src_base[s] + within[s, e])
                rows[at:at + n] = np.arange(b, b + n, dtype=np.int32)
                at += n
    return (experts + lo).astype(np.int32), start, rows


class EPMoELayerA2A:
    """The expert-parallel layer on one rank, row all-to-all form (host-planned: one device-to-host read of the counts per
    step, so it suits prompt-sized steps; every row is bit-identical to the single-GPU layer's).  `blobs` holds this rank's experts only ([E/N][stride] uint8); the router gate,
    bias and the shared expert are replicated."""

    def __init__(self, gate_w, bias, blobs, layout, args, n_expert_total: int, shared_blob=None, max_tokens: int = 64,
                 max_recv_rows: Optional[int] = None, group=None):
        import torch
        import torch.distributed as dist
        from . import moe
        self.torch, self.dist, self.moe = torch, dist, moe
        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.E, self.L, self.args = n_expert_total, layout, args
        self.first = ep_partition(n_expert_total, self.world)
        self.gate_w, self.bias, self.blobs, self.shared_blob = gate_w, bias, blobs, shared_blob
        dev = blobs.device
        self.dev = dev
        El, stride = blobs.shape
        assert El == n_expert_total // self.world
        self.blob_addr = blobs.data_ptr() + np.arange(El, dtype=np.int64) * stride
        n = max_tokens * args.k
        self.max_tokens, self.n_pairs = max_tokens, n
        self.max_recv = max_recv_rows or n * self.world
        f32, i32 = torch.float32, torch.int32
        self.logits = torch.empty((max_tokens, n_expert_total), dtype=f32, device=dev)
        self.ids = torch.empty((max_tokens, args.k), dtype=i32, device=dev)
        self.w = torch.empty((max_tokens, args.k), dtype=f32, device=dev)
        self.cnt_all = torch.empty((self.world, n_expert_total), dtype=i32, device=dev)
        self.rows_back = torch.empty((n, layout.n_embd), dtype=f32, device=dev)
        self.y = torch.empty((max_tokens, layout.n_embd), dtype=f32, device=dev)
        self.scratch = torch.empty(moe.native_expert_scratch_bytes(layout, self.max_recv), dtype=torch.uint8, device=dev)
        self.side = torch.cuda.Stream(device=dev)
        self.time_experts, self.last_expert_ms, self.last_groups = False, 0.0, 0
        if shared_blob is not None:
            self.s_out = torch.empty((max_tokens, layout.n_embd), dtype=f32, device=dev)
            self.s_scratch = torch.empty(C.c_size_t(moe.capi.lib().bsx_gated_mlp_scratch_bytes(C.byref(layout), max_tokens)).value,
                                         dtype=torch.uint8, device=dev)

    def forward(self, x):
        torch, dist, moe = self.torch, self.dist, self.moe
        a, L = self.args, self.L
        T = x.shape[0]
        n = T * a.k
        cur = torch.cuda.current_stream()
        # 1. route and dispatch the rank's own tokens
        moe.router_x(x, self.gate_w, self.bias, a, self.logits, self.ids, self.w)
        cnt, off, slot, src, _, _ = moe.dispatch(self.ids[:T].reshape(-1), a.k, self.E)
        # the shared expert runs beside the exchange on its own stream
        if self.shared_blob is not None:
            self.side.wait_stream(cur)
            with torch.cuda.stream(self.side):
                moe.gated_mlp(L, self.shared_blob, x, cap_tok=self.max_tokens, out=self.s_out[:T], scratch=self.s_scratch)
        # 2. counts of every rank -> split sizes and the receive plan (one device-to-host read per step)
        dist.all_gather_into_tensor(self.cnt_all, cnt, group=self.group)
        cnt_all = self.cnt_all.cpu().numpy()
        send, recv = ep_splits(cnt_all, self.rank)
        experts, start, rows = ep_recv_plan(cnt_all, self.rank)
        n_recv = int(recv.sum())
        assert n_recv <= self.max_recv, "receive buffer too small for this routing"
        # 3. rows in send order, then the all-to-all
        xs = moe.gather_rows(x, src[:n])
        xr = torch.empty((max(n_recv, 1), L.n_embd), dtype=x.dtype, device=self.dev)
        dist.all_to_all_single(xr[:n_recv], xs, recv.tolist(), send.tolist(), group=self.group)
        # 4. local grouped experts over the received rows; output row = receive row
        out = torch.empty((max(n_recv, 1), L.n_embd), dtype=torch.float32, device=self.dev)
        if n_recv:
            g = len(experts)
            ptr = torch.from_numpy(self.blob_addr[experts - int(self.first[self.rank])]).to(self.dev)
            st = torch.from_numpy(np.concatenate([start, start[-1:]])).to(self.dev)
            ent = torch.from_numpy(rows).to(self.dev)
            ng = torch.tensor([g], dtype=torch.int32, device=self.dev)
            if self.time_experts:
                t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                t0.record(cur)
            moe.native_expert_grouped(L, ptr, st, ng, ent, ent, g, n_recv, xr, self.scratch, out, n_x_rows=n_recv)
            if self.time_experts:
                t1.record(cur)
                t1.synchronize()
                self.last_expert_ms, self.last_groups = t0.elapsed_time(t1), g
        # 5. results back to their tokens' ranks (the mirror exchange), then the combine
        dist.all_to_all_single(self.rows_back[:n], out[:n_recv], send.tolist(), recv.tolist(), group=self.group)
        shared = None
        if self.shared_blob is not None:
            cur.wait_stream(self.side)
            shared = self.s_out[:T]
        return moe.moe_combine(self.rows_back[:n], slot.reshape(T, a.k), self.w[:T], shared, None, self.y[:T])


class EPMoELayer:
    """The expert-parallel layer on one rank for decode-sized steps, collective form.  Every size is fixed by (world,
    max_tokens), nothing is read back to the host, every rank passes the same number of tokens per step, and capture()
    records the step - collectives included - into a CUDA graph.

    Step: the rank's activations are all-gathered on a side stream WHILE the router runs on them (the exchange needs no
    routing); the routing ([ids | weights], one small buffer) is all-gathered after the selection; one kernel (bsx_ep_plan) turns
    all gathered pairs into the groups of the experts held here plus the shared expert's group over the rank's own tokens; the
    grouped experts run; one kernel (bsx_combine_partial_ep) sums each token's local pairs and, on the token's owner, adds the
    shared row; a reduce-scatter adds the ranks' partial rows and leaves every rank its own tokens' finished rows.  The
    cross-rank sum is NCCL's, so results match the single-GPU layer to fp32 rounding, not bit for bit.
    packed: blobs and the shared blob are in the plane layout of moe.pack_experts (block-scaled FP4 tensor cores)."""

    DATA_PLANE = ("NCCL all-gather of the bf16 rows (beside the router) and of the routing, local grouped experts, "
                  "reduce-scatter of fp32 partial rows")
    LAUNCHES = 8      # logits, selection, plan, x images + pass list, gate/up, h images, down, partial combine (+ 3 NCCL kernels)

    def __init__(self, gate_w, bias, blobs, layout, args, n_expert_total: int, shared_blob=None, max_tokens: int = 64, group=None,
                 packed: bool = False, replicas=None):
        """replicas: {expert id: blob tensor} of hot experts this rank (and every other rank: the same ids everywhere) holds a
        copy of besides its own block (choose_replicas picks them from load counts).  A pair naming one runs on the rank that
        owns its token."""
        import torch
        import torch.distributed as dist
        from . import capi, moe
        self.torch, self.dist, self.moe, self.capi = torch, dist, moe, capi
        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.E, self.L, self.args, self.packed = n_expert_total, layout, args, packed
        first = ep_partition(n_expert_total, self.world)
        self.lo, self.hi = int(first[self.rank]), int(first[self.rank + 1])
        self.gate_w, self.bias, self.blobs, self.shared_blob = gate_w, bias, blobs, shared_blob
        dev = blobs.device
        self.dev = dev
        El, stride = blobs.shape
        assert El == self.hi - self.lo
        table = np.zeros(n_expert_total, np.int64)                 # 0 = an expert another rank holds
        table[self.lo:self.hi] = blobs.data_ptr() + np.arange(El, dtype=np.int64) * stride
        self.replicas, self.replicated = replicas or {}, None
        if self.replicas:
            mask = np.zeros(n_expert_total, np.uint8)
            for e, blob in self.replicas.items():
                table[e] = blob.data_ptr()
                mask[e] = 1
            self.replicated = torch.from_numpy(mask).to(dev)
        self.blob_table = torch.from_numpy(table).to(dev)
        W, T, k, H = self.world, max_tokens, args.k, layout.n_embd
        self.max_tokens = T
        n = W * T * k
        assert n <= 8192, "bsx_ep_plan takes at most 8192 gathered pairs"
        rows = n + (T if shared_blob is not None else 0)
        f32, i32 = torch.float32, torch.int32
        self.logits = torch.empty((T, n_expert_total), dtype=f32, device=dev)
        self.route = torch.empty(2 * T * k, dtype=i32, device=dev)           # [ids T x k | weight bits T x k] of the rank's own tokens
        self.ids = self.route[:T * k].view(T, k)
        self.w = self.route[T * k:].view(f32).view(T, k)
        self.route_all = torch.empty(W * 2 * T * k, dtype=i32, device=dev)   # the ranks' buffers, one after the other
        self.ptr = torch.zeros(n_expert_total + 3, dtype=torch.int64, device=dev)
        self.start = torch.zeros(n_expert_total + 3, dtype=i32, device=dev)
        self.n_groups = torch.zeros(1, dtype=i32, device=dev)
        self.ent_dst = torch.zeros(rows, dtype=i32, device=dev)
        self.ent_tok = torch.zeros(rows, dtype=i32, device=dev)
        self.rows = torch.empty((rows, H), dtype=f32, device=dev)
        if packed:
            self.scratch = torch.empty(capi.lib().bsx_experts_packed_scratch_bytes(C.byref(layout), rows), dtype=torch.uint8, device=dev)
        else:
            self.scratch = torch.empty(moe.native_expert_scratch_bytes(layout, rows), dtype=torch.uint8, device=dev)
        self.status = torch.zeros(1, dtype=i32, device=dev)
        self.y_part = torch.empty((W * T, H), dtype=f32, device=dev)
        self.y = torch.empty((T, H), dtype=f32, device=dev)
        self.x_all = None
        self.side = torch.cuda.Stream(device=dev)
        self.events = None       # set to a list to collect (name, event) marks between the stages
        self.graph = None

    def check_status(self):
        """Raises moe.KernelWaitTimeout if a kernel of a step since the last check gave up on a bounded wait; clears the word."""
        self.moe.read_status(self.status, "EPMoELayer")

    def _mark(self, name):
        if self.events is not None:
            ev = self.torch.cuda.Event(enable_timing=True)
            ev.record(self.torch.cuda.current_stream())
            self.events.append((name, ev))

    def capture(self, x_example):
        """Records forward() into a CUDA graph (NCCL collectives included).  Every rank must capture, and replay, in step."""
        torch = self.torch
        self.x_static = torch.zeros((self.max_tokens, self.L.n_embd), dtype=x_example.dtype, device=self.dev)
        side = torch.cuda.Stream(device=self.dev)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(3):
                self.forward(self.x_static)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        # thread-local capture mode: the process group's watchdog thread polls its events while this thread captures
        with torch.cuda.graph(self.graph, capture_error_mode="thread_local"):
            self.forward(self.x_static)
        return self

    def forward_graphed(self, x=None):
        """x may be a pinned host tensor; None: the caller has already written self.x_static."""
        if x is not None:
            self.x_static.copy_(x, non_blocking=True)
        self.graph.replay()
        return self.y

    def forward(self, x):
        torch, dist, moe, capi = self.torch, self.dist, self.moe, self.capi
        lib, a, L = capi.lib(), self.args, self.L
        T, k, W, H = x.shape[0], a.k, self.world, L.n_embd
        assert T == self.max_tokens, "the collective form exchanges fixed-size buffers: pass max_tokens rows"
        cur = torch.cuda.current_stream()
        st = moe._stream(cur)
        p = moe._p
        self._mark("start")
        # 1. everyone gets every token's activations - on the side stream, beside the router
        if self.x_all is None or self.x_all.dtype != x.dtype:
            self.x_all = torch.empty((W * T, H), dtype=x.dtype, device=self.dev)
        self.side.wait_stream(cur)
        with torch.cuda.stream(self.side):
            dist.all_gather_into_tensor(self.x_all, x, group=self.group)
        # 2. route the rank's own tokens; ids and weights land in one buffer, which is then gathered
        moe.router_x(x, self.gate_w, self.bias, a, self.logits, self.ids, self.w)
        self._mark("router")
        dist.all_gather_into_tensor(self.route_all, self.route, group=self.group)
        self._mark("all_gather_route")
        # 3. all gathered pairs -> the groups of the experts held here (+ the shared expert over the rank's own tokens)
        n = W * T * k
        shared = self.shared_blob is not None
        capi.check("bsx_ep_plan", lib.bsx_ep_plan(p(self.route_all), n, k, T * k, 2 * T * k, self.E, p(self.blob_table),
                                                   self.shared_blob.data_ptr() if shared else 0, self.rank * T, T if (shared or self.replicas) else 0,
                                                   p(self.replicated), p(self.ptr), p(self.start), p(self.n_groups), p(self.ent_dst), p(self.ent_tok), st))
        self._mark("plan")
        cur.wait_stream(self.side)           # the gathered activations are needed from here on
        self._mark("all_gather_x_wait")
        # 4. the local experts over the rows routed to them (a pair's output lands on row = its index; shared rows after them)
        cap_groups, cap_rows = self.hi - self.lo + len(self.replicas) + (1 if shared else 0), n + (T if shared else 0)
        if self.packed:
            moe.native_expert_grouped_packed(L, self.ptr, self.start, self.n_groups, self.ent_dst, self.ent_tok, cap_groups, cap_rows, self.x_all,
                                             self.scratch, self.rows, self.status, n_x_rows=W * T)
        else:
            moe.native_expert_grouped(L, self.ptr, self.start, self.n_groups, self.ent_dst, self.ent_tok, cap_groups, cap_rows, self.x_all, self.scratch,
                                      self.rows, n_x_rows=W * T)
        self._mark("experts")
        # 5. each token's local pairs summed here (its owner adds the shared row), the ranks' partial rows reduced onto the owner
        capi.check("bsx_combine_partial_ep", lib.bsx_combine_partial_ep(p(self.rows), self.route_all.data_ptr() + 4 * T * k, p(self.route_all), T, 2 * T * k,
                                                                         self.lo, self.hi, W * T, k, H, p(self.rows[n:]) if shared else None,
                                                                         self.rank * T, T if (shared or self.replicas) else 0, p(self.replicated), p(self.y_part), st))
        self._mark("combine_partial")
        dist.reduce_scatter_tensor(self.y, self.y_part, op=dist.ReduceOp.SUM, group=self.group)
        self._mark("reduce_scatter")
        return self.y


class _NcclUniqueId(C.Structure):
    """ncclUniqueId: 128 opaque bytes, passed to ncclCommInitRank BY VALUE (a ctypes array would decay to a pointer)"""
    _fields_ = [("internal", C.c_byte * 128)]


class NcclComm:
    """An NCCL communicator of this process's own, made through NCCL's C API with ctypes (ncclGetUniqueId on rank 0, the id
    broadcast over the existing torch.distributed group, ncclCommInitRank everywhere): what a C++ host would hand to
    bsx_ep_layer.  torch keeps its own communicators private, so the layer behind the C ABI gets this one.  The library is the
    libnccl the process has already loaded (torch's), found by its soname - the same one bsx_ep_layer resolves."""

    def __init__(self, group=None):
        import torch
        import torch.distributed as dist
        self.lib = C.CDLL("libnccl.so.2", mode=C.RTLD_GLOBAL)
        self.lib.ncclGetUniqueId.argtypes = [C.POINTER(_NcclUniqueId)]
        self.lib.ncclCommInitRank.argtypes = [C.POINTER(C.c_void_p), C.c_int, _NcclUniqueId, C.c_int]
        self.lib.ncclCommDestroy.argtypes = [C.c_void_p]
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        uid = _NcclUniqueId()
        if rank == 0:
            rc = self.lib.ncclGetUniqueId(C.byref(uid))
            assert rc == 0, f"ncclGetUniqueId: {rc}"
        # the id travels as a byte tensor on the group's own backend (a CUDA tensor for nccl, a CPU tensor for gloo)
        on_gpu = dist.get_backend(group) == "nccl"
        t = torch.frombuffer(bytearray(bytes(uid)), dtype=torch.uint8).clone()
        t = t.cuda() if on_gpu else t
        dist.broadcast(t, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
        uid = _NcclUniqueId.from_buffer_copy(bytes(t.cpu().numpy().tobytes()))
        self.handle = C.c_void_p()
        rc = self.lib.ncclCommInitRank(C.byref(self.handle), world, uid, rank)
        assert rc == 0, f"ncclCommInitRank: {rc}"
        self.rank, self.world = rank, world

    def destroy(self):
        if self.handle:
            self.lib.ncclCommDestroy(self.handle)
            self.handle = C.c_void_p()


class EPMoELayerNative:
    """EPMoELayer's step as ONE call behind the C ABI (bsx_ep_layer): the collectives are issued by the library on an NCCL
    communicator the caller owns, so a C or C++ host gets the expert-parallel layer without this module.  Same arguments,
    same buffers' meaning, same result as EPMoELayer (bit for bit: the same kernels and the same collectives in the same order)."""

    DATA_PLANE = EPMoELayer.DATA_PLANE + "; the whole step is one C ABI call (bsx_ep_layer) on the caller's ncclComm_t"
    LAUNCHES = EPMoELayer.LAUNCHES

    def __init__(self, gate_w, bias, blobs, layout, args, n_expert_total: int, comm: NcclComm, shared_blob=None, max_tokens: int = 64,
                 packed: bool = False, replicas=None):
        import torch
        from . import capi, moe
        self.torch, self.moe, self.capi, self.comm = torch, moe, capi, comm
        assert capi.lib().bsx_ep_available() == 1, "no NCCL library in the process"
        self.rank, self.world = comm.rank, comm.world
        first = ep_partition(n_expert_total, self.world)
        self.lo, self.hi = int(first[self.rank]), int(first[self.rank + 1])
        self.gate_w, self.bias, self.blobs, self.shared_blob = gate_w, bias, blobs, shared_blob
        dev = blobs.device
        self.dev, self.L, self.args, self.E, self.max_tokens = dev, layout, args, n_expert_total, max_tokens
        El, stride = blobs.shape
        assert El == self.hi - self.lo
        table = np.zeros(n_expert_total, np.int64)
        table[self.lo:self.hi] = blobs.data_ptr() + np.arange(El, dtype=np.int64) * stride
        self.replicas, self.replicated = replicas or {}, None
        if self.replicas:
            mask = np.zeros(n_expert_total, np.uint8)
            for e, blob in self.replicas.items():
                table[e] = blob.data_ptr()
                mask[e] = 1
            self.replicated = torch.from_numpy(mask).to(dev)
        self.blob_table = torch.from_numpy(table).to(dev)
        d = capi.EPLayerDesc()
        d.layout = layout
        d.n_expert, d.top_k, d.gate_kind = n_expert_total, args.k, args.gate
        d.n_group, d.topk_group, d.packed = args.n_group, args.topk_group, 1 if packed else 0
        d.e_lo, d.n_local, d.n_replicas = self.lo, El, len(self.replicas)
        d.weight_scale = args.weight_scale
        d.gate, d.bias = gate_w.data_ptr(), (bias.data_ptr() if bias is not None else None)
        d.blob_table = self.blob_table.data_ptr()
        d.shared_blob = shared_blob.data_ptr() if shared_blob is not None else 0
        d.replicated = self.replicated.data_ptr() if self.replicated is not None else None
        self.desc = d
        lib = capi.lib()
        nbytes = lib.bsx_ep_layer_workspace_bytes(C.byref(d), max_tokens, self.world)
        assert nbytes > 0, "bsx_ep_layer_workspace_bytes refused the layer"
        self.workspace = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        self.y = torch.empty((max_tokens, layout.n_embd), dtype=torch.float32, device=dev)
        self.side = torch.cuda.Stream(device=dev)
        self.ev_fork, self.ev_join = torch.cuda.Event(), torch.cuda.Event()
        # the events must exist as CUDA objects before their handles are passed on
        self.ev_fork.record(torch.cuda.current_stream())
        self.ev_join.record(torch.cuda.current_stream())
        self.graph = None

    def check_status(self):
        """Raises moe.KernelWaitTimeout if a kernel of a step since the last check gave up on a bounded wait; clears the word."""
        self.moe.read_status(self.status, "EPMoELayerNative")

    def forward(self, x):
        torch, capi, moe = self.torch, self.capi, self.moe
        assert x.shape[0] == self.max_tokens, "the collective form exchanges fixed-size buffers: pass max_tokens rows"
        cur = torch.cuda.current_stream()
        kind = capi.X_BF16 if x.dtype == torch.bfloat16 else capi.X_F32
        capi.check("bsx_ep_layer", capi.lib().bsx_ep_layer(C.byref(self.desc), self.comm.handle, x.data_ptr(), kind, x.shape[0], self.workspace.data_ptr(),
                                                           self.y.data_ptr(), self.status.data_ptr(), moe._stream(cur), self.side.cuda_stream,
                                                           self.ev_fork.cuda_event, self.ev_join.cuda_event))
        return self.y

    def capture(self, x_example):
        """Records forward() into a CUDA graph (NCCL's kernels included).  Every rank must capture, and replay, in step."""
        torch = self.torch
        self.x_static = torch.zeros((self.max_tokens, self.L.n_embd), dtype=x_example.dtype, device=self.dev)
        warm = torch.cuda.Stream(device=self.dev)
        warm.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(warm):
            for _ in range(3):
                self.forward(self.x_static)
        torch.cuda.current_stream().wait_stream(warm)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph, capture_error_mode="thread_local"):
            self.forward(self.x_static)
        return self

    def forward_graphed(self, x=None):
        if x is not None:
            self.x_static.copy_(x, non_blocking=True)
        self.graph.replay()
        return self.y


class EPPrefillMoELayer:
    """The expert-parallel layer for prompt-sized batches, collective form: every rank routes its own T tokens (tensor-core
    gate product + selection), all-gathers activations and routing, dispatches all pairs, runs bsx_experts_prefill over the
    experts it holds (blob_table = 0 for the others, whose tiles the kernel skips), sums its experts' weighted rows per
    token (bsx_combine_partial) and reduce-scatters the partial sums to the tokens' owners.  The shared expert (replicated)
    runs on the rank's own tokens as a one-expert prefill call and is added last.  Fixed sizes, no host reads."""

    def __init__(self, gate_w, bias, blobs, layout, args, n_expert_total: int, shared_blob=None, max_tokens: int = 4096, group=None,
                 packed: bool = False):
        import torch
        import torch.distributed as dist
        from . import capi, moe
        self.torch, self.dist, self.moe, self.capi = torch, dist, moe, capi
        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.E, self.L, self.args, self.packed = n_expert_total, layout, args, packed
        first = ep_partition(n_expert_total, self.world)
        self.lo, self.hi = int(first[self.rank]), int(first[self.rank + 1])
        self.gate_w, self.bias, self.blobs, self.shared_blob = gate_w, bias, blobs, shared_blob
        dev = blobs.device
        self.dev = dev
        El, stride = blobs.shape
        assert El == self.hi - self.lo
        table = np.zeros(n_expert_total, np.int64)
        table[self.lo:self.hi] = blobs.data_ptr() + np.arange(El, dtype=np.int64) * stride
        self.blob_table = torch.from_numpy(table).to(dev)
        W, T, k, H = self.world, max_tokens, args.k, layout.n_embd
        self.max_tokens = T
        n = W * T * k
        f32, i32, u8 = torch.float32, torch.int32, torch.uint8
        lib = capi.lib()
        self.logits = torch.empty((T, n_expert_total), dtype=f32, device=dev)
        self.rscratch = torch.empty(lib.bsx_router_logits_prefill_scratch_bytes(T, n_expert_total, H), dtype=u8, device=dev)
        self.ids = torch.empty((T, k), dtype=i32, device=dev)
        self.w = torch.empty((T, k), dtype=f32, device=dev)
        self.route = torch.empty((T, 2 * k), dtype=i32, device=dev)
        self.route_all = torch.empty((W * T, 2 * k), dtype=i32, device=dev)
        self.ids_all = torch.empty((W * T, k), dtype=i32, device=dev)
        self.w_all = torch.empty((W * T, k), dtype=f32, device=dev)
        self.x_all = None
        self.cnt = torch.empty(n_expert_total, dtype=i32, device=dev)
        self.off = torch.empty(n_expert_total + 1, dtype=i32, device=dev)
        self.slot = torch.empty(n, dtype=i32, device=dev)
        self.src = torch.empty(n, dtype=i32, device=dev)
        self.tiles = torch.zeros((n // 128 + n_expert_total, 2), dtype=i32, device=dev)
        self.n_tiles = torch.zeros(1, dtype=i32, device=dev)
        self.dscratch = torch.empty(lib.bsx_dispatch_scratch_bytes(n, n_expert_total), dtype=u8, device=dev)
        scr = lib.bsx_experts_prefill_packed_scratch_bytes if packed else lib.bsx_experts_prefill_scratch_bytes
        self.scratch = torch.empty(scr(C.byref(layout), W * T, n), dtype=u8, device=dev)
        self.dm = torch.empty((n, H), dtype=f32, device=dev)
        self.status = torch.zeros(1, dtype=i32, device=dev)
        self.y_part = torch.empty((W * T, H), dtype=f32, device=dev)
        self.y_sum = torch.empty((T, H), dtype=f32, device=dev)
        self.y = torch.empty((T, H), dtype=f32, device=dev)
        self.ones = torch.ones((T, 1), dtype=f32, device=dev)
        if shared_blob is not None:
            # the shared expert as a one-expert dispatch of the rank's own tokens: rows in token order
            self.s_table = torch.tensor([shared_blob.data_ptr()], dtype=torch.int64, device=dev)
            self.s_off = torch.tensor([0, T], dtype=i32, device=dev)
            self.s_src = torch.arange(T, dtype=i32, device=dev)
            nt = (T + 127) // 128
            self.s_tiles = torch.stack([torch.zeros(nt, dtype=i32), torch.arange(nt, dtype=i32) * 128], dim=1).contiguous().to(dev)
            self.s_ntiles = torch.tensor([nt], dtype=i32, device=dev)
            self.s_scratch = torch.empty(scr(C.byref(layout), T, T), dtype=u8, device=dev)
            self.s_dm = torch.empty((T, H), dtype=f32, device=dev)

    def check_status(self):
        """Raises moe.KernelWaitTimeout if a kernel of a step since the last check gave up on a bounded wait; clears the word."""
        self.moe.read_status(self.status, "EPPrefillMoELayer")

    def forward(self, x):
        torch, dist, moe, capi = self.torch, self.dist, self.moe, self.capi
        lib, a, L = capi.lib(), self.args, self.L
        T, k, W, H = x.shape[0], a.k, self.world, L.n_embd
        assert T == self.max_tokens, "the collective form exchanges fixed-size buffers: pass max_tokens rows"
        st = moe._stream(torch.cuda.current_stream())
        p = moe._p
        kind = moe._x_kind(x)
        capi.check("bsx_router_logits_prefill", lib.bsx_router_logits_prefill(p(x), kind, p(self.gate_w), T, a.n_expert, a.n_embd, p(self.logits),
                                                                              p(self.rscratch), p(self.status), st))
        moe.router_select(self.logits, self.bias, a, self.ids, self.w)
        self.route[:, :k].copy_(self.ids)
        self.route[:, k:].view(torch.float32).copy_(self.w)
        if self.x_all is None or self.x_all.dtype != x.dtype:
            self.x_all = torch.empty((W * T, H), dtype=x.dtype, device=self.dev)
        dist.all_gather_into_tensor(self.x_all, x, group=self.group)
        dist.all_gather_into_tensor(self.route_all, self.route, group=self.group)
        self.ids_all.copy_(self.route_all[:, :k])
        self.w_all.copy_(self.route_all[:, k:].view(torch.float32))
        n = W * T * k
        capi.check("bsx_dispatch", lib.bsx_dispatch(p(self.ids_all), n, k, self.E, p(self.cnt), p(self.off), p(self.slot), p(self.src), 128,
                                                     p(self.tiles), p(self.n_tiles), p(self.dscratch), st))
        if self.packed:
            capi.check("bsx_experts_prefill_packed", lib.bsx_experts_prefill_packed(C.byref(L), p(self.blob_table), p(self.off), p(self.src), p(self.tiles),
                                                                                    p(self.n_tiles), self.tiles.shape[0], n, p(self.x_all), kind, W * T, self.E,
                                                                                    p(self.scratch), p(self.dm), p(self.status), st))
        else:
            capi.check("bsx_experts_prefill", lib.bsx_experts_prefill(C.byref(L), p(self.blob_table), p(self.off), p(self.src), p(self.tiles), p(self.n_tiles),
                                                                      self.tiles.shape[0], n, p(self.x_all), kind, W * T, p(self.scratch), p(self.dm),
                                                                      p(self.status), st))
        capi.check("bsx_combine_partial", lib.bsx_combine_partial(p(self.dm), p(self.slot), p(self.w_all), p(self.ids_all), self.lo, self.hi, W * T, k, H,
                                                                   p(self.y_part), st))
        if self.shared_blob is None:
            dist.reduce_scatter_tensor(self.y, self.y_part, op=dist.ReduceOp.SUM, group=self.group)
            return self.y
        if self.packed:
            capi.check("bsx_experts_prefill_packed", lib.bsx_experts_prefill_packed(C.byref(L), p(self.s_table), p(self.s_off), p(self.s_src), p(self.s_tiles),
                                                                                    p(self.s_ntiles), self.s_tiles.shape[0], T, p(x), kind, T, 1,
                                                                                    p(self.s_scratch), p(self.s_dm), p(self.status), st))
        else:
            capi.check("bsx_experts_prefill", lib.bsx_experts_prefill(C.byref(L), p(self.s_table), p(self.s_off), p(self.s_src), p(self.s_tiles), p(self.s_ntiles),
                                                                      self.s_tiles.shape[0], T, p(x), kind, T, p(self.s_scratch), p(self.s_dm), p(self.status), st))
        dist.reduce_scatter_tensor(self.y_sum, self.y_part, op=dist.ReduceOp.SUM, group=self.group)
        capi.check("bsx_combine", lib.bsx_combine(p(self.y_sum), None, p(self.ones), p(self.s_dm), None, T, 1, H, p(self.y), st))
        return self.y
