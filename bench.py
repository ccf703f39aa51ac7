#!/usr/bin/env python
"""MoE-layer throughput benchmark: `python bench.py --gpus N --steps K --warmup W [--impl reference]`.

Workload at N = 1 (BASELINE.json configs[1], the configuration the metric is quoted on): a Flash-Next-style MoE layer at
decode - hidden 2048, 512 routed experts + 1 shared expert, intermediate 512, softmax top-10 renormalised, NVFP4 experts
(E2M1 codes, UE4M3 scale per 16, fp32 scale per matrix) quantised from N(0, 0.02^2), bf16 activations N(0, 1), 64 tokens per
step.  A step is one pass of the layer over one batch: router -> plan -> grouped experts (+ shared) -> combine.  Inputs are
seeded synthetic data of those shapes and distributions (no dataset or checkpoint is involved).

The JSON line carries: `value` = tokens/s with inputs resident in HBM (CUDA events, max over ranks); `e2e` = the same through
the public call with host buffers (pinned host -> device copy of the step's activations and device -> host read of its
output inside the timed region); `roofline` = the dominant kernel (the routed experts' gate/up stream) against the measured
HBM copy bandwidth; `cpu_baseline` = the reference engine's own CPU expert-offload path (its thread pool and AVX kernels,
compiled from a reference checkout into oracle/_ref) on the same layer and tokens, timed on this box's host cores.

`--impl reference` times that CPU path alone (all host threads), printing the same line with "impl": "reference".
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

CFG = dict(workload="flash-next-style MoE layer decode, 64 tokens/step", hidden=2048, n_expert=512, n_shared=1, intermediate=512,
           top_k=10, router="softmax fp32 top-10 renormalised", expert_format="NVFP4 (ggml block_nvfp4 + fp32 tail scales)",
           activations="bf16", tokens_per_step=64)
H, E, I, K_TOP, T = 2048, 512, 512, 10, 64
LAYER_COPIES = 4   # the step cycles through copies of the layer (3.6 GB) so the 126 MB L2 cannot hold the weights


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), "measured (MEASURED_PEAKS.json)"
    return 6650.0, "fallback (earlier measurement on this pool)"


SHAPES = {
    # flash-next-style layer (the decode line's layer): softmax top-10 of 512 + 1 shared
    "c1": dict(H=2048, E=512, I=512, k=10, gate="softmax", n_group=1, topk_group=1, scale=1.0, bias=False, zipf=True,
               name="flash-next-style MoE layer"),
    # v4-flash-style layer: sigmoid + bias, 8 groups keep 4, top-8 of 256 + 1 shared, weights x 2.5
    "c3": dict(H=7168, E=256, I=2048, k=8, gate="sigmoid", n_group=8, topk_group=4, scale=2.5, bias=True, zipf=False,
               name="v4-flash-style MoE layer"),
    # the c3 layer with IQ1_M routed experts and a Q6_K shared expert (decode only; random valid blocks)
    "c4": dict(H=7168, E=256, I=2048, k=8, gate="sigmoid", n_group=8, topk_group=4, scale=2.5, bias=True, zipf=False,
               name="v4-flash-style MoE layer, IQ1_M routed + Q6_K shared experts", routed_type=29, shared_type=14),
}


def random_codebook_blobs(device, type_id, n, H_, I_, seed):
    """n expert blobs of random valid blocks of a ggml K/IQ format - uniform over the valid codes, as the reference's own
    tests make IQ1_M weights (it has no quantiser for that format: tests/kernels/iq1s_parity.cpp:65-93).  IQ1_M (56 bytes per
    256 values): random bytes with a finite fp16 super-scale in [2^-7, 2^-6) in the top nibbles of the four scale words.
    Q6_K (210 bytes per 256 values): random ql / qh, int8 scales in [-32, 31], fp16 d = 2^-12."""
    g = torch.Generator(device=device).manual_seed(seed)
    bb = 56 if type_id == 29 else 210
    nb = 3 * I_ * H_ // 256
    raw = torch.randint(0, 256, (n, nb, bb), generator=g, device=device, dtype=torch.int16)
    if type_id == 29:
        d = 0x2000 + torch.randint(0, 0x400, (n, nb), generator=g, device=device, dtype=torch.int32)
        for j in range(4):                     # scale word j (bytes 48 + 2 j, 49 + 2 j): its top nibble = nibble j of d
            raw[:, :, 49 + 2 * j] = (raw[:, :, 49 + 2 * j] & 0x0F) | ((((d >> (4 * j)) & 0xF) << 4).to(torch.int16))
    else:
        raw[:, :, 192:208] = (raw[:, :, 192:208] & 0x3F) - 32          # int8 scales
        raw[:, :, 192:208] = raw[:, :, 192:208] & 0xFF
        raw[:, :, 208] = 0x00
        raw[:, :, 209] = 0x0C                                           # fp16 0x0C00 = 2^-12
    blob_bytes = nb * bb
    stride = (blob_bytes + 15) // 16 * 16
    out = torch.zeros((n, stride), dtype=torch.uint8, device=device)
    out[:, :blob_bytes] = raw.to(torch.uint8).reshape(n, -1)
    return out, blob_bytes


def make_layer_weights(device, seed=0, E=E, H=H, I=I, first=0, count=None):
    """gate [E][H] fp32 and NVFP4 blobs quantised from N(0, 0.02^2): experts first .. first + count - 1 of E + 1 (the last,
    index E, is the shared expert).  Every expert's values depend only on (seed, its index)."""
    from basalt_b200 import pack
    if count is not None:
        gate = (torch.randn((E, H), generator=torch.Generator(device=device).manual_seed(seed), device=device) * 0.02).float()
        blob_bytes = 3 * I * (H // 64 * 36) + 16
        stride = (blob_bytes + 15) // 16 * 16
        blobs = torch.zeros((count, stride), dtype=torch.uint8, device=device)
        for i in range(count):
            g = torch.Generator(device=device).manual_seed(seed * 100003 + 1 + first + i)
            G = torch.randn((I, H), generator=g, device=device) * 0.02
            U = torch.randn((I, H), generator=g, device=device) * 0.02
            D = torch.randn((H, I), generator=g, device=device) * 0.02
            blobs[i, :blob_bytes] = pack.pack_nvfp4_expert(G, U, D)
        return gate, blobs, blob_bytes
    g = torch.Generator(device=device).manual_seed(seed)
    gate = (torch.randn((E, H), generator=g, device=device) * 0.02).float()
    blob_bytes = 3 * I * (H // 64 * 36) + 16
    stride = (blob_bytes + 15) // 16 * 16
    blobs = torch.zeros((E + 1, stride), dtype=torch.uint8, device=device)
    for e in range(E + 1):
        G = torch.randn((I, H), generator=g, device=device) * 0.02
        U = torch.randn((I, H), generator=g, device=device) * 0.02
        D = torch.randn((H, I), generator=g, device=device) * 0.02
        blobs[e, :blob_bytes] = pack.pack_nvfp4_expert(G, U, D)
    return gate, blobs, blob_bytes


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled every 200 ms while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index=0):
        self.rows, self.proc, self.index = [], None, index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc:
            time.sleep(0.25)
            self.proc.terminate()
            self.thread.join(timeout=2)

    def summary(self):
        sm = [float(r[0]) for r in self.rows if len(r) >= 7 and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) >= 7 and r[1].replace(".", "").isdigit()]
        reasons = set()
        for r in self.rows:
            if len(r) >= 7:
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


# --------------------------------------------------------------------------------------------------------- CPU reference arm
def cpu_reference_layer(gate, blobs_host, blob_bytes, xs_host, steps, warmup, workers=None):
    """The reference engine's CPU expert-offload path (ExpertPool::run_split_multi_native over its AVX kernels, from
    oracle/_ref/libref_cpu.so) for the same layer: the oracle's CPU router / dispatch / combine around it.  Returns
    (seconds per step list, cores used, kind)."""
    from oracle import oracle as O
    R = O.ref_cpu()
    n_thr = workers or max(1, (os.cpu_count() or 2))
    gate = np.ascontiguousarray(gate, np.float32)
    times = []
    if R is not None:
        pool = R.ref_pool_create(max(1, n_thr - 1))     # the host thread drains too (pool.hpp:57-76)
        ptrs = (C.c_void_p * E)(*[blobs_host[e].ctypes.data for e in range(E)])
        sptr = (C.c_void_p * 1)(blobs_host[E].ctypes.data)
        s_off = np.array([0, T], np.int32)
        s_src = np.arange(T, dtype=np.int32)
    L = O.Layout(O.T_NVFP4, O.T_NVFP4, H, I)
    for it in range(warmup + steps):
        x = xs_host[it % len(xs_host)]
        t0 = time.perf_counter()
        logits = O.router_logits(x, gate)
        ids, w = O.router_select(logits, None, K_TOP, O.GATE_SOFTMAX)
        cnt, off, slot, src, _ = O.dispatch(ids, K_TOP, E)
        rows = np.zeros((T * K_TOP, H), np.float32)
        shared = np.zeros((T, H), np.float32)
        if R is not None:
            assert R.ref_pool_layer(pool, 40, 40, H, I, 0.0, ptrs, E, off, src, x, T, rows) == 0
            assert R.ref_pool_layer(pool, 40, 40, H, I, 0.0, sptr, 1, s_off, s_src, x, T, shared) == 0
        else:   # the plain-C port: dequantise and multiply, one expert at a time
            for e in range(E):
                if cnt[e]:
                    rows[off[e]:off[e + 1]] = O.expert_forward(L, blobs_host[e][:blob_bytes], x[src[off[e]:off[e + 1]]])
            shared = O.expert_forward(L, blobs_host[E][:blob_bytes], x)
        y = O.combine(rows, slot, w, shared)
        dt = time.perf_counter() - t0
        if it >= warmup:
            times.append(dt)
    if R is not None:
        R.ref_pool_destroy(pool)
    return times, n_thr, ("reference" if R is not None else "port"), y


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    dev = torch.device("cuda:0" if torch.cuda.is_available() else "cpu")
    gate, blobs, blob_bytes = make_layer_weights(dev)
    gate_h, blobs_h = gate.cpu().numpy(), blobs.cpu().numpy()
    del gate, blobs
    rng = np.random.default_rng(1)
    xs = [torch.from_numpy(rng.standard_normal((T, H)).astype(np.float32)).bfloat16().float().numpy() for _ in range(4)]
    times, cores, kind, _ = cpu_reference_layer(gate_h, blobs_h, blob_bytes, xs, args.steps, args.warmup)
    ms = 1e3 * sum(times) / len(times)
    val = T / (ms / 1e3)
    line = {"impl": "reference", "metric": "MoE-layer tokens/s (decode)", "value": val, "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "int8 x NVFP4 dot products, fp32 accumulation (the reference's CPU arithmetic)", "data": "synthetic",
            "config": CFG,
            "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": cores, "kind": kind,
                             "sample": f"{args.steps} full layer steps of 64 tokens (all 640 routed rows + shared expert)"},
            "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


# --------------------------------------------------------------------------------------------------------- the B200 arm
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--copies", type=int, default=LAYER_COPIES, help="layer copies the steps cycle through (1 for a small profiler capture)")
    ap.add_argument("--experts", default="packed", choices=["packed", "fp16"],
                    help="decode expert kernels: packed = blobs repacked at load into planes, block-scaled FP4 tensor cores (tcgen05 kind::mxf4nvf4); "
                         "fp16 = ggml blobs in place, fp16 activation images, mma.sync")
    ap.add_argument("--input-norm", default="none", choices=["none", "fused", "separate"],
                    help="decode workload: the layer also applies its input RMS norm (the reference's norm_pack step) - fused with the FP4 "
                         "activation images, or as a launch of its own")
    ap.add_argument("--act", default="bf16", choices=["bf16", "fp32"], help="decode workload: element type of the activation rows given to the layer")
    ap.add_argument("--no-fork", action="store_true", help="decode workload: the activation-image kernel runs on the step's own stream, ahead of the router, "
                                                           "instead of where the layer would put it (a forked branch beside the router for up to 16 tokens)")
    ap.add_argument("--no-graph", action="store_true", help="launch every kernel of a step from the host instead of replaying the layer's CUDA graph")
    ap.add_argument("--decode-tokens", type=int, default=T, help="tokens per decode step and GPU (the reference's decode configs: 1, 8, 64; the metric is quoted on 64)")
    ap.add_argument("--workload", default="decode", choices=["decode", "prefill"],
                    help="decode: 64 tokens a step (the default line); prefill: --tokens rows a step, Zipf(1.1) expert popularity, tcgen05 grouped experts")
    ap.add_argument("--tokens", type=int, default=4096, help="rows per step of the prefill workload, per GPU (4096 or 16384 in the reference's configs)")
    ap.add_argument("--shape", default="c1", choices=sorted(SHAPES), help="layer of the prefill workload: c1 (H 2048, 512 experts) or c3 (H 7168, 256 experts)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.workload == "decode" and args.shape != "c1":
        # the decode step on another layer shape (c3: the v4-flash / DeepSeek-style layer); the default line stays c1
        sh = SHAPES[args.shape]
        globals().update(H=sh["H"], E=sh["E"], I=sh["I"], K_TOP=sh["k"])
        CFG.update(workload=f"{sh['name']} decode, {T} tokens/step", hidden=sh["H"], n_expert=sh["E"], intermediate=sh["I"], top_k=sh["k"],
                   router=f"{sh['gate']} + bias, {sh['n_group']} groups keep {sh['topk_group']}, top-{sh['k']}, x {sh['scale']}" if sh["bias"] else sh["gate"])
    if args.decode_tokens != T:
        assert 1 <= args.decode_tokens <= 64
        globals()["T"] = args.decode_tokens
        CFG.update(workload=CFG["workload"].replace("64 tokens/step", f"{args.decode_tokens} tokens/step"), tokens_per_step=args.decode_tokens)
    if args.impl == "reference":
        return run_reference_arm(args)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the MoE layer has no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        # with NCCL_DEBUG=VERSION in the environment NCCL prints its version banner to stdout at the first collective; the JSON
        # line below is always the last line of stdout
        dist.init_process_group("nccl", device_id=dev)
    from basalt_b200 import build, capi, moe
    if rank == 0:
        build.build()
    if world > 1:
        dist.barrier()
    lib = capi.lib()
    if args.workload == "prefill":
        return run_prefill(args, dev, rank, world)
    if world > 1:
        return run_expert_parallel(args, rank, world, dev)

    sh = SHAPES[args.shape]
    if "routed_type" in sh:
        return run_decode_codebook(args, dev, sh)
    gate, blobs, blob_bytes = make_layer_weights(dev, E=E, H=H, I=I, first=0, count=E + 1) if args.shape != "c1" else make_layer_weights(dev)
    L = moe.native_expert_layout(capi.TYPE_NVFP4, capi.TYPE_NVFP4, H, I)
    assert L.bytes == blob_bytes
    rargs = moe.RouterArgs(n_expert=E, n_embd=H, k=K_TOP, weight_scale=sh["scale"], gate=capi.GATE_SOFTMAX if sh["gate"] == "softmax" else capi.GATE_SIGMOID,
                           n_group=sh["n_group"], topk_group=sh["topk_group"])
    bias = (torch.randn(E, generator=torch.Generator(device=dev).manual_seed(7), device=dev) * 0.01).float() if sh["bias"] else None
    layers = []
    use_packed = args.experts == "packed"
    if use_packed:
        blobs_ggml = blobs
        blobs = moe.pack_experts(L, blobs_ggml)       # the load-time step: the same bytes in plane order
        torch.cuda.synchronize()
        if args.shape != "c1":
            del blobs_ggml
    for c in range(args.copies):
        b = blobs if c == 0 else blobs.clone()
        norm_w = None if args.input_norm == "none" else 1.0 + 0.1 * torch.randn(H, generator=torch.Generator(device=dev).manual_seed(3), device=dev)
        layers.append(moe.MoELayer(gate if c == 0 else gate.clone(), bias, b[:E], L, rargs, shared_blob=b[E], max_tokens=T, packed=use_packed,
                                   norm_w=norm_w, norm_fused=args.input_norm != "separate", fork_images=False if args.no_fork else None))
    n_batches = 8
    g = torch.Generator(device=dev).manual_seed(1 + rank)
    xs = [torch.randn((T, H), generator=g, device=dev).bfloat16() for _ in range(n_batches)]
    if args.act == "fp32":
        xs = [x.float() for x in xs]
    stream = torch.cuda.Stream(device=dev)

    use_graph = not args.no_graph
    if use_graph:
        with torch.cuda.stream(stream):
            for ly in layers:
                ly.capture(xs[0])
        torch.cuda.synchronize()

    def step(i, x=None):
        xx = xs[i % n_batches] if x is None else x
        if use_graph:
            return layers[i % args.copies].forward_graphed(xx)
        return layers[i % args.copies].forward(xx, None, stream)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    with torch.cuda.stream(stream):
        for i in range(args.warmup):
            step(i)
        barrier()
        # ---- resident-input throughput
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler(local) as clocks:
            ev0.record(stream)
            for i in range(args.steps):
                step(i)
            ev1.record(stream)
            barrier()
        ms_total = ev0.elapsed_time(ev1)
        # ---- end to end: pinned host activations in, host output out, every step
        x_host = [x.cpu().pin_memory() for x in xs]
        xin = torch.empty((T, H), dtype=xs[0].dtype, device=dev)
        y_host = torch.empty((T, H), dtype=torch.float32).pin_memory()
        def e2e_step(i):
            # pinned host rows -> device (with a graph: straight into its input buffer), the step, the result -> pinned host
            if use_graph:
                y_host.copy_(step(i, x_host[i % n_batches]), non_blocking=True)
            else:
                xin.copy_(x_host[i % n_batches], non_blocking=True)
                y_host.copy_(step(i, xin), non_blocking=True)

        for i in range(3):
            e2e_step(i)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for i in range(args.steps):
            e2e_step(i)
            stream.synchronize()          # the caller reads the step's result before it issues the next step
        e1.record(stream)
        barrier()
        ms_e2e = e0.elapsed_time(e1)
        # ---- per-stage device times for the roofline (same steps, events between the C ABI calls)
        stage_ms, gu_bytes = instrumented_pass(layers, xs, None, stream, min(args.steps, 100), L)
        barrier()
        # ---- the run is only a number if no kernel gave up on a bounded wait and a step's output is right
        for ly in layers:
            ly.check_status()
        if use_packed and args.input_norm == "none" and args.shape == "c1":
            y_fast = step(0, xs[0]).clone()
            twin = moe.MoELayer(gate, bias, blobs_ggml[:E], L, rargs, shared_blob=blobs_ggml[E], max_tokens=T)   # ggml blobs in place, fp16 images
            y_ref = twin.forward(xs[0], None, stream)
            stream.synchronize()
            err = float((y_fast - y_ref).norm() / y_ref.norm())
            if not err < 1e-3:
                raise SystemExit(f"bench: the timed path's output differs from the in-place fp16 path (relative L2 {err:.3e})")
            del twin

    times = torch.tensor([ms_total, ms_e2e], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms_total, ms_e2e = times.tolist()
    if rank != 0:
        return
    ms_step = ms_total / args.steps
    peak, peak_src = measured_peaks()
    gu_ms = stage_ms["experts_gate_up"]
    achieved = gu_bytes / (gu_ms * 1e-3) / 1e9
    line = {
        "metric": "MoE-layer tokens/s (decode)", "value": T * world / (ms_step * 1e-3), "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None,
        "dtype": ("NVFP4 weights x 4-term FP4 activations on tcgen05 kind::mxf4nvf4 (block-scaled), fp32 accumulation" if use_packed
                  else "fp16 x NVFP4 tensor-core products (mma.sync), fp32 accumulation"), "data": "synthetic",
        "config": dict(CFG, l2_policy=(f"weights cycle through {args.copies} layer copies ({0.906 * args.copies:.1f} GB) and each step touches ~650 MB: larger than L2" if (T == 64 and args.shape == "c1") else
                                  f"weights cycle through {args.copies} layer copies ({0.906 * args.copies:.1f} GB); use --copies so that copies x touched experts exceed the 126 MB L2"),
                       parallelism="single GPU" if world == 1 else f"ep{world}",
                       expert_kernels="packed planes + tcgen05 block-scaled FP4" if use_packed else "ggml blobs in place + fp16 images + mma.sync",
                       launch="one CUDA graph per step (input copied into its static buffer, device to device)" if use_graph else "one host launch per kernel",
                       input_norm={"none": "not part of the step (rows arrive normed)", "fused": "RMS norm inside the step, fused with the FP4 activation images",
                                   "separate": "RMS norm inside the step, a launch of its own"}[args.input_norm]),
        "e2e": {"value": T * world / (ms_e2e / args.steps * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": T * H * xs[0].element_size(), "d2h_bytes_per_step": T * H * 4},
        "gpu_launches": (9 if args.input_norm == "separate" else 8) * args.steps,   # (norm,) logits, select, plan, 2 x activation images, gate/up, down, combine (the shared expert rides in the grouped call)
        "roofline": {"bound": "hbm", "kernel": ("nvf4_stream_kernel<gate/up>" if use_packed else "nvfp4_mma_kernel<gate/up>") + " (routed + shared experts; stage time includes the activation-image kernel)", "achieved": achieved, "peak": peak,
                     "unit": "GB/s", "frac": achieved / peak, "peak_source": peak_src,
                     # dram__bytes_read.sum + dram__bytes_write.sum of one gate/up launch of this workload at 64 tokens (seeded, so the
                     # same experts every run), from the ncu captures summarised in profiles/nvf4_stream_kernel_c1_t64.md and
                     # profiles/nvfp4_mma_kernel_c1_t64.md; not measured by this run
                     "traffic": ((450646784 if use_packed else 451744256) if (T == 64 and args.shape == "c1") else None), "traffic_source": "ncu capture (profiles/)",
                     "algorithmic_bytes_per_launch": gu_bytes, "kernel_ms": gu_ms, "frac_of_nominal_8TBs": achieved / 8000.0},
        "stage_ms": stage_ms,
        "clocks": clocks.summary(),
    }
    if not args.no_cpu_baseline and args.shape == "c1":
        try:
            gate_h, blobs_h = gate.cpu().numpy(), (blobs_ggml if use_packed else blobs).cpu().numpy()
            xh = [x.float().cpu().numpy() for x in xs[:4]]
            tms, cores, kind, _ = cpu_reference_layer(gate_h, blobs_h, blob_bytes, xh, 20, 3)
            sec = sum(tms) / len(tms)
            line["cpu_baseline"] = {"value": T / sec, "unit": "tokens/s", "cores": cores, "kind": kind,
                                    "sample": "20 full layer steps of 64 tokens on the same weights (reference CPU expert pool; oracle router/dispatch/combine)"}
        except Exception as exc:   # the baseline is reported, never required
            line["cpu_baseline"] = {"value": None, "unit": "tokens/s", "cores": 0, "kind": "port", "sample": f"failed: {exc}"}
    print(json.dumps(line))


def run_expert_parallel(args, rank, world, dev):
    """N > 1: the same layer with its 512 routed experts sharded over the ranks in contiguous blocks (expert parallel), 64
    tokens per rank and step (weak scaling: per-GPU tokens fixed), rows exchanged by NCCL all-to-all before and after the
    local grouped experts; router and shared expert replicated.  Device time, max over ranks."""
    import torch.distributed as dist
    from basalt_b200 import capi, ep, moe
    gate, blobs, blob_bytes = make_layer_weights(dev)          # the same seed on every rank: identical replicated weights
    El = E // world
    L = moe.native_expert_layout(capi.TYPE_NVFP4, capi.TYPE_NVFP4, H, I)
    rargs = moe.RouterArgs(n_expert=E, n_embd=H, k=K_TOP, weight_scale=1.0, gate=capi.GATE_SOFTMAX)
    layers = []
    use_packed = args.experts == "packed"
    mine = torch.cat([blobs[rank * El:(rank + 1) * El], blobs[E:E + 1]])      # the rank's routed experts + the shared one
    if use_packed:
        mine = moe.pack_experts(L, mine)
    for c in range(args.copies):
        b = mine.clone()
        layers.append(ep.EPMoELayer(gate.clone(), None, b[:El], L, rargs, E, shared_blob=b[El], max_tokens=T, packed=use_packed))
    del blobs
    n_batches = 8
    g = torch.Generator(device=dev).manual_seed(1 + rank)
    xs = [torch.randn((T, H), generator=g, device=dev).bfloat16() for _ in range(n_batches)]
    stream = torch.cuda.Stream(device=dev)

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    use_graph = not args.no_graph

    def fwd(i, x=None):
        ly, xx = layers[i % args.copies], (xs[i % n_batches] if x is None else x)
        return ly.forward_graphed(xx) if use_graph else ly.forward(xx)

    with torch.cuda.stream(stream):
        if use_graph:
            for ly in layers:
                ly.capture(xs[0])
            barrier()
        for i in range(args.warmup):
            fwd(i)
        barrier()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler(dev.index or 0) as clocks:
            ev0.record(stream)
            for i in range(args.steps):
                fwd(i)
            ev1.record(stream)
            barrier()
        ms_total = ev0.elapsed_time(ev1)
        x_host = [x.cpu().pin_memory() for x in xs]
        xin = torch.empty((T, H), dtype=torch.bfloat16, device=dev)
        y_host = torch.empty((T, H), dtype=torch.float32).pin_memory()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for i in range(args.steps):
            if use_graph:
                y_host.copy_(fwd(i, x_host[i % n_batches]), non_blocking=True)
            else:
                xin.copy_(x_host[i % n_batches], non_blocking=True)
                y_host.copy_(fwd(i, xin), non_blocking=True)
            stream.synchronize()
        e1.record(stream)
        barrier()
        ms_e2e = e0.elapsed_time(e1)
        # the local expert stage alone, for the roofline: bytes of the experts this rank touched / device time of the call
        ly = layers[0]
        ly.time_experts = True
        exp_ms, exp_bytes = [], []
        for i in range(min(args.steps, 50)):
            ly.forward(xs[i % n_batches])
            stream.synchronize()
            exp_ms.append(ly.last_expert_ms)
            exp_bytes.append(ly.last_groups * (L.bytes - 16))
        ly.time_experts = False
        barrier()
    times = torch.tensor([ms_total, ms_e2e], dtype=torch.float64, device=dev)
    dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms_total, ms_e2e = times.tolist()
    if rank != 0:
        return
    ms_step = ms_total / args.steps
    peak, peak_src = measured_peaks()
    k_ms, k_bytes = sum(exp_ms) / len(exp_ms), sum(exp_bytes) / len(exp_bytes)
    achieved = k_bytes / (k_ms * 1e-3) / 1e9
    line = {
        "metric": "MoE-layer tokens/s (decode)", "value": T * world / (ms_step * 1e-3), "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None,
        "dtype": ("NVFP4 weights x 4-term FP4 activations on tcgen05 kind::mxf4nvf4 (block-scaled), fp32 accumulation" if use_packed
                  else "fp16 x NVFP4 tensor-core products (mma.sync), fp32 accumulation"), "data": "synthetic",
        "config": dict(CFG, tokens_per_step=T * world, tokens_per_gpu=T,
                       parallelism=f"ep{world}: {E // world} routed experts per GPU, router and shared expert replicated; NCCL all-gather of bf16 rows and routing, reduce-scatter of fp32 partial sums",
                       l2_policy=f"each rank cycles through {args.copies} copies of its expert shard",
                       expert_kernels="packed planes + tcgen05 block-scaled FP4" if use_packed else "ggml blobs in place + fp16 images + mma.sync",
                       launch="one CUDA graph per step, collectives included" if use_graph else "one host launch per kernel"),
        "e2e": {"value": T * world / (ms_e2e / args.steps * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": T * H * 2 * world,
                "d2h_bytes_per_step": T * H * 4 * world},
        "gpu_launches": 13 * args.steps,   # logits, select, 3 dispatch, plan, 2 x images, gate/up, down, partial combine, combine (+ torch's 4 small copies, 3 NCCL kernels)
        "roofline": {"bound": "hbm", "kernel": "rank 0's local grouped experts (image prep, gate/up, down)", "achieved": achieved, "peak": peak,
                     "unit": "GB/s", "frac": achieved / peak, "peak_source": peak_src, "traffic": None, "algorithmic_bytes_per_launch": k_bytes,
                     "kernel_ms": k_ms},
        "clocks": clocks.summary(),
    }
    print(json.dumps(line))


def run_decode_codebook(args, dev, sh):
    """The decode step with K/IQ-format experts (configs[4]'s layer on one GPU): IQ1_M routed experts and a Q6_K shared
    expert, both read in place by the plain kernels (one warp per weight row, fp32 FMA) - the formats have no tensor-core
    path yet.  Reported: tokens/s and the bytes of the touched blobs over the expert stage's time."""
    from basalt_b200 import capi, moe
    rt, st_ = sh["routed_type"], sh["shared_type"]
    gate = (torch.randn((E, H), generator=torch.Generator(device=dev).manual_seed(0), device=dev) * 0.02).float()
    bias = (torch.randn(E, generator=torch.Generator(device=dev).manual_seed(7), device=dev) * 0.01).float()
    blobs, rb = random_codebook_blobs(dev, rt, E, H, I, 11)
    shared, sb = random_codebook_blobs(dev, st_, 1, H, I, 12)
    L = moe.native_expert_layout(rt, rt, H, I)
    Ls = moe.native_expert_layout(st_, st_, H, I)
    assert L.bytes == rb and Ls.bytes == sb
    rargs = moe.RouterArgs(n_expert=E, n_embd=H, k=K_TOP, weight_scale=sh["scale"], gate=capi.GATE_SIGMOID, n_group=sh["n_group"],
                           topk_group=sh["topk_group"])
    layers = [moe.MoELayer(gate, bias, blobs if c == 0 else blobs.clone(), L, rargs, shared_blob=(shared if c == 0 else shared.clone())[0],
                           shared_layout=Ls, max_tokens=T) for c in range(args.copies)]
    g = torch.Generator(device=dev).manual_seed(1)
    xs = [torch.randn((T, H), generator=g, device=dev).bfloat16() for _ in range(4)]
    stream = torch.cuda.Stream(device=dev)
    with torch.cuda.stream(stream):
        for i in range(args.warmup):
            layers[i % args.copies].forward(xs[i % 4], None, stream)
        torch.cuda.synchronize()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler(dev.index or 0) as clocks:
            ev0.record(stream)
            for i in range(args.steps):
                layers[i % args.copies].forward(xs[i % 4], None, stream)
            ev1.record(stream)
            torch.cuda.synchronize()
        ms_step = ev0.elapsed_time(ev1) / args.steps
        x_host = [x.cpu().pin_memory() for x in xs]
        xin = torch.empty((T, H), dtype=torch.bfloat16, device=dev)
        y_host = torch.empty((T, H), dtype=torch.float32).pin_memory()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for i in range(args.steps):
            xin.copy_(x_host[i % 4], non_blocking=True)
            y_host.copy_(layers[i % args.copies].forward(xin, None, stream), non_blocking=True)
            stream.synchronize()
        e1.record(stream)
        torch.cuda.synchronize()
        ms_e2e = e0.elapsed_time(e1) / args.steps
        touched = sum(int(torch.unique(layers[0].ids[:T]).numel()) for _ in range(1))
    peak, peak_src = measured_peaks()
    bytes_step = touched * rb + sb
    line = {
        "metric": "MoE-layer tokens/s (decode)", "value": T / (ms_step * 1e-3), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp32 FMA on weights decoded in registers (IQ1_M codebook, Q6_K)", "data": "synthetic (random valid blocks)",
        "config": dict(workload=f"{sh['name']} decode, {T} tokens/step", hidden=H, n_expert=E, n_shared=1, intermediate=I, top_k=K_TOP,
                       expert_format="IQ1_M routed (56 B / 256 values), Q6_K shared (210 B / 256 values)", activations="bf16", tokens_per_step=T,
                       l2_policy=f"weights cycle through {args.copies} layer copies; a step touches {bytes_step / 1e9:.2f} GB", parallelism="single GPU",
                       expert_kernels="ggml blobs in place, plain kernels (experts_simple.cu)"),
        "e2e": {"value": T / (ms_e2e * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": T * H * 2, "d2h_bytes_per_step": T * H * 4},
        "gpu_launches": 12 * args.steps,
        "roofline": {"bound": "hbm", "kernel": "whole step (the expert kernels dominate)", "achieved": bytes_step / (ms_step * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                     "frac": bytes_step / (ms_step * 1e-3) / 1e9 / peak, "peak_source": peak_src, "traffic": None, "algorithmic_bytes_per_launch": bytes_step},
        "clocks": clocks.summary(),
    }
    print(json.dumps(line))


def zipf_logits(n_tokens, n_expert, gen, dev, s=1.1):
    """[T][E] fp32 scores whose top-k sets follow Zipf(s) popularity: log p_e + Gumbel noise, the popularity ranks dealt to
    expert ids by a seeded permutation (top-k of such scores = sampling k experts without replacement from p)."""
    p = torch.arange(1, n_expert + 1, device=dev, dtype=torch.float64) ** (-s)
    logp = torch.log(p / p.sum()).float()[torch.randperm(n_expert, generator=gen, device=dev)]
    u = torch.rand((n_tokens, n_expert), generator=gen, device=dev).clamp_(1e-20, 1.0 - 1e-7)
    return (logp[None, :] - torch.log(-torch.log(u))).contiguous()


def run_prefill(args, dev, rank=0, world=1):
    """The prompt-sized workload: --tokens rows a step per GPU on the layer --shape names.  c1: expert popularity Zipf(1.1)
    (scores drawn; the reference's prompt benches have no dataset for this path either); c3: the router's own scores.
    One step = gate product (tensor cores) + selection + dispatch with the 128-row tile list + grouped experts on the tcgen05
    tensor cores (routed + shared) + combine.  With N > 1 ranks the routed experts are sharded (expert parallel, collective
    form: all-gather, local experts, reduce-scatter) and every rank brings --tokens rows (weak scaling).  The roofline is the
    tensor one: 6 H I flops per expert row over the measured bf16 peak (the products run as kind::f16 on exactly decoded
    weights); the HBM time of the touched blobs is reported beside it."""
    from basalt_b200 import capi, ep, moe
    import torch.distributed as dist
    sh = SHAPES[args.shape]
    Hs, Es, Is, ks = sh["H"], sh["E"], sh["I"], sh["k"]
    Tn = args.tokens
    El = Es // world
    gate, own, blob_bytes = make_layer_weights(dev, E=Es, H=Hs, I=Is, first=rank * El, count=El)
    _, shared, _ = make_layer_weights(dev, E=Es, H=Hs, I=Is, first=Es, count=1)
    L = moe.native_expert_layout(capi.TYPE_NVFP4, capi.TYPE_NVFP4, Hs, Is)
    assert L.bytes == blob_bytes
    gk = capi.GATE_SOFTMAX if sh["gate"] == "softmax" else capi.GATE_SIGMOID
    rargs = moe.RouterArgs(n_expert=Es, n_embd=Hs, k=ks, weight_scale=sh["scale"], gate=gk, n_group=sh["n_group"], topk_group=sh["topk_group"])
    g = torch.Generator(device=dev).manual_seed(1 + rank)
    bias = (torch.randn(Es, generator=torch.Generator(device=dev).manual_seed(7), device=dev) * 0.01).float() if sh["bias"] else None
    use_packed = args.experts == "packed"
    if use_packed:
        own, shared = moe.pack_experts(L, own), moe.pack_experts(L, shared)
        torch.cuda.synchronize()
    if world == 1:
        layer = moe.PrefillMoELayer(gate, bias, own, L, rargs, shared_blob=shared[0], max_tokens=Tn, packed=use_packed)
    else:
        layer = ep.EPPrefillMoELayer(gate, bias, own, L, rargs, Es, shared_blob=shared[0], max_tokens=Tn, packed=use_packed)
    n_batches = 2
    xs = [torch.randn((Tn, Hs), generator=g, device=dev).bfloat16() for _ in range(n_batches)]
    lgs = [zipf_logits(Tn, Es, g, dev) if (sh["zipf"] and world == 1) else None for _ in range(n_batches)]
    stream = torch.cuda.Stream(device=dev)

    def fwd(i, x=None):
        xx = xs[i % n_batches] if x is None else x
        return layer.forward(xx, lgs[i % n_batches], stream) if world == 1 else layer.forward(xx)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    barrier()
    with torch.cuda.stream(stream):
        for i in range(args.warmup):
            fwd(i)
        barrier()
        if int(layer.status.item()) != 0:
            raise SystemExit("the prefill kernel reported a bounded wait that ran out (status %d)" % int(layer.status.item()))
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler(dev.index or 0) as clocks:
            ev0.record(stream)
            for i in range(args.steps):
                fwd(i)
            ev1.record(stream)
            barrier()
        ms_step = ev0.elapsed_time(ev1) / args.steps
        # end to end: pinned host rows in, host result out, every step
        x_host = [x.cpu().pin_memory() for x in xs]
        xin = torch.empty((Tn, Hs), dtype=torch.bfloat16, device=dev)
        y_host = torch.empty((Tn, Hs), dtype=torch.float32).pin_memory()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n_e2e = max(3, args.steps // 2)
        barrier()
        e0.record(stream)
        for i in range(n_e2e):
            xin.copy_(x_host[i % n_batches], non_blocking=True)
            y_host.copy_(fwd(i, xin), non_blocking=True)
            stream.synchronize()
        e1.record(stream)
        barrier()
        ms_e2e = e0.elapsed_time(e1) / n_e2e
        stage_ms, touched, cnt = {}, float(El), None
        if world == 1:
            names = ["router_logits", "router_select", "dispatch", "experts", "combine"]
            acc = {n: 0.0 for n in names}
            n_inst = min(args.steps, 10)
            touched = 0
            for i in range(n_inst):
                layer.events = []
                fwd(i)
                stream.synchronize()
                evs = layer.events
                for (_, a), (nme, b) in zip(evs[:-1], evs[1:]):
                    acc[nme] += a.elapsed_time(b)
                touched += int((layer.cnt > 0).sum().item())
            layer.events = None
            stage_ms = {k: v / n_inst for k, v in acc.items()}
            touched /= n_inst
            cnt = layer.cnt.cpu().numpy()
    status = int(layer.status.item())
    times = torch.tensor([ms_step, ms_e2e], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms_step, ms_e2e = times.tolist()
    if rank != 0:
        return
    flops = 6.0 * Hs * Is * (Tn * ks + Tn) * world
    peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text()) if (ROOT / "MEASURED_PEAKS.json").exists() else {}
    tpeak = float(peaks.get("bf16_tflops", 1590.0))
    hbm = float(peaks.get("hbm_gbs", 6650.0))
    # the tensor roofline of the expert stage (one GPU: its own stage time; N GPUs: the whole step, per GPU)
    exp_ms = stage_ms["experts"] if world == 1 else ms_step
    achieved = flops / world / (exp_ms * 1e-3) / 1e12
    blob_b = touched * (L.bytes - 16)
    roof = {"bound": "tensor", "kernel": (("prefill_nvf4_kernel" if use_packed else "prefill_gemm_kernel") + "<gate/up> + <down> (+ activation images)") if world == 1 else "whole step per GPU (experts + collectives)",
            "achieved": achieved, "peak": tpeak, "unit": "TFLOP/s", "frac": achieved / tpeak,
            "peak_source": "measured bf16 burst (MEASURED_PEAKS.json)" if peaks else "fallback", "traffic": None,
            "algorithmic_flops_per_launch": flops / world, "kernel_ms": exp_ms, "hbm_ms_of_touched_blobs": blob_b / (hbm * 1e9) * 1e3,
            "tensor_ms_at_peak": flops / world / (tpeak * 1e12) * 1e3, "experts_touched": touched}
    if cnt is not None:
        roof.update(max_rows_per_expert=int(cnt.max()), median_rows_per_expert=float(np.median(cnt[:Es])))
    line = {
        "metric": "MoE-layer tokens/s (prefill)", "value": Tn * world / (ms_step * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": ("NVFP4 weights x 4-term FP4 activations on tcgen05 kind::mxf4nvf4 (block-scaled), fp32 accumulation in tensor memory" if use_packed
                  else "fp16 x (NVFP4 decoded exactly to fp16) on tcgen05 kind::f16, fp32 accumulation in tensor memory"), "data": "synthetic",
        "config": dict(workload=f"{sh['name']} prefill, {Tn} tokens/step per GPU" + (", Zipf(1.1) expert popularity" if lgs[0] is not None else ""),
                       hidden=Hs, n_expert=Es, n_shared=1, intermediate=Is, top_k=ks, router=sh["gate"], n_group=sh["n_group"], topk_group=sh["topk_group"],
                       expert_format="NVFP4 (ggml block_nvfp4 + fp32 tail scales)", activations="bf16", tokens_per_step=Tn * world,
                       l2_policy=f"every step reads all touched expert blobs ({blob_b / 1e9:.2f} GB per GPU): larger than L2",
                       parallelism="single GPU" if world == 1 else f"ep{world}: {El} routed experts per GPU; all-gather of bf16 rows and routing, reduce-scatter of fp32 partial sums"),
        "e2e": {"value": Tn * world / (ms_e2e * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": Tn * Hs * 2 * world, "d2h_bytes_per_step": Tn * Hs * 4 * world},
        "gpu_launches": (12 if world == 1 else 16) * args.steps,   # image prep x2, gate GEMM, selection, 3 dispatch, activation prep, gate/up, down, combine (+ shared expert's three and the partial combine with N > 1)
        "roofline": roof, "stage_ms": stage_ms, "status_word": status, "clocks": clocks.summary(),
    }
    print(json.dumps(line))


def instrumented_pass(layers, xs, xr, stream, steps, L):
    """Re-runs the steps with CUDA events between the C ABI calls; returns mean ms per stage and the gate/up launch's
    algorithmic bytes (distinct experts touched, the shared one included, x gate+up bytes + activation images in + h out),
    averaged over steps."""
    from basalt_b200 import capi
    from basalt_b200.moe import _p, _stream, _x_kind
    lib = capi.lib()
    st = _stream(stream)
    names = ["router", "plan", "experts_gate_up", "experts_down", "combine"]
    acc = {n: 0.0 for n in names}
    gu_bytes = 0.0
    for i in range(steps):
        ly, x = layers[i % len(layers)], xs[i % len(xs)]
        a = ly.args
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(6)]
        n = T * a.k
        ev[0].record(stream)
        capi.check("router", lib.bsx_router_x(_p(x), _x_kind(x), _p(ly.gate_w), _p(ly.bias), T, a.n_expert, a.n_embd, a.k, a.gate, a.weight_scale, a.n_group, a.topk_group, 0.0,
                                              None, 0, _p(ly.logits), _p(ly.ids), _p(ly.w), st))
        ev[1].record(stream)
        capi.check("plan", lib.bsx_moe_plan_shared(_p(ly.ids), T, a.k, a.n_expert, _p(ly.blob_table), ly.shared_blob.data_ptr(), _p(ly.ptr), _p(ly.start),
                                                   _p(ly.n_groups), _p(ly.dst), _p(ly.tok), st))
        ev[2].record(stream)
        for phase in (1, 2):
            lib.bsx_experts_set_phase(phase)
            if ly.packed:
                capi.check("experts", lib.bsx_experts_grouped_packed(C.byref(ly.L), _p(ly.ptr), _p(ly.start), _p(ly.n_groups), _p(ly.dst), _p(ly.tok),
                                                                      min(n, a.n_expert) + 1, n + T, _p(x), _x_kind(x), T, _p(ly.scratch), _p(ly.rows),
                                                                      capi.OUT_F32, _p(ly.status), st))
            else:
                capi.check("experts", lib.bsx_experts_grouped_rows(C.byref(ly.L), _p(ly.ptr), _p(ly.start), _p(ly.n_groups), _p(ly.dst), _p(ly.tok),
                                                                    min(n, a.n_expert) + 1, n + T, _p(x), _x_kind(x), T, _p(ly.scratch), _p(ly.rows),
                                                                    capi.OUT_F32, st))
            ev[2 + phase].record(stream)
        lib.bsx_experts_set_phase(0)
        capi.check("combine", lib.bsx_combine(_p(ly.rows), None, _p(ly.w), _p(ly.rows[n:n + T]), None, T, a.k, L.n_embd, _p(ly.y), st))
        ev[5].record(stream)
        stream.synchronize()
        for j, nme in enumerate(names):
            acc[nme] += ev[j].elapsed_time(ev[j + 1])
        groups = int(ly.n_groups.item())      # distinct routed experts touched + the shared expert
        # gate + up blob bytes of the touched experts, the activation images read (bf16 rows: 2 B a value as fp16, or 4 FP4 terms
        # = 2.25 B with their scales), the SwiGLU rows written
        gu_bytes += groups * 2 * L.n_ff * L.gu_row + (n + T) * L.n_embd * 2 + (n + T) * L.n_ff * 4
    return {k: v / steps for k, v in acc.items()}, gu_bytes / steps


if __name__ == "__main__":
    main()
