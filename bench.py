#!/usr/bin/env python
"""MoE-layer throughput benchmark: `python bench.py --gpus N --steps K --warmup W [--impl reference]`.

The line's own workload (N = 1): a Flash-Next-style MoE layer at decode - hidden 2048, 512 routed experts + 1 shared expert,
intermediate 512, softmax top-10 renormalised, NVFP4 experts (E2M1 codes, UE4M3 scale per 16, fp32 scale per matrix) quantised
from N(0, 0.02^2), bf16 activations N(0, 1), 64 tokens per step.  A step is one pass of the layer over one batch: router ->
plan -> grouped experts (+ shared) -> combine, issued by the one-call layer entry (bsx_moe_layer).  Inputs are seeded synthetic
data of those shapes and distributions (no dataset or checkpoint is involved).

The JSON line carries: `value` = tokens/s with inputs resident in HBM (CUDA events, max over ranks); `e2e` = the same through
the public call with host buffers (pinned host -> device copy of the step's activations and device -> host read of its
output inside the timed region); `roofline` = the dominant kernel (the routed experts' gate/up stream) against the measured
HBM copy bandwidth; `cpu_baseline` = the reference engine's own CPU expert-offload path (its thread pool and AVX kernels,
compiled from a reference checkout into oracle/_ref) on the same layer and tokens, timed on this box's host cores, with the CPU
model, the instruction set that ran and a second leg with its AVX2 kernels forced; `workloads` = the other configurations of the
same layer family, each a short run of this script's own code: decode at 1 and 8 tokens, the DeepSeek-style layer (hidden 7168,
256 + 1 experts of 2048, sigmoid + bias, 8 groups keep 4, top-8) at 64-token decode, the same shape with IQ1_M routed experts
and a Q6_K shared expert, and the prompt-sized steps (16,384 tokens on the first layer, 8192 on the second).

`--impl reference` times that CPU path alone (all host threads), printing the same line with "impl": "reference".
`--workload` / `--shape` / `--decode-tokens` make one of the other configurations the line's own workload.
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

LAYER_COPIES = 4   # the 64-token step cycles through copies of the layer (3.6 GB) so the 126 MB L2 cannot hold the weights

SHAPES = {
    # flash-next-style layer (the decode line's layer): softmax top-10 of 512 + 1 shared
    "c1": dict(H=2048, E=512, I=512, k=10, gate="softmax", n_group=1, topk_group=1, scale=1.0, bias=False, zipf=True,
               name="flash-next-style MoE layer", router="softmax fp32 top-10 renormalised"),
    # v4-flash / DeepSeek-style layer: sigmoid + bias, 8 groups keep 4, top-8 of 256 + 1 shared, weights x 2.5
    "c3": dict(H=7168, E=256, I=2048, k=8, gate="sigmoid", n_group=8, topk_group=4, scale=2.5, bias=True, zipf=False,
               name="v4-flash-style MoE layer", router="sigmoid + bias, 8 groups keep 4, top-8, x 2.5"),
    # the c3 layer with IQ1_M routed experts and a Q6_K shared expert (decode only; random valid blocks)
    "c4": dict(H=7168, E=256, I=2048, k=8, gate="sigmoid", n_group=8, topk_group=4, scale=2.5, bias=True, zipf=False,
               name="v4-flash-style MoE layer, IQ1_M routed + Q6_K shared experts", router="sigmoid + bias, 8 groups keep 4, top-8, x 2.5",
               routed_type=29, shared_type=14),
}


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return dict(hbm=float(d["hbm_gbs"]), bf16=float(d.get("bf16_tflops", 1590.0)), source="measured (MEASURED_PEAKS.json)")
    return dict(hbm=6650.0, bf16=1590.0, source="fallback (earlier measurement on this pool)")


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
        raw[:, :, 192:208] = ((raw[:, :, 192:208] & 0x3F) - 32) & 0xFF           # int8 scales
        raw[:, :, 208] = 0x00
        raw[:, :, 209] = 0x0C                                                    # fp16 0x0C00 = 2^-12
    blob_bytes = nb * bb
    stride = (blob_bytes + 15) // 16 * 16
    out = torch.zeros((n, stride), dtype=torch.uint8, device=device)
    out[:, :blob_bytes] = raw.to(torch.uint8).reshape(n, -1)
    return out, blob_bytes


def make_layer_weights(device, seed=0, E=512, H=2048, I=512, first=0, count=None):
    """gate [E][H] fp32 and NVFP4 blobs quantised from N(0, 0.02^2): experts first .. first + count - 1 of E + 1 (the last,
    index E, is the shared expert).  Every expert's values depend only on (seed, its index)."""
    from basalt_b200 import pack
    gate = (torch.randn((E, H), generator=torch.Generator(device=device).manual_seed(seed), device=device) * 0.02).float()
    if count is None:
        first, count = 0, E + 1
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


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled every 200 ms while the timed region runs (a read-only query)."""
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
def host_cpu():
    """model name and physical core count of the host, from /proc/cpuinfo"""
    name, cores = "", set()
    try:
        phys = core = None
        for line in open("/proc/cpuinfo"):
            if line.startswith("model name") and not name:
                name = line.split(":", 1)[1].strip()
            elif line.startswith("physical id"):
                phys = line.split(":", 1)[1].strip()
            elif line.startswith("core id"):
                core = line.split(":", 1)[1].strip()
            elif not line.strip():
                if phys is not None and core is not None:
                    cores.add((phys, core))
                phys = core = None
    except OSError:
        pass
    return name, (len(cores) or (os.cpu_count() or 1))


def cpu_reference_layer(gate, blobs_host, blob_bytes, xs_host, steps, warmup, sh, T, workers=None, avx2=False):
    """The reference engine's CPU expert-offload path (ExpertPool::run_split_multi_native over its AVX kernels, from
    oracle/_ref/libref_cpu.so) for the same layer: the oracle's CPU router / dispatch / combine around it.  avx2: the
    reference's AVX2 kernels called directly (a row-split thread pool of the same size), whatever else the CPU has.
    Returns (seconds per step list, threads used, kind, last y)."""
    from oracle import oracle as O
    E, H, I, K_TOP = sh["E"], sh["H"], sh["I"], sh["k"]
    R = O.ref_cpu()
    n_thr = workers or max(1, (os.cpu_count() or 2))
    gate = np.ascontiguousarray(gate, np.float32)
    times = []
    pool = None
    if R is not None:
        if not avx2:
            pool = R.ref_pool_create(max(1, n_thr - 1))     # the host thread drains too (pool.hpp:57-76)
        ptrs = (C.c_void_p * E)(*[blobs_host[e].ctypes.data for e in range(E)])
        sptr = (C.c_void_p * 1)(blobs_host[E].ctypes.data)
        s_off = np.array([0, T], np.int32)
        s_src = np.arange(T, dtype=np.int32)
    elif avx2:
        raise RuntimeError("the AVX2 leg needs oracle/_ref/libref_cpu.so")
    L = O.Layout(O.T_NVFP4, O.T_NVFP4, H, I)
    y = None
    for it in range(warmup + steps):
        x = xs_host[it % len(xs_host)]
        t0 = time.perf_counter()
        logits = O.router_logits(x, gate)
        ids, w = O.router_select(logits, None, K_TOP, O.GATE_SOFTMAX)
        cnt, off, slot, src, _ = O.dispatch(ids, K_TOP, E)
        rows = np.zeros((T * K_TOP, H), np.float32)
        shared = np.zeros((T, H), np.float32)
        if R is not None and avx2:
            assert R.ref_avx2_layer(n_thr, H, I, ptrs, E, off, src, x, T, rows) == 0
            assert R.ref_avx2_layer(n_thr, H, I, sptr, 1, s_off, s_src, x, T, shared) == 0
        elif R is not None:
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
    if pool is not None:
        R.ref_pool_destroy(pool)
    return times, n_thr, ("reference" if R is not None else "port"), y


def cpu_info():
    """the host CPU as the reference names it and the instruction set its kernels pick"""
    from oracle import oracle as O
    name, cores = host_cpu()
    isa = "unknown"
    R = O.ref_cpu()
    if R is not None and hasattr(R, "ref_cpu_info"):
        buf = C.create_string_buffer(160)
        isa = {3: "avx512 (F, BW, VL, VNNI, VBMI)", 2: "avx2", 0: "none"}.get(R.ref_cpu_info(buf, 160), "unknown")
        name = buf.value.decode("utf-8", "replace") or name
    return name, cores, isa


def cpu_baseline_block(gate_h, blobs_h, blob_bytes, xh, sh, T, steps, with_avx2=True):
    tms, thr, kind, _ = cpu_reference_layer(gate_h, blobs_h, blob_bytes, xh, steps, 3, sh, T)
    sec = sum(tms) / len(tms)
    name, cores, isa = cpu_info()
    out = {"value": T / sec, "unit": "tokens/s", "cores": thr, "physical_cores": cores, "cpu_model": name, "isa": isa if kind == "reference" else "plain C",
           "kind": kind, "sample": f"{steps} full layer steps of {T} tokens on the same weights (reference CPU expert pool; oracle router/dispatch/combine)"}
    if with_avx2 and kind == "reference":
        try:
            t2, thr2, _, _ = cpu_reference_layer(gate_h, blobs_h, blob_bytes, xh, max(3, steps // 2), 2, sh, T, avx2=True)
            out["avx2_forced"] = {"value": T / (sum(t2) / len(t2)), "unit": "tokens/s", "cores": thr2,
                                  "sample": f"{max(3, steps // 2)} steps; the reference's nvfp4_256_* AVX2 kernels called directly, rows split over the threads"}
        except Exception as exc:
            out["avx2_forced"] = {"value": None, "sample": f"failed: {exc}"}
    return out


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sh = SHAPES["c1"]
    T = 64
    dev = torch.device("cuda:0" if torch.cuda.is_available() else "cpu")
    gate, blobs, blob_bytes = make_layer_weights(dev)
    gate_h, blobs_h = gate.cpu().numpy(), blobs.cpu().numpy()
    del gate, blobs
    rng = np.random.default_rng(1)
    xs = [torch.from_numpy(rng.standard_normal((T, sh["H"])).astype(np.float32)).bfloat16().float().numpy() for _ in range(4)]
    times, thr, kind, _ = cpu_reference_layer(gate_h, blobs_h, blob_bytes, xs, args.steps, args.warmup, sh, T)
    ms = 1e3 * sum(times) / len(times)
    val = T / (ms / 1e3)
    name, cores, isa = cpu_info()
    line = {"impl": "reference", "metric": "MoE-layer tokens/s (decode)", "value": val, "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "int8 x NVFP4 dot products, fp32 accumulation (the reference's CPU arithmetic)", "data": "synthetic",
            "config": decode_config(sh, T),
            "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": thr, "physical_cores": cores, "cpu_model": name, "isa": isa, "kind": kind,
                             "sample": f"{args.steps} full layer steps of 64 tokens (all 640 routed rows + shared expert)"},
            "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


# --------------------------------------------------------------------------------------------------------- decode on one GPU
def decode_config(sh, T):
    return dict(workload=f"{sh['name']} decode, {T} tokens/step", hidden=sh["H"], n_expert=sh["E"], n_shared=1, intermediate=sh["I"], top_k=sh["k"],
                router=sh["router"], expert_format="NVFP4 (ggml block_nvfp4 + fp32 tail scales)", activations="bf16", tokens_per_step=T)


class Weights:
    """one layer's synthetic weights on the device: gate, bias, ggml blobs (kept when asked), packed blobs"""

    def __init__(self, dev, key, keep_ggml=False):
        from basalt_b200 import capi, moe
        sh = SHAPES[key]
        self.sh, self.key = sh, key
        self.gate, blobs, self.blob_bytes = make_layer_weights(dev, E=sh["E"], H=sh["H"], I=sh["I"])
        self.L = moe.native_expert_layout(capi.TYPE_NVFP4, capi.TYPE_NVFP4, sh["H"], sh["I"])
        assert self.L.bytes == self.blob_bytes
        self.bias = (torch.randn(sh["E"], generator=torch.Generator(device=dev).manual_seed(7), device=dev) * 0.01).float() if sh["bias"] else None
        self.packed = moe.pack_experts(self.L, blobs)
        torch.cuda.synchronize()
        self.ggml = blobs if keep_ggml else None
        self.rargs = moe.RouterArgs(n_expert=sh["E"], n_embd=sh["H"], k=sh["k"], weight_scale=sh["scale"],
                                    gate=capi.GATE_SOFTMAX if sh["gate"] == "softmax" else capi.GATE_SIGMOID, n_group=sh["n_group"], topk_group=sh["topk_group"])


def make_decode_layers(w: Weights, T, copies, kind, experts="packed", input_norm="none", no_fork=False, pdl=True):
    from basalt_b200 import moe
    sh, E = w.sh, w.sh["E"]
    dev = w.gate.device
    layers = []
    src = w.packed if experts == "packed" else w.ggml
    for c in range(copies):
        b = src if c == 0 else src.clone()
        norm_w = None if input_norm == "none" else 1.0 + 0.1 * torch.randn(sh["H"], generator=torch.Generator(device=dev).manual_seed(3), device=dev)
        if kind == "native":
            layers.append(moe.NativeMoELayer(w.gate if c == 0 else w.gate.clone(), w.bias, b[:E], w.L, w.rargs, shared_blob=b[E], max_tokens=T,
                                             packed=experts == "packed", norm_w=norm_w, pdl=pdl))
        else:
            layers.append(moe.MoELayer(w.gate if c == 0 else w.gate.clone(), w.bias, b[:E], w.L, w.rargs, shared_blob=b[E], max_tokens=T,
                                       packed=experts == "packed", norm_w=norm_w, norm_fused=input_norm != "separate", fork_images=False if no_fork else None))
    return layers


def run_decode(w: Weights, T, steps, warmup, copies, dev, kind="native", experts="packed", input_norm="none", act="bf16", graph=True, no_fork=False,
               stages=False, check=False, pdl=True):
    """times the decode step at T tokens: resident inputs, end to end, and (stages) per-stage device times; returns a dict"""
    from basalt_b200 import moe
    sh = w.sh
    H, E, k = sh["H"], sh["E"], sh["k"]
    layers = make_decode_layers(w, T, copies, kind, experts, input_norm, no_fork, pdl)
    n_batches = 8
    g = torch.Generator(device=dev).manual_seed(1)
    xs = [torch.randn((T, H), generator=g, device=dev).bfloat16() for _ in range(n_batches)]
    if act == "fp32":
        xs = [x.float() for x in xs]
    stream = torch.cuda.Stream(device=dev)
    if graph:
        with torch.cuda.stream(stream):
            for ly in layers:
                ly.capture(xs[0])
        torch.cuda.synchronize()

    def step(i, x=None):
        xx = xs[i % n_batches] if x is None else x
        ly = layers[i % copies]
        if graph:
            return ly.forward_graphed(xx)
        return ly.forward(xx, None, stream)

    out = {}
    with torch.cuda.stream(stream):
        for i in range(warmup):
            step(i)
        torch.cuda.synchronize()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler(dev.index or 0) as clocks:
            ev0.record(stream)
            for i in range(steps):
                step(i)
            ev1.record(stream)
            torch.cuda.synchronize()
        out["ms_step"] = ev0.elapsed_time(ev1) / steps
        out["clocks"] = clocks.summary()
        # ---- end to end: pinned host activations in, host output out, every step
        x_host = [x.cpu().pin_memory() for x in xs]
        xin = torch.empty((T, H), dtype=xs[0].dtype, device=dev)
        y_host = torch.empty((T, H), dtype=torch.float32).pin_memory()

        def e2e_step(i):
            if graph:
                y_host.copy_(step(i, x_host[i % n_batches])[:T], non_blocking=True)
            else:
                xin.copy_(x_host[i % n_batches], non_blocking=True)
                y_host.copy_(step(i, xin), non_blocking=True)

        for i in range(3):
            e2e_step(i)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n_e2e = steps
        e0.record(stream)
        for i in range(n_e2e):
            e2e_step(i)
            stream.synchronize()          # the caller reads the step's result before it issues the next step
        e1.record(stream)
        torch.cuda.synchronize()
        out["ms_e2e"] = e0.elapsed_time(e1) / n_e2e
        # distinct experts a step touches (for the step's algorithmic bytes)
        touched = []
        for i in range(min(8, n_batches)):
            ly = layers[i % copies]
            (ly.forward(xs[i], None, stream) if kind != "native" else ly.forward(xs[i], None, stream))
            stream.synchronize()
            touched.append(int(torch.unique(ly.ids[:T]).numel()))
        out["experts_touched"] = sum(touched) / len(touched)
        if stages:
            calls = make_decode_layers(w, T, copies, "calls", experts, "none", True) if kind == "native" else layers
            out["stage_ms"], out["gu_bytes"] = instrumented_pass(calls, xs, stream, min(steps, 100), w.L, T)
            if calls is not layers:
                del calls
        # ---- the run is only a number if no kernel gave up on a bounded wait and a step's output is right
        for ly in layers:
            ly.check_status()
        if check and w.ggml is not None and experts == "packed" and input_norm == "none":
            y_fast = step(0, xs[0])[:T].clone()
            twin = moe.MoELayer(w.gate, w.bias, w.ggml[:E], w.L, w.rargs, shared_blob=w.ggml[E], max_tokens=T)   # ggml blobs in place, fp16 images
            y_ref = twin.forward(xs[0], None, stream)
            stream.synchronize()
            err = float((y_fast - y_ref).norm() / y_ref.norm())
            if not err < 1e-3:
                raise SystemExit(f"bench: the timed path's output differs from the in-place fp16 path (relative L2 {err:.3e})")
            out["output_check_rel_l2_vs_fp16_path"] = err
            del twin
    L = w.L
    blob = L.bytes - 16
    out["bytes_step"] = (out["experts_touched"] + 1) * blob + E * H * 4 + T * H * (xs[0].element_size() + 4) + T * k * 8
    out["launches"] = ({"none": 7, "fused": 7, "separate": 8}[input_norm] if kind == "native" else {"none": 8, "fused": 8, "separate": 9}[input_norm])
    del layers
    torch.cuda.empty_cache()
    return out


def instrumented_pass(layers, xs, stream, steps, L, T):
    """Re-runs the steps call by call with CUDA events between the C ABI calls; returns mean ms per stage and the gate/up launch's
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
        if ly.packed:
            # the x images belong to the head of the step, where the one-call entry runs them beside the logits kernel
            capi.check("x_images", lib.bsx_experts_packed_x_images(C.byref(ly.L), _p(x), _x_kind(x), T, n + T, _p(ly.scratch), st))
        capi.check("router", lib.bsx_router_x(_p(x), _x_kind(x), _p(ly.gate_w), _p(ly.bias), T, a.n_expert, a.n_embd, a.k, a.gate, a.weight_scale, a.n_group, a.topk_group, 0.0,
                                              None, 0, _p(ly.logits), _p(ly.ids), _p(ly.w), st))
        ev[1].record(stream)
        capi.check("plan", lib.bsx_moe_plan_shared(_p(ly.ids), T, a.k, a.n_expert, _p(ly.blob_table), ly.shared_blob.data_ptr(), _p(ly.ptr), _p(ly.start),
                                                   _p(ly.n_groups), _p(ly.dst), _p(ly.tok), st))
        ev[2].record(stream)
        for phase in (capi.EXPERT_STAGE_GU, capi.EXPERT_STAGE_DOWN):
            Lp = capi.ExpertLayout.from_buffer_copy(ly.L)     # the same layout, one stage of the two
            Lp.options = phase
            if ly.packed:
                capi.check("experts", lib.bsx_experts_grouped_packed(C.byref(Lp), _p(ly.ptr), _p(ly.start), _p(ly.n_groups), _p(ly.dst), _p(ly.tok),
                                                                      min(n, a.n_expert) + 1, n + T, _p(x), _x_kind(x), -T, _p(ly.scratch), _p(ly.rows),
                                                                      capi.OUT_F32, _p(ly.status), st))
            else:
                capi.check("experts", lib.bsx_experts_grouped_rows(C.byref(Lp), _p(ly.ptr), _p(ly.start), _p(ly.n_groups), _p(ly.dst), _p(ly.tok),
                                                                    min(n, a.n_expert) + 1, n + T, _p(x), _x_kind(x), T, _p(ly.scratch), _p(ly.rows),
                                                                    capi.OUT_F32, st))
            ev[2 + phase].record(stream)
        capi.check("combine", lib.bsx_combine(_p(ly.rows), None, _p(ly.w), _p(ly.rows[n:n + T]), None, T, a.k, L.n_embd, _p(ly.y), st))
        ev[5].record(stream)
        stream.synchronize()
        for j, nme in enumerate(names):
            acc[nme] += ev[j].elapsed_time(ev[j + 1])
        groups = int(ly.n_groups.item())      # distinct routed experts touched + the shared expert
        gu_bytes += groups * 2 * L.n_ff * L.gu_row + (n + T) * L.n_embd * 2 + (n + T) * L.n_ff * 4
    return {k: v / steps for k, v in acc.items()}, gu_bytes / steps


def decode_line(args, w, T, r, world=1):
    sh = w.sh
    pk = peaks()
    use_packed = args.experts == "packed"
    ms_step = r["ms_step"]
    line = {
        "metric": "MoE-layer tokens/s (decode)", "value": T * world / (ms_step * 1e-3), "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": ("NVFP4 weights x 4-term FP4 activations on tcgen05 kind::mxf4nvf4 (block-scaled), fp32 accumulation" if use_packed
                  else "fp16 x NVFP4 tensor-core products (mma.sync), fp32 accumulation"), "data": "synthetic",
        "config": dict(decode_config(sh, T),
                       l2_policy=f"weights cycle through {args.copies} layer copies ({w.packed.numel() * args.copies / 1e9:.1f} GB); a step touches {r['bytes_step'] / 1e6:.0f} MB, "
                                 f"so {args.copies} steps touch {r['bytes_step'] * args.copies / 1e6:.0f} MB before a copy repeats (L2: 126 MB)",
                       parallelism="single GPU",
                       expert_kernels="packed planes + tcgen05 block-scaled FP4" if use_packed else "ggml blobs in place + fp16 images + mma.sync",
                       layer_call=("one C ABI call per step (bsx_moe_layer): programmatic dependent launches, selection + plan + pass list in one kernel"
                                   if args.layer == "native" else "one C ABI call per operator (router, plan, experts, combine)"),
                       launch="one CUDA graph per step (input copied into its static buffer, device to device)" if not args.no_graph else "one host launch per kernel",
                       input_norm={"none": "not part of the step (rows arrive normed)", "fused": "RMS norm inside the step, fused with the FP4 activation images",
                                   "separate": "RMS norm inside the step, a launch of its own"}[args.input_norm]),
        "e2e": {"value": T * world / (r["ms_e2e"] * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": T * sh["H"] * (2 if args.act == "bf16" else 4),
                "d2h_bytes_per_step": T * sh["H"] * 4},
        "gpu_launches": r["launches"] * args.steps,
        "clocks": r["clocks"],
    }
    step_gbs = r["bytes_step"] / (ms_step * 1e-3) / 1e9
    line["step_roofline"] = {"bound": "hbm", "what": "every byte the step must read or write once (touched blobs, gate matrix, rows) over the whole step's device time",
                             "algorithmic_bytes": r["bytes_step"], "achieved": step_gbs, "peak": pk["hbm"], "unit": "GB/s", "frac": step_gbs / pk["hbm"],
                             "experts_touched": r["experts_touched"]}
    if "stage_ms" in r:
        gu_ms = r["stage_ms"]["experts_gate_up"]
        achieved = r["gu_bytes"] / (gu_ms * 1e-3) / 1e9
        line["roofline"] = {"bound": "hbm", "kernel": ("nvf4_stream_kernel<gate/up>" if use_packed else "nvfp4_mma_kernel<gate/up>") +
                            " (routed + shared experts; the stage's CUDA events also span the one-block kernel that lists the passes)", "achieved": achieved, "peak": pk["hbm"],
                            "unit": "GB/s", "frac": achieved / pk["hbm"], "peak_source": pk["source"],
                            # dram__bytes_read.sum + dram__bytes_write.sum of one gate/up launch of this workload at 64 tokens (seeded, so the same
                            # experts every run), from the ncu capture summarised in profiles/nvf4_stream_kernel_c1_t64.md; not measured by this run
                            "traffic": ((450112000 if use_packed else 451744256) if (T == 64 and w.key == "c1") else None),
                            "traffic_source": ("dram__bytes_read.sum + dram__bytes_write.sum of one launch, ncu capture of source revision b1578ff "
                                               "(profiles/nvf4_stream_kernel_c1_t64.md); per launch on the same workload, not measured by this run"),
                            "algorithmic_bytes_per_launch": r["gu_bytes"], "kernel_ms": gu_ms, "frac_of_nominal_8TBs": achieved / 8000.0}
        line["stage_ms"] = r["stage_ms"]
    else:
        line["roofline"] = dict(line["step_roofline"], kernel="whole step", peak_source=pk["source"], traffic=None)
    if "output_check_rel_l2_vs_fp16_path" in r:
        line["output_check_rel_l2_vs_fp16_path"] = r["output_check_rel_l2_vs_fp16_path"]
    return line


def short(line, keys=("ms_per_step", "value", "unit")):
    """a workload's entry in the headline's `workloads` array"""
    out = {"workload": line["config"]["workload"], "metric": line["metric"]}
    for k in keys:
        out[k] = line[k]
    out["steps"] = line["steps"]
    out["e2e"] = line["e2e"]["value"]
    r = line.get("step_roofline") or line["roofline"]
    out["roofline"] = {k: r[k] for k in ("bound", "achieved", "peak", "unit", "frac") if k in r}
    for extra in ("algorithmic_bytes", "algorithmic_flops_per_launch", "kernel_ms", "hbm_ms_of_touched_blobs", "tensor_ms_at_peak", "experts_touched", "frac_of_fp4_peak"):
        if extra in r:
            out["roofline"][extra] = r[extra]
    out["roofline"]["peak_source"] = peaks()["source"]
    if "stage_ms" in line and line["stage_ms"]:
        out["stage_ms"] = line["stage_ms"]
    out["clocks"] = line.get("clocks")
    return out


# --------------------------------------------------------------------------------------------------------- K / I-quant decode
def run_decode_codebook(args, dev, sh, steps=None, warmup=None, copies=None):
    """The decode step with K/IQ-format experts (the DeepSeek-style layer on one GPU): IQ1_M routed experts and a Q6_K shared
    expert, both read in place by the integer tensor-core kernels (experts_kq.cu: int8 activation terms, mma.sync u8 x s8).
    Reported: tokens/s and the bytes of the touched blobs over the step's time."""
    from basalt_b200 import capi, moe
    steps, warmup, copies = steps or args.steps, warmup or args.warmup, copies or args.copies
    H, E, I, K_TOP, T = sh["H"], sh["E"], sh["I"], sh["k"], args.decode_tokens
    rt, st_ = sh["routed_type"], sh["shared_type"]
    gate = (torch.randn((E, H), generator=torch.Generator(device=dev).manual_seed(0), device=dev) * 0.02).float()
    bias = (torch.randn(E, generator=torch.Generator(device=dev).manual_seed(7), device=dev) * 0.01).float()
    blobs, rb = random_codebook_blobs(dev, rt, E, H, I, 11)
    shared, sb = random_codebook_blobs(dev, st_, 1, H, I, 12)
    L = moe.native_expert_layout(rt, rt, H, I)
    Ls = moe.native_expert_layout(st_, st_, H, I)
    assert L.bytes == rb and Ls.bytes == sb
    if getattr(args, "plain_experts", False):      # the warp-per-row kernels instead (what every format without a tensor-core kernel runs)
        L.options |= capi.EXPERT_PLAIN
        Ls.options |= capi.EXPERT_PLAIN
    rargs = moe.RouterArgs(n_expert=E, n_embd=H, k=K_TOP, weight_scale=sh["scale"], gate=capi.GATE_SIGMOID, n_group=sh["n_group"],
                           topk_group=sh["topk_group"])
    layers = [moe.NativeMoELayer(gate, bias, blobs if c == 0 else blobs.clone(), L, rargs, shared_blob=(shared if c == 0 else shared.clone())[0],
                                 shared_layout=Ls, max_tokens=T) for c in range(copies)]
    g = torch.Generator(device=dev).manual_seed(1)
    xs = [torch.randn((T, H), generator=g, device=dev).bfloat16() for _ in range(4)]
    stream = torch.cuda.Stream(device=dev)
    with torch.cuda.stream(stream):
        for i in range(warmup):
            layers[i % copies].forward(xs[i % 4], None, stream)
        torch.cuda.synchronize()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler(dev.index or 0) as clocks:
            ev0.record(stream)
            for i in range(steps):
                layers[i % copies].forward(xs[i % 4], None, stream)
            ev1.record(stream)
            torch.cuda.synchronize()
        ms_step = ev0.elapsed_time(ev1) / steps
        x_host = [x.cpu().pin_memory() for x in xs]
        xin = torch.empty((T, H), dtype=torch.bfloat16, device=dev)
        y_host = torch.empty((T, H), dtype=torch.float32).pin_memory()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for i in range(steps):
            xin.copy_(x_host[i % 4], non_blocking=True)
            y_host.copy_(layers[i % copies].forward(xin, None, stream), non_blocking=True)
            stream.synchronize()
        e1.record(stream)
        torch.cuda.synchronize()
        ms_e2e = e0.elapsed_time(e1) / steps
        touched = int(torch.unique(layers[(steps - 1) % copies].ids[:T]).numel())
    pk = peaks()
    bytes_step = touched * rb + sb
    gbs = bytes_step / (ms_step * 1e-3) / 1e9
    line = {
        "metric": "MoE-layer tokens/s (decode)", "value": T / (ms_step * 1e-3), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "two int8 activation terms x integer weight codes (IQ1_M codebook, Q6_K) on mma.sync u8/s8 -> s32, block scales in fp32", "data": "synthetic (random valid blocks)",
        "config": dict(workload=f"{sh['name']} decode, {T} tokens/step", hidden=H, n_expert=E, n_shared=1, intermediate=I, top_k=K_TOP, router=sh["router"],
                       expert_format="IQ1_M routed (56 B / 256 values), Q6_K shared (210 B / 256 values)", activations="bf16", tokens_per_step=T,
                       l2_policy=f"weights cycle through {copies} layer copies; a step touches {bytes_step / 1e9:.2f} GB: larger than L2", parallelism="single GPU",
                       expert_kernels=("ggml blobs in place, warp-per-row fp32 kernels (experts_simple.cu)" if getattr(args, "plain_experts", False)
                                       else "ggml blobs in place, integer tensor-core kernels (experts_kq.cu)")),
        "e2e": {"value": T / (ms_e2e * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": T * H * 2, "d2h_bytes_per_step": T * H * 4},
        "gpu_launches": 11 * steps,   # logits, selection + plan, 2 x (images, product) routed, shared plan, 2 x (images, product) shared... combine
        "roofline": {"bound": "hbm", "kernel": "whole step (kq_mma_kernel<IQ1_M> gate/up and down dominate)", "achieved": gbs, "peak": pk["hbm"], "unit": "GB/s",
                     "frac": gbs / pk["hbm"], "peak_source": pk["source"], "traffic": None, "algorithmic_bytes": bytes_step, "experts_touched": touched},
        "clocks": clocks.summary(),
    }
    del layers
    torch.cuda.empty_cache()
    return line


def run_prefill_codebook(args, dev, sh, tokens=4096, steps=3, warmup=3):
    """The prompt-sized step over K/IQ-format experts read in place (the path the reference runs as its int8 MMQ product): the
    DeepSeek-style layer's IQ1_M routed experts, `tokens` rows a step, through router GEMM -> selection -> dispatch with the tile
    list -> bsx_experts_prefill (decoder warps feeding tcgen05 kind::f16) -> combine.  No shared expert in this entry: the routed
    product is what it measures.  Tensor roofline against the measured bf16 peak (the weights are decoded to fp16 operands)."""
    from basalt_b200 import capi, moe
    H, E, I, K_TOP = sh["H"], sh["E"], sh["I"], sh["k"]
    rt = sh["routed_type"]
    gate = (torch.randn((E, H), generator=torch.Generator(device=dev).manual_seed(0), device=dev) * 0.02).float()
    bias = (torch.randn(E, generator=torch.Generator(device=dev).manual_seed(7), device=dev) * 0.01).float()
    blobs, rb = random_codebook_blobs(dev, rt, E, H, I, 11)
    L = moe.native_expert_layout(rt, rt, H, I)
    assert L.bytes == rb
    rargs = moe.RouterArgs(n_expert=E, n_embd=H, k=K_TOP, weight_scale=sh["scale"], gate=capi.GATE_SIGMOID, n_group=sh["n_group"],
                           topk_group=sh["topk_group"])
    layer = moe.PrefillMoELayer(gate, bias, blobs, L, rargs, shared_blob=None, max_tokens=tokens, packed=False)
    g = torch.Generator(device=dev).manual_seed(1)
    xs = [torch.randn((tokens, H), generator=g, device=dev).bfloat16() for _ in range(2)]
    stream = torch.cuda.Stream(device=dev)
    with torch.cuda.stream(stream):
        for i in range(warmup):
            layer.forward(xs[i % 2], None, stream)
        torch.cuda.synchronize()
        layer.check_status()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler(dev.index or 0) as clocks:
            ev0.record(stream)
            for i in range(steps):
                layer.forward(xs[i % 2], None, stream)
            ev1.record(stream)
            torch.cuda.synchronize()
        ms_step = ev0.elapsed_time(ev1) / steps
        x_host = [x.cpu().pin_memory() for x in xs]
        xin = torch.empty((tokens, H), dtype=torch.bfloat16, device=dev)
        y_host = torch.empty((tokens, H), dtype=torch.float32).pin_memory()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for i in range(steps):
            xin.copy_(x_host[i % 2], non_blocking=True)
            y_host.copy_(layer.forward(xin, None, stream), non_blocking=True)
            stream.synchronize()
        e1.record(stream)
        torch.cuda.synchronize()
        ms_e2e = e0.elapsed_time(e1) / steps
        layer.events = []
        layer.forward(xs[0], None, stream)
        stream.synchronize()
        stage_ms = {nme: a.elapsed_time(b) for (_, a), (nme, b) in zip(layer.events[:-1], layer.events[1:])}
        layer.events = None
        layer.check_status()
    pk = peaks()
    flops = 6.0 * H * I * tokens * K_TOP
    achieved = flops / (stage_ms["experts"] * 1e-3) / 1e12
    line = {
        "metric": "MoE-layer tokens/s (prefill)", "value": tokens / (ms_step * 1e-3), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp16 x (IQ1_M decoded to fp16, scaled by 16) on tcgen05 kind::f16, fp32 accumulation in tensor memory", "data": "synthetic (random valid blocks)",
        "config": dict(workload=f"{sh['name']} prefill, IQ1_M routed experts in place, {tokens} tokens/step (no shared expert)", hidden=H, n_expert=E, n_shared=0,
                       intermediate=I, top_k=K_TOP, router=sh["router"], expert_format="IQ1_M (56 B / 256 values)", activations="bf16", tokens_per_step=tokens,
                       l2_policy="every step reads every touched expert blob", parallelism="single GPU"),
        "e2e": {"value": tokens / (ms_e2e * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": tokens * H * 2, "d2h_bytes_per_step": tokens * H * 4},
        "gpu_launches": 10 * steps,
        "roofline": {"bound": "tensor", "kernel": "prefill_gemm_kernel<IQ1_M> gate/up + down", "achieved": achieved, "peak": pk["bf16"], "unit": "TFLOP/s",
                     "frac": achieved / pk["bf16"], "peak_source": pk["source"], "traffic": None, "algorithmic_flops_per_launch": flops,
                     "kernel_ms": stage_ms["experts"]},
        "stage_ms": stage_ms, "clocks": clocks.summary(),
    }
    del layer, blobs
    torch.cuda.empty_cache()
    return line


# --------------------------------------------------------------------------------------------------------- prompt-sized steps
def zipf_logits(n_tokens, n_expert, gen, dev, s=1.1):
    """[T][E] fp32 scores whose top-k sets follow Zipf(s) popularity: log p_e + Gumbel noise, the popularity ranks dealt to
    expert ids by a seeded permutation (top-k of such scores = sampling k experts without replacement from p)."""
    p = torch.arange(1, n_expert + 1, device=dev, dtype=torch.float64) ** (-s)
    logp = torch.log(p / p.sum()).float()[torch.randperm(n_expert, generator=gen, device=dev)]
    u = torch.rand((n_tokens, n_expert), generator=gen, device=dev).clamp_(1e-20, 1.0 - 1e-7)
    return (logp[None, :] - torch.log(-torch.log(u))).contiguous()


def run_prefill(args, dev, rank=0, world=1, shape=None, tokens=None, steps=None, warmup=None, weights=None):
    """The prompt-sized workload: `tokens` rows a step per GPU on the layer `shape` names.  c1: expert popularity Zipf(1.1)
    (scores drawn; the reference's prompt benches have no dataset for this path either); c3: the router's own scores.
    One step = gate product (tensor cores) + selection + dispatch with the 128-row tile list + grouped experts on the tcgen05
    tensor cores (routed + shared) + combine.  With N > 1 ranks the routed experts are sharded (expert parallel, collective
    form: all-gather, local experts, reduce-scatter) and every rank brings `tokens` rows (weak scaling).  The roofline is the
    tensor one: 6 H I flops per expert row over the measured bf16 peak (four FP4 MMAs per K-step cost the tensor time of one
    fp16 MMA); the HBM time of the touched blobs is reported beside it.  Returns the JSON line as a dict (rank 0) or None."""
    from basalt_b200 import capi, ep, moe
    import torch.distributed as dist
    shape, Tn = shape or args.shape, tokens or args.tokens
    steps, warmup = steps or args.steps, warmup or args.warmup
    sh = SHAPES[shape]
    Hs, Es, Is, ks = sh["H"], sh["E"], sh["I"], sh["k"]
    El = Es // world
    use_packed = args.experts == "packed"
    L = moe.native_expert_layout(capi.TYPE_NVFP4, capi.TYPE_NVFP4, Hs, Is)
    if weights is not None and world == 1 and use_packed:
        gate, own, shared, bias = weights.gate, weights.packed[:Es], weights.packed[Es:Es + 1], weights.bias
    else:
        gate, own, blob_bytes = make_layer_weights(dev, E=Es, H=Hs, I=Is, first=rank * El, count=El)
        _, shared, _ = make_layer_weights(dev, E=Es, H=Hs, I=Is, first=Es, count=1)
        assert L.bytes == blob_bytes
        bias = (torch.randn(Es, generator=torch.Generator(device=dev).manual_seed(7), device=dev) * 0.01).float() if sh["bias"] else None
        if use_packed:
            own, shared = moe.pack_experts(L, own), moe.pack_experts(L, shared)
            torch.cuda.synchronize()
    gk = capi.GATE_SOFTMAX if sh["gate"] == "softmax" else capi.GATE_SIGMOID
    rargs = moe.RouterArgs(n_expert=Es, n_embd=Hs, k=ks, weight_scale=sh["scale"], gate=gk, n_group=sh["n_group"], topk_group=sh["topk_group"])
    g = torch.Generator(device=dev).manual_seed(1 + rank)
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
        for i in range(warmup):
            fwd(i)
        barrier()
        layer.check_status()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler(dev.index or 0) as clocks:
            ev0.record(stream)
            for i in range(steps):
                fwd(i)
            ev1.record(stream)
            barrier()
        ms_step = ev0.elapsed_time(ev1) / steps
        # end to end: pinned host rows in, host result out, every step
        x_host = [x.cpu().pin_memory() for x in xs]
        xin = torch.empty((Tn, Hs), dtype=torch.bfloat16, device=dev)
        y_host = torch.empty((Tn, Hs), dtype=torch.float32).pin_memory()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n_e2e = max(3, steps // 2)
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
            n_inst = min(steps, 10)
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
    layer.check_status()
    times = torch.tensor([ms_step, ms_e2e], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms_step, ms_e2e = times.tolist()
    del layer
    torch.cuda.empty_cache()
    if rank != 0:
        return None
    pk = peaks()
    flops = 6.0 * Hs * Is * (Tn * ks + Tn) * world
    # the tensor roofline of the expert stage (one GPU: its own stage time; N GPUs: the whole step, per GPU)
    exp_ms = stage_ms["experts"] if world == 1 else ms_step
    achieved = flops / world / (exp_ms * 1e-3) / 1e12
    blob_b = touched * (L.bytes - 16)
    roof = {"bound": "tensor", "kernel": (("prefill_nvf4_kernel" if use_packed else "prefill_gemm_kernel") + "<gate/up> + <down> (+ activation images)") if world == 1 else "whole step per GPU (experts + collectives)",
            "achieved": achieved, "peak": pk["bf16"], "unit": "TFLOP/s", "frac": achieved / pk["bf16"],
            "peak_source": pk["source"] + ": the bf16 burst figure, because an activation row enters as four FP4 terms, so a K-step costs four FP4 MMAs = the tensor time of one fp16 MMA",
            "frac_of_fp4_peak": achieved / (4.0 * pk["bf16"]), "fp4_peak_assumed": "4 x the measured bf16 burst peak (no FP4 figure is measured on this pool)",
            "traffic": None, "algorithmic_flops_per_launch": flops / world, "kernel_ms": exp_ms, "hbm_ms_of_touched_blobs": blob_b / (pk["hbm"] * 1e9) * 1e3,
            "tensor_ms_at_peak": flops / world / (pk["bf16"] * 1e12) * 1e3, "experts_touched": touched}
    if cnt is not None:
        roof.update(max_rows_per_expert=int(cnt.max()), median_rows_per_expert=float(np.median(cnt[:Es])))
    line = {
        "metric": "MoE-layer tokens/s (prefill)", "value": Tn * world / (ms_step * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": steps,
        "warmup": warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": ("NVFP4 weights x 4-term FP4 activations on tcgen05 kind::mxf4nvf4 (block-scaled), fp32 accumulation in tensor memory" if use_packed
                  else "fp16 x (NVFP4 decoded exactly to fp16) on tcgen05 kind::f16, fp32 accumulation in tensor memory"), "data": "synthetic",
        "config": dict(workload=f"{sh['name']} prefill, {Tn} tokens/step per GPU" + (", Zipf(1.1) expert popularity" if lgs[0] is not None else ""),
                       hidden=Hs, n_expert=Es, n_shared=1, intermediate=Is, top_k=ks, router=sh["gate"], n_group=sh["n_group"], topk_group=sh["topk_group"],
                       expert_format="NVFP4 (ggml block_nvfp4 + fp32 tail scales)", activations="bf16", tokens_per_step=Tn * world,
                       l2_policy=f"every step reads all touched expert blobs ({blob_b / 1e9:.2f} GB per GPU): larger than L2",
                       parallelism="single GPU" if world == 1 else f"ep{world}: {El} routed experts per GPU; all-gather of bf16 rows and routing, reduce-scatter of fp32 partial sums"),
        "e2e": {"value": Tn * world / (ms_e2e * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": Tn * Hs * 2 * world, "d2h_bytes_per_step": Tn * Hs * 4 * world},
        "gpu_launches": (12 if world == 1 else 16) * steps,   # image prep x2, gate GEMM, selection, 3 dispatch, activation prep, gate/up, down, combine (+ shared expert's three and the partial combine with N > 1)
        "roofline": roof, "stage_ms": stage_ms, "clocks": clocks.summary(),
    }
    return line


# --------------------------------------------------------------------------------------------------------- N > 1: expert parallel
def run_expert_parallel(args, rank, world, dev):
    """N > 1: the same layer with its 512 routed experts sharded over the ranks in contiguous blocks (expert parallel), 64
    tokens per rank and step (weak scaling: per-GPU tokens fixed); router and shared expert replicated; the token rows travel by
    NCCL collectives over NVLink (ep.py says which).  Device time, max over ranks."""
    import torch.distributed as dist
    from basalt_b200 import capi, ep, moe
    sh = SHAPES["c1"]
    H, E, I, K_TOP, T = sh["H"], sh["E"], sh["I"], sh["k"], args.decode_tokens
    El = E // world
    gate, mine, blob_bytes = make_layer_weights(dev, first=rank * El, count=El)        # every expert's values depend on its index only
    _, shared, _ = make_layer_weights(dev, first=E, count=1)
    L = moe.native_expert_layout(capi.TYPE_NVFP4, capi.TYPE_NVFP4, H, I)
    rargs = moe.RouterArgs(n_expert=E, n_embd=H, k=K_TOP, weight_scale=1.0, gate=capi.GATE_SOFTMAX)
    use_packed = args.experts == "packed"
    mine = torch.cat([mine, shared])
    if use_packed:
        mine = moe.pack_experts(L, mine)
    # the timed layers: the whole step as one C ABI call (bsx_ep_layer) on a communicator of this process's own
    comm = ep.NcclComm()
    layers = []
    for c in range(args.copies):
        b = mine.clone()
        layers.append(ep.EPMoELayerNative(gate.clone(), None, b[:El], L, rargs, E, comm, shared_blob=b[El], max_tokens=T, packed=use_packed))
    # the same step driven call by call from Python, for the per-stage times only (events between the stages)
    probe = ep.EPMoELayer(gate, None, mine[:El], L, rargs, E, shared_blob=mine[El], max_tokens=T, packed=use_packed)
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
        # per-stage device times of the step (events between the stages, launched call by call) and the local expert stage's bytes
        ly = probe
        stage_acc, exp_bytes = {}, []
        n_inst = min(args.steps, 30)
        for i in range(n_inst):
            ly.events = []
            ly.forward(xs[i % n_batches])
            stream.synchronize()
            evs = ly.events
            for (_, a), (nme, b) in zip(evs[:-1], evs[1:]):
                stage_acc[nme] = stage_acc.get(nme, 0.0) + a.elapsed_time(b)
            exp_bytes.append(int(ly.n_groups.item()) * (L.bytes - 16))
            dist.barrier()
        ly.events = None
        stage_ms = {k: v / n_inst for k, v in stage_acc.items()}
        for ly in layers + [probe]:
            ly.check_status()
        # the one-call step and the call-by-call step are the same kernels and collectives: their rows must agree
        y_nat = layers[0].forward(xs[0]).clone()
        y_py = probe.forward(xs[0]).clone()
        torch.cuda.synchronize()
        rel_check = float((y_nat - y_py).norm() / y_py.norm())
        assert rel_check < 1e-5, f"bsx_ep_layer differs from the call-by-call step (relative L2 {rel_check})"
        barrier()
    times = torch.tensor([ms_total, ms_e2e] + [stage_ms[k] for k in sorted(stage_ms)], dtype=torch.float64, device=dev)
    dist.all_reduce(times, op=dist.ReduceOp.MAX)
    vals = times.tolist()
    ms_total, ms_e2e = vals[0], vals[1]
    stage_max = dict(zip(sorted(stage_ms), vals[2:]))
    data_plane, launches_per_step = layers[0].DATA_PLANE, layers[0].LAUNCHES
    wl = None
    if not args.no_workloads and T == 64:
        # the DeepSeek-style layer, 8192 prompt tokens in total split over the ranks (strong scaling across N): every rank joins
        for l_ in layers:
            if l_.graph is not None:
                l_.graph.reset()
        layers.clear()
        del mine, ly, probe
        torch.cuda.empty_cache()
        wp = argparse.Namespace(**vars(args))
        wp.experts = "packed"
        n_tok = 8192 // world
        pl = run_prefill(wp, dev, rank, world, shape="c3", tokens=n_tok, steps=5, warmup=3)
        if pl is not None:
            pl["config"]["workload"] = f"{SHAPES['c3']['name']} prefill, 8192 tokens/step in total ({n_tok} per GPU x {world} GPUs: total work fixed as N grows)"
            wl = [short(pl)]
    if rank != 0:
        return
    ms_step = ms_total / args.steps
    pk = peaks()
    k_ms, k_bytes = stage_ms.get("experts", 0.0), sum(exp_bytes) / len(exp_bytes)
    achieved = k_bytes / (k_ms * 1e-3) / 1e9 if k_ms else 0.0
    line = {
        "metric": "MoE-layer tokens/s (decode)", "value": T * world / (ms_step * 1e-3), "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None,
        "dtype": ("NVFP4 weights x 4-term FP4 activations on tcgen05 kind::mxf4nvf4 (block-scaled), fp32 accumulation" if use_packed
                  else "fp16 x NVFP4 tensor-core products (mma.sync), fp32 accumulation"), "data": "synthetic",
        "config": dict(decode_config(sh, T), tokens_per_step=T * world, tokens_per_gpu=T,
                       parallelism=f"ep{world}: {E // world} routed experts per GPU, router and shared expert replicated; " + data_plane,
                       l2_policy=f"each rank cycles through {args.copies} copies of its expert shard",
                       expert_kernels="packed planes + tcgen05 block-scaled FP4" if use_packed else "ggml blobs in place + fp16 images + mma.sync",
                       launch="one CUDA graph per step, collectives included" if use_graph else "one host launch per kernel"),
        "e2e": {"value": T * world / (ms_e2e / args.steps * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": T * H * 2 * world,
                "d2h_bytes_per_step": T * H * 4 * world},
        "gpu_launches": launches_per_step * args.steps,
        "roofline": {"bound": "hbm", "kernel": "rank 0's local grouped experts (image prep, gate/up, down)", "achieved": achieved, "peak": pk["hbm"],
                     "unit": "GB/s", "frac": achieved / pk["hbm"], "peak_source": pk["source"], "traffic": None, "algorithmic_bytes_per_launch": k_bytes,
                     "kernel_ms": k_ms},
        "stage_ms": stage_max, "stage_ms_note": "max over ranks, steps launched call by call with events between the stages (the timed steps replay one graph)",
        "clocks": clocks.summary(),
    }
    line["check"] = {"one_call_step_vs_call_by_call_rel_l2": rel_check, "status_words": "clear"}
    if stage_max:
        outside = {k: v for k, v in stage_max.items() if k != "experts"}
        top = max(outside, key=outside.get) if outside else None
        line["limiter"] = (f"local experts {stage_max.get('experts', 0.0) * 1e3:.0f} us of {sum(stage_max.values()) * 1e3:.0f} us of stages; largest stage outside them: "
                           f"{top} {outside[top] * 1e3:.0f} us" if top else "local experts")
    if wl:
        line["workloads"] = wl
    print(json.dumps(line))


# --------------------------------------------------------------------------------------------------------- main
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-workloads", action="store_true", help="only the line's own workload (no `workloads` array): for profiler captures and quick runs")
    ap.add_argument("--copies", type=int, default=None, help="layer copies the steps cycle through (1 for a small profiler capture); default 4 at 64 tokens, 16 below")
    ap.add_argument("--experts", default="packed", choices=["packed", "fp16"],
                    help="decode expert kernels: packed = blobs repacked at load into planes, block-scaled FP4 tensor cores (tcgen05 kind::mxf4nvf4); "
                         "fp16 = ggml blobs in place, fp16 activation images, mma.sync")
    ap.add_argument("--layer", default="native", choices=["native", "calls"],
                    help="native: one C ABI call per step (bsx_moe_layer); calls: one call per operator, as the reference's layer loop issues them")
    ap.add_argument("--no-pdl", action="store_true", help="with --layer native: plain launches instead of programmatic dependent launches")
    ap.add_argument("--input-norm", default="none", choices=["none", "fused", "separate"],
                    help="decode workload: the layer also applies its input RMS norm (the reference's norm_pack step) - fused with the FP4 "
                         "activation images, or as a launch of its own")
    ap.add_argument("--act", default="bf16", choices=["bf16", "fp32"], help="decode workload: element type of the activation rows given to the layer")
    ap.add_argument("--no-fork", action="store_true", help="with --layer calls: the activation-image kernel runs on the step's own stream")
    ap.add_argument("--no-graph", action="store_true", help="launch every kernel of a step from the host instead of replaying the layer's CUDA graph")
    ap.add_argument("--decode-tokens", type=int, default=64, help="tokens per decode step and GPU (the reference's decode configs: 1, 8, 64; the metric is quoted on 64)")
    ap.add_argument("--workload", default="decode", choices=["decode", "prefill"],
                    help="decode: 64 tokens a step (the default line); prefill: --tokens rows a step, Zipf(1.1) expert popularity, tcgen05 grouped experts")
    ap.add_argument("--tokens", type=int, default=4096, help="rows per step of the prefill workload, per GPU (4096 or 16384 in the reference's configs)")
    ap.add_argument("--plain-experts", action="store_true", help="with --shape c4: the warp-per-row kernels instead of the integer tensor-core ones")
    ap.add_argument("--shape", default="c1", choices=sorted(SHAPES), help="layer: c1 (H 2048, 512 experts), c3 (H 7168, 256 experts), c4 (c3 with IQ1_M / Q6_K blobs)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    T = args.decode_tokens
    assert 1 <= T <= 64
    if args.copies is None:
        args.copies = (LAYER_COPIES if T >= 32 else 16) if args.shape == "c1" else 1
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
    from basalt_b200 import build, capi
    if rank == 0:
        build.build()
    if world > 1:
        dist.barrier()
    capi.lib()
    if args.workload == "prefill" and "routed_type" in SHAPES[args.shape]:
        print(json.dumps(run_prefill_codebook(args, dev, SHAPES[args.shape], tokens=args.tokens, steps=max(args.steps // 20, 3), warmup=3)))
        return
    if args.workload == "prefill":
        line = run_prefill(args, dev, rank, world)
        if line is not None:
            print(json.dumps(line))
        return
    if world > 1:
        return run_expert_parallel(args, rank, world, dev)
    sh = SHAPES[args.shape]
    if "routed_type" in sh:
        print(json.dumps(run_decode_codebook(args, dev, sh)))
        return

    headline = args.shape == "c1" and T == 64
    w = Weights(dev, args.shape, keep_ggml=args.shape == "c1")
    r = run_decode(w, T, args.steps, args.warmup, args.copies, dev, kind=args.layer, experts=args.experts, input_norm=args.input_norm, act=args.act,
                   graph=not args.no_graph, no_fork=args.no_fork, stages=True, check=args.shape == "c1", pdl=not args.no_pdl)
    line = decode_line(args, w, T, r)
    if not args.no_cpu_baseline and args.shape == "c1":
        try:
            g = torch.Generator(device=dev).manual_seed(1)
            xh = [torch.randn((T, sh["H"]), generator=g, device=dev).bfloat16().float().cpu().numpy() for _ in range(4)]
            line["cpu_baseline"] = cpu_baseline_block(w.gate.cpu().numpy(), w.ggml.cpu().numpy(), w.blob_bytes, xh, sh, T, 20 if T == 64 else 10)
        except Exception as exc:   # the baseline is reported, never required
            line["cpu_baseline"] = {"value": None, "unit": "tokens/s", "cores": 0, "kind": "port", "sample": f"failed: {exc}"}
    if headline and not args.no_workloads:
        # the other configurations, each a short run: same code paths, fewer steps
        wl = []
        sub = argparse.Namespace(**vars(args))
        sub.steps, sub.warmup = 20, 5
        for t_small in (1, 8):
            sub.copies, sub.decode_tokens = 16, t_small
            rs = run_decode(w, t_small, 50, 10, 16, dev, kind=args.layer, experts=args.experts, graph=not args.no_graph, pdl=not args.no_pdl)
            sub.steps = 50
            wl.append(short(decode_line(sub, w, t_small, rs)))
        sub.steps = 20
        wp = argparse.Namespace(**vars(args))
        wp.experts = "packed"
        pl = run_prefill(wp, dev, shape="c1", tokens=16384, steps=10, warmup=3, weights=w)
        wl.append(short(pl))
        del w
        torch.cuda.empty_cache()
        w3 = Weights(dev, "c3")
        sub.copies, sub.decode_tokens = 1, 64
        r3 = run_decode(w3, 64, 20, 5, 1, dev, kind=args.layer, experts="packed", graph=not args.no_graph, stages=True, pdl=not args.no_pdl)
        wl.append(short(decode_line(sub, w3, 64, r3)))
        pl3 = run_prefill(wp, dev, shape="c3", tokens=8192, steps=5, warmup=3, weights=w3)
        wl.append(short(pl3))
        del w3
        torch.cuda.empty_cache()
        sub.decode_tokens = 64
        wl.append(short(run_decode_codebook(sub, dev, SHAPES["c4"], steps=10, warmup=3, copies=1)))
        wl.append(short(run_prefill_codebook(sub, dev, SHAPES["c4"], tokens=4096, steps=3, warmup=3)))
        line["workloads"] = wl
    print(json.dumps(line))


if __name__ == "__main__":
    main()
