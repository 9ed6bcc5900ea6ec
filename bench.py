#!/usr/bin/env python
"""Benchmark of the quantized projection path on B200.

One step = every quantized projection of one decoded token of the synthetic
27B-class hybrid model (tessera_b200/workload.py: 497 projections, Q4_K/Q6_K
mix, about 14.6 GB of weights streamed per token at one GPU), driven through
the backend interface exactly as the reference's ProjectBatch drives its
backend.  Attention, the delta-rule scan, norms and sampling are not part of
the path and are not run.  Under `--gpus N` (torchrun) the projections are
tensor-parallel: column-parallel ones take n/N rows, row-parallel ones k/N
columns followed by an all-reduce of the 5120 partial sums.

Prints one JSON line (rank 0).  `--impl reference` times the reference's own
CPU functions for the same path instead.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from tessera_b200 import synth, workload  # noqa: E402

METRIC = "decode_projection_tok_s"
UNIT = "tok/s"


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


def config_dict(world: int):
    return {
        "workload": "27B-class decode step, quantized projections only (configs[3] shapes: hidden 5120, "
                    "64 layers, FFN 17408, vocab 151936, Q4_K/Q6_K mix), m=1",
        "projections_per_step": len(workload.decode_projections()),
        "parameters": workload.total_parameters(),
        "weight_bytes_per_rank": workload.total_weight_bytes(0, world),
        "parallelism": f"tp{world}",
        "allreduce": "none" if world == 1 else "in the row-parallel launch, peer stores over NVLink",
        "cache": "weights streamed per step exceed L2 a hundredfold; no flush needed",
    }


# --------------------------------------------------------------------------
# clocks
class ClockSampler:
    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {
            nv.nvmlClocksThrottleReasonSwPowerCap: "sw_power_cap",
            nv.nvmlClocksThrottleReasonHwSlowdown: "hw_slowdown",
            nv.nvmlClocksThrottleReasonSwThermalSlowdown: "sw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonHwThermalSlowdown: "hw_thermal_slowdown",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.01)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": []}
        return {"sm_mhz": float(np.median(self.samples)), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


# --------------------------------------------------------------------------
# CPU arms
def cpu_sample_shapes():
    """One projection of each distinct (dtype, n, k) with its multiplicity."""
    shapes = {}
    for p in workload.decode_projections():
        shapes.setdefault((p.dtype, p.n, p.k), 0)
        shapes[(p.dtype, p.n, p.k)] += 1
    return shapes


_CPU_INPUTS = {}
CPU_SAMPLE_ROWS = 4096


def run_cpu_sample(oracle, threads: int, budget_s: float, pool=None):
    """Times the CPU implementation on up to CPU_SAMPLE_ROWS rows of one
    projection per distinct shape, repeats the pass until `budget_s` of CPU
    work is spent, and scales by rows and multiplicity to a whole step.
    Returns (tok/s, description)."""
    shapes = cpu_sample_shapes()
    if not _CPU_INPUTS:
        for (dtype, n, k) in shapes:
            rows = min(n, CPU_SAMPLE_ROWS)
            w = synth.q4k_weights(rows, k, seed=1) if dtype == "q4k" else synth.q6k_weights(rows, k, seed=1)
            _CPU_INPUTS[(dtype, n, k)] = (rows, w, synth.activations(1, k, seed=2))
    spent, passes, est = 0.0, 0, []
    while spent < budget_s or passes == 0:
        step_s = 0.0
        for (dtype, n, k), count in shapes.items():
            rows, w, a = _CPU_INPUTS[(dtype, n, k)]
            fn = oracle.gemm_q4k if dtype == "q4k" else oracle.gemm_q6k
            t0 = time.perf_counter()
            if pool is None:
                fn(a, w, 1, rows, k, threads=threads)
            else:
                rb = (k // 256) * (144 if dtype == "q4k" else 210)
                chunk = (rows + threads - 1) // threads
                jobs = [(r0, min(rows, r0 + chunk)) for r0 in range(0, rows, chunk)]
                list(pool.map(lambda j: fn(a, w[j[0] * rb:j[1] * rb], 1, j[1] - j[0], k), jobs))
            dt = time.perf_counter() - t0
            spent += dt
            step_s += dt * (n / rows) * count
        est.append(step_s)
        passes += 1
    return 1.0 / float(np.median(est)), (
        f"up to {CPU_SAMPLE_ROWS} rows of one projection of each of the {len(shapes)} distinct shapes, "
        f"{passes} passes, {spent:.1f} s of CPU work on {threads} threads, scaled by rows and multiplicity to a full step")


def cpu_qgemv_rows(oracle, threads: int, pool=None, rows: int = 2048):
    """The CPU implementation on `rows` rows of the 17408 x 5120 decode GEMV in each weight
    format (m = 1), scaled to the whole matrix: microseconds and GB/s of weight bytes, to stand
    beside the GPU's single-projection table."""
    n, k = 17408, 5120
    a = synth.activations(1, k, seed=2)
    out = []
    for fmt in ("q4k", "q6k", "mxfp4", "fp8"):
        if fmt == "q4k":
            w, rb, fn = synth.q4k_weights(rows, k, seed=1), (k // 256) * 144, oracle.gemm_q4k
        elif fmt == "q6k":
            w, rb, fn = synth.q6k_weights(rows, k, seed=1), (k // 256) * 210, oracle.gemm_q6k
        elif fmt == "mxfp4":
            w, rb, fn = synth.mxfp4_weights(rows, k, seed=1), k // 2 + k // 32, oracle.gemm_mxfp4
        else:
            (w, sc), rb = synth.fp8_weights(rows, k, seed=1), k + 4
            fn = lambda a_, w_, m_, n_, k_, threads=0: oracle.gemm_fp8(a_, w_, sc[:n_], m_, n_, k_, threads=threads)
        parts = None
        if pool is not None and fmt in ("mxfp4", "fp8"):
            # row ranges per thread, each repacked in the format's own layout (outside the timing)
            chunk = (rows + threads - 1) // threads
            cuts = [(r0, min(rows, r0 + chunk)) for r0 in range(0, rows, chunk)]
            if fmt == "mxfp4":
                blob, scales = w[: rows * k // 2], w[rows * k // 2:]
                parts = [np.concatenate([blob[r0 * k // 2:r1 * k // 2], scales[r0 * k // 32:r1 * k // 32]]) for r0, r1 in cuts]
            else:
                parts = [(np.ascontiguousarray(w[r0 * k:r1 * k]), np.ascontiguousarray(sc[r0:r1])) for r0, r1 in cuts]
        best = None
        for _ in range(3):
            t0 = time.perf_counter()
            if pool is None:
                fn(a, w, 1, rows, k, threads=threads)
            elif fmt in ("q4k", "q6k"):
                chunk = (rows + threads - 1) // threads
                jobs = [(r0, min(rows, r0 + chunk)) for r0 in range(0, rows, chunk)]
                list(pool.map(lambda j: fn(a, w[j[0] * rb:j[1] * rb], 1, j[1] - j[0], k), jobs))
            elif fmt == "mxfp4":
                list(pool.map(lambda j: oracle.gemm_mxfp4(a, j, 1, j.size // rb, k), parts))
            else:
                list(pool.map(lambda j: oracle.gemm_fp8(a, j[0], j[1], 1, j[1].size, k), parts))
            dt = time.perf_counter() - t0
            best = dt if best is None else min(best, dt)
        us = best * 1e6 * n / rows
        out.append({"fmt": fmt, "m": 1, "n": n, "k": k, "us": round(us, 1), "gbs": round(n * rb / us / 1e3, 2),
                    "threads": threads, "rows_timed": rows})
    return out


def reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from concurrent.futures import ThreadPoolExecutor
    from oracle.oracle import Oracle, reference_available
    threads = os.cpu_count() or 1
    if reference_available():
        oracle, kind = Oracle(reference=True), "reference"
        pool = ThreadPoolExecutor(threads)
    else:
        oracle, kind, pool = Oracle(), "port", None
    for _ in range(max(args.warmup, 0)):
        run_cpu_sample(oracle, threads, 1.0, pool)
    values, sample = [], ""
    t0 = time.perf_counter()
    for _ in range(max(args.steps, 1)):
        v, sample = run_cpu_sample(oracle, threads, min(20.0, max(1.0, 90.0 / max(args.steps, 1))), pool)
        values.append(v)
    total = time.perf_counter() - t0
    value = float(np.mean(values))
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 / value, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": config_dict(args.gpus),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "wall_s": total,
        "qgemv_cpu": cpu_qgemv_rows(oracle, threads, pool),
    }
    print(json.dumps(line))


# --------------------------------------------------------------------------
# GPU arm
def qgemv_table(stream, hbm_peak, only=None, tensor_peak=None):
    """Device time per launch of the single-projection shapes the metric names: the Q4_K
    decode GEMV (17408 x 5120, m = 1) and the MXFP4 / FP8 projections at m = 1, 4, 16 over
    5120 x 5120, 17408 x 5120 and 5120 x 17408.  Each case rotates through enough private
    weight copies to exceed L2 three times over, runs from a CUDA graph and is timed with
    events on the launching stream; bytes are the algorithmic ones (weights once,
    activations in, outputs out)."""
    import ctypes
    import torch
    from tessera_b200 import capi
    lib = capi.load_library()
    st = ctypes.c_void_p(stream.cuda_stream)
    shapes = [(17408, 5120), (5120, 5120), (5120, 17408)]
    cases = [("q4k", 1, 17408, 5120), ("q4k", 1, 17408, 5120, 2), ("q6k", 1, 17408, 5120)]
    cases += [(f, m, n, k) for f in ("mxfp4", "fp8", "w4a8") for (n, k) in shapes for m in (1, 4, 16)]
    cases += [("bf16", 1, 17408, 5120), ("f32", 1, 256, 2048)]  # a bf16 checkpoint's projection; a router gate
    # a prefill chunk on the tcgen05 tile: tensor-bound
    cases += [("q4k", 512, 17408, 5120), ("q6k", 512, 17408, 5120), ("mxfp4", 512, 17408, 5120), ("fp8", 512, 17408, 5120)]
    if only is not None:
        cases = [only]
    rows, cache = [], {}
    group_backend = None
    for case in cases:
        fmt, m, n, k = case[:4]
        group = case[4] if len(case) > 4 else 1   # weight tensors per launch (Q4_K / Q6_K: tsr_gemv_group)
        # a case that names its group size, 1 included, goes through the merged-launch entry
        # point (the launch splits k as it sees fit); the others through the typed launchers
        grouped = len(case) > 4
        if grouped and group_backend is None:
            from tessera_b200.backend import CreateBackend
            group_backend = CreateBackend(stream=stream.cuda_stream)
            group_backend.SetDeviceIndex(torch.cuda.current_device())
            group_backend.Init()
        if (fmt, n, k) not in cache:
            cache.clear()
            torch.cuda.empty_cache()
            scale = None
            if fmt == "q4k":
                host = synth.q4k_weights(n, k, seed=11)
            elif fmt == "q6k":
                host = synth.q6k_weights(n, k, seed=11)
            elif fmt in ("mxfp4", "w4a8"):
                host = synth.mxfp4_weights(n, k, seed=11)
            elif fmt in ("bf16", "f32"):
                dense = np.random.default_rng(11).standard_normal((n, k)).astype(np.float32) * 0.05
                host = ((dense.view(np.uint32) >> 16).astype(np.uint16) if fmt == "bf16" else dense).reshape(-1).view(np.uint8)
            else:
                host, scale = synth.fp8_weights(n, k, seed=11)
                scale = torch.from_numpy(scale).cuda()
            first = torch.from_numpy(host).cuda()
            copies = max(3, int(np.ceil(400e6 / host.size)))
            copies = (copies + group - 1) // group * group
            cache[(fmt, n, k)] = ([first] + [first.clone() for _ in range(copies - 1)], scale, host.size)
        ws, scale, wbytes = cache[(fmt, n, k)]
        a = torch.from_numpy(synth.activations(m, k, seed=12)).cuda()
        c = torch.empty(m * n, dtype=torch.float32, device="cuda")
        # W4A8: per-token FP8 codes and factors (quantize_fp8_pack_rows), then the unsplit
        # gemm_mxfp4_wmma contract; the row-reference bytes are not read by the unsplit launch
        a8 = torch.empty(m * k, dtype=torch.uint8, device="cuda")
        a_scale = torch.empty(m, dtype=torch.float32, device="cuda")
        wref = torch.zeros(n, dtype=torch.uint8, device="cuda")

        outs = [torch.empty(m * n, dtype=torch.float32, device="cuda") for _ in range(group)]

        def launch(i):
            w = ctypes.c_void_p(ws[i % len(ws)].data_ptr())
            pa, pc = ctypes.c_void_p(a.data_ptr()), ctypes.c_void_p(c.data_ptr())
            if grouped:
                wp = (ctypes.c_void_p * group)(*[ws[(i * group + j) % len(ws)].data_ptr() for j in range(group)])
                cp = (ctypes.c_void_p * group)(*[o.data_ptr() for o in outs])
                nn = (ctypes.c_uint64 * group)(*([n] * group))
                rc = lib.tsr_gemv_group(group_backend._ctx, 0 if fmt == "q4k" else 1, pa, wp, cp, nn, group, m, k)
            elif fmt == "q4k":
                rc = lib.tsr_gemm_q4k(pa, w, pc, m, n, k, 1, st)
            elif fmt == "q6k":
                rc = lib.tsr_gemm_q6k(pa, w, pc, m, n, k, 1, st)
            elif fmt in ("bf16", "f32"):
                rc = lib.tsr_gemm_dense(1 if fmt == "bf16" else 0, pa, w, pc, m, n, k, st)
            elif fmt == "mxfp4":
                rc = lib.tsr_gemm_mxfp4(pa, w, pc, m, n, k, st)
            elif fmt == "w4a8":
                rc = lib.tsr_quantize_fp8_pack(pa, ctypes.c_void_p(a8.data_ptr()), ctypes.c_void_p(a_scale.data_ptr()),
                                               m, k, st)
                rc = rc or lib.tsr_gemm_mxfp4_w4a8(ctypes.c_void_p(a8.data_ptr()), w, ctypes.c_void_p(a_scale.data_ptr()),
                                                   ctypes.c_void_p(wref.data_ptr()), pc, m, n, k, 1, st)
            else:
                rc = lib.tsr_gemm_fp8(pa, w, ctypes.c_void_p(scale.data_ptr()), pc, m, n, k, st)
            if rc != 0:
                raise RuntimeError(f"{fmt} projection returned status {rc}")
        per_graph = 2 * len(ws) // group
        with torch.cuda.stream(stream):
            launch(0)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream, capture_error_mode="thread_local"):
                for i in range(per_graph):
                    launch(i)
            for _ in range(3):
                graph.replay()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            reps = 10
            e0.record(stream)
            for _ in range(reps):
                graph.replay()
            e1.record(stream)
            torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / (reps * per_graph)
        gbs = (group * (wbytes + m * n * 4) + m * k * 4) / us / 1e3
        row = {"fmt": fmt, "m": m, "n": n, "k": k, "us": round(us, 2), "gbs": round(gbs, 1),
               "frac": round(gbs / hbm_peak, 3)}
        if grouped:
            row["weights_per_launch"] = group
        if m >= 128:  # the tensor roofline: 2 m n k over the measured dense bf16 rate
            row["tflops"] = round(2.0 * m * n * k / us / 1e6, 1)
            if tensor_peak:
                row["tensor_frac"] = round(row["tflops"] / tensor_peak, 3)
        rows.append(row)
    cache.clear()
    if group_backend is not None:
        group_backend.close()
    return rows


def moe_row(stream, hbm_peak, hidden=2048, inter=512, experts=256, top_k=8):
    """Routed experts of one token and layer at the MoE configuration's shape (256 experts of
    2048 -> 512 -> 2048 in Q4_K, eight selected): moe_experts_gate_up_q4k followed by
    moe_experts_down_q4k, through the name-keyed launch, from a CUDA graph whose launches rotate
    through disjoint expert sets (the tensors hold 453 MB, so nothing is served from L2).
    Bytes: the selected experts' rows once (gate + up + down), activations and outputs."""
    import torch
    from tessera_b200.backend import CreateBackend, KernelLaunch
    backend = CreateBackend(stream=stream.cuda_stream)
    backend.SetDeviceIndex(torch.cuda.current_device())
    backend.Init()
    per_gu = inter * (hidden // 256) * 144
    per_d = hidden * (inter // 256) * 144
    g = np.random.default_rng(21)
    one_gu = synth.q4k_weights(inter, hidden, seed=21, index=1)
    one_d = synth.q4k_weights(hidden, inter, seed=21, index=2)
    gate = backend.upload(np.tile(one_gu, experts))
    up = backend.upload(np.tile(one_gu[::-1].copy(), experts))
    down = backend.upload(np.tile(one_d, experts))
    x = backend.upload((g.standard_normal(hidden) * 0.02).astype(np.float32))
    wts = backend.upload(np.full(top_k, 1.0 / top_k, dtype=np.float32))
    phi = backend.AllocateBuffer(top_k * inter * 4)
    out = backend.AllocateBuffer(hidden * 4)
    rounds = experts // top_k
    perm = g.permutation(experts).astype(np.uint32)
    ids = [backend.upload(perm[r * top_k:(r + 1) * top_k].copy()) for r in range(rounds)]
    k_gu, k_d = backend.LoadKernel("moe_experts_gate_up_q4k"), backend.LoadKernel("moe_experts_down_q4k")

    def layer(r):
        backend.LaunchKernel(k_gu, KernelLaunch(buffers=[x, gate, up, ids[r], phi], scalars=[hidden, inter, top_k, per_gu, per_gu]))
        backend.LaunchKernel(k_d, KernelLaunch(buffers=[phi, down, ids[r], wts, out], scalars=[hidden, inter, top_k, per_d, 0]))

    with torch.cuda.stream(stream):
        layer(0)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream, capture_error_mode="thread_local"):
            for r in range(rounds):
                layer(r)
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 10
        e0.record(stream)
        for _ in range(reps):
            graph.replay()
        e1.record(stream)
        torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / (reps * rounds)
    nbytes = top_k * (2 * per_gu + per_d) + hidden * 4 * 2 + top_k * inter * 4 * 2
    backend.close()
    return {"fmt": "moe_q4k", "hidden": hidden, "inter": inter, "experts": experts, "top_k": top_k, "launches": 2,
            "us": round(us, 2), "gbs": round(nbytes / us / 1e3, 1), "frac": round(nbytes / us / 1e3 / hbm_peak, 3)}


def delta_row(stream, hbm_peak, heads=48, dk=128, dv=128, layers=48):
    """The gated delta-rule step of the linear-attention layers (delta_step_heads, one token):
    every layer has its own recurrent state (48 heads x 128 x 128 fp32 = 3.1 MB, 151 MB over the 48
    layers, more than L2), read once and written once per step.  From a CUDA graph of the 48
    launches; bytes = state in and out, k, q, v, o."""
    import torch
    from tessera_b200.backend import CreateBackend, KernelLaunch
    backend = CreateBackend(stream=stream.cuda_stream)
    backend.SetDeviceIndex(torch.cuda.current_device())
    backend.Init()
    g = np.random.default_rng(31)
    states = [backend.upload((g.standard_normal(heads * dk * dv) * 0.1).astype(np.float32)) for _ in range(layers)]
    k = backend.upload((g.standard_normal(heads * dk) * 0.05).astype(np.float32))
    q = backend.upload(g.standard_normal(heads * dk).astype(np.float32))
    v = backend.upload(g.standard_normal(heads * dv).astype(np.float32))
    alpha = backend.upload(np.full(heads, 0.9, dtype=np.float32))
    beta = backend.upload(np.full(heads, 0.5, dtype=np.float32))
    o = backend.AllocateBuffer(heads * dv * 4)
    kern = backend.LoadKernel("delta_step_heads")
    with torch.cuda.stream(stream):
        def step():
            for s_ in states:
                backend.LaunchKernel(kern, KernelLaunch(buffers=[s_, k, v, q, o, alpha, beta], scalars=[heads, dk, dv, 1, 0, 0, 0]))
        step()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream, capture_error_mode="thread_local"):
            step()
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 10
        e0.record(stream)
        for _ in range(reps):
            graph.replay()
        e1.record(stream)
        torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / (reps * layers)
    nbytes = 2 * heads * dk * dv * 4 + 2 * heads * dk * 4 + 2 * heads * dv * 4
    backend.close()
    return {"fmt": "delta_step_heads", "heads": heads, "dk": dk, "dv": dv, "us": round(us, 2),
            "gbs": round(nbytes / us / 1e3, 1), "frac": round(nbytes / us / 1e3 / hbm_peak, 3)}


def attention_row(stream, hbm_peak, tag="f32", n=4096, heads=24, kv_heads=4, head_dim=256, layers=16):
    """One decode token's attention over the key / value cache (ids attention / attention_q8 / attention_fp8):
    every full-attention layer has its own cache (4096 keys x 4 kv heads x 256: 33.5 MB in fp32, 8.4 MB in
    FP8; 16 layers hold more than L2), read once per token.  From a CUDA graph of the 16 launches
    (two kernels each: chunks, merge); bytes = keys + values + scales + q + out."""
    import torch
    from tessera_b200.backend import CreateBackend, KernelLaunch
    backend = CreateBackend(stream=stream.cuda_stream)
    backend.SetDeviceIndex(torch.cuda.current_device())
    backend.Init()
    g = np.random.default_rng(37)
    row = kv_heads * head_dim
    esz = {"f32": 4, "f16": 2, "q8": 1, "fp8": 1}[tag]

    def cache():
        if tag == "f32":
            return backend.upload(g.standard_normal((n, row)).astype(np.float32))
        if tag == "f16":
            return backend.upload(g.standard_normal((n, row)).astype(np.float16).view(np.uint8))
        if tag == "q8":
            return backend.upload(g.integers(-127, 128, (n, row)).astype(np.int8).view(np.uint8))
        b = g.integers(0, 256, (n, row)).astype(np.uint8)
        b[(b & 0x7F) == 0x7F] = 0x3C
        return backend.upload(b)
    caches = [(cache(), cache()) for _ in range(layers)]
    scale = backend.upload(np.full(n, 0.01, dtype=np.float32))
    q = backend.upload(g.standard_normal(heads * head_dim).astype(np.float32))
    o = backend.AllocateBuffer(heads * head_dim * 4)
    if tag in ("f32", "f16"):
        kern = backend.LoadKernel("attention")
        launches = [KernelLaunch(buffers=[q, k, v, o], scalars=[1, n, heads, kv_heads, head_dim, n - 1, 0, 0, int(tag == "f16"), 1])
                    for k, v in caches]
    else:
        kern = backend.LoadKernel("attention_" + tag)
        launches = [KernelLaunch(buffers=[q, k, v, scale, scale, o],
                                 scalars=[1, n, heads, kv_heads, head_dim, n - 1, 0, 0, 0 if tag == "q8" else 2])
                    for k, v in caches]
    with torch.cuda.stream(stream):
        def step():
            for l in launches:
                backend.LaunchKernel(kern, l)
        step()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream, capture_error_mode="thread_local"):
            step()
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 10
        e0.record(stream)
        for _ in range(reps):
            graph.replay()
        e1.record(stream)
        torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / (reps * layers)
    nbytes = 2 * n * row * esz + (2 * n * 4 if esz == 1 else 0) + 2 * heads * head_dim * 4
    backend.close()
    return {"fmt": "attention_" + tag, "keys": n, "heads": heads, "kv_heads": kv_heads, "head_dim": head_dim,
            "us": round(us, 2), "gbs": round(nbytes / us / 1e3, 1), "frac": round(nbytes / us / 1e3 / hbm_peak, 3)}


class Recorder:
    """Stands in for the backend while the projection planner runs: kernels and buffers come
    from the real backend, launches are recorded instead of issued.  The recorded list is the
    reference's own launch sequence for the step (gemm_*_vec, gemm_vec_reduce, ...), submitted
    later with one tsr_launch_many call per step."""

    def __init__(self, backend, batch):
        self.backend, self.batch = backend, batch

    def LoadKernel(self, name, code=b""):
        return self.backend.LoadKernel(name, code)

    def AllocateBuffer(self, nbytes, kind=0):
        return self.backend.AllocateBuffer(nbytes, kind)

    def LaunchKernel(self, kernel, launch):
        self.batch.add(kernel, launch)


def profile_traffic(name):
    """`dram_bytes_per_launch: N` of a committed ncu summary, or None."""
    path = os.path.join(ROOT, "profiles", name)
    try:
        with open(path) as f:
            for line in f:
                if line.strip().startswith("dram_bytes_per_launch:"):
                    return int(line.split(":", 1)[1].strip().split()[0])
    except OSError:
        pass
    return None


def tp_parity(backend, comm, dist, rank, world, local):
    """Config 2 on the running ranks, outside the timed region: the 17408 -> 5120 down projection
    and the 6144 -> 5120 output projection, Q4_K, Q6_K and MXFP4, m = 1 and 16.  Every rank cuts
    its k range out of one full seeded tensor with the library's slicer, projects it and the
    library sums over ranks; the result is compared on all outputs with the same projection of
    the whole tensor on this GPU (the un-sharded TP = 1 result) and, by checksum, across ranks.
    The flat collective is checked bit for bit against the rank-order sum of the gathered inputs."""
    import hashlib
    from tessera_b200 import tp_check
    from tessera_b200.backend import KernelLaunch
    from tessera_b200.tp import rank_order_sum
    worst, identical, cases = 0.0, True, []
    for fmt, n, k in (("q4k", 5120, 17408), ("mxfp4", 5120, 17408), ("q6k", 5120, 17408), ("q4k", 5120, 6144)):
        for m in (1, 16):
            case = tp_check.make_case(fmt, m, n, k, seed=7)
            a, w, k_local = tp_check.rank_inputs(case, rank, world)
            ab, wb = backend.upload(a), backend.upload(w)
            out = backend.AllocateBuffer(m * n * 4)
            fa, fw = backend.upload(case.activations), backend.upload(case.weight)
            full = backend.AllocateBuffer(m * n * 4)
            tp_check.launch_unsharded(backend, case, fa, fw, full)
            want = backend.download(full, np.float32, m * n)
            for rep in range(2):  # the second pass replays what the first one queued
                tp_check.launch_rank(backend, case, ab, wb, out, k_local)
                got = backend.download(out, np.float32, m * n)
                err = tp_check.max_rel_err(got, want)
                worst = max(worst, err)
                sums = [None] * world
                dist.all_gather_object(sums, hashlib.sha1(got.tobytes()).hexdigest())
                identical = identical and len(set(sums)) == 1
            cases.append({"fmt": fmt, "m": m, "n": n, "k": k, "k_local": k_local, "max_rel_err": err})
            for buf in (ab, wb, out, fa, fw, full):
                buf.release()
    # the end of an FFN block (silu_mul, down projection with the sum over ranks, residual add:
    # one launch per rank once queued) against the same three steps over the whole k
    for fmt, m in (("q4k", 1), ("q6k", 1), ("q4k", 4)):
        n, k = 5120, 17408
        case = tp_check.make_case(fmt, m, n, k, seed=11)
        gen = np.random.default_rng(12)
        up_full = gen.standard_normal((m, k)).astype(np.float32)
        resid = gen.standard_normal(m * n).astype(np.float32)
        _, w, k_local = tp_check.rank_inputs(case, rank, world)
        from tessera_b200.tp import ROW, slice_shape
        _, cols, c0, _ = slice_shape(tp_check.FORMATS[fmt], ROW, n, k, rank, world)
        bufs = {
            "g": backend.upload(np.ascontiguousarray(case.activations[:, c0:c0 + cols])),
            "u": backend.upload(np.ascontiguousarray(up_full[:, c0:c0 + cols])),
            "act": backend.AllocateBuffer(m * cols * 4), "w": backend.upload(w), "down": backend.AllocateBuffer(m * n * 4),
            "res": backend.upload(resid), "fin": backend.AllocateBuffer(m * n * 4),
            "fg": backend.upload(case.activations), "fu": backend.upload(up_full), "fact": backend.AllocateBuffer(m * k * 4),
            "fw": backend.upload(case.weight), "fdown": backend.AllocateBuffer(m * n * 4), "ffin": backend.AllocateBuffer(m * n * 4),
        }
        tp_check.launch_ffn_tail(backend, case, bufs["fg"], bufs["fu"], bufs["fact"], bufs["fw"], bufs["fdown"], bufs["res"],
                                 bufs["ffin"], k, sharded=False)
        want = backend.download(bufs["ffin"], np.float32, m * n)
        want_act = backend.download(bufs["fact"], np.float32, m * k).reshape(m, k)[:, c0:c0 + cols]
        for rep in range(2):
            tp_check.launch_ffn_tail(backend, case, bufs["g"], bufs["u"], bufs["act"], bufs["w"], bufs["down"], bufs["res"],
                                     bufs["fin"], k_local, sharded=True)
            got = backend.download(bufs["fin"], np.float32, m * n)
            got_act = backend.download(bufs["act"], np.float32, m * cols).reshape(m, cols)
            err = max(tp_check.max_rel_err(got, want), tp_check.max_rel_err(got_act, want_act))
            worst = max(worst, err)
            sums = [None] * world
            dist.all_gather_object(sums, hashlib.sha1(got.tobytes()).hexdigest())
            identical = identical and len(set(sums)) == 1
        cases.append({"fmt": fmt, "m": m, "n": n, "k": k, "k_local": k_local, "steps": "silu_mul+down+add", "max_rel_err": err})
        for buf in bufs.values():
            buf.release()
    # flat all-reduce and its [m][n] form against the rank-order sum of everybody's input
    exact = True
    kern = backend.LoadKernel("allreduce_sum")
    for m, n in ((1, 5120), (16, 5120), (3, 520)):
        x = (np.random.default_rng(100 + rank).standard_normal(m * n) * 10.0 ** rank).astype(np.float32)
        xb = backend.upload(x)
        backend.LaunchKernel(kern, KernelLaunch(buffers=[xb], scalars=[m, n]))
        got = backend.download(xb, np.float32, m * n)
        parts = [None] * world
        dist.all_gather_object(parts, x)
        exact = exact and bool(np.array_equal(got, rank_order_sum(parts)))
        xb.release()
    errors = comm.error_count()
    result = {"max_rel_err": worst, "ranks_bit_identical": bool(identical), "allreduce_equals_rank_order_sum": exact,
              "tolerance": 2e-3, "peer_wait_errors": errors, "cases": cases}
    flags = [None] * world
    dist.all_gather_object(flags, (worst, identical, exact, errors))
    ok = all(f[0] <= 2e-3 and f[1] and f[2] and f[3] == 0 for f in flags)
    return result, ok


def collective_table(backend, dist, stream, local):
    """The library's peer-memory all-reduce and NCCL's on the same payloads (the row-parallel
    partial sums of m = 1 and m = 16: 20 KB and 320 KB of fp32), 200 calls back to back, timed
    with events on the launching stream, max over ranks.  peer_us: the calls go through the
    backend's deferred queue and replay as one CUDA graph, as they do inside a decode step;
    peer_eager_us and nccl_eager_us: every call issued by the host as it is made (both then
    include the host's per-call cost)."""
    import torch
    from tessera_b200.backend import KernelLaunch, LaunchBatch
    kern = backend.LoadKernel("allreduce_sum")
    rows = []
    for m in (1, 16):
        n = workload.HIDDEN
        xb = backend.upload(np.ones(m * n, dtype=np.float32))
        t = torch.ones(m * n, dtype=torch.float32, device=f"cuda:{local}")
        reps = 200
        batch = LaunchBatch()
        for _ in range(reps):
            batch.add(kern, KernelLaunch(buffers=[xb], scalars=[m, n]))

        def peer_graph():
            backend.LaunchMany(batch)
            backend.Flush()

        def peer_eager():
            for _ in range(reps):
                backend.LaunchKernel(kern, KernelLaunch(buffers=[xb], scalars=[m, n]))
                backend.Flush()

        def nccl():
            for _ in range(reps):
                dist.all_reduce(t)
        times = {}
        for name, fn in (("peer_us", peer_graph), ("peer_eager_us", peer_eager), ("nccl_eager_us", nccl)):
            for _ in range(3):  # the third identical queue is already a graph replay
                fn()
            torch.cuda.synchronize()
            dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            fn()
            e1.record(stream)
            torch.cuda.synchronize()
            ms = torch.tensor([e0.elapsed_time(e1)], device=f"cuda:{local}")
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
            times[name] = round(float(ms.item()) * 1e3 / reps, 2)
        rows.append({"floats": m * n, "bytes": m * n * 4, **times})
        xb.release()
    return rows


def gpu_arm(args):
    import torch
    import torch.distributed as dist

    from tessera_b200.backend import CreateBackend, KernelLaunch, LaunchBatch
    from tessera_b200.project import GemmKernelName, Projector

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    stream = torch.cuda.Stream()
    backend = CreateBackend(stream=stream.cuda_stream)
    backend.SetDeviceIndex(local)
    backend.Init()
    comm = None
    if world > 1:
        from tessera_b200.tp import TpComm
        comm = TpComm(local, rank, world, 16 * workload.HIDDEN)
        comm.connect(dist)
        backend.BindTensorParallel(comm)
    # Launches queue in the backend until the next copy or synchronisation, are merged there
    # and replayed as a CUDA graph from the second identical step on (TSR_BENCH_DEFERRED=0:
    # every launch of the reference's sequence is issued as it is made).
    deferred = int(os.environ.get("TSR_BENCH_DEFERRED", "1"))
    backend.SetDeferred(deferred)

    with torch.cuda.stream(stream):
        parity, parity_ok, collective = None, True, None
        if world > 1:
            if not args.no_tp_parity:
                parity, parity_ok = tp_parity(backend, comm, dist, rank, world, local)
            if not args.no_collective_table:
                collective = collective_table(backend, dist, stream, local)

        plan = workload.decode_projections()
        # ---- weights: one seeded host tensor per distinct local shape, a private
        # device copy per projection (distinct addresses, so nothing stays in L2)
        templates = {}
        weights = []
        for p in plan:
            n, k = workload.shard(p, rank, world) if args.shard_of <= 1 else workload.shard(p, 0, args.shard_of)
            key = (p.dtype, n, k)
            if key not in templates:
                host = synth.q4k_weights(n, k, seed=3) if p.dtype == "q4k" else synth.q6k_weights(n, k, seed=3)
                templates[key] = backend.upload(host)
            buf = backend.AllocateBuffer(templates[key].Size())
            backend.CopyD2D(templates[key], 0, buf, 0, buf.Size())
            weights.append((p, n, k, buf))
        backend.Synchronize()
        for t in templates.values():
            t.release()
        templates.clear()

        # ---- activations (host) and outputs: one output buffer per projection of a layer so
        # that projections which share their input stay independent of each other
        act_len = {"x": workload.HIDDEN}
        for p, n, k, _ in weights:
            act_len[p.act] = max(act_len.get(p.act, 0), k)
        host_act = {name: synth.activations(1, ln, seed=5, index=i).reshape(-1)
                    for i, (name, ln) in enumerate(act_len.items())}
        dev_act = {name: backend.upload(h) for name, h in host_act.items()}
        out_bufs = {}
        for p, n, k, _ in weights:
            if p.name != "output":
                out_bufs[p.name] = max(out_bufs.get(p.name, 0), n)
        out_bufs = {name: backend.AllocateBuffer(n * 4) for name, n in out_bufs.items()}
        logits_n = weights[-1][1]
        logits_buf = backend.AllocateBuffer(logits_n * 4)
        logits_host = np.empty(logits_n, dtype=np.float32)

        x_odd = backend.upload(host_act["x"])  # a second copy of the hidden state, see record()

        def record(only=None):
            """The reference's launch sequence for the step, as ProjectBatch makes it; the
            row-parallel projections of a tensor-parallel run use the ids that end with the sum
            over ranks instead of ProjectBatch + TpReduce.  With `only` (a subset of tensor
            names) the layers alternate between two copies of the hidden state, so that the
            backend merges what it merges inside the whole step (the projections of one layer
            that share their input) and not neighbours from different layers."""
            batch = LaunchBatch()
            proj = Projector(Recorder(backend, batch))
            for p, n, k, w in weights:
                if only is not None and p.name not in only:
                    continue
                dst = logits_buf if p.name == "output" else out_bufs[p.name]
                act = dev_act[p.act]
                if only is not None and p.act == "x" and p.layer % 2 == 1:
                    act = x_odd
                if world > 1 and p.kind == workload.ROW:
                    kern = backend.LoadKernel(GemmKernelName(p.dtype) + "_allreduce")
                    batch.add(kern, KernelLaunch(buffers=[act, w, dst], scalars=[1, n, k]))
                    continue
                proj.ProjectBatch(p.dtype, act, w, dst, 1, n, k)
            return batch, proj

        def token_mixers(keys):
            """Buffers and launches of what sits between a layer's input projections and its output
            projection (src/models/qwen3_5/trunk.cpp:360-455,745-775 of the reference), one decode token
            at position keys - 1.  Full-attention layers: qgate_split, per-head rmsnorm of q and k,
            mrope, the cache rows' append, attention over a private fp32 cache of `keys` rows,
            sigmoid_gate.  Linear-attention layers: ssm_gate, conv1d_state, l2norm, repeat_heads,
            delta_step_heads on a private recurrent state, rmsnorm_gated.  Returns (emit, keep)."""
            W = workload
            f = lambda n: backend.AllocateBuffer(n * 4)
            load = backend.LoadKernel
            g = np.random.default_rng(17)
            q_dim, kv_dim = W.Q_HEADS * W.HEAD_DIM, W.KV_HEADS * W.HEAD_DIM
            k_heads, head_k = 16, 128
            key_dim, width = k_heads * head_k, 4
            eps = int(np.float32(1e-6).view(np.uint32))
            fb = lambda v: int(np.float32(v).view(np.uint32))
            full_layers = [l for l in range(W.LAYERS) if l % W.FULL_ATTENTION_INTERVAL == W.FULL_ATTENTION_INTERVAL - 1]
            row = (g.standard_normal((1, kv_dim)) * 0.5).astype(np.float32)
            template = backend.upload(np.repeat(row, keys, axis=0))
            caches = {}
            for l in full_layers:
                caches[l] = (backend.AllocateBuffer(keys * kv_dim * 4), backend.AllocateBuffer(keys * kv_dim * 4))
                for c in caches[l]:
                    backend.CopyD2D(template, 0, c, 0, c.Size())
            states = {l: backend.upload((g.standard_normal(W.SSM_HEADS * head_k * 128) * 0.1).astype(np.float32))
                      for l in range(W.LAYERS) if l not in caches}
            hists = {l: backend.upload(g.standard_normal(W.SSM_QKV * (width - 1)).astype(np.float32)) for l in states}
            backend.Synchronize()
            template.release()
            b = dict(q=f(q_dim), gate=f(q_dim), pos=backend.upload(np.full((1, 3), keys - 1, dtype=np.uint64)),
                     head_w=backend.upload(np.ones(W.HEAD_DIM, dtype=np.float32)),
                     conv_w=backend.upload((g.standard_normal((W.SSM_QKV, width)) * 0.02).astype(np.float32)),
                     a_log=backend.upload((-np.exp(g.standard_normal(W.SSM_HEADS))).astype(np.float32)),
                     dt=backend.upload(g.standard_normal(W.SSM_HEADS).astype(np.float32)),
                     ssm_w=backend.upload(np.ones(128, dtype=np.float32)),
                     alpha=f(W.SSM_HEADS), beta=f(W.SSM_HEADS), q_l=f(key_dim), k_l=f(key_dim), v_l=f(W.SSM_INNER),
                     q_exp=f(W.SSM_HEADS * head_k), k_exp=f(W.SSM_HEADS * head_k), core=f(W.SSM_INNER))
            kern = {n: load(n) for n in ("qgate_split", "rmsnorm", "mrope", "copy_d2d", "attention", "sigmoid_gate", "ssm_gate",
                                         "conv1d_state", "l2norm", "repeat_heads", "delta_step_heads", "rmsnorm_gated")}

            def emit(batch, layer):
                add = lambda name, buffers, scalars: batch.add(kern[name], KernelLaunch(buffers=buffers, scalars=scalars))
                attn = dev_act["attn"]
                if layer in caches:
                    kc, vc = caches[layer]
                    add("qgate_split", [out_bufs["attn_q"], b["q"], b["gate"]], [W.Q_HEADS, W.HEAD_DIM, 1])
                    add("rmsnorm", [b["q"], b["head_w"], b["q"]], [W.Q_HEADS, W.HEAD_DIM, eps])
                    add("rmsnorm", [out_bufs["attn_k"], b["head_w"], out_bufs["attn_k"]], [W.KV_HEADS, W.HEAD_DIM, eps])
                    add("mrope", [b["q"], b["pos"]], [1, W.Q_HEADS, W.HEAD_DIM, 64, fb(1e7), 11, 11, 10])
                    add("mrope", [out_bufs["attn_k"], b["pos"]], [1, W.KV_HEADS, W.HEAD_DIM, 64, fb(1e7), 11, 11, 10])
                    add("copy_d2d", [out_bufs["attn_k"], kc], [0, (keys - 1) * kv_dim * 4, kv_dim * 4])
                    add("copy_d2d", [out_bufs["attn_v"], vc], [0, (keys - 1) * kv_dim * 4, kv_dim * 4])
                    add("attention", [b["q"], kc, vc, attn], [1, keys, W.Q_HEADS, W.KV_HEADS, W.HEAD_DIM, keys - 1, 0, 0, 0, 1])
                    add("sigmoid_gate", [attn, b["gate"], attn], [q_dim])
                else:
                    add("ssm_gate", [b["a_log"], b["dt"], out_bufs["ssm_alpha"], out_bufs["ssm_beta"], b["alpha"], b["beta"]],
                        [W.SSM_HEADS, 1])
                    add("conv1d_state", [out_bufs["attn_qkv"], b["conv_w"], hists[layer], b["q_l"], b["k_l"], b["v_l"], hists[layer]],
                        [W.SSM_QKV, width, key_dim, 0, 1, 0])
                    add("l2norm", [b["q_l"], b["q_l"]], [k_heads, head_k, fb(1e-6), fb(1.0 / np.sqrt(float(head_k)))])
                    add("l2norm", [b["k_l"], b["k_l"]], [k_heads, head_k, fb(1e-6), fb(1.0)])
                    add("repeat_heads", [b["q_l"], b["q_exp"]], [W.SSM_HEADS, head_k, W.SSM_HEADS // k_heads, 1])
                    add("repeat_heads", [b["k_l"], b["k_exp"]], [W.SSM_HEADS, head_k, W.SSM_HEADS // k_heads, 1])
                    add("delta_step_heads", [states[layer], b["k_exp"], b["v_l"], b["q_exp"], b["core"], b["alpha"], b["beta"]],
                        [W.SSM_HEADS, head_k, 128, 1, 0, 0, 0])
                    add("rmsnorm_gated", [b["core"], b["ssm_w"], out_bufs["attn_gate"], attn], [W.SSM_HEADS, 128, eps, 0, 0])
            return emit, (caches, states, hists, b)

        def record_with_elementwise(mixers=None):
            """The same projections with the elementwise steps the reference's forward queues
            around them (src/models/qwen3_5/trunk.cpp:279-322,440-470 of the reference): rmsnorm
            before the projections that read the hidden state, silu_mul between ffn_gate / ffn_up
            and ffn_down, the residual add after each row-parallel projection.  The hidden state
            itself is not advanced (the adds write a scratch vector), so the step repeats.  With
            `mixers` (token_mixers' emit) every layer also runs what lies between its input and
            output projections: the whole forward of the token."""
            batch = LaunchBatch()
            proj = Projector(Recorder(backend, batch))
            hid = workload.HIDDEN
            norm_w = backend.upload(np.ones(hid, dtype=np.float32))
            scratch = backend.AllocateBuffer(hid * 4)
            resid = backend.upload(host_act["x"][:hid])
            rms, silu, add = backend.LoadKernel("rmsnorm"), backend.LoadKernel("silu_mul"), backend.LoadKernel("add")
            eps = int(np.float32(1e-6).view(np.uint32))
            normed_for = None   # (layer, half) whose rmsnorm is already queued
            for p, n, k, w in weights:
                dst = logits_buf if p.name == "output" else out_bufs[p.name]
                if p.act == "x":
                    half = (p.layer, p.name.startswith("ffn"))
                    if half != normed_for:
                        batch.add(rms, KernelLaunch(buffers=[resid, norm_w, dev_act["x"]], scalars=[1, hid, eps]))
                        normed_for = half
                if p.name == "ffn_down":
                    batch.add(silu, KernelLaunch(buffers=[out_bufs["ffn_gate"], out_bufs["ffn_up"], dev_act["ffn"]], scalars=[k]))
                if mixers is not None and p.name in ("attn_output", "ssm_out"):
                    mixers(batch, p.layer)
                if world > 1 and p.kind == workload.ROW:
                    kern = backend.LoadKernel(GemmKernelName(p.dtype) + "_allreduce")
                    batch.add(kern, KernelLaunch(buffers=[dev_act[p.act], w, dst], scalars=[1, n, k]))
                else:
                    proj.ProjectBatch(p.dtype, dev_act[p.act], w, dst, 1, n, k)
                if p.kind == workload.ROW:
                    batch.add(add, KernelLaunch(buffers=[resid, dst, scratch], scalars=[n]))
            return batch, (proj, norm_w, scratch, resid)

        step, keep_step = record(only=set(args.only.split(",")) if args.only else None)
        if args.elementwise_step:   # experiment: time the step with its elementwise neighbours as the step
            step, keep_step = record_with_elementwise()
        dominant = ("ffn_gate", "ffn_up")
        dom, keep_dom = record(only=dominant)
        h2d_bytes = host_act["x"].nbytes
        d2h_bytes = logits_host.nbytes

        def run_step():
            backend.LaunchMany(step)
            backend.Flush()

        def run_dom():
            backend.LaunchMany(dom)
            backend.Flush()

        def e2e_step():
            backend.CopyH2D(dev_act["x"], host_act["x"])
            backend.LaunchMany(step)
            backend.CopyD2H(logits_buf, logits_host)

        def barrier():
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()

        def timed(fn, steps):
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(steps):
                fn()
            e1.record(stream)
            barrier()
            ms = e0.elapsed_time(e1)
            if world > 1:
                t = torch.tensor([ms], device=f"cuda:{local}")
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms = float(t.item())
            return ms

        warmup = max(args.warmup, 3)
        for _ in range(warmup):
            run_step()
        backend.Synchronize()
        api0, dev0, graphs0 = backend.LaunchStats()
        with ClockSampler(local) as clocks:
            ms_total = timed(run_step, args.steps)
            api1, dev1, graphs1 = backend.LaunchStats()
            for _ in range(2):
                e2e_step()
            ms_e2e = timed(e2e_step, args.steps)
            for _ in range(3):
                run_dom()
            backend.Synchronize()
            _, devd0, _ = backend.LaunchStats()
            ms_dom = timed(run_dom, args.steps)
            _, devd1, _ = backend.LaunchStats()

            # ---- the step with its elementwise neighbours, folded into the projection launches
            # and as launches of their own (outside the metric: it is quoted on the projections)
            with_elementwise, full_forward, prefill, verify = None, None, None, None
            step_bytes_n1 = workload.total_weight_bytes(0, 1)
            if deferred == 1 and not args.only and not args.no_elementwise:
                full, keep_full = record_with_elementwise()

                def run_full():
                    backend.LaunchMany(full)
                    backend.Flush()

                with_elementwise = {"launches_queued_per_step": len(full)}
                for mode, tag in ((1, "folded"), (3, "unfolded")):
                    backend.SetDeferred(mode)
                    for _ in range(3):
                        run_full()
                    backend.Synchronize()
                    _, k0, _ = backend.LaunchStats()
                    ms = timed(run_full, args.steps)
                    _, k1, _ = backend.LaunchStats()
                    with_elementwise["kernels_per_step_" + tag] = (k1 - k0) // args.steps
                    with_elementwise["ms_per_step_" + tag] = ms / args.steps
                backend.SetDeferred(deferred)
                if world == 1 and args.shard_of <= 1:
                    # the whole forward of one token: the step above plus every layer's token mixer
                    keys = 4096
                    emit, keep_mixers = token_mixers(keys)
                    forward, keep_forward = record_with_elementwise(mixers=emit)

                    def run_forward():
                        backend.LaunchMany(forward)
                        backend.Flush()

                    for _ in range(3):
                        run_forward()
                    backend.Synchronize()
                    _, k0, _ = backend.LaunchStats()
                    ms = timed(run_forward, args.steps)
                    _, k1, _ = backend.LaunchStats()
                    full_forward = {"context_keys": keys, "kv_cache": "f32", "launches_queued_per_token": len(forward),
                                    "kernels_per_token": (k1 - k0) // args.steps, "ms_per_token": ms / args.steps,
                                    "tok_s": args.steps / (ms * 1e-3)}
                    del forward, keep_forward, emit, keep_mixers
                    # batches: every projection of the model over 16 tokens (a speculative-verify step) and over 512
                    # (a prefill chunk) at once, through the ids ProjectBatch picks for the batch; activations and
                    # outputs resident
                    peaks_now, _ = measured_peaks()
                    tensor_peak = peaks_now.get("bf16_tflops_sustained", peaks_now.get("bf16_tflops", 1590.0))
                    for chunk in (16, 512):
                        pre_act = {name: backend.upload(synth.activations(chunk, ln, seed=6, index=i))
                                   for i, (name, ln) in enumerate(act_len.items())}
                        pre_out = {}
                        for p_, n_, _, _ in weights:
                            pre_out[p_.name] = max(pre_out.get(p_.name, 0), n_)
                        pre_out = {name: backend.AllocateBuffer(chunk * n_ * 4) for name, n_ in pre_out.items()}
                        pre_batch = LaunchBatch()
                        pre_proj = Projector(Recorder(backend, pre_batch))
                        flops = 0.0
                        for p_, n_, k_, w_ in weights:
                            pre_proj.ProjectBatch(p_.dtype, pre_act[p_.act], w_, pre_out[p_.name], chunk, n_, k_)
                            flops += 2.0 * chunk * n_ * k_

                        def run_batched():
                            backend.LaunchMany(pre_batch)
                            backend.Flush()

                        for _ in range(3):
                            run_batched()
                        backend.Synchronize()
                        pre_steps = max(3, args.steps // 4)
                        ms = timed(run_batched, pre_steps)
                        tf = flops * pre_steps / (ms * 1e-3) / 1e12
                        row = {"tokens": chunk, "ms": ms / pre_steps, "tok_s": chunk * pre_steps / (ms * 1e-3), "tflops": tf}
                        if chunk >= 128:
                            row["tensor_frac"] = tf / tensor_peak
                            row["tensor_peak"] = "bf16_tflops_sustained (a seconds-long loop)" if "bf16_tflops_sustained" in peaks_now else "bf16_tflops"
                            prefill = row
                        else:
                            row["hbm_gbs"] = step_bytes_n1 / (ms * 1e-3 / pre_steps) / 1e9
                            verify = row
                        del pre_batch, pre_proj
                        for b_ in list(pre_act.values()) + list(pre_out.values()):
                            b_.release()

    value = args.steps / (ms_total * 1e-3)
    e2e_value = args.steps / (ms_e2e * 1e-3)
    kernels_per_step = (dev1 - dev0) // args.steps
    # ---- roofline of the dominant kernel: the launch that serves ffn_gate and ffn_up of a layer
    peaks, peak_kind = measured_peaks()
    gate = next(x for x in weights if x[0].name == "ffn_gate")
    n_g, k_g = gate[1], gate[2]
    dom_kernels = max(1, (devd1 - devd0) // args.steps)
    dom_projections = sum(1 for p, _, _, _ in weights if p.name in dominant)
    per_launch = dom_projections // dom_kernels  # weight tensors one launch serves
    alg_bytes = per_launch * (workload.weight_bytes("q4k", n_g, k_g) + n_g * 4) + k_g * 4
    t_launch_s = ms_dom * 1e-3 / (args.steps * dom_kernels)
    achieved = alg_bytes / t_launch_s / 1e9
    traffic = profile_traffic("gemv_q4k_group_gate_up.md") if (n_g, k_g, per_launch) == (17408, 5120, 2) else None
    roofline = {
        "bound": "hbm", "kernel": "gemv_q4k_staged_kernel (ffn_gate + ffn_up of a layer in one launch)"
                                  if per_launch == 2 else "gemv_q4k_staged_kernel (gemm_q4k_vec)",
        "shape": [1, per_launch * n_g, k_g], "weights_per_launch": per_launch,
        "achieved": achieved, "peak": peaks["hbm_gbs"], "peak_kind": peak_kind, "unit": "GB/s",
        "frac": achieved / peaks["hbm_gbs"], "us_per_launch": t_launch_s * 1e6,
        "algorithmic_bytes": alg_bytes, "traffic": traffic,
        "launches_timed": args.steps * dom_kernels,
    }
    step_bytes = workload.total_weight_bytes(rank, world) if args.shard_of <= 1 else workload.total_weight_bytes(0, args.shard_of)
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": warmup, "ms_per_step": ms_total / args.steps, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None,
        "dtype": "f32 accumulate over Q4_K/Q6_K (int8 digits on the staged path)",
        "data": "synthetic", "config": config_dict(world) if args.shard_of <= 1 else {"experiment": f"rank 0 shard of tp{args.shard_of} on one GPU"},
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": d2h_bytes},
        "gpu_launches": kernels_per_step * args.steps,
        "kernels_per_step": kernels_per_step,
        "api_launches_per_step": (api1 - api0) // args.steps,
        "graph_launches_per_step": (graphs1 - graphs0) / args.steps,
        "submission": {0: "every launch issued as made", 1: "deferred queue, merged launches, CUDA graph replay",
                       2: "deferred queue, merged launches, no graphs"}.get(deferred, str(deferred)),
        "step_hbm_gbs_per_gpu": step_bytes / (ms_total * 1e-3 / args.steps) / 1e9,
        "roofline": roofline, "clocks": clocks.summary(),
    }
    if with_elementwise is not None:
        line["with_elementwise"] = with_elementwise
    if full_forward is not None:
        line["full_forward"] = full_forward
    if verify is not None:
        line["verify"] = verify
    if prefill is not None:
        line["prefill"] = prefill
    if parity is not None:
        line["tp_parity"] = parity
    if collective is not None:
        line["collective"] = collective
    if rank == 0 and world == 1 and not args.no_qgemv:
        # free the step's weights first: the table below wants a few hundred MB per case
        backend.SetDeferred(0)
        for _, _, _, buf in weights:
            buf.release()
        weights.clear()
        line["qgemv"] = qgemv_table(stream, peaks["hbm_gbs"], tensor_peak=peaks.get("bf16_tflops"))
        line["qgemv"].append(moe_row(stream, peaks["hbm_gbs"]))
        line["qgemv"].append(delta_row(stream, peaks["hbm_gbs"]))
        line["qgemv"].append(attention_row(stream, peaks["hbm_gbs"], "f32"))
        line["qgemv"].append(attention_row(stream, peaks["hbm_gbs"], "fp8"))
        from oracle.oracle import Oracle
        threads = os.cpu_count() or 1
        v, sample = run_cpu_sample(Oracle(), threads, 12.0)
        line["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample,
                                "qgemv": cpu_qgemv_rows(Oracle(), threads)}
    if rank == 0:
        print(json.dumps(line))
    backend.Synchronize()
    failed = comm is not None and comm.error_count() != 0
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if failed:
        raise RuntimeError("a tensor-parallel wait on a peer gave up; the results are not valid")
    if not parity_ok:
        raise RuntimeError("tensor-parallel parity check failed: " + json.dumps(parity))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--case", default=None, metavar="FMT:M:N:K[:G]",
                    help="time one projection (q4k, q6k, mxfp4, fp8, w4a8, bf16, f32; `moe` for the routed experts of one token, `delta` for the delta-rule state step, `attn:f32|f16|q8|fp8[:KEYS]` for one token's attention over the cache) "
                         "instead of the decode step, e.g. "
                         "q4k:1:17408:5120; with G (q4k, q6k): G weight tensors of that shape in one merged launch\n"
                         "that picks its own split of k")
    ap.add_argument("--only", default=None, metavar="NAMES",
                    help="experiment: the step holds only these projections (comma separated tensor names)")
    ap.add_argument("--no-qgemv", action="store_true", help="skip the single-projection table and the CPU baseline")
    ap.add_argument("--no-tp-parity", action="store_true",
                    help="experiment: skip the tensor-parallel parity check before the timed region")
    ap.add_argument("--shard-of", type=int, default=1, metavar="W",
                    help="experiment (1 GPU): the step holds rank 0's shard of a W-way tensor-parallel run, without "
                         "the sums over ranks (per-launch costs of the small shapes; not the metric)")
    ap.add_argument("--elementwise-step", action="store_true",
                    help="experiment: the timed step is the one with its rmsnorm / silu_mul / add neighbours (not the metric)")
    ap.add_argument("--no-elementwise", action="store_true",
                    help="skip the extra timing of the step with its rmsnorm / silu_mul / add neighbours")
    ap.add_argument("--no-collective-table", action="store_true",
                    help="skip the peer-memory / NCCL all-reduce comparison of a tensor-parallel run")
    args = ap.parse_args()
    if args.impl == "reference":
        reference_arm(args)
    elif args.case:
        import torch
        fields = args.case.split(":")
        if fields[0] == "delta":
            peaks, kind = measured_peaks()
            torch.cuda.set_device(0)
            print(json.dumps({"case": args.case, "peak_kind": kind, **delta_row(torch.cuda.Stream(), peaks["hbm_gbs"])}))
            return
        if fields[0] == "attn":
            peaks, kind = measured_peaks()
            torch.cuda.set_device(0)
            row = attention_row(torch.cuda.Stream(), peaks["hbm_gbs"], fields[1], int(fields[2]) if len(fields) > 2 else 4096)
            print(json.dumps({"case": args.case, "peak_kind": kind, **row}))
            return
        if fields[0] == "moe":
            peaks, kind = measured_peaks()
            torch.cuda.set_device(0)
            print(json.dumps({"case": args.case, "peak_kind": kind, **moe_row(torch.cuda.Stream(), peaks["hbm_gbs"])}))
            return
        fmt, (m, n, k) = fields[0], fields[1:4]
        only = (fmt, int(m), int(n), int(k)) + ((int(fields[4]),) if len(fields) > 4 else ())
        peaks, kind = measured_peaks()
        torch.cuda.set_device(0)
        row = qgemv_table(torch.cuda.Stream(), peaks["hbm_gbs"], only=only, tensor_peak=peaks.get("bf16_tflops"))[0]
        print(json.dumps({"case": args.case, "peak_kind": kind, **row}))
    else:
        gpu_arm(args)


if __name__ == "__main__":
    main()
