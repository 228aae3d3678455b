#!/usr/bin/env python
"""Benchmark of the GEMM hot path through the drop-in C ABI (libcublas.so.12 / libcublasLt.so.12 / libnccl.so.2).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One JSON line on stdout (rank 0). A "step" is one GEMM call of the workload:

  N = 1   cfg2_f16_tn_8192: cublasGemmEx, fp16 A/B (opA = T, opB = N), fp32 C, M = N = K = 8192, alpha = 1, beta = 0,
          operands normal(0, 0.02) rounded to fp16, seed 1. The three matrices hold 512 MiB, four times the L2, so every
          step streams its operands from HBM (no flush needed between steps).
  N > 1   cfg5b_bf16_32768_nsharded: the 32768^3 bf16 -> fp32 product split along N, rank r computing the column block
          C[:, r*32768/N : (r+1)*32768/N] with cublasLtMatmul in column chunks whose results are all-gathered over NVLink
          through this repository's libnccl.so.2 while the next chunk is multiplied (strong scaling: total work fixed).

`value` is the whole-job rate with operands resident in HBM; `e2e` is the same metric through the same C-ABI call but from
pinned HOST buffers, the host-to-device copies of A and B and the device-to-host copy of C inside the timed region.
`--impl reference` times k0zi/Vulkanizer's own CPU GEMM for this path (oracle/_ref, compiled from its sources) on the host
cores, on a bounded sample of the workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            d = json.loads(path.read_text())
            return d, "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.rows = []
        self.proc = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def stop(self, t0: float, t1: float):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        rows = [r for (t, r) in self.rows if t0 - 0.05 <= t <= t1 + 0.15 and len(r) >= 7] or [r for (_, r) in self.rows if len(r) >= 7]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        mhz = [float(r[0]) for r in rows if r[0].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[3 + i] == "Active" for r in rows)]
        return {"sm_mhz": statistics.median(mhz) if mhz else None, "sm_max_mhz": float(rows[0][1]) if rows[0][1].isdigit() else None,
                "reasons": reasons, "samples": len(rows), "power_w_max": max(float(r[2]) for r in rows if r[2].replace(".", "").isdigit())}


def physical_gpu_index(local: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local])
        except Exception:
            return local
    return local


# ---------------------------------------------------------------------------------------------------------------------
# CPU arm: the reference's own code for this path on the host cores
# ---------------------------------------------------------------------------------------------------------------------

def reference_sample_of(workload: str):
    """Which bounded sample of `workload` the host cores are timed on: (operand type, opA, opB, size, scale of the normal
    inputs). The reference's CPU GEMM takes f32, f16 and bf16; int8 operands go in as their values in f32 (timing only:
    the reference has no int8 product)."""
    spec = WORKLOADS.get(workload)
    if workload == "cfg5b_bf16_32768_nsharded":
        return "bf16", "T", "N", 2048, 1.0
    if spec is None:
        return "f16", "T", "N", 2048, 0.02
    kind = "f32" if spec["ab"] in ("s8", "f32") else spec["ab"]
    return kind, spec["ta"], spec["tb"], 2048 if spec["call"] != "sgemm" else 512, float(spec["dist"][1]) if spec["dist"][0] == "normal" else 1.0


def cpu_reference_sample(size: int = 2048, reps: int = 3, kind: str = "f16", ta: str = "T", tb: str = "N", scale: float = 0.02):
    """size^3 through the reference's staged CPU GEMM (packTransposed -> hostGemm on all cores -> epilogue), or through
    the C restatement when the compiled reference is absent. Returns (tflops, cores, kind, sample)."""
    import numpy as np
    from oracle import pyoracle as orc
    from vulkanizer_b200 import synth

    a = orc.to_storage(synth.normal(1, size * size, scale), kind)
    b = orc.to_storage(synth.normal(1, size * size, scale, first=size * size), kind)
    c = np.zeros(size * size, dtype=np.float32)
    code, opa, opb = orc.TYPE_CODE[kind], int(ta == "T"), int(tb == "T")
    ref = orc.reference()
    times = []
    if ref is not None:
        cores = ref.vkref_hardware_threads()
        for _ in range(reps + 1):
            t = time.perf_counter()
            used = ref.vkref_staged_gemm(opa, opb, size, size, size, 1.0, a.ctypes.data, code, size, b.ctypes.data, code, size, 0.0, c.ctypes.data, 0, size)
            times.append(time.perf_counter() - t)
        how, cores = "reference", used or cores
    else:
        size = min(size, 512)
        a, b, c = a[:size * size], b[:size * size], c[:size * size]
        for _ in range(2):
            t = time.perf_counter()
            orc.gemm_f32(bool(opa), bool(opb), size, size, size, 1, 1.0, a, kind, size, 0, b, kind, size, 0, 0.0, c, "f32", size, 0)
            times.append(time.perf_counter() - t)
        how, cores = "port", 1
    best = statistics.median(times[1:])
    return (2.0 * size ** 3 / best / 1e12, cores, how,
            f"{kind} {ta}{tb} {size}^3, alpha=1 beta=0, median of {len(times) - 1} runs after one warm-up")


def run_reference_arm(args):
    """The reference's own CPU implementation of the path on the host cores, on a bounded sample of the workload the other arm
    runs with the same arguments (one GPU: --workload or the headline configuration; several: the column-sharded product)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    world = int(os.environ.get("WORLD_SIZE", "1"))
    workload = args.workload or ("cfg5b_bf16_32768_nsharded" if max(world, args.gpus) > 1 else "cfg2_f16_tn_8192")
    kind, ta, tb, size, scale = reference_sample_of(workload)
    times = []
    tf = cores = how = sample = None
    for _ in range(max(1, args.warmup // 3)):
        cpu_reference_sample(min(size, 1024), 1, kind, ta, tb, scale)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        tf, cores, how, sample = cpu_reference_sample(size, 1, kind, ta, tb, scale)
        times.append(tf)
        if time.perf_counter() - t0 > 120:
            break
    value = statistics.median(times)
    line = {"impl": "reference", "metric": "gemm_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": len(times),
            "warmup": args.warmup, "ms_per_step": 2.0 * size ** 3 / value / 1e9, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": WORKLOADS.get(workload, {}).get("ab", "bf16"), "data": "synthetic",
            "config": {"workload": f"{workload} (bounded sample: {size}^3 per step on the host cores)", "m": size, "n": size, "k": size},
            "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": how, "sample": sample},
            "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------------------------------
# GPU arm, one GPU: configuration 2
# ---------------------------------------------------------------------------------------------------------------------

WORKLOADS = {
    # name: call, A/B type, C type, opA, opB, m, n, k, batch, alpha, beta, distribution, seed, bound
    "cfg1_sgemm_nn_512": dict(call="sgemm", ab="f32", c="f32", ta="N", tb="N", m=512, n=512, k=512, batch=1, alpha=1.0, beta=0.5,
                              dist=("uniform", 1.0), seed=0, bound="ffma"),
    "cfg2_f16_tn_8192": dict(call="gemmex", ab="f16", c="f32", ta="T", tb="N", m=8192, n=8192, k=8192, batch=1, alpha=1.0, beta=0.0,
                             dist=("normal", 0.02), seed=1, bound="tensor"),
    "cfg2_bf16_tn_8192": dict(call="gemmex", ab="bf16", c="f32", ta="T", tb="N", m=8192, n=8192, k=8192, batch=1, alpha=1.0, beta=0.0,
                              dist=("normal", 0.02), seed=1, bound="tensor"),
    "cfg3_s8_tn_11008x512x4096": dict(call="gemmex", ab="s8", c="s32", ta="T", tb="N", m=11008, n=512, k=4096, batch=1, alpha=1, beta=0,
                                      dist=("int8", 127), seed=2, bound="tensor"),
    "cfg3_s8_tn_4096x512x11008": dict(call="gemmex", ab="s8", c="s32", ta="T", tb="N", m=4096, n=512, k=11008, batch=1, alpha=1, beta=0,
                                      dist=("int8", 127), seed=2, bound="tensor"),
    "cfg4_f16_tn_batched_qk": dict(call="strided", ab="f16", c="f32", ta="T", tb="N", m=1024, n=1024, k=128, batch=256,
                                   alpha=128 ** -0.5, beta=0.0, dist=("normal", 1.0), seed=3, bound="hbm"),
    "cfg5a_f16_gemv_4096": dict(call="gemmex", ab="f16", c="f32", ta="T", tb="N", m=4096, n=1, k=4096, batch=1, alpha=1.0, beta=0.0,
                                dist=("normal", 0.02), seed=4, bound="hbm"),
    "cfg5a_f16_gemv_11008": dict(call="gemmex", ab="f16", c="f32", ta="T", tb="N", m=11008, n=1, k=4096, batch=1, alpha=1.0, beta=0.0,
                                 dist=("normal", 0.02), seed=4, bound="hbm"),
    # a smaller sibling of cfg2 for profiler captures (operands 96 MiB + C 64 MiB)
    "profile_f16_tn_4096": dict(call="gemmex", ab="f16", c="f32", ta="T", tb="N", m=4096, n=4096, k=4096, batch=1, alpha=1.0, beta=0.0,
                                dist=("normal", 0.02), seed=1, bound="tensor"),
    "profile_s8_tn_4096": dict(call="gemmex", ab="s8", c="s32", ta="T", tb="N", m=4096, n=4096, k=4096, batch=1, alpha=1, beta=0,
                               dist=("int8", 127), seed=2, bound="tensor"),
}
ELEM = {"f32": 4, "f16": 2, "bf16": 2, "s8": 1, "s32": 4}
L2_BYTES = 126 * 1024 * 1024


def host_operand(torch, spec, count: int, first: int):
    """Pinned host tensor with `count` elements of the workload's distribution (element i depends on seed and i only)."""
    import numpy as np
    from vulkanizer_b200 import synth

    kind, (dist, scale), seed = spec["ab"], spec["dist"], spec["seed"]
    tdt = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16, "s8": torch.int8}[kind]
    host = torch.empty(count, dtype=tdt).pin_memory()
    raw = host.view(torch.int16).numpy().view(np.uint16) if kind in ("f16", "bf16") else host.numpy()
    for start, n in synth.blocks(count):
        if dist == "int8":
            raw[start:start + n] = synth.int8_uniform(seed, n, first=first + start)
            continue
        v = synth.normal(seed, n, scale, first=first + start) if dist == "normal" else synth.uniform(seed, n, -scale, scale, first=first + start)
        if kind == "f32":
            raw[start:start + n] = v
        elif kind == "f16":
            raw[start:start + n] = v.astype(np.float16).view(np.uint16)
        else:
            u = v.view(np.uint32).astype(np.uint64)
            raw[start:start + n] = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    return host


def yardstick(torch, kind: str) -> float:
    """The rate NVIDIA's own library reaches on this box for a dense product of `kind`, measured now with CUDA events: the
    denominator for the kernels MEASURED_PEAKS.json has no figure for. 's8': int8 -> int32 8192^3 (TOP/s); 'f32': fp32 4096^3."""
    size, reps = (8192, 10) if kind == "s8" else (4096, 5)
    if kind == "s8":
        a = torch.randint(-127, 128, (size, size), dtype=torch.int8, device="cuda")
        b = torch.randint(-127, 128, (size, size), dtype=torch.int8, device="cuda").t()
        run = lambda: torch._int_mm(a, b)
    else:
        torch.backends.cuda.matmul.allow_tf32 = False
        a = torch.randn(size, size, device="cuda")
        b = torch.randn(size, size, device="cuda")
        run = lambda: torch.matmul(a, b)
    for _ in range(3):
        run()
    torch.cuda.synchronize()
    best = float("inf")
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(reps):
        start.record()
        run()
        stop.record()
        torch.cuda.synchronize()
        best = min(best, start.elapsed_time(stop))
    del a, b
    return 2.0 * size ** 3 / (best * 1e-3) / 1e12


def run_single_gpu(args):
    import torch
    from vulkanizer_b200 import capi

    name = args.workload or "cfg2_f16_tn_8192"
    spec = WORKLOADS[name]
    torch.cuda.set_device(0)
    torch.zeros(1, device="cuda")
    m, n, k, batch = spec["m"], spec["n"], spec["k"], spec["batch"]
    ab, ct = spec["ab"], spec["c"]
    ta = capi.OP_T if spec["ta"] == "T" else capi.OP_N
    tb = capi.OP_T if spec["tb"] == "T" else capi.OP_N
    rows_a, cols_a = (k, m) if ta == capi.OP_T else (m, k)
    rows_b, cols_b = (n, k) if tb == capi.OP_T else (k, n)
    lda, ldb, ldc = rows_a, rows_b, m
    sA, sB, sC = rows_a * cols_a, rows_b * cols_b, m * n
    cuda_type = {"f32": capi.CUDA_R_32F, "f16": capi.CUDA_R_16F, "bf16": capi.CUDA_R_16BF, "s8": capi.CUDA_R_8I, "s32": capi.CUDA_R_32I}
    compute = capi.COMPUTE_32I if ab == "s8" else capi.COMPUTE_32F
    ctorch = torch.int32 if ct == "s32" else torch.float32
    bytes_in = (sA + sB) * batch * ELEM[ab]
    bytes_out = sC * batch * ELEM[ct]
    algorithmic_bytes = bytes_in + bytes_out * (2 if spec["beta"] != 0 else 1)

    hostA = host_operand(torch, spec, sA * batch, 0)
    hostB = host_operand(torch, spec, sB * batch, sA * batch)
    hostC = torch.empty(sC * batch, dtype=ctorch).pin_memory()
    # Small workloads would be served from L2 if the same buffers were reused: rotate through enough copies of
    # the operands that a step never finds its inputs cached.
    copies = 1 if algorithmic_bytes > 2 * L2_BYTES else int(2 * L2_BYTES // algorithmic_bytes) + 2
    dAs = [hostA.cuda() for _ in range(copies)]
    dBs = [hostB.cuda() for _ in range(copies)]
    dCs = [torch.zeros(sC * batch, dtype=ctorch, device="cuda") for _ in range(copies)]
    if spec["beta"] != 0:
        for c in dCs:
            c.copy_(torch.from_numpy(__import__("vulkanizer_b200.synth", fromlist=["x"]).uniform(spec["seed"] + 100, sC * batch)).to(ctorch))
    blas = capi.Cublas()
    stream = torch.cuda.Stream()
    blas.set_stream(stream.cuda_stream)
    counter = [0]

    def call(i):
        A, B, Cd = dAs[i % copies].data_ptr(), dBs[i % copies].data_ptr(), dCs[i % copies].data_ptr()
        if spec["call"] == "sgemm":
            blas.sgemm(ta, tb, m, n, k, spec["alpha"], A, lda, B, ldb, spec["beta"], Cd, ldc)
        elif spec["call"] == "strided":
            blas.gemm_strided_batched_ex(ta, tb, m, n, k, spec["alpha"], A, cuda_type[ab], lda, sA, B, cuda_type[ab], ldb, sB, spec["beta"],
                                         Cd, cuda_type[ct], ldc, sC, batch, compute)
        else:
            blas.gemm_ex(ta, tb, m, n, k, spec["alpha"], A, cuda_type[ab], lda, B, cuda_type[ab], ldb, spec["beta"], Cd, cuda_type[ct], ldc,
                         compute, capi.GEMM_DEFAULT_TENSOR_OP)

    def step():
        call(counter[0])
        counter[0] += 1

    # Launch-bound workloads (a few microseconds of kernel) are replayed from a CUDA graph holding whole passes over the
    # rotating buffers (at least 32 calls, so that the cost of launching the graph itself is spread thin), so that the
    # device time per step is the kernel's and not the host's call overhead.
    flops = 2.0 * m * n * k * batch
    use_graph = flops < 2e11
    graph = None
    with torch.cuda.stream(stream):
        for _ in range(max(3, args.warmup)):
            step()
        stream.synchronize()
        path = blas.last_path()
        if use_graph:
            graph = torch.cuda.CUDAGraph()
            graph_calls = copies * -(-32 // copies)
            with torch.cuda.graph(graph, stream=stream):
                for i in range(graph_calls):
                    call(i)
            graph.replay()
            stream.synchronize()
    launches0 = blas.launch_count()
    sampler = ClockSampler(physical_gpu_index(0))
    time.sleep(0.3)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.time()
    with torch.cuda.stream(stream):
        stream.synchronize()
        if use_graph:
            replays = max(1, -(-args.steps // graph_calls))
            steps_done = replays * graph_calls
            start.record(stream)
            for _ in range(replays):
                graph.replay()
            stop.record(stream)
            graph_launches = steps_done
        else:
            steps_done = args.steps
            start.record(stream)
            for _ in range(steps_done):
                step()
            stop.record(stream)
            graph_launches = 0
        stream.synchronize()
    t1 = time.time()
    clocks = sampler.stop(t0, t1)
    launches = blas.launch_count() - launches0 + graph_launches
    total_ms = start.elapsed_time(stop)
    kernel_ms = total_ms / steps_done
    value_tf = flops * steps_done / (total_ms * 1e-3) / 1e12
    assert blas.device_status() == 0, "a bounded wait in the tcgen05 kernel gave up"

    # tensor-bound products of seconds' worth: the same call back to back for two seconds, against the sustained cuBLAS
    # figure (the timed region above is a burst of a few milliseconds at the full clock)
    sustained = None
    if spec["bound"] == "tensor" and not use_graph and ab != "s8":
        sampler2 = ClockSampler(physical_gpu_index(0))
        with torch.cuda.stream(stream):
            stream.synchronize()
            t_s0 = time.time()
            done_calls = 0
            start.record(stream)
            while time.time() - t_s0 < 2.0:
                for _ in range(10):
                    step()
                done_calls += 10
                stream.synchronize()
            stop.record(stream)
            stream.synchronize()
        t_s1 = time.time()
        clocks2 = sampler2.stop(t_s0, t_s1)
        sus_tf = flops * done_calls / (start.elapsed_time(stop) * 1e-3) / 1e12
        sus_peak = float(measured_peaks()[0].get("bf16_tflops_sustained", FALLBACK_PEAKS["bf16_tflops_sustained"]))
        sustained = {"achieved": sus_tf, "peak": sus_peak, "frac": sus_tf / sus_peak, "unit": "TFLOP/s", "seconds": round(t_s1 - t_s0, 2), "calls": done_calls,
                     "sm_mhz": clocks2.get("sm_mhz"), "reasons": clocks2.get("reasons"),
                     "peak_source": "measured: cuBLAS bf16 8192^3 back to back for seconds (bf16_tflops_sustained)"}

    # End to end through the same C-ABI calls from pinned host buffers: copy A and B in, multiply, copy C out, every
    # step. A product with enough columns (or batch entries) goes in blocks: block j of B travels to the device while block
    # j - 1 is multiplied and block j - 2 of C travels back, on three streams, so both directions of the host link stay busy.
    blocks = 8 if (batch == 1 and n >= 2048 and n % 8 == 0 and spec["call"] == "gemmex" and spec["tb"] == "N") else 1
    copy_in, copy_out = torch.cuda.Stream(), torch.cuda.Stream()
    # Two sets of device buffers take turns, so that the operands of step s + 1 travel while step s is still being multiplied
    # and its result is still on its way back: the link to the host, not the GPU, bounds this figure, and it is busy in both
    # directions the whole time.
    sets = 2 if blocks > 1 else 1
    eA = [dAs[0]] + [torch.empty_like(dAs[0]) for _ in range(sets - 1)]
    eB = [dBs[0]] + [torch.empty_like(dBs[0]) for _ in range(sets - 1)]
    eC = [dCs[0]] + [torch.empty_like(dCs[0]) for _ in range(sets - 1)]
    in_done = [[torch.cuda.Event() for _ in range(blocks + 1)] for _ in range(sets)]
    out_ready = [[torch.cuda.Event() for _ in range(blocks)] for _ in range(sets)]
    out_done = [[torch.cuda.Event() for _ in range(blocks)] for _ in range(sets)]
    step_done = [torch.cuda.Event() for _ in range(sets)]
    e2e_count = [0]

    def step_e2e():
        if blocks == 1:
            dAs[0].copy_(hostA, non_blocking=True)
            dBs[0].copy_(hostB, non_blocking=True)
            call(0)
            hostC.copy_(dCs[0], non_blocking=True)
            return
        b = e2e_count[0] % sets
        e2e_count[0] += 1
        A_d, B_d, C_d = eA[b], eB[b], eC[b]
        cols = n // blocks
        copy_in.wait_event(step_done[b])  # the products of the step that last used this set have read its A and B
        with torch.cuda.stream(copy_in):
            A_d.copy_(hostA, non_blocking=True)
            in_done[b][blocks].record(copy_in)
            for j in range(blocks):
                B_d[j * cols * ldb:(j + 1) * cols * ldb].copy_(hostB[j * cols * ldb:(j + 1) * cols * ldb], non_blocking=True)
                in_done[b][j].record(copy_in)
        stream.wait_event(in_done[b][blocks])
        for j in range(blocks):
            stream.wait_event(in_done[b][j])
            stream.wait_event(out_done[b][j])  # this block of C has left for the host (the step before last wrote it)
            blas.gemm_ex(ta, tb, m, cols, k, spec["alpha"], A_d.data_ptr(), cuda_type[ab], lda, B_d.data_ptr() + j * cols * ldb * ELEM[ab],
                         cuda_type[ab], ldb, spec["beta"], C_d.data_ptr() + j * cols * ldc * ELEM[ct], cuda_type[ct], ldc, compute,
                         capi.GEMM_DEFAULT_TENSOR_OP)
            out_ready[b][j].record(stream)
            copy_out.wait_event(out_ready[b][j])
            with torch.cuda.stream(copy_out):
                hostC[j * cols * ldc:(j + 1) * cols * ldc].copy_(C_d[j * cols * ldc:(j + 1) * cols * ldc], non_blocking=True)
                out_done[b][j].record(copy_out)
        step_done[b].record(stream)

    with torch.cuda.stream(stream):
        for e in step_done:
            e.record(stream)
        for per_set in out_done:
            for e in per_set:
                e.record(stream)
        for _ in range(2 * sets):
            step_e2e()
        stream.wait_stream(copy_out)
        stream.synchronize()
        e2e_steps = max(3, min(args.steps, 10))
        copy_in.wait_stream(stream)
        copy_out.wait_stream(stream)
        start.record(stream)
        for _ in range(e2e_steps):
            step_e2e()
        stream.wait_stream(copy_out)
        stop.record(stream)
        stream.synchronize()
    e2e_tf = flops * e2e_steps / (start.elapsed_time(stop) * 1e-3) / 1e12

    peaks, peak_kind = measured_peaks()
    bound = spec["bound"]
    if bound == "hbm":
        peak = float(peaks.get("hbm_gbs", FALLBACK_PEAKS["hbm_gbs"]))
        achieved, unit, source = algorithmic_bytes / (kernel_ms * 1e-3) / 1e9, "GB/s", f"{peak_kind}: device copy bandwidth"
    elif bound == "ffma":
        # the fp32 yardstick is measured here: cuBLAS SGEMM (TF32 off) on 4096^3, the FFMA rate NVIDIA's own kernel reaches on this box
        peak, bound = yardstick(torch, "f32"), "tensor"
        achieved, unit, source = flops / (kernel_ms * 1e-3) / 1e12, "TFLOP/s", "measured here: cuBLAS fp32 4096^3 (TF32 off) through torch.matmul, best of 5 (CUDA cores, not tensor cores)"
    elif ab == "s8":
        # the int8 yardstick is measured here: no int8 figure is on record in MEASURED_PEAKS.json
        peak = yardstick(torch, "s8")
        achieved, unit = flops / (kernel_ms * 1e-3) / 1e12, "TFLOP/s"
        source = "measured here: cuBLAS int8 8192^3 through torch._int_mm, best of 10, CUDA events"
    else:
        peak = float(peaks.get("bf16_tflops", FALLBACK_PEAKS["bf16_tflops"]))
        achieved, unit = flops / (kernel_ms * 1e-3) / 1e12, "TFLOP/s"
        source = f"{peak_kind}: cuBLAS bf16 8192^3 burst"
    traffic = None
    traffic_file = ROOT / "profiles" / "traffic.json"
    if traffic_file.exists():
        try:
            traffic = json.loads(traffic_file.read_text()).get(name)
        except Exception:
            traffic = None

    headline = name == "cfg2_f16_tn_8192"
    cpu_tf, cores, cpu_kind, sample = cpu_reference_sample(2048, 3) if headline else (None, None, None, None)
    path_names = {capi.PATH_GEMV: "gemvRowsBulk", capi.PATH_SGEMM: "sgemmKernel", capi.PATH_UMMA: "ummaGemmKernel", capi.PATH_GENERIC: "genericGemmKernel"}
    line = {
        "metric": "gemm_tflops", "value": value_tf, "unit": "TFLOP/s", "n_gpus": 1, "steps": steps_done, "warmup": max(3, args.warmup),
        "ms_per_step": kernel_ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": ab, "data": "synthetic",
        "config": {"workload": name, "call": {"sgemm": "cublasSgemm_v2", "strided": "cublasGemmStridedBatchedEx", "gemmex": "cublasGemmEx"}[spec["call"]],
                   "opA": spec["ta"], "opB": spec["tb"], "m": m, "n": n, "k": k, "batch": batch, "a_b_type": ab, "c_type": ct,
                   "alpha": spec["alpha"], "beta": spec["beta"], "seed": spec["seed"], "distribution": list(spec["dist"]),
                   "l2": (f"{copies} rotating operand sets, {copies * algorithmic_bytes >> 20} MiB > L2" if copies > 1 else
                          f"operands of one step hold {algorithmic_bytes >> 20} MiB > L2") + ", no flush",
                   "timing": "CUDA graph replay of whole passes over the operand sets, at least 32 calls per graph" if use_graph else "back-to-back calls on one stream"},
        "roofline": {"bound": bound, "achieved": achieved, "peak": peak, "unit": unit, "frac": achieved / peak, "traffic": traffic,
                     "peak_source": source, "kernel": path_names.get(path, str(path)), "kernel_ms": kernel_ms,
                     "algorithmic_bytes": algorithmic_bytes, "algorithmic_flop": flops},
        "roofline_sustained": sustained,
        "e2e": {"value": e2e_tf, "unit": "TFLOP/s", "h2d_bytes_per_step": bytes_in, "d2h_bytes_per_step": bytes_out,
                "how": (f"{blocks} column blocks: copy in, cublasGemmEx and copy out overlap on three streams, two sets of device buffers in turn" if blocks > 1 else
                        "copy in, one call, copy out, on one stream")},
        "gpu_launches": launches, "clocks": clocks,
    }
    if cpu_tf is not None:
        line["cpu_baseline"] = {"value": cpu_tf, "unit": "TFLOP/s", "cores": cores, "kind": cpu_kind, "sample": sample}
    print(json.dumps(line), flush=True)
    blas.destroy()


# ---------------------------------------------------------------------------------------------------------------------
# GPU arm, one GPU: the fused attention that follows configuration 4's Q K^T (vkzbAttentionForward)
# ---------------------------------------------------------------------------------------------------------------------

ATTENTION_WORKLOADS = {
    # configuration 4's operands (256 heads of 1024 queries and keys, head dimension 128, f16) with a V of the same shape
    "f4_attention_f16_256x1024x1024x128": dict(ab="f16", heads=256, num_q=1024, num_k=1024, dim=128, mask=0, dist=("normal", 1.0), seed=3, bound="tensor"),
    "f4_attention_f16_256x1024x1024x128_causal": dict(ab="f16", heads=256, num_q=1024, num_k=1024, dim=128, mask=1, dist=("normal", 1.0), seed=3, bound="tensor"),
    "f4_attention_bf16_64x4096x4096x128": dict(ab="bf16", heads=64, num_q=4096, num_k=4096, dim=128, mask=0, dist=("normal", 1.0), seed=3, bound="tensor"),
    # a few heads for profiler captures
    "profile_attention_f16_64x1024x1024x128": dict(ab="f16", heads=64, num_q=1024, num_k=1024, dim=128, mask=0, dist=("normal", 1.0), seed=3, bound="tensor"),
}


def run_attention(args):
    """One step = one vkzbAttentionForward over all heads. FLOPs counted: 4 numQ numK dim per head (half of that under the
    causal mask), the two products only. The check against the fp64 oracle runs on one head, outside the timed region."""
    import numpy as np
    import torch
    from vulkanizer_b200 import capi

    name = args.workload
    spec = ATTENTION_WORKLOADS[name]
    torch.cuda.set_device(0)
    torch.zeros(1, device="cuda")
    heads, num_q, num_k, dim, mask, ab = spec["heads"], spec["num_q"], spec["num_k"], spec["dim"], spec["mask"], spec["ab"]
    scale = dim ** -0.5
    tdt = torch.float16 if ab == "f16" else torch.bfloat16
    cuda_type = capi.CUDA_R_16F if ab == "f16" else capi.CUDA_R_16BF
    count_q, count_k = heads * num_q * dim, heads * num_k * dim
    hostQ = host_operand(torch, spec, count_q, 0)
    hostK = host_operand(torch, spec, count_k, count_q)
    hostV = host_operand(torch, spec, count_k, count_q + count_k)
    hostO = torch.empty(count_q, dtype=tdt).pin_memory()
    algorithmic_bytes = (2 * count_q + 2 * count_k) * 2
    copies = 1 if algorithmic_bytes > 2 * L2_BYTES else int(2 * L2_BYTES // algorithmic_bytes) + 2
    dQ, dK, dV = ([h.cuda() for _ in range(copies)] for h in (hostQ, hostK, hostV))
    dO = [torch.zeros(count_q, dtype=tdt, device="cuda") for _ in range(copies)]
    lib = capi.cublas_library()
    stream = torch.cuda.Stream()
    counter = [0]

    def call(i):
        j = i % copies
        status = capi.attention_forward(stream.cuda_stream, cuda_type, 1, heads, heads, num_q, num_k, dim, mask, scale, dQ[j].data_ptr(), (dim, num_q * dim, 0),
                                        dK[j].data_ptr(), (dim, num_k * dim, 0), dV[j].data_ptr(), (dim, num_k * dim, 0), dO[j].data_ptr(), (dim, num_q * dim, 0))
        assert status == 0, f"vkzbAttentionForward: status {status}"

    def step():
        call(counter[0])
        counter[0] += 1

    flops = 4.0 * heads * num_q * num_k * dim * (0.5 if mask else 1.0)
    with torch.cuda.stream(stream):
        for _ in range(max(3, args.warmup)):
            step()
        stream.synchronize()
    launches0 = int(lib.vkzbLaunchCount())
    sampler = ClockSampler(physical_gpu_index(0))
    time.sleep(0.3)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.time()
    with torch.cuda.stream(stream):
        start.record(stream)
        for _ in range(args.steps):
            step()
        stop.record(stream)
        stream.synchronize()
    t1 = time.time()
    clocks = sampler.stop(t0, t1)
    launches = int(lib.vkzbLaunchCount()) - launches0
    kernel_ms = start.elapsed_time(stop) / args.steps
    value_tf = flops / (kernel_ms * 1e-3) / 1e12
    assert lib.vkzbAttentionStatus() == 0, "a bounded wait in the attention kernel gave up"

    # parity: the last head of the first operand set against the fp64 oracle, with the tolerance of the reference's attention test
    from oracle import pyoracle as orc
    call(0)
    stream.synchronize()
    h = heads - 1
    pick = lambda t, n: t[h * n * dim:(h + 1) * n * dim].float().cpu().numpy().reshape(1, 1, n, dim)
    want, _ = orc.attention_fp64(pick(dQ[0], num_q), pick(dK[0], num_k), pick(dV[0], num_k), scale, mask)
    err = float((np.abs(pick(dO[0], num_q) - want) / (1.0 + np.abs(want))).max())
    tolerance = 6e-3 if ab == "f16" else 4e-2
    assert err <= tolerance, f"attention differs from the fp64 oracle: {err}"

    def step_e2e():
        dQ[0].copy_(hostQ, non_blocking=True)
        dK[0].copy_(hostK, non_blocking=True)
        dV[0].copy_(hostV, non_blocking=True)
        call(0)
        hostO.copy_(dO[0], non_blocking=True)

    with torch.cuda.stream(stream):
        for _ in range(2):
            step_e2e()
        stream.synchronize()
        e2e_steps = max(3, min(args.steps, 10))
        start.record(stream)
        for _ in range(e2e_steps):
            step_e2e()
        stop.record(stream)
        stream.synchronize()
    e2e_tf = flops * e2e_steps / (start.elapsed_time(stop) * 1e-3) / 1e12

    # the host cores on one head of the same problem through the oracle (numpy, fp64)
    t_c0 = time.time()
    orc.attention_fp64(pick(dQ[0], num_q), pick(dK[0], num_k), pick(dV[0], num_k), scale, mask)
    cpu_tf = flops / heads / (time.time() - t_c0) / 1e12

    peaks, peak_kind = measured_peaks()
    peak = float(peaks.get("bf16_tflops", FALLBACK_PEAKS["bf16_tflops"]))
    traffic = None
    traffic_file = ROOT / "profiles" / "traffic.json"
    if traffic_file.exists():
        try:
            traffic = json.loads(traffic_file.read_text()).get(name)
        except Exception:
            traffic = None
    line = {
        "metric": "attention_tflops", "value": value_tf, "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps, "warmup": max(3, args.warmup),
        "ms_per_step": kernel_ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": ab, "data": "synthetic",
        "config": {"workload": name, "call": "vkzbAttentionForward", "heads": heads, "num_q": num_q, "num_k": num_k, "head_dim": dim, "mask": mask,
                   "scale": scale, "seed": spec["seed"], "distribution": list(spec["dist"]),
                   "l2": (f"{copies} rotating operand sets, {copies * algorithmic_bytes >> 20} MiB > L2" if copies > 1 else
                          f"operands of one step hold {algorithmic_bytes >> 20} MiB > L2") + ", no flush",
                   "timing": "back-to-back calls on one stream"},
        "roofline": {"bound": "tensor", "achieved": value_tf, "peak": peak, "unit": "TFLOP/s", "frac": value_tf / peak, "traffic": traffic,
                     "peak_source": f"{peak_kind}: cuBLAS bf16 8192^3 burst", "kernel": "attentionKernel", "kernel_ms": kernel_ms,
                     "algorithmic_bytes": algorithmic_bytes, "algorithmic_flop": flops},
        "parity_checked": {"head": h, "max_error": err, "tolerance": tolerance, "against": "fp64 oracle (oracle/pyoracle.py attention_fp64)"},
        "e2e": {"value": e2e_tf, "unit": "TFLOP/s", "h2d_bytes_per_step": (count_q + 2 * count_k) * 2, "d2h_bytes_per_step": count_q * 2,
                "how": "copy Q, K, V in, one call, copy O out, on one stream"},
        "cpu_baseline": {"value": cpu_tf, "unit": "TFLOP/s", "cores": os.cpu_count(), "kind": "port",
                         "sample": f"one head ({num_q} x {num_k} x {dim}) through the numpy fp64 oracle, BLAS threads as numpy chooses"},
        "gpu_launches": launches, "clocks": clocks,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None, help="one of the names in WORKLOADS or ATTENTION_WORKLOADS (default: the headline configuration)")
    ap.add_argument("--chunk-columns", type=int, default=0, help="sharded run: columns per rank and round of the pipelined gather (default: chosen by rank count)")
    ap.add_argument("--gather", default="auto", choices=["auto", "fused", "pipelined", "hybrid"], help="sharded run: how the column blocks reach every rank")
    ap.add_argument("--timeline", action="store_true", help="sharded run: device time of every round's product and gather of one extra step, on stderr")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference_arm(args)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1 or args.gpus > 1 or args.workload == "cfg5b_bf16_32768_nsharded":
        import bench_multi_gpu
        return bench_multi_gpu.run(args)
    if args.workload in ATTENTION_WORKLOADS:
        return run_attention(args)
    return run_single_gpu(args)


if __name__ == "__main__":
    main()
