"""Multi-GPU arm of bench.py (benchmark code, not part of the library): the N-sharded large GEMM with its column blocks
gathered over NVLink, and the batch-sharded attention-score product.

Workload cfg5b_bf16_32768_nsharded: D = A^T B with A, B 32768 x 32768 bf16 (normal(0, 1), seed 5), D 32768 x 32768 fp32,
alpha = 1, beta = 0, through cublasLtMatmul. The columns of B and D are dealt to the ranks block-cyclically: column chunk
c (W columns) belongs to rank c mod G, so that the G chunks of one "round" lie side by side in D and ncclAllGather, whose
result layout is rank-major, can gather them in place (send = the rank's own chunk inside the receive region). Rank r
multiplies its chunk of round j on the compute stream and gathers round j on a second stream while round j + 1 is being
multiplied; A (2 GiB) is replicated, every rank ends with the whole of D. This is the partitioning of k0zi/Vulkanizer's
`partOf(g, rows=false, first, count)` (src/cublas/cublas.cpp:542-546) applied across GPUs, with the exchange step its
libnccl surface provides (src/nccl/nccl.cpp:691-695). Strong scaling: the total work is fixed.

Two ways of getting every rank's columns everywhere are built. "Pipelined" (what runs by default): the block-cyclic,
chunk-pipelined products + ncclAllGather described above. "Fused" (--gather fused): each rank multiplies its column
block with cublasLtMatmul calls whose epilogue stores every finished tile not only to its own D but, through peer-mapped
addresses (vkzbNcclExchangeBuffer + vkzbSetOutputMirrors), to the other ranks' D as well, so the NVLink traffic is spread
over the whole product and nothing is left to gather; barriers of libnccl.so.2 order the ranks around the step. It measures
slower at every rank count (the remote stores hold up the epilogue: 28.1 / 17.3 / 9.1 ms at 2 / 4 / 8 GPUs against
26.9 / 14.5 / 8.3), and is kept as the form in which one kernel does the product and the exchange.

Operands are the seeded synthetic ones of vulkanizer_b200/synth.py (seed 5; element i of A^T's storage is value i of the
stream, element i of B's value m * k + i), made on the GPU by the torch form of that generator. After the timed region every
rank checks a sample of D (rows across the matrix, columns from EVERY rank's block) against the fp64 oracle on operands
regenerated on the host with the numpy form; the bench line carries the result as `parity_checked`. Every line for more than
one GPU also carries `scaling_baseline`: the time of the same whole product on rank 0 alone, measured in the same run.

torch.distributed (gloo) is only the plumbing: it carries the 128-byte communicator id, the barrier around the timed region and
the maximum over the ranks' device times. All GPU work goes through this repository's libcublasLt.so.12 and libnccl.so.2.
"""
from __future__ import annotations

import json
import os
import time

import numpy as np


def round_widths(n: int, ranks: int, forced: int = 0):
    if forced:
        assert (n // ranks) % forced == 0 and forced % 256 == 0, "--chunk-columns must be a multiple of 256 that divides a rank's share"
        return [forced] * (n // ranks // forced)
    return default_round_widths(n, ranks)


def default_round_widths(n: int, ranks: int):
    """Chunk widths (columns per rank) of the successive rounds: uniform, 1024 columns where the share allows four rounds.
    1024 columns are 512 tile pairs of 256 x 256, 6.9 waves over 74 CTA pairs, so almost no SM idles at the end of a
    chunk; and with equal chunks the gather of round j always hides behind the product of round j + 1. Only the last round's
    gather is exposed. (Rounds that shrink towards the end were measured slower, at 8 ranks, where a wide round's gather
    outlasts the narrower product after it, and at 4 ranks, where the gather takes under half a product's time: 14.5 ms with
    equal rounds, 14.8 - 15.0 with the last round cut into halves, 14.6 into a half and two quarters.)"""
    per_rank = n // ranks
    assert n % ranks == 0 and per_rank % 256 == 0, "the column count must be a multiple of 256 x ranks"
    if ranks == 1:
        return [min(2048, per_rank)] * (per_rank // min(2048, per_rank))
    width = 1024 if ranks < 8 else 512  # 8 GPUs: the link is busy most of the step, and 512 measured 4 % faster than 1024
    while width > 256 and (per_rank % width or per_rank // width < 4):
        width //= 2
    return [width] * (per_rank // width)


def column_chunks(n: int, ranks: int, widths=None):
    """Rounds of `ranks` chunks side by side: [(round, width, first column of the round, [first column of rank r's chunk])].
    Chunk c of a round belongs to rank c, so the round's columns lie in rank order, the layout ncclAllGather produces."""
    widths = widths or round_widths(n, ranks)
    assert sum(widths) * ranks == n, "the rounds must cover every column exactly once"
    rounds, first = [], 0
    for j, w in enumerate(widths):
        rounds.append((j, w, first, [first + r * w for r in range(ranks)]))
        first += ranks * w
    return rounds


def shard(units: int, ranks: int, rank: int):
    """First unit and number of units of `rank` when `units` independent units are dealt to `ranks` ranks in contiguous shares
    that differ by at most one (the shape of k0zi/Vulkanizer's partOf, src/cublas/cublas.cpp:542-546)."""
    first = units * rank // ranks
    return first, units * (rank + 1) // ranks - first


def run_batch_sharded(args):
    """The batched attention-score product (256 entries of 1024 x 1024 x 128, fp16 in, fp32 out) with its batch entries dealt
    to the ranks: entries [r * 256 / G, (r + 1) * 256 / G) on rank r, operands resident per shard, no data-path collective
    (k0zi/Vulkanizer cuts batches the same way, src/cublas/cublas.cpp:542-546). Time = common start to the last rank done."""
    import torch
    import torch.distributed as dist

    from bench import WORKLOADS, ClockSampler, measured_peaks, physical_gpu_index, FALLBACK_PEAKS, host_operand
    from vulkanizer_b200 import capi

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29511")
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.cuda.set_device(local)
    torch.zeros(1, device="cuda")
    name = "cfg4_f16_tn_batched_qk"
    spec = WORKLOADS[name]
    m, n, k, batch = spec["m"], spec["n"], spec["k"], spec["batch"]
    first, count = shard(batch, world, rank)
    sA, sB, sC = k * m, k * n, m * n
    # the rank's own entries of the same seeded operands every rank count would produce
    hostA = host_operand(torch, spec, sA * count, first * sA)
    hostB = host_operand(torch, spec, sB * count, batch * sA + first * sB)
    hostC = torch.empty(sC * count, dtype=torch.float32).pin_memory()
    copies = max(2, int(2 * (126 << 20) // max(1, (sA + sB) * 2 * count + sC * 4 * count)) + 2)  # more than L2 between reuses
    dAs = [hostA.cuda() for _ in range(copies)]
    dBs = [hostB.cuda() for _ in range(copies)]
    dCs = [torch.zeros(sC * count, dtype=torch.float32, device="cuda") for _ in range(copies)]
    blas = capi.Cublas()
    stream = torch.cuda.Stream()
    blas.set_stream(stream.cuda_stream)

    def call(i):
        blas.gemm_strided_batched_ex(capi.OP_T, capi.OP_N, m, n, k, spec["alpha"], dAs[i % copies].data_ptr(), capi.CUDA_R_16F, k, sA,
                                     dBs[i % copies].data_ptr(), capi.CUDA_R_16F, k, sB, spec["beta"], dCs[i % copies].data_ptr(),
                                     capi.CUDA_R_32F, m, sC, count, capi.COMPUTE_32F)

    warmup = max(3, args.warmup)
    with torch.cuda.stream(stream):
        for i in range(warmup):
            call(i)
        stream.synchronize()
    launches0 = blas.launch_count()
    sampler = ClockSampler(physical_gpu_index(local))
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    dist.barrier()
    torch.cuda.synchronize()
    t0 = time.time()
    with torch.cuda.stream(stream):
        start.record(stream)
        for i in range(args.steps):
            call(i)
        stop.record(stream)
        stream.synchronize()
    dist.barrier()
    t1 = time.time()
    clocks = sampler.stop(t0, t1)
    ms = torch.tensor([start.elapsed_time(stop)], dtype=torch.float64)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    launches = blas.launch_count() - launches0
    assert blas.device_status() == 0

    def step_e2e():
        dAs[0].copy_(hostA, non_blocking=True)
        dBs[0].copy_(hostB, non_blocking=True)
        call(0)
        hostC.copy_(dCs[0], non_blocking=True)

    e2e_steps = max(3, min(args.steps, 10))
    with torch.cuda.stream(stream):
        step_e2e()
        stream.synchronize()
        dist.barrier()
        start.record(stream)
        for _ in range(e2e_steps):
            step_e2e()
        stop.record(stream)
        stream.synchronize()
    e2e_ms = torch.tensor([start.elapsed_time(stop)], dtype=torch.float64)
    dist.all_reduce(e2e_ms, op=dist.ReduceOp.MAX)
    if rank == 0:
        peaks, kind = measured_peaks()
        flops = 2.0 * m * n * k * batch
        per_step_ms = float(ms.item()) / args.steps
        algorithmic = (sA + sB) * 2 * batch + sC * 4 * batch
        peak = float(peaks.get("hbm_gbs", FALLBACK_PEAKS["hbm_gbs"]))
        achieved = algorithmic / world / (per_step_ms * 1e-3) / 1e9  # per GPU: each shard is bound by its own HBM
        line = {
            "metric": "gemm_tflops", "value": flops / (per_step_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": warmup, "ms_per_step": per_step_ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16",
            "data": "synthetic",
            "config": {"workload": name, "call": "cublasGemmStridedBatchedEx", "opA": "T", "opB": "N", "m": m, "n": n, "k": k, "batch": batch,
                       "a_b_type": "f16", "c_type": "f32", "alpha": spec["alpha"], "beta": 0.0, "seed": spec["seed"],
                       "parallelism": f"batch-sharded x{world}", "entries_per_rank": count, "collective": "none",
                       "l2": f"{copies} rotating operand sets per rank, no flush", "timing": "back-to-back calls, common start, max over ranks"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "traffic": None,
                         "peak_source": f"{kind}: device copy bandwidth, per GPU", "kernel": "ummaGemmKernel", "kernel_ms": per_step_ms,
                         "algorithmic_bytes": algorithmic // world},
            "e2e": {"value": flops * e2e_steps / (float(e2e_ms.item()) * 1e-3) / 1e12, "unit": "TFLOP/s",
                    "h2d_bytes_per_step": (sA + sB) * 2 * batch, "d2h_bytes_per_step": sC * 4 * batch},
            "gpu_launches": launches * world, "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    blas.destroy()
    dist.barrier()
    dist.destroy_process_group()


def run(args):
    if args.workload == "cfg4_f16_tn_batched_qk":
        return run_batch_sharded(args)
    import torch
    import torch.distributed as dist

    from bench import ClockSampler, measured_peaks, physical_gpu_index, FALLBACK_PEAKS
    from vulkanizer_b200 import capi

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29511")
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.cuda.set_device(local)
    torch.zeros(1, device="cuda")

    from vulkanizer_b200 import synth

    size = 32768
    m = n = k = size
    # fused: products whose tiles go straight to every rank's D; pipelined: chunked products + ncclAllGather.
    # Measured, 32768^3: 2 GPUs 28.1 ms fused / 26.9 pipelined, 4 GPUs 17.3 / 14.5, 8 GPUs 9.1 / 8.3. The
    # mirrored bulk stores push back into the epilogue (every tile waits for seven or three or one remote copies of itself),
    # while a gather behind the next round's product costs the product nothing; so the pipelined form is what runs unless
    # the fused one is asked for.
    fused = world > 1 and args.gather == "fused"
    # hybrid: pipelined, except that the last round's product stores its tiles to every rank itself, so that no gather is left
    # over when the last product ends (the price: that one product's epilogue waits for the remote copies)
    hybrid = world > 1 and args.gather == "hybrid"
    # (fused: 2048 columns per call. One call over a rank's whole share ran a quarter slower at 2 GPUs: over tens of
    # milliseconds the CTAs of one persistent kernel drift apart along k and stop finding each other's operand slices in L2.)
    rounds = column_chunks(n, world, round_widths(n, world, getattr(args, "chunk_columns", 0)))
    if fused:
        per_rank, w = n // world, min(2048, n // world)
        rounds = [(j, w, None, [r * per_rank + j * w for r in range(world)]) for j in range(per_rank // w)]
    mine_cols = sum(w for _, w, _, _ in rounds)  # columns this rank computes

    # the communicator id travels through the process group
    box = [capi.NcclComm.unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    comm = capi.NcclComm(world, rank, box[0])

    # Operands, seed 5: A^T's storage (k x m, lda = k) holds values 0 .. m k - 1 of the stream, column j of B values
    # m k + j k .. of it. A is identical on every rank: each makes its share and the shares are gathered through this
    # repository's libnccl; of B a rank makes only the columns it multiplies.
    A = torch.empty(m * k, dtype=torch.bfloat16, device="cuda")
    a_first, a_count = shard(m, world, rank)
    assert m % world == 0
    synth.fill_normal_torch(torch, A[a_first * k:(a_first + a_count) * k], 5, 1.0, first=a_first * k)
    if world > 1:
        comm.all_gather(A.data_ptr() + 2 * a_first * k, A.data_ptr(), a_count * k, "bfloat16", 0)
        torch.cuda.synchronize()
    Bmine = torch.empty(mine_cols * k, dtype=torch.bfloat16, device="cuda")  # the rank's chunks, one after another
    b_offset = []  # element offset of round j's chunk inside Bmine
    off = 0
    for j, w, _, firsts in rounds:
        b_offset.append(off)
        synth.fill_normal_torch(torch, Bmine[off:off + w * k], 5, 1.0, first=m * k + firsts[rank] * k)
        off += w * k
    D = torch.zeros(m * n, dtype=torch.float32, device="cuda")  # column-major m x n, ldd = m: 4 GiB at full size

    lt = capi.CublasLt()
    compute, gather = torch.cuda.Stream(), torch.cuda.Stream()
    bf16, f32 = capi.CUDA_R_16BF, capi.CUDA_R_32F
    events = [torch.cuda.Event() for _ in rounds]

    mirrors = []
    if fused or hybrid:
        peers = comm.exchange_buffer(D.data_ptr())
        mirrors = [peers[p] for p in range(world) if p != rank]
    if fused:
        lt.set_output_mirrors(D.data_ptr(), D.numel() * 4, mirrors)

    def step():
        if fused:
            comm.barrier(compute.cuda_stream)  # nobody still reads the D this step overwrites
        for j, w, round_first, firsts in rounds:
            mine = D.data_ptr() + 4 * firsts[rank] * m
            stored_everywhere = hybrid and j == len(rounds) - 1
            if stored_everywhere:
                lt.set_output_mirrors(D.data_ptr(), D.numel() * 4, mirrors)
            lt.matmul(capi.OP_T, capi.OP_N, m, w, k, 1.0, A.data_ptr(), bf16, k, Bmine.data_ptr() + 2 * b_offset[j], bf16, k, 0.0,
                      mine, f32, m, mine, f32, m, stream=compute.cuda_stream)
            if stored_everywhere:
                lt.set_output_mirrors(0, 0, [])
            elif world > 1 and not fused:
                events[j].record(compute)
                gather.wait_event(events[j])
                comm.all_gather(mine, D.data_ptr() + 4 * round_first * m, w * m, "float32", gather.cuda_stream)
        if world > 1 and not fused:
            compute.wait_stream(gather)  # the step ends when every rank's columns have arrived
        if fused or hybrid:
            # every rank's (last) product is finished, so every tile it stored has landed here; behind the gathers, because a
            # communicator's operations run one after another, whatever stream they were given
            comm.barrier(compute.cuda_stream)

    for _ in range(max(3, args.warmup)):
        step()
    torch.cuda.synchronize()
    assert lt.last_path() == capi.PATH_UMMA
    launches0 = lt.launch_count()
    sampler = ClockSampler(physical_gpu_index(local)) if rank == 0 else None
    dist.barrier()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.time()
    start.record(compute)
    for _ in range(args.steps):
        step()
    stop.record(compute)
    torch.cuda.synchronize()
    dist.barrier()
    t1 = time.time()
    ms = torch.tensor([start.elapsed_time(stop)], dtype=torch.float64)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    total_ms = float(ms.item())
    clocks = sampler.stop(t0, t1) if sampler else None
    launches = lt.launch_count() - launches0
    assert comm.async_error() == 0, "a device-side barrier of the gather gave up"

    if getattr(args, "timeline", False) and world > 1 and not fused:
        # one more step with an event around every round's product and gather: where the step's time goes (rank 0, stderr)
        marks = {"g0": [], "g1": [], "c0": [], "c1": []}
        dist.barrier()
        torch.cuda.synchronize()
        origin = torch.cuda.Event(enable_timing=True)
        origin.record(compute)
        gather.wait_event(origin)
        for j, w, round_first, firsts in rounds:
            mine = D.data_ptr() + 4 * firsts[rank] * m
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
            ev[0].record(compute)
            lt.matmul(capi.OP_T, capi.OP_N, m, w, k, 1.0, A.data_ptr(), bf16, k, Bmine.data_ptr() + 2 * b_offset[j], bf16, k, 0.0, mine, f32, m, mine, f32, m,
                      stream=compute.cuda_stream)
            ev[1].record(compute)
            gather.wait_event(ev[1])
            ev[2].record(gather)
            comm.all_gather(mine, D.data_ptr() + 4 * round_first * m, w * m, "float32", gather.cuda_stream)
            ev[3].record(gather)
            for key, e in zip(("c0", "c1", "g0", "g1"), ev):
                marks[key].append(e)
        compute.wait_stream(gather)
        torch.cuda.synchronize()
        if rank == 0:
            import sys
            rows_t = [{"round": j, "product_ms": [round(origin.elapsed_time(marks["c0"][j]), 3), round(origin.elapsed_time(marks["c1"][j]), 3)],
                       "gather_ms": [round(origin.elapsed_time(marks["g0"][j]), 3), round(origin.elapsed_time(marks["g1"][j]), 3)]} for j in range(len(rounds))]
            print(json.dumps({"timeline": rows_t}), file=sys.stderr, flush=True)

    # Parity, outside the timed region: a sample of D on EVERY rank (each holds all of D after the step) against the fp64
    # oracle, with operands regenerated on the host by the numpy form of the generator: rows spread over the matrix, and
    # from every rank's column block its first and its last column.
    from oracle import pyoracle as orc
    rows = sorted(set(range(rank * 131 % 997, m, 997)) | {m - 1})
    cols = sorted({c for _, w, _, firsts in (rounds[0], rounds[-1]) for q in range(world) for c in (firsts[q], firsts[q] + w - 1)})
    a_rows = np.concatenate([orc.to_storage(synth.normal(5, k, 1.0, first=i * k), "bf16") for i in rows])   # row i of op(A): k values
    b_cols = np.concatenate([orc.to_storage(synth.normal(5, k, 1.0, first=m * k + j * k), "bf16") for j in cols])
    want = orc.dots_fp64(True, False, k, a_rows, "bf16", k, b_cols, "bf16", k, list(range(len(rows))), list(range(len(cols))))
    got = D.view(n, m)[torch.tensor(cols, device="cuda")][:, torch.tensor(rows, device="cuda")].T.cpu().numpy().astype(np.float64)
    rel = float(np.max(np.abs(got - want) / np.maximum(1.0, np.abs(want))))
    worst = torch.tensor([rel], dtype=torch.float64)
    dist.all_reduce(worst, op=dist.ReduceOp.MAX)
    parity = {"rows": len(rows), "cols": len(cols), "ranks_checked": world, "max_rel": float(worst.item()), "tolerance": 1e-2,
              "oracle": "oracle.pyoracle.dots_fp64 on operands regenerated by vulkanizer_b200.synth (numpy)"}
    assert parity["max_rel"] <= parity["tolerance"], f"the gathered result differs from the oracle: {parity}"

    # The same whole product on rank 0 alone, in the same run, as the denominator of the scaling efficiency: 32768 columns in
    # calls of 2048, B made 2048 columns at a time into a buffer that the timed calls then reuse (its content is irrelevant
    # to the time; A and D are the ones above).
    baseline_ms = None
    if world > 1:
        if rank == 0:
            Bblock = torch.empty(2048 * k, dtype=torch.bfloat16, device="cuda")
            synth.fill_normal_torch(torch, Bblock, 5, 1.0, first=m * k)
            lt.set_output_mirrors(0, 0, [])

            def alone():
                for c in range(0, n, 2048):
                    lt.matmul(capi.OP_T, capi.OP_N, m, 2048, k, 1.0, A.data_ptr(), bf16, k, Bblock.data_ptr(), bf16, k, 0.0, D.data_ptr() + 4 * c * m, f32, m,
                              D.data_ptr() + 4 * c * m, f32, m, stream=compute.cuda_stream)

            alone()
            torch.cuda.synchronize()
            start.record(compute)
            for _ in range(3):
                alone()
            stop.record(compute)
            torch.cuda.synchronize()
            baseline_ms = start.elapsed_time(stop) / 3
            if fused:
                lt.set_output_mirrors(D.data_ptr(), D.numel() * 4, [peers[p] for p in range(world) if p != rank])
        dist.barrier()

    # end to end: the rank's inputs come from pinned host memory, its own columns of D go back
    hostA = torch.empty(m * k, dtype=torch.bfloat16).pin_memory()
    hostB = torch.empty(Bmine.numel(), dtype=torch.bfloat16).pin_memory()
    hostD = torch.empty(mine_cols * m, dtype=torch.float32).pin_memory()
    hostA.copy_(A)
    hostB.copy_(Bmine)
    e2e_steps = 2

    def step_e2e():
        with torch.cuda.stream(compute):
            A.copy_(hostA, non_blocking=True)
            Bmine.copy_(hostB, non_blocking=True)
        step()
        with torch.cuda.stream(compute):
            for j, w, _, firsts in rounds:
                hostD[b_offset[j] // k * m:(b_offset[j] // k + w) * m].copy_(D[firsts[rank] * m:(firsts[rank] + w) * m], non_blocking=True)

    step_e2e()
    torch.cuda.synchronize()
    dist.barrier()
    start.record(compute)
    for _ in range(e2e_steps):
        step_e2e()
    stop.record(compute)
    torch.cuda.synchronize()
    e2e_ms = torch.tensor([start.elapsed_time(stop)], dtype=torch.float64)
    dist.all_reduce(e2e_ms, op=dist.ReduceOp.MAX)

    flops = 2.0 * m * n * k
    if rank == 0:
        peaks, peak_kind = measured_peaks()
        peak = float(peaks.get("bf16_tflops_sustained", FALLBACK_PEAKS["bf16_tflops_sustained"])) * world
        value = flops * args.steps / (total_ms * 1e-3) / 1e12
        gathered_bytes = (world - 1) * (n // world) * m * 4
        line = {
            "metric": "gemm_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup),
            "ms_per_step": total_ms / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": {"workload": "cfg5b_bf16_32768_nsharded", "call": "cublasLtMatmul with output mirrors (tiles stored to every rank over NVLink)" if fused else "cublasLtMatmul + ncclAllGather", "opA": "T", "opB": "N", "m": m, "n": n,
                       "k": k, "a_b_type": "bf16", "c_type": "f32", "alpha": 1, "beta": 0, "seed": 5, "parallelism": f"n-sharded x{world}", "gather": "fused into the GEMM epilogue" if fused else ("none" if world == 1 else "ncclAllGather, chunk-pipelined" + ("; the last round stored to every rank by the GEMM epilogue" if hybrid else "")),
                       "chunk_columns": [w for _, w, _, _ in rounds], "rounds": len(rounds),
                       "l2": "operands of one step hold 8 GiB > L2, no flush", "timing": "CUDA events on the compute stream, maximum over ranks"},
            "roofline": {"bound": "tensor", "achieved": value, "peak": peak, "unit": "TFLOP/s", "frac": value / peak, "traffic": None,
                         "peak_source": f"{peak_kind}: cuBLAS bf16 sustained x {world} GPUs (the step is a long loop of GEMMs)",
                         "kernel": "ummaGemmKernel<256>", "nvlink_bytes_in_per_gpu_per_step": gathered_bytes,
                         "nvlink_floor_ms": gathered_bytes / 770e9 * 1e3},
            "e2e": {"value": flops * e2e_steps / (float(e2e_ms.item()) * 1e-3) / 1e12, "unit": "TFLOP/s",
                    "h2d_bytes_per_step": (hostA.numel() + hostB.numel()) * 2 * world, "d2h_bytes_per_step": hostD.numel() * 4 * world},
            "gpu_launches": launches * world, "clocks": clocks, "parity_checked": parity,
        }
        if baseline_ms:
            line["scaling_baseline"] = {"workload": "the same 32768^3 product on rank 0 alone, 3 steps, this run", "ms_per_step_1gpu": baseline_ms,
                                        "efficiency": baseline_ms / (world * total_ms / args.steps)}
        print(json.dumps(line), flush=True)
    if fused:
        lt.set_output_mirrors(0, 0, [])
    torch.cuda.synchronize()
    dist.barrier()
    comm.destroy()
    lt.destroy()
    dist.barrier()
    dist.destroy_process_group()
