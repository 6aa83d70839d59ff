#!/usr/bin/env python
"""Benchmark of the quantized-matmul hot path on B200.

Headline (one JSON line): int8 tensor-op throughput of the fused Q8_0 SwiGLU FFN at the
prefill shape M=512, K=1024, n_ff=3072 (x -> quantize -> gate|up GEMM + SiLU*mul + re-quantize
-> down GEMM).  One step = one FFN pass over one batch of 512 synthetic token rows.
  value     whole-job TOPS with inputs resident in HBM (all ranks; weak scaling: every rank
            runs its own 512-row batch, no collective)
  e2e       the same metric through the host-pointer C ABI call (pinned host x in, host out)
  roofline  the dominant kernel (gate|up tcgen05 GEMM with fused epilogue), timed with CUDA
            events on the launching stream
  cpu_baseline / --impl reference: the CPU oracle port of the reference's AVX2 path, timed on
            this box's host cores
Secondary figures (GEMV GB/s, decode tok/s, Q4_K, the 1-GPU times of the sharded sweep) are carried in
"also" at N=1, each with the CPU oracle's time for the same work beside it.  With N > 1 GPUs the line also
carries "sharded_sweep": BASELINE config 5 (W [32768, 8192] split by row across the ranks, every rank ends
with the whole [M, 32768] result) per M, with each exchange, against the 1-GPU time measured in the same run.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import tempfile
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

M, E, FF = 512, 1024, 3072
OPS_GATE_UP = 2 * M * E * (2 * FF)
OPS_DOWN = 2 * M * FF * E
OPS_STEP = OPS_GATE_UP + OPS_DOWN          # 9.664 G int8-op
METRIC = "Q8_0 fused FFN prefill int8 GEMM throughput (M=512,K=1024,n_ff=3072)"


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"], d["bf16_tflops"], d.get("bf16_tflops_sustained", d["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, 1400.0, "fallback"


class ClockSampler:
    """Polls SM clock and throttle reasons through NVML (read-only) while a region runs."""

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz, self._stop = [], set(), None, threading.Event()
        self._t = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nv = None

    def _run(self):
        nv = self._nv
        names = {nv.nvmlClocksEventReasonHwSlowdown: "hw_slowdown",
                 nv.nvmlClocksEventReasonHwThermalSlowdown: "hw_thermal_slowdown",
                 nv.nvmlClocksEventReasonSwThermalSlowdown: "sw_thermal_slowdown",
                 nv.nvmlClocksEventReasonSwPowerCap: "sw_power_cap"}
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)
                for bit, name in names.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.002)

    def __enter__(self):
        if self._nv is not None:
            self._t = threading.Thread(target=self._run, daemon=True)
            self._t.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._t:
            self._t.join()

    def summary(self):
        return {"sm_mhz": int(statistics.median(self.samples)) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


def ffn_weights_bytes(pkg):
    return (pkg.synth.q8_0_weight(FF, E, seed=0), pkg.synth.q8_0_weight(FF, E, seed=1),
            pkg.synth.q8_0_weight(E, FF, seed=2))


def cpu_ffn_tops(pkg, threads: int, reps: int):
    """The oracle's AVX2 path (quantize, gate, up, SiLU*mul, re-quantize, down per token) on host cores."""
    from oracle import orc
    g, u, d = ffn_weights_bytes(pkg)
    x = pkg.synth.normal((M, E), seed=3)
    orc.ffn_swiglu_q8_0(g, u, d, x[:32], E, FF, orc.SEM_AVX2, threads)  # warm the pool and caches
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        orc.ffn_swiglu_q8_0(g, u, d, x, E, FF, orc.SEM_AVX2, threads)
        times.append(time.perf_counter() - t0)
    return OPS_STEP / statistics.median(times) / 1e12, times


def run_reference(args, rank, world):
    """--impl reference: the reference's CPU implementation of the path (C port of its AVX2
    kernels; the Rust crate cannot be built offline) on all host threads, same config/metric."""
    if rank != 0:
        return
    from __graft_entry__ import load_package
    pkg = load_package()
    threads = args.threads or os.cpu_count() or 1
    from oracle import orc
    g, u, d = ffn_weights_bytes(pkg)
    x = pkg.synth.normal((M, E), seed=3)
    for _ in range(max(args.warmup, 1)):
        orc.ffn_swiglu_q8_0(g, u, d, x[:64], E, FF, orc.SEM_AVX2, threads)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        orc.ffn_swiglu_q8_0(g, u, d, x, E, FF, orc.SEM_AVX2, threads)
    dt = time.perf_counter() - t0
    tops = OPS_STEP * args.steps / dt / 1e12
    line = {"impl": "reference", "metric": METRIC, "value": tops, "unit": "TOPS", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
            "config": {"workload": "configs[1]: Q8_0 prefill GEMM + fused FFN, M=512 K=1024 n_ff=3072",
                       "semantics": "avx2"},
            "cpu_baseline": {"value": tops, "unit": "TOPS", "cores": threads, "kind": "port",
                             "sample": f"{args.steps} full M=512 batches, {threads} threads, row-partitioned GEMVs"},
            "e2e": {"value": tops, "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


_WEIGHTS = {}


def q8_weight_cached(pkg, n, k, seed=0):
    """Synthetic Q8_0 weight bytes, generated once per (shape, seed) in this process."""
    key = (n, k, seed)
    if key not in _WEIGHTS:
        _WEIGHTS[key] = pkg.synth.q8_0_weight(n, k, seed=seed)
    return _WEIGHTS[key]


def cpu_gemv(pkg, n, k, threads, m=1, budget_s=2.0):
    """The oracle's AVX2 GEMV (quantize + row-partitioned matmul, all host threads) on the same shape."""
    from oracle import orc
    wb = q8_weight_cached(pkg, n, k)
    x = pkg.synth.normal((m, k), seed=1)
    orc.q8_forward_batched(wb, x, k, n, orc.SEM_AVX2, threads)
    times, t_all = [], time.perf_counter()
    while len(times) < 3 or (time.perf_counter() - t_all < budget_s and len(times) < 200):
        t0 = time.perf_counter()
        orc.q8_forward_batched(wb, x, k, n, orc.SEM_AVX2, threads)
        times.append(time.perf_counter() - t0)
    t = statistics.median(times)
    algo = n * (k // 32) * 34 + m * (k + (k // 32) * 4) + m * n * 4
    return {"us": t * 1e6, "gbs": algo / t / 1e9, "cores": threads, "kind": "port",
            "sample": f"{len(times)} calls of the C oracle's AVX2 path (quantize + GEMV, {threads} threads, rows split "
                      f"ceil(n/threads) per thread; the reference's default is min(cores, 8) threads), median"}


def gemv_bandwidth(pkg, ctx, torch, stream, n, k, copies, sem, min_ms=250.0, dependent_launch=False):
    """GB/s of the decode GEMV with `copies` distinct weight buffers so every launch streams from HBM.  The timed
    region is at least `min_ms` long (graph replays back to back).  dependent_launch: the GEMVs of the graph are
    launched with programmatic stream serialization, so a GEMV's weight fetch overlaps its predecessor's tail."""
    ctx.set_semantics(sem)
    wb = q8_weight_cached(pkg, n, k)
    ws = [pkg.QuantizedTensor.from_bytes(wb, pkg.GGML_Q8_0, k, n) for _ in range(copies)]
    x = torch.from_numpy(pkg.synth.normal((1, k), seed=1)).cuda()
    q8 = torch.empty(k, dtype=torch.uint8, device="cuda")
    sc = torch.empty(k // 32, dtype=torch.float32, device="cuda")
    out = torch.empty(n, dtype=torch.float32, device="cuda")
    pkg.quantize_q8_0_dev(ctx, x.data_ptr(), 1, k, q8.data_ptr(), sc.data_ptr())

    def burst():
        for w in ws:
            pkg.matmul_q8_0_prequantized_dev(w, q8.data_ptr(), sc.data_ptr(), 1, out.data_ptr())

    for _ in range(3):
        burst()
    stream.synchronize()
    # one launch alone, cold L2 (the weight copy used was last touched `copies` launches ago)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    lat = []
    with torch.cuda.stream(stream):
        for w in ws[:min(copies, 8)]:
            e0.record(stream)
            pkg.matmul_q8_0_prequantized_dev(w, q8.data_ptr(), sc.data_ptr(), 1, out.data_ptr())
            e1.record(stream)
            stream.synchronize()
            lat.append(e0.elapsed_time(e1) * 1e3)
    ctx.set_dependent_launch(dependent_launch)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        burst()
    ctx.set_dependent_launch(False)
    graph.replay()
    stream.synchronize()
    with torch.cuda.stream(stream):
        for _ in range(2):
            graph.replay()
        e0.record(stream)
        for _ in range(4):
            graph.replay()
        e1.record(stream)
    stream.synchronize()
    iters = max(3, int(min_ms / max(e0.elapsed_time(e1) / 4, 1e-3)) + 1)
    with torch.cuda.stream(stream):
        e0.record(stream)
        for _ in range(iters):
            graph.replay()
        e1.record(stream)
    stream.synchronize()
    total_ms = e0.elapsed_time(e1)
    per = total_ms / 1e3 / (iters * copies)
    algo = n * (k // 32) * 34 + k + (k // 32) * 4 + n * 4   # weights + pre-quantized x + y
    for w in ws:
        w.free()
    return {"shape": [n, k], "us_per_gemv": per * 1e6, "gbs": algo / per / 1e9, "algorithmic_bytes": algo,
            "distinct_weight_copies": copies, "launch": "cuda-graph" + (" + dependent launch" if dependent_launch else ""),
            "timed_ms": total_ms, "gemvs_timed": iters * copies, "single_launch_us_median": statistics.median(lat)}


def q4k_bench(pkg, ctx, torch, stream, hbm_peak, iters=10, cpu_threads=0):
    """BASELINE config 3: W [4096, 4096] Q4_K, M in {1, 8, 256}; both reference paths (dequantize-and-matmul,
    Q4_K x Q8_K).  16 distinct weight copies (151 MB > L2) rotate inside one CUDA graph."""
    n = k = 4096
    ctx.set_semantics(pkg.SEM_AVX2)
    ctx.set_stream(stream.cuda_stream)
    wb = pkg.synth.q4_k_weight(n, k, seed=0)
    ws = [pkg.QuantizedTensor.from_bytes(wb, pkg.GGML_Q4_K, k, n) for _ in range(16)]
    res = {}
    for m in (1, 8, 256):
        x = torch.from_numpy(pkg.synth.normal((m, k), seed=1)).cuda()
        out = torch.empty((m, n), dtype=torch.float32, device="cuda")
        for name, fn in (("dequant", pkg.matmul_q4_k_dequant_dev), ("q8k", pkg.matmul_q4_k_q8k_dev),
                         ("q8k_dependent_launch", pkg.matmul_q4_k_q8k_dev)):
            # the last variant launches quantizer and matmul as programmatic dependents: the matmul fetches its first
            # weight chunks while the quantizer runs
            ctx.set_dependent_launch(name == "q8k_dependent_launch")

            def burst():
                for w in ws:
                    fn(w, x.data_ptr(), m, out.data_ptr())
            for _ in range(2):
                burst()
            stream.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                burst()
            graph.replay()
            stream.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            with torch.cuda.stream(stream):
                e0.record(stream)
                for _ in range(iters):
                    graph.replay()
                e1.record(stream)
            stream.synchronize()
            per = e0.elapsed_time(e1) / 1e3 / (iters * len(ws))
            algo = n * (k // 256) * 144 + m * k * 4 + m * n * 4
            ctx.set_dependent_launch(False)
            res[f"{name}_m{m}"] = {"us": per * 1e6, "gbs": algo / per / 1e9, "frac_of_hbm_peak": algo / per / 1e9 / hbm_peak,
                                   "tflops": 2.0 * m * n * k / per / 1e12, "algorithmic_bytes": algo}
    for w in ws:
        w.free()
    if cpu_threads:
        # CPU oracle beside it: Q4_KKernel::forward_prepared (Q8_K activation + vec_dot_q4k_q8k) and
        # QuantizedLinear::forward_dequant, row-partitioned as the reference does; M > 1 = per-row loop,
        # timed on a bounded sample of rows and scaled
        from oracle import orc
        xr = pkg.synth.normal((k,), seed=1)
        t0 = time.perf_counter()
        reps = 0
        while time.perf_counter() - t0 < 1.5 or reps < 2:
            buf = np.zeros(n, np.float32)
            for ith in range(1):
                orc.q4k_forward_prepared(wb, xr, k, n, 0, 1, orc.SEM_AVX2, buf)
            reps += 1
        per_row_q8k = (time.perf_counter() - t0) / reps
        t0 = time.perf_counter()
        orc.q4k_forward_dequant(wb, n, k, xr)
        per_row_deq = time.perf_counter() - t0
        res["cpu_baseline"] = {"q8k_us_per_row": per_row_q8k * 1e6, "dequant_us_per_row": per_row_deq * 1e6, "cores": 1,
                               "kind": "port",
                               "sample": f"{reps} rows through the C oracle's Q4_K x Q8_K path and 1 row through its "
                                         "dequantize-then-dot path, one thread; M rows cost M times this (per-row loop)"}
    return res


FORWARDS = {"session": 0, "text": 1, "text_f32kv": 2, "logits": 3, "logits_f32kv": 4}


def decode_bench(pkg, ctx, cfg, path, batch, n_prompt, n_gen, sem, forward="session", lean=False):
    ctx.set_semantics(sem)
    model = pkg.Qwen3Model.from_file(path)
    s = pkg.Qwen3Session(model, n_prompt + n_gen, batch=batch, forward=FORWARDS[forward])
    prompts = np.stack([pkg.synth.prompt_tokens(cfg["vocab"], n_prompt, seed=1000 + b) for b in range(batch)])
    toks = s.generate(prompts, n_gen)
    res = {"batch": batch, "prompt": n_prompt, "gen": n_gen, "tok_s": batch * n_gen / (s.gen_ms / 1e3),
           "gen_ms": s.gen_ms, "prefill_ms": s.prefill_ms, "first_tokens": [int(t) for t in toks[0, :4]],
           "prefill": "prompt positions as rows through every operator; cache rows bit-identical to the reference's "
                      "token loop (AVX2: eight-lane order on CUDA cores)"}
    if forward == "session" and not lean:
        s.set_prefill(pkg.PREFILL_TOKEN_LOOP)
        s.generate(prompts, 1)
        res["prefill_ms_token_loop"] = s.prefill_ms
        if sem == pkg.SEM_AVX2:
            s.set_prefill(pkg.PREFILL_BATCHED_TENSOR)
            t2 = s.generate(prompts, n_gen)
            res["prefill_ms_tensor_cores"] = s.prefill_ms
            res["tensor_core_prefill_same_tokens"] = bool(np.array_equal(t2, toks))
    s.free()
    model.free()
    return res, toks


def cpu_decode(pkg, cfg, tensors, threads, n_prompt=8, n_gen=6):
    """The oracle's Qwen3Session on host cores for a bounded sample (short prompt, a few generated tokens):
    seconds per step, which is what a token costs the reference's CPU path at batch 1."""
    from oracle import orc
    model = orc.Qwen3(cfg, tensors)
    prompt = pkg.synth.prompt_tokens(cfg["vocab"], n_prompt, seed=1000)
    model.generate(prompt[:2], 1, sem=orc.SEM_AVX2, threads=threads)   # page the weights in, start the pool
    t0 = time.perf_counter()
    model.generate(prompt, n_gen, sem=orc.SEM_AVX2, threads=threads)
    dt = time.perf_counter() - t0
    steps = n_prompt + n_gen - 1
    return {"value": steps / dt, "unit": "tok/s", "cores": threads, "kind": "port",
            "sample": f"{steps} steps ({n_prompt} prompt + {n_gen} generated tokens, positions 0..{steps - 1}) of the C "
                      f"oracle's Qwen3Session, {threads} threads; one sequence (batch B costs B times this)"}


def sharded_sweep(args, pkg, ctx, torch, dist, rank, world, stream, hbm_peak, bf16_peak, ms=(1, 16, 256, 4096),
                  cpu_threads=0):
    """BASELINE config 5: W [32768, 8192] Q8_0 split by row across the ranks, x [M, 8192] replicated, every rank
    ends with the whole [M, 32768] f32 result.  Per M, device times (CUDA events on the context's stream, max
    over ranks): the 1-GPU matmul of the whole weight (every rank runs it alone on its own GPU), the local
    shard, and the shard plus each exchange -- NCCL all-gather + un-shard, fused peer stores, copy-engine peer
    copies overlapped with the matmul.  The results of all exchanges are compared bit for bit with the 1-GPU
    result.  Library defaults: AVX2 semantics, m > 32 on the tensor cores."""
    n, k = 32768, 8192
    ctx.set_semantics(pkg.SEM_AVX2)
    npr = n // world
    s_row, e_row = pkg.sharding.shard_rows(n, world, rank)
    shard_bytes = pkg.synth.q8_0_weight_rows(n, k, seed=0, row_begin=s_row, row_end=e_row)
    if world > 1:
        # the whole weight for the 1-GPU reference: all-gather of the shards' bytes
        mine = torch.from_numpy(shard_bytes).cuda()
        allb = torch.empty(world * mine.numel(), dtype=torch.uint8, device="cuda")
        dist.all_gather_into_tensor(allb, mine)
        full_bytes = allb.cpu().numpy()
        del mine, allb
    else:
        full_bytes = shard_bytes
    w_full = pkg.QuantizedTensor.from_bytes(full_bytes, pkg.GGML_Q8_0, k, n)
    comm = None
    if world > 1:
        def bcast(obj):
            box = [obj]
            dist.broadcast_object_list(box, src=0)
            return box[0]
        comm = pkg.NcclComm(ctx, world, rank, bcast)
    lin = pkg.sharding.ShardedLinear(pkg, shard_bytes, k, n, rank, world, comm=comm) if world > 1 else None
    peer = pkg.sharding.PeerShardedLinear(pkg, shard_bytes, k, n, rank, world, m_max=max(ms)) if world > 1 else None

    def timed(fn, iters):
        with torch.cuda.stream(stream):
            for _ in range(3):
                fn()
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(iters):
                fn()
            e1.record(stream)
            torch.cuda.synchronize()
            ctx.check_status()
            if world > 1:
                dist.barrier()
        t = torch.tensor([e0.elapsed_time(e1) / iters], dtype=torch.float64, device="cuda")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    results = {}
    for m in ms:
        x = torch.from_numpy(pkg.synth.normal((m, k), seed=1)).cuda()
        ref_full = torch.empty((m, n), dtype=torch.float32, device="cuda")
        iters = max(3, min(args.steps, 50 if m <= 256 else 10))
        ops = 2.0 * m * k * n
        r = {"ms_1gpu": timed(lambda: pkg.matmul_q8_0_dev(w_full, x.data_ptr(), m, ref_full.data_ptr()), iters)}
        r["tops_1gpu"] = ops / (r["ms_1gpu"] / 1e3) / 1e12
        r["weight_gbs_1gpu"] = n * (k // 32) * 34 / (r["ms_1gpu"] / 1e3) / 1e9
        r["frac_of_hbm_peak_1gpu"] = r["weight_gbs_1gpu"] / hbm_peak
        r["frac_of_int8_peak_1gpu"] = r["tops_1gpu"] / (2.0 * bf16_peak)
        if world > 1:
            out_local = torch.empty((m, npr), dtype=torch.float32, device="cuda")
            gathered = torch.empty((world, m, npr), dtype=torch.float32, device="cuda")
            out_full = torch.empty((m, n), dtype=torch.float32, device="cuda")
            r["ms_local_shard"] = timed(lambda: lin.forward_dev(x, out_local), iters)
            r["ms_nccl_allgather"] = timed(lambda: lin.forward_dev(x, out_local, gathered, out_full), iters)
            same = {"nccl_allgather": bool(torch.equal(out_full.view(torch.int32), ref_full.view(torch.int32)))}
            for name, mode in (("fused_peer_stores", pkg.EXCHANGE_FUSED_STORES), ("peer_copy_overlapped", pkg.EXCHANGE_PEER_COPY),
                               ("peer_push_overlapped", pkg.EXCHANGE_PEER_PUSH)):
                r["ms_" + name] = timed(lambda: peer.forward_dev(x.data_ptr(), m, mode), iters)
                got = np.empty((m, n), np.float32)
                ctx.d2h(got, peer.out_ptr)
                same[name] = bool(np.array_equal(got.view(np.uint32), ref_full.cpu().numpy().view(np.uint32)))
                if world > 1:
                    dist.barrier()
            best = min(("nccl_allgather", "fused_peer_stores", "peer_copy_overlapped", "peer_push_overlapped"), key=lambda nm: r["ms_" + nm])
            r["best_exchange"] = best
            r["ms_best"] = r["ms_" + best]
            r["speedup_vs_1gpu"] = r["ms_1gpu"] / r["ms_best"]
            r["efficiency_vs_1gpu"] = r["ms_1gpu"] / (world * r["ms_best"])
            r["whole_job_tops"] = ops / (r["ms_best"] / 1e3) / 1e12          # exchange included
            r["frac_of_int8_peak_all_gpus"] = r["whole_job_tops"] / (world * 2.0 * bf16_peak)
            r["per_gpu_weight_gbs"] = npr * (k // 32) * 34 / (r["ms_best"] / 1e3) / 1e9
            r["frac_of_hbm_peak"] = r["per_gpu_weight_gbs"] / hbm_peak
            r["exchange_bytes_in_per_gpu"] = (world - 1) * m * npr * 4
            r["exchange_gbs_in_per_gpu"] = r["exchange_bytes_in_per_gpu"] / (max(r["ms_best"] - r["ms_local_shard"], 1e-6) / 1e3) / 1e9
            r["bits_equal_1gpu_result"] = same
        results[f"M={m}"] = r
    _WEIGHTS[(n, k, 0)] = full_bytes   # the GEMV bandwidth leg and the CPU baseline use the same bytes
    if cpu_threads and rank == 0:
        results["cpu_baseline"] = cpu_gemv(pkg, n, k, cpu_threads)
        results["cpu_baseline"]["what"] = "M=1 (one GEMV of the whole weight); M rows cost M times this (per-row loop)"
    if peer is not None:
        peer.close()
    if comm is not None:
        comm.destroy()
    w_full.free()
    return results


def run_sharded(args, pkg, ctx, torch, dist, rank, world, stream, hbm_peak, bf16_peak):
    results = sharded_sweep(args, pkg, ctx, torch, dist, rank, world, stream, hbm_peak, bf16_peak,
                            cpu_threads=args.threads or os.cpu_count() or 1)
    if rank == 0:
        top = results["M=4096"]
        print(json.dumps({"metric": "sharded Q8_0 GEMM sweep (N=32768,K=8192,M=4096): whole-job int8 throughput, exchange included",
                          "value": top.get("whole_job_tops", top["tops_1gpu"]), "unit": "TOPS",
                          "n_gpus": world, "scaling": "strong", "higher_is_better": True, "dtype": "int8", "data": "synthetic",
                          "config": {"workload": "configs[4]: sharded Q8_0 GEMM sweep", "semantics": "avx2"},
                          "results": results}), flush=True)


GEMV_SHAPES = {"c1_3072x1024": (3072, 1024, 160, True), "logits_151936x1024": (151936, 1024, 4, False),
               "c5_m1_32768x8192": (32768, 8192, 3, False)}


def gemv_suite(pkg, ctx, torch, stream, hbm_peak, sems, cpu_threads):
    """The HBM-bound decode GEMVs (configs[0] shape, the logits shape, the config-5 M=1 shape).  The small
    configs[0] GEMV (3.3 MB, a few microseconds) is timed twice: launches fully serialised, and with
    programmatic dependent launch inside the graph (how the decode step runs it)."""
    res = {}
    for name, (n, k, copies, small) in GEMV_SHAPES.items():
        for sem_name, sem in sems:
            r = gemv_bandwidth(pkg, ctx, torch, stream, n, k, copies, sem)
            r["frac_of_hbm_peak"] = r["gbs"] / hbm_peak
            res[f"{name}_{sem_name}"] = r
            if small:
                r2 = gemv_bandwidth(pkg, ctx, torch, stream, n, k, copies, sem, dependent_launch=True)
                r2["frac_of_hbm_peak"] = r2["gbs"] / hbm_peak
                res[f"{name}_{sem_name}_dependent_launch"] = r2
        if cpu_threads:
            res[f"{name}_cpu_baseline"] = cpu_gemv(pkg, n, k, cpu_threads)
    return res


def run_gemv(args, pkg, ctx, torch, stream, hbm_peak, peak_kind):
    """--workload gemv: one JSON line, `roofline` for the logits GEMV."""
    ctx.set_stream(stream.cuda_stream)
    res = gemv_suite(pkg, ctx, torch, stream, hbm_peak, (("avx2", pkg.SEM_AVX2), ("neon", pkg.SEM_NEON)),
                     args.threads or os.cpu_count() or 1)
    top = res["logits_151936x1024_avx2"]
    print(json.dumps({"metric": "Q8_0 decode GEMV achieved HBM bandwidth (logits shape 151936x1024, M=1)",
                      "value": top["gbs"], "unit": "GB/s", "n_gpus": 1, "higher_is_better": True, "dtype": "int8",
                      "data": "synthetic", "config": {"workload": "decode GEMVs, pre-quantized x, distinct weight copies > L2"},
                      "roofline": {"bound": "hbm", "kernel": "q8_gemv_short_kernel<AVX2,16,1>", "achieved": top["gbs"],
                                   "peak": hbm_peak, "unit": "GB/s", "frac": top["gbs"] / hbm_peak,
                                   "peak_source": f"copy bandwidth, of {peak_kind}",
                                   # dram__bytes_read.sum + dram__bytes_write.sum of one launch in a committed ncu capture
                                   "traffic": 169306000},
                      "results": res}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=50)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--threads", type=int, default=0, help="CPU threads of the reference arm / cpu baseline (0 = all)")
    ap.add_argument("--semantics", default="avx2", choices=["neon", "scalar", "avx2"],
                    help="which instruction-set variant of the reference the device reproduces (avx2 = an x86 host, "
                         "the library default and what the reference arm runs)")
    ap.add_argument("--no-also", action="store_true", help="skip the secondary figures (GEMV, decode)")
    ap.add_argument("--decode-batch", type=int, default=1)
    ap.add_argument("--decode-prompt", type=int, default=512)
    ap.add_argument("--decode-gen", type=int, default=128)
    ap.add_argument("--decode-forward", default="session", choices=sorted(FORWARDS),
                    help="which of the reference's copies of the forward the session reproduces "
                         "(text_f32kv holds at most 512 positions)")
    ap.add_argument("--decode-lean", action="store_true",
                    help="decode workload: skip the token-loop and tensor-core prefill comparisons (short runs under a profiler)")
    ap.add_argument("--workload", default="ffn", choices=["ffn", "sharded", "gemv", "decode", "q4k"],
                    help="ffn: the headline line; sharded: BASELINE config 5 (separate JSON line)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    if args.impl == "reference":
        return run_reference(args, rank, world)

    import torch
    import torch.distributed as dist
    from __graft_entry__ import load_package
    pkg = load_package()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")
    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        import datetime
        # a rank that fails must not leave the others waiting for the default ten minutes
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank), timeout=datetime.timedelta(seconds=180))
    ctx = pkg.context(local_rank)
    sem = {"neon": pkg.SEM_NEON, "scalar": pkg.SEM_SCALAR, "avx2": pkg.SEM_AVX2}[args.semantics]
    ctx.set_semantics(sem)
    stream = torch.cuda.Stream()
    ctx.set_stream(stream.cuda_stream)
    hbm_peak, bf16_peak, bf16_sus, peak_kind = measured_peaks()
    sm_count, l2_bytes, _ = ctx.device_info()
    if args.workload == "q4k":
        # BASELINE config 3 on its own: W [4096, 4096] Q4_K, M in {1, 8, 256}, both reference paths
        if rank == 0:
            res = q4k_bench(pkg, ctx, torch, stream, hbm_peak, iters=max(3, min(args.steps, 10)))
            top = res["q8k_m1"]
            print(json.dumps({"metric": "Q4_K x Q8_K matmul (4096x4096, M=1) achieved bandwidth", "value": top["gbs"],
                              "unit": "GB/s", "n_gpus": 1, "higher_is_better": True, "dtype": "int8", "data": "synthetic",
                              "config": {"workload": "configs[2]: Q4_K 4096x4096, M in {1,8,256}, 16 weight copies > L2"},
                              "roofline": {"bound": "hbm", "kernel": "q8k_quantize_kernel + q4k_q8k_matmul_kernel<AVX2,1>",
                                           "achieved": top["gbs"], "peak": hbm_peak, "unit": "GB/s",
                                           "frac": top["gbs"] / hbm_peak, "peak_source": f"copy bandwidth, of {peak_kind}",
                                           "traffic": None},
                              "results": res}), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return
    if args.workload == "decode":
        # BASELINE config 4 on its own: Qwen3-0.6B-architecture greedy decode (synthetic GGUF, seed 0)
        if rank == 0:
            ctx.set_stream(None)
            cfg = dict(pkg.synth.QWEN3_0_6B)
            path = os.path.join(tempfile.gettempdir(), "rmi_qwen3_0_6b_seed0.gguf")
            if not os.path.exists(path):
                pkg.synth.write_qwen3_gguf(path, cfg, pkg.synth.qwen3_tensors(cfg, 0))
            res, _ = decode_bench(pkg, ctx, cfg, path, args.decode_batch, args.decode_prompt, args.decode_gen, sem,
                                  args.decode_forward, lean=args.decode_lean)
            kv = 28 * (args.decode_prompt + args.decode_gen // 2) * 1024 * 2 * 2
            roof = hbm_peak * 1e9 / (633233408 + args.decode_batch * kv) * args.decode_batch
            print(json.dumps({"metric": "Qwen3-0.6B-architecture greedy decode throughput", "value": res["tok_s"],
                              "unit": "tok/s", "n_gpus": 1, "higher_is_better": True, "dtype": "int8", "data": "synthetic",
                              "config": {"workload": "configs[3]: decode", "batch": args.decode_batch,
                                         "prompt": args.decode_prompt, "gen": args.decode_gen, "semantics": args.semantics,
                                         "forward": args.decode_forward},
                              "roofline": {"bound": "hbm", "achieved": res["tok_s"], "peak": roof, "unit": "tok/s",
                                           "frac": res["tok_s"] / roof,
                                           "peak_source": f"copy bandwidth ({peak_kind}) / bytes per step (weights once + KV per sequence)"},
                              "result": res}), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return
    if args.workload == "gemv":
        if rank == 0:
            run_gemv(args, pkg, ctx, torch, stream, hbm_peak, peak_kind)
        if world > 1:
            dist.destroy_process_group()
        return
    if args.workload == "sharded":
        run_sharded(args, pkg, ctx, torch, dist, rank, world, stream, hbm_peak, bf16_peak)
        if world > 1:
            dist.destroy_process_group()
        return

    # R distinct weight/input/output sets, > L2 in total, rotated every step
    g, u, d = ffn_weights_bytes(pkg)
    set_bytes = (2 * FF * E + E * FF) * (1 + 4 / 32) + 2 * M * E * 4
    R = int(max(4, -(-2 * l2_bytes // set_bytes)))
    sets = []
    for r in range(R):
        wgu = pkg.QuantizedTensor.from_bytes(g, pkg.GGML_Q8_0, E, FF).fuse_vstack(
            pkg.QuantizedTensor.from_bytes(u, pkg.GGML_Q8_0, E, FF))
        wd = pkg.QuantizedTensor.from_bytes(d, pkg.GGML_Q8_0, FF, E)
        x = torch.from_numpy(pkg.synth.normal((M, E), seed=3 + 17 * r + 1000 * rank)).cuda()
        out = torch.empty((M, E), dtype=torch.float32, device="cuda")
        sets.append((wgu, wd, x, out))

    def step(i):
        wgu, wd, x, out = sets[i % R]
        pkg.ffn_swiglu_q8_0_dev(wgu, wd, x.data_ptr(), M, out.data_ptr())

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # The step's kernels (quantizer, gate|up GEMM, down GEMM) run as programmatic dependents
    # (rmi_set_dependent_launch): each sets up its barriers and tensor memory while its predecessor drains.  The same
    # steps without it are timed beside (value_plain_launch).
    ctx.set_dependent_launch(False)
    for i in range(max(args.warmup, R)):   # also builds the tcgen05 weight layout of every set
        step(i)
    barrier()
    p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    n_plain = max(3, min(args.steps, 4 * R))
    p0.record(stream)
    for i in range(n_plain):
        step(i)
    p1.record(stream)
    barrier()
    ms_plain = p0.elapsed_time(p1) / n_plain
    ctx.set_dependent_launch(True)
    for i in range(max(3, args.warmup)):
        step(i)
    barrier()
    launches0 = ctx.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clocks:
        barrier()
        e0.record(stream)
        for i in range(args.steps):
            step(i)
        e1.record(stream)
        barrier()
    launches = ctx.launch_count() - launches0
    ms = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_total = float(ms.item())
    value = world * OPS_STEP * args.steps / (ms_total / 1e3) / 1e12

    # AVX2 semantics: the same steps on the bit-exact CUDA-core kernels (rmi_set_prefill_exact), reported beside
    exact = None
    if sem == pkg.SEM_AVX2:
        ctx.set_prefill_exact(True)
        n_exact = max(3, min(args.steps, 2 * R))
        for i in range(3):
            step(i)
        barrier()
        x0, x1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        x0.record(stream)
        for i in range(n_exact):
            step(i)
        x1.record(stream)
        barrier()
        ctx.set_prefill_exact(False)
        ms_x = x0.elapsed_time(x1) / n_exact
        exact = {"value": OPS_STEP / (ms_x / 1e3) / 1e12, "unit": "TOPS", "ms_per_step": ms_x, "steps": n_exact,
                 "what": "same FFN steps with rmi_set_prefill_exact(1): CUDA-core kernels that reproduce the reference's "
                         "eight-lane AVX2 accumulation bit for bit (per GPU)"}

    # per-kernel timing of the same steps (second pass, events around the tagged launches)
    ksteps = min(args.steps, 2000)
    ctx.prof_enable(True)
    for i in range(ksteps):
        step(i)
    n_k, ms_k = ctx.prof_read("gemm_tc_swiglu")
    n_d, ms_d = ctx.prof_read("gemm_tc")
    ctx.prof_enable(False)
    roofline = None
    int8_peak = 2.0 * bf16_peak   # no int8 figure is measured on this pool: dense int8 = 2 x the measured bf16 peak
    if n_k:
        achieved = OPS_GATE_UP / (ms_k / n_k / 1e3) / 1e12
        roofline = {"bound": "tensor", "kernel": "gemm_tc_kernel<128,SWIGLU_Q8> (gate|up GEMM, fused SiLU*mul + re-quantize)",
                    "achieved": achieved, "peak": int8_peak, "unit": "TFLOP/s", "frac": achieved / int8_peak,
                    "peak_source": f"2 x bf16 {peak_kind} ({bf16_peak} TFLOP/s burst); of {peak_kind}",
                    "frac_of_bf16_peak": achieved / bf16_peak, "avg_kernel_us": ms_k / n_k * 1e3, "launches": n_k,
                    "down_gemm_avg_us": (ms_d / n_d * 1e3) if n_d else None,
                    "down_gemm_tops": (OPS_DOWN / (ms_d / n_d / 1e3) / 1e12) if n_d else None,
                    # dram__bytes_read.sum + dram__bytes_write.sum of one launch of this kernel on this workload in a
                    # committed ncu capture (a constant, not measured by this run); algorithmic bytes 7.65 MB
                    "traffic": 7703552, "traffic_source": "constant from an ncu capture of one launch of this kernel on this workload"}
    else:   # AVX2 semantics keep every M on the CUDA-core kernels
        n_g, ms_g = ctx.prof_read("q8_gemv")
        roofline = {"bound": "tensor", "kernel": "q8_gemv_kernel (CUDA cores; AVX2 semantics)", "achieved": value,
                    "peak": int8_peak, "unit": "TFLOP/s", "frac": value / int8_peak, "traffic": None}

    # end to end through the host-pointer C ABI: every step's x comes from pinned host memory and its result
    # goes back to pinned host memory.  Headline: the pipelined entry point (copies of neighbouring steps overlap
    # the arithmetic); the one-call-per-step entry point is reported beside it.
    e2e_steps = min(args.steps, 304)
    NBUF_H = 4
    hxs = [torch.from_numpy(pkg.synth.normal((M, E), seed=99 + rank + 7 * j)).pin_memory() for j in range(NBUF_H)]
    houts = [torch.empty((M, E), dtype=torch.float32).pin_memory() for _ in range(NBUF_H)]
    lib, C = pkg.lib(), __import__("ctypes")

    def e2e_serial_step(i):
        wgu, wd = sets[i % R][0], sets[i % R][1]
        st = lib.rmi_ffn_swiglu_q8_0(ctx.handle, wgu._h, wd._h, C.c_void_p(hxs[i % NBUF_H].data_ptr()), C.c_size_t(M),
                                     C.c_void_p(houts[i % NBUF_H].data_ptr()))
        if st != 0:
            raise RuntimeError(lib.rmi_last_error().decode())

    def e2e_pipelined(n):
        pkg.ffn_swiglu_q8_0_pipelined([sets[i % R][0] for i in range(n)], [sets[i % R][1] for i in range(n)],
                                      [hxs[i % NBUF_H].data_ptr() for i in range(n)],
                                      [houts[i % NBUF_H].data_ptr() for i in range(n)], M)

    def timed(fn):
        barrier()
        t0 = time.perf_counter()
        fn()
        torch.cuda.synchronize()
        dt = torch.tensor([(time.perf_counter() - t0) * 1e3], dtype=torch.float64, device="cuda")
        barrier()
        if world > 1:
            dist.all_reduce(dt, op=dist.ReduceOp.MAX)
        return float(dt.item())

    for i in range(5):
        e2e_serial_step(i)
    serial_ms = timed(lambda: [e2e_serial_step(i) for i in range(e2e_steps)])
    e2e_pipelined(8)
    e2e_ms_v = timed(lambda: e2e_pipelined(e2e_steps))
    e2e_ms = torch.tensor([e2e_ms_v], dtype=torch.float64, device="cuda")
    e2e = {"value": world * OPS_STEP * e2e_steps / (float(e2e_ms.item()) / 1e3) / 1e12, "unit": "TOPS",
           "h2d_bytes_per_step": M * E * 4, "d2h_bytes_per_step": M * E * 4, "steps": e2e_steps,
           "serial_value": world * OPS_STEP * e2e_steps / (serial_ms / 1e3) / 1e12,
           "api": "rmi_ffn_swiglu_q8_0_pipelined (host pointers, pinned; copies of neighbouring steps overlap the "
                  "arithmetic); serial_value = one rmi_ffn_swiglu_q8_0 call per step"}

    ctx.set_dependent_launch(False)
    line = {"metric": METRIC, "value": value, "unit": "TOPS", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_total / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "int8", "data": "synthetic",
            "config": {"workload": "configs[1]: Q8_0 prefill GEMM + fused FFN, M=512 K=1024 n_ff=3072",
                       "semantics": args.semantics, "l2_hygiene": f"{R} distinct weight/input/output sets "
                       f"({R * set_bytes / 1e6:.0f} MB > L2 {l2_bytes / 1e6:.0f} MB) rotated every step",
                       "int8_ops_per_step": OPS_STEP, "parallelism": f"replicas x{world}, no collective",
                       "launch": "programmatic dependent launch (rmi_set_dependent_launch(1)); value_plain_launch = "
                                 "the same steps launched plainly, this rank"},
            "value_plain_launch": OPS_STEP / (ms_plain / 1e3) / 1e12,
            "roofline": roofline, "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks.summary()}
    if exact is not None:
        line["avx2_bit_exact_cuda_cores"] = exact
    if world > 1:
        # BASELINE config 5 across these GPUs (strong scaling, the one exchange of the path)
        try:
            ctx.set_stream(stream.cuda_stream)
            sweep = sharded_sweep(args, pkg, ctx, torch, dist, rank, world, stream, hbm_peak, bf16_peak)
            line["sharded_sweep"] = {"workload": "configs[4]: W [32768, 8192] Q8_0 split by row across the GPUs, x [M, 8192] "
                                                 "replicated, whole [M, 32768] f32 result on every GPU", "scaling": "strong",
                                     "semantics": "avx2", "n_gpus": world, "results": sweep}
        except Exception as ex:
            line["sharded_sweep"] = {"error": repr(ex)}

    if rank == 0 and world == 1:
        threads = args.threads or os.cpu_count() or 1
        tops, times = cpu_ffn_tops(pkg, threads, reps=3)
        line["cpu_baseline"] = {"value": tops, "unit": "TOPS", "cores": threads, "kind": "port",
                                "sample": f"3 full M=512 batches (median {statistics.median(times) * 1e3:.1f} ms), "
                                          f"AVX2 path of the C oracle, {threads} threads"}
        if not args.no_also:
            also = {}
            try:
                ctx.set_stream(stream.cuda_stream)
                # config 5 on one GPU (the 1-GPU column of the sharded sweep), with the CPU's GEMV beside it
                also["sharded_c5_1gpu"] = sharded_sweep(args, pkg, ctx, torch, dist, 0, 1, stream, hbm_peak, bf16_peak,
                                                        cpu_threads=threads)
            except Exception as ex:   # secondary figures never break the headline line
                also["sharded_error"] = repr(ex)
            try:
                ctx.set_stream(stream.cuda_stream)
                also.update({"gemv_" + k_: v for k_, v in
                             gemv_suite(pkg, ctx, torch, stream, hbm_peak, (("avx2", pkg.SEM_AVX2),), threads).items()})
                also["hbm_peak_gbs"] = hbm_peak
            except Exception as ex:
                also["gemv_error"] = repr(ex)
            try:
                also["q4_k_4096x4096"] = q4k_bench(pkg, ctx, torch, stream, hbm_peak, cpu_threads=threads)
            except Exception as ex:
                also["q4k_error"] = repr(ex)
            try:
                ctx.set_stream(None)
                cfg = dict(pkg.synth.QWEN3_0_6B)
                path = os.path.join(tempfile.gettempdir(), "rmi_qwen3_0_6b_seed0.gguf")
                tensors = pkg.synth.qwen3_tensors(cfg, 0)
                if not os.path.exists(path):
                    pkg.synth.write_qwen3_gguf(path, cfg, tensors)
                for b in (1, 32):
                    res, _ = decode_bench(pkg, ctx, cfg, path, b, 512, 128, pkg.SEM_AVX2)
                    kv = 28 * (512 + 64) * 1024 * 2 * 2
                    res["roofline_tok_s"] = hbm_peak * 1e9 / (633233408 + b * kv) * b
                    res["frac_of_roofline"] = res["tok_s"] / res["roofline_tok_s"]
                    also[f"decode_qwen3_0_6b_b{b}_avx2"] = res
                also["decode_cpu_baseline"] = cpu_decode(pkg, cfg, tensors, threads)
            except Exception as ex:
                also["decode_error"] = repr(ex)
            line["also"] = also
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
