#!/usr/bin/env python
"""bench.py -- headline benchmark of the B200 back end for SimpLang's tensor hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--size S]

Metric: int8 GEMM throughput (TOPS = 2*M*N*K / t / 1e12) of `tensor_matmul` on
u8[M,K] x s8[K,N] -> i32[M,N], M = N = K = 8192, seeded uniform inputs -- the upper end of the
reference's "INT8 tensor_matmul" sweep and the largest single-GPU cube the metric is quoted on.
A step is one GEMM over device-resident operands (384 MB touched per step, larger than the 126 MB
L2, so no flush is needed between steps).  At N > 1 the columns of B are sharded over the ranks
(N/R columns each, A replicated) and the shards of C are gathered into every rank's row-major C by the
GEMM epilogue itself (stores to peer memory over NVLink): total work is fixed, so scaling is "strong".
`without_gather` times the same shards with C left column-sharded, `link` relates the step to the NVLink floor.

The second half of the metric, LLaMA decode tokens/s, is the `decode` record of the same line: the f32 110M
model on one GPU and the W4 3B model tensor-parallel over all ranks (16 prompt tokens + greedy tokens, random-init
weights), device-timed and wall-clock through simp_llama_generate, each with its HBM roofline and an in-run check
(a second run gives the same tokens; the tensor-parallel run gives the tokens of the single-GPU run).

Prints ONE JSON line (rank 0).  `value` is the device-timed throughput (CUDA events on the stream the
kernel runs on, max over ranks); `e2e` is the same metric through the host-pointer entry point
(simp_host_tensor_matmul_i8: pinned host operands in, host result out, copies inside the timed
region); `roofline` reports the tensor-core kernel against the calibrated int8 peak; `cpu_baseline`
is the reference's own OpenMP VNNI kernel timed on this machine's host cores.

`--impl reference` times only the CPU side (the reference has no GPU code): its VNNI kernel on the same 8192^3
problem per step (a slab of rows per step when --steps would make that run too long) on all host cores, and the CPU
restatement of the two decode models on a bounded number of tokens.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

NOMINAL_INT8_TOPS = 4500.0  # B200 dense int8, vendor figure
# dram__bytes_read.sum + dram__bytes_write.sum per launch.  4096^3 is the ncu capture summarised in
# profiles/gemm_i8_tcgen05_2cta_8192.md; 8192^3 is too large to capture under the profiling size rule and is
# scaled from it by the units processed (reads x4, plus the full 256 MB result, which no longer stays in L2).
NCU_TRAFFIC_BYTES = {4096: 52_200_000, 8192: 393_000_000}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock, power and throttle reasons through NVML (read-only) while the timed region runs."""

    def __init__(self, device_index, period_s=0.01):
        self.idx = device_index
        self.period = period_s
        self.samples = []
        self._stop = False
        self._thread = None
        self._nvml = None

    def start(self):
        import threading
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nvml = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(self.idx)
            self._max = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nvml = None
            return
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()

    def _run(self):
        n = self._nvml
        while not self._stop:
            try:
                sm = n.nvmlDeviceGetClockInfo(self._h, n.NVML_CLOCK_SM)
                pw = n.nvmlDeviceGetPowerUsage(self._h) / 1000.0
                rs = n.nvmlDeviceGetCurrentClocksEventReasons(self._h)
                self.samples.append((sm, pw, rs))
            except Exception:
                pass
            time.sleep(self.period)

    def stop(self):
        if self._nvml is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["NVML unavailable"]}
        self._stop = True
        self._thread.join(timeout=2)
        n = self._nvml
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": float(self._max), "reasons": ["no samples"]}
        names = {"hw_slowdown": n.nvmlClocksEventReasonHwSlowdown,
                 "hw_thermal_slowdown": n.nvmlClocksEventReasonHwThermalSlowdown,
                 "sw_thermal_slowdown": n.nvmlClocksEventReasonSwThermalSlowdown,
                 "sw_power_cap": n.nvmlClocksEventReasonSwPowerCap}
        power = [p for _, p, _ in self.samples]
        thr = (max(power) + min(power)) / 2
        loaded = [s for s in self.samples if s[1] >= thr] or self.samples
        reasons = sorted(k for k, bit in names.items() if any(r & bit for _, _, r in loaded))
        return {"sm_mhz": statistics.median(s for s, _, _ in loaded), "sm_max_mhz": float(self._max),
                "power_w_max": max(power), "samples": len(self.samples), "samples_under_load": len(loaded),
                "reasons": reasons}


def gen_inputs(M, K, N, seed_a=1, seed_b=2, a_unsigned=True):
    rng_a, rng_b = np.random.default_rng(seed_a), np.random.default_rng(seed_b)
    if a_unsigned:
        A = rng_a.integers(0, 256, (M, K), dtype=np.uint8)
    else:
        A = rng_a.integers(-128, 128, (M, K), dtype=np.int8)
    B = rng_b.integers(-128, 128, (K, N), dtype=np.int8)
    return A, B


# --------------------------------------------------------------------------------------------- CPU legs
def cpu_reference_gemm(n, repeats, warmup, rows=None):
    """Times the reference's own OpenMP VNNI GEMM (oracle/_ref, compiled from the reference checkout;
    s8 x s8 with B pre-transposed) on all host cores: `vnni_matmul_multicore<n>` for the whole n^3 problem, or
    -- `rows` given -- the reference's non-square VNNI kernel on a slab of `rows` rows of the same problem
    (same K and N, OpenMP over the rows).  Without AVX512-VNNI or the prebuilt objects: the oracle's OpenMP
    restatement on a smaller cube.  Returns (tera-ops per step, [seconds per step], description, kind, cores)."""
    import oracle
    cores = oracle.use_all_cores()
    rng = np.random.default_rng(3)
    if oracle.ref("multicore") is not None and (rows is None or oracle.ref("qkv") is not None):
        m = n if rows is None else rows
        A = rng.integers(-128, 128, (m, n), dtype=np.int8)
        Bt = rng.integers(-128, 128, (n, n), dtype=np.int8)
        if rows is None:
            fn = lambda: oracle.ref_vnni_square(A, Bt, multicore=True)
            what = f"reference vnni_matmul_multicore<{n}> (s8 x s8, B pre-transposed), {n}^3 per step"
        else:
            fn = lambda: oracle.ref_vnni_mnk(A, Bt, threads=cores)
            what = (f"reference vnni_matmul_i8 (s8 x s8, B pre-transposed, OpenMP over rows), a slab of {m} rows of the "
                    f"{n}^3 problem per step")
        for _ in range(warmup):
            fn()
        times = []
        for _ in range(repeats):
            t = time.perf_counter()
            fn()
            times.append(time.perf_counter() - t)
        return 2.0 * m * n * n / 1e12, times, what, "reference", cores
    n = min(n, 1024)
    A = rng.integers(-128, 128, (n, n), dtype=np.int8)
    Bt = rng.integers(-128, 128, (n, n), dtype=np.int8)
    times = []
    for i in range(warmup + repeats):
        t = time.perf_counter()
        oracle.tensor_matmul_i8(A, Bt, b_transposed=True, threads=0)
        if i >= warmup:
            times.append(time.perf_counter() - t)
    return 2.0 * n ** 3 / 1e12, times, f"oracle OpenMP scalar loop (no AVX512-VNNI here), {n}^3 per step", "port", cores


_TENSORS = {}


def model_tensors(which):
    """Seeded random-init tensors of a decode configuration (cached: the GPU leg and the CPU baseline share them)."""
    from simplang_b200 import synth
    if which not in _TENSORS:
        threads = len(os.sched_getaffinity(0))
        if which == "f32_110m":
            _TENSORS[which] = (synth.STORIES_110M, synth.llama_f32_tensors(synth.STORIES_110M, 0), None)
        else:
            t, off = synth.llama_w4_tensors(synth.LLAMA_3B_W4, 0, threads=threads)
            _TENSORS[which] = (synth.LLAMA_3B_W4, t, off)
    return _TENSORS[which]


def cpu_decode_baseline(which, n_tokens):
    """Tokens/s of the CPU restatement of the model (oracle, OpenMP over rows, all host cores) on a bounded
    number of tokens: the first is a warm-up, the rest are timed."""
    import oracle
    from simplang_b200 import synth
    cores = oracle.use_all_cores()
    cfg, t, off = model_tensors(which)
    m = oracle.Llama(cfg, t, threads=cores) if off is None else oracle.Llama(cfg, t, w4=True, offsets=off, threads=cores)
    tok = int(synth.prompt_tokens(16, cfg["vocab_size"])[0])
    logits = m.forward(tok, 0)
    t0 = time.perf_counter()
    for pos in range(1, n_tokens + 1):
        tok = int(oracle.argmax(logits))
        logits = m.forward(tok, pos)
    dt = time.perf_counter() - t0
    return {"tok_s": n_tokens / dt, "unit": "tokens/s", "cores": cores, "kind": "port",
            "sample": f"oracle restatement of the model, {n_tokens} greedy tokens from position 1 after 1 warm-up token"}


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    n = args.size
    total_steps = args.steps + args.warmup
    budget_s = 150.0
    # the whole problem per step when the run then ends within the budget, else a slab of its rows per step
    _, probe, _, _, _ = cpu_reference_gemm(n, 1, 1)
    rows = None
    if probe[0] * total_steps > budget_s:
        rows = int(n * budget_s / (probe[0] * total_steps)) // 64 * 64
        rows = max(64, min(rows, n))
    tera_ops, times, sample, kind, cores = cpu_reference_gemm(n, args.steps, args.warmup, rows=rows)
    total = sum(times)
    value = tera_ops * len(times) / total
    line = {
        "impl": "reference", "metric": "int8_gemm_tops", "value": value, "unit": "TOPS", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / len(times),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "u8", "data": "synthetic",
        "config": {"workload": f"int8 tensor_matmul {args.size}^3 u8 x s8 -> i32 (CPU arm: see cpu_baseline.sample)"},
        "cpu_baseline": {"value": value, "unit": "TOPS", "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    if not args.no_decode:
        line["decode"] = {"f32_110m": cpu_decode_baseline("f32_110m", 32), "w4_3b": cpu_decode_baseline("w4_3b", 4)}
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------------- decode legs
def decode_bytes_per_token(cfg, w4, steps, ranks):
    """Bytes that must stream from HBM per token and GPU: the weights (every projection and the f32 classifier), the
    average key/value cache read over the run and one embedding row."""
    d, h, L, V = cfg["dim"], cfg["hidden_dim"], cfg["n_layers"], cfg["vocab_size"]
    nw = L * (4 * d * d + 3 * d * h)
    if w4:
        wbytes = nw // 2 + 4 * nw // cfg["group_size"] + 4 * V * d
    else:
        wbytes = 4 * (nw + V * d)
    kv = 2 * L * d * 4 * (steps + 1) / 2.0
    return (wbytes + kv) / ranks + 4 * d, wbytes / ranks, kv / ranks


def shared_w4_tensors(cfg, rank, world, barrier):
    """The 3B W4 tensors, generated once per node: rank 0 writes them to a memory-backed directory, the other ranks
    map the files (every rank's loader keeps only its own row slices)."""
    if world == 1:
        _, t, off = model_tensors("w4_3b")
        return t, off, None
    base = "/dev/shm" if os.path.isdir("/dev/shm") else "/tmp"
    d = os.path.join(base, f"simp_bench_{os.environ.get('MASTER_PORT', '0')}_{os.getuid()}")
    if rank == 0:
        _, t, off = model_tensors("w4_3b")
        os.makedirs(d, exist_ok=True)
        for k, v in t.items():
            np.save(os.path.join(d, k + ".npy"), v)
        with open(os.path.join(d, "offsets.json"), "w") as f:
            json.dump(off, f)
    barrier()
    if rank != 0:
        with open(os.path.join(d, "offsets.json")) as f:
            off = json.load(f)
        t = {k[:-4]: np.load(os.path.join(d, k), mmap_mode="r") for k in os.listdir(d) if k.endswith(".npy")}
    return t, off, d


def run_decode_leg(sg, which, rank, world, barrier, local_rank, peaks):
    """One model of the decode half of the metric: 16 teacher-forced prompt tokens, then greedy tokens (256 for the
    f32 110M model, 128 for the 3B W4 model).  Device-timed over the whole generation (CUDA events inside
    simp_llama_generate) and wall-clock around the same call with the token ids copied back (`e2e`)."""
    from simplang_b200 import synth
    shm_dir = None
    if which == "f32_110m":
        cfg, w4, n_new, tp = synth.STORIES_110M, False, 256, 1
        if rank != 0:      # single-GPU configuration: rank 0 runs it, the others wait
            barrier()
            return None
        model = sg.Llama(cfg, model_tensors(which)[1])
    else:
        cfg, w4, n_new, tp = synth.LLAMA_3B_W4, True, 128, world
        t, off, shm_dir = shared_w4_tensors(cfg, rank, world, barrier)
        model = sg.Llama(cfg, t, w4=True, offsets=off, tp_size=world)
    prompt = synth.prompt_tokens(16, cfg["vocab_size"])
    steps = 16 + n_new - 1
    model.generate(prompt, 8)          # warm-up: builds the graph, first touches
    model.generate(prompt, n_new)
    if tp > 1:
        barrier()
    sampler = ClockSampler(local_rank, period_s=0.002)
    if rank == 0:
        sampler.start()
    toks1, _, ms = model.generate(prompt, n_new)
    t0 = time.perf_counter()
    toks2, _, _ = model.generate(prompt, n_new)
    wall = time.perf_counter() - t0
    clocks = sampler.stop() if rank == 0 else None
    sg.check(sg.lib().simp_gpu_check_device_status())
    if tp > 1:
        import torch
        import torch.distributed as dist
        tt = torch.tensor([ms, wall * 1e3], device="cuda")
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms, wall = float(tt[0].item()), float(tt[1].item()) / 1e3
    launches = model.kernels_per_token()
    check = {"second_run_identical": bool(np.array_equal(toks1, toks2))}
    if not check["second_run_identical"]:
        raise SystemExit(f"bench: {which}: two runs of the same generation differ -- refusing to report a number")
    model.close()
    if tp > 1:
        barrier()
        if rank == 0:   # the same generation on one GPU must give the same tokens
            single = sg.Llama(cfg, t, w4=True, offsets=off, tp_size=1)
            ref_toks, _, _ = single.generate(prompt, n_new)
            single.close()
            same = int(np.sum(ref_toks == toks1))
            check["tokens_equal_to_single_gpu"] = f"{same}/{n_new}"
            if same != n_new:
                raise SystemExit(f"bench: {which}: tensor-parallel tokens differ from the single-GPU run ({same}/{n_new})")
        barrier()
        if rank == 0 and shm_dir:
            import shutil
            shutil.rmtree(shm_dir, ignore_errors=True)
    elif which == "f32_110m" and world > 1:
        barrier()
    if rank != 0:
        return None
    per_gpu, wbytes, kv = decode_bytes_per_token(cfg, w4, steps, tp)
    us = ms * 1e3 / steps
    gbs = per_gpu / us / 1e3
    return {
        "tok_s": 1e6 / us, "unit": "tokens/s", "us_per_token": us, "tokens": steps, "n_gpus": tp,
        "workload": ("LLaMA-2-style 110M f32, dim 768, 12 layers, vocab 32000, seq_len 1024" if not w4 else
                     "LLaMA 3B W4 (symmetric int4, groups of 64), dim 3200, 26 layers, 32 heads, FFN 8640, vocab 32000, "
                     "seq_len 2048" + (f", tensor parallel over {tp} ranks" if tp > 1 else "")) +
                    f"; batch 1, 16 prompt tokens + {n_new} greedy, random-init weights",
        "e2e": {"tok_s": steps / wall, "ms_total": wall * 1e3, "h2d_bytes": int(prompt.nbytes), "d2h_bytes": int(toks2.nbytes),
                "api": "simp_llama_generate (prompt ids in, generated ids out, wall clock around the call)"},
        "kernels_per_token": launches,
        "roofline": {"bound": "hbm", "bytes_per_token_per_gpu": int(per_gpu), "weight_bytes_per_gpu": int(wbytes),
                     "avg_kv_bytes_per_gpu": int(kv), "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": gbs / peaks["hbm_gbs"], "peak_basis": f"copy bandwidth, {peaks['source']}"},
        "clocks": clocks, "check": check,
    }


# --------------------------------------------------------------------------------------------- GPU arm
def run_ours(args):
    import simplang_b200 as sg

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    sg.init(local_rank)

    S = args.size
    M = K = N = S
    assert N % world == 0 and (N // world) % 32 == 0, "N must split into 32-column multiples per rank"
    Nl = N // world
    A, B = gen_inputs(M, K, N)
    B_local = np.ascontiguousarray(B[:, rank * Nl:(rank + 1) * Nl])

    dA, dB = sg.DeviceBuffer.from_numpy(A), sg.DeviceBuffer.from_numpy(B_local)
    c_ptr = None
    if world > 1:
        import ctypes as C
        from simplang_b200 import dist as sd
        sd.init_from_env(sg)
        cptr = C.c_void_p()
        sg.check(sg.lib().simp_dist_symm_alloc(M * N * 4, C.byref(cptr)))  # full row-major C on every rank
        c_ptr = cptr.value
        fused = os.environ.get("SIMP_BENCH_ALLGATHER", "fused") == "fused"
        if not fused:
            dC = sg.DeviceBuffer(world * M * Nl * 4)
        dC_local = sg.DeviceBuffer(M * Nl * 4)

        def step():
            if fused:  # all-gather fused into the GEMM epilogue (stores to every rank's C)
                sg.check(sg.lib().simp_dist_matmul_i8_nsharded_fused(dA.ptr, dB.ptr, c_ptr, M, K, Nl, 1, 0))
            else:      # GEMM, then NCCL all-gather of the column blocks
                sg.check(sg.lib().simp_dist_matmul_i8_nsharded(dA.ptr, dB.ptr, dC.ptr, M, K, Nl, 1, 0))

        def step_local():   # the same shard of the product, C left column-sharded (no exchange)
            sg.matmul_i8(dA, dB, dC_local, M, K, Nl, a_unsigned=True, b_transposed=False)
    else:
        fused = False
        dC = sg.DeviceBuffer(M * N * 4)

        def step():
            sg.matmul_i8(dA, dB, dC, M, K, N, a_unsigned=True, b_transposed=False)

    def barrier():
        if dist is not None:
            dist.barrier()
            import torch
            torch.cuda.synchronize()
        sg.sync()

    def max_over_ranks(v):
        if dist is None:
            return v
        import torch
        t = torch.tensor([v], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def timed(fn, steps, sample=False):
        barrier()
        sampler = ClockSampler(local_rank, period_s=0.002)
        if sample and rank == 0:
            sampler.start()
        barrier()
        e0, e1 = sg.Event(), sg.Event()
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        ms = max_over_ranks(e0.elapsed_ms(e1))
        return ms, (sampler.stop() if sample and rank == 0 else None)

    for _ in range(max(args.warmup, 3)):
        step()
    ms_total, clocks = timed(step, args.steps, sample=True)
    sg.check(sg.lib().simp_gpu_check_device_status())

    ops = 2.0 * M * N * K
    ms_step = ms_total / args.steps
    tops = ops / (ms_step * 1e-3) / 1e12

    # in-run parity spot check: EVERY rank checks rows of its own copy of C against the exact integer product
    rows = sorted({(7 * rank) % M, (M // 2 + 1 + 13 * rank) % M, M - 1 - rank, (M // world) * rank})
    if world > 1 and fused:
        Cg = np.empty((len(rows), N), np.int32)
        for i, r in enumerate(rows):
            sg.check(sg.lib().simp_gpu_download(Cg[i].ctypes.data, c_ptr + 4 * r * N, 4 * N))
    elif world > 1:
        blocks = dC.to_numpy(np.int32, (world, M, Nl))
        Cg = np.concatenate([blocks[r][rows] for r in range(world)], axis=1)  # column blocks -> rows of C
    else:
        Cg = dC.to_numpy(np.int32, (M, N))[rows]
    exact = (A[rows].astype(np.int64) @ B.astype(np.int64)).astype(np.int32)
    ok = float(np.array_equal(Cg, exact))
    if max_over_ranks(1.0 - ok) != 0.0:
        raise SystemExit(f"bench: rank {rank}: GPU result differs from the exact product -- refusing to report a number"
                         if not ok else "bench: another rank's result differs from the exact product")

    # ---- a long pass of the same step (single GPU): what the kernel sustains once the power cap is reached
    sustained = None
    if world == 1 and not args.no_sustained:
        n_long = max(200, int(2000.0 / max(ms_step, 1e-3)))
        ms_long, clk_long = timed(step, n_long, sample=True)
        sustained = {"value": ops / (ms_long / n_long * 1e-3) / 1e12, "unit": "TOPS", "steps": n_long,
                     "seconds": ms_long / 1e3, "clocks": clk_long}

    # ---- N > 1: the same shards with C left column-sharded (no exchange), and the link figures of the exchange
    without_gather = None
    link = None
    if world > 1:
        for _ in range(3):
            step_local()
        ms_local, _ = timed(step_local, args.steps)
        ms_local /= args.steps
        without_gather = {"value": ops / (ms_local * 1e-3) / 1e12, "unit": "TOPS", "ms_per_step": ms_local,
                          "note": "every rank computes its column block of C and keeps it (no all-gather)"}
        out_bytes = 4.0 * M * Nl * (world - 1)      # leaves (and enters) every GPU per step
        link_ms = out_bytes / 770e9 * 1e3
        link = {"bytes_out_per_gpu_per_step": int(out_bytes), "achieved_gb_s_per_gpu": out_bytes / (ms_step * 1e-3) / 1e9,
                "peer_copy_gb_s": 770.0, "link_floor_ms": link_ms, "math_ms": ms_local,
                "frac_of_max_math_link": max(link_ms, ms_local) / ms_step}

    # ---- N > 1: the largest cube of the sweep, 16384^3, where the math per exchanged byte is twice that of 8192^3
    cube16k = None
    if world > 1 and not args.no_big and S == 8192:
        import ctypes as C
        S2 = 16384
        Nl2 = S2 // world
        rng2 = np.random.default_rng(77)
        A2 = rng2.integers(0, 256, (S2, S2), dtype=np.uint8)
        B2 = rng2.integers(-128, 128, (S2, S2), dtype=np.int8)
        dA2 = sg.DeviceBuffer.from_numpy(A2)
        dB2 = sg.DeviceBuffer.from_numpy(np.ascontiguousarray(B2[:, rank * Nl2:(rank + 1) * Nl2]))
        cp2 = C.c_void_p()
        sg.check(sg.lib().simp_dist_symm_alloc(S2 * S2 * 4, C.byref(cp2)))

        def step2():
            sg.check(sg.lib().simp_dist_matmul_i8_nsharded_fused(dA2.ptr, dB2.ptr, cp2.value, S2, S2, Nl2, 1, 0))

        for _ in range(3):
            step2()
        n2 = max(3, min(args.steps, 10))
        ms2, _ = timed(step2, n2)
        ms2 /= n2
        sg.check(sg.lib().simp_gpu_check_device_status())
        # every rank checks 3 rows of a 2048-column slice that ANOTHER rank computed
        src = (rank + 1) % world
        c_lo = src * Nl2
        rows2 = [(5 * rank + 1) % S2, S2 // 2 + rank, S2 - 1 - rank]
        got2 = np.empty((3, 2048), np.int32)
        for i, r in enumerate(rows2):
            sg.check(sg.lib().simp_gpu_download(got2[i].ctypes.data, cp2.value + 4 * (r * S2 + c_lo), 4 * 2048))
        exact2 = (A2[rows2].astype(np.float64) @ B2[:, c_lo:c_lo + 2048].astype(np.float64)).astype(np.int64).astype(np.int32)
        ok2 = float(np.array_equal(got2, exact2))
        if max_over_ranks(1.0 - ok2) != 0.0:
            raise SystemExit("bench: 16384^3 gathered result differs from the exact product")
        ops2 = 2.0 * S2 ** 3
        out2 = 4.0 * S2 * Nl2 * (world - 1)
        cube16k = {"value": ops2 / (ms2 * 1e-3) / 1e12, "unit": "TOPS", "ms_per_step": ms2, "steps": n2,
                   "workload": "int8 tensor_matmul 16384^3, N-sharded, all-gather fused into the GEMM epilogue",
                   "bytes_out_per_gpu_per_step": int(out2), "achieved_gb_s_per_gpu": out2 / (ms2 * 1e-3) / 1e9,
                   "link_floor_ms": out2 / 770e9 * 1e3, "check": "3 rows x 2048 columns of a peer's block exact on every rank"}
        dA2.free(); dB2.free()
        sg.check(sg.lib().simp_dist_symm_free(cp2.value))
        del A2, B2

    # ---- e2e through the host-pointer entry point (every rank computes its shard; max over ranks)
    hA = sg.pinned_empty((M, K), np.uint8); hA[...] = A
    hB = sg.pinned_empty((K, Nl), np.int8); hB[...] = B_local
    hC = sg.pinned_empty((M, Nl), np.int32)
    e2e_steps = max(2, min(args.steps, 5))
    sg.host_tensor_matmul_i8(hA, hB, hC)  # warm-up (allocates staging)
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        sg.host_tensor_matmul_i8(hA, hB, hC)
    t_e2e = max_over_ranks((time.perf_counter() - t0) / e2e_steps)
    e2e_tops = ops / t_e2e / 1e12
    del hA, hB, hC

    # ---- int8 MMA issue ceiling of the same tiling (single GPU only): the GEMM kernel with its TMA loads and
    # epilogue traffic switched off, run last so that it cannot disturb the timed region or the result check
    mma_ceiling = None
    if world == 1 and (M // 256) * (N // 256) >= 74:
        os.environ["SIMP_GEMM_I8_ABLATE"] = "mma"
        try:
            dScratch = sg.DeviceBuffer(M * N * 4)
            for _ in range(3):
                sg.matmul_i8(dA, dB, dScratch, M, K, N, a_unsigned=True, b_transposed=False)
            sg.sync()
            f0, f1 = sg.Event(), sg.Event()
            f0.record()
            for _ in range(10):
                sg.matmul_i8(dA, dB, dScratch, M, K, N, a_unsigned=True, b_transposed=False)
            f1.record()
            sg.sync()
            mma_ceiling = ops / (f0.elapsed_ms(f1) / 10 * 1e-3) / 1e12
            dScratch.free()
        finally:
            os.environ.pop("SIMP_GEMM_I8_ABLATE", None)

    # ---- the GEMM buffers are released before the decode legs
    dA.free(); dB.free()
    if world > 1:
        dC_local.free()
        sg.check(sg.lib().simp_dist_symm_free(c_ptr))
        if not fused:
            dC.free()
    else:
        dC.free()

    peaks = measured_peaks()
    decode = None
    if not args.no_decode:
        decode = {}
        for which in ("f32_110m", "w4_3b"):
            decode[which] = run_decode_leg(sg, which, rank, world, barrier, local_rank, peaks)

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    peak_int8 = 2.0 * peaks["bf16_tflops"]
    line = {
        "metric": "int8_gemm_tops", "value": tops, "unit": "TOPS", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "u8", "data": "synthetic",
        "config": {"workload": f"int8 tensor_matmul {S}^3: u8[M,K] x s8[K,N] -> i32, seeded uniform, row-major",
                   "sharding": "single GPU" if world == 1 else (f"N-sharded over {world} ranks, all-gather of C fused into the GEMM epilogue (every tile stored to all peers over NVLink by the kernel itself)"
                                                                   if fused else f"N-sharded over {world} ranks + NCCL all-gather of the column blocks of C"),
                   "l2": "384 MB touched per step at 8192^3 (> 126 MB L2): no flush between steps",
                   "decode": "second half of the metric: see the `decode` record (f32 110M on one GPU; W4 3B tensor-parallel over all ranks)"},
        "clocks": clocks,
        "e2e": {"value": e2e_tops, "unit": "TOPS", "h2d_bytes_per_step": int(M * K + K * Nl) * world,
                "d2h_bytes_per_step": int(4 * M * Nl) * world, "ms_per_step": 1e3 * t_e2e, "steps": e2e_steps,
                "api": "simp_host_tensor_matmul_i8 (pinned host operands; C in row chunks x column blocks, upload / compute / download overlapped)"},
        "gpu_launches": args.steps,
        "roofline": {"bound": "tensor", "achieved": tops / world, "peak": peak_int8, "unit": "TOP/s",
                     "frac": tops / world / peak_int8,
                     "peak_basis": f"2 x cuBLAS bf16 burst ({peaks['bf16_tflops']} TFLOP/s, {peaks['source']}); "
                                   "int8 MMA issues at twice the bf16 rate",
                     "frac_of_nominal_4500": tops / world / NOMINAL_INT8_TOPS,
                     "mma_issue_ceiling": mma_ceiling,
                     "mma_issue_ceiling_note": "same kernel and tiling without TMA loads and epilogue traffic, 10 launches: "
                                               "measured int8 pipe ceiling at whatever clock a 10-launch burst runs at "
                                               "(see `clocks` for the timed region and `sustained.clocks` for a 2 s pass)",
                     "frac_of_mma_issue_ceiling": (tops / mma_ceiling) if mma_ceiling else None,
                     "traffic": NCU_TRAFFIC_BYTES.get(S), "algorithmic_bytes": int(M * K + K * N + 4 * M * N),
                     "kernel": "gemm_i8_tcgen05_2cta_kernel" if (M // 256) * (N // world // 256) >= 74 else "gemm_i8_tcgen05_kernel"},
    }
    if sustained:
        line["sustained"] = sustained
    if without_gather:
        line["without_gather"] = without_gather
        line["link"] = link
    if cube16k:
        line["cube_16384"] = cube16k
    if decode:
        line["decode"] = decode
    if world == 1 and not args.no_cpu:
        tera, times, sample, kind, cores = cpu_reference_gemm(min(S, 8192), 2, 1)
        line["cpu_baseline"] = {"value": tera / min(times), "unit": "TOPS", "cores": cores, "kind": kind,
                                "sample": sample + ", best of 2 after 1 warm-up"}
        if decode:
            line["cpu_baseline"]["decode"] = {"f32_110m": cpu_decode_baseline("f32_110m", 32),
                                              "w4_3b": cpu_decode_baseline("w4_3b", 4)}
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--size", type=int, default=8192)
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--no-decode", action="store_true", help="skip the LLaMA decode legs")
    ap.add_argument("--no-sustained", action="store_true", help="skip the 2-second pass of the GEMM step")
    ap.add_argument("--no-big", action="store_true", help="skip the 16384^3 sub-record of the multi-GPU arm")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
