"""Per-op sweep of the bandwidth-bound kernels (f32 GEMV, W4 GEMV, rmsnorm, softmax, silu) and of the
int8 GEMM at the configured shapes.  Prints one JSON line per case with the achieved GB/s (or TOPS), the
algorithmic bytes used, and the fraction of the measured roofline.

    python -m simplang_b200.opbench [--iters 50] [--only gemv_f32,gemm_f32,w4,rowops,gemm_i8,gemm_i4,mma_peak,decode110m,decode3b,decode_i8,prefill_i8]

Each case rotates over enough independent operand copies that the working set exceeds twice the
126 MB L2, so every iteration streams from HBM the way consecutive layers of a decode step do.
Timing: CUDA events on the library stream, 3 warm-up passes, mean over `iters` launches.
"""
from __future__ import annotations

import argparse
import json
import os

import numpy as np

import simplang_b200 as sg

L2_BYTES = 126 << 20
WORLD = int(os.environ.get("WORLD_SIZE", "1"))
RANK = int(os.environ.get("RANK", "0"))
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def hbm_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return json.load(open(p))["hbm_gbs"], "measured"
    return 6650.0, "fallback"


SHAPE_FILTER = None  # e.g. [32000, 3200]: run only the case with this shape (for single-kernel ncu captures)


def want(shape):
    return SHAPE_FILTER is None or list(shape) == SHAPE_FILTER


def copies_for(nbytes):
    return max(2, min(256, int(2 * L2_BYTES // max(nbytes, 1)) + 1))


def timed(fn, ncopies, iters):
    for i in range(3 * min(ncopies, 4)):
        fn(i % ncopies)
    sg.sync()
    e0, e1 = sg.Event(), sg.Event()
    e0.record()
    for i in range(iters):
        fn(i % ncopies)
    e1.record()
    sg.sync()
    return e0.elapsed_ms(e1) / iters


def emit(op, shape, ms, nbytes, extra=None):
    peak, src = hbm_peak()
    gbs = nbytes / (ms * 1e-3) / 1e9
    line = {"op": op, "shape": shape, "us": round(ms * 1e3, 3), "algorithmic_bytes": int(nbytes),
            "gb_s": round(gbs, 1), "frac_of_hbm_peak": round(gbs / peak, 4), "peak_gb_s": peak, "peak": src}
    if extra:
        line.update(extra)
    print(json.dumps(line), flush=True)


def bench_gemv_f32(iters):
    rng = np.random.default_rng(0)
    for rows, cols in [(768, 768), (2048, 768), (768, 2048), (32000, 768), (3200, 3200), (32000, 3200), (65536, 4096)]:
        if not want((rows, cols)):
            continue
        nb = 4 * (rows * cols + cols + rows)
        nc = copies_for(nb)
        A = sg.DeviceBuffer.from_numpy((0.02 * rng.standard_normal(rows * cols)).astype(np.float32))
        bufs = [A] + [sg.DeviceBuffer(rows * cols * 4) for _ in range(nc - 1)]
        for b in bufs[1:]:
            sg.check(sg.lib().simp_gpu_memset(b.ptr, 0, b.nbytes))
        x = sg.DeviceBuffer.from_numpy(rng.standard_normal(cols).astype(np.float32))
        y = sg.DeviceBuffer(rows * 4)
        ms = timed(lambda i: sg.matmul_f32(bufs[i], 0, x, 0, y, 0, rows, cols, 1, accumulate=False), nc, iters)
        emit("gemv_f32", [rows, cols], ms, nb, {"copies": nc})
        del bufs


def bench_gemm_f32(iters):
    """tensor_matmul on f32 with more than one right-hand side: the projection shapes of
    examples/llama2/llama32_1b_fp32_prefill.sl:51-199 (M tokens x [2048 -> 2048 / 512 / 8192, 8192 -> 2048]).
    M = 8 / 64: f32 FMA kernels bound by the weight stream; M >= 128: 3 x TF32 on the tensor cores (f32 accuracy), whose
    rate is also reported against the FP32 pipe's own peak (148 SMs x 128 FMA per clock) for comparison."""
    rng = np.random.default_rng(5)
    ffma_peak = 148 * 128 * 2 * 1.965e9 / 1e12   # TFLOP/s at the maximum clock
    for m, k, n in [(8, 2048, 2048), (8, 2048, 8192), (64, 2048, 2048), (512, 2048, 2048), (512, 2048, 8192), (512, 8192, 2048),
                    (4096, 4096, 4096), (8192, 8192, 8192)]:
        if not want((m, k, n)):
            continue
        nb = 4 * (m * k + k * n + m * n)
        nc = copies_for(4 * k * n)
        A = sg.DeviceBuffer.from_numpy(rng.standard_normal(m * k).astype(np.float32))
        Bs = [sg.DeviceBuffer.from_numpy((0.02 * rng.standard_normal(k * n)).astype(np.float32)) for _ in range(min(nc, 8))]
        Cb = sg.DeviceBuffer(m * n * 4)
        ms = timed(lambda i: sg.matmul_f32(A, 0, Bs[i % len(Bs)], 0, Cb, 0, m, k, n, accumulate=False), len(Bs), iters)
        tf = 2.0 * m * k * n / (ms * 1e-3) / 1e12
        emit("tensor_matmul_f32", [m, k, n], ms, nb, {"tflops": round(tf, 2), "frac_of_ffma_peak": round(tf / ffma_peak, 3),
                                                      "ffma_peak_tflops": round(ffma_peak, 1)})
        del Bs


def bench_w4(iters):
    rng = np.random.default_rng(1)
    gs = 64
    for rows, cols in [(3200, 3200), (9600, 3200), (8640, 3200), (3200, 8640), (26 * 8640, 3200), (65536, 8192)]:
        if not want((rows, cols)):
            continue
        nb = rows * cols // 2 + 4 * rows * cols // gs + 4 * cols + 4 * rows
        nc = copies_for(nb)
        qbytes, ngroups = rows * cols // 2, rows * cols // gs
        q = sg.DeviceBuffer.from_numpy(rng.integers(0, 256, nc * qbytes, dtype=np.uint8))
        s = sg.DeviceBuffer.from_numpy((0.01 * rng.random(nc * ngroups)).astype(np.float32))
        x = sg.DeviceBuffer.from_numpy(rng.standard_normal(cols).astype(np.float32))
        y = sg.DeviceBuffer(rows * 4)
        ms = timed(lambda i: sg.matmul_w4(q, s, None, x, y, rows, cols, gs, i * rows * cols, scale_mode=1), nc, iters)
        emit("gemv_w4_sym_gs64", [rows, cols], ms, nb, {"copies": nc})
        del q, s


def bench_rowops(iters):
    rng = np.random.default_rng(2)
    for rows, n in [(4096, 768), (4096, 3200), (4096, 4096), (16384, 4096)]:
        if not want((rows, n)):
            continue
        nb = 4 * (2 * rows * n + n)
        nc = copies_for(nb)
        xs = [sg.DeviceBuffer.from_numpy(rng.standard_normal(rows * n).astype(np.float32)) for _ in range(min(nc, 8))]
        ys = [sg.DeviceBuffer(rows * n * 4) for _ in range(len(xs))]
        w = sg.DeviceBuffer.from_numpy(np.ones(n, np.float32))
        ms = timed(lambda i: sg.rmsnorm_f32(xs[i], w, ys[i], rows, n), len(xs), iters)
        emit("rmsnorm", [rows, n], ms, nb, {"copies": len(xs)})
        ms = timed(lambda i: sg.softmax_f32(xs[i], ys[i], rows, n), len(xs), iters)
        emit("softmax", [rows, n], ms, 8 * rows * n, {"copies": len(xs)})
        ms = timed(lambda i: sg.silu_f32(xs[i], None, ys[i], rows * n), len(xs), iters)
        emit("silu", [rows * n], ms, 8 * rows * n, {"copies": len(xs)})
        ms = timed(lambda i: sg.silu_f32(xs[i], xs[(i + 1) % len(xs)], ys[i], rows * n), len(xs), iters)
        emit("silu_mul", [rows * n], ms, 12 * rows * n, {"copies": len(xs)})
        del xs, ys


def bench_gemm_i8(iters):
    rng = np.random.default_rng(3)
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    peak = 2 * (json.load(open(peaks_path))["bf16_tflops"] if os.path.exists(peaks_path) else 1590.0)
    cases = [(1024, 1024, 1024), (2048, 2048, 2048), (4096, 4096, 4096), (8192, 8192, 8192), (16384, 16384, 16384),
             (512, 3200, 9600), (512, 3200, 8640), (512, 8640, 3200)]
    for M, K, N in cases:
        if not want((M, K, N)):
            continue
        A = sg.DeviceBuffer.from_numpy(rng.integers(0, 256, (M, K), dtype=np.uint8))
        for b_t in (False, True):
            B = sg.DeviceBuffer.from_numpy(rng.integers(-128, 128, (K, N), dtype=np.int8))
            Cd = sg.DeviceBuffer(M * N * 4)
            it = max(3, min(iters, int(2e14 / (2.0 * M * N * K))))
            ms = timed(lambda i: sg.matmul_i8(A, B, Cd, M, K, N, a_unsigned=True, b_transposed=b_t), 1, it)
            tops = 2.0 * M * N * K / (ms * 1e-3) / 1e12
            # the same call recorded once and replayed: device time without the per-call launch cost of the host
            per = 20
            with sg.Recording() as rec:
                for _ in range(per):
                    sg.matmul_i8(A, B, Cd, M, K, N, a_unsigned=True, b_transposed=b_t)
            reps = max(1, it // per)
            rec.replay(1)
            sg.sync()
            e0, e1 = sg.Event(), sg.Event()
            e0.record()
            rec.replay(reps)
            e1.record()
            sg.sync()
            ms_r = e0.elapsed_ms(e1) / (reps * per)
            rec.close()
            tops_r = 2.0 * M * N * K / (ms_r * 1e-3) / 1e12
            print(json.dumps({"op": "gemm_i8", "shape": [M, K, N], "b_transposed": b_t, "us": round(ms * 1e3, 2),
                              "tops": round(tops, 1), "us_replayed": round(ms_r * 1e3, 2), "tops_replayed": round(tops_r, 1),
                              "frac_of_2x_bf16_burst": round(max(tops, tops_r) / peak, 4),
                              "frac_of_nominal_4500": round(max(tops, tops_r) / 4500, 4)}), flush=True)
            del B, Cd


def bench_mma_peak(iters):
    """Issue ceiling of the int8 tensor pipe for the 2-CTA tiling: the GEMM kernel run with its TMA loads and
    its epilogue traffic switched off (SIMP_GEMM_I8_ABLATE=mma; the result buffer is not written).  This is
    the measured int8 figure next to the calibrated 2 x bf16 one."""
    rng = np.random.default_rng(3)
    M = K = N = 8192
    A = sg.DeviceBuffer.from_numpy(rng.integers(0, 256, (M, K), dtype=np.uint8))
    B = sg.DeviceBuffer.from_numpy(rng.integers(-128, 128, (K, N), dtype=np.int8))
    Cd = sg.DeviceBuffer(M * N * 4)
    out = {}
    for mode in ("mma", None):
        if mode:
            os.environ["SIMP_GEMM_I8_ABLATE"] = mode
        else:
            os.environ.pop("SIMP_GEMM_I8_ABLATE", None)
        ms = timed(lambda i: sg.matmul_i8(A, B, Cd, M, K, N, a_unsigned=True, b_transposed=False), 1, min(iters, 20))
        out[mode or "full"] = 2.0 * M * N * K / (ms * 1e-3) / 1e12
    print(json.dumps({"op": "int8 MMA issue ceiling (2-CTA tiling, 8192^3, no loads / no epilogue)",
                      "tops_mma_only": round(out["mma"], 1), "tops_full_kernel": round(out["full"], 1),
                      "full_over_mma_only": round(out["full"] / out["mma"], 4)}), flush=True)


def bench_gemm_i4(iters):
    """Packed i4 x i4 -> i16 tensor_matmul at the sizes of the reference's benchmark (bench_int4_matmul.sl: 32 ... 1024)."""
    rng = np.random.default_rng(4)
    for n in (32, 64, 128, 256, 384, 512, 768, 1024, 4096):
        A = sg.DeviceBuffer.from_numpy(rng.integers(0, 256, (n, n // 2), dtype=np.uint8))
        B = sg.DeviceBuffer.from_numpy(rng.integers(0, 256, (n, n // 2), dtype=np.uint8))
        Cd = sg.DeviceBuffer(n * n * 2)
        call = lambda i: sg.check(sg.lib().simp_gpu_matmul_i4(A.ptr, B.ptr, Cd.ptr, n, n, n))
        ms = timed(call, 1, iters)
        with sg.Recording() as rec:
            for _ in range(10):
                call(0)
        rec.replay(1)
        sg.sync()
        e0, e1 = sg.Event(), sg.Event()
        e0.record()
        rec.replay(5)
        e1.record()
        sg.sync()
        ms_r = e0.elapsed_ms(e1) / 50
        rec.close()
        print(json.dumps({"op": "gemm_i4", "n": n, "us": round(ms * 1e3, 2), "us_replayed": round(ms_r * 1e3, 2),
                          "giops_replayed": round(2.0 * n ** 3 / (ms_r * 1e-3) / 1e9, 1)}), flush=True)


DECODE_TOKENS = 128


def bench_decode(which, n_new=None):
    """Greedy decode tokens/s of the two model configurations (random init), device-timed over the
    whole generation (prompt of 16 teacher-forced tokens + n_new generated)."""
    from simplang_b200 import synth
    n_new = n_new or DECODE_TOKENS
    peak, src = hbm_peak()
    if which == "110m":
        cfg = synth.STORIES_110M
        m = sg.Llama(cfg, synth.llama_f32_tensors(cfg, 0))
        d, h, L, V = cfg["dim"], cfg["hidden_dim"], cfg["n_layers"], cfg["vocab_size"]
        wbytes = 4 * (L * (4 * d * d + 3 * d * h) + V * d)
        name = "llama 110M f32 decode"
    else:
        cfg = synth.LLAMA_3B_W4
        t, off = synth.llama_w4_tensors(cfg, 0, threads=max(2, 16 // WORLD))
        m = sg.Llama(cfg, t, w4=True, offsets=off, tp_size=WORLD)  # tensor-parallel under torchrun
        d, h, L, V, gs = cfg["dim"], cfg["hidden_dim"], cfg["n_layers"], cfg["vocab_size"], cfg["group_size"]
        nw = L * (4 * d * d + 3 * d * h)
        wbytes = nw // 2 + 4 * nw // gs + 4 * V * d
        name = "llama 3B W4 decode"
    prompt = synth.prompt_tokens(16, cfg["vocab_size"])
    m.generate(prompt, 8)
    toks, _, ms = m.generate(prompt, n_new)
    steps = 16 + n_new - 1
    us = ms * 1e3 / steps
    kv = 2 * cfg["n_layers"] * cfg["dim"] * 4 * (steps / 2)
    if WORLD > 1:
        name += f" (tensor-parallel x{WORLD}, rank {RANK})"
        wbytes //= WORLD
    if RANK != 0:
        m.close()
        return
    print(json.dumps({"op": name, "tokens": steps, "us_per_token": round(us, 1), "tok_s": round(1e6 / us, 1),
                      "weight_bytes_per_token": int(wbytes), "avg_kv_bytes_per_token": int(kv),
                      "gb_s": round((wbytes + kv) / us / 1e3, 1), "frac_of_hbm_peak": round((wbytes + kv) / us / 1e3 / peak, 4),
                      "peak_gb_s": peak, "peak": src}), flush=True)
    m.close()


def bench_decode_marks():
    """Block-level time marks of one layer of the 3B W4 token graph.  Needs the instrumented library
    (`python -m simplang_b200.build --trace`, loaded through SIMP_GPU_LIB): thread 0 of every block of the four
    projection launches and of the attention launch of layer 1 writes %globaltimer marks; printed for the last token of
    the run as min / median / max over blocks, ns relative to the first block of the q/k/v launch."""
    import ctypes as C
    from simplang_b200 import synth
    L = sg.lib()
    if not hasattr(L, "simp_debug_w4_trace"):
        raise SystemExit("decode3b_marks needs the instrumented library: python -m simplang_b200.build --trace, then "
                         "SIMP_GPU_LIB=simplang_b200/libsimp_gpu_trace.so")
    cfg = synth.LLAMA_3B_W4
    t, off = synth.llama_w4_tensors(cfg, 0, threads=16)
    m = sg.Llama(cfg, t, w4=True, offsets=off)
    prompt = synth.prompt_tokens(16, cfg["vocab_size"])
    m.generate(prompt, 8)
    _, _, ms = m.generate(prompt, DECODE_TOKENS)
    print(json.dumps({"op": "llama 3B W4 decode (instrumented build)", "us_per_token": round(ms * 1e3 / (15 + DECODE_TOKENS), 1)}))
    n = 5 * 148 * 16
    buf = np.zeros(n, np.uint64)
    L.simp_debug_w4_trace.argtypes = [C.c_void_p, C.c_size_t]
    sg.check(L.simp_debug_w4_trace(buf.ctypes.data, n))
    marks = buf.reshape(5, 148, 16).astype(np.int64)
    base = marks[0, :, 0].min()
    proj = {0: "start", 1: "weights requested", 2: "predecessor done", 3: "input packed", 4: "first tile ready", 5: "batch done", 15: "end"}
    for k, name in enumerate(["q/k/v", "wo", "gate/up", "down"]):
        for mk, what in proj.items():
            v = marks[k, :, mk]
            v = v[v > 0] - base
            if len(v):
                print(json.dumps({"launch": name, "mark": what, "min_ns": int(v.min()), "median_ns": int(np.median(v)), "max_ns": int(v.max()), "blocks": int(len(v))}))
    att = {0: "start", 2: "rows requested", 3: "predecessor done", 4: "q/k/v staged", 7: "rows landed", 8: "scores done", 9: "softmax done",
           5: "values done", 6: "output stored"}
    for mk, what in att.items():
        v = marks[4, :cfg["n_heads"], mk]
        v = v[v > 0] - base
        if len(v):
            print(json.dumps({"launch": "attention", "mark": what, "min_ns": int(v.min()), "median_ns": int(np.median(v)), "max_ns": int(v.max()), "blocks": int(len(v))}))
    m.close()


def bench_decode_i8():
    """The int8 LLaMA-3.2-1B-style model as its host times it (bench_llama32_1b_int8.cpp): forwards of one
    int8 input at positions 0 / 127 / 511 / 1023 / 2047 / 4095 (5 each) and a 64-token loop from position 128."""
    from simplang_b200 import synth
    peak, src = hbm_peak()
    cfg = synth.LLAMA32_1B_INT8
    t = synth.llama_i8_tensors(cfg, 0, "bench")
    x = synth.llama_i8_input(cfg)
    m = sg.LlamaI8(cfg, t)
    d, h, L, V = cfg["dim"], cfg["hidden_dim"], cfg["n_layers"], cfg["vocab_size"]
    kvd = cfg["n_kv_heads"] * cfg["head_dim"]
    wbytes = L * (2 * d * d + 2 * kvd * d + 3 * h * d) + 4 * V * d
    m.decode_loop(x, 0, 3)
    for pos in (0, 127, 511, 1023, 2047, 4095):
        ms = min(m.decode_loop(x, pos, 1)[1] for _ in range(5))
        kvb = 2 * L * (pos + 1) * kvd
        print(json.dumps({"op": "llama-3.2-1B int8 forward", "pos": pos, "us_per_token": round(ms * 1e3, 1),
                          "tok_s": round(1e3 / ms, 1), "weight_bytes_per_token": int(wbytes), "kv_bytes": int(kvb),
                          "frac_of_hbm_peak": round((wbytes + kvb) / (ms * 1e-3) / 1e9 / peak, 4), "peak": src}), flush=True)
    m.reset_cache()
    _, ms = m.decode_loop(x, 128, 64)
    us = ms * 1e3 / 64
    kvb = 2 * L * 160 * kvd
    print(json.dumps({"op": "llama-3.2-1B int8 decode loop (64 tokens from pos 128)", "us_per_token": round(us, 1),
                      "tok_s": round(1e6 / us, 1), "weight_bytes_per_token": int(wbytes),
                      "gb_s": round((wbytes + kvb) / us / 1e3, 1),
                      "frac_of_hbm_peak": round((wbytes + kvb) / us / 1e3 / peak, 4), "peak_gb_s": peak, "peak": src}), flush=True)
    m.close()


def bench_prefill_i8():
    """Prefill of the int8 LLaMA-3.2-1B-style model as its host times it (bench_llama32_1b_int8_prefill.cpp):
    seq_len 8 ... 256, prompt tokens per second; the seven projections per layer are tcgen05 int8 GEMMs."""
    from simplang_b200 import synth
    cfg = dict(synth.LLAMA32_1B_INT8, max_seq_len=256)
    t = synth.llama_i8_tensors(cfg, 0, "bench")
    m = sg.LlamaI8(cfg, t)
    d, h, L = cfg["dim"], cfg["hidden_dim"], cfg["n_layers"]
    kvd = cfg["n_kv_heads"] * cfg["head_dim"]
    w_params = L * (2 * d * d + 2 * kvd * d + 3 * h * d)
    for M in (8, 16, 32, 64, 128, 256):
        x = np.random.default_rng(M).integers(-64, 64, (M, d), dtype=np.int8)
        m.prefill(x, M)
        ms = min(m.prefill(x, M)[3] for _ in range(5))
        print(json.dumps({"op": "llama-3.2-1B int8 prefill", "seq_len": M, "ms": round(ms, 3),
                          "prompt_tok_s": round(M / ms * 1e3, 1), "gemm_tops": round(2.0 * M * w_params / (ms * 1e-3) / 1e12, 2),
                          "weight_gb_s": round(w_params / (ms * 1e-3) / 1e9, 1)}), flush=True)
    m.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--only", default="gemv_f32,w4,rowops,gemm_i8")
    ap.add_argument("--shape", default=None, help="run only the case with this shape, e.g. 32000x3200")
    ap.add_argument("--tokens", type=int, default=128, help="generated tokens of the decode workloads (small for profiler runs)")
    args = ap.parse_args()
    global SHAPE_FILTER, DECODE_TOKENS
    DECODE_TOKENS = args.tokens
    if args.shape:
        SHAPE_FILTER = [int(v) for v in args.shape.lower().split("x")]
    sg.init(int(os.environ.get("LOCAL_RANK", "0")))
    if WORLD > 1:  # torchrun: tensor-parallel decode
        import torch
        import torch.distributed as dist
        from simplang_b200 import dist as sd
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        dist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0"))))
        sd.init_from_env(sg)
    which = set(args.only.split(","))
    if "gemv_f32" in which:
        bench_gemv_f32(args.iters)
    if "gemm_f32" in which:
        bench_gemm_f32(args.iters)
    if "w4" in which:
        bench_w4(args.iters)
    if "rowops" in which:
        bench_rowops(args.iters)
    if "gemm_i8" in which:
        bench_gemm_i8(args.iters)
    if "gemm_i4" in which:
        bench_gemm_i4(args.iters)
    if "mma_peak" in which:
        bench_mma_peak(args.iters)
    if "decode110m" in which:
        bench_decode("110m")
    if "decode3b_marks" in which:
        bench_decode_marks()
    if "decode3b" in which:
        bench_decode("3b")
    if "decode_i8" in which:
        bench_decode_i8()
    if "prefill_i8" in which:
        bench_prefill_i8()
    sg.check(sg.lib().simp_gpu_check_device_status())


if __name__ == "__main__":
    main()
