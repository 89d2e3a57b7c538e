"""GPU tests of the multi-GPU paths (need >= 2 GPUs, the 4-rank cases >= 4; skipped otherwise): the N-sharded int8
GEMM -- every rank must end with all column blocks, bit-exact against the oracle, in the NCCL form and in the form
that fuses the exchange into the GEMM epilogue -- and tensor-parallel W4 decode against the CPU oracle."""
import os
import socket
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    import torch
    import torch.distributed as dist
    import oracle
    import simplang_b200 as sg
    from simplang_b200 import dist as sd
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        sg.init(rank)
        sd.init_from_env(sg)
        M, K, N = 256, 512, 1024
        rng = np.random.default_rng(3)
        A = rng.integers(0, 256, (M, K), dtype=np.uint8)
        B = rng.integers(-128, 128, (K, N), dtype=np.int8)
        lo, hi = sd.column_shard(N, world, rank)
        dA = sg.DeviceBuffer.from_numpy(A)
        dB = sg.DeviceBuffer.from_numpy(np.ascontiguousarray(B[:, lo:hi]))
        dC = sg.DeviceBuffer(world * M * (hi - lo) * 4)
        sg.check(sg.lib().simp_dist_matmul_i8_nsharded(dA.ptr, dB.ptr, dC.ptr, M, K, hi - lo, 1, 0))
        full = sd.assemble_column_blocks(dC.to_numpy(np.int32, (world, M, hi - lo)))
        assert np.array_equal(full, oracle.tensor_matmul_i8(A, B))
        # fused form: the epilogue writes every tile into every rank's row-major C (CUDA IPC peers)
        import ctypes as C
        # (2048, 4096, 8192): two waves of 256 x 256 tiles per rank; on 2 ranks the stores to the peer are paced
        for (M2, K2, N2) in ((256, 512, 1024), (1024, 2048, 4096), (300, 256, 96 * world), (2048, 4096, 8192)):
            A2 = rng.integers(0, 256, (M2, K2), dtype=np.uint8)
            B2 = rng.integers(-128, 128, (K2, N2), dtype=np.int8)
            lo2, hi2 = sd.column_shard(N2, world, rank)
            dA2 = sg.DeviceBuffer.from_numpy(A2)
            dB2 = sg.DeviceBuffer.from_numpy(np.ascontiguousarray(B2[:, lo2:hi2]))
            cptr = C.c_void_p()
            sg.check(sg.lib().simp_dist_symm_alloc(M2 * N2 * 4, C.byref(cptr)))
            sg.check(sg.lib().simp_gpu_memset(cptr, 0xff, M2 * N2 * 4))
            sg.check(sg.lib().simp_dist_barrier())
            sg.check(sg.lib().simp_dist_matmul_i8_nsharded_fused(dA2.ptr, dB2.ptr, cptr, M2, K2, hi2 - lo2, 1, 0))
            full2 = np.empty((M2, N2), np.int32)
            sg.check(sg.lib().simp_gpu_download(full2.ctypes.data, cptr, full2.nbytes))
            assert np.array_equal(full2, oracle.tensor_matmul_i8(A2, B2)), (M2, K2, N2)
            sg.check(sg.lib().simp_dist_barrier())
            sg.sync()
            dist.barrier()
            sg.check(sg.lib().simp_dist_symm_free(cptr))
        # a column block that is not a multiple of 32 columns would spill into the neighbour's block: refused
        cptr = C.c_void_p()
        sg.check(sg.lib().simp_dist_symm_alloc(256 * 48 * world * 4, C.byref(cptr)))
        rc = sg.lib().simp_dist_matmul_i8_nsharded_fused(dA.ptr, dB.ptr, cptr, 256, 512, 48, 1, 0)
        assert rc != 0 and b"multiples of 32" in sg.lib().simp_gpu_last_error()
        dist.barrier()
        sg.check(sg.lib().simp_dist_symm_free(cptr))
        np.save(os.path.join(out_dir, f"ok{rank}.npy"), np.array([1]))
        sg.check(sg.lib().simp_dist_shutdown())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_nsharded_gemm(gpu, tmp_path, world):
    import ctypes
    n = ctypes.c_int()
    gpu.check(gpu.lib().simp_gpu_device_count(ctypes.byref(n)))
    if n.value < world:
        pytest.skip(f"needs at least {world} GPUs")
    import torch.multiprocessing as mp
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all(os.path.exists(tmp_path / f"ok{r}.npy") for r in range(world))


def _tp_worker(rank, world, port, out_dir, which):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    import torch
    import torch.distributed as dist
    import oracle
    import simplang_b200 as sg
    from simplang_b200 import dist as sd, synth
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        sg.init(rank)
        sd.init_from_env(sg)
        if which == "tiny":
            cfg = dict(dim=256, hidden_dim=512, n_layers=3, n_heads=8, n_kv_heads=8, vocab_size=320, seq_len=64,
                       group_size=64)
            n_prompt, n_new = 4, 24
        elif which == "ragged":
            # per-rank row counts that are not whole 16-row tiles (as the 3B model's 8640 / 8 = 1080 hidden rows on 8
            # ranks): 2144 / 4 = 536 hidden rows and 88 classifier rows per rank
            cfg = dict(dim=512, hidden_dim=2144, n_layers=2, n_heads=8, n_kv_heads=8, vocab_size=88 * world, seq_len=64,
                       group_size=32)
            n_prompt, n_new = 4, 20
        else:
            cfg = synth.LLAMA_3B_W4
            n_prompt, n_new = 16, 16
        t, off = synth.llama_w4_tensors(cfg, 11, threads=8)
        prompt = synth.prompt_tokens(n_prompt, cfg["vocab_size"])
        m = sg.Llama(cfg, t, w4=True, offsets=off, tp_size=world)
        toks, trace, ms = m.generate(prompt, n_new, trace_logits=True)
        if rank == 0:
            om = oracle.Llama(cfg, t, w4=True, offsets={k + "_off": v for k, v in off.items()}, threads=0)
            tok, ref, worst = int(prompt[0]), [], 0.0
            for pos in range(n_prompt + n_new - 1):
                lg = om.forward(tok, pos)
                worst = max(worst, float(np.max(np.abs(trace[pos] - lg)) / np.max(np.abs(lg))))
                nxt = oracle.argmax(lg)
                tok = int(prompt[pos + 1]) if pos + 1 < n_prompt else nxt
                if pos + 1 >= n_prompt:
                    ref.append(nxt)
            assert worst <= 1e-3, worst
            assert list(toks) == ref
            print(f"TP{world} {which}: worst logit err {worst:.2e}, {(n_prompt + n_new - 1) / ms * 1e3:.0f} tok/s")
        allt = [None] * world
        dist.all_gather_object(allt, toks.tolist())
        assert all(a == allt[0] for a in allt)  # every rank generated the same sequence
        np.save(os.path.join(out_dir, f"tp_{which}_{rank}.npy"), np.array([1]))
        m.close()
        sg.check(sg.lib().simp_dist_shutdown())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("which,world", [("tiny", 2), ("ragged", 2), ("3b", 2), ("tiny", 4), ("ragged", 4), ("3b", 4)])
def test_tensor_parallel_w4_decode(gpu, tmp_path, which, world):
    import ctypes
    n = ctypes.c_int()
    gpu.check(gpu.lib().simp_gpu_device_count(ctypes.byref(n)))
    if n.value < world:
        pytest.skip(f"needs at least {world} GPUs")
    import torch.multiprocessing as mp
    mp.spawn(_tp_worker, args=(world, _free_port(), str(tmp_path), which), nprocs=world, join=True)
    assert all(os.path.exists(tmp_path / f"tp_{which}_{r}.npy") for r in range(world))
