"""CPU tests of the multi-GPU host logic with world_size 2 over gloo: shard arithmetic, the unique-id
rendezvous, and the N-sharded GEMM emulated per rank with the oracle (each rank multiplies A by its column
block of B; the gathered blocks must assemble to the unsharded product, bit for bit)."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    import oracle
    from simplang_b200 import dist as sd
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        uid = sd.exchange_unique_id(lambda: bytes(range(128)), rank, world)
        assert uid == bytes(range(128))
        M, K, N = 48, 64, 96
        rng = np.random.default_rng(7)  # same seed on every rank: A replicated, B sliced
        A = rng.integers(0, 256, (M, K), dtype=np.uint8)
        B = rng.integers(-128, 128, (K, N), dtype=np.int8)
        lo, hi = sd.column_shard(N, world, rank)
        mine = oracle.tensor_matmul_i8(A, np.ascontiguousarray(B[:, lo:hi]), threads=1)
        gathered = [torch.empty((M, hi - lo), dtype=torch.int32) for _ in range(world)]
        dist.all_gather(gathered, torch.from_numpy(mine))
        full = sd.assemble_column_blocks(np.stack([g.numpy() for g in gathered]))
        assert np.array_equal(full, oracle.tensor_matmul_i8(A, B, threads=1))
        np.save(os.path.join(out_dir, f"ok{rank}.npy"), np.array([1]))
    finally:
        dist.destroy_process_group()


def test_world2_gloo(tmp_path):
    import torch.multiprocessing as mp
    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert all(os.path.exists(tmp_path / f"ok{r}.npy") for r in range(2))


def test_shard_arithmetic():
    from simplang_b200 import dist as sd
    assert sd.column_shard(8192, 8, 3) == (3072, 4096)
    assert sd.row_shard(8640, 8, 7) == (7560, 8640)
    with pytest.raises(ValueError):
        sd.column_shard(100, 8, 0)
    with pytest.raises(ValueError):
        sd.column_shard(8 * 24, 8, 0)  # 24 columns per rank: not a multiple of 16
    blocks = np.arange(2 * 3 * 4).reshape(2, 3, 4)
    full = sd.assemble_column_blocks(blocks)
    assert full.shape == (3, 8) and full[1, 5] == blocks[1, 1, 1]
