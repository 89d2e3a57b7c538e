"""Host-side helpers for the multi-GPU paths: shard arithmetic, assembling gathered blocks, and the
rendezvous that carries the NCCL unique id from rank 0 to the other ranks over ``torch.distributed``
(any backend: ``nccl`` on GPUs, ``gloo`` in CPU tests).  The collectives themselves run inside
``libsimp_gpu.so`` (``simp_dist_*``)."""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

ID_BYTES = 128


def column_shard(n: int, world: int, rank: int, multiple: int = 16):
    """Half-open column range [lo, hi) of rank's block when n columns are split evenly over `world` ranks.
    Every block has the same width (the all-gather needs equal counts) and that width must be a multiple of
    `multiple` (16 bytes of int8 = what a TMA row needs)."""
    if n % world != 0 or (n // world) % multiple != 0:
        raise ValueError(f"{n} columns do not split into {world} blocks that are multiples of {multiple}")
    w = n // world
    return rank * w, (rank + 1) * w


def assemble_column_blocks(blocks: np.ndarray) -> np.ndarray:
    """[world, M, n_local] gathered column blocks -> the row-major [M, world*n_local] matrix."""
    world, m, nl = blocks.shape
    return np.ascontiguousarray(blocks.transpose(1, 0, 2).reshape(m, world * nl))


def row_shard(rows: int, world: int, rank: int):
    """Row range of rank's shard for the column-parallel projections of tensor-parallel decode."""
    if rows % world != 0:
        raise ValueError(f"{rows} rows do not split evenly over {world} ranks")
    w = rows // world
    return rank * w, (rank + 1) * w


def exchange_unique_id(make_id, rank: int, world: int) -> bytes:
    """Rank 0 calls make_id() -> bytes; every rank returns the same bytes.  Uses the default process group."""
    import torch
    import torch.distributed as dist
    buf = torch.zeros(ID_BYTES, dtype=torch.uint8)
    if rank == 0:
        raw = make_id()
        assert len(raw) == ID_BYTES
        buf = torch.frombuffer(bytearray(raw), dtype=torch.uint8).clone()
    if world > 1:
        backend = dist.get_backend()
        if backend == "nccl":
            buf = buf.cuda()
        dist.broadcast(buf, src=0)
        buf = buf.cpu()
    return bytes(buf.numpy().tobytes())


def init_from_env(sg):
    """Initialises the library's communicator from RANK / WORLD_SIZE / LOCAL_RANK (torchrun).  Requires an
    initialised torch.distributed default group when WORLD_SIZE > 1.  Returns (rank, world)."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    def make_id():
        b = (C.c_uint8 * ID_BYTES)()
        sg.check(sg.lib().simp_dist_unique_id(b, ID_BYTES))
        return bytes(b)

    uid = exchange_unique_id(make_id, rank, world) if world > 1 else bytes(ID_BYTES)
    ub = (C.c_uint8 * ID_BYTES).from_buffer_copy(uid)
    sg.check(sg.lib().simp_dist_init(rank, world, ub, ID_BYTES))
    return rank, world
