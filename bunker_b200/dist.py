"""Process-group plumbing for the tensor-parallel path: one process per GPU, torch.distributed for the
rendezvous, barriers and the exchange of CUDA IPC handles.  No tensor of the decode path goes through it."""
from __future__ import annotations

import os

import numpy as np


def env_rank() -> tuple[int, int, int]:
    return (int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")),
            int(os.environ.get("LOCAL_RANK", os.environ.get("RANK", "0"))))


def init(backend: str | None = None):
    """Join the process group described by RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT.  Returns (rank, world)."""
    import torch
    import torch.distributed as dist
    rank, world, local = env_rank()
    if world == 1:
        return rank, world
    if not dist.is_initialized():
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        if backend == "nccl":
            torch.cuda.set_device(local)
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group(backend=backend, rank=rank, world_size=world)
    return rank, world


def _device():
    import torch
    import torch.distributed as dist
    return torch.device("cuda", torch.cuda.current_device()) if dist.get_backend() == "nccl" else torch.device("cpu")


def all_gather_bytes(payload: bytes) -> list[bytes]:
    """Every rank contributes len(payload) bytes (same length everywhere); returns them in rank order."""
    import torch
    import torch.distributed as dist
    if not dist.is_initialized():
        return [payload]
    dev = _device()
    mine = torch.tensor(list(payload), dtype=torch.uint8, device=dev)
    outs = [torch.empty_like(mine) for _ in range(dist.get_world_size())]
    dist.all_gather(outs, mine)
    return [bytes(o.cpu().numpy().tobytes()) for o in outs]


def barrier() -> None:
    import torch.distributed as dist
    if dist.is_initialized():
        dist.barrier()


def max_over_ranks(x: float) -> float:
    import torch
    import torch.distributed as dist
    if not dist.is_initialized():
        return x
    t = torch.tensor([x], dtype=torch.float64, device=_device())
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def shutdown() -> None:
    import torch.distributed as dist
    if dist.is_initialized():
        dist.destroy_process_group()
