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


class PeerLost(RuntimeError):
    """A tensor-parallel peer has left (or stopped answering) between two steps."""


class StepGate:
    """Host-side liveness check between decode steps, over the process group's key-value store.

    A tensor-parallel step exchanges partial sums with every peer on the device; a rank that is gone would leave the
    others waiting on the device until their bounded waits give up.  The gate moves that discovery to the host and
    before the launch: every rank posts `gate/<step>/<rank>` and then looks for the same key of its peers; a rank
    that leaves on purpose posts `left/<rank>` first.  A missing key after `timeout_s`, or a `left` key, raises
    PeerLost -- an error code path, never a hang and never a GPU fault.  A rank leaves only between steps, with none
    of its kernels in flight."""

    def __init__(self, store=None, rank: int | None = None, world: int | None = None, poll_s: float = 0.005):
        import torch.distributed as dist
        if store is None:
            from torch.distributed.distributed_c10d import _get_default_store
            store = _get_default_store()
        self.store = store
        self.rank = dist.get_rank() if rank is None else rank
        self.world = dist.get_world_size() if world is None else world
        self.poll_s = poll_s

    def leave(self) -> None:
        self.store.set(f"left/{self.rank}", b"1")

    def arrive(self, step: int, timeout_s: float = 5.0) -> None:
        import time
        self.store.set(f"gate/{step}/{self.rank}", b"1")
        deadline = time.monotonic() + timeout_s
        for r in range(self.world):
            if r == self.rank:
                continue
            while not self.store.check([f"gate/{step}/{r}"]):
                if self.store.check([f"left/{r}"]):
                    raise PeerLost(f"rank {r} left before step {step}")
                if time.monotonic() > deadline:
                    raise PeerLost(f"rank {r} did not reach step {step} within {timeout_s} s")
                time.sleep(self.poll_s)


def shutdown() -> None:
    import torch.distributed as dist
    if dist.is_initialized():
        dist.destroy_process_group()
