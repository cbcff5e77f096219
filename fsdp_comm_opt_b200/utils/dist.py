"""Process-group bring-up and small distributed helpers (reference: train.py:65-70, 386-394)."""
from __future__ import annotations

import os
from contextlib import contextmanager
from datetime import timedelta

import torch
import torch.distributed as dist


def init_distributed(device_type: str = "auto", timeout_s: float | None = None):
    """Reads RANK / WORLD_SIZE / LOCAL_RANK, picks cuda:local_rank (NCCL) or cpu (gloo), and
    initialises the default process group eagerly.  Returns ``(rank, world_size, device)``."""
    rank = int(os.getenv("RANK", "0"))
    world = int(os.getenv("WORLD_SIZE", "1"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29511")
    use_cuda = device_type == "cuda" or (device_type == "auto" and torch.cuda.is_available())
    kwargs = {}
    if timeout_s is not None:
        kwargs["timeout"] = timedelta(seconds=timeout_s)
    if use_cuda:
        local_rank = int(os.getenv("LOCAL_RANK", rank % max(torch.cuda.device_count(), 1)))
        device = torch.device(f"cuda:{local_rank}")
        torch.cuda.set_device(device)
        if not dist.is_initialized():
            dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device, **kwargs)
    else:
        device = torch.device("cpu")
        if not dist.is_initialized():
            dist.init_process_group("gloo", rank=rank, world_size=world, **kwargs)
    return rank, world, device


@contextmanager
def rank0_first():
    """Rank 0 runs the body, then everyone else (e.g. to fill a shared cache once)."""
    rank = dist.get_rank() if dist.is_initialized() else 0
    if rank == 0:
        yield
    if dist.is_initialized():
        dist.barrier()
    if rank > 0:
        yield
    if dist.is_initialized():
        dist.barrier()


def all_reduce_max(value: float, device) -> float:
    """MAX over ranks of a host scalar (used for device-timed metrics)."""
    if not dist.is_initialized() or dist.get_world_size() == 1:
        return value
    t = torch.tensor([value], dtype=torch.float64, device=device if device.type == "cuda" else "cpu")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())
