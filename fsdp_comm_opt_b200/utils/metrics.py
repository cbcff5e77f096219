"""Logging set-up and memory statistics (reference: train.py:72-79, 374-383)."""
from __future__ import annotations

import logging

import torch


def setup_logging(rank: int, level=logging.INFO) -> logging.Logger:
    logging.basicConfig(format=f"[rank={rank}] [%(asctime)s] %(levelname)s:%(message)s", level=level, force=True)
    return logging.getLogger("fsdp_comm_opt_b200")


def get_mem_stats(device=None) -> dict:
    if device is None or torch.device(device).type != "cuda" or not torch.cuda.is_available():
        return {k: 0.0 for k in ("total_gb", "curr_alloc_gb", "peak_alloc_gb", "curr_resv_gb", "peak_resv_gb")}
    mem = torch.cuda.memory_stats(device)
    props = torch.cuda.get_device_properties(device)
    return {
        "total_gb": 1e-9 * props.total_memory,
        "curr_alloc_gb": 1e-9 * mem["allocated_bytes.all.current"],
        "peak_alloc_gb": 1e-9 * mem["allocated_bytes.all.peak"],
        "curr_resv_gb": 1e-9 * mem["reserved_bytes.all.current"],
        "peak_resv_gb": 1e-9 * mem["reserved_bytes.all.peak"],
    }
