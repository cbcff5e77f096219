"""Symmetric-memory channels for the fused collective kernels (filled in by ``symm_impl``)."""
from __future__ import annotations

import os

import torch


def available(group) -> bool:
    """True when the fused symmetric-memory transport can be used for ``group``."""
    if os.environ.get("ZC_DISABLE_SYMM", "0") == "1" or not torch.cuda.is_available():
        return False
    try:
        from . import symm_impl
    except ImportError:
        return False
    return symm_impl.available(group)


def channel_for(group, device, kind: str):
    from . import symm_impl

    return symm_impl.channel_for(group, device, kind)
