"""Host-side check of the device-side status words.

The fused kernels never trap or spin forever: a wait that runs out records a code in a status word
and the kernel returns.  ``check_device_status()`` reads every such word (this synchronises the
device, so call it where the loop synchronises anyway, e.g. next to ``loss.item()``) and raises.
"""
from __future__ import annotations

import torch


def check_device_status(deep: bool = False) -> None:
    """``deep`` also reads back the canary regions around the symmetric staging buffers (a few small
    device reads per channel: for checkpoints and log lines, not for every step)."""
    if not torch.cuda.is_available():
        return
    from ..ops import attention
    from .. import _lib
    from ..parallel import symm_impl

    health = _lib.cuda().zc_health_read_and_clear()  # cleared first: the channel checks below may raise
    for ch in symm_impl.all_channels():
        ch.check_status()
        if deep:
            ch.check_canaries()
    if health != 0:
        raise RuntimeError("the device health word was set (a fused collective gave up) but no channel reported it")
    if attention.status_read_and_clear() != 0:
        raise RuntimeError("an attention kernel reported an expired bounded wait")
    if _lib.cuda().zc_gemm_status_read_and_clear() != 0:
        raise RuntimeError("the tcgen05 GEMM reported an expired bounded wait")
