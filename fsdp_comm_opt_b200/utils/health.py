"""Host-side check of the device-side status words.

The fused kernels never trap or spin forever: a wait that runs out records a code in a status word
and the kernel returns.  ``check_device_status()`` reads every such word (this synchronises the
device, so call it where the loop synchronises anyway, e.g. next to ``loss.item()``) and raises.
"""
from __future__ import annotations

import torch


def check_device_status() -> None:
    if not torch.cuda.is_available():
        return
    from ..ops import attention
    from .. import _lib
    from ..parallel import symm_impl

    for ch in symm_impl.all_channels():
        ch.check_status()
    if attention.status_read_and_clear() != 0:
        raise RuntimeError("an attention kernel reported an expired bounded wait")
    if _lib.cuda().zc_gemm_status_read_and_clear() != 0:
        raise RuntimeError("the tcgen05 GEMM reported an expired bounded wait")
