"""Per-buffer absmax int8 quantisation used by ``QuantizedAllGather``.

Packed layout of one rank's contribution: ``[fp32 scale (4 B) | pad to 16 B | numel int8]``.
The reference packs ``[4 B scale | int8...]`` with torch ops (main/comm.py:37-58); the 16-byte
header here keeps the int8 payload aligned for 128-bit accesses.  Same arithmetic:
scale = max(absmax / 127, 1e-8), q = clamp(round_half_even(x / scale), -127, 127).
"""
from __future__ import annotations

import torch

from .. import _lib

HEADER = 16


def packed_bytes(numel: int) -> int:
    return HEADER + (numel + 15) // 16 * 16


def quantize_pack(x: torch.Tensor, out: torch.Tensor) -> None:
    """Quantise contiguous ``x`` into ``out`` (uint8, ``packed_bytes(x.numel())`` long)."""
    n = x.numel()
    if out.dtype != torch.uint8 or out.numel() < packed_bytes(n) or not out.is_contiguous():
        raise ValueError("out must be a contiguous uint8 buffer of packed_bytes(numel)")
    if x.is_cuda:
        code = {torch.bfloat16: 0, torch.float32: 1, torch.float16: 2}.get(x.dtype)
        if code is None:
            raise TypeError(f"unsupported dtype {x.dtype}")
        lib = _lib.cuda()
        _lib.check(lib.zc_quant_int8(x.data_ptr(), n, code, out.data_ptr(), _lib.stream_ptr(x.device)),
                   "zc_quant_int8")
        return
    xf = x.reshape(-1).float()
    scale = torch.clamp(xf.abs().max() / 127.0, min=1e-8)
    q = torch.clamp(torch.round(xf / scale), -127, 127).to(torch.int8)
    out[:4].copy_(scale.reshape(1).view(torch.uint8))
    out[4:HEADER].zero_()
    out[HEADER:HEADER + n].copy_(q.view(torch.uint8))


def dequantize_unpack(gathered: torch.Tensor, numel: int, out: torch.Tensor) -> None:
    """``gathered`` is ``[world, packed_bytes(numel)]`` uint8; ``out`` receives world*numel values."""
    world = gathered.shape[0]
    if out.numel() != world * numel:
        raise ValueError("out must hold world * numel elements")
    if gathered.is_cuda:
        code = {torch.bfloat16: 0, torch.float32: 1, torch.float16: 2}.get(out.dtype)
        if code is None or not out.is_contiguous():
            raise TypeError(f"unsupported output {out.dtype}")
        lib = _lib.cuda()
        _lib.check(lib.zc_dequant_int8(gathered.data_ptr(), gathered.stride(0), world, numel, code,
                                       out.data_ptr(), _lib.stream_ptr(out.device)), "zc_dequant_int8")
        return
    scales = gathered[:, :4].contiguous().view(torch.float32).view(world, 1)
    q = gathered[:, HEADER:HEADER + numel].contiguous().view(torch.int8).to(torch.float32)
    out.view(world, numel).copy_((q * scales).to(out.dtype))
