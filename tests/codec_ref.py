"""Pure-PyTorch restatement of the v1 codec math, independent of the C++ codec.

Used as a second oracle: the scalar C++ codec and the CUDA kernels must both agree with it.
Split layout only (the fused layout is the same fields in a different order).
"""
import torch

BLOCK = 4096


def split_fields(x_bf16: torch.Tensor):
    v = x_bf16.view(torch.int16).to(torch.int32) & 0xFFFF
    sm = ((v >> 8) & 0x80) | (v & 0x7F)
    e = (v >> 7) & 0xFF
    return sm.to(torch.uint8), e


def encode_work(x_bf16: torch.Tensor, base: int):
    """x: 1-D bf16 with numel % 4096 == 0.  Returns dict of sm, planes (3 x N/32 int32),
    block_off (nb), outliers (uint8)."""
    n = x_bf16.numel()
    assert n % BLOCK == 0
    sm, e = split_fields(x_bf16)
    inwin = (e >= base) & (e < base + 7)
    code = torch.where(inwin, e - base + 1, torch.zeros_like(e))
    bits = code.view(n // 32, 32)
    weights = (1 << torch.arange(32, dtype=torch.int64))
    planes = []
    for p in range(3):
        w = (((bits >> p) & 1).to(torch.int64) * weights).sum(1)
        planes.append(w.to(torch.int64))
    esc_mask = code == 0
    outliers = e[esc_mask].to(torch.uint8)
    per_block = esc_mask.view(n // BLOCK, BLOCK).sum(1)
    block_off = torch.cumsum(per_block, 0) - per_block
    return dict(sm=sm, planes=planes, block_off=block_off.to(torch.int32), outliers=outliers)


def det_stream(fields, n: int, base: int) -> torch.Tensor:
    nb = n // BLOCK
    size = (n + n // 8 * 3 + nb * 4 + 4 + 127) // 128 * 128
    out = torch.zeros(size, dtype=torch.uint8)
    out[:n] = fields["sm"]
    off = n
    for p in range(3):
        w = fields["planes"][p]
        w32 = torch.where(w >= 2 ** 31, w - 2 ** 32, w).to(torch.int32)
        out[off:off + n // 8] = w32.view(torch.uint8)
        off += n // 8
    out[off:off + 4 * nb] = fields["block_off"].view(torch.uint8)
    off += 4 * nb
    out[off:off + 4] = torch.tensor([base], dtype=torch.int32).view(torch.uint8)
    return out
