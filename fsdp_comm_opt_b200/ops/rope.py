"""Rotary position embedding applied in place to the q and k heads of a packed qkv tensor.

Pairing is "rotate half": element i of a head pairs with element i + D/2 (the Llama convention
of HF ``apply_rotary_pos_emb``, which the reference inherits through ``AutoModelForCausalLM``).
The backward pass is the same rotation with the sine negated.
"""
from __future__ import annotations

import torch

from .. import _lib


_TABLES: dict = {}


def cached_tables(seq_len: int, head_dim: int, theta: float, device) -> tuple[torch.Tensor, torch.Tensor]:
    """fp32 cos/sin tables, cached per (seq_len, head_dim, theta, device).  Modules fetch them here
    instead of receiving them as forward arguments: FSDP2's mixed-precision policy casts floating
    point forward inputs to the parameter dtype, which would silently turn the tables into bf16."""
    key = (int(seq_len), int(head_dim), float(theta), str(device))
    t = _TABLES.get(key)
    if t is None:
        if len(_TABLES) > 16:
            _TABLES.clear()
        t = _TABLES[key] = rope_tables(seq_len, head_dim, theta, device)
    return t


def rope_tables(seq_len: int, head_dim: int, theta: float, device) -> tuple[torch.Tensor, torch.Tensor]:
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32, device=device) / head_dim))
    t = torch.arange(seq_len, dtype=torch.float32, device=device)
    ang = torch.outer(t, inv)
    return ang.cos().contiguous(), ang.sin().contiguous()


def _rotate(qkv: torch.Tensor, cos, sin, n_rot_heads: int, head_dim: int, seq_len: int, sign: float):
    """qkv: [T, H_total*D] contiguous, token t sits at position t % seq_len."""
    T = qkv.shape[0]
    total_heads = qkv.shape[1] // head_dim
    if cos.dtype != torch.float32 or sin.dtype != torch.float32 or cos.shape != (seq_len, head_dim // 2):
        raise TypeError("rope tables must be fp32 [seq_len, head_dim/2]")
    if qkv.is_cuda:
        if qkv.dtype != torch.bfloat16 or not qkv.is_contiguous():
            raise TypeError("CUDA rope expects contiguous bf16")
        cos, sin = cos.contiguous(), sin.contiguous()
        _lib.check(_lib.cuda().zc_rope_inplace(
            qkv.data_ptr(), cos.data_ptr(), sin.data_ptr(), T, seq_len, n_rot_heads, total_heads,
            head_dim, float(sign), _lib.stream_ptr(qkv.device)), "zc_rope_inplace")
        return qkv
    half = head_dim // 2
    v = qkv.view(T // seq_len, seq_len, total_heads, head_dim)
    rot = v[:, :, :n_rot_heads].float()
    c = cos[None, :, None, :]
    s = sin[None, :, None, :] * sign
    a, b = rot[..., :half], rot[..., half:]
    out = torch.cat([a * c - b * s, b * c + a * s], dim=-1)
    v[:, :, :n_rot_heads] = out.to(qkv.dtype)
    return qkv


def apply_rope(qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, n_rot_heads: int,
               head_dim: int, seq_len: int) -> torch.Tensor:
    """Out-of-place, differentiable form for standalone use: returns a rotated copy of ``qkv``
    ``[T, H*D]``.  Inside the models the rotation is fused into the attention op instead."""
    return _Rope.apply(qkv, cos, sin, n_rot_heads, head_dim, seq_len)


class _Rope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, cos, sin, n_rot_heads, head_dim, seq_len):
        ctx.save_for_backward(cos, sin)
        ctx.meta = (n_rot_heads, head_dim, seq_len)
        return _rotate(qkv.detach().contiguous().clone(), cos, sin, n_rot_heads, head_dim, seq_len, 1.0)

    @staticmethod
    def backward(ctx, dout):
        cos, sin = ctx.saved_tensors
        n_rot_heads, head_dim, seq_len = ctx.meta
        return _rotate(dout.contiguous().clone(), cos, sin, n_rot_heads, head_dim, seq_len, -1.0), None, None, None, None, None
