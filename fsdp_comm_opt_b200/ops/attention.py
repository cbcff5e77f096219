"""Causal grouped-query attention, forward and backward.

Layout: one packed projection ``[B, S, Hq + 2*Hkv, D]`` (q heads, then k heads, then v heads),
output ``[B, S, Hq, D]`` contiguous; the backward returns one packed gradient of the same shape,
so the qkv projection's backward reads it without a concatenation.
CUDA tensors run the sm_100a flash-style kernels (``zc_attn_fwd_2q`` / ``zc_attn_bwd_kt`` for head
dimension 128, ``zc_attn_fwd_ws`` / ``zc_attn_bwd_ws`` for 64: online softmax, log-sum-exp saved for
the backward, no S x S tensor in memory); CPU tensors run fp32 matmul/softmax.  The reference reaches PyTorch SDPA through HF attention modules.
"""
from __future__ import annotations

import math
import os

import torch

from .. import _lib


_FWD_IMPL = os.environ.get("ZC_ATTN_FWD", "2q")
_BWD_IMPL = os.environ.get("ZC_ATTN_BWD", "kt")


def status_read_and_clear() -> int:
    """Non-zero when a bounded wait inside an attention kernel expired since the last call
    (synchronises the device)."""
    lib = _lib.cuda()
    return (int(lib.zc_attn_status_read_and_clear()) | int(lib.zc_attn_ws_status_read_and_clear())
            | int(lib.zc_attn_bwd_ws_status_read_and_clear()) | int(lib.zc_attn_fwd_2q_status_read_and_clear()))


def _strides(t):
    return t.stride(0), t.stride(1), t.stride(2)


def _ref_attention(q, k, v, scale):
    B, S, Hq, D = q.shape
    Hkv = k.shape[2]
    g = Hq // Hkv
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(g, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(g, dim=1)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    mask = torch.ones(S, S, dtype=torch.bool, device=q.device).tril()
    s = s.masked_fill(~mask, float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.matmul(p, vf).permute(0, 2, 1, 3)


class _Attention(torch.autograd.Function):
    """Attention over a packed ``[B, S, Hq + 2*Hkv, D]`` projection (q heads, k heads, v heads)."""

    @staticmethod
    def forward(ctx, qkv, Hq, Hkv, scale, cos, sin):
        B, S, Ht, D = qkv.shape
        ctx.heads = (Hq, Hkv)
        ctx.scale = scale
        ctx.rope = (cos, sin)
        if cos is not None:
            # rotate q and k heads in place in the projection's output buffer; the projection's
            # backward never reads its own output, so autograd does not need to know
            from .rope import _rotate

            if not qkv.is_contiguous():
                raise ValueError("packed qkv must be contiguous when RoPE is fused")
            _rotate(qkv.detach().view(B * S, Ht * D), cos, sin, Hq + Hkv, D, S, 1.0)
        q, k, v = qkv[:, :, :Hq], qkv[:, :, Hq:Hq + Hkv], qkv[:, :, Hq + Hkv:]
        if not qkv.is_cuda:
            with torch.enable_grad():
                packed = qkv.detach().requires_grad_(True)
                o = _ref_attention(packed[:, :, :Hq], packed[:, :, Hq:Hq + Hkv], packed[:, :, Hq + Hkv:], scale)
            ctx.cpu_graph = (packed, o)
            return o.detach().to(qkv.dtype).contiguous()
        if qkv.dtype != torch.bfloat16 or D not in (64, 128) or qkv.stride(3) != 1:
            raise TypeError("CUDA attention expects bf16, head_dim 64 or 128, contiguous heads")
        o = torch.empty(B, S, Hq, D, dtype=qkv.dtype, device=qkv.device)
        lse = torch.empty(B, Hq, S, dtype=torch.float32, device=qkv.device)
        lib = _lib.cuda()
        # default: two query tiles per CTA, one softmax thread per row; ZC_ATTN_FWD=ws / simple select
        # the earlier warp-specialised and single-role kernels
        fwd = {"simple": lib.zc_attn_fwd, "ws": lib.zc_attn_fwd_ws}.get(_FWD_IMPL, lib.zc_attn_fwd_2q)
        _lib.check(fwd(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(), B, S, Hq, Hkv, D,
            *_strides(q), *_strides(k), *_strides(v), float(scale), _lib.stream_ptr(qkv.device)),
            "zc_attn_fwd")
        ctx.save_for_backward(qkv, o, lse)
        return o

    @staticmethod
    def backward(ctx, do):
        Hq, Hkv = ctx.heads
        if getattr(ctx, "cpu_graph", None) is not None:
            packed, o = ctx.cpu_graph
            (dqkv,) = torch.autograd.grad(o, (packed,), do.float())
            dqkv = dqkv.to(do.dtype).contiguous()
            ctx.cpu_graph = None
            return _Attention._unrope(ctx, dqkv), None, None, None, None, None
        qkv, o, lse = ctx.saved_tensors
        B, S, Ht, D = qkv.shape
        q, k, v = qkv[:, :, :Hq], qkv[:, :, Hq:Hq + Hkv], qkv[:, :, Hq + Hkv:]
        do = do.contiguous()
        dqkv = torch.empty_like(qkv)
        dq, dk, dv = dqkv[:, :, :Hq], dqkv[:, :, Hq:Hq + Hkv], dqkv[:, :, Hq + Hkv:]
        delta = torch.empty(B, Hq, S, dtype=torch.float32, device=qkv.device)
        lib = _lib.cuda()
        # default: key-row kernel (64-query iterations, pipelined); ZC_ATTN_BWD=ws / simple select
        # the earlier warp-specialised and single-role kernels
        bwd = {"simple": lib.zc_attn_bwd, "ws": lib.zc_attn_bwd_ws}.get(_BWD_IMPL, lib.zc_attn_bwd_kt)
        _lib.check(bwd(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), do.data_ptr(), lse.data_ptr(),
            delta.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), B, S, Hq, Hkv, D,
            *_strides(q), *_strides(k), *_strides(v), *_strides(dq), *_strides(dk), *_strides(dv),
            float(ctx.scale), _lib.stream_ptr(qkv.device)), "zc_attn_bwd")
        return _Attention._unrope(ctx, dqkv), None, None, None, None, None

    @staticmethod
    def _unrope(ctx, dqkv):
        cos, sin = ctx.rope
        if cos is not None:
            from .rope import _rotate

            Hq, Hkv = ctx.heads
            B, S, Ht, D = dqkv.shape
            _rotate(dqkv.view(B * S, Ht * D), cos, sin, Hq + Hkv, D, S, -1.0)
        return dqkv


def causal_attention(qkv: torch.Tensor, n_q_heads: int, n_kv_heads: int, scale: float | None = None,
                     rope_cos: torch.Tensor | None = None, rope_sin: torch.Tensor | None = None) -> torch.Tensor:
    """``qkv`` is ``[B, S, n_q_heads + 2*n_kv_heads, D]``; returns ``[B, S, n_q_heads, D]``.

    With ``rope_cos``/``rope_sin`` (``[S, D/2]`` fp32) the rotary embedding is applied to the q and
    k heads first, in place in ``qkv``, and undone on the gradient in the backward pass.
    """
    if scale is None:
        scale = 1.0 / math.sqrt(qkv.shape[-1])
    return _Attention.apply(qkv, n_q_heads, n_kv_heads, scale, rope_cos, rope_sin)
