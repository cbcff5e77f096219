"""SwiGLU activation on a packed ``[T, 2F]`` tensor holding ``[gate | up]``: out = silu(gate) * up.

One kernel forward, one kernel backward (recomputes the sigmoid; nothing but the packed input is
saved).  The reference runs HF's ``act_fn(gate_proj(x)) * up_proj(x)`` as separate ATen kernels.
"""
from __future__ import annotations

import torch

from .. import _lib


class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        T, F2 = gu.shape
        F = F2 // 2
        ctx.save_for_backward(gu)
        if gu.is_cuda:
            if gu.dtype != torch.bfloat16 or not gu.is_contiguous():
                raise TypeError("CUDA swiglu expects contiguous bf16")
            out = torch.empty(T, F, dtype=gu.dtype, device=gu.device)
            _lib.check(_lib.cuda().zc_swiglu_fwd(gu.data_ptr(), out.data_ptr(), T, F,
                                                 _lib.stream_ptr(gu.device)), "zc_swiglu_fwd")
            return out
        g, u = gu[:, :F].float(), gu[:, F:].float()
        return (torch.nn.functional.silu(g) * u).to(gu.dtype)

    @staticmethod
    def backward(ctx, dy):
        (gu,) = ctx.saved_tensors
        T, F2 = gu.shape
        F = F2 // 2
        if gu.is_cuda:
            dy = dy.contiguous()
            dgu = torch.empty_like(gu)
            _lib.check(_lib.cuda().zc_swiglu_bwd(gu.data_ptr(), dy.data_ptr(), dgu.data_ptr(), T, F,
                                                 _lib.stream_ptr(gu.device)), "zc_swiglu_bwd")
            return dgu
        g, u, d = gu[:, :F].float(), gu[:, F:].float(), dy.float()
        s = torch.sigmoid(g)
        dg = d * u * s * (1 + g * (1 - s))
        du = d * g * s
        return torch.cat([dg, du], dim=1).to(gu.dtype)


def swiglu(gu: torch.Tensor) -> torch.Tensor:
    return _SwiGLU.apply(gu)
