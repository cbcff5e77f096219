"""RMSNorm (optionally fused with the preceding residual add) as an autograd function.

CUDA tensors run the sm_100a kernels ``zc_rmsnorm_fwd`` / ``zc_rmsnorm_bwd``; CPU tensors run
the same arithmetic in fp32 PyTorch.  The reference gets RMSNorm from HF ``LlamaRMSNorm`` (five
ATen elementwise/reduction kernels per call, reference: train.py:35, 48).
"""
from __future__ import annotations

import torch

from .. import _lib


def _use_cuda(x: torch.Tensor) -> bool:
    return x.is_cuda


class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, eps, residual):
        shape = x.shape
        cols = shape[-1]
        x2 = x.reshape(-1, cols)
        rows = x2.shape[0]
        if _use_cuda(x):
            if x.dtype != torch.bfloat16:
                raise TypeError("CUDA rms_norm expects bf16 activations")
            x2 = x2.contiguous()
            w = weight.to(torch.bfloat16).contiguous()
            y = torch.empty_like(x2)
            rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
            if residual is not None:
                r2 = residual.reshape(-1, cols).contiguous()
                h = torch.empty_like(x2)
            else:
                r2, h = None, x2
            _lib.check(_lib.cuda().zc_rmsnorm_fwd(
                x2.data_ptr(), _lib.ptr(r2), w.data_ptr(), y.data_ptr(),
                h.data_ptr() if residual is not None else None, rstd.data_ptr(), rows, cols,
                float(eps), _lib.stream_ptr(x.device)), "zc_rmsnorm_fwd")
        else:
            h = x2 if residual is None else (x2.float() + residual.reshape(-1, cols).float()).to(x.dtype)
            hf = h.float()
            rstd = torch.rsqrt(hf.pow(2).mean(-1) + eps)
            y = (hf * rstd[:, None] * weight.float()).to(x.dtype)
            w = weight
        ctx.save_for_backward(h, w, rstd)
        ctx.has_residual = residual is not None
        ctx.shape = shape
        ctx.wdtype = weight.dtype
        if residual is not None:
            return y.view(shape), h.view(shape)
        return y.view(shape), None

    @staticmethod
    def backward(ctx, dy, dh_out):
        h, w, rstd = ctx.saved_tensors
        rows, cols = h.shape
        dy2 = dy.reshape(rows, cols)
        if _use_cuda(h):
            dy2 = dy2.contiguous()
            dx = torch.empty_like(h)
            lib = _lib.cuda()
            dw32 = torch.empty(cols, dtype=torch.float32, device=h.device)
            # one row of partial column sums per CTA, summed by a second small kernel
            partials = torch.empty(int(lib.zc_rmsnorm_bwd_ctas(rows)), cols, dtype=torch.float32, device=h.device)
            dh2 = dh_out.reshape(rows, cols).contiguous() if dh_out is not None else None
            _lib.check(lib.zc_rmsnorm_bwd(
                dy2.data_ptr(), h.data_ptr(), w.data_ptr(), rstd.data_ptr(), _lib.ptr(dh2),
                dx.data_ptr(), dw32.data_ptr(), partials.data_ptr(), rows, cols, _lib.stream_ptr(h.device)),
                "zc_rmsnorm_bwd")
            dw = dw32.to(ctx.wdtype)
        else:
            hf, dyf, wf = h.float(), dy2.float(), w.float()
            xhat = hf * rstd[:, None]
            g = dyf * wf
            dxf = rstd[:, None] * (g - xhat * (g * xhat).mean(-1, keepdim=True))
            if dh_out is not None:
                dxf = dxf + dh_out.reshape(rows, cols).float()
            dx = dxf.to(h.dtype)
            dw = (dyf * xhat).sum(0).to(ctx.wdtype)
        dx = dx.view(ctx.shape)
        return dx, dw, None, (dx if ctx.has_residual else None)


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    y, _ = _RMSNorm.apply(x, weight, eps, None)
    return y


def add_rms_norm(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, eps: float = 1e-5):
    """Returns ``(rms_norm(x + residual), x + residual)`` from one kernel."""
    y, h = _RMSNorm.apply(x, weight, eps, residual)
    return y, h
