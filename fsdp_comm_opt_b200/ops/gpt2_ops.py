"""LayerNorm and fused bias + tanh-GELU for the GPT-2 decoder family, as autograd functions.

CUDA tensors (bf16) run the sm_100a kernels of ``csrc/gpt2_ops.cu``; CPU tensors run the same
arithmetic in fp32 PyTorch.  The reference gets these ops from HF ``GPT2Block`` (ATen LayerNorm,
``NewGELUActivation`` and separate bias adds: about ten elementwise kernels per MLP).
"""
from __future__ import annotations

import math

import torch

from .. import _lib

_K = math.sqrt(2.0 / math.pi)
_C = 0.044715


class _LayerNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, eps):
        shape = x.shape
        cols = shape[-1]
        x2 = x.reshape(-1, cols)
        rows = x2.shape[0]
        if x.is_cuda:
            if x.dtype != torch.bfloat16:
                raise TypeError("CUDA layer_norm expects bf16 activations")
            x2 = x2.contiguous()
            w = weight.to(torch.bfloat16).contiguous()
            b = bias.to(torch.bfloat16).contiguous()
            y = torch.empty_like(x2)
            mean = torch.empty(rows, dtype=torch.float32, device=x.device)
            rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
            _lib.check(_lib.cuda().zc_layernorm_fwd(
                x2.data_ptr(), w.data_ptr(), b.data_ptr(), y.data_ptr(), mean.data_ptr(), rstd.data_ptr(), rows, cols,
                float(eps), _lib.stream_ptr(x.device)), "zc_layernorm_fwd")
        else:
            xf = x2.float()
            mean = xf.mean(-1)
            rstd = torch.rsqrt((xf - mean[:, None]).pow(2).mean(-1) + eps)
            y = ((xf - mean[:, None]) * rstd[:, None] * weight.float() + bias.float()).to(x.dtype)
            w = weight
        ctx.save_for_backward(x2, w, mean, rstd)
        ctx.shape = shape
        ctx.dtypes = (weight.dtype, bias.dtype)
        return y.view(shape)

    @staticmethod
    def backward(ctx, dy):
        x2, w, mean, rstd = ctx.saved_tensors
        rows, cols = x2.shape
        dy2 = dy.reshape(rows, cols)
        if x2.is_cuda:
            lib = _lib.cuda()
            dy2 = dy2.contiguous()
            dx = torch.empty_like(x2)
            dwdb = torch.empty(2, cols, dtype=torch.float32, device=x2.device)
            partials = torch.empty(int(lib.zc_layernorm_bwd_ctas(rows)), 2, cols, dtype=torch.float32, device=x2.device)
            _lib.check(lib.zc_layernorm_bwd(
                dy2.data_ptr(), x2.data_ptr(), w.data_ptr(), mean.data_ptr(), rstd.data_ptr(), dx.data_ptr(),
                dwdb.data_ptr(), partials.data_ptr(), rows, cols, _lib.stream_ptr(x2.device)), "zc_layernorm_bwd")
            dw, db = dwdb[0].to(ctx.dtypes[0]), dwdb[1].to(ctx.dtypes[1])
        else:
            xf, dyf = x2.float(), dy2.float()
            xhat = (xf - mean[:, None]) * rstd[:, None]
            g = dyf * w.float()
            dxf = rstd[:, None] * (g - g.mean(-1, keepdim=True) - xhat * (g * xhat).mean(-1, keepdim=True))
            dx = dxf.to(x2.dtype)
            dw = (dyf * xhat).sum(0).to(ctx.dtypes[0])
            db = dyf.sum(0).to(ctx.dtypes[1])
        return dx.view(ctx.shape), dw, db, None


def layer_norm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    """LayerNorm over the last dimension with weight and bias."""
    return _LayerNorm.apply(x, weight, bias, eps)


def _gelu_ref(a: torch.Tensor):
    t = torch.tanh(_K * (a + _C * a.pow(3)))
    return 0.5 * a * (1.0 + t), t


class _BiasGelu(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, bias):
        shape = x.shape
        cols = shape[-1]
        x2 = x.reshape(-1, cols)
        if x.is_cuda:
            if x.dtype != torch.bfloat16:
                raise TypeError("CUDA bias_gelu expects bf16 activations")
            x2 = x2.contiguous()
            b = bias.to(torch.bfloat16).contiguous()
            y = torch.empty_like(x2)
            _lib.check(_lib.cuda().zc_bias_gelu_fwd(x2.data_ptr(), b.data_ptr(), y.data_ptr(), x2.shape[0], cols,
                                                    _lib.stream_ptr(x.device)), "zc_bias_gelu_fwd")
        else:
            b = bias
            y = _gelu_ref(x2.float() + bias.float())[0].to(x.dtype)
        ctx.save_for_backward(x2, b)
        ctx.shape = shape
        ctx.bdtype = bias.dtype
        return y.view(shape)

    @staticmethod
    def backward(ctx, dy):
        x2, b = ctx.saved_tensors
        rows, cols = x2.shape
        dy2 = dy.reshape(rows, cols)
        if x2.is_cuda:
            dy2 = dy2.contiguous()
            dx = torch.empty_like(x2)
            _lib.check(_lib.cuda().zc_bias_gelu_bwd(x2.data_ptr(), b.data_ptr(), dy2.data_ptr(), dx.data_ptr(), rows,
                                                    cols, _lib.stream_ptr(x2.device)), "zc_bias_gelu_bwd")
        else:
            a = x2.float() + b.float()
            _, t = _gelu_ref(a)
            dt = (1.0 - t * t) * _K * (1.0 + 3.0 * _C * a * a)
            dx = (dy2.float() * (0.5 * (1.0 + t) + 0.5 * a * dt)).to(x2.dtype)
        db = dx.float().sum(0).to(ctx.bdtype)
        return dx.view(ctx.shape), db


def bias_gelu(x: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """``gelu_tanh(x + bias)`` with ``bias`` broadcast over the last dimension."""
    return _BiasGelu.apply(x, bias)
