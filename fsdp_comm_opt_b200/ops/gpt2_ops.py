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


def _grad_target(param: torch.Tensor, cols: int):
    """Where a kernel can write the gradient of a small parameter directly: ``param.main_grad`` (the
    view of a sharded engine's flat gradient buffer) when it is a contiguous bf16 or fp32 vector.
    Returns ``(tensor, accumulate)`` or ``(None, False)``."""
    mg = getattr(param, "main_grad", None)
    if (mg is None or not mg.is_cuda or mg.dtype not in (torch.bfloat16, torch.float32) or mg.numel() != cols
            or not mg.is_contiguous() or mg.data_ptr() % 8):
        return None, False
    return mg, bool(getattr(param, "main_grad_written", False))


def bias_grad(dy2: torch.Tensor, bias: torch.Tensor):
    """Gradient of a bias added to every row of a ``[rows, cols]`` bf16 output whose gradient is ``dy2``:
    its column sums (fp32 accumulation), written into ``bias.main_grad`` when the parameter has one
    (returns None then), else returned in the bias's dtype."""
    rows, cols = dy2.shape
    if not dy2.is_cuda:
        return dy2.float().sum(0).to(bias.dtype)
    lib = _lib.cuda()
    if dy2.stride(1) != 1 or dy2.stride(0) % 8 or cols % 8 or dy2.data_ptr() % 16:
        dy2 = dy2.contiguous()
    target, acc = _grad_target(bias, cols)
    out = target if target is not None else torch.empty(cols, dtype=torch.float32, device=dy2.device)
    partials = torch.empty(int(lib.zc_bf16_column_sum_blocks(rows)), cols, dtype=torch.float32, device=dy2.device)
    _lib.check(lib.zc_bf16_column_sum(dy2.data_ptr(), rows, cols, dy2.stride(0), out.data_ptr(),
                                      int(out.dtype == torch.bfloat16), int(acc), partials.data_ptr(),
                                      _lib.stream_ptr(dy2.device)), "zc_bf16_column_sum")
    if target is not None:
        bias.main_grad_written = True
        return None
    return out.to(bias.dtype)


class _LayerNorm(torch.autograd.Function):
    """``y = LayerNorm(h) * w + b`` with ``h = x`` or, given a residual, ``h = x + residual`` (returned
    as the second output): the residual add of the previous block runs inside the norm kernel, and the
    gradient arriving through ``h`` is added inside the backward kernel.  The parameters are kept by
    reference: when they carry ``main_grad`` the backward kernel writes their gradients there."""

    @staticmethod
    def forward(ctx, x, weight, bias, eps, residual):
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
            if residual is not None:
                r2 = residual.reshape(-1, cols).contiguous()
                h = torch.empty_like(x2)
            else:
                r2, h = None, x2
            _lib.check(_lib.cuda().zc_layernorm_fwd(
                x2.data_ptr(), _lib.ptr(r2), w.data_ptr(), b.data_ptr(), y.data_ptr(),
                h.data_ptr() if residual is not None else None, mean.data_ptr(), rstd.data_ptr(), rows, cols,
                float(eps), _lib.stream_ptr(x.device)), "zc_layernorm_fwd")
        else:
            h = x2 if residual is None else (x2.float() + residual.reshape(-1, cols).float()).to(x.dtype)
            hf = h.float()
            mean = hf.mean(-1)
            rstd = torch.rsqrt((hf - mean[:, None]).pow(2).mean(-1) + eps)
            y = ((hf - mean[:, None]) * rstd[:, None] * weight.float() + bias.float()).to(x.dtype)
            w = weight
        ctx.save_for_backward(h, w, mean, rstd)
        ctx.shape = shape
        ctx.params = (weight, bias)
        ctx.has_residual = residual is not None
        return y.view(shape), (h.view(shape) if residual is not None else None)

    @staticmethod
    def backward(ctx, dy, dh_out):
        h, w, mean, rstd = ctx.saved_tensors
        weight, bias = ctx.params
        rows, cols = h.shape
        dy2 = dy.reshape(rows, cols)
        if h.is_cuda:
            lib = _lib.cuda()
            dy2 = dy2.contiguous()
            dh2 = dh_out.reshape(rows, cols).contiguous() if dh_out is not None else None
            dx = torch.empty_like(h)
            tw, acc_w = _grad_target(weight, cols)
            tb, acc_b = _grad_target(bias, cols)
            direct = tw is not None and tb is not None and tw.dtype == tb.dtype
            if direct:
                gw, gb = tw, tb
            else:
                dwdb = torch.empty(2, cols, dtype=torch.float32, device=h.device)
                gw, gb, acc_w, acc_b = dwdb[0], dwdb[1], False, False
            partials = torch.empty(int(lib.zc_layernorm_bwd_ctas(rows)), 2, cols, dtype=torch.float32, device=h.device)
            _lib.check(lib.zc_layernorm_bwd(
                dy2.data_ptr(), h.data_ptr(), w.data_ptr(), mean.data_ptr(), rstd.data_ptr(), _lib.ptr(dh2),
                dx.data_ptr(), gw.data_ptr(), gb.data_ptr(), int(gw.dtype == torch.bfloat16), int(acc_w), int(acc_b),
                partials.data_ptr(), rows, cols, _lib.stream_ptr(h.device)), "zc_layernorm_bwd")
            if direct:
                weight.main_grad_written = bias.main_grad_written = True
                dw = db = None
            else:
                dw, db = gw.to(weight.dtype), gb.to(bias.dtype)
        else:
            hf, dyf = h.float(), dy2.float()
            xhat = (hf - mean[:, None]) * rstd[:, None]
            g = dyf * w.float()
            dxf = rstd[:, None] * (g - g.mean(-1, keepdim=True) - xhat * (g * xhat).mean(-1, keepdim=True))
            if dh_out is not None:
                dxf = dxf + dh_out.reshape(rows, cols).float()
            dx = dxf.to(h.dtype)
            dw = (dyf * xhat).sum(0).to(weight.dtype)
            db = dyf.sum(0).to(bias.dtype)
        dx = dx.view(ctx.shape)
        return dx, dw, db, None, (dx if ctx.has_residual else None)


def layer_norm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    """LayerNorm over the last dimension with weight and bias."""
    return _LayerNorm.apply(x, weight, bias, eps, None)[0]


def add_layer_norm(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor,
                   eps: float = 1e-5):
    """Returns ``(layer_norm(x + residual), x + residual)`` from one kernel."""
    return _LayerNorm.apply(x, weight, bias, eps, residual)


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
        ctx.bias = bias
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
        db = bias_grad(dx, ctx.bias)
        return dx.view(ctx.shape), db


def bias_gelu(x: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """``gelu_tanh(x + bias)`` with ``bias`` broadcast over the last dimension."""
    return _BiasGelu.apply(x, bias)
