"""bf16 linear layers: ``linear(x, w) = x @ w^T`` with the three GEMMs of training.

Backends (``set_backend``):
  ``"tcgen05_2sm"``  the hand-written sm_100a kernel in ``csrc/gemm_tcgen05_2sm.cu``: clusters of two
                 CTAs, ``tcgen05.mma.cta_group::2`` on 256 x 256 tiles with the B operand split between
                 the pair, TMA loads into 128B-swizzled shared memory, TMEM accumulators, persistent
                 over tiles with a split-K tail.  Any M, N, K; rows a multiple of 8 elements apart.
  ``"tcgen05"``  the one-SM kernel in ``csrc/gemm_tcgen05.cu`` (128 x 256 tiles; M % 128, N % 128,
                 K % 64).
  ``"cublas"``   ``torch.matmul`` (cuBLASLt), kept as the comparison column of the benchmarks.
  ``"auto"``     the two-SM kernel whenever the shape allows it, else the library.
Forward uses K-major operands; dgrad and wgrad use the MN-major descriptor forms, so no transposed
copy of the weight or the activations is made.  CPU tensors always use ``torch.matmul``.
"""
from __future__ import annotations

import os

import torch

from .. import _lib

_BACKEND = os.environ.get("ZC_GEMM_BACKEND", "auto")


def set_backend(name: str) -> None:
    global _BACKEND
    if name not in ("auto", "tcgen05", "tcgen05_2sm", "cublas"):
        raise ValueError(name)
    _BACKEND = name


def get_backend() -> str:
    return _BACKEND


def _rows_ok(t: torch.Tensor) -> bool:
    """Row-major 2-D operand the kernels can address: unit column stride, rows a multiple of 16 bytes
    apart (a slice ``buf[:, :n]`` of a padded buffer qualifies), 16-byte aligned base."""
    return (t.dim() == 2 and t.stride(1) == 1 and t.stride(0) % 8 == 0 and t.stride(0) >= t.shape[1]
            and t.data_ptr() % 16 == 0)


def _pad8(n: int) -> int:
    return (n + 7) // 8 * 8


def _kernel_for(a: torch.Tensor, b: torch.Tensor, M: int, N: int, K: int, trans_a: bool, trans_b: bool):
    """Which hand-written kernel will run this GEMM: "2sm", "1sm", or None for the library."""
    if (not a.is_cuda or a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16 or _BACKEND == "cublas"
            or min(M, N, K) <= 0 or not (_rows_ok(a) and _rows_ok(b))):
        return None
    two_sm_ok = M >= 128 and N >= 128 and K >= 64 and not (trans_a and trans_b)
    one_sm_ok = (M % 128 == 0 and N % 128 == 0 and K % 64 == 0 and a.is_contiguous() and b.is_contiguous())
    if _BACKEND in ("auto", "tcgen05_2sm") and two_sm_ok:
        return "2sm"
    if _BACKEND in ("tcgen05", "tcgen05_2sm") and one_sm_ok:
        return "1sm"
    return None


def gemm(a: torch.Tensor, b: torch.Tensor, trans_a: bool, trans_b: bool,
         out: torch.Tensor | None = None, accumulate: bool = False, bias: torch.Tensor | None = None) -> torch.Tensor:
    """C[M,N] (+)= op(A) @ op(B) for row-major 2-D bf16 tensors.

    op(A) is A ``[M,K]`` (or A^T of a stored ``[K,M]`` when ``trans_a``); op(B) is B ``[K,N]`` (or
    B^T of a stored ``[N,K]`` when ``trans_b``).  Operands and ``out`` may be row slices or column
    slices of wider buffers as long as rows stay a multiple of 8 elements apart.  When N is not a
    multiple of 8 (GPT-2's vocabulary of 50257) the result allocated here is a ``[:, :N]`` view of a
    buffer whose rows are padded to the next multiple of 8, so that the next GEMM and the loss kernel
    can read it with aligned rows; its padding columns hold zeros.  ``bias`` ([N]) is added to every
    row in the kernel's epilogue (the two-SM kernel), else by a separate add.
    """
    M, K = (a.shape[1], a.shape[0]) if trans_a else (a.shape[0], a.shape[1])
    N = b.shape[0] if trans_b else b.shape[1]
    kind = _kernel_for(a, b, M, N, K, trans_a, trans_b)
    if kind is not None and out is not None and not (_rows_ok(out) and out.dtype == torch.bfloat16
                                                     and (kind == "1sm" and out.is_contiguous()
                                                          or kind == "2sm" and out.stride(0) >= _pad8(N))):
        kind = None
    if kind is not None:
        if out is None:
            out = torch.empty(M, N, dtype=a.dtype, device=a.device) if N % 8 == 0 else \
                torch.empty(M, _pad8(N), dtype=a.dtype, device=a.device)[:, :N]
            accumulate = False
        lib = _lib.cuda()
        if kind == "2sm":
            fused_bias = (bias is not None and bias.dtype == torch.bfloat16 and bias.is_contiguous()
                          and bias.numel() == N and bias.data_ptr() % 16 == 0)
            _lib.check(lib.zc_gemm_bf16_2sm_bias(
                a.data_ptr(), b.data_ptr(), out.data_ptr(), bias.data_ptr() if fused_bias else None, M, N, K,
                a.stride(0), b.stride(0), out.stride(0), int(trans_a), int(trans_b), int(accumulate),
                _lib.stream_ptr(a.device)), "zc_gemm_bf16_2sm")
            if bias is not None and not fused_bias:
                out.add_(bias.to(out.dtype))
        else:
            _lib.check(lib.zc_gemm_bf16(
                a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, int(trans_a), int(trans_b),
                int(accumulate), _lib.stream_ptr(a.device)), "zc_gemm_bf16")
            if bias is not None:
                out.add_(bias.to(out.dtype))
        return out
    A = a.t() if trans_a else a
    B = b.t() if trans_b else b
    if out is None:
        res = torch.matmul(A, B)
    elif accumulate:
        res = out.addmm_(A, B)
    else:
        res = torch.matmul(A, B, out=out)
    if bias is not None:
        res.add_(bias.to(res.dtype))
    return res


class _Linear(torch.autograd.Function):
    """``y = x w^T``.  The weight is kept by reference (not as a saved tensor): under the sharded
    engines its storage is released after forward and gathered again before backward, and backward
    must read whatever the parameter points at then.  When the weight carries ``main_grad`` (a view
    of the engine's flat gradient buffer) the weight-gradient GEMM writes there directly and no
    ``.grad`` tensor is produced."""

    @staticmethod
    def forward(ctx, x, w, bias=None):
        ctx.save_for_backward(x)
        ctx.w = w
        ctx.bias = bias
        x2 = x.reshape(-1, x.shape[-1])
        b = None if bias is None else (bias if bias.dtype == x.dtype else bias.to(x.dtype))
        y = gemm(x2, w, False, True, bias=b)   # [T,K] @ [N,K]^T (+ bias in the epilogue)
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        w = ctx.w
        x2 = x.reshape(-1, x.shape[-1])
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not (dy2.is_contiguous() or _rows_ok(dy2)):
            dy2 = dy2.contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, w, False, False).view(x.shape)      # [T,N] @ [N,K]
        if ctx.needs_input_grad[1]:
            mg = getattr(w, "main_grad", None)
            if mg is not None and mg.dtype == dy2.dtype:
                gemm(dy2, x2, True, False, out=mg, accumulate=bool(w.main_grad_written))
                w.main_grad_written = True
            else:
                dw = gemm(dy2, x2, True, False)                # [T,N]^T @ [T,K]
        db = None
        if ctx.bias is not None and ctx.needs_input_grad[2]:
            from .gpt2_ops import bias_grad

            db = bias_grad(dy2, ctx.bias)                      # column sums, into bias.main_grad when it has one
        return dx, dw, db


def linear(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """``x [..., K] @ w[N, K]^T (+ bias)``."""
    if x.dtype != w.dtype:
        w = w.to(x.dtype)
    return _Linear.apply(x, w, bias)
