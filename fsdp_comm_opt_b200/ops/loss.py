"""Token cross-entropy over bf16 logits with the gradient produced in the same pass.

``cross_entropy(logits, labels)`` returns the mean loss over labels != ignore_index.  On CUDA one
kernel per call reads each logits row twice (online max/sum, then gradient) and overwrites the
row with d(loss)/d(logits); backward only rescales.  HF's loss path, which the reference uses
(train.py:252), upcasts the whole ``[T, V]`` logits tensor to fp32 first.
"""
from __future__ import annotations

import torch

from .. import _lib

IGNORE_INDEX = -100

# Set (by the training engines, around ``loss.backward()``) when the loss is the root of the backward
# pass and its incoming gradient is therefore exactly 1: the [T, V] gradient buffer is then handed on
# as it is instead of being multiplied by one (a full read + write of the logits-sized tensor).
_UNIT_GRAD = False


class unit_loss_grad:
    """Context manager: promise that d(total)/d(loss) == 1 for backward passes started inside."""

    def __enter__(self):
        global _UNIT_GRAD
        self._prev, _UNIT_GRAD = _UNIT_GRAD, True
        return self

    def __exit__(self, *exc):
        global _UNIT_GRAD
        _UNIT_GRAD = self._prev


class _CrossEntropy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, labels, ignore_index):
        T, V = logits.shape
        valid = (labels != ignore_index)
        count = valid.sum().clamp_min(1).to(torch.float32)
        if logits.is_cuda:
            if logits.dtype != torch.bfloat16 or logits.stride(1) != 1 or logits.stride(0) < V:
                raise TypeError("CUDA cross_entropy expects bf16 logits with unit column stride")
            inv = (1.0 / count).reshape(1).contiguous()
            row_loss = torch.empty(T, dtype=torch.float32, device=logits.device)
            lab = labels.to(torch.int64).contiguous()
            # rows may be padded (the GEMM's [:, :V] view of aligned rows when V % 8 != 0): the kernel
            # takes the row stride and zeroes the padding
            _lib.check(_lib.cuda().zc_ce_fwd_bwd_ld(
                logits.data_ptr(), lab.data_ptr(), row_loss.data_ptr(), inv.data_ptr(), T, V, logits.stride(0),
                int(ignore_index), _lib.stream_ptr(logits.device)), "zc_ce_fwd_bwd")
            ctx.grad_logits = logits.detach()  # the buffer now holds d(loss)/d(logits)
            return row_loss.sum() * inv[0]
        lf = logits.float()
        lse = torch.logsumexp(lf, dim=-1)
        safe = labels.clamp_min(0)
        picked = lf.gather(1, safe[:, None])[:, 0]
        row = torch.where(valid, lse - picked, torch.zeros_like(lse))
        grad = torch.softmax(lf, dim=-1)
        grad[torch.arange(T), safe] -= 1.0
        grad = grad * (valid[:, None] / count)
        ctx.grad_logits = grad.to(logits.dtype)
        return row.sum() / count

    @staticmethod
    def backward(ctx, dloss):
        grad = ctx.grad_logits
        ctx.grad_logits = None
        if _UNIT_GRAD:
            return grad, None, None
        if grad.is_cuda:
            # scale in place to keep one [T, V] buffer
            return grad.mul_(dloss.to(grad.dtype)), None, None
        return grad * dloss.to(grad.dtype), None, None


def cross_entropy(logits: torch.Tensor, labels: torch.Tensor, ignore_index: int = IGNORE_INDEX) -> torch.Tensor:
    """``logits`` [T, V] is consumed (overwritten with its gradient on CUDA)."""
    return _CrossEntropy.apply(logits, labels, ignore_index)
