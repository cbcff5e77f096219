"""Fused AdamW on the local shards of FSDP2 parameters.

``FusedAdamW`` keeps the state layout of ``torch.optim.AdamW`` (``step``, ``exp_avg``,
``exp_avg_sq`` per parameter, DTensor-sharded like the parameter), so
``torch.distributed.checkpoint.state_dict.get_state_dict`` / ``set_state_dict`` work unchanged
and checkpoints are interchangeable with the reference's optimizer
(reference: train.py:146 ``torch.optim.AdamW(..., fused=True)``).

On CUDA each shard is updated by one launch of ``zc_adamw`` (one read of p, g, m, v and one write
of p, m, v; bias correction and decoupled weight decay folded in; optional gradient zeroing in the
same pass).  The launch is guarded by the library's health word: when a fused collective of the step
ran into its bounded wait (and therefore left wrong data behind) the kernel returns without
touching parameters or moments, so the bad step is never applied even though the host only learns
of it at its next synchronisation.  CPU tensors use the same arithmetic in PyTorch.
"""
from __future__ import annotations

import math

import torch

from .. import _lib

_DT = {torch.bfloat16: 0, torch.float32: 1, torch.float16: 2}


def _local(t: torch.Tensor) -> torch.Tensor:
    return t._local_tensor if hasattr(t, "_local_tensor") else t


class FusedAdamW(torch.optim.Optimizer):
    def __init__(self, params, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 1e-2, zero_grad_in_step: bool = False):
        if lr < 0 or eps < 0 or not 0 <= betas[0] < 1 or not 0 <= betas[1] < 1:
            raise ValueError("invalid AdamW hyper-parameters")
        defaults = dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)
        super().__init__(params, defaults)
        self.zero_grad_in_step = zero_grad_in_step
        self.kernel_launches = 0

    def ensure_state(self) -> None:
        """Create the (zero) moments of every parameter that has none yet, so that a checkpoint can
        be loaded into, or saved from, an optimizer that has not stepped."""
        for group in self.param_groups:
            for p in group["params"]:
                st = self.state[p]
                if len(st) == 0:
                    st["step"] = torch.zeros((), dtype=torch.float32)
                    st["exp_avg"] = torch.zeros_like(p, memory_format=torch.preserve_format)
                    st["exp_avg_sq"] = torch.zeros_like(p, memory_format=torch.preserve_format)

    @torch.no_grad()
    def step(self, closure=None, split_at: int | None = None, between=None):
        """``split_at`` / ``between``: update elements ``[0, split_at)`` of every (flat) parameter first, call
        ``between()``, then update the rest.  The flat-shard engine uses it to start gathering the
        first groups of the next step while the rest of the shards are still being updated."""
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            lr = group["lr"]
            lr = float(lr) if not isinstance(lr, torch.Tensor) else float(lr.item())
            b1, b2 = group["betas"]
            eps, wd = group["eps"], group["weight_decay"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if len(st) == 0:
                    st["step"] = torch.zeros((), dtype=torch.float32)
                    st["exp_avg"] = torch.zeros_like(p, memory_format=torch.preserve_format)
                    st["exp_avg_sq"] = torch.zeros_like(p, memory_format=torch.preserve_format)
                st["step"] += 1
                step = int(st["step"].item())  # CPU scalar tensor: no device sync
                bc1 = 1.0 - b1 ** step
                bc2 = 1.0 - b2 ** step
                pl, gl = _local(p), _local(p.grad)
                ml, vl = _local(st["exp_avg"]), _local(st["exp_avg_sq"])
                if pl.numel() == 0:
                    continue
                if pl.is_cuda:
                    if not (pl.is_contiguous() and gl.is_contiguous()):
                        raise ValueError("FusedAdamW needs contiguous shards")
                    lib = _lib.cuda()
                    with torch.cuda.device(pl.device):
                        guard = lib.zc_health_word()
                    n = pl.numel()
                    cut = n if split_at is None else max(0, min(n, int(split_at) // 8 * 8))
                    for lo, hi in ((0, cut), (cut, n)):
                        if hi > lo:
                            _lib.check(lib.zc_adamw_guarded(
                                pl.data_ptr() + lo * pl.element_size(), gl.data_ptr() + lo * gl.element_size(),
                                ml.data_ptr() + lo * ml.element_size(), vl.data_ptr() + lo * vl.element_size(), hi - lo,
                                _DT[pl.dtype], _DT[gl.dtype], _DT[ml.dtype], float(lr), float(b1), float(b2),
                                float(eps), float(wd), float(bc1), float(bc2), int(self.zero_grad_in_step),
                                guard, _lib.stream_ptr(pl.device)), "zc_adamw")
                            self.kernel_launches += 1
                        if hi == cut and between is not None and cut < n:
                            between()
                            between = None
                else:
                    g = gl.float()
                    pf = pl.float()
                    m = ml.float().mul_(b1).add_(g, alpha=1 - b1)
                    v = vl.float().mul_(b2).addcmul_(g, g, value=1 - b2)
                    pf.mul_(1 - lr * wd)
                    denom = (v.sqrt() / math.sqrt(bc2)).add_(eps)
                    pf.addcdiv_(m, denom, value=-lr / bc1)
                    pl.copy_(pf), ml.copy_(m), vl.copy_(v)
                    if self.zero_grad_in_step:
                        gl.zero_()
        if between is not None:
            between()
        return loss
