"""Llama-shape decoder (RMSNorm, RoPE, grouped-query causal attention, SwiGLU) built from the
package's own ops.  Parameters are laid out for FSDP2 and for the fused kernels: one packed
``wqkv`` and one packed ``wgu`` (gate|up) weight per block, large matrices first and norm vectors
last so that every matrix shard starts on a codec chunk boundary in the all-gather buffer.

The reference instantiates HF ``AutoModelForCausalLM`` (train.py:86-88) and relies on
``model.model.layers`` for layer discovery (train.py:99-104); the same attribute path exists here.
Calling convention matches HF causal LMs: ``model(input_ids=..., labels=...)`` returns an object
with ``.loss`` and ``.logits``; labels are shifted by one inside the model.
"""
from __future__ import annotations

from typing import NamedTuple, Optional

import torch
import torch.nn as nn
from torch.utils.checkpoint import checkpoint

from ..ops import attention as attn_ops
from ..ops import gemm, loss as loss_ops, norm, rope, swiglu
from .config import ModelConfig


class CausalLMOutput(NamedTuple):
    """A pytree (named tuple), so FSDP2 finds the loss tensor and registers its pre-backward hook."""

    loss: Optional[torch.Tensor]
    logits: Optional[torch.Tensor]


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.empty(dim))

    def reset_parameters(self):
        nn.init.ones_(self.weight)

    def forward(self, x, residual=None):
        """``rms_norm(x)``, or ``rms_norm(x + residual)`` from one kernel when a pending residual
        branch is handed over."""
        if residual is None:
            return norm.rms_norm(x, self.weight, self.eps)
        return norm.add_rms_norm(residual, x, self.weight, self.eps)[0]


class Embedding(nn.Embedding):
    """Token / position table initialised with the model's ``init_std``."""

    def __init__(self, num_embeddings: int, embedding_dim: int, init_std: float):
        self.init_std = init_std
        super().__init__(num_embeddings, embedding_dim)

    def reset_parameters(self):
        nn.init.normal_(self.weight, mean=0.0, std=self.init_std)


class Linear(nn.Module):
    """Bias-free linear layer on the package GEMM."""

    def __init__(self, in_features: int, out_features: int, init_std: float):
        super().__init__()
        self.in_features, self.out_features, self.init_std = in_features, out_features, init_std
        self.weight = nn.Parameter(torch.empty(out_features, in_features))

    def reset_parameters(self):
        nn.init.normal_(self.weight, mean=0.0, std=self.init_std)

    def forward(self, x):
        return gemm.linear(x, self.weight)


class LlamaBlock(nn.Module):
    def __init__(self, cfg: ModelConfig):
        super().__init__()
        self.cfg = cfg
        d, hd = cfg.d_model, cfg.head_dim
        self.wqkv = Linear(d, (cfg.n_heads + 2 * cfg.n_kv_heads) * hd, cfg.init_std)
        self.wo = Linear(cfg.n_heads * hd, d, cfg.init_std)
        self.wgu = Linear(d, 2 * cfg.ffn, cfg.init_std)
        self.wd = Linear(cfg.ffn, d, cfg.init_std)
        self.attn_norm = RMSNorm(d, cfg.norm_eps)
        self.mlp_norm = RMSNorm(d, cfg.norm_eps)

    def forward(self, x, delta=None):
        """The residual stream is ``x + delta``: a block hands its MLP output to the next block
        unadded, and the next block's first normalisation kernel does the add (so no stand-alone
        elementwise add runs between blocks).  Returns ``(x, delta)``."""
        cfg = self.cfg
        B, S, d = x.shape
        hd, Hq, Hkv = cfg.head_dim, cfg.n_heads, cfg.n_kv_heads
        cos, sin = rope.cached_tables(S, hd, cfg.rope_theta, x.device)
        if delta is None:
            h = self.attn_norm(x)
        else:
            h, x = norm.add_rms_norm(delta, x, self.attn_norm.weight, self.attn_norm.eps)
        qkv = self.wqkv(h).view(B, S, Hq + 2 * Hkv, hd)
        o = attn_ops.causal_attention(qkv, Hq, Hkv, None, cos, sin)
        a = self.wo(o.view(B, S, Hq * hd))
        h2, x = norm.add_rms_norm(a, x, self.mlp_norm.weight, self.mlp_norm.eps)
        gu = self.wgu(h2).view(B * S, 2 * cfg.ffn)
        m = self.wd(swiglu.swiglu(gu)).view(B, S, d)
        return x, m


class LlamaBackbone(nn.Module):
    def __init__(self, cfg: ModelConfig):
        super().__init__()
        self.embed_tokens = Embedding(cfg.vocab_size, cfg.d_model, cfg.init_std)
        self.layers = nn.ModuleList(LlamaBlock(cfg) for _ in range(cfg.n_layers))
        self.norm = RMSNorm(cfg.d_model, cfg.norm_eps)


class LlamaForCausalLM(nn.Module):
    def __init__(self, cfg: ModelConfig):
        super().__init__()
        self.config = cfg
        self.model = LlamaBackbone(cfg)
        self.lm_head = Linear(cfg.d_model, cfg.vocab_size, cfg.init_std)
        if cfg.tie_embeddings:
            self.lm_head.weight = self.model.embed_tokens.weight
        self.activation_checkpointing = False

    def init_weights(self):
        """Calls ``reset_parameters`` on every submodule, as the reference does after
        ``to_empty`` (train.py:125-128)."""
        self.apply(lambda m: m.reset_parameters() if hasattr(m, "reset_parameters") else None)

    def forward(self, input_ids: torch.Tensor, labels: Optional[torch.Tensor] = None,
                return_logits: bool = False, **_ignored) -> CausalLMOutput:
        B, S = input_ids.shape
        x, delta = self.model.embed_tokens(input_ids), None
        for layer in self.model.layers:
            if self.activation_checkpointing and torch.is_grad_enabled():
                x, delta = checkpoint(layer, x, delta, use_reentrant=False)
            else:
                x, delta = layer(x, delta)
        x = self.model.norm(x, delta)
        logits = self.lm_head(x)
        loss = None
        if labels is not None:
            shifted = torch.full_like(labels, loss_ops.IGNORE_INDEX)
            shifted[:, :-1] = labels[:, 1:]
            keep = logits.detach().clone() if return_logits else None
            loss = loss_ops.cross_entropy(logits.view(B * S, -1), shifted.reshape(-1))
            logits = keep
        return CausalLMOutput(loss=loss, logits=logits)
