"""GPT-2-shape decoder (LayerNorm, learned positions, biased projections, tanh-GELU MLP, tied
output embedding): the family of the reference's shipped run (run.sh:1, GPT-2-XL), discovered by
the reference at ``model.transformer.h`` (train.py:99-100).  Attention, GEMMs, LayerNorm, the fused
bias + GELU of the MLP, the loss and the optimizer are the package's own ops.  Bias adds run in the
GEMM epilogue, residual adds inside the LayerNorm that follows them, and the gradients of biases and
norm parameters are written by their kernels straight into a sharded engine's gradient buffer.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint

from ..ops import attention as attn_ops
from ..ops import gemm, gpt2_ops, loss as loss_ops
from .config import ModelConfig
from .llama import CausalLMOutput, Embedding


class BiasLinear(nn.Module):
    def __init__(self, in_features: int, out_features: int, init_std: float):
        super().__init__()
        self.init_std = init_std
        self.weight = nn.Parameter(torch.empty(out_features, in_features))
        self.bias = nn.Parameter(torch.empty(out_features))

    def reset_parameters(self):
        nn.init.normal_(self.weight, mean=0.0, std=self.init_std)
        nn.init.zeros_(self.bias)

    def forward(self, x):
        return gemm.linear(x, self.weight, self.bias)


class GPT2Block(nn.Module):
    def __init__(self, cfg: ModelConfig):
        super().__init__()
        self.cfg = cfg
        d = cfg.d_model
        self.c_attn = BiasLinear(d, 3 * d, cfg.init_std)
        self.c_proj = BiasLinear(d, d, cfg.init_std)
        self.c_fc = BiasLinear(d, cfg.ffn, cfg.init_std)
        self.c_mlp_proj = BiasLinear(cfg.ffn, d, cfg.init_std)
        self.ln_1 = nn.LayerNorm(d, eps=cfg.norm_eps)
        self.ln_2 = nn.LayerNorm(d, eps=cfg.norm_eps)

    def forward(self, x, delta=None):
        """``x`` is the residual stream before the previous block's MLP output ``delta`` was added: the
        sum is formed inside ``ln_1``.  Returns the residual stream after attention and this block's MLP
        output, to be added by the next norm."""
        cfg = self.cfg
        B, S, d = x.shape
        H, hd = cfg.n_heads, cfg.head_dim
        if delta is None:
            ln1 = gpt2_ops.layer_norm(x, self.ln_1.weight, self.ln_1.bias, self.ln_1.eps)
        else:
            ln1, x = gpt2_ops.add_layer_norm(x, delta, self.ln_1.weight, self.ln_1.bias, self.ln_1.eps)
        qkv = self.c_attn(ln1).view(B, S, 3 * H, hd)
        if x.is_cuda and hd not in (64, 128):
            q, k, v = (t.transpose(1, 2) for t in qkv.split(H, dim=2))
            o = F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(B, S, d)
        else:
            o = attn_ops.causal_attention(qkv, H, H).view(B, S, d)
        ln2, x = gpt2_ops.add_layer_norm(x, self.c_proj(o), self.ln_2.weight, self.ln_2.bias, self.ln_2.eps)
        h = gpt2_ops.bias_gelu(gemm.linear(ln2, self.c_fc.weight), self.c_fc.bias)
        return x, self.c_mlp_proj(h)


class GPT2Backbone(nn.Module):
    def __init__(self, cfg: ModelConfig):
        super().__init__()
        self.wte = Embedding(cfg.vocab_size, cfg.d_model, cfg.init_std)
        self.wpe = Embedding(cfg.max_seq, cfg.d_model, cfg.init_std)
        self.h = nn.ModuleList(GPT2Block(cfg) for _ in range(cfg.n_layers))
        self.ln_f = nn.LayerNorm(cfg.d_model, eps=cfg.norm_eps)


class GPT2ForCausalLM(nn.Module):
    def __init__(self, cfg: ModelConfig):
        super().__init__()
        self.config = cfg
        self.transformer = GPT2Backbone(cfg)
        self.activation_checkpointing = False

    def init_weights(self):
        self.apply(lambda m: m.reset_parameters() if hasattr(m, "reset_parameters") else None)

    def forward(self, input_ids: torch.Tensor, labels: Optional[torch.Tensor] = None,
                return_logits: bool = False, **_ignored) -> CausalLMOutput:
        B, S = input_ids.shape
        t = self.transformer
        pos = torch.arange(S, device=input_ids.device)
        x, m = t.wte(input_ids), t.wpe(pos)[None].expand(B, S, -1)   # the position add runs in the first norm
        for blk in t.h:
            if self.activation_checkpointing and torch.is_grad_enabled():
                x, m = checkpoint(blk, x, m, use_reentrant=False)
            else:
                x, m = blk(x, m)
        x, _ = gpt2_ops.add_layer_norm(x, m, t.ln_f.weight, t.ln_f.bias, t.ln_f.eps)
        logits = gemm.linear(x, t.wte.weight)  # tied output embedding
        loss = None
        if labels is not None:
            shifted = torch.full_like(labels, loss_ops.IGNORE_INDEX)
            shifted[:, :-1] = labels[:, 1:]
            keep = logits.detach().clone() if return_logits else None
            loss = loss_ops.cross_entropy(logits.view(B * S, -1), shifted.reshape(-1))
            logits = keep
        return CausalLMOutput(loss=loss, logits=logits)
