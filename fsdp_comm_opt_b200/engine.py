"""``TrainEngine``: the public training API.  One object owns the model (built on the meta
device, FSDP2-wrapped, materialised as shards), the fused optimizer and the LR schedule;
``step(input_ids)`` takes a batch of token ids in (pinned) host memory, runs forward, backward and
the optimizer update, and returns the loss as a Python float.  ``train.py`` is the CLI around the
same pieces; ``bench.py`` times this call.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist

from .models import ModelConfig, build_model, get_config
from .ops.adamw import FusedAdamW
from .parallel.fsdp import FSDPPlan, apply_fsdp


@dataclass
class EngineConfig:
    model: str | ModelConfig = "llama3-8b"
    lr: float = 3e-5
    weight_decay: float = 1e-2
    master_dtype: torch.dtype = torch.bfloat16
    quantize: bool = True
    zip_ccl: bool = True
    compress_rs: bool = True
    act_ckpt: bool = False
    forward_prefetch_distance: int = 1
    transport: str = "auto"
    codec_version: str = "auto"
    seed: int = 0


class TrainEngine:
    def __init__(self, cfg: EngineConfig, device: torch.device):
        if not dist.is_initialized():
            raise RuntimeError("initialise torch.distributed first (utils.dist.init_distributed)")
        self.cfg, self.device = cfg, device
        torch.manual_seed(cfg.seed)
        mcfg = get_config(cfg.model) if isinstance(cfg.model, str) else cfg.model
        self.model_config = mcfg
        with torch.device("meta"):
            model = build_model(mcfg).to(cfg.master_dtype)
        self.plan = FSDPPlan(quantize=cfg.quantize, zip_ccl=cfg.zip_ccl, compress_rs=cfg.compress_rs,
                             forward_prefetch_distance=cfg.forward_prefetch_distance, transport=cfg.transport,
                             codec_version=cfg.codec_version, act_ckpt=cfg.act_ckpt)
        apply_fsdp(model, self.plan)
        model.to_empty(device=device)
        model.init_weights()
        self.model = model
        self.optimizer = FusedAdamW(model.parameters(), lr=cfg.lr, weight_decay=cfg.weight_decay)
        self.lr_scheduler = torch.optim.lr_scheduler.CosineAnnealingLR(self.optimizer, T_max=1000,
                                                                       eta_min=cfg.lr * 1e-2)
        self.global_step = 0

    def step_on_device(self, input_ids: torch.Tensor) -> torch.Tensor:
        """One optimizer step on a batch already on the device; returns the loss tensor."""
        self.model.unshard()
        out = self.model(input_ids=input_ids, labels=input_ids)
        out.loss.backward()
        self.optimizer.step()
        self.lr_scheduler.step()
        self.optimizer.zero_grad(set_to_none=True)
        self.global_step += 1
        return out.loss.detach()

    def step(self, input_ids_host: torch.Tensor) -> float:
        """Host batch in, loss out: H2D copy, one optimizer step, D2H read of the loss."""
        ids = input_ids_host.to(self.device, non_blocking=True)
        return float(self.step_on_device(ids).item())
