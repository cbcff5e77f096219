"""``TrainEngine``: the public training API.  One object owns the model (built on the meta
device, sharded, materialised as shards), the fused optimizer and the LR schedule;
``step(input_ids)`` takes a batch of token ids in (pinned) host memory, runs forward, backward and
the optimizer update, and returns the loss as a Python float.  ``train.py`` is the CLI around the
same pieces; ``bench.py`` times this call.

Two sharding back ends share the comm hooks, the model code and the optimizer kernel:

``"flat"``   (default) the package's own flat-shard ZeRO-3 engine (``parallel/flat_shard.py``):
             parameters and gradients live in flat buffers that the collectives read and write
             directly, one AdamW launch per step.
``"fsdp2"``  PyTorch FSDP2 ``fully_shard`` with the hooks installed through
             ``set_custom_all_gather`` / ``set_custom_reduce_scatter``, which is how the reference
             wires them (reference: train.py:93-123).  Needed for CPU offload.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist

from .models import ModelConfig, build_model, get_config, shard_groups
from .ops.adamw import FusedAdamW
from .ops.loss import unit_loss_grad
from .parallel.flat_shard import FlatShardEngine, FlatShardPlan
from .parallel.fsdp import FSDPPlan, apply_fsdp, make_hook_factories


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
    wire: str = "auto"              # "auto" | "nibble" | "compressed" | "verbatim": what the collectives put on the wire
    seed: int = 0
    sharding: str = "flat"          # "flat" | "fsdp2"
    cpu_offload: bool = False       # fsdp2 only
    error_feedback: bool = True
    time_collectives: bool = False  # flat only: CUDA-event timing of every collective
    reshard_after_forward: object = "auto"   # flat only: True | False | "auto" (see FlatShardPlan)


def build_sharded(cfg: EngineConfig, device: torch.device):
    """Model on the meta device -> sharded and initialised.  Returns ``(model, plan, flat_engine)``;
    ``flat_engine`` is None for the FSDP2 back end."""
    mcfg = get_config(cfg.model) if isinstance(cfg.model, str) else cfg.model
    torch.manual_seed(cfg.seed)
    plan = FSDPPlan(quantize=cfg.quantize, zip_ccl=cfg.zip_ccl, compress_rs=cfg.compress_rs,
                    cpu_offload=cfg.cpu_offload, forward_prefetch_distance=cfg.forward_prefetch_distance,
                    transport=cfg.transport, codec_version=cfg.codec_version, act_ckpt=cfg.act_ckpt,
                    error_feedback=cfg.error_feedback, wire=cfg.wire)
    if cfg.sharding == "fsdp2":
        with torch.device("meta"):
            model = build_model(mcfg).to(cfg.master_dtype)
        apply_fsdp(model, plan)
        model.to_empty(device="cpu" if cfg.cpu_offload else device)
        model.init_weights()
        return model, plan, None
    if cfg.sharding != "flat":
        raise ValueError(f"unknown sharding back end {cfg.sharding!r}")
    if cfg.cpu_offload:
        raise ValueError("CPU offload needs sharding='fsdp2'")
    with torch.device("meta"):
        model = build_model(mcfg)
    ag_factory, rs_factory = make_hook_factories(plan, reduce_out_dtype=cfg.master_dtype)
    fplan = FlatShardPlan(ag_hook_factory=ag_factory, rs_hook_factory=rs_factory,
                          forward_prefetch_distance=cfg.forward_prefetch_distance,
                          master_dtype=cfg.master_dtype, act_ckpt=cfg.act_ckpt,
                          time_collectives=cfg.time_collectives, reshard_after_forward=cfg.reshard_after_forward)
    flat = FlatShardEngine(model, shard_groups(model), fplan, device)
    return model, plan, flat


class TrainEngine:
    def __init__(self, cfg: EngineConfig, device: torch.device):
        if not dist.is_initialized():
            raise RuntimeError("initialise torch.distributed first (utils.dist.init_distributed)")
        self.cfg, self.device = cfg, device
        self.model_config = get_config(cfg.model) if isinstance(cfg.model, str) else cfg.model
        self.model, self.plan, self.flat = build_sharded(cfg, device)
        params = self.flat.parameters_for_optimizer() if self.flat is not None else self.model.parameters()
        self.optimizer = FusedAdamW(params, lr=cfg.lr, weight_decay=cfg.weight_decay)
        self.lr_scheduler = torch.optim.lr_scheduler.CosineAnnealingLR(self.optimizer, T_max=1000,
                                                                       eta_min=cfg.lr * 1e-2)
        self.global_step = 0

    def step_on_device(self, input_ids: torch.Tensor) -> torch.Tensor:
        """One optimizer step on a batch already on the device; returns the loss tensor."""
        if self.flat is not None:
            self.flat.begin_step()
            out = self.model(input_ids=input_ids, labels=input_ids)
            self.flat.backward(out.loss)
            self.flat.optimizer_step(self.optimizer, self.lr_scheduler)
        else:
            self.model.unshard()
            out = self.model(input_ids=input_ids, labels=input_ids)
            with unit_loss_grad():
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

    def comm_report(self) -> dict:
        """What the collectives of this engine actually ran on (see ``parallel.fsdp.comm_report``)."""
        from .parallel.fsdp import comm_report

        return comm_report(self.plan)
