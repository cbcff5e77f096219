"""FSDP2 wrapping: the one parallelism strategy (ZeRO-3 style full-shard data parallel).

``apply_fsdp`` reproduces the reference's wrapping (reference: train.py:93-123): every decoder
layer becomes its own FSDP2 group with ``reshard_after_forward=True`` and a bf16-compute /
fp32-reduce mixed-precision policy, then the root module is wrapped; layer i explicitly prefetches
layers i+1..i+distance in forward; a fresh comm hook instance is installed per FSDP module.
On top of the reference: a gradient reduce-scatter hook, a choice of reduce dtype, and
activation checkpointing per block.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch
from torch.distributed.fsdp import CPUOffloadPolicy, FSDPModule, MixedPrecisionPolicy, fully_shard

from ..models import decoder_layers
from .hooks import QuantizedAllGather, ZipCCLAllGather, ZipCCLReduceScatter


@dataclass
class FSDPPlan:
    quantize: bool = False            # -q: install a custom all-gather (int8 unless zip_ccl)
    zip_ccl: bool = False             # --zip-ccl: lossless compressed all-gather
    compress_rs: bool = False         # --compress-rs: compressed reduce-scatter with error feedback
    cpu_offload: bool = False
    forward_prefetch_distance: int = 1
    param_dtype: torch.dtype = torch.bfloat16
    reduce_dtype: torch.dtype = torch.float32
    transport: str = "auto"
    codec_version: str = "auto"
    wire: str = "auto"               # "auto" (nibble on the fused transport, bit planes on lib) | "nibble" | "compressed" | "verbatim"
    error_feedback: bool = True
    act_ckpt: bool = False
    mesh: Optional[object] = None
    rs_hooks: list = field(default_factory=list)
    ag_hooks: list = field(default_factory=list)


def _install_hooks(m: FSDPModule, plan: FSDPPlan) -> None:
    if plan.quantize:
        if plan.zip_ccl:
            hook = ZipCCLAllGather(codec_version=plan.codec_version, transport=plan.transport, wire=plan.wire)
        else:
            hook = QuantizedAllGather(transport=plan.transport)
        m.set_custom_all_gather(hook)
        plan.ag_hooks.append(hook)
    if plan.compress_rs:
        rs = ZipCCLReduceScatter(error_feedback=plan.error_feedback, reduce_dtype=plan.reduce_dtype,
                                 transport=plan.transport, wire=plan.wire)
        m.set_custom_reduce_scatter(rs)
        plan.rs_hooks.append(rs)


def make_hook_factories(plan: FSDPPlan, reduce_out_dtype: torch.dtype = torch.bfloat16):
    """Constructors of one all-gather and one reduce-scatter hook per shard group for the flat-shard
    engine, from the same flags ``apply_fsdp`` reads.  ``None`` means the plain library collective.
    Every hook made is also listed in ``plan.ag_hooks`` / ``plan.rs_hooks``."""
    ag = rs = None
    if plan.quantize:
        def ag():
            hook = (ZipCCLAllGather(codec_version=plan.codec_version, transport=plan.transport, wire=plan.wire) if plan.zip_ccl
                    else QuantizedAllGather(transport=plan.transport))
            plan.ag_hooks.append(hook)
            return hook
    if plan.compress_rs:
        def rs():
            hook = ZipCCLReduceScatter(error_feedback=plan.error_feedback, reduce_dtype=reduce_out_dtype,
                                       transport=plan.transport, wire=plan.wire)
            plan.rs_hooks.append(hook)
            return hook
    return ag, rs


def comm_report(plan: FSDPPlan) -> dict:
    """What the installed hooks ran on so far: the transport each kind of hook resolved to, calls and
    wire bytes per element of the fused channels (synchronises the device).  Raises when compression
    was requested on CUDA with ``transport="symm"`` semantics expected but every call fell back."""
    from . import symm_impl

    rep: dict = {"all_gather": "library", "reduce_scatter": "library"}
    if plan.ag_hooks:
        rep["all_gather"] = sorted({getattr(h, "last_transport", None) or "not called" for h in plan.ag_hooks})
    if plan.rs_hooks:
        rep["reduce_scatter"] = sorted({getattr(h, "last_transport", None) or "not called" for h in plan.rs_hooks})
    chans = {}
    for ch in symm_impl.all_channels():
        wire = ch.wire_bytes()
        chans[ch.kind] = {"calls": ch.calls, "wire_bytes": wire,
                          "wire_bytes_per_element": round(wire / ch.elements, 4) if ch.elements else None,
                          "push_ctas": ch.push_ctas, "dec_ctas": ch.dec_ctas,
                          "multicast": bool(getattr(ch, "mc_ptr", 0))}
    rep["channels"] = chans
    return rep


def apply_fsdp(model: torch.nn.Module, plan: FSDPPlan) -> torch.nn.Module:
    # With bf16 parameters the gradients entering the reduce-scatter are bf16 values and FSDP2
    # casts the reduced result back to bf16.  The compressed reduce-scatter hook accumulates in
    # fp32 internally whatever its input dtype, so handing it bf16 rows is numerically the same as
    # the fp32 hand-off and removes FSDP2's bf16->fp32 copy-in and fp32->bf16 cast (two passes over
    # every gradient).  Without the hook the reference policy (fp32 reduce) is kept.
    first = next(model.parameters(), None)
    if (plan.compress_rs and plan.reduce_dtype == torch.float32 and first is not None
            and first.dtype == torch.bfloat16 and plan.param_dtype == torch.bfloat16):
        plan.reduce_dtype = torch.bfloat16
    cfg = dict(
        reshard_after_forward=True,
        offload_policy=CPUOffloadPolicy() if plan.cpu_offload else None,
        mp_policy=MixedPrecisionPolicy(param_dtype=plan.param_dtype, reduce_dtype=plan.reduce_dtype),
    )
    if cfg["offload_policy"] is None:
        del cfg["offload_policy"]
    if plan.mesh is not None:
        cfg["mesh"] = plan.mesh
    layers = decoder_layers(model)
    fsdp_layers = []
    for layer in layers:
        m = fully_shard(layer, **cfg)
        fsdp_layers.append(m)
        _install_hooks(m, plan)
    if plan.forward_prefetch_distance > 0:
        for i, m in enumerate(fsdp_layers):
            nxt = fsdp_layers[i + 1: i + 1 + plan.forward_prefetch_distance]
            if nxt:
                m.set_modules_to_forward_prefetch(nxt)
    root = fully_shard(model, **cfg)
    _install_hooks(root, plan)
    if plan.act_ckpt:
        model.activation_checkpointing = True
    return root
