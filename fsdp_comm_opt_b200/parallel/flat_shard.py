"""Flat-shard ZeRO-3 engine: full-shard data parallelism laid out so that the collectives move
the parameters and gradients themselves, with nothing copied in or out around them.

The reference shards with PyTorch FSDP2 (reference: train.py:93-123): every parameter is split
on dim 0, so each all-gather is preceded by a copy-in of the shards into a flat buffer and
followed by a ``split_with_sizes_copy`` into per-parameter tensors, and each reduce-scatter is
preceded by a ``chunk_cat`` of the gradients.  Here a group (one decoder block, the embedding, the
head) owns ONE flat bf16 buffer of ``W * S`` elements that holds all its parameters back to back
(each starting on a 256-byte boundary); rank r keeps elements ``[r*S, (r+1)*S)`` as its shard.

* all-gather:  input = the shard, output = the flat buffer; the module's parameters are views
  into that buffer, so the gathered bytes are the weights the GEMMs read.
* backward:    the weight-gradient GEMMs write straight into views of a flat gradient buffer of
  the same layout (``param.main_grad``); other gradients are copied there once.
* reduce-scatter: input = the flat gradient buffer (row j is the slice rank j owns), output = this
  rank's slice of ONE gradient tensor that covers every group.
* optimizer:   one fused AdamW launch over all shards of all groups (one master tensor).
* world size 1: parameters are views of the master tensor and gradients views of the gradient
  tensor for the whole run; a step contains no communication and no copy at all.

The collectives themselves are the same hook objects FSDP2 would call (``ZipCCLAllGather``,
``QuantizedAllGather``, ``ZipCCLReduceScatter`` or plain NCCL / gloo), invoked on two side streams;
buffers come from pools with explicit events, so nothing is allocated in steady state.
Schedule: forward gathers group i+1..i+d while group i computes and releases group i afterwards;
backward gathers group i-1 while group i computes and reduce-scatters group i's gradients as soon
as its backward is complete.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

PARAM_ALIGN = 128          # elements: every parameter starts on a 256-byte boundary
SHARD_ALIGN = 4096         # elements: a shard is a whole number of codec blocks (v1) / chunks (v2)


# ---------------------------------------------------------------------------------------------
# plain collectives with the hook call signature
# ---------------------------------------------------------------------------------------------
class PlainAllGather:
    """``dist.all_gather_into_tensor`` behind the hook protocol."""

    def __call__(self, output_tensor, input_tensor, group, async_op: bool = False):
        return dist.all_gather_into_tensor(output_tensor, input_tensor, group=group, async_op=async_op)


class PlainReduceScatter:
    """Reduce-scatter with fp32 accumulation, as the reference's mixed-precision policy does
    (reference: train.py:96 ``reduce_dtype=torch.float32``): rows are widened to fp32, summed by
    the library and the averaged result is rounded once into ``output_tensor``."""

    def __call__(self, output_tensor, input_tensor, group, op=None, async_op: bool = False):
        world = dist.get_world_size(group)
        x = input_tensor.view(-1)
        x32 = x if x.dtype == torch.float32 else x.to(torch.float32)
        out32 = output_tensor.view(-1) if output_tensor.dtype == torch.float32 else torch.empty(
            x.numel() // world, dtype=torch.float32, device=x.device)
        dist.reduce_scatter_tensor(out32, x32, op=dist.ReduceOp.SUM, group=group)
        out32.mul_(1.0 / world)
        if out32.data_ptr() != output_tensor.data_ptr():
            output_tensor.view(-1).copy_(out32)
        return None


# ---------------------------------------------------------------------------------------------
# layout
# ---------------------------------------------------------------------------------------------
@dataclass
class GroupSpec:
    """Modules whose parameters are gathered and reduced together.

    ``modules`` run back to back in forward (hooks go on the first and the last one).
    ``persistent``: gathered at the start of the step and kept until the end of backward (groups
    whose parameters are used at both ends of the step, e.g. tied embeddings).
    ``backward_needs_params``: False for modules whose backward does not read the weights
    (embedding lookups), which saves their re-gather in backward.
    """

    name: str
    modules: list
    persistent: bool = False
    backward_needs_params: bool = True
    extra_params: list = field(default_factory=list)   # parameters used outside module.forward


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


class _Slot:
    __slots__ = ("param", "fqn", "offset", "numel", "shape")

    def __init__(self, param, fqn, offset, numel, shape):
        self.param, self.fqn, self.offset, self.numel, self.shape = param, fqn, offset, numel, shape


class _Pool:
    """Fixed-layout buffers handed out and taken back with the event after which they are free.

    A buffer that has just been released is free only once its last reader has finished on the
    device (a reduce-scatter still running, a layer still computing), and the host runs many layers
    ahead of the device, so handing the newest release straight back would make the next user wait
    for exactly the work it is meant to overlap.  The pool therefore grows to ``depth`` buffers per
    layout before it reuses any, and then reuses the one released longest ago."""

    def __init__(self, device, dtype, depth: int):
        self.device, self.dtype, self.depth = device, dtype, depth
        self._free: dict = {}
        self._count: dict = {}
        self.allocated = 0

    def get(self, key, numel, stream):
        lst = self._free.get(key)
        if self._count.get(key, 0) < self.depth or not lst:
            self._count[key] = self._count.get(key, 0) + 1
            self.allocated += 1
            return torch.zeros(numel, dtype=self.dtype, device=self.device)  # padding stays zero for good
        t, ev = lst.pop(0)
        if ev is not None and stream is not None:
            stream.wait_event(ev)
        return t

    def put(self, key, tensor, event):
        self._free.setdefault(key, []).append((tensor, event))


SHARDED, PENDING, UNSHARDED = 0, 1, 2


class ShardGroup:
    def __init__(self, spec: GroupSpec, slots: list, world: int, index: int):
        self.spec, self.name, self.slots, self.index = spec, spec.name, slots, index
        end = slots[-1].offset + slots[-1].numel if slots else 0
        self.numel = end
        self.padded = _round_up(max(end, 1), world * SHARD_ALIGN)
        self.shard_numel = self.padded // world
        self.layout_key = (self.padded,) + tuple((s.offset, s.numel) for s in slots)
        self.state = SHARDED
        self.full = None          # gathered flat parameters (compute dtype)
        self.full_grad = None     # flat gradients (compute dtype)
        self.ag_event = None
        self.shard = None         # view of the master tensor
        self.shard_c = None       # the same shard in the compute dtype (what the all-gather sends)
        self.grad_shard = None    # view of the gradient tensor
        self.ag_hook = None
        self.rs_hook = None
        self.grads_ready = False  # gradient buffer handed out for this backward
        self.view_cache = {}      # (buffer address, dtype) -> (buffer, per-parameter views)


@dataclass
class FlatShardPlan:
    ag_hook_factory: Optional[Callable[[], object]] = None
    rs_hook_factory: Optional[Callable[[], object]] = None
    forward_prefetch_distance: int = 1
    # True: a group's gathered parameters are released after its forward and gathered again for its
    # backward (ZeRO-3, what the reference asks FSDP2 for, reference: train.py:94).  False: they are
    # kept until the group's backward, which halves the all-gathers of a step.  "auto": keep them when
    # all gathered parameters together take less than `keep_params_fraction` of the device's memory
    # (16 GB of a 180 GB B200 for an 8B model), release them otherwise.
    reshard_after_forward: object = "auto"
    keep_params_fraction: float = 0.2
    compute_dtype: torch.dtype = torch.bfloat16
    master_dtype: torch.dtype = torch.bfloat16
    act_ckpt: bool = False
    prefetch_next_step: bool = True
    time_collectives: bool = False   # bracket every collective with CUDA events (read by comm_stats)


class _PostBackward(torch.autograd.Function):
    """Identity on a group's inputs whose backward runs once the group's backward is complete."""

    @staticmethod
    def forward(ctx, engine, group, *inputs):
        ctx.engine, ctx.group = engine, group
        ctx.set_materialize_grads(False)
        return inputs

    @staticmethod
    def backward(ctx, *grads):
        ctx.engine._post_backward(ctx.group)
        return (None, None) + grads


class FlatShardEngine:
    """Owns the sharded storage of ``model`` and drives gather / compute / reduce for one step.

    Usage::

        eng = FlatShardEngine(model_on_meta, groups, plan, device)
        eng.begin_step(); out = model(...); eng.backward(out.loss); eng.optimizer_step(opt)
    """

    def __init__(self, model: nn.Module, specs: list, plan: FlatShardPlan, device: torch.device,
                 process_group=None):
        self.model, self.plan, self.device = model, plan, device
        self.pg = process_group if process_group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.pg)
        self.rank = dist.get_rank(self.pg)
        self.cuda = device.type == "cuda"
        self.in_backward = False
        self._rs_events: list = []
        self._comm_log: list = []   # (kind, start event, end event, payload bytes)
        self._shards_ready = None
        cd = plan.compute_dtype

        # ---- group layout ------------------------------------------------------------------
        self._realize_parameters()
        fqn_of = {id(p): n for n, p in model.named_parameters(remove_duplicate=True)}
        seen: set = set()
        self.groups: list[ShardGroup] = []
        for gi, spec in enumerate(specs):
            slots, off = [], 0
            plist = [p for m in spec.modules for p in m.parameters()] + list(spec.extra_params)
            for p in plist:
                if id(p) in seen:
                    continue
                seen.add(id(p))
                off = _round_up(off, PARAM_ALIGN)
                numel = 1
                for d in p.full_shape:
                    numel *= d
                slots.append(_Slot(p, fqn_of[id(p)], off, numel, p.full_shape))
                off += numel
            self.groups.append(ShardGroup(spec, slots, self.world, gi))
        missing = [n for n, p in model.named_parameters() if id(p) not in seen]
        if missing:
            raise ValueError(f"parameters outside every shard group: {missing[:4]} ...")

        # ---- persistent storage: one tensor per role over all groups --------------------------
        total = sum(g.shard_numel for g in self.groups)
        self.master = torch.zeros(total, dtype=plan.master_dtype, device=device)
        grad_dtype = cd if (self.world == 1 or plan.master_dtype == cd) else torch.float32
        self.grad_master = torch.zeros(total, dtype=grad_dtype, device=device)
        self.master_c = self.master if plan.master_dtype == cd else torch.zeros(total, dtype=cd, device=device)
        off = 0
        for g in self.groups:
            g.shard = self.master[off:off + g.shard_numel]
            g.shard_c = self.master_c[off:off + g.shard_numel]
            g.grad_shard = self.grad_master[off:off + g.shard_numel]
            off += g.shard_numel
            g.ag_hook = plan.ag_hook_factory() if plan.ag_hook_factory else PlainAllGather()
            g.rs_hook = plan.rs_hook_factory() if plan.rs_hook_factory else PlainReduceScatter()
        self.master_param = nn.Parameter(self.master, requires_grad=True)
        self.master_param.grad = self.grad_master

        # parameters: the group computing, the one being gathered, one draining; gradients: the group
        # being written, the one being reduce-scattered
        self._param_pool = _Pool(device, cd, depth=3)
        self._grad_pool = _Pool(device, cd, depth=2)
        if self.cuda:
            self.ag_stream = torch.cuda.Stream(device, priority=-1)
            self.rs_stream = torch.cuda.Stream(device, priority=-1)
        else:
            self.ag_stream = self.rs_stream = None

        raf = plan.reshard_after_forward
        if raf == "auto":
            full_bytes = sum(g.padded for g in self.groups) * torch.empty(0, dtype=cd).element_size()
            if self.cuda and self.world > 1:
                total_mem = torch.cuda.get_device_properties(device).total_memory
                raf = full_bytes > plan.keep_params_fraction * total_mem
            else:
                raf = True
        self.reshard_after_forward = bool(raf)
        self._materialize()
        self._install_hooks()
        if plan.act_ckpt:
            model.activation_checkpointing = True

    # ------------------------------------------------------------------------------------------
    # construction helpers
    # ------------------------------------------------------------------------------------------
    def _realize_parameters(self) -> None:
        """Swap every (meta-device) parameter for an empty one on the device; the full shape is kept
        on the parameter as ``full_shape``.  A parameter shared by several modules stays shared."""
        cd, repl = self.plan.compute_dtype, {}
        for mod in self.model.modules():
            for name, p in list(mod._parameters.items()):
                if p is None:
                    continue
                q = repl.get(id(p))
                if q is None:
                    q = nn.Parameter(torch.empty(0, dtype=cd, device=self.device), requires_grad=p.requires_grad)
                    q.full_shape = tuple(p.shape)
                    repl[id(p)] = q
                mod._parameters[name] = q

    @staticmethod
    def _slot_views(g: ShardGroup, flat: torch.Tensor):
        """Per-parameter views of a flat buffer of this group's layout.  The buffers come from small
        pools and return every step, so the views are made once per buffer and kept (with a reference
        to the buffer, which makes its address a safe key): a step then costs one attribute store per
        parameter instead of a slice, a view and their dispatch."""
        key = (flat.data_ptr(), flat.dtype)
        hit = g.view_cache.get(key)
        if hit is None:
            if len(g.view_cache) >= 8:
                g.view_cache.pop(next(iter(g.view_cache)))
            hit = (flat, [flat[s.offset:s.offset + s.numel].view(s.shape) for s in g.slots])
            g.view_cache[key] = hit
        return hit[1]

    def _replace_param_storage(self, g: ShardGroup, flat: torch.Tensor) -> None:
        for s, v in zip(g.slots, self._slot_views(g, flat)):
            s.param.data = v

    def _materialize(self) -> None:
        """Initialise every group's parameters (the same values on every rank: every rank draws the
        full group from the same generator state) and keep this rank's slice."""
        cd = self.plan.compute_dtype
        for g in self.groups:
            flat = torch.zeros(g.padded, dtype=self.plan.master_dtype, device=self.device)
            for s in g.slots:
                s.param.data = flat[s.offset:s.offset + s.numel].view(s.shape)
            for m in g.spec.modules:
                for sub in m.modules():
                    if hasattr(sub, "reset_parameters"):
                        sub.reset_parameters()
            g.shard.copy_(flat[self.rank * g.shard_numel:(self.rank + 1) * g.shard_numel])
            del flat
        self._sync_compute_copy()
        for g in self.groups:
            if self.world == 1:
                g.full, g.full_grad, g.state = g.shard_c, g.grad_shard, UNSHARDED
                self._replace_param_storage(g, g.full)
                self._set_main_grads(g)
            else:
                for s in g.slots:
                    s.param.data = torch.empty(0, dtype=cd, device=self.device)
        self._record_shards_ready()

    def _sync_compute_copy(self) -> None:
        if self.master_c is not self.master:
            self.master_c.copy_(self.master)

    def _record_shards_ready(self) -> None:
        if self.cuda:
            self._shards_ready = torch.cuda.Event()
            self._shards_ready.record(torch.cuda.current_stream(self.device))

    def _install_hooks(self) -> None:
        for g in self.groups:
            first, last = g.spec.modules[0], g.spec.modules[-1]
            first.register_forward_pre_hook(self._make_pre_forward(g), with_kwargs=True)
            last.register_forward_hook(self._make_post_forward(g))

    # ------------------------------------------------------------------------------------------
    # gather / release
    # ------------------------------------------------------------------------------------------
    def _current(self):
        return torch.cuda.current_stream(self.device) if self.cuda else None

    def _stamp(self, stream):
        if not (self.cuda and self.plan.time_collectives):
            return None
        ev = torch.cuda.Event(enable_timing=True)
        ev.record(stream)
        return ev

    def comm_stats(self, reset: bool = True) -> dict:
        """Device time of the collectives logged since the last call (needs ``time_collectives``):
        per kind the number of calls, the summed milliseconds on this rank and the bus bandwidth
        ``payload * (W-1)/W / time`` in GB/s, with the payload counted uncompressed (what a plain
        collective would move), as nccl-tests does.  The ``*_exposed`` kinds are the time the compute
        stream stood still waiting for a gather / for the last reduce-scatters, i.e. the part of the
        communication that nothing overlapped.  Synchronises on the last logged event."""
        out: dict = {}
        if not self._comm_log:
            return out
        self._comm_log[-1][2].synchronize()
        for kind, a, b, nbytes in self._comm_log:
            if not b.query():
                b.synchronize()
            d = out.setdefault(kind, {"calls": 0, "ms": 0.0, "bytes": 0})
            d["calls"] += 1
            d["ms"] += a.elapsed_time(b)
            d["bytes"] += nbytes
        for d in out.values():
            d["bus_gbs"] = d["bytes"] * (self.world - 1) / self.world / max(d["ms"], 1e-9) / 1e6 if d["bytes"] else None
        if reset:
            self._comm_log.clear()
        return out

    def _issue_unshard(self, g: ShardGroup, urgent: bool = False) -> None:
        if g.state != SHARDED or self.world == 1:
            return
        if hasattr(g.ag_hook, "urgent"):
            g.ag_hook.urgent = urgent
        buf = self._param_pool.get(g.layout_key, g.padded, self.ag_stream)
        if self.cuda:
            self.ag_stream.wait_event(self._shards_ready)
            with torch.cuda.stream(self.ag_stream):
                t0 = self._stamp(self.ag_stream)
                g.ag_hook(buf, g.shard_c, self.pg)
                g.ag_event = torch.cuda.Event(enable_timing=self.plan.time_collectives)
                g.ag_event.record(self.ag_stream)
                if t0 is not None:
                    self._comm_log.append(("all_gather", t0, g.ag_event, g.padded * buf.element_size()))
        else:
            g.ag_hook(buf, g.shard_c, self.pg)
        g.full = buf
        self._replace_param_storage(g, buf)
        g.state = PENDING

    def _wait_unshard(self, g: ShardGroup) -> None:
        if g.state == SHARDED:
            self._issue_unshard(g, urgent=True)  # nobody prefetched it: the step is waiting
        if g.state == PENDING:
            if g.ag_event is not None:
                cur = self._current()
                t0 = self._stamp(cur)
                cur.wait_event(g.ag_event)
                if t0 is not None:   # how long compute stood still for this gather
                    self._comm_log.append(("all_gather_exposed", t0, self._stamp(cur), 0))
                g.ag_event = None
            g.state = UNSHARDED

    def _reshard(self, g: ShardGroup) -> None:
        if self.world == 1 or g.state == SHARDED:
            return
        self._wait_unshard(g)  # never hand back a buffer a collective is still writing
        ev = None
        if self.cuda:
            ev = torch.cuda.Event()
            ev.record(self._current())
        self._param_pool.put(g.layout_key, g.full, ev)
        g.full = None
        g.state = SHARDED

    # ------------------------------------------------------------------------------------------
    # gradients
    # ------------------------------------------------------------------------------------------
    def _set_main_grads(self, g: ShardGroup) -> None:
        for s, v in zip(g.slots, self._slot_views(g, g.full_grad)):
            s.param.main_grad = v
            s.param.main_grad_written = False

    def _prepare_grads(self, g: ShardGroup) -> None:
        if g.grads_ready:
            return
        if self.world > 1:
            g.full_grad = self._grad_pool.get(g.layout_key, g.padded, self._current())
            self._set_main_grads(g)
        else:
            for s in g.slots:
                s.param.main_grad_written = False
        g.grads_ready = True

    def _collect_grads(self, g: ShardGroup) -> None:
        """Gradients that autograd produced as ``.grad`` move into the flat buffer; parameters that
        received none are zeroed.  Ops that wrote ``main_grad`` themselves are left alone."""
        with torch.no_grad():
            for s in g.slots:
                p = s.param
                if p.grad is not None:
                    if p.main_grad_written:
                        p.main_grad.add_(p.grad.to(p.main_grad.dtype))
                    else:
                        p.main_grad.copy_(p.grad)
                    p.grad = None
                    p.main_grad_written = True
                elif not p.main_grad_written:
                    p.main_grad.zero_()

    def _post_backward(self, g: ShardGroup) -> None:
        if not g.grads_ready or (g.spec.persistent and self.in_backward):
            return
        self._collect_grads(g)
        g.grads_ready = False
        if self.world == 1:
            return
        self._reshard(g)
        if self.cuda:
            ev = torch.cuda.Event()
            ev.record(self._current())
            self.rs_stream.wait_event(ev)
            if hasattr(g.rs_hook, "urgent"):
                # backward of the groups before this one is still to come, except at the very end
                g.rs_hook.urgent = not self.in_backward or g.index <= 1
            with torch.cuda.stream(self.rs_stream):
                t0 = self._stamp(self.rs_stream)
                g.rs_hook(g.grad_shard, g.full_grad, self.pg, op=dist.ReduceOp.AVG)
                done = torch.cuda.Event(enable_timing=self.plan.time_collectives)
                done.record(self.rs_stream)
                if t0 is not None:
                    self._comm_log.append(("reduce_scatter", t0, done, g.padded * g.full_grad.element_size()))
            self._rs_events.append(done)
        else:
            g.rs_hook(g.grad_shard, g.full_grad, self.pg, op=dist.ReduceOp.AVG)
            done = None
        for s in g.slots:
            s.param.main_grad = None
        self._grad_pool.put(g.layout_key, g.full_grad, done)
        g.full_grad = None

    # ------------------------------------------------------------------------------------------
    # module hooks
    # ------------------------------------------------------------------------------------------
    def _make_pre_forward(self, g: ShardGroup):
        def hook(module, args, kwargs):
            self._wait_unshard(g)
            if not self.in_backward:
                d = self.plan.forward_prefetch_distance
                for nxt in self.groups[g.index + 1: g.index + 1 + d]:
                    self._issue_unshard(nxt)
            if not torch.is_grad_enabled():
                return None
            flat = list(args)
            idx = [i for i, a in enumerate(flat) if torch.is_tensor(a) and a.requires_grad]
            if not idx:
                return None
            outs = _PostBackward.apply(self, g, *[flat[i] for i in idx])
            for i, o in zip(idx, outs):
                flat[i] = o
            return tuple(flat), kwargs

        return hook

    def _make_post_forward(self, g: ShardGroup):
        def pre_backward(grad):
            self._pre_backward(g)
            return grad

        def hook(module, args, output):
            if torch.is_grad_enabled():
                outs = output if isinstance(output, (tuple, list)) else (output,)
                for o in outs:
                    if torch.is_tensor(o) and o.requires_grad:
                        o.register_hook(pre_backward)
            if self.in_backward or g.spec.persistent:
                return None
            last = g.index == len(self.groups) - 1
            if (self.reshard_after_forward or not torch.is_grad_enabled()) and not (last and torch.is_grad_enabled()):
                self._reshard(g)
            return None

        return hook

    def _pre_backward(self, g: ShardGroup) -> None:
        if g.grads_ready:
            return
        if g.spec.backward_needs_params:
            self._wait_unshard(g)
        self._prepare_grads(g)
        # the group computed before this one in forward is the next one backward reaches
        for j in range(g.index - 1, -1, -1):
            prev = self.groups[j]
            if prev.spec.backward_needs_params and not prev.spec.persistent:
                self._issue_unshard(prev)
                break

    # ------------------------------------------------------------------------------------------
    # step API
    # ------------------------------------------------------------------------------------------
    def begin_step(self) -> None:
        """Start gathering the first groups (the counterpart of the reference loop's
        ``model.unshard()``, reference: train.py:241)."""
        if self.world == 1:
            return
        for g in self.groups:
            if g.spec.persistent:
                self._issue_unshard(g, urgent=True)
        n = 1 + max(0, self.plan.forward_prefetch_distance)
        for g in self.groups[:n]:
            self._issue_unshard(g, urgent=True)  # nothing to hide behind at the start of a step

    def backward(self, loss: torch.Tensor) -> None:
        self.in_backward = True
        try:
            for g in self.groups:
                if g.spec.persistent:
                    self._pre_backward(g)
            from ..ops.loss import unit_loss_grad

            with unit_loss_grad():   # the loss is the root of this backward pass
                loss.backward()
        finally:
            self.in_backward = False
        # groups whose inputs carry no gradient (embedding) and persistent groups finish here
        for g in reversed(self.groups):
            if g.grads_ready:
                self._post_backward(g)
        for g in self.groups:
            self._reshard(g)

    def wait_for_gradients(self) -> None:
        if self.cuda:
            cur = self._current()
            t0 = self._stamp(cur) if self._rs_events else None
            for ev in self._rs_events:
                cur.wait_event(ev)
            if t0 is not None:       # how long the optimizer waited for the last reduce-scatters
                self._comm_log.append(("reduce_scatter_exposed", t0, self._stamp(cur), 0))
        self._rs_events.clear()

    def optimizer_step(self, optimizer, lr_scheduler=None) -> None:
        """Update all shards, then start the next step's first gathers.  With more than one rank and
        a ``FusedAdamW`` the update is cut in two: the shards of the first groups (whose gathers the
        next forward waits for) are updated first, their gathers start, and the rest of the update
        runs beside them."""
        self.wait_for_gradients()
        self.master_param.grad = self.grad_master
        early = self._early_groups() if (self.world > 1 and self.plan.prefetch_next_step and self.cuda
                                         and self.master_c is self.master) else []
        if early and hasattr(optimizer, "kernel_launches"):
            cut = sum(g.shard_numel for g in self.groups[:len(early)])

            def start_first_gathers():
                self._record_shards_ready()
                for g in early:
                    self._issue_unshard(g, urgent=True)

            optimizer.step(split_at=cut, between=start_first_gathers)
        else:
            optimizer.step()
        if lr_scheduler is not None:
            lr_scheduler.step()
        self._sync_compute_copy()
        self._record_shards_ready()
        if self.plan.prefetch_next_step:
            self.begin_step()

    def _early_groups(self) -> list:
        """The leading groups whose gathers ``begin_step`` issues (a prefix of the group list; persistent
        groups elsewhere in the list are left to ``begin_step``)."""
        n = 1 + max(0, self.plan.forward_prefetch_distance)
        return list(self.groups[:n])

    # ------------------------------------------------------------------------------------------
    # state
    # ------------------------------------------------------------------------------------------
    def parameters_for_optimizer(self):
        return [self.master_param]

    def _gather_full(self, flat_shard: torch.Tensor, g: ShardGroup) -> torch.Tensor:
        if self.world == 1:
            return flat_shard
        out = torch.empty(g.padded, dtype=flat_shard.dtype, device=flat_shard.device)
        dist.all_gather_into_tensor(out, flat_shard.contiguous(), group=self.pg)
        return out

    def full_state_dict(self) -> dict:
        """Unsharded parameters by fully-qualified name, on the CPU (collective)."""
        sd = {}
        for g in self.groups:
            full = self._gather_full(g.shard, g)
            for s in g.slots:
                sd[s.fqn] = full[s.offset:s.offset + s.numel].view(s.shape).detach().cpu().clone()
        return sd

    def load_full_state_dict(self, sd: dict) -> None:
        with torch.no_grad():
            for g in self.groups:
                flat = torch.zeros(g.padded, dtype=self.plan.master_dtype, device=self.device)
                for s in g.slots:
                    flat[s.offset:s.offset + s.numel].copy_(sd[s.fqn].reshape(-1).to(self.device))
                g.shard.copy_(flat[self.rank * g.shard_numel:(self.rank + 1) * g.shard_numel])
        self._sync_compute_copy()
        self._record_shards_ready()

    def sharded_tensors(self, optimizer=None) -> dict:
        """``{name: local flat shard}`` of every group (and of the optimizer moments when given):
        the tensors a sharded checkpoint stores.  Views, so loading into them is in place."""
        out = {f"model.{g.name}": g.shard for g in self.groups}
        if optimizer is not None:
            optimizer.ensure_state()
            st = optimizer.state[self.master_param]
            off = 0
            for g in self.groups:
                out[f"optim.exp_avg.{g.name}"] = st["exp_avg"][off:off + g.shard_numel]
                out[f"optim.exp_avg_sq.{g.name}"] = st["exp_avg_sq"][off:off + g.shard_numel]
                off += g.shard_numel
        return out

    def after_load(self) -> None:
        self._sync_compute_copy()
        self._record_shards_ready()

    def memory_summary(self) -> dict:
        return {"param_buffers": self._param_pool.allocated, "grad_buffers": self._grad_pool.allocated,
                "shard_elements": int(self.master.numel()), "reshard_after_forward": self.reshard_after_forward}
