"""Sharded checkpoint save / resume in the reference's layout (reference: train.py:151-205,
297-311): ``<exp_dir>/checkpoint`` is a PyTorch DCP directory with the sharded ``model`` and
``optimizer`` state dicts (``StateDictOptions(full_state_dict=False, cpu_offload=True)``), rank 0
writes ``lr_scheduler.pt`` and ``state.json``.  In addition every rank writes
``rank-<r>/comm_state.pt`` with the error-feedback residuals of its reduce-scatter hooks: they
are per-rank, unsharded-size training state that the reference does not have.

The flat-shard engine stores the same container (a DCP directory of ``Shard(0)`` DTensors plus the
two side files), but its entries are the groups' flat shards (``model.<group>``,
``optim.exp_avg.<group>``, ``optim.exp_avg_sq.<group>``) rather than one entry per parameter;
``FlatShardEngine.full_state_dict()`` gives the per-parameter view by fully-qualified name."""
from __future__ import annotations

import json
from pathlib import Path

import torch
import torch.distributed as dist
from torch.distributed.checkpoint import load, save
from torch.distributed.checkpoint.state_dict import StateDictOptions, get_state_dict, set_state_dict

CKPT_OPTS = StateDictOptions(full_state_dict=False, cpu_offload=True)


def _barrier():
    if dist.is_initialized():
        dist.barrier()


def save_checkpoint(exp_dir: Path, model, optimizer, lr_scheduler, state: dict, rs_hooks=()) -> None:
    rank = dist.get_rank() if dist.is_initialized() else 0
    _barrier()
    model_sd, optim_sd = get_state_dict(model, optimizer, options=CKPT_OPTS)  # on ALL ranks
    save(dict(model=model_sd, optimizer=optim_sd), checkpoint_id=exp_dir / "checkpoint")
    if rs_hooks:
        rdir = exp_dir / f"rank-{rank}"
        rdir.mkdir(parents=True, exist_ok=True)
        torch.save([h.state_dict() for h in rs_hooks], rdir / "comm_state.pt")
    if rank == 0:
        torch.save(lr_scheduler.state_dict(), exp_dir / "lr_scheduler.pt")
        with open(exp_dir / "state.json", "w") as fp:
            json.dump(state, fp)
    _barrier()


def try_resume(exp_dir: Path, model, optimizer, lr_scheduler, device, rs_hooks=()):
    """Returns the saved ``state`` dict when ``state.json`` exists, else ``None``."""
    if not (exp_dir / "state.json").exists():
        return None
    rank = dist.get_rank() if dist.is_initialized() else 0
    model_sd, optim_sd = get_state_dict(model, optimizer, options=CKPT_OPTS)
    load(dict(model=model_sd, optimizer=optim_sd), checkpoint_id=exp_dir / "checkpoint")
    set_state_dict(model, optimizer, model_state_dict=model_sd, optim_state_dict=optim_sd, options=CKPT_OPTS)
    lr_scheduler.load_state_dict(torch.load(exp_dir / "lr_scheduler.pt", map_location=device, weights_only=True))
    comm = exp_dir / f"rank-{rank}" / "comm_state.pt"
    if rs_hooks and comm.exists():
        states = torch.load(comm, map_location="cpu", weights_only=True)
        _load_residuals(rs_hooks, states, device)
    with open(exp_dir / "state.json") as fp:
        return json.load(fp)


def _load_residuals(rs_hooks, states, device) -> None:
    """Residuals are stored per hook in installation order; a count or size mismatch means the
    checkpoint belongs to another model or world size and is refused rather than misapplied."""
    if len(states) != len(rs_hooks):
        raise ValueError(f"checkpoint has residuals of {len(states)} reduce-scatter hooks, the model has {len(rs_hooks)}")
    for h, s in zip(rs_hooks, states):
        h.load_state_dict(s, device=device)


# ---------------------------------------------------------------------------------------------
# flat-shard engine
# ---------------------------------------------------------------------------------------------
def _flat_state(flat, optimizer) -> dict:
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.tensor import DTensor, Shard

    mesh = getattr(flat, "_ckpt_mesh", None)
    if mesh is None:
        mesh = flat._ckpt_mesh = init_device_mesh(flat.device.type, (flat.world,))
    sd = {k: DTensor.from_local(t, mesh, [Shard(0)], run_check=False)
          for k, t in flat.sharded_tensors(optimizer).items()}
    sd["optim.step"] = optimizer.state[flat.master_param]["step"]
    return sd


def save_flat_checkpoint(exp_dir: Path, flat, optimizer, lr_scheduler, state: dict, rs_hooks=()) -> None:
    rank = dist.get_rank() if dist.is_initialized() else 0
    _barrier()
    save(_flat_state(flat, optimizer), checkpoint_id=exp_dir / "checkpoint")
    if rs_hooks:
        rdir = exp_dir / f"rank-{rank}"
        rdir.mkdir(parents=True, exist_ok=True)
        torch.save([h.state_dict() for h in rs_hooks], rdir / "comm_state.pt")
    if rank == 0:
        torch.save(lr_scheduler.state_dict(), exp_dir / "lr_scheduler.pt")
        with open(exp_dir / "state.json", "w") as fp:
            json.dump(state, fp)
    _barrier()


def try_resume_flat(exp_dir: Path, flat, optimizer, lr_scheduler, device, rs_hooks=()):
    if not (exp_dir / "state.json").exists():
        return None
    rank = dist.get_rank() if dist.is_initialized() else 0
    sd = _flat_state(flat, optimizer)
    load(sd, checkpoint_id=exp_dir / "checkpoint")   # in place: the entries are views of the engine's storage
    optimizer.state[flat.master_param]["step"].copy_(sd["optim.step"])
    flat.after_load()
    lr_scheduler.load_state_dict(torch.load(exp_dir / "lr_scheduler.pt", map_location=device, weights_only=True))
    comm = exp_dir / f"rank-{rank}" / "comm_state.pt"
    if rs_hooks and comm.exists():
        states = torch.load(comm, map_location="cpu", weights_only=True)
        _load_residuals(rs_hooks, states, device)
    with open(exp_dir / "state.json") as fp:
        return json.load(fp)
