"""FSDP2 training entry point with compressed collectives.

Keeps every flag of the reference script (reference: train.py:426-448) and its loop structure
(reference: train.py:229-311: ``model.unshard()`` -> batch to device -> forward -> backward ->
optimizer / LR step -> zero_grad -> profiler step -> logging -> checkpoint), and adds

  --synthetic / --model-shape   build a named shape locally and train on random tokens
                                (the reference needs the HF hub for config, tokenizer and data)
  --device {auto,cuda,cpu}      CPU runs use gloo and the scalar codec
  --compress-rs                 compressed gradient reduce-scatter with error feedback
  --act-ckpt                    activation checkpointing per decoder block
  --steps N                     stop after N optimizer steps
  --transport / --codec         symm | lib | auto,  v1 | v2 | auto
  --wire                        auto | nibble | compressed | verbatim (cheap 4-bit codes, bit planes, raw bf16;
                                auto = nibble on the fused transport, bit planes on the library transport)
  --master-dtype fp32           keep fp32 master weights (communication stays bf16)
  --sharding {flat,fsdp2}       the package's flat-shard ZeRO-3 engine (default) or PyTorch FSDP2
                                (the reference's wrapping; chosen automatically for --cpu-offload)

``-m`` takes a named shape, the hub id of one (``openai-community/gpt2-xl``) or a local directory
with a HF ``config.json``.  Phases are timed with CUDA events (no synchronisation inside a step);
every ``--log-freq`` steps the log also carries the device time and bus bandwidth of the
collectives and the wire bytes per element of the compressed ones.  Expired device-side waits
are checked next to the loss read of every step and before every checkpoint.
``ZC_FAULT_INJECT="rank=1,step=3,kind=raise"`` makes a rank fail on the host between steps.

Launch: ``torchrun --nproc-per-node N --master-addr 127.0.0.1 train.py --synthetic ...``.
"""
from __future__ import annotations

import argparse
import contextlib
import math
import os
from pathlib import Path

import torch
from torch import distributed as dist
from torch.distributed.elastic.multiprocessing.errors import record
from torch.profiler import ProfilerActivity
from torch.utils.data import DataLoader
from torch.utils.data.distributed import DistributedSampler

from fsdp_comm_opt_b200.engine import EngineConfig, build_sharded
from fsdp_comm_opt_b200.models import get_config
from fsdp_comm_opt_b200.ops.adamw import FusedAdamW
from fsdp_comm_opt_b200.ops.loss import unit_loss_grad
from fsdp_comm_opt_b200.parallel.fsdp import comm_report
from fsdp_comm_opt_b200.utils import checkpoint as ckpt
from fsdp_comm_opt_b200.utils.data import SyntheticTokens, collate, load_text_dataset
from fsdp_comm_opt_b200.utils.dist import all_reduce_max, init_distributed, rank0_first
from fsdp_comm_opt_b200.utils.failure import FaultInjector, Heartbeat
from fsdp_comm_opt_b200.utils.health import check_device_status
from fsdp_comm_opt_b200.utils.metrics import get_mem_stats, setup_logging
from fsdp_comm_opt_b200.utils.timing import PhaseTimer


def _get_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser()
    # reference flags
    p.add_argument("-e", "--experiment-name", default=None)
    p.add_argument("-d", "--dataset-name", default=None)
    p.add_argument("--dataset-subset", default=None)
    p.add_argument("-m", "--model-name", default=None)
    p.add_argument("--save-dir", default="../outputs")
    p.add_argument("--seed", default=0, type=int)
    p.add_argument("--num-epochs", default=100, type=int)
    p.add_argument("--lr", default=3e-5, type=float)
    p.add_argument("-b", "--batch-size", default=1, type=int)
    p.add_argument("--log-freq", default=10, type=int)
    p.add_argument("--ckpt-freq", default=500, type=int)
    p.add_argument("-s", "--seq-length", default=1024, type=int)
    p.add_argument("--cpu-offload", default=False, action="store_true")
    p.add_argument("-p", "--profiler", default=False, action="store_true")
    p.add_argument("--profiler-wait", default=10, type=int)
    p.add_argument("--profiler-warmup", default=5, type=int)
    p.add_argument("--profiler-active", default=2, type=int)
    p.add_argument("--forward-prefetch-distance", default=1, type=int)
    p.add_argument("-q", "--quantize", default=False, action="store_true")
    p.add_argument("--zip-ccl", default=False, action="store_true")
    # additions
    p.add_argument("--synthetic", default=False, action="store_true")
    p.add_argument("--model-shape", default=None, help="tiny | small | llama3-8b | llama2-13b | 34b | gpt2-tiny | gpt2-xl")
    p.add_argument("--device", default="auto", choices=["auto", "cuda", "cpu"])
    p.add_argument("--compress-rs", default=False, action="store_true")
    p.add_argument("--no-error-feedback", default=False, action="store_true")
    p.add_argument("--act-ckpt", default=False, action="store_true")
    p.add_argument("--steps", default=None, type=int)
    p.add_argument("--transport", default="auto", choices=["auto", "symm", "lib"])
    p.add_argument("--codec", default="auto", choices=["auto", "v1", "v2"])
    p.add_argument("--wire", default="auto", choices=["auto", "nibble", "compressed", "verbatim"],
                   help="what the fused collectives move: lossless exponent-coded records with 4-bit codes (nibble), "
                        "with bit planes (compressed: smallest wire, more codec work), or the raw bf16 bytes on the "
                        "same one-kernel protocol (verbatim)")
    p.add_argument("--master-dtype", default="bf16", choices=["bf16", "fp32"])
    p.add_argument("--num-samples", default=1 << 14, type=int, help="synthetic dataset length")
    p.add_argument("--heartbeat-timeout", default=0.0, type=float,
                   help="> 0: ranks publish a heartbeat each step and abort when a peer is silent that long")
    p.add_argument("--loss-log", default=None, help="rank 0 appends 'step loss' lines to this file")
    p.add_argument("--sharding", default="flat", choices=["flat", "fsdp2"])
    p.add_argument("--reshard-after-forward", default="auto", choices=["auto", "true", "false"],
                   help="flat sharding: release gathered parameters after forward (the reference's ZeRO-3 setting), keep "
                        "them until backward, or decide by the memory they take (auto)")
    p.add_argument("--dist-timeout", default=None, type=float,
                   help="seconds after which a collective whose peer never joins fails instead of waiting "
                        "(process-group timeout; the default is the backend's)")
    p.add_argument("--tokenizer", default=None,
                   help="tokenizer name or local directory for text data (default: the model name; 'bytes' = built-in byte-level)")
    return p


def _comm_metrics(flat, plan, steps: int, device) -> dict:
    """Per-step device time (max over ranks) and bus GB/s of the collectives since the last log line,
    and the wire bytes per element of the fused compressed channels (compression ratio = that / 2)."""
    out: dict = {}
    if flat is not None:
        for kind, d in flat.comm_stats().items():
            out[f"comm/{kind}_ms_per_step"] = all_reduce_max(d["ms"] / max(steps, 1), device)
            if d["bus_gbs"] is not None:
                out[f"comm/{kind}_bus_gbs"] = d["bus_gbs"]
    if device.type == "cuda":
        rep = comm_report(plan)
        out["comm/transport"] = {"all_gather": rep["all_gather"], "reduce_scatter": rep["reduce_scatter"]}
        for kind, ch in rep["channels"].items():
            if ch["wire_bytes_per_element"] is not None:
                out[f"comm/{kind}_wire_bytes_per_elem"] = ch["wire_bytes_per_element"]
                out[f"comm/{kind}_ratio_vs_bf16"] = ch["wire_bytes_per_element"] / 2.0
    return out


@record
def main(argv=None):
    args = _get_parser().parse_args(argv)
    if not args.synthetic and (args.dataset_name is None or args.model_name is None):
        raise SystemExit("either --synthetic with --model-shape, or -d/--dataset-name and -m/--model-name")

    rank, world_size, device = init_distributed(args.device, timeout_s=args.dist_timeout)
    local_rank = device.index or 0
    LOGGER = setup_logging(rank)
    LOGGER.debug(os.environ)
    LOGGER.debug(args)

    master_dtype = torch.bfloat16 if args.master_dtype == "bf16" else torch.float32
    torch.manual_seed(args.seed)

    # ---- model on the meta device (no memory), shard, then materialise the shards ---------------
    shape_name = args.model_shape or args.model_name
    cfg = get_config(shape_name)
    sharding = "fsdp2" if args.cpu_offload else args.sharding
    ecfg = EngineConfig(model=cfg, lr=args.lr, master_dtype=master_dtype, quantize=args.quantize,
                        zip_ccl=args.zip_ccl, compress_rs=args.compress_rs, act_ckpt=args.act_ckpt,
                        forward_prefetch_distance=args.forward_prefetch_distance, transport=args.transport,
                        codec_version=args.codec, wire=args.wire, seed=args.seed, sharding=sharding, cpu_offload=args.cpu_offload,
                        error_feedback=not args.no_error_feedback, time_collectives=True,
                        reshard_after_forward={"auto": "auto", "true": True, "false": False}[args.reshard_after_forward])
    model, plan, flat = build_sharded(ecfg, device)
    LOGGER.info(f"Training {cfg.num_params()} model parameters ({sharding} sharding)")
    LOGGER.info(f"Initialized model uses {get_mem_stats(device)['curr_alloc_gb']}gb")

    # ---- data ---------------------------------------------------------------------------------
    if args.synthetic:
        train_data = SyntheticTokens(cfg.vocab_size, args.seq_length, args.num_samples, args.seed)
    else:
        with rank0_first():
            train_data = load_text_dataset(args.dataset_name, args.dataset_subset,
                                           args.tokenizer or args.model_name, args.seq_length, cfg.max_seq,
                                           vocab_size=cfg.vocab_size)
    dataloader = DataLoader(train_data, batch_size=args.batch_size, collate_fn=collate,
                            sampler=DistributedSampler(train_data, shuffle=True, drop_last=True))
    LOGGER.debug(f"{len(dataloader)} batches per epoch")

    optimizer = FusedAdamW(flat.parameters_for_optimizer() if flat is not None else model.parameters(), lr=args.lr)
    lr_scheduler = torch.optim.lr_scheduler.CosineAnnealingLR(optimizer, T_max=1000, eta_min=args.lr * 1e-2)

    # ---- experiment directory / resume --------------------------------------------------------
    is_experiment = args.experiment_name is not None
    exp_dir = Path(args.save_dir)
    if is_experiment:
        exp_dir = exp_dir / args.experiment_name
    state = {"epoch": 0, "global_step": 0, "epoch_step": 0, "running_loss": 0}
    resumed = False
    if is_experiment:
        if flat is not None:
            loaded = ckpt.try_resume_flat(exp_dir, flat, optimizer, lr_scheduler, device, plan.rs_hooks)
        else:
            loaded = ckpt.try_resume(exp_dir, model, optimizer, lr_scheduler, device, plan.rs_hooks)
        if loaded is not None:
            state, resumed = loaded, True
        LOGGER.info(f"Resumed={resumed} | {state}")
    dist.barrier()
    if is_experiment and ((exp_dir.is_mount() and rank == 0) or (not exp_dir.is_mount() and local_rank == 0)):
        exp_dir.mkdir(parents=True, exist_ok=True)
    dist.barrier()
    if is_experiment:
        (exp_dir / f"rank-{rank}").mkdir(parents=True, exist_ok=True)

    timers = {k: PhaseTimer(device) for k in ["data", "forward", "backward", "update"]}
    injector = FaultInjector.from_env()
    heartbeat = Heartbeat.from_default_store(rank, world_size, args.heartbeat_timeout) if args.heartbeat_timeout > 0 else None

    activities = [ProfilerActivity.CPU] + ([ProfilerActivity.CUDA] if device.type == "cuda" else [])
    prof_ctx = torch.profiler.profile(
        activities=activities,
        schedule=torch.profiler.schedule(wait=args.profiler_wait, warmup=args.profiler_warmup,
                                         active=args.profiler_active, repeat=1),
        on_trace_ready=torch.profiler.tensorboard_trace_handler(str(exp_dir / "log" / f"rank-{rank}")),
        record_shapes=False, with_stack=False, profile_memory=False, with_modules=False,
    ) if args.profiler else contextlib.nullcontext()

    def save_checkpoint():
        if device.type == "cuda":
            check_device_status(deep=True)  # never persist a step whose collectives gave up or strayed
        if flat is not None:
            ckpt.save_flat_checkpoint(exp_dir, flat, optimizer, lr_scheduler, state, plan.rs_hooks)
        else:
            ckpt.save_checkpoint(exp_dir, model, optimizer, lr_scheduler, state, plan.rs_hooks)

    done = False
    with prof_ctx as prof:
        for state["epoch"] in range(state["epoch"], args.num_epochs):
            LOGGER.info(f"Begin epoch {state['epoch']} at step {state['epoch_step']}")
            dataloader.sampler.set_epoch(state["epoch"])
            batches = iter(dataloader)
            progress = None
            if rank == 0:
                from tqdm import tqdm

                progress = tqdm(total=len(dataloader), initial=0, disable=None)
            for i_step in range(len(dataloader)):
                injector.maybe_fail(rank, state["global_step"])  # host-side, nothing in flight
                if heartbeat is not None:
                    heartbeat.beat_and_check(state["global_step"])
                # start gathering the first groups' parameters
                if flat is not None:
                    flat.begin_step()
                else:
                    model.unshard()
                with timers["data"], torch.no_grad():
                    batch = next(batches)
                    batch = {k: v.to(device=device, non_blocking=True) for k, v in batch.items()}
                if i_step < state["epoch_step"]:
                    if progress is not None:
                        progress.update(1)
                    continue  # fast-forward when resuming
                with timers["forward"], torch.profiler.record_function("STEP::forward"):
                    outputs = model(**batch)
                    del batch
                with timers["backward"], torch.profiler.record_function("STEP::backward"):
                    if flat is not None:
                        flat.backward(outputs.loss)
                    else:
                        with unit_loss_grad():
                            outputs.loss.backward()
                with timers["update"], torch.profiler.record_function("STEP::update"):
                    if flat is not None:
                        flat.optimizer_step(optimizer, lr_scheduler)
                    else:
                        optimizer.step()
                        lr_scheduler.step()
                        optimizer.zero_grad(set_to_none=not args.cpu_offload)
                if prof is not None:
                    prof.step()
                if progress is not None:
                    progress.update(1)

                state["global_step"] += 1
                state["epoch_step"] += 1
                loss_value = outputs.loss.item()  # the one host synchronisation of a step
                if device.type == "cuda":
                    check_device_status()  # an expired device-side wait becomes an exception here
                if not math.isfinite(loss_value):
                    # stop before the next checkpoint can save the state: the last good one is on disk
                    raise FloatingPointError(f"non-finite loss {loss_value} at step {state['global_step']} "
                                             f"on rank {rank}; resume from the last checkpoint")
                state["running_loss"] += loss_value
                if args.loss_log and rank == 0:
                    with open(args.loss_log, "a") as fp:
                        fp.write(f"{state['global_step']} {loss_value:.8f}\n")

                if state["global_step"] % args.log_freq == 0:
                    tok_per_step = world_size * args.batch_size * args.seq_length
                    ms_local = sum(t.avg_elapsed_ms() for t in timers.values())
                    ms_per_step = all_reduce_max(ms_local, device)  # slowest rank sets the pace
                    info = {
                        "global_step": state["global_step"],
                        "lr": lr_scheduler.get_last_lr()[0],
                        "running_loss": state["running_loss"] / args.log_freq,
                        "epoch": state["epoch"],
                        "epoch_progress": state["epoch_step"] / len(dataloader),
                        "num_batches_remaining": len(dataloader) - i_step,
                        **get_mem_stats(device),
                        "tokens_per_s": 1000 * tok_per_step / max(ms_per_step, 1e-9),
                        "time/total": ms_per_step,
                        **{f"time/{k}": t.avg_elapsed_ms() for k, t in timers.items()},
                    }
                    info.update(_comm_metrics(flat, plan, args.log_freq, device))
                    LOGGER.info(info)
                    if device.type == "cuda":
                        check_device_status(deep=True)
                        torch.cuda.reset_peak_memory_stats(device)
                    state["running_loss"] = 0
                    for t in timers.values():
                        t.reset()

                if is_experiment and state["global_step"] % args.ckpt_freq == 0:
                    save_checkpoint()

                if args.steps is not None and state["global_step"] >= args.steps:
                    done = True
                    break
            if progress is not None:
                progress.close()
            if done:
                break
            state["epoch_step"] = 0
    dist.barrier()
    dist.destroy_process_group()
    return state


if __name__ == "__main__":
    main()
