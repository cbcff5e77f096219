"""Throughput benchmark: FSDP training tokens/s of a Llama-3-8B-shape model (bf16, seq 4096,
micro-batch 1 per GPU, AdamW, synthetic uniform tokens, random N(0, 0.02) weights).

    python bench.py --gpus 1 --steps 5 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...      # the unmodified reference hooks from baseline/_ref

Two measurements per run, both the maximum over ranks:
  value      device-timed: K optimizer steps between CUDA events, inputs already on the device
  e2e.value  end to end through ``TrainEngine.step``: every step copies its token batch from pinned
             host memory and reads the loss back to the host
Rank 0 prints one JSON line.  SM clocks and throttle reasons are sampled with nvidia-smi while the
timed regions run.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))

MODEL_SHAPES = {
    # name: (vocab, d_model, layers, heads, kv_heads, ffn, rope_theta)
    "llama3-8b": (128256, 4096, 32, 32, 8, 14336, 500000.0),
    "llama2-13b": (32000, 5120, 40, 40, 40, 13824, 10000.0),
    "34b": (32000, 8192, 48, 64, 8, 22016, 1000000.0),
    "small": (32768, 1024, 4, 8, 2, 4096, 500000.0),
    # GPT-2 family (rope_theta None): the reference's shipped run is GPT-2-XL, batch 2 per GPU, seq 1024
    "gpt2-xl": (50257, 1600, 48, 25, 25, 6400, None),
}


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU every 200 ms while running."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), line.strip()))

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self, t0: float, t1: float) -> dict:
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for t, line in self.rows:
            if t < t0 or t > t1:
                continue
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0])), mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="llama3-8b", choices=sorted(MODEL_SHAPES))
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--micro-batch", type=int, default=1)
    ap.add_argument("--ref-variant", default="zip", choices=["zip", "int8", "nccl"],
                    help="reference arm: its shipped run uses -q --zip-ccl (zip)")
    ap.add_argument("--transport", default="auto", choices=["auto", "symm", "lib"])
    ap.add_argument("--no-compress", action="store_true", help="ours: stock NCCL collectives")
    ap.add_argument("--wire", default="auto", choices=["auto", "nibble", "compressed", "verbatim"],
                    help="ours: what the fused collectives move: lossless exponent-coded records in nibble mode "
                         "(default) or with bit planes (compressed: the smallest wire), or the raw bf16 bytes "
                         "(verbatim: a comparison arm without codec work)")
    ap.add_argument("--act-ckpt", action="store_true")
    ap.add_argument("--gemm", default=None, choices=[None, "auto", "tcgen05", "tcgen05_2sm", "cublas"])
    ap.add_argument("--reshard-after-forward", default="auto", choices=["auto", "true", "false"],
                    help="ours (flat): release gathered parameters after forward (ZeRO-3) or keep them until backward")
    ap.add_argument("--comm-stats", action="store_true",
                    help="ours: bracket every collective with CUDA events and report per-step device time, bus "
                         "GB/s and the time compute stood still waiting for communication (a few events per "
                         "collective; off for the headline runs)")
    ap.add_argument("--strict-comm", action="store_true",
                    help="fail instead of warning when compressed collectives did not run on the fused transport")
    ap.add_argument("--sharding", default="flat", choices=["flat", "fsdp2"], help="ours: sharding back end")
    ap.add_argument("--kernel-table", type=int, default=0, metavar="N",
                    help="after the timed runs, trace two more steps with torch.profiler and print the N "
                         "kernels with the most device time on rank 0 (shares only: traced steps are not timed)")
    return ap.parse_args()


def make_ours(args, device):
    sys.path.insert(0, ROOT)
    from fsdp_comm_opt_b200 import _lib
    from fsdp_comm_opt_b200.engine import EngineConfig, TrainEngine
    from fsdp_comm_opt_b200.ops import gemm

    if args.gemm:
        gemm.set_backend(args.gemm)
    comp = not args.no_compress
    eng = TrainEngine(EngineConfig(model=args.model, quantize=comp, zip_ccl=comp, compress_rs=comp,
                                   transport=args.transport, wire=args.wire, act_ckpt=args.act_ckpt,
                                   sharding=args.sharding, time_collectives=args.comm_stats,
                                   reshard_after_forward={"auto": "auto", "true": True, "false": False}[
                                       args.reshard_after_forward]), device)
    info = {"gemm_backend": gemm.get_backend(), "native_lib": str(_lib.cuda_lib_path()), "sharding": args.sharding,
            "reshard_after_forward": eng.flat.reshard_after_forward if eng.flat is not None else True,
            "comm_requested": ("nccl" if not comp else "zip all-gather + compressed reduce-scatter (nibble-mode records)"
                               if args.wire in ("auto", "nibble") else
                               "zip all-gather + compressed reduce-scatter (bit-plane records)" if args.wire == "compressed"
                               else "fused all-gather + reduce-scatter, verbatim bf16 wire")}
    make_ours.engine = eng
    return eng.step_on_device, eng.step, info, _lib


def make_reference(args, device, world):
    """Stock FSDP2 + the reference's unmodified hook classes and extension from baseline/_ref, an HF
    Llama model built from a local config, torch fused AdamW: the reference's train.py flow
    (which cannot run offline because it needs the HF hub) with synthetic tokens."""
    ref_root = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_root, "main")):
        raise RuntimeError("baseline/_ref is missing (reference not installed)")
    sys.path.insert(0, ref_root)
    import torch
    from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard
    from transformers import AutoModelForCausalLM, LlamaConfig
    from transformers.models.llama.modeling_llama import LlamaRMSNorm

    v, d, L, H, Hkv, ffn, theta = MODEL_SHAPES[args.model]
    is_gpt2 = theta is None
    if is_gpt2:
        from transformers import GPT2Config

        cfg = GPT2Config(vocab_size=v, n_embd=d, n_layer=L, n_head=H, n_inner=ffn, n_positions=max(args.seq, 1024),
                         use_cache=False, resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0)
    else:
        cfg = LlamaConfig(vocab_size=v, hidden_size=d, intermediate_size=ffn, num_hidden_layers=L,
                          num_attention_heads=H, num_key_value_heads=Hkv,
                          max_position_embeddings=max(args.seq, 4096), rope_theta=theta, use_cache=False,
                          tie_word_embeddings=False)
    with torch.device("meta"):
        model = AutoModelForCausalLM.from_config(cfg, dtype=torch.bfloat16)
    fsdp_config = dict(reshard_after_forward=True,
                       mp_policy=MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32))
    hook_cls = None
    if args.ref_variant != "nccl":
        import main.comm as ref_comm
        import main.zipccl_comm as ref_zip

        assert ref_zip.__file__.startswith(ref_root) and ref_comm.__file__.startswith(ref_root)
        hook_cls = ref_zip.ZipCCLAllGather if args.ref_variant == "zip" else ref_comm.QuantizedAllGather
    layers = list(model.transformer.h if is_gpt2 else model.model.layers)
    fl = []
    for dec in layers:
        m = fully_shard(dec, **fsdp_config)
        fl.append(m)
        if hook_cls is not None:
            m.set_custom_all_gather(hook_cls())
    for i, m in enumerate(fl):
        if fl[i + 1:i + 2]:
            m.set_modules_to_forward_prefetch(fl[i + 1:i + 2])
    root = fully_shard(model, **fsdp_config)
    if hook_cls is not None:
        root.set_custom_all_gather(hook_cls())
    model.to_empty(device=device)
    torch.manual_seed(0)
    with torch.no_grad():
        for mod in model.modules():
            if isinstance(mod, (torch.nn.Linear, torch.nn.Embedding)):
                torch.nn.init.normal_(mod.weight, mean=0.0, std=0.02)
            elif isinstance(mod, (LlamaRMSNorm, torch.nn.LayerNorm)):
                torch.nn.init.ones_(mod.weight)
            elif type(mod).__name__ == "Conv1D":  # GPT-2 projections
                torch.nn.init.normal_(mod.weight, mean=0.0, std=0.02)
            if getattr(mod, "bias", None) is not None and isinstance(mod.bias, torch.Tensor) and mod.bias.dim() == 1:
                torch.nn.init.zeros_(mod.bias)
        if not is_gpt2:
            hd = d // H
            inv = 1.0 / (theta ** (torch.arange(0, hd, 2, dtype=torch.float32, device=device) / hd))
            model.model.rotary_emb.inv_freq = inv
            model.model.rotary_emb.original_inv_freq = inv.clone()
    opt = torch.optim.AdamW(model.parameters(), lr=3e-5, fused=True)
    sched = torch.optim.lr_scheduler.CosineAnnealingLR(opt, T_max=1000, eta_min=3e-7)

    def step_on_device(ids):
        model.unshard()
        out = model(input_ids=ids, labels=ids)
        out.loss.backward()
        opt.step()
        sched.step()
        opt.zero_grad(set_to_none=True)
        return out.loss.detach()

    def step(host_ids):
        return float(step_on_device(host_ids.to(device, non_blocking=True)).item())

    return step_on_device, step, {"ref_variant": args.ref_variant}, None


def kernel_table(step_fn, batch, top: int, device) -> list:
    """Device time per kernel name over two traced steps (every rank traces, so collectives match up)."""
    import torch
    from torch.profiler import ProfilerActivity, profile

    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        step_fn(batch)
        step_fn(batch)
        torch.cuda.synchronize(device)
    rows = sorted(prof.key_averages(), key=lambda e: -e.device_time_total)
    total = sum(e.device_time_total for e in rows) or 1.0
    return [{"kernel": e.key[:90], "launches_per_step": e.count / 2, "ms_per_step": round(e.device_time_total / 2e3, 3),
             "share": round(e.device_time_total / total, 4)} for e in rows[:top]]


def main():
    args = parse_args()
    try:
        import torch
        import torch.distributed as dist
    except Exception as e:  # pragma: no cover
        print(json.dumps({"impl": args.impl, "unavailable": f"torch import failed: {e}"}))
        return 0
    if not torch.cuda.is_available():
        print(json.dumps({"impl": args.impl, "unavailable": "no CUDA device"}))
        return 0
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            print(json.dumps({"impl": args.impl, "unavailable":
                              f"--gpus {args.gpus} needs torch.distributed.run with --nproc-per-node {args.gpus}"}))
            return 0
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29541")
    device = torch.device(f"cuda:{local_rank}")
    torch.cuda.set_device(device)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)

    try:
        if args.impl == "ours":
            step_dev, step_host, info, lib = make_ours(args, device)
        else:
            step_dev, step_host, info, lib = make_reference(args, device, world)
    except Exception as e:
        if args.impl == "reference":
            if rank == 0:
                print(json.dumps({"impl": "reference", "unavailable": f"{type(e).__name__}: {e}"[:300]}))
            dist.destroy_process_group()
            return 0
        raise

    vocab = MODEL_SHAPES[args.model][0]
    B, S = args.micro_batch, args.seq
    g = torch.Generator().manual_seed(1234 + rank)
    n_batches = args.warmup + args.steps
    host_batches = [torch.randint(0, vocab, (B, S), generator=g, dtype=torch.int64).pin_memory()
                    for _ in range(n_batches)]
    dev_batches = [b.to(device) for b in host_batches]

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()

    def run(kind):
        fn, batches = (step_dev, dev_batches) if kind == "device" else (step_host, host_batches)
        for i in range(args.warmup):
            fn(batches[i])
        torch.cuda.synchronize(device)
        dist.barrier()
        torch.cuda.synchronize(device)
        if lib is not None:
            lib.reset_launch_count()
        t_wall0 = time.time()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        last = None
        for i in range(args.steps):
            last = fn(batches[args.warmup + i])
        e1.record()
        torch.cuda.synchronize(device)
        dist.barrier()
        torch.cuda.synchronize(device)
        t_wall1 = time.time()
        ms = e0.elapsed_time(e1) if kind == "device" else 1000.0 * (t_wall1 - t_wall0)
        t = torch.tensor([ms], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        launches = lib.launch_count() if lib is not None else None
        return float(t.item()), float(last) if last is not None else None, launches, (t_wall0, t_wall1)

    try:
        dev_ms, dev_loss, launches, (d0, d1) = run("device")
        e2e_ms, e2e_loss, _, (x0, x1) = run("e2e")
        if args.impl == "ours":
            # A step that produced a non-finite loss did not train (and runs fast: NaN operands draw
            # little power): such a number must not be reported.  Build the engine again and measure
            # once more; a second failure ends the run with an error.
            import gc
            import math

            def any_rank_bad(*vals):
                bad = torch.tensor([float(any(v is None or not math.isfinite(v) for v in vals))], device=device)
                dist.all_reduce(bad, op=dist.ReduceOp.MAX)
                return bool(bad.item())

            if any_rank_bad(dev_loss, e2e_loss):
                if rank == 0:
                    print("[bench] non-finite loss in the timed steps: rebuilding the engine and measuring again",
                          file=sys.stderr, flush=True)
                make_ours.engine = None
                step_dev = step_host = None
                gc.collect()
                torch.cuda.empty_cache()
                step_dev, step_host, info, lib = make_ours(args, device)
                dev_ms, dev_loss, launches, (d0, d1) = run("device")
                e2e_ms, e2e_loss, _, (x0, x1) = run("e2e")
                info["remeasured"] = "first attempt gave a non-finite loss"
                if any_rank_bad(dev_loss, e2e_loss):
                    raise RuntimeError(f"non-finite loss twice (device run {dev_loss}, end-to-end run {e2e_loss})")
    except torch.OutOfMemoryError as e:
        if args.impl != "reference":
            raise
        # the reference has no activation checkpointing: some shapes do not fit its arm
        if rank == 0:
            sampler.stop()
            print(json.dumps({"impl": "reference", "unavailable":
                              f"out of device memory on {args.model} at {world} GPUs (the reference has no activation "
                              f"checkpointing): {str(e)[:120]}"}))
        os._exit(0)  # the other ranks are inside collectives; do not wait for them
    comm = None
    if args.impl == "ours":
        # a bounded device-side wait that expired would have left wrong data behind: fail loudly
        from fsdp_comm_opt_b200.utils.health import check_device_status

        check_device_status()
        # what the collectives actually ran on (not what the flags asked for)
        comm = make_ours.engine.comm_report()
        if args.comm_stats and make_ours.engine.flat is not None:
            n_steps = 2 * (args.warmup + args.steps)
            comm["per_step"] = {k: {"calls": v["calls"] / n_steps, "ms": round(v["ms"] / n_steps, 3),
                                    "bus_gbs": None if v["bus_gbs"] is None else round(v["bus_gbs"], 1)}
                                for k, v in make_ours.engine.flat.comm_stats().items()}
        if world > 1 and not args.no_compress and args.transport != "lib":
            ran = set(comm["all_gather"]) | set(comm["reduce_scatter"])
            if ran != {"symm"}:
                from fsdp_comm_opt_b200.parallel import symm_impl as _symm

                why = _symm.why_unavailable(dist.group.WORLD)
                comm["fused_transport_unavailable"] = why
                msg = (f"compressed collectives were requested but ran on {sorted(ran)}: the fused "
                       f"symmetric-memory transport was not available ({why})")
                if args.strict_comm:
                    raise RuntimeError(msg)
                if rank == 0:
                    print("WARNING: " + msg, file=sys.stderr)
    table = None
    if args.kernel_table > 0:  # every rank runs the traced steps (they contain collectives)
        table = kernel_table(step_dev, dev_batches[-1], args.kernel_table, device)
    if rank == 0:
        time.sleep(0.3)
        sampler.stop()
    tokens = world * B * S * args.steps
    value = tokens / (dev_ms / 1000.0)
    e2e_value = tokens / (e2e_ms / 1000.0)
    if rank == 0:
        clocks = sampler.summary(d0, x1)
        out = {
            "metric": "FSDP training tokens/sec (max over ranks, device-timed)",
            "impl": args.impl,
            "value": value,
            "unit": "tokens/s",
            "n_gpus": world,
            "steps": args.steps,
            "warmup": args.warmup,
            "ms_per_step": dev_ms / args.steps,
            "higher_is_better": True,
            "scaling": "weak",
            "vs_baseline": None,
            "dtype": "bf16",
            "data": "synthetic uniform random tokens, random N(0,0.02) init (no datasets or checkpoints offline)",
            "config": {"model": args.model, "global_batch": world * B, "seq_len": S,
                       "parallelism": f"fsdp{world}" if world > 1 else "fsdp1 (single GPU, full shard of one)",
                       "optimizer": "AdamW", "act_ckpt": args.act_ckpt,
                       "l2": "inputs larger than L2: every step streams >16 GB of weights and activations",
                       **info},
            "e2e": {"value": e2e_value, "unit": "tokens/s", "ms_per_step": e2e_ms / args.steps,
                    "h2d_bytes_per_step": B * S * 8, "d2h_bytes_per_step": 4,
                    "api": "TrainEngine.step(pinned host token ids) -> float loss" if args.impl == "ours"
                    else "reference hooks + FSDP2 + HF model step, batch.to(device) then loss.item()"},
            "gpu_launches": launches,
            "comm": comm,
            "clocks": clocks,
            "loss": {"device_run_last": dev_loss, "e2e_run_last": e2e_loss},
        }
        print(json.dumps(out))
        if table is not None:
            print(json.dumps({"kernel_table": table}))
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
