"""Compressed-collective sweep against NCCL.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        -m fsdp_comm_opt_b200.parallel.bench_collectives [--min-log2 20 --max-log2 30 --iters 4]
        [--budget exclusive|in-step] [--wire nibble|compressed|verbatim]

For total tensor sizes 2^20 .. 2^30 elements (powers of 4) it times
  * all-gather of bf16 shards   (parameter-like N(0, 0.02) data): fused symm kernel vs NCCL
  * reduce-scatter of fp32 rows (gradient-like N(0, 1e-3) data with 1% of entries x100, rounded to
    bf16-representable values as FSDP produces them): fused symm kernel vs NCCL fp32
and reports, per line of JSON: bus GB/s of both (nccl-tests convention: bytes * (W-1)/W / time, with
the UNCOMPRESSED payload as bytes, so a compressed collective can exceed the link rate), the
measured wire bytes per element and the compression ratio they mean, the max abs error against NCCL, and the achieved fraction of the
NVLink roofline (compressed bytes that must leave a GPU / 770 GB/s measured peer bandwidth).
Timing: CUDA events on the launching stream, 2 warm-up calls, max over ranks; inputs alternate
between two buffers so consecutive calls do not hit the same L2 lines for sizes under the L2.
``--budget exclusive`` (default): the collective is alone on the GPU, as in this sweep, and gets the
CTA budget of the whole machine (``hook.exclusive = True``); ``--budget in-step``: the budget it has
inside a training step, which leaves room for the GEMMs and for a second collective in flight.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from ..utils.dist import init_distributed
from .hooks import ZipCCLAllGather, ZipCCLReduceScatter

PEER_GBS = 770.0


def _timed(fn, iters, device):
    for _ in range(2):
        fn(0)
    torch.cuda.synchronize(device)
    dist.barrier()
    torch.cuda.synchronize(device)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(iters):
        fn(i)
    e1.record()
    torch.cuda.synchronize(device)
    t = torch.tensor([e0.elapsed_time(e1) / iters], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--min-log2", type=int, default=20)
    ap.add_argument("--max-log2", type=int, default=30)
    ap.add_argument("--iters", type=int, default=4)
    ap.add_argument("--transport", default="symm", choices=["symm", "lib"])
    ap.add_argument("--budget", default="exclusive", choices=["exclusive", "in-step"])
    ap.add_argument("--wire", default="nibble", choices=["nibble", "compressed", "verbatim"])
    args = ap.parse_args()
    rank, world, device = init_distributed("cuda")
    from . import symm_impl

    group = dist.group.WORLD
    ag = ZipCCLAllGather(transport=args.transport, wire=args.wire)
    rs = ZipCCLReduceScatter(transport=args.transport, wire=args.wire)
    ag.exclusive = rs.exclusive = args.budget == "exclusive"
    for lg in range(args.min_log2, args.max_log2 + 1, 2):
        total = 1 << lg
        shard = total // world
        g = torch.Generator(device=device).manual_seed(1000 * lg + rank)
        # ---------------- all-gather ------------------------------------------------------------
        xs = [(torch.randn(shard, generator=g, device=device) * 0.02).to(torch.bfloat16) for _ in range(2)]
        out = torch.empty(world * shard, dtype=torch.bfloat16, device=device)
        ref = torch.empty_like(out)
        dist.all_gather_into_tensor(ref, xs[0])
        ag(out, xs[0], group)
        torch.cuda.synchronize(device)
        err = float((out.float() - ref.float()).abs().max().item())
        ch = symm_impl.channel_for(group, device, "ag") if args.transport == "symm" else None
        w0 = ch.wire_bytes() if ch else 0
        ms_z = _timed(lambda i: ag(out, xs[i & 1], group), args.iters, device)
        w1 = ch.wire_bytes() if ch else 0
        ms_n = _timed(lambda i: dist.all_gather_into_tensor(ref, xs[i & 1]), args.iters, device)
        payload = 2.0 * shard * world
        wire_pe = (w1 - w0) / ((args.iters + 2) * shard * (world - 1)) if ch else None
        roof_ms = (wire_pe * shard * (world - 1) / (PEER_GBS * 1e6)) if wire_pe else None
        if rank == 0:
            print(json.dumps({"op": "all_gather", "elements": total, "world": world, "budget": args.budget, "wire": args.wire, "data": "params N(0,0.02)",
                              "zip_ms": round(ms_z, 4), "nccl_ms": round(ms_n, 4),
                              "zip_bus_gbs": round(payload * (world - 1) / world / ms_z / 1e6, 1),
                              "nccl_bus_gbs": round(payload * (world - 1) / world / ms_n / 1e6, 1),
                              "wire_bytes_per_elem": None if wire_pe is None else round(wire_pe, 4),
                              "compression_ratio_vs_bf16": None if not wire_pe else round(2.0 / wire_pe, 3),
                              "frac_of_nvlink_roofline": None if roof_ms is None else round(roof_ms / ms_z, 3),
                              "max_abs_err": err}), flush=True)
        del xs, out, ref
        # ---------------- reduce-scatter ----------------------------------------------------------
        rows = []
        for _ in range(2):
            x = torch.randn(world * shard, generator=g, device=device) * 1e-3
            mask = torch.rand(world * shard, generator=g, device=device) < 0.01
            x = torch.where(mask, x * 100, x).to(torch.bfloat16).float()
            rows.append(x)
        out = torch.empty(shard, dtype=torch.float32, device=device)
        ref = torch.empty_like(out)
        dist.reduce_scatter_tensor(ref, rows[0].clone(), op=dist.ReduceOp.AVG)
        rs(out, rows[0], group, dist.ReduceOp.AVG)
        torch.cuda.synchronize(device)
        err = float((out - ref).abs().max().item())
        ref0 = ref.clone()   # fp32 sum of rows[0]: the timing loops below overwrite `ref`
        ch = symm_impl.channel_for(group, device, "rs") if args.transport == "symm" else None
        w0 = ch.wire_bytes() if ch else 0
        ms_z = _timed(lambda i: rs(out, rows[i & 1], group, dist.ReduceOp.AVG), args.iters, device)
        w1 = ch.wire_bytes() if ch else 0
        scratch = [r.clone() for r in rows]
        ms_n = _timed(lambda i: dist.reduce_scatter_tensor(ref, scratch[i & 1], op=dist.ReduceOp.AVG), args.iters, device)
        payload = 4.0 * shard * world
        wire_pe = (w1 - w0) / ((args.iters + 2) * shard * (world - 1)) if ch else None
        roof_ms = (wire_pe * shard * (world - 1) / (PEER_GBS * 1e6)) if wire_pe else None
        if rank == 0:
            print(json.dumps({"op": "reduce_scatter", "elements": total, "world": world, "budget": args.budget, "wire": args.wire,
                              "data": "grads N(0,1e-3) + 1% x100 outliers, fp32 input",
                              "zip_ms": round(ms_z, 4), "nccl_ms": round(ms_n, 4),
                              "zip_bus_gbs": round(payload * (world - 1) / world / ms_z / 1e6, 1),
                              "nccl_bus_gbs": round(payload * (world - 1) / world / ms_n / 1e6, 1),
                              "wire_bytes_per_elem": None if wire_pe is None else round(wire_pe, 4),
                              "compression_ratio_vs_fp32": None if not wire_pe else round(4.0 / wire_pe, 3),
                              "frac_of_nvlink_roofline": None if roof_ms is None else round(roof_ms / ms_z, 3),
                              "max_abs_err": err}), flush=True)
        # ---------------- reduce-scatter of bf16 rows (what the flat-shard engine hands over) --------
        rows16 = [r.to(torch.bfloat16) for r in rows]
        del rows, scratch
        out16 = torch.empty(shard, dtype=torch.bfloat16, device=device)
        ref16 = torch.empty_like(out16)
        rs(out16, rows16[0], group, dist.ReduceOp.AVG)
        torch.cuda.synchronize(device)
        err = float((out16.float() - ref0).abs().max().item())   # against the fp32 NCCL result of the same rows
        ms_z = _timed(lambda i: rs(out16, rows16[i & 1], group, dist.ReduceOp.AVG), args.iters, device)
        scratch = [r.clone() for r in rows16]
        ms_n = _timed(lambda i: dist.reduce_scatter_tensor(ref16, scratch[i & 1], op=dist.ReduceOp.AVG), args.iters, device)
        payload = 2.0 * shard * world
        if rank == 0:
            print(json.dumps({"op": "reduce_scatter_bf16", "elements": total, "world": world, "budget": args.budget,
                              "data": "same gradients as bf16 rows; NCCL column = bf16 reduce-scatter (bf16 accumulation)",
                              "zip_ms": round(ms_z, 4), "nccl_ms": round(ms_n, 4),
                              "zip_bus_gbs": round(payload * (world - 1) / world / ms_z / 1e6, 1),
                              "nccl_bus_gbs": round(payload * (world - 1) / world / ms_n / 1e6, 1),
                              "max_abs_err_vs_fp32_sum": err}), flush=True)
        del rows16, scratch, out, ref, ref0, out16, ref16
        torch.cuda.empty_cache()
    for ch in symm_impl.all_channels():
        ch.check_status()
        ch.check_canaries()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
