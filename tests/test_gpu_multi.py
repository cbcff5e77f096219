"""Multi-GPU tests (2 ranks, NCCL, NVLS off): fused symmetric-memory collectives against the
uncompressed NCCL collectives, the NCCL-transport hooks, bounded-wait failure reporting, and a
short FSDP run.  Skipped with fewer than 2 GPUs."""
import os

import pytest
import torch

from mp_util import run_ranks

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]

# number of ranks for the collective tests (2 by default; ZC_TEST_WORLD=8 on a full box)
WORLD = int(os.environ.get("ZC_TEST_WORLD", "2"))


def _bits(t):
    return t.view(torch.int16)


def _ag_case(rank, world, transport):
    import torch.distributed as dist
    from fsdp_comm_opt_b200.parallel.hooks import ZipCCLAllGather

    dev = torch.device("cuda", rank)
    if transport == "symm-unicast":          # per-peer stores
        os.environ["ZC_SYMM_MULTICAST"] = "0"
        transport = "symm"
    elif transport == "symm":                # NVSwitch multicast stores where the fabric has them
        os.environ["ZC_SYMM_MULTICAST"] = "1"
    hook = ZipCCLAllGather(transport=transport)
    sizes = [1 << 20, 777, 65536 * 3 + 5, 1 << 22, 4096, 1 << 20, (1 << 20) + 8]
    if transport == "symm":
        from fsdp_comm_opt_b200.parallel import symm_impl

        # size the channel once: growing it later would start a new buffer and a new byte counter
        assert symm_impl.available(dist.group.WORLD)
        symm_impl.channel_for(dist.group.WORLD, dev, "ag").reserve(max(sizes))
    for it, n in enumerate(sizes):
        g = torch.Generator().manual_seed(100 * it + rank)
        x = (torch.randn(n, generator=g) * 0.02).to(torch.bfloat16).to(dev)
        ref = torch.zeros(world * n, dtype=torch.bfloat16, device=dev)
        dist.all_gather_into_tensor(ref, x)
        out = torch.zeros(world * n, dtype=torch.bfloat16, device=dev)
        if it % 2 == 0:                      # FSDP2 style: input is a view of the output
            inp = out.narrow(0, n * rank, n)
            inp.copy_(x)
        else:
            inp = x
        w = hook(out, inp, dist.group.WORLD, async_op=(it % 3 == 0))
        if w is not None:
            w.wait()
        torch.cuda.synchronize()
        assert torch.equal(_bits(out), _bits(ref)), (transport, it, n)
    if transport == "symm":
        from fsdp_comm_opt_b200.parallel import symm_impl

        for ch in symm_impl.all_channels():
            ch.check_status()
            ch.check_canaries()
            pushed = ch.wire_bytes()
            raw = 2 * sum(sizes) * (world - 1)
            assert 0.6 * raw < pushed < 0.8 * raw, (pushed, raw)   # ~1.4 of 2 bytes per element


@pytest.mark.parametrize("transport", ["symm", "symm-unicast", "lib"])
def test_zip_all_gather_nccl_ranks(transport):
    run_ranks(_ag_case, WORLD, (transport,), backend="nccl")


def _int8_case(rank, world):
    """The fused int8 all-gather gives every rank (the source included) the values the NCCL-transport
    hook gives, and both stay within the quantisation error of the inputs: half a step from the
    rounding to int8 plus up to half a step from writing the result as bf16 (a value of up to 127
    steps rounded to 8 significant bits)."""
    import torch.distributed as dist
    from fsdp_comm_opt_b200.parallel.hooks import QuantizedAllGather
    from fsdp_comm_opt_b200.parallel import symm_impl

    dev = torch.device("cuda", rank)
    fused, lib = QuantizedAllGather(transport="symm"), QuantizedAllGather(transport="lib")
    for it, n in enumerate([1 << 20, 1000, 65536 * 3 + 7, 1 << 22, 1 << 20]):
        g = torch.Generator().manual_seed(31 * it + rank)
        x = (torch.randn(n, generator=g) * (0.02 * (rank + 1))).to(torch.bfloat16).to(dev)
        full = torch.zeros(world * n, dtype=torch.bfloat16, device=dev)
        dist.all_gather_into_tensor(full, x)
        a = torch.zeros(world * n, dtype=torch.bfloat16, device=dev)
        b = torch.zeros(world * n, dtype=torch.bfloat16, device=dev)
        if it % 2 == 0:                      # FSDP2 style: input is a view of the output
            inp = a.narrow(0, n * rank, n)
            inp.copy_(x)
        else:
            inp = x
        w = fused(a, inp, dist.group.WORLD, async_op=(it % 2 == 1))
        if w is not None:
            w.wait()
        lib(b, x, dist.group.WORLD)
        torch.cuda.synchronize()
        for r in range(world):
            seg = slice(r * n, (r + 1) * n)
            step = full[seg].float().abs().max().item() / 127.0
            assert (a[seg].float() - full[seg].float()).abs().max().item() <= 1.0 * step + 1e-8, (it, r)
            # same arithmetic on both transports; allow one quantisation step where x/scale rounds apart
            assert (a[seg].float() - b[seg].float()).abs().max().item() <= 1.01 * step, (it, r)
        assert (a != b).float().mean().item() < 1e-3
    for ch in symm_impl.all_channels():
        ch.check_status()


def test_int8_all_gather_fused_matches_library_transport():
    run_ranks(_int8_case, WORLD, backend="nccl")


def _rs_case(rank, world, transport):
    import torch.distributed as dist
    from fsdp_comm_opt_b200.parallel.hooks import ZipCCLReduceScatter

    dev = torch.device("cuda", rank)
    hook = ZipCCLReduceScatter(transport=transport)
    for it, shard in enumerate([1 << 20, 5000, 65536 * 2 + 3, 1 << 21, 1 << 20]):
        g = torch.Generator().manual_seed(7 * it + rank)
        x = (torch.randn(world * shard, generator=g) * 1e-3).to(torch.bfloat16).float().to(dev)
        ref = torch.zeros(shard, device=dev)
        dist.reduce_scatter_tensor(ref, x.clone(), op=dist.ReduceOp.AVG)
        out = torch.zeros(shard, device=dev)
        hook(out, x, dist.group.WORLD, dist.ReduceOp.AVG)
        torch.cuda.synchronize()
        assert torch.allclose(out, ref, rtol=1e-6, atol=1e-9), (transport, it, (out - ref).abs().max().item())
        # bf16 input and output
        xb = x.to(torch.bfloat16)
        outb = torch.zeros(shard, dtype=torch.bfloat16, device=dev)
        hook(outb, xb, dist.group.WORLD, dist.ReduceOp.SUM)
        refb = torch.zeros(shard, device=dev)
        dist.reduce_scatter_tensor(refb, x.clone(), op=dist.ReduceOp.SUM)
        torch.cuda.synchronize()
        assert torch.allclose(outb.float(), refb, rtol=1e-2, atol=1e-6)
    # true fp32 gradients: error feedback keeps the running sum closer than plain rounding
    shard = 1 << 18
    ef, no = ZipCCLReduceScatter(transport=transport), ZipCCLReduceScatter(error_feedback=False, transport=transport)
    const = (torch.randn(world * shard, generator=torch.Generator().manual_seed(rank)) * 1e-3).to(dev)
    acc_ref, acc_ef, acc_no = (torch.zeros(shard, device=dev) for _ in range(3))
    for _ in range(24):
        r, a, b = (torch.zeros(shard, device=dev) for _ in range(3))
        dist.reduce_scatter_tensor(r, const.clone(), op=dist.ReduceOp.SUM)
        ef(a, const.clone(), dist.group.WORLD, dist.ReduceOp.SUM)
        no(b, const.clone(), dist.group.WORLD, dist.ReduceOp.SUM)
        acc_ref += r; acc_ef += a; acc_no += b
    torch.cuda.synchronize()
    e1, e2 = (acc_ef - acc_ref).abs().max().item(), (acc_no - acc_ref).abs().max().item()
    assert e1 < e2 / 3, (e1, e2)
    if transport == "symm":
        from fsdp_comm_opt_b200.parallel import symm_impl

        for ch in symm_impl.all_channels():
            ch.check_status()
            ch.check_canaries()


@pytest.mark.parametrize("transport", ["symm", "lib"])
def test_compressed_reduce_scatter_nccl_ranks(transport):
    run_ranks(_rs_case, WORLD, (transport,), backend="nccl")


def _verbatim_case(rank, world):
    """The verbatim wire (raw bf16 bytes on the fused protocol): the all-gather is bit exact, with
    multicast stores and with per-peer stores, and the reduce-scatter gives the bits of the compressed
    one (same rounding, same order of the fp32 sum); 2 bytes per element cross the links."""
    import torch.distributed as dist
    from fsdp_comm_opt_b200.parallel import symm_impl
    from fsdp_comm_opt_b200.parallel.hooks import ZipCCLAllGather, ZipCCLReduceScatter

    dev = torch.device("cuda", rank)
    grp = dist.group.WORLD
    assert symm_impl.available(grp)
    sizes = [1 << 20, 777, 65536 * 3 + 5, 4096]
    symm_impl.channel_for(grp, dev, "ag").reserve(max(sizes))
    ag = ZipCCLAllGather(transport="symm", wire="verbatim")
    for it, n in enumerate(sizes):
        g = torch.Generator().manual_seed(7 * it + rank)
        x = (torch.randn(n, generator=g) * 0.02).to(torch.bfloat16).to(dev)
        ref = torch.zeros(world * n, dtype=torch.bfloat16, device=dev)
        dist.all_gather_into_tensor(ref, x)
        out = torch.zeros(world * n, dtype=torch.bfloat16, device=dev)
        w = ag(out, x, grp, async_op=(it % 2 == 0))
        if w is not None:
            w.wait()
        torch.cuda.synchronize()
        assert torch.equal(_bits(out), _bits(ref)), (it, n)
    ch = symm_impl.channel_for(grp, dev, "ag")
    nchunks = sum((n + 1023) // 1024 for n in sizes)
    assert ch.wire_bytes() == 2048 * nchunks * (world - 1)
    for dtype in (torch.float32, torch.bfloat16):
        shard = 50_000
        g = torch.Generator().manual_seed(99 + rank)
        x = (torch.randn(world * shard, generator=g) * 1e-3).to(dtype).to(dev)
        outs = []
        for wire in ("compressed", "verbatim", "nibble"):
            hook = ZipCCLReduceScatter(transport="symm", wire=wire)
            o = torch.zeros(shard, dtype=dtype, device=dev)
            hook(o, x.clone(), grp, dist.ReduceOp.AVG)
            torch.cuda.synchronize()
            outs.append(o)
        assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2]), dtype
    for c in symm_impl.all_channels():
        c.check_status()
        c.check_canaries()


def test_verbatim_wire_on_the_fused_transport():
    run_ranks(_verbatim_case, WORLD, (), backend="nccl")


def _back_to_back_case(rank, world, wire):
    """Many collectives of changing sizes queued on one stream with no host synchronisation in between
    (the way a training step issues them), results checked only at the end: exercises the reuse of the
    two parity buffers and of the flags while ranks run ahead of one another."""
    import torch.distributed as dist
    from fsdp_comm_opt_b200.parallel import symm_impl
    from fsdp_comm_opt_b200.parallel.hooks import ZipCCLAllGather, ZipCCLReduceScatter

    dev = torch.device("cuda", rank)
    grp = dist.group.WORLD
    sizes = [1 << 23, 300_000, 1 << 25, 4096, (1 << 22) + 1024, 70_000, 1 << 24, 1 << 20]
    symm_impl.channel_for(grp, dev, "ag").reserve(max(sizes))
    symm_impl.channel_for(grp, dev, "rs").reserve(max(sizes))
    ag = ZipCCLAllGather(transport="symm", wire=wire)
    rs = ZipCCLReduceScatter(transport="symm", wire=wire, error_feedback=False)
    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    side = torch.cuda.Stream(dev)
    xs, outs, refs, rxs, routs, rrefs = [], [], [], [], [], []
    for rep in range(3):
        for n in sizes:
            x = (torch.randn(n, generator=g, device=dev) * 0.02).bfloat16()
            ref = torch.empty(world * n, dtype=torch.bfloat16, device=dev)
            dist.all_gather_into_tensor(ref, x)
            xs.append(x), refs.append(ref), outs.append(torch.zeros(world * n, dtype=torch.bfloat16, device=dev))
            shard = n // world // 8 * 8
            rx = (torch.randn(world * shard, generator=g, device=dev) * 1e-3).bfloat16()
            rref = torch.empty(shard, dtype=torch.float32, device=dev)
            dist.reduce_scatter_tensor(rref, rx.float(), op=dist.ReduceOp.SUM)
            rxs.append(rx), rrefs.append(rref), routs.append(torch.zeros(shard, dtype=torch.float32, device=dev))
    torch.cuda.synchronize()
    dist.barrier()
    side.wait_stream(torch.cuda.current_stream(dev))
    for i in range(len(xs)):                      # all-gathers on this stream, reduce-scatters on another
        ag(outs[i], xs[i], grp, async_op=True)
        with torch.cuda.stream(side):
            rs(routs[i], rxs[i], grp, dist.ReduceOp.SUM, async_op=True)
        if i % 5 == rank:                         # ranks drift apart
            torch.cuda._sleep(3_000_000)
    torch.cuda.synchronize()
    for i in range(len(xs)):
        assert torch.equal(_bits(outs[i]), _bits(refs[i])), ("all_gather", wire, i, xs[i].numel())
        assert torch.allclose(routs[i], rrefs[i], rtol=1e-5, atol=1e-7), ("reduce_scatter", wire, i)
    for c in symm_impl.all_channels():
        c.check_status()
        c.check_canaries()


@pytest.mark.parametrize("wire", ["compressed", "nibble", "verbatim"])
def test_back_to_back_collectives_without_host_sync(wire):
    run_ranks(_back_to_back_case, WORLD, (wire,), backend="nccl")


def _timeout_case(rank, world):
    """Rank 1 never joins one collective; rank 0's bounded wait must expire into a status word,
    surface as SymmTimeout on the host, and leave the context usable."""
    import torch.distributed as dist
    from fsdp_comm_opt_b200.parallel import symm_impl

    dev = torch.device("cuda", rank)
    assert symm_impl.available(dist.group.WORLD)
    os.environ["ZC_SYMM_MULTICAST"] = "0"   # failure paths are exercised on plain peer stores
    ch = symm_impl.channel_for(dist.group.WORLD, dev, "timeout-test")
    ch.timeout_s = 1.0
    n = 1 << 16
    ch.reserve(n)
    x = torch.ones(n, dtype=torch.bfloat16, device=dev)
    out = torch.zeros(world * n, dtype=torch.bfloat16, device=dev)
    if rank == 0:
        ch.all_gather(out, x)
        with pytest.raises(symm_impl.SymmTimeout) as ei:
            ch.check_status()
        assert ei.value.code == 2 and ei.value.peer == 1
        ch.check_status()                       # cleared
        y = torch.arange(10, device=dev).sum()  # the context still works
        assert int(y) == 45
    torch.cuda.synchronize()
    dist.barrier()


def test_bounded_wait_reports_missing_peer():
    run_ranks(_timeout_case, 2, backend="nccl")


def _train(rank, world, extra, loss_log):
    import train

    train.main(["--synthetic", "--model-shape", "small", "--device", "cuda", "-b", "1", "-s", "512", "--lr", "1e-4",
                "--log-freq", "100", "--num-samples", "64", "--steps", "4", "--loss-log", loss_log] + extra)


def _losses(path):
    return [float(l.split()[1]) for l in open(path).read().split("\n") if l]


def test_fsdp_two_gpus_symm_vs_lib_vs_uncompressed(tmp_path):
    logs = {k: str(tmp_path / f"{k}.log") for k in ("none", "lib", "symm")}
    run_ranks(_train, 2, init_pg=False, backend="nccl", args=([], logs["none"]))
    run_ranks(_train, 2, init_pg=False, backend="nccl", args=(["-q", "--zip-ccl", "--transport", "lib"], logs["lib"]))
    run_ranks(_train, 2, init_pg=False, backend="nccl",
              args=(["-q", "--zip-ccl", "--compress-rs", "--transport", "symm"], logs["symm"]))
    a, b, c = (_losses(logs[k]) for k in ("none", "lib", "symm"))
    assert len(a) == len(b) == len(c) == 4
    # the all-gather is lossless (bit-exact gathers are asserted in _ag_case); the curves themselves agree
    # to fp32 summation order only: the attention backward adds its dQ tiles with bulk reductions whose
    # order is not fixed from run to run
    assert a[0] == b[0] and all(abs(x - y) / x < 5e-4 for x, y in zip(a, b)), (a, b)
    assert all(abs(x - y) / x < 0.01 for x, y in zip(a, c)), (a, c)


def test_fsdp2_back_end_two_gpus_compressed_vs_uncompressed(tmp_path):
    """The same hooks through PyTorch FSDP2 (``--sharding fsdp2``), which is how the reference wires them."""
    logs = {k: str(tmp_path / f"{k}.log") for k in ("none", "symm")}
    run_ranks(_train, 2, init_pg=False, backend="nccl", args=(["--sharding", "fsdp2"], logs["none"]))
    run_ranks(_train, 2, init_pg=False, backend="nccl",
              args=(["--sharding", "fsdp2", "-q", "--zip-ccl", "--compress-rs", "--transport", "symm"], logs["symm"]))
    a, c = _losses(logs["none"]), _losses(logs["symm"])
    assert len(a) == len(c) == 4
    assert all(abs(x - y) / x < 0.01 for x, y in zip(a, c)), (a, c)


def _side_stream_case(rank, world):
    """The Work of an async fused all-gather launched on a side stream orders the *default* stream
    after the kernel (c10d semantics: ``wait()`` blocks the current stream, not the host)."""
    import torch.distributed as dist
    from fsdp_comm_opt_b200.parallel.hooks import ZipCCLAllGather

    dev = torch.device("cuda", rank)
    hook = ZipCCLAllGather(transport="symm")
    n = 1 << 22
    side = torch.cuda.Stream(dev)
    for it in range(3):
        g = torch.Generator().manual_seed(5 * it + rank)
        x = (torch.randn(n, generator=g) * 0.02).to(torch.bfloat16).to(dev)
        ref = torch.zeros(world * n, dtype=torch.bfloat16, device=dev)
        dist.all_gather_into_tensor(ref, x)
        out = torch.zeros(world * n, dtype=torch.bfloat16, device=dev)
        torch.cuda.synchronize()
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            work = hook(out, x, dist.group.WORLD, async_op=True)
        assert work is not None
        work.wait()                      # called on the default stream
        got = out.clone()                # default-stream read: must see the gathered data
        torch.cuda.synchronize()
        assert work.is_completed()
        assert torch.equal(_bits(got), _bits(ref)), it


def test_async_work_orders_another_stream_after_the_kernel():
    run_ranks(_side_stream_case, 2, backend="nccl")
