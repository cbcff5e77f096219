"""Comm hooks and AggregatedWork on CPU/gloo ranks against the uncompressed collectives."""
from datetime import timedelta

import pytest
import torch
import torch.distributed as dist

from mp_util import run_ranks


def _bits(t):
    return t.view(torch.int16)


def _ag_case(rank, world, version, async_op):
    from fsdp_comm_opt_b200.parallel.hooks import ZipCCLAllGather

    hook = ZipCCLAllGather(codec_version=version)
    for n in (1, 777, 4096, 10001):
        g = torch.Generator().manual_seed(100 + rank)
        out = torch.zeros(world * n, dtype=torch.bfloat16)
        inp = out.narrow(0, n * rank, n)          # FSDP2 passes a view of the output
        inp.copy_((torch.randn(n, generator=g) * 0.02).to(torch.bfloat16))
        ref = torch.zeros_like(out)
        dist.all_gather_into_tensor(ref, inp.clone())
        work = hook(out, inp, dist.group.WORLD, async_op=async_op)
        if async_op:
            assert isinstance(work, dist.Work)
            work.wait()            # wait(None) must work
            assert work.is_completed() and work.is_success() and work.exception() is None
        else:
            assert work is None
        assert torch.equal(_bits(out), _bits(ref)), (version, n)
    # non-bf16 input goes through uncompressed and stays exact
    x = torch.full((8,), float(rank) + 0.123456789, dtype=torch.float32)
    out = torch.zeros(world * 8, dtype=torch.float32)
    hook(out, x, dist.group.WORLD)
    assert torch.equal(out.view(world, 8)[:, 0], torch.arange(world, dtype=torch.float32) + 0.123456789)


@pytest.mark.parametrize("version", ["v1", "v2"])
@pytest.mark.parametrize("async_op", [False, True])
def test_zip_all_gather_is_bit_exact(version, async_op):
    run_ranks(_ag_case, 2, (version, async_op))


def test_zip_all_gather_world3():
    run_ranks(_ag_case, 3, ("v2", False))


def _quant_case(rank, world):
    from fsdp_comm_opt_b200.parallel.hooks import QuantizedAllGather

    n = 3000
    g = torch.Generator().manual_seed(rank)
    x = (torch.randn(n, generator=g) * (0.01 * (rank + 1))).to(torch.bfloat16)
    ref = torch.zeros(world * n, dtype=torch.bfloat16)
    dist.all_gather_into_tensor(ref, x)
    for async_op in (False, True):
        out = torch.zeros(world * n, dtype=torch.bfloat16)
        w = QuantizedAllGather()(out, x, dist.group.WORLD, async_op=async_op)
        if w is not None:
            w.wait(timedelta(seconds=30))
        for r in range(world):
            seg, rseg = out[r * n:(r + 1) * n].float(), ref[r * n:(r + 1) * n].float()
            scale = rseg.abs().max() / 127
            assert (seg - rseg).abs().max() <= scale * 1.01   # scale/2 plus bf16 rounding of the result (127*scale*2^-8)
    # bypass for small / integer inputs
    out = torch.zeros(world * 4, dtype=torch.int64)
    QuantizedAllGather()(out, torch.full((4,), rank, dtype=torch.int64), dist.group.WORLD)
    assert out.tolist() == sum(([r] * 4 for r in range(world)), [])
    out = torch.zeros(world * 4, dtype=torch.bfloat16)
    QuantizedAllGather(min_quantize_numel=100)(out, torch.full((4,), 1.2345, dtype=torch.bfloat16), dist.group.WORLD)
    assert torch.equal(out, torch.full((world * 4,), 1.2345, dtype=torch.bfloat16))


def test_quantized_all_gather_error_bound():
    run_ranks(_quant_case, 2)


def _rs_case(rank, world):
    from fsdp_comm_opt_b200.parallel.hooks import ZipCCLReduceScatter

    shard = 5000
    g = torch.Generator().manual_seed(7 + rank)
    # bf16-representable fp32 input: compressed RS must equal the fp32 collective up to summation order
    x = (torch.randn(world * shard, generator=g) * 1e-3).to(torch.bfloat16).float()
    ref = torch.zeros(shard)
    dist.reduce_scatter_tensor(ref, x.clone(), op=dist.ReduceOp.SUM)
    for op, scale in ((dist.ReduceOp.SUM, 1.0), (dist.ReduceOp.AVG, 1.0 / world)):
        hook = ZipCCLReduceScatter()
        out = torch.zeros(shard)
        hook(out, x.clone(), dist.group.WORLD, op)
        assert torch.allclose(out, ref * scale, rtol=1e-6, atol=1e-9)
        assert hook._residual is not None and float(hook._residual.abs().max()) == 0.0
    pm = dist._make_nccl_premul_sum(0.25) if hasattr(dist, "_make_nccl_premul_sum") else None
    if pm is not None:
        out = torch.zeros(shard)
        ZipCCLReduceScatter()(out, x.clone(), dist.group.WORLD, pm)
        assert torch.allclose(out, ref * 0.25, rtol=1e-6, atol=1e-9)
    # true fp32 input: error feedback keeps the accumulated sum close over many steps
    hook = ZipCCLReduceScatter(error_feedback=True, residual_dtype=torch.float32)
    hook_off = ZipCCLReduceScatter(error_feedback=False)
    acc_ref, acc_ef, acc_no = torch.zeros(shard), torch.zeros(shard), torch.zeros(shard)
    const = torch.randn(world * shard, generator=g) * 1e-3
    for _ in range(40):
        r = torch.zeros(shard)
        dist.reduce_scatter_tensor(r, const.clone(), op=dist.ReduceOp.SUM)
        a, b = torch.zeros(shard), torch.zeros(shard)
        hook(a, const.clone(), dist.group.WORLD, dist.ReduceOp.SUM)
        hook_off(b, const.clone(), dist.group.WORLD, dist.ReduceOp.SUM)
        acc_ref += r; acc_ef += a; acc_no += b
    err_ef = (acc_ef - acc_ref).abs().max().item()
    err_no = (acc_no - acc_ref).abs().max().item()
    assert err_ef < err_no / 5, (err_ef, err_no)
    sd = hook.state_dict()
    h2 = ZipCCLReduceScatter(residual_dtype=torch.float32)
    h2.load_state_dict(sd)
    assert torch.equal(h2._residual, hook._residual)


def test_compressed_reduce_scatter_and_error_feedback():
    run_ranks(_rs_case, 2)


def _work_case(rank, world):
    import threading

    from fsdp_comm_opt_b200.parallel.work import AggregatedWork

    calls = []
    t = torch.ones(4) * (rank + 1)
    w = dist.all_reduce(t, async_op=True)
    agg = AggregatedWork([w], postprocess_fn=lambda: calls.append(1))
    threads = [threading.Thread(target=agg.wait) for _ in range(4)] + [threading.Thread(target=agg.is_completed)]
    [th.start() for th in threads]
    [th.join() for th in threads]
    assert agg.wait(timedelta(seconds=5)) is True
    assert calls == [1], "postprocess must run exactly once"
    assert t[0].item() == sum(range(1, world + 1))
    assert agg.result() is not None
    t2 = torch.ones(2)
    agg2 = AggregatedWork([dist.all_reduce(t2, async_op=True)], postprocess_fn=lambda: calls.append(2))
    agg2.get_future().wait()
    assert calls == [1, 2]

    def boom():
        raise ValueError("decode failed")

    agg3 = AggregatedWork([dist.all_reduce(torch.ones(1), async_op=True)], postprocess_fn=boom)
    with pytest.raises(ValueError):
        agg3.wait()
    assert isinstance(agg3.exception(), ValueError) and not agg3.is_success()
    with pytest.raises(ValueError):
        agg3.wait()
    agg4 = AggregatedWork([], postprocess_fn=lambda: calls.append(4))
    agg4.block_current_stream()
    assert calls[-1] == 4


def test_aggregated_work_semantics():
    run_ranks(_work_case, 2)


def _verbatim_case(rank, world):
    """``wire="verbatim"`` away from the fused transport: the all-gather is the plain library
    collective, the reduce-scatter keeps its arithmetic (same result as the compressed wire)."""
    import torch.distributed as dist
    from fsdp_comm_opt_b200.parallel.hooks import ZipCCLAllGather, ZipCCLReduceScatter

    g = torch.Generator().manual_seed(50 + rank)
    x = (torch.randn(5000, generator=g) * 0.02).to(torch.bfloat16)
    out = torch.zeros(world * 5000, dtype=torch.bfloat16)
    ref = torch.zeros_like(out)
    dist.all_gather_into_tensor(ref, x)
    hook = ZipCCLAllGather(wire="verbatim")
    w = hook(out, x, dist.group.WORLD, async_op=True)
    if w is not None:
        w.wait()
    assert torch.equal(_bits(out), _bits(ref)) and hook.last_transport == "lib"
    rows = torch.randn(world * 3000, generator=g) * 1e-3
    o1, o2 = torch.zeros(3000), torch.zeros(3000)
    ZipCCLReduceScatter(wire="verbatim")(o1, rows.clone(), dist.group.WORLD, dist.ReduceOp.AVG)
    ZipCCLReduceScatter()(o2, rows.clone(), dist.group.WORLD, dist.ReduceOp.AVG)
    assert torch.equal(o1, o2)
    # nibble-mode records on the library transport's v2 protocol: still bit exact, same reduce-scatter result
    out_n = torch.zeros_like(out)
    hook_n = ZipCCLAllGather(wire="nibble", codec_version="v2")
    hook_n(out_n, x, dist.group.WORLD)
    assert torch.equal(_bits(out_n), _bits(ref))
    o3 = torch.zeros(3000)
    ZipCCLReduceScatter(wire="nibble")(o3, rows.clone(), dist.group.WORLD, dist.ReduceOp.AVG)
    assert torch.equal(o3, o2)
    with pytest.raises(ValueError):
        ZipCCLAllGather(wire="zstd")


def test_verbatim_wire_on_the_library_transport():
    run_ranks(_verbatim_case, 2)
