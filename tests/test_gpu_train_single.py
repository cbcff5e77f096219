"""train.py on one GPU: both sharding back ends, CPU offload (FSDP2 only), activation checkpointing."""
import pytest

from mp_util import run_ranks

pytestmark = pytest.mark.gpu


def _train(rank, world, extra, loss_log):
    import train

    train.main(["--synthetic", "--model-shape", "small", "--device", "cuda", "-b", "1", "-s", "512", "--lr", "1e-4",
                "--log-freq", "2", "--num-samples", "4", "--steps", "6", "--loss-log", loss_log] + extra)


def _losses(path):
    return [float(l.split()[1]) for l in open(path).read().split("\n") if l]


def test_flat_and_fsdp2_back_ends_train_on_one_gpu(tmp_path):
    logs = {k: str(tmp_path / f"{k}.log") for k in ("flat", "flat_ckpt", "fsdp2")}
    run_ranks(_train, 1, init_pg=False, backend="nccl", args=(["-q", "--zip-ccl", "--compress-rs"], logs["flat"]))
    run_ranks(_train, 1, init_pg=False, backend="nccl", args=(["--act-ckpt"], logs["flat_ckpt"]))
    run_ranks(_train, 1, init_pg=False, backend="nccl", args=(["--sharding", "fsdp2", "-q", "--zip-ccl"], logs["fsdp2"]))
    a, b, c = (_losses(logs[k]) for k in ("flat", "flat_ckpt", "fsdp2"))
    assert len(a) == len(b) == len(c) == 6
    assert a[-1] < a[0] and c[-1] < c[0]       # four samples, repeated: the loss falls
    assert a == b                              # recomputation is exact
    assert abs(a[0] - c[0]) < 0.2              # same shape, different initial values


def test_cpu_offload_runs_through_fsdp2(tmp_path):
    """``--cpu-offload`` (reference: train.py:95, 125, 261) keeps parameters, gradients and optimizer
    state on the host; it selects the FSDP2 back end."""
    log = str(tmp_path / "off.log")
    run_ranks(_train, 1, init_pg=False, backend="nccl", args=(["--cpu-offload", "--model-shape", "tiny"], log))
    ls = _losses(log)
    assert len(ls) == 6 and all(l == l for l in ls)
