"""Spawn ``world`` gloo ranks on CPU and run ``fn(rank, world, *args)`` in each."""
import os
import socket
import traceback

import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _entry(rank, world, port, fn, args, errq, init_pg, backend="gloo"):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      OMP_NUM_THREADS="1")
    try:
        if backend == "nccl":
            import torch

            os.environ["LOCAL_RANK"] = str(rank)
            os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
            torch.cuda.set_device(rank)
        if init_pg:
            if backend == "nccl":
                import torch

                dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
            else:
                dist.init_process_group("gloo", rank=rank, world_size=world)
        fn(rank, world, *args)
        if init_pg and dist.is_initialized():
            dist.barrier()
            dist.destroy_process_group()
    except BaseException:
        errq.put((rank, traceback.format_exc()))
        raise


def run_ranks(fn, world=2, args=(), init_pg=True, timeout=240, backend="gloo"):
    """``init_pg=False``: ``fn`` brings up (and tears down) its own process group from the env."""
    ctx = mp.get_context("spawn")
    errq = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_entry, args=(r, world, port, fn, args, errq, init_pg, backend)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout)
    errs = []
    while not errq.empty():
        errs.append(errq.get())
    for p in procs:
        if p.is_alive():
            p.kill()
            errs.append((-1, "rank timed out"))
    assert not errs, "\n".join(f"[rank {r}] {e}" for r, e in errs)
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
