"""The flat-shard engine on CPU/gloo ranks: loss parity between plain and compressed collectives,
between world sizes, with activation checkpointing, against the FSDP2 back end, and the state
round trip."""
import torch

from mp_util import run_ranks


def _batches(rank, n, vocab=8192, B=2, S=32):
    g = torch.Generator().manual_seed(100 + rank)
    two = [torch.randint(0, vocab, (B, S), generator=g) for _ in range(2)]
    return [two[i % 2] for i in range(n)]  # two alternating batches: the loss falls as they are memorised


def _run(rank, world, kind, steps, out_path, model="tiny"):
    from fsdp_comm_opt_b200.engine import EngineConfig, TrainEngine

    kw = dict(model=model, lr=1e-3, quantize=False, zip_ccl=False, compress_rs=False)
    if kind == "zip":
        kw.update(quantize=True, zip_ccl=True)
    elif kind == "zip+rs":
        kw.update(quantize=True, zip_ccl=True, compress_rs=True)
    elif kind == "ckpt":
        kw.update(act_ckpt=True)
    elif kind == "keep":
        kw.update(reshard_after_forward=False, quantize=True, zip_ccl=True, compress_rs=True)
    elif kind == "fp32":
        kw.update(master_dtype=torch.float32, quantize=True, zip_ccl=True, compress_rs=True)
    eng = TrainEngine(EngineConfig(**kw), torch.device("cpu"))
    losses = [eng.step(b) for b in _batches(rank, steps, eng.model_config.vocab_size)]
    if rank == 0:
        torch.save({"losses": losses, "pool": eng.flat.memory_summary()}, out_path)


def _load(p):
    return torch.load(p, weights_only=True)


def test_flat_engine_lossless_hooks_give_identical_curves(tmp_path):
    paths = {k: str(tmp_path / f"{k.replace('+', '_')}.pt") for k in ("plain", "zip", "zip+rs", "ckpt", "keep")}
    for kind, p in paths.items():
        run_ranks(_run, 2, args=(kind, 5, p))
    base = _load(paths["plain"])["losses"]
    assert len(base) == 5 and base[-1] < base[0]
    assert _load(paths["zip"])["losses"] == base          # lossless all-gather
    assert _load(paths["zip+rs"])["losses"] == base       # bf16 rows, fp32 sum of two ranks
    assert _load(paths["ckpt"])["losses"] == base         # recomputation is exact
    assert _load(paths["keep"])["losses"] == base         # parameters kept gathered until backward
    assert _load(paths["keep"])["pool"]["reshard_after_forward"] is False
    pool = _load(paths["plain"])["pool"]
    # steady state: a handful of buffers, not one per layer and step
    assert pool["param_buffers"] <= 9 and pool["grad_buffers"] <= 6, pool


def test_flat_engine_gpt2_family_and_fp32_master(tmp_path):
    a, b = str(tmp_path / "a.pt"), str(tmp_path / "b.pt")
    run_ranks(_run, 2, args=("zip+rs", 4, a, "gpt2-tiny"))
    la = _load(a)["losses"]
    assert len(la) == 4 and la[-1] < la[0]
    run_ranks(_run, 2, args=("fp32", 4, b))
    lb = _load(b)["losses"]
    assert len(lb) == 4 and lb[-1] < lb[0]


def _one_vs_two(rank, world, out_path):
    """World size 2 against a single process that sees both ranks' batches as one batch."""
    from fsdp_comm_opt_b200.engine import EngineConfig, TrainEngine

    eng = TrainEngine(EngineConfig(model="tiny", lr=1e-3, quantize=False, zip_ccl=False, compress_rs=False),
                      torch.device("cpu"))
    if world == 1:
        b0, b1 = _batches(0, 3), _batches(1, 3)
        losses = [eng.step(torch.cat([x, y])) for x, y in zip(b0, b1)]
    else:
        mine = [eng.step(b) for b in _batches(rank, 3)]
        t = torch.tensor(mine)
        import torch.distributed as dist

        dist.all_reduce(t)
        losses = (t / world).tolist()
    if rank == 0:
        torch.save(losses, out_path)


def test_flat_engine_matches_single_process_on_the_global_batch(tmp_path):
    a, b = str(tmp_path / "w1.pt"), str(tmp_path / "w2.pt")
    run_ranks(_one_vs_two, 1, args=(a,))
    run_ranks(_one_vs_two, 2, args=(b,))
    l1, l2 = _load(a), _load(b)
    assert abs(l1[0] - l2[0]) < 2e-3, (l1, l2)            # same weights, same tokens
    assert all(abs(x - y) < 2e-2 for x, y in zip(l1, l2)), (l1, l2)


def _flat_vs_fsdp2(rank, world, out_path):
    from fsdp_comm_opt_b200.engine import EngineConfig, TrainEngine

    common = dict(model="tiny", lr=1e-3, quantize=True, zip_ccl=True, compress_rs=False)
    flat = TrainEngine(EngineConfig(sharding="flat", **common), torch.device("cpu"))
    sd = flat.flat.full_state_dict()
    ref = TrainEngine(EngineConfig(sharding="fsdp2", **common), torch.device("cpu"))
    from torch.distributed.checkpoint.state_dict import StateDictOptions, set_model_state_dict

    set_model_state_dict(ref.model, sd, options=StateDictOptions(full_state_dict=True, broadcast_from_rank0=False))
    la = [flat.step(b) for b in _batches(rank, 3)]
    lb = [ref.step(b) for b in _batches(rank, 3)]
    # round trip of the flat engine's own state
    sd2 = flat.flat.full_state_dict()
    flat.flat.load_full_state_dict(sd2)
    sd3 = flat.flat.full_state_dict()
    same = all(torch.equal(sd2[k], sd3[k]) for k in sd2)
    if rank == 0:
        torch.save({"flat": la, "fsdp2": lb, "same": same, "keys": sorted(sd)[:3]}, out_path)


def test_flat_engine_against_the_fsdp2_back_end(tmp_path):
    p = str(tmp_path / "x.pt")
    run_ranks(_flat_vs_fsdp2, 2, args=(p,))
    r = _load(p)
    assert r["same"]
    assert abs(r["flat"][0] - r["fsdp2"][0]) < 1e-3, r    # identical weights: same first loss
    assert all(abs(x - y) < 2e-2 for x, y in zip(r["flat"], r["fsdp2"])), r
