"""End-to-end CPU/gloo runs of train.py: loss parity of compressed vs uncompressed collectives,
checkpoint save -> resume, flag surface, heartbeat failure detection."""
import json
import os
import time

import pytest
import torch

from mp_util import run_ranks

COMMON = ["--synthetic", "--model-shape", "tiny", "--device", "cpu", "-b", "2", "-s", "32", "--lr", "1e-3",
          "--log-freq", "100", "--num-samples", "64"]


def _train(rank, world, extra, loss_log):
    import train  # train.main owns the process group (run_ranks(..., init_pg=False))

    train.main(COMMON + extra + ["--loss-log", loss_log])


def _losses(path):
    return [float(l.split()[1]) for l in open(path).read().split("\n") if l]


def test_loss_parity_compressed_vs_uncompressed(tmp_path):
    a, b, c, d = (str(tmp_path / f"{n}.log") for n in "abcd")
    run_ranks(_train, 2, init_pg=False, args=(["--steps", "6"], a))
    run_ranks(_train, 2, init_pg=False, args=(["--steps", "6", "-q", "--zip-ccl"], b))
    run_ranks(_train, 2, init_pg=False, args=(["--steps", "6", "--master-dtype", "fp32"], c))
    run_ranks(_train, 2, init_pg=False, args=(["--steps", "6", "-q", "--zip-ccl", "--compress-rs", "--master-dtype", "fp32"], d))
    la, lb, lc, ld = _losses(a), _losses(b), _losses(c), _losses(d)
    assert len(la) == len(lb) == len(lc) == len(ld) == 6
    assert la == lb, "lossless all-gather must give a bitwise identical loss curve"
    assert all(abs(x - y) / x < 0.01 for x, y in zip(lc, ld)), (lc, ld)


def test_checkpoint_resume_continues_the_curve(tmp_path):
    full, part = str(tmp_path / "full.log"), str(tmp_path / "part.log")
    save = ["--save-dir", str(tmp_path), "--ckpt-freq", "3", "-q", "--zip-ccl", "--compress-rs",
            "--master-dtype", "fp32"]
    run_ranks(_train, 2, init_pg=False, args=(save + ["-e", "full", "--steps", "6"], full))
    run_ranks(_train, 2, init_pg=False, args=(save + ["-e", "part", "--steps", "3"], part))
    exp = tmp_path / "part"
    assert (exp / "state.json").exists() and (exp / "lr_scheduler.pt").exists()
    assert (exp / "checkpoint" / ".metadata").exists()
    assert (exp / "checkpoint" / "__0_0.distcp").exists() and (exp / "checkpoint" / "__1_0.distcp").exists()
    assert (exp / "rank-1" / "comm_state.pt").exists()
    assert json.load(open(exp / "state.json"))["global_step"] == 3
    run_ranks(_train, 2, init_pg=False, args=(save + ["-e", "part", "--steps", "6"], part))
    lf, lp = _losses(full), _losses(part)
    assert len(lp) == 6
    assert all(abs(x - y) < 2e-3 for x, y in zip(lf, lp)), (lf, lp)


def test_flag_surface_matches_reference():
    import train

    opts = {s for a in train._get_parser()._actions for s in a.option_strings}
    ref = {"-e", "--experiment-name", "-d", "--dataset-name", "--dataset-subset", "-m", "--model-name",
           "--save-dir", "--seed", "--num-epochs", "--lr", "-b", "--batch-size", "--log-freq", "--ckpt-freq",
           "-s", "--seq-length", "--cpu-offload", "-p", "--profiler", "--profiler-wait", "--profiler-warmup",
           "--profiler-active", "--forward-prefetch-distance", "-q", "--quantize", "--zip-ccl"}
    assert ref <= opts
    assert {"--synthetic", "--model-shape", "--device", "--compress-rs", "--act-ckpt", "--steps", "--wire",
            "--transport", "--codec", "--sharding"} <= opts


def _gpt2_quant_actckpt(rank, world, loss_log):
    _train(rank, world, ["--steps", "3", "-q", "--act-ckpt", "--model-shape", "gpt2-tiny",
                         "--forward-prefetch-distance", "2"], loss_log)


def test_gpt2_family_int8_hook_and_activation_checkpointing(tmp_path):
    log = str(tmp_path / "g.log")
    run_ranks(_gpt2_quant_actckpt, 2, init_pg=False, args=(log,))
    ls = _losses(log)
    assert len(ls) == 3 and all(8.0 < l < 10.0 for l in ls)


def test_verbatim_wire_trains_like_the_compressed_one(tmp_path):
    """``--wire verbatim`` changes what crosses the links, not the arithmetic: same loss curve."""
    a, b = str(tmp_path / "a.log"), str(tmp_path / "b.log")
    common = ["--steps", "4", "-q", "--zip-ccl", "--compress-rs", "--model-shape", "gpt2-tiny"]
    run_ranks(_train, 2, init_pg=False, args=(common, a))
    run_ranks(_train, 2, init_pg=False, args=(common + ["--wire", "verbatim"], b))
    assert _losses(a) == _losses(b) and len(_losses(a)) == 4


def _heartbeat_case(rank, world):
    import torch.distributed as dist
    from fsdp_comm_opt_b200.utils.failure import FaultInjector, Heartbeat, PeerFailure

    hb = Heartbeat.from_default_store(rank, world, timeout_s=1.0, startup_grace_s=5.0)
    inj = FaultInjector(rank=1, step=2, kind="raise")
    caught = None
    for step in range(6):
        try:
            inj.maybe_fail(rank, step)
        except RuntimeError:
            # the failing rank stops stepping (between steps, nothing in flight) but stays alive
            time.sleep(4.0)
            return
        try:
            hb.beat_and_check(step)
        except PeerFailure as e:
            caught = e
            break
        time.sleep(0.6)
    assert rank == 0 and caught is not None and caught.rank == 1 and caught.last_step == 1


def test_heartbeat_reports_a_silent_rank_on_the_host():
    run_ranks(_heartbeat_case, 2)


def test_fault_injector_env_parsing(monkeypatch):
    from fsdp_comm_opt_b200.utils.failure import FaultInjector

    monkeypatch.setenv("ZC_FAULT_INJECT", "rank=1,step=3,kind=raise")
    inj = FaultInjector.from_env()
    assert (inj.rank, inj.step, inj.kind) == (1, 3, "raise")
    inj.maybe_fail(0, 3)
    with pytest.raises(RuntimeError):
        inj.maybe_fail(1, 3)


def _train_with_env(rank, world, extra, loss_log, env):
    os.environ.update(env)
    _train(rank, world, extra, loss_log)


def _spawn_exit_codes(fn, world, args):
    """Like ``run_ranks`` but for runs that are expected to die: returns the ranks' exit codes."""
    import torch.multiprocessing as mp

    from mp_util import _entry, _free_port

    ctx = mp.get_context("spawn")
    errq, port = ctx.SimpleQueue(), _free_port()
    procs = [ctx.Process(target=_entry, args=(r, world, port, fn, args, errq, False, "gloo")) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(180)
    for p in procs:
        if p.is_alive():
            p.kill()
    return [p.exitcode for p in procs]


def test_rank_failure_then_resume_from_last_checkpoint(tmp_path):
    """Rank 1 raises on the host before step 5 (the injector runs between steps, nothing in flight);
    rank 0's next collective runs into the process-group timeout, so the whole job ends with an
    error instead of hanging.  Starting the same command again resumes from the checkpoint written
    after step 4 and continues the loss curve of an uninterrupted run (the recovery path of the
    reference: rerun with the same ``-e``, train.py:168-190)."""
    full, part = str(tmp_path / "full.log"), str(tmp_path / "part.log")
    common = ["--save-dir", str(tmp_path), "--ckpt-freq", "2", "-q", "--zip-ccl", "--compress-rs", "--steps", "8",
              "--dist-timeout", "8"]
    run_ranks(_train, 2, init_pg=False, args=(common + ["-e", "full"], full))
    codes = _spawn_exit_codes(_train_with_env, 2, (common + ["-e", "part"], part,
                                                   {"ZC_FAULT_INJECT": "rank=1,step=4,kind=raise"}))
    assert all(c != 0 for c in codes), codes                       # both ranks ended with an error
    assert json.load(open(tmp_path / "part" / "state.json"))["global_step"] == 4
    assert len(_losses(part)) == 4
    run_ranks(_train, 2, init_pg=False, args=(common + ["-e", "part"], part))    # no fault this time
    lf, lp = _losses(full), _losses(part)
    assert len(lp) == 8
    assert all(abs(x - y) < 2e-3 for x, y in zip(lf, lp)), (lf, lp)


def _train_plain(rank, world, argv):
    import train

    train.main(argv)


def test_text_file_dataset_with_byte_tokenizer(tmp_path):
    """The reference's data path (tokenise everything, concatenate, cut into blocks, labels = ids;
    reference: train.py:316-371) on a local text file with the built-in byte-level tokenizer."""
    text = tmp_path / "corpus.txt"
    text.write_text("\n".join(f"line {i}: the quick brown fox jumps over the lazy dog {i * 7919}" for i in range(400)))
    log = str(tmp_path / "t.log")
    run_ranks(_train_plain, 2, init_pg=False, args=([
        "-d", str(text), "-m", "tiny", "--tokenizer", "bytes", "--device", "cpu", "-b", "2", "-s", "32",
        "--lr", "1e-3", "--log-freq", "100", "--steps", "4", "-q", "--zip-ccl", "--loss-log", log],))
    ls = _losses(log)
    assert len(ls) == 4 and ls[-1] < ls[0]          # byte text is learnable, unlike random tokens

    from fsdp_comm_opt_b200.utils.data import load_text_dataset

    ds = load_text_dataset(str(text), None, "bytes", 32, 4096, vocab_size=8192, num_proc=1)
    item = ds[0]
    assert item["input_ids"].shape == (32,) and torch.equal(item["input_ids"], item["labels"])
    assert int(item["input_ids"].max()) < 256


def test_model_names_resolve_like_the_reference_launch_line(tmp_path):
    from fsdp_comm_opt_b200.models import get_config

    assert get_config("openai-community/gpt2-xl") is get_config("gpt2-xl")       # reference: run.sh:1
    hf = {"model_type": "llama", "vocab_size": 1000, "hidden_size": 64, "num_hidden_layers": 2,
          "num_attention_heads": 4, "num_key_value_heads": 2, "intermediate_size": 128, "rope_theta": 5e5}
    (tmp_path / "config.json").write_text(json.dumps(hf))
    cfg = get_config(str(tmp_path))                                               # a local HF directory
    assert (cfg.d_model, cfg.n_kv_heads, cfg.ffn, cfg.rope_theta) == (64, 2, 128, 5e5)
    with pytest.raises(KeyError):
        get_config("no-such/model")


def test_profiler_flag_writes_a_trace(tmp_path):
    run_ranks(_train_plain, 1, init_pg=False, args=(COMMON + [
        "--steps", "3", "-p", "--profiler-wait", "0", "--profiler-warmup", "1", "--profiler-active", "1",
        "-e", "prof", "--save-dir", str(tmp_path)],))
    traces = list((tmp_path / "prof" / "log" / "rank-0").glob("*"))
    assert traces, "the tensorboard trace handler wrote nothing"
