"""Host-side failure detection and fault injection.

The reference only has ``@record`` plus torchrun's error file (reference: train.py:15, 60); a
dead rank shows up there as an NCCL hang.  Here every rank publishes a heartbeat through the
process group's key-value store *between* steps and checks its peers before the next launch, so a
rank that died, raised or stalled is reported as ``PeerFailure`` on the host while no kernel or
collective of the survivors is in flight.  Device-side waits inside the fused kernels are bounded
and report through a status word (see ``parallel/symm.py``); nothing here touches the GPU.

``FaultInjector`` makes failures on the host for tests: a rank raises, exits, or goes silent at
a chosen step (``ZC_FAULT_INJECT="rank=1,step=3,kind=raise"``).
"""
from __future__ import annotations

import os
import time
from dataclasses import dataclass

import torch.distributed as dist


class PeerFailure(RuntimeError):
    def __init__(self, rank: int, silent_s: float, last_step: int):
        super().__init__(f"rank {rank} sent no heartbeat for {silent_s:.1f}s (last step {last_step})")
        self.rank, self.silent_s, self.last_step = rank, silent_s, last_step


class Heartbeat:
    """``beat_and_check(step)``: publish ``step:time`` and verify that every peer has published
    within ``timeout_s``.  Peers that have not started yet get ``startup_grace_s``."""

    def __init__(self, store, rank: int, world_size: int, timeout_s: float, startup_grace_s: float = 60.0,
                 prefix: str = "zc_hb"):
        self.store, self.rank, self.world, self.timeout_s = store, rank, world_size, timeout_s
        self.grace = startup_grace_s
        self.prefix = prefix
        self.t0 = time.time()

    @classmethod
    def from_default_store(cls, rank: int, world_size: int, timeout_s: float, **kw):
        from torch.distributed.distributed_c10d import _get_default_store

        return cls(_get_default_store(), rank, world_size, timeout_s, **kw)

    def _key(self, r: int) -> str:
        return f"{self.prefix}/{r}"

    def beat(self, step: int) -> None:
        self.store.set(self._key(self.rank), f"{step}:{time.time():.3f}")

    def check(self) -> None:
        now = time.time()
        for r in range(self.world):
            if r == self.rank:
                continue
            try:
                if hasattr(self.store, "check") and not self.store.check([self._key(r)]):
                    raise KeyError
                step_s, ts_s = self.store.get(self._key(r)).decode().split(":")
                silent, last = now - float(ts_s), int(step_s)
            except (KeyError, RuntimeError, ValueError):
                silent, last = now - self.t0, -1
                if silent < self.grace:
                    continue
            if silent > self.timeout_s:
                raise PeerFailure(r, silent, last)

    def beat_and_check(self, step: int) -> None:
        self.beat(step)
        self.check()


@dataclass
class FaultInjector:
    rank: int = -1
    step: int = -1
    kind: str = "raise"   # raise | exit | silent

    @classmethod
    def from_env(cls, var: str = "ZC_FAULT_INJECT"):
        spec = os.environ.get(var, "")
        inj = cls()
        for part in filter(None, spec.split(",")):
            k, v = part.split("=")
            setattr(inj, k, int(v) if k in ("rank", "step") else v)
        return inj

    def maybe_fail(self, rank: int, step: int) -> None:
        """Call between steps, with nothing in flight on the device."""
        if rank != self.rank or step != self.step:
            return
        if self.kind == "raise":
            raise RuntimeError(f"injected failure on rank {rank} at step {step}")
        if self.kind == "exit":
            os._exit(17)
        if self.kind == "silent":
            time.sleep(3600)
