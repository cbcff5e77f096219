"""Symmetric-memory channels that drive the fused collective kernels (``csrc/symm_collectives.cu``).

A ``Channel`` owns one symmetric buffer per (process group, device, role): control words, arrival
flags and two parities of staging slots.  The buffer is allocated with
``torch.distributed._symmetric_memory`` and exchanged once by rendezvous (a collective, so every
rank must create and grow channels in the same order -- FSDP2 calls its hooks in the same order on
every rank).  After that a collective is ONE kernel launch on the current stream: no NCCL call, no
host sync, no allocation.  The reference has no counterpart: all of its traffic goes through
``dist.all_gather_into_tensor`` (reference: main/zipccl_comm.py:106-132).

Sequence numbers: every call on a channel increments ``seq``; the kernels use ``seq & 1`` as the
staging parity and wait (bounded) for the peers' ``done >= seq - 2`` before reusing a parity.

Failure reporting: a device wait that runs out sets status words in the control block and the
library's per-device health word; the kernel then returns normally.  The fused AdamW kernel reads
the health word on the device and leaves parameters and moments untouched when it is set, so a
step whose collectives gave up is never applied, without any host synchronisation in the step.
``check_status()`` (synchronising) turns the status words into ``SymmTimeout``; the training loop
calls it where it synchronises anyway (next to the loss read) and before every checkpoint.
The ``Work`` returned on the async path carries an event recorded on the launch stream, so
``wait()`` orders the caller's stream after the kernel; it does not poll the status words.
"""
from __future__ import annotations

import ctypes
import logging
import os

import torch
import torch.distributed as dist

from .. import _lib
from ..ops import codec
from .work import AggregatedWork

_CHANNELS: dict = {}
_AVAILABLE: dict = {}
_WHY: dict = {}
LOGGER = logging.getLogger("fsdp_comm_opt_b200.symm")

CTRL_WORDS = 1024
CW_STATUS, CW_STATUS_PEER, CW_STATUS_GROUP, CW_WIRE_LO, CW_HEALTH_PTR = 65, 66, 67, 68, 72
GUARD = 4096          # canary bytes in front of and behind every symmetric buffer
CANARY = 0xA5


class SymmCorruption(RuntimeError):
    """A canary region next to a symmetric buffer was overwritten, or a bounds-checked store was refused."""


class SymmTimeout(RuntimeError):
    """A bounded device-side wait expired (peer did not arrive in time)."""

    def __init__(self, code: int, peer: int, group: int):
        what = {1: "waiting for a peer to release the staging buffer", 2: "waiting for a peer's data",
                3: "refusing a store outside the destination slot (bounds-checked build)"}.get(code, "?")
        super().__init__(f"fused collective timed out {what}: peer rank {peer}, group {group}")
        self.code, self.peer, self.group = code, peer, group


def _symm_mod():
    import torch.distributed._symmetric_memory as symm_mem

    return symm_mem


def available(group) -> bool:
    """True when symmetric memory can be rendezvoused for ``group`` (probed once, collectively).
    ``why_unavailable(group)`` gives the reason after a False."""
    key = group.group_name if hasattr(group, "group_name") else str(group)
    if key in _AVAILABLE:
        return _AVAILABLE[key]
    if os.environ.get("ZC_DISABLE_SYMM", "0") == "1" or not torch.cuda.is_available():
        _AVAILABLE[key], _WHY[key] = False, "disabled by ZC_DISABLE_SYMM or no CUDA device"
        return False
    ok, why = False, ""
    if dist.get_backend(group) != "nccl":
        why = f"backend is {dist.get_backend(group)}, not nccl"
    elif dist.get_world_size(group) < 2:
        why = "world size 1"
    elif not hasattr(_lib.cuda()._lib, "zc_symm_all_gather"):
        why = "libzc_cuda.so has no fused collective kernels"
    else:
        try:
            symm_mem = _symm_mod()
            t = symm_mem.empty(4096, dtype=torch.uint8, device=torch.device("cuda", torch.cuda.current_device()))
            hdl = symm_mem.rendezvous(t, group)
            ok = hdl is not None and len(hdl.buffer_ptrs) == dist.get_world_size(group)
            if not ok:
                why = "rendezvous returned no peer pointers"
        except (RuntimeError, ImportError, AttributeError, NotImplementedError) as e:
            why = f"{type(e).__name__}: {e}"
    # every rank must agree, otherwise some would wait in a kernel for peers that use NCCL
    flag = torch.tensor([1 if ok else 0], device=torch.device("cuda", torch.cuda.current_device()))
    dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
    agreed = bool(flag.item())
    if ok and not agreed:
        why = "another rank could not rendezvous symmetric memory"
    if not agreed:
        LOGGER.warning("symmetric-memory transport unavailable: %s", why)
    _AVAILABLE[key], _WHY[key] = agreed, why
    return agreed


def why_unavailable(group) -> str:
    key = group.group_name if hasattr(group, "group_name") else str(group)
    return _WHY.get(key, "")


_WIRE_CODE = {"compressed": 0, "verbatim": 1, "nibble": 2}


class Channel:
    def __init__(self, group, device: torch.device, kind: str):
        self.group, self.device, self.kind = group, device, kind
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.seq = 0
        self.nc_max = 0
        self.buf = None
        self.hdl = None
        # a peer may lag by a checkpoint write or a profiler flush; NCCL would simply wait, so the
        # bound is generous (tests set ``timeout_s`` to a second)
        self.timeout_s = float(os.environ.get("ZC_SYMM_TIMEOUT_S", "120"))
        self.calls = 0
        self.elements = 0
        self._wire_carry = 0   # bytes counted in buffers that were since replaced by larger ones
        sm = torch.cuda.get_device_properties(device).multi_processor_count
        # The codec is integer-ALU work, the GEMMs it overlaps with are tensor-pipe work, and a
        # collective CTA needs only 8 KB of shared memory, so two of them fit beside a GEMM CTA on
        # every SM.  One pusher and one decoder CTA per SM keeps the wall time of a collective
        # short; fewer CTAs make it encode-bound (measured: 24+37 CTAs -> 89 GB/s bus at 2 GPUs).
        # Progress argument for two collectives in flight at once (FSDP overlaps the next all-gather
        # with a reduce-scatter): pusher CTAs never wait, so they always retire; only decoder CTAs
        # hold an SM slot while they wait for a peer.  Beside a resident GEMM CTA an SM still has
        # room for two collective CTAs (2 x sm slots); keeping the decoders of both kernels below
        # that (2 x (sm - 20)) always leaves slots through which every kernel's pushers drain, on
        # every rank, whatever order the ranks scheduled the two kernels in.
        self.push_ctas = int(os.environ.get("ZC_SYMM_PUSH_CTAS", str(sm)))
        self.dec_ctas = int(os.environ.get("ZC_SYMM_DEC_CTAS", str(max(8, sm - 20))))
        # Budget of a collective that runs in the shadow of a layer's GEMMs (``urgent=False``).
        # Measured on Llama-3-8B at two ranks: a small budget (32 + 48 CTAs) makes every collective run
        # for milliseconds beside the GEMMs and slows them all that time (260 ms per step); the full
        # budget gets the same codec work out of the way in a fraction of a millisecond (240 ms per
        # step).  So background collectives default to the full budget too; ZC_SYMM_BG_* lowers it.
        self.bg_push_ctas = int(os.environ.get("ZC_SYMM_BG_PUSH_CTAS", str(self.push_ctas)))
        self.bg_dec_ctas = int(os.environ.get("ZC_SYMM_BG_DEC_CTAS", str(self.dec_ctas)))
        # Budget of a collective that has the GPU to itself (``exclusive=True``: no GEMM resident, no
        # second collective whose pushers need slots, so the progress argument above does not bind).
        # Measured at four ranks, 2^28 elements: the all-gather is bound by its decoders (148 + 276 CTAs:
        # 0.56 ms against 0.68 ms with the in-step budget, NCCL 0.76 ms), the reduce-scatter by both halves
        # (296 + 296: 0.87 ms against 1.02 ms, NCCL fp32 1.36 ms); more all-gather pushers than one per SM
        # only take issue slots from its decoders (296 + 296: 0.66 ms).
        if kind == "rs":
            self.excl_push_ctas, self.excl_dec_ctas = 2 * sm, 2 * sm
        else:
            self.excl_push_ctas, self.excl_dec_ctas = sm, max(8, 2 * sm - 20)
        self._lib = _lib.cuda()
        self._lib._lib.zc_symm_buffer_bytes.restype = ctypes.c_int64
        self._lib._lib.zc_symm_buffer_bytes.argtypes = [ctypes.c_int, ctypes.c_int64]

    # -- buffer management -----------------------------------------------------------------------
    def reserve(self, numel_per_source: int) -> None:
        """Make sure messages of ``numel_per_source`` elements per source fit (collective when it
        has to grow: allocates a new symmetric buffer and rendezvouses it)."""
        nc = codec.v2_num_chunks(numel_per_source)
        if nc <= self.nc_max:
            return
        symm_mem = _symm_mod()
        if self.buf is not None:
            torch.cuda.synchronize(self.device)
            dist.barrier(group=self.group)  # nobody may still be pushing into the old buffer
            # the byte counter lives in the buffer that is about to be replaced
            self._wire_carry += int(self._ctrl()[CW_WIRE_LO:CW_WIRE_LO + 2].view(torch.int64).item())
        nc_max = max(nc, 1024)
        nbytes = int(self._lib._lib.zc_symm_buffer_bytes(self.world, nc_max))
        # [guard | buffer the kernels see | guard]: the guards carry a fixed pattern that no kernel may
        # touch; check_canaries() reads them back (peers write into this allocation over NVLink, so a
        # wrong offset on ANY rank shows up here)
        raw = symm_mem.empty(nbytes + 2 * GUARD, dtype=torch.uint8, device=self.device)
        raw[:GUARD].fill_(CANARY)
        raw[GUARD + nbytes:].fill_(CANARY)
        buf = raw[GUARD:GUARD + nbytes]
        # flags must start below any sequence number; zero the control block and the flag area
        flag_bytes = (2 * self.world * ((nc_max + 63) // 64) * 4 + 127) // 128 * 128
        buf[: CTRL_WORDS * 4 + flag_bytes].zero_()
        # where the kernels report a wait that ran out besides the status words: the library's health
        # word, which the fused optimizer step reads on the device
        with torch.cuda.device(self.device):
            health = int(self._lib.zc_health_word() or 0)
        buf[CW_HEALTH_PTR * 4:CW_HEALTH_PTR * 4 + 8].view(torch.int64).fill_(health)
        torch.cuda.synchronize(self.device)
        hdl = symm_mem.rendezvous(raw, self.group)
        dist.barrier(group=self.group)
        self.raw, self.buf, self.hdl, self.nc_max, self.seq = raw, buf, hdl, nc_max, 0
        self._peer_table = torch.tensor([int(p) + GUARD for p in hdl.buffer_ptrs], dtype=torch.int64, device=self.device)
        self.peers_dev = self._peer_table.data_ptr()
        self.local_ptr = int(hdl.buffer_ptrs[self.rank]) + GUARD
        # NVSwitch multicast mapping of the buffer (0 when the fabric or the driver has none): the
        # all-gather then stores its payload once instead of once per peer.  Measured at 2^28
        # elements: 387 against 471 GB/s bus on two ranks (the store also lands in the sender's own
        # copy) and 459 against 460 on eight (the receiving side's decode is the limit, not the
        # bytes leaving the GPU), so it is opt-in: ZC_SYMM_MULTICAST=1 turns it on.
        mc = int(getattr(hdl, "multicast_ptr", 0) or 0)
        self.mc_ptr = (mc + GUARD) if (mc and os.environ.get("ZC_SYMM_MULTICAST", "0") == "1") else 0

    def _next_seq(self) -> int:
        self.seq += 1
        return self.seq

    # -- status ----------------------------------------------------------------------------------
    def _ctrl(self) -> torch.Tensor:
        return self.buf[: CTRL_WORDS * 4].view(torch.int32)

    def check_status(self) -> None:
        """Synchronises the device and raises ``SymmTimeout`` when a bounded wait expired."""
        if self.buf is None:
            return
        c = self._ctrl()[CW_STATUS:CW_STATUS + 3].tolist()
        if c[0] != 0:
            self._ctrl()[CW_STATUS:CW_STATUS + 3].zero_()
            with torch.cuda.device(self.device):
                self._lib.zc_health_read_and_clear()  # this report consumes the failure
            if c[0] == 3:
                raise SymmCorruption(f"a store outside its slot was refused: peer rank {c[1]}, chunk {c[2]}")
            raise SymmTimeout(c[0], c[1], c[2])

    def check_canaries(self) -> None:
        """Synchronises and raises ``SymmCorruption`` when a guard region around the buffer changed."""
        if self.buf is None:
            return
        n = self.buf.numel()
        front, back = self.raw[:GUARD], self.raw[GUARD + n:]
        bad = int((front != CANARY).sum().item()) + int((back != CANARY).sum().item())
        if bad:
            raise SymmCorruption(f"{bad} canary bytes around the {self.kind!r} staging buffer of rank {self.rank} "
                                 "were overwritten")

    def wire_bytes(self) -> int:
        """Bytes this rank has pushed over NVLink on this channel so far (synchronises)."""
        if self.buf is None:
            return 0
        return self._wire_carry + int(self._ctrl()[CW_WIRE_LO:CW_WIRE_LO + 2].view(torch.int64).item())

    # -- collectives -----------------------------------------------------------------------------
    def _budget(self, urgent: bool, exclusive: bool = False):
        if exclusive:
            return self.excl_push_ctas, self.excl_dec_ctas
        return (self.push_ctas, self.dec_ctas) if urgent else (min(self.push_ctas, self.bg_push_ctas),
                                                                min(self.dec_ctas, self.bg_dec_ctas))

    def all_gather(self, output_tensor: torch.Tensor, x: torch.Tensor, mode: str = "zip", async_op: bool = False,
                   urgent: bool = True, wire: str = "compressed", exclusive: bool = False):
        """``mode="zip"``: lossless v2 codec (``wire`` "compressed" or "nibble"), or with ``wire="verbatim"`` the
        raw bf16 bytes on the same protocol.  ``mode="int8"``: per-shard absmax int8 (every rank, the source included, ends
        up with the dequantised values)."""
        if mode not in ("zip", "int8"):
            raise ValueError(f"unknown all-gather mode {mode!r}")
        if x.dtype != torch.bfloat16 or output_tensor.dtype != torch.bfloat16:
            raise TypeError("the fused all-gather moves bf16 tensors")
        n = x.numel()
        self.reserve(n)
        seq = self._next_seq()
        fn = self._lib.zc_symm_all_gather if mode == "zip" else self._lib.zc_symm_all_gather_int8
        push, dec = self._budget(urgent, exclusive)
        args = (x.data_ptr(), output_tensor.data_ptr(), self.peers_dev, self.local_ptr, self.mc_ptr or None, n, self.rank,
                self.world, self.nc_max, seq, push, dec, self.timeout_s)
        if mode == "zip":
            args += (_WIRE_CODE[wire],)
        _lib.check(fn(*args, _lib.stream_ptr(self.device)), "zc_symm_all_gather")
        self.calls += 1
        self.elements += n * (self.world - 1)
        return self._work() if async_op else None

    def _work(self) -> AggregatedWork:
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(self.device))
        return AggregatedWork([], ready_event=ev)

    def reduce_scatter(self, output_tensor: torch.Tensor, x: torch.Tensor, scale: float, residual, async_op=False,
                       urgent: bool = True, wire: str = "compressed", exclusive: bool = False):
        shard = x.numel() // self.world
        if output_tensor.numel() != shard or output_tensor.dtype not in (torch.float32, torch.bfloat16):
            raise ValueError("output must hold numel/world fp32 or bf16 elements")
        if residual is not None and residual.dtype != torch.bfloat16:
            raise TypeError("the fused reduce-scatter keeps its residual in bf16")
        self.reserve(shard)
        seq = self._next_seq()
        push, dec = self._budget(urgent, exclusive)
        _lib.check(self._lib.zc_symm_reduce_scatter(
            x.data_ptr(), output_tensor.data_ptr(), _lib.ptr(residual), self.peers_dev, self.local_ptr, shard,
            self.rank, self.world, self.nc_max, seq, int(x.dtype == torch.float32),
            int(output_tensor.dtype == torch.float32), float(scale), push, dec,
            self.timeout_s, _WIRE_CODE[wire], _lib.stream_ptr(self.device)), "zc_symm_reduce_scatter")
        self.calls += 1
        self.elements += shard * (self.world - 1)
        return self._work() if async_op else None


def channel_for(group, device: torch.device, kind: str) -> Channel:
    key = (group.group_name if hasattr(group, "group_name") else str(group), str(device), kind)
    ch = _CHANNELS.get(key)
    if ch is None:
        ch = _CHANNELS[key] = Channel(group, device, kind)
    return ch


def all_channels():
    return list(_CHANNELS.values())
