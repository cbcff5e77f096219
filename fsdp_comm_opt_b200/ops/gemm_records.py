"""A linear layer whose weight arrives as v2 codec records: decode fused with the consumer GEMM.

What a compressed all-gather delivers is a buffer of v2 records.  The plain path decodes the whole
weight to bf16 in HBM and then runs the GEMM, which reads it back.  Here the weight is decoded one
slab of output rows at a time into a small ring of bf16 buffers (two or three slabs of a few MB: they
stay in the 126 MB L2), and the GEMM of slab ``s`` runs on the main stream while the decoder, on a
side stream, expands slab ``s + 1`` beside it on the same SMs.  The decoded weight as a whole never
exists in memory, and the GEMM reads its B operand from L2 lines the decoder has just written.

Decoder and GEMM are the hand-written kernels of this package (``zc_v2_decode``,
``gemm_2sm_kernel``); the hand-off per slab is a CUDA event in each direction (slab decoded / ring
slot free), so nothing spins on the device.

The product is formed as ``y^T[N, M] = W[N, K] @ x[M, K]^T`` so that a slab of weight rows gives a
contiguous block of output rows.  (The reference has no counterpart: it decompresses into the FSDP
all-gather output and lets cuBLAS read that, ``main/zipccl_comm.py:134-152``.)
"""
from __future__ import annotations

import torch

from . import codec
from .gemm import gemm

_CHUNK = codec.V2_CHUNK
_SLOT = codec.V2_SLOT


class RecordLinear:
    """``y^T = W @ x^T`` for a weight ``W[N, K]`` held as v2 records of its row-major flat layout.

    ``slab_rows`` weight rows are decoded at a time (``slab_rows * K`` must be a multiple of the
    1024-element chunk so that a slab is a whole number of records); ``ring`` slabs are in flight.
    """

    def __init__(self, N: int, K: int, device, *, slab_rows: int = 1024, ring: int = 3):
        if (slab_rows * K) % _CHUNK or N % slab_rows:
            raise ValueError(f"slab_rows={slab_rows} must divide N={N} and slab_rows*K must be a multiple of {_CHUNK}")
        if slab_rows % 8 or K % 8:
            raise ValueError("slab_rows and K must be multiples of 8")
        self.N, self.K, self.slab_rows, self.ring = N, K, slab_rows, ring
        self.device = torch.device(device)
        self.buf = torch.empty(ring, slab_rows, K, dtype=torch.bfloat16, device=self.device)
        self.side = torch.cuda.Stream(self.device, priority=-1) if self.device.type == "cuda" else None
        self._decoded = [None] * ring
        self._free = [None] * ring

    def __call__(self, x: torch.Tensor, records: torch.Tensor, headers: torch.Tensor,
                 out: torch.Tensor | None = None) -> torch.Tensor:
        N, K, R = self.N, self.K, self.slab_rows
        M = x.shape[0]
        if x.shape[1] != K:
            raise ValueError("x must be [M, K]")
        if out is None:
            out = torch.empty(N, M, dtype=torch.bfloat16, device=x.device)
        slabs = N // R
        cps = R * K // _CHUNK     # records per slab
        if self.side is None:     # CPU: the same slab walk, in order
            for s in range(slabs):
                w = self.buf[s % self.ring]
                codec.v2_decode(records[s * cps * _SLOT:(s + 1) * cps * _SLOT], headers[s * cps:(s + 1) * cps], R * K,
                                w.view(-1))
                out[s * R:(s + 1) * R] = (w.float() @ x.float().t()).to(out.dtype)
            return out
        main = torch.cuda.current_stream(self.device)
        start = torch.cuda.Event()
        start.record(main)
        self.side.wait_event(start)       # records and headers are ready on the caller's stream

        def decode(s):
            slot = s % self.ring
            with torch.cuda.stream(self.side):
                if self._free[slot] is not None:
                    self.side.wait_event(self._free[slot])
                codec.v2_decode(records[s * cps * _SLOT:(s + 1) * cps * _SLOT], headers[s * cps:(s + 1) * cps], R * K,
                                self.buf[slot].view(-1))
                ev = torch.cuda.Event()
                ev.record(self.side)
                self._decoded[slot] = ev

        for s in range(min(self.ring - 1, slabs)):
            decode(s)
        for s in range(slabs):
            if s + self.ring - 1 < slabs:
                decode(s + self.ring - 1)
            slot = s % self.ring
            main.wait_event(self._decoded[slot])
            gemm(self.buf[slot], x, False, True, out=out[s * R:(s + 1) * R])
            ev = torch.cuda.Event()
            ev.record(main)
            self._free[slot] = ev
        return out


def linear_t_plain(x: torch.Tensor, records: torch.Tensor, headers: torch.Tensor, N: int, K: int,
                   w_buf: torch.Tensor | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """The unfused path with the same result layout: decode all of W, then one GEMM."""
    w = codec.v2_decode(records, headers, N * K, None if w_buf is None else w_buf.view(-1)).view(N, K)
    if x.device.type == "cpu":
        y = (w.float() @ x.float().t()).to(torch.bfloat16)
        if out is not None:
            out.copy_(y)
            return out
        return y
    return gemm(w, x, False, True, out=out)
