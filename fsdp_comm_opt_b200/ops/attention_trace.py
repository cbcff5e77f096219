"""Phase timeline of the attention kernels, read from their SM-clock trace hooks.

    python -m fsdp_comm_opt_b200.ops.attention_trace {fwd,bwd} [--seq 4096] [--heads 32] [--kv-heads 8]

CTA 0 of ``zc_attn_fwd_2q`` / ``zc_attn_bwd_kt`` (the heaviest CTA of the launch) stamps
``clock64()`` at the phase boundaries of one softmax/compute warp and of its MMA issuer threads
into a device buffer installed with ``zc_attn_*_set_trace``.  This prints the per-block (forward)
or per-iteration (backward) cycle counts of each phase, which is how the kernels were tuned: it
shows directly whether a block is spent waiting for the tensor core, for the previous P V product,
or in the element-wise arithmetic.  The stamps are taken between ``asm volatile`` instructions, so
plain arithmetic may be scheduled across a boundary; read them as phase totals, not instruction
timings.
"""
from __future__ import annotations

import argparse
import ctypes

import torch

from . import attention
from .. import _lib


def _install(name: str, buf):
    fn = getattr(_lib.cuda()._lib, name)
    fn.argtypes = [ctypes.c_void_p]
    fn.restype = None
    fn(buf.data_ptr() if buf is not None else None)


def _rows(t, slot, idxs, n):
    out = []
    for i in idxs:
        r = [int(x) for x in t[slot, i, :n]]
        out.append((i, [r[k + 1] - r[k] for k in range(n - 1)], int(t[slot, i + 1, 0]) - r[0]))
    return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("which", choices=["fwd", "bwd"])
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    args = ap.parse_args()
    B, S, Hq, Hkv, D = 1, args.seq, args.heads, args.kv_heads, 128
    dev = torch.device("cuda")
    torch.manual_seed(0)
    qkv = (torch.randn(B, S, Hq + 2 * Hkv, D, device=dev) * 0.5).bfloat16().requires_grad_()
    g = torch.randn(B, S, Hq, D, device=dev).bfloat16()
    if args.which == "fwd":
        run = lambda: attention.causal_attention(qkv.detach(), Hq, Hkv)
        tr = torch.zeros(2 * 128 * 8, dtype=torch.int64, device=dev)
        setter, shape = "zc_attn_fwd_2q_set_trace", (2, 128, 8)
    else:
        run = lambda: torch.autograd.grad(attention.causal_attention(qkv, Hq, Hkv), qkv, g)
        tr = torch.zeros(3 * 256 * 8, dtype=torch.int64, device=dev)
        setter, shape = "zc_attn_bwd_kt_set_trace", (3, 256, 8)
    for _ in range(3):
        run()
    torch.cuda.synchronize()
    _install(setter, tr)
    run()
    torch.cuda.synchronize()
    _install(setter, None)
    t = tr.view(*shape).cpu()
    n_units = min(shape[1] - 2, (S // 64) - 2)
    picks = list(range(1, 5)) + list(range(n_units - 6, n_units - 2))
    if args.which == "fwd":
        print("softmax warp 2 (tile 0), cycles per 64-key block: "
              "[wait S, load S, max/alpha, wait P buffer (+rescale), exp+store P, fence+arrive] | block total")
        for i, d, tot in _rows(t, 0, picks, 7):
            print(f"  block {i:3d}: {d} | {tot}")
        print("MMA issuer of tile 0: [issue S(j+1), wait P(j), issue P V(j)] | loop total")
        for i, d, tot in _rows(t, 1, picks, 4):
            print(f"  block {i:3d}: {d} | {tot}")
    else:
        print("compute thread 64, cycles per 64-query iteration: [wait S^T/dP^T, load+barrier, element-wise, "
              "wait P^T/dS^T buffer, store+fence+barrier, wait dQ^T, drain+barrier+reduce] | iteration total")
        for i, d, tot in _rows(t, 0, picks, 8):
            print(f"  iter {i:3d}: {d} | {tot}")
        print("issuer of S^T and dP^T: [wait Q/dO, wait accumulators free, issue 16 MMAs] | loop total")
        for i, d, tot in _rows(t, 1, picks, 4):
            print(f"  iter {i:3d}: {d} | {tot}")
        print("issuer of dV, dK and dQ^T: [wait P^T/dS^T, wait dQ^T buffer free, issue 16 MMAs] | loop total")
        for i, d, tot in _rows(t, 2, picks, 4):
            print(f"  iter {i:3d}: {d} | {tot}")


if __name__ == "__main__":
    main()
