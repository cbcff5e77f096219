"""Small single-kernel workloads for profiler captures.

    python -m fsdp_comm_opt_b200.ops.profile_case {gemm,gemm_wgrad,attn_fwd,attn_bwd,v2_encode,v2_decode,v1_encode,
                                                   rmsnorm,ce,adamw}

Each case launches its kernel a few times on inputs larger than the 126 MB L2 but well under a GB,
so a capture of one launch (``ncu -k regex:<kernel> -c 1``) ends by itself in seconds.
"""
from __future__ import annotations

import sys

import torch

from . import attention, codec, gemm, loss, norm
from .. import _lib


def main(case: str, reps: int = 3) -> None:
    dev = torch.device("cuda")
    torch.manual_seed(0)
    if case in ("gemm", "gemm_wgrad"):
        M, N, K = 4096, 8192, 4096          # A 32 MB + B 64 MB + C 64 MB
        gemm.set_backend("tcgen05")
        if case == "gemm":
            a = torch.randn(M, K, device=dev).bfloat16(); b = torch.randn(N, K, device=dev).bfloat16()
            fn = lambda: gemm.gemm(a, b, False, True)
        else:
            a = torch.randn(K, M, device=dev).bfloat16(); b = torch.randn(K, N, device=dev).bfloat16()
            fn = lambda: gemm.gemm(a, b, True, False)
    elif case in ("attn_fwd", "attn_bwd"):
        B, S, Hq, Hkv, D = 1, 4096, 32, 8, 128
        qkv = (torch.randn(B, S, Hq + 2 * Hkv, D, device=dev) * 0.5).bfloat16().requires_grad_()
        if case == "attn_fwd":
            fn = lambda: attention.causal_attention(qkv.detach(), Hq, Hkv)
        else:
            g = torch.randn(B, S, Hq, D, device=dev).bfloat16()
            fn = lambda: torch.autograd.grad(attention.causal_attention(qkv, Hq, Hkv), qkv, g)
    elif case in ("v2_encode", "v2_decode", "v1_encode"):
        n = 1 << 27                          # 256 MB of bf16
        x = (torch.randn(n, device=dev) * 0.02).bfloat16()
        rec, hdr = codec.v2_encode(x)
        out = torch.empty_like(x)
        if case == "v2_encode":
            fn = lambda: codec.v2_encode(x, rec, hdr)
        elif case == "v2_decode":
            fn = lambda: codec.v2_decode(rec, hdr, n, out)
        else:
            n_8 = torch.tensor([n], dtype=torch.int32, device=dev)
            bases = torch.full((256,), 116, dtype=torch.int32, device=dev)
            det = torch.empty(codec.v1_det_bytes(n), dtype=torch.uint8, device=dev)
            scr = torch.empty(n, dtype=torch.uint8, device=dev); esc = torch.empty(n, dtype=torch.uint8, device=dev)
            gc = torch.zeros(1, dtype=torch.int32, device=dev)
            fn = lambda: codec.v1_compress_split_store(x, n_8, bases, det, scr, esc, gc, 1)
    elif case == "rmsnorm":
        x = torch.randn(32768, 4096, device=dev).bfloat16(); w = torch.ones(4096, device=dev).bfloat16()
        fn = lambda: norm.rms_norm(x, w, 1e-5)
    elif case == "ce":
        lg = torch.randn(2048, 128256, device=dev).bfloat16(); lab = torch.randint(0, 128256, (2048,), device=dev)
        fn = lambda: loss.cross_entropy(lg, lab)
    elif case == "adamw":
        n = 1 << 27
        p = torch.randn(n, device=dev).bfloat16(); g = torch.randn(n, device=dev).bfloat16()
        m = torch.zeros_like(p); v = torch.zeros_like(p)
        lib = _lib.cuda()
        fn = lambda: lib.zc_adamw(p.data_ptr(), g.data_ptr(), m.data_ptr(), v.data_ptr(), n, 0, 0, 0, 1e-4, 0.9, 0.999,
                                  1e-8, 0.01, 0.1, 0.001, 0, _lib.stream_ptr())
    else:
        raise SystemExit(f"unknown case {case}")
    for _ in range(reps):
        fn()
    torch.cuda.synchronize()
    print(f"{case}: ok")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else "gemm")
