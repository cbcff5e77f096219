"""Device-timed micro-benchmarks of the hot kernels against their roofline denominators.

    python -m fsdp_comm_opt_b200.ops.bench_ops [--peaks MEASURED_PEAKS.json] [--only gemm,attn,codec,refcodec,recgemm,beside,elt]
        [--case SUBSTRING] [--gemm-backends tcgen05_2sm,tcgen05,cublas] [--iters N] [--warmup W]

``--case`` keeps the cases whose name contains the substring; with ``--iters 1 --warmup 1`` and one
backend the program launches a handful of kernels, which is the form to run under a profiler.

Every number: >= 3 warm-up launches, CUDA events on the launching stream around ``iters`` launches,
inputs larger than the 126 MB L2 or an L2 flush between launches (stated per line).  Fractions are
"of measured" peaks when the peaks file exists, else "of fallback" (6.65 TB/s, 1.59 PFLOP/s).
Prints one JSON object per line.
"""
from __future__ import annotations

import argparse
import json
import os

import torch

from . import attention, codec, gemm, loss, norm, swiglu
from .. import _lib


def _time(fn, iters=10, warmup=3, flush=None):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        if flush is not None:
            flush.add_(1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    return total / iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--peaks", default="MEASURED_PEAKS.json")
    ap.add_argument("--only", default="gemm,attn,codec,elt")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--case", default="", help="only cases whose name contains this")
    ap.add_argument("--gemm-backends", default="tcgen05_2sm,tcgen05,cublas")
    args = ap.parse_args()
    if os.path.exists(args.peaks):
        pk = json.load(open(args.peaks))
        hbm, tf, tag = pk["hbm_gbs"], pk["bf16_tflops"], "of measured"
    else:
        hbm, tf, tag = 6650.0, 1590.0, "of fallback"
    dev = torch.device("cuda")
    flush = torch.zeros(256 << 20, dtype=torch.uint8, device=dev)  # 256 MB > L2
    only = set(args.only.split(","))

    def emit(**kw):
        print(json.dumps(kw), flush=True)

    if "gemm" in only:
        shapes = [("fwd wgu", 4096, 28672, 4096, False, True), ("fwd wd", 4096, 4096, 14336, False, True),
                  ("fwd qkv", 4096, 6144, 4096, False, True), ("fwd wo", 4096, 4096, 4096, False, True),
                  ("dgrad wgu", 4096, 4096, 28672, False, False), ("dgrad wd", 4096, 14336, 4096, False, False),
                  ("wgrad wgu", 28672, 4096, 4096, True, False), ("wgrad wd", 4096, 14336, 4096, True, False),
                  ("lm_head", 4096, 128256, 4096, False, True), ("mid 4096x8192x4096", 4096, 8192, 4096, False, True),
                  ("square 8192", 8192, 8192, 8192, False, True)]
        backends = [b for b in args.gemm_backends.split(",") if b]
        for name, M, N, K, ta, tb in shapes:
            if args.case not in name:
                continue
            a = torch.randn((K, M) if ta else (M, K), device=dev).bfloat16()
            b = torch.randn((N, K) if tb else (K, N), device=dev).bfloat16()
            out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
            res = {}
            for be in backends:
                gemm.set_backend(be)
                ms = _time(lambda: gemm.gemm(a, b, ta, tb, out=out), args.iters, args.warmup, flush=flush)
                res["tflops_" + be] = round(2.0 * M * N * K / ms / 1e9, 1)
            gemm.set_backend("auto")
            status = int(_lib.cuda().zc_gemm_status_read_and_clear())
            ours = res.get("tflops_tcgen05_2sm", res.get("tflops_tcgen05"))
            emit(kernel="gemm_bf16", case=name, M=M, N=N, K=K, **res, status=status,
                 frac=round(ours / tf, 3) if ours else None, frac_of=tag, l2="flushed between launches")
    if "attn" in only:
        for B, S, Hq, Hkv, D in [(1, 4096, 32, 8, 128), (2, 4096, 40, 40, 128), (1, 8192, 32, 8, 128)]:
            if args.case not in f"B{B} S{S} H{Hq}/{Hkv}":
                continue
            qkv = (torch.randn(B, S, Hq + 2 * Hkv, D, device=dev) * 0.5).bfloat16().requires_grad_()
            o = attention.causal_attention(qkv, Hq, Hkv)
            g = torch.randn_like(o)
            fl = 4.0 * B * Hq * S * S * D / 2
            ms_f = _time(lambda: attention.causal_attention(qkv.detach(), Hq, Hkv), args.iters, args.warmup, flush=flush)
            ms_b = _time(lambda: torch.autograd.grad(attention.causal_attention(qkv, Hq, Hkv), qkv, g), args.iters,
                         args.warmup, flush=flush) - ms_f
            # the library attention the reference's model gets (PyTorch SDPA), forward and backward
            q, k, v = (t.transpose(1, 2).contiguous().requires_grad_() for t in
                       qkv.detach().split([Hq, Hkv, Hkv], dim=2))
            sdpa = lambda: torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
            with torch.no_grad():
                ms_sdpa = _time(sdpa, args.iters, args.warmup, flush=flush)
            go = torch.randn_like(sdpa())
            ms_sdpa_fb = _time(lambda: torch.autograd.grad(sdpa(), (q, k, v), go), args.iters, args.warmup, flush=flush)
            ms_sdpa_b = ms_sdpa_fb - ms_sdpa
            emit(kernel="attn", B=B, S=S, Hq=Hq, Hkv=Hkv, D=D, fwd_tflops=round(fl / ms_f / 1e9, 1),
                 bwd_tflops=round(2.5 * fl / max(ms_b, 1e-6) / 1e9, 1), sdpa_fwd_tflops=round(fl / ms_sdpa / 1e9, 1),
                 sdpa_bwd_tflops=round(2.5 * fl / max(ms_sdpa_b, 1e-6) / 1e9, 1),
                 ms=dict(fwd=round(ms_f, 4), bwd=round(ms_b, 4), sdpa_fwd=round(ms_sdpa, 4), sdpa_bwd=round(ms_sdpa_b, 4)),
                 frac_fwd=round(fl / ms_f / 1e9 / tf, 3), frac_of=tag, l2="flushed between launches")
    if "codec" in only:
        n = 1 << (27 if args.case == "2^27" else 28)  # 256 / 512 MB of bf16 > L2
        x = (torch.randn(n, device=dev) * 0.02).bfloat16()
        rec, hdr = codec.v2_encode(x)
        out = torch.empty_like(x)
        used = int(codec.v2_record_bytes(hdr).sum().item()) + 4 * hdr.numel()
        ms_e = _time(lambda: codec.v2_encode(x, rec, hdr), args.iters, args.warmup)
        ms_d = _time(lambda: codec.v2_decode(rec, hdr, n, out), args.iters, args.warmup)
        # the decoder with the CTA budget it has inside a fused collective (one 8-warp CTA per SM)
        lib = _lib.cuda()
        nsm = torch.cuda.get_device_properties(dev).multi_processor_count
        for ctas in (nsm, nsm // 2):
            ms_c = _time(lambda: lib.zc_v2_decode_ctas(rec.data_ptr(), hdr.data_ptr(), n, out.data_ptr(), ctas,
                                                       _lib.stream_ptr()), args.iters, args.warmup)
            emit(kernel="v2_decode_capped", ctas=ctas, elems=n, gbs=round((2 * n + used) / ms_c / 1e6, 1),
                 frac=round((2 * n + used) / ms_c / 1e6 / hbm, 3), frac_of=tag, gelems_per_s=round(n / ms_c / 1e6, 1))
        rec_n, hdr_n = codec.v2_encode(x, nibble=True)
        used_n = int(codec.v2_record_bytes(hdr_n).sum().item()) + 4 * hdr_n.numel()
        ms_en = _time(lambda: codec.v2_encode(x, rec_n, hdr_n, nibble=True), args.iters, args.warmup)
        ms_dn = _time(lambda: codec.v2_decode(rec_n, hdr_n, n, out, nibble=True), args.iters, args.warmup)
        emit(kernel="v2_encode_nibble", elems=n, gbs=round((2 * n + used_n) / ms_en / 1e6, 1),
             frac=round((2 * n + used_n) / ms_en / 1e6 / hbm, 3), frac_of=tag, bytes_per_elem=round(used_n / n, 4),
             gelems_per_s=round(n / ms_en / 1e6, 1), plane_mode_gelems_per_s=round(n / ms_e / 1e6, 1))
        emit(kernel="v2_decode_nibble", elems=n, gbs=round((2 * n + used_n) / ms_dn / 1e6, 1),
             frac=round((2 * n + used_n) / ms_dn / 1e6 / hbm, 3), frac_of=tag,
             gelems_per_s=round(n / ms_dn / 1e6, 1), plane_mode_gelems_per_s=round(n / ms_d / 1e6, 1))
        emit(kernel="v2_encode", elems=n, gbs=round((2 * n + used) / ms_e / 1e6, 1),
             frac=round((2 * n + used) / ms_e / 1e6 / hbm, 3), frac_of=tag, bytes_per_elem=round(used / n, 4),
             l2="input larger than L2")
        emit(kernel="v2_decode", elems=n, gbs=round((2 * n + used) / ms_d / 1e6, 1),
             frac=round((2 * n + used) / ms_d / 1e6 / hbm, 3), frac_of=tag, l2="input larger than L2")
        per = codec.pad_to_block(n)
        n_8 = torch.tensor([per], dtype=torch.int32, device=dev)
        bases = torch.full((256,), 116, dtype=torch.int32, device=dev)
        det = torch.empty(codec.v1_det_bytes(per), dtype=torch.uint8, device=dev)
        scr = torch.empty(per, dtype=torch.uint8, device=dev)
        esc = torch.empty(per, dtype=torch.uint8, device=dev)
        gc = torch.zeros(1, dtype=torch.int32, device=dev)
        ms_e1 = _time(lambda: codec.v1_compress_split_store(x, n_8, bases, det, scr, esc, gc, 1), args.iters)
        cnt = int(gc[0])
        ms_d1 = _time(lambda: codec.v1_decompress_split_store(det, esc, n_8, gc, out, 1), args.iters)
        b1 = det.numel() + cnt
        emit(kernel="v1_encode_split", elems=n, gbs=round((2 * n + b1 + 2 * cnt) / ms_e1 / 1e6, 1),
             frac=round((2 * n + b1 + 2 * cnt) / ms_e1 / 1e6 / hbm, 3), frac_of=tag, bytes_per_elem=round(b1 / n, 4))
        emit(kernel="v1_decode_split", elems=n, gbs=round((2 * n + b1) / ms_d1 / 1e6, 1),
             frac=round((2 * n + b1) / ms_d1 / 1e6 / hbm, 3), frac_of=tag)
    if "recgemm" in only:
        # decode fused with the consumer GEMM (weight given as v2 records) against decode, then GEMM
        from .gemm_records import RecordLinear, linear_t_plain
        M, N, K = 4096, 28672, 4096
        w = (torch.randn(N, K, device=dev) * 0.02).bfloat16()
        x = torch.randn(M, K, device=dev).bfloat16()
        rec, hdr = codec.v2_encode(w.view(-1))
        y = torch.empty(N, M, dtype=torch.bfloat16, device=dev)
        ms_g = _time(lambda: gemm.gemm(w, x, False, True, out=y), args.iters, args.warmup, flush=flush)
        wbuf = torch.empty_like(w)
        ms_d = _time(lambda: codec.v2_decode(rec, hdr, N * K, wbuf.view(-1)), args.iters, args.warmup, flush=flush)
        ms_p = _time(lambda: linear_t_plain(x, rec, hdr, N, K, w_buf=wbuf, out=y), args.iters, args.warmup, flush=flush)
        ref = y.clone()
        del w
        for slab_rows, ring in ((512, 3), (1024, 3), (2048, 3), (4096, 2)):
            rl = RecordLinear(N, K, dev, slab_rows=slab_rows, ring=ring)
            ms_f = _time(lambda: rl(x, rec, hdr, out=y), args.iters, args.warmup, flush=flush)
            emit(kernel="gemm_from_records", M=M, N=N, K=K, slab_rows=slab_rows, ring=ring,
                 ring_mb=round(ring * slab_rows * K * 2 / 2**20, 1), fused_ms=round(ms_f, 4),
                 decode_then_gemm_ms=round(ms_p, 4), gemm_alone_ms=round(ms_g, 4), decode_alone_ms=round(ms_d, 4),
                 fused_over_plain=round(ms_p / ms_f, 3),
                 max_abs_diff_vs_plain=float((y.float() - ref.float()).abs().max().item()),
                 l2="flushed between launches")
            del rl
    if "beside" in only:
        # What a GEMM loop pays for work that runs beside it on a high-priority side stream (the
        # position of the collectives during training): decode, encode, or a plain device copy of the
        # same kind of buffer.  hidden = (t_gemm + t_side - t_both) / min(t_gemm, t_side): 1 if the
        # side work is free, 0 if the two simply add up.
        M, N, K = 4096, 14336, 4096
        x = (torch.randn(M, K, device=dev) * 0.05).bfloat16()
        w = (torch.randn(N, K, device=dev) * 0.02).bfloat16()
        y = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
        n = 1 << 27
        src = (torch.randn(n, device=dev) * 0.02).bfloat16()
        rec, hdr = codec.v2_encode(src)
        out, out2 = torch.empty_like(src), torch.empty_like(src)
        lib = _lib.cuda()
        side = torch.cuda.Stream(priority=-1)
        main_s = torch.cuda.current_stream()
        nsm = torch.cuda.get_device_properties(dev).multi_processor_count

        def gemms():
            for _ in range(24):
                gemm.gemm(x, w, False, True, out=y)

        def both(main_fn, side_fn):
            t = None
            for _ in range(max(3, args.warmup)):
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                es = torch.cuda.Event()
                e0.record(main_s)
                side.wait_event(e0)
                if side_fn is not None:
                    with torch.cuda.stream(side):
                        side_fn()
                es.record(side)
                if main_fn is not None:
                    main_fn()
                main_s.wait_event(es)
                e1.record(main_s)
                torch.cuda.synchronize()
                t = e0.elapsed_time(e1)
            return t

        def rep(fn, r):
            def f():
                for _ in range(r):
                    fn()
            return f

        kinds = {
            "v2_decode, one CTA per SM": (lambda: lib.zc_v2_decode_ctas(rec.data_ptr(), hdr.data_ptr(), n, out.data_ptr(), nsm,
                                                                        _lib.stream_ptr()), n),
            "v2_decode, 64 CTAs": (lambda: lib.zc_v2_decode_ctas(rec.data_ptr(), hdr.data_ptr(), n, out.data_ptr(), 64,
                                                                 _lib.stream_ptr()), n),
            "v2_encode": (lambda: codec.v2_encode(src, rec, hdr), n),
            "device copy (bf16)": (lambda: out2.copy_(src), n),
        }
        t_g = both(gemms, None)
        for name, (fn, elems) in kinds.items():
            t1 = both(None, fn)
            r = max(1, int(round(0.8 * t_g / t1)))
            t_s = both(None, rep(fn, r))
            t_b = both(gemms, rep(fn, r))
            emit(kernel="gemm_beside", side=name, gemm_loop_ms=round(t_g, 3), side_alone_ms=round(t_s, 3),
                 together_ms=round(t_b, 3), hidden=round((t_g + t_s - t_b) / min(t_g, t_s), 3),
                 gemm_ms_paid_per_g_elem=round((t_b - t_g) / (r * elems / 1e9), 3) if t_b > t_g else 0.0,
                 side_g_elems=round(r * elems / 1e9, 2))
    if "refcodec" in only:
        # the reference's own kernels (built from its sources under baseline/_ref) on the same input,
        # beside this package's v1 and v2 kernels: encode = its K3 + K4 launches, decode = its K9
        import glob
        import importlib.util

        root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
        hits = glob.glob(os.path.join(root, "baseline", "_ref", "zipccl", "hopper_fastzip2*.so"))
        if not hits:
            emit(kernel="reference_codec", unavailable="baseline/_ref/zipccl/hopper_fastzip2*.so not found")
        else:
            spec = importlib.util.spec_from_file_location("hopper_fastzip2", hits[0])
            ref = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(ref)
            n = 1 << 27
            x = (torch.randn(n, device=dev) * 0.02).bfloat16()
            n_8 = torch.full((1,), n, dtype=torch.int32, device=dev)
            bases = torch.full((256,), 116, dtype=torch.int32, device=dev)
            det = torch.empty(codec.v1_det_bytes(n), dtype=torch.uint8, device=dev)
            scr = torch.empty(codec.align128(n), dtype=torch.uint8, device=dev)
            esc = torch.empty(codec.align128(n), dtype=torch.uint8, device=dev)
            gc = torch.zeros(1, dtype=torch.int32, device=dev)
            out = torch.empty_like(x)

            def enc(fn):
                gc.zero_()
                fn(x, n_8, bases, det, scr, esc, gc, 1)

            ms_re = _time(lambda: enc(ref.compress_split_store), args.iters, args.warmup)
            cnt = int(gc[0])
            stride = codec.align128(cnt)
            nbytes = torch.full((1,), stride, dtype=torch.int32, device=dev)
            escv = esc[:stride]
            ms_rd = _time(lambda: ref.decompress_split_store_unpad(det, escv, n_8, nbytes, out, n, 1), args.iters,
                          args.warmup)
            ok_ref = bool(torch.equal(out.view(torch.int16), x.view(torch.int16)))
            ms_oe = _time(lambda: enc(codec.v1_compress_split_store), args.iters, args.warmup)
            ms_od = _time(lambda: codec.v1_decompress_split_store_unpad(det, escv, n_8, nbytes, out, n, 1),
                          args.iters, args.warmup)
            ok_ours = bool(torch.equal(out.view(torch.int16), x.view(torch.int16)))
            rec, hdr = codec.v2_encode(x)
            ms_2e = _time(lambda: codec.v2_encode(x, rec, hdr), args.iters, args.warmup)
            ms_2d = _time(lambda: codec.v2_decode(rec, hdr, n, out), args.iters, args.warmup)
            b1 = det.numel() + cnt
            emit(kernel="codec_vs_reference", elems=n, ms_encode=dict(reference=round(ms_re, 4), v1=round(ms_oe, 4),
                                                                      v2=round(ms_2e, 4)),
                 ms_decode=dict(reference=round(ms_rd, 4), v1=round(ms_od, 4), v2=round(ms_2d, 4)),
                 gbs_encode=dict(reference=round((2 * n + b1 + 2 * cnt) / ms_re / 1e6, 1),
                                 v1=round((2 * n + b1 + 2 * cnt) / ms_oe / 1e6, 1)),
                 gbs_decode=dict(reference=round((2 * n + b1) / ms_rd / 1e6, 1), v1=round((2 * n + b1) / ms_od / 1e6, 1)),
                 roundtrip_exact=dict(reference=ok_ref, v1=ok_ours), l2="input larger than L2")
    if "elt" in only:
        T, d, F_, V = 16384, 4096, 14336, 128256
        x = torch.randn(T, d, device=dev).bfloat16()
        w = torch.ones(d, device=dev).bfloat16()
        ms = _time(lambda: norm.rms_norm(x, w, 1e-5), args.iters)
        emit(kernel="rmsnorm_fwd", rows=T, cols=d, gbs=round(4 * T * d / ms / 1e6, 1), frac=round(4 * T * d / ms / 1e6 / hbm, 3), frac_of=tag)
        gu = torch.randn(T, 2 * F_, device=dev).bfloat16()
        ms = _time(lambda: swiglu.swiglu(gu), args.iters)
        emit(kernel="swiglu_fwd", rows=T, F=F_, gbs=round(6 * T * F_ / ms / 1e6, 1), frac=round(6 * T * F_ / ms / 1e6 / hbm, 3), frac_of=tag)
        lg = torch.randn(4096, V, device=dev).bfloat16()
        lab = torch.randint(0, V, (4096,), device=dev)
        ms = _time(lambda: loss.cross_entropy(lg, lab), args.iters)
        emit(kernel="ce_fwd_bwd", rows=4096, V=V, gbs=round(4 * 4096 * V / ms / 1e6, 1), frac=round(4 * 4096 * V / ms / 1e6 / hbm, 3), frac_of=tag,
             note="algorithmic bytes: one read + one write of the logits")
        n = 1 << 28
        p = torch.randn(n, device=dev).bfloat16(); g = torch.randn(n, device=dev).bfloat16()
        m = torch.zeros_like(p); v = torch.zeros_like(p)
        lib = _lib.cuda()
        ms = _time(lambda: lib.zc_adamw(p.data_ptr(), g.data_ptr(), m.data_ptr(), v.data_ptr(), n, 0, 0, 0, 1e-4, 0.9, 0.999,
                                        1e-8, 0.01, 0.1, 0.001, 0, _lib.stream_ptr()), args.iters)
        emit(kernel="adamw_bf16", elems=n, gbs=round(14 * n / ms / 1e6, 1), frac=round(14 * n / ms / 1e6 / hbm, 3), frac_of=tag)


if __name__ == "__main__":
    main()
