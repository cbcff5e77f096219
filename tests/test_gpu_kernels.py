"""GPU numerics: every CUDA kernel against a plain PyTorch fp32 reference (or, for the lossless
codec, against the scalar C++ codec byte for byte)."""
import math

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu

from fsdp_comm_opt_b200 import _lib
from fsdp_comm_opt_b200.ops import adamw, attention, codec, gpt2_ops, loss, norm, quant, rope, swiglu
from zipccl import hopper_fastzip2 as hz

DEV = "cuda"


def bits(t):
    return t.view(torch.int16)


def gauss(n, std=0.02, seed=0, device=DEV):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(n, generator=g) * std).to(torch.bfloat16).to(device)


def rand_bits(n, seed=0, device=DEV):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, 65536, (n,), generator=g, dtype=torch.int32).to(torch.int16).view(torch.bfloat16).to(device)


def test_native_library_is_loaded():
    assert _lib.cuda_lib_path().exists()
    assert _lib.cuda().zc_v2_encode is not None


# ------------------------------------------------------------------ codec
@pytest.mark.parametrize("n", [1, 1000, 1024, 4097, 1 << 20, (1 << 20) + 77])
@pytest.mark.parametrize("maker", [gauss, rand_bits])
def test_v2_gpu_matches_cpu_bytes_and_roundtrips(n, maker):
    x = maker(n, seed=3)
    rec, hdr = codec.v2_encode(x)
    rec_c, hdr_c = codec.v2_encode(x.cpu())
    assert torch.equal(hdr.cpu(), hdr_c)
    sizes = codec.v2_record_bytes(hdr_c)
    r = rec.cpu().view(-1, 2048)
    rc = rec_c.view(-1, 2048)
    mask = torch.arange(2048)[None, :] < sizes[:, None]
    assert torch.equal(r[mask], rc[mask])
    out = codec.v2_decode(rec, hdr, n)
    assert torch.equal(bits(out), bits(x))
    # GPU decodes CPU streams too
    out2 = codec.v2_decode(rec_c.to(DEV), hdr_c.to(DEV), n)
    assert torch.equal(bits(out2), bits(x))


@pytest.mark.parametrize("n", [1000, 4097, 1 << 20, (1 << 20) + 77])
@pytest.mark.parametrize("maker", [gauss, rand_bits])
def test_v2_nibble_mode_gpu_matches_cpu_bytes_and_roundtrips(n, maker):
    x = maker(n, seed=4)
    if maker is gauss:
        x[::700] = 2.0                                   # escapes below the window
    rec, hdr = codec.v2_encode(x, nibble=True)
    rec_c, hdr_c = codec.v2_encode(x.cpu(), nibble=True)
    assert torch.equal(hdr.cpu(), hdr_c)
    sizes = codec.v2_record_bytes(hdr_c)
    mask = torch.arange(2048)[None, :] < sizes[:, None]
    assert torch.equal(rec.cpu().view(-1, 2048)[mask], rec_c.view(-1, 2048)[mask])
    assert torch.equal(bits(codec.v2_decode(rec, hdr, n, nibble=True)), bits(x))
    assert torch.equal(bits(codec.v2_decode(rec_c.to(DEV), hdr_c.to(DEV), n, nibble=True)), bits(x))
    assert torch.equal(bits(codec.v2_decode(rec.cpu(), hdr.cpu(), n, nibble=True)), bits(x.cpu()))


def test_v2_unaligned_output_and_input():
    x = gauss(5000 + 3, seed=5)[3:]          # 6-byte offset: not 16-byte aligned
    rec, hdr = codec.v2_encode(x.contiguous() if False else x)
    buf = torch.zeros(5000 + 1, dtype=torch.bfloat16, device=DEV)
    out = codec.v2_decode(rec, hdr, 5000, buf[1:])
    assert torch.equal(bits(out), bits(x))


def _split_encode(x, base, n_works=1):
    n = x.numel()
    per = codec.pad_to_block((n + n_works - 1) // n_works)
    dev = x.device
    n_8 = torch.full((n_works,), per, dtype=torch.int32, device=dev)
    bases = torch.full((256,), base, dtype=torch.int32, device=dev)
    det = torch.zeros(n_works * codec.v1_det_bytes(per), dtype=torch.uint8, device=dev)
    scratch = torch.zeros(n_works * per, dtype=torch.uint8, device=dev)
    esc = torch.zeros(n_works * codec.align128(per), dtype=torch.uint8, device=dev)
    gc = torch.zeros(n_works, dtype=torch.int32, device=dev)
    hz.compress_split_store(x, n_8, bases, det, scratch, esc, gc, n_works)
    return n_8, det, esc, gc


@pytest.mark.parametrize("n,n_works", [(4096, 1), (10000, 1), (3 * 8192, 3), (1 << 20, 1), (8 * 12288, 8)])
@pytest.mark.parametrize("base", [116, 0, 252])
def test_v1_split_gpu_matches_cpu_bytes(n, n_works, base):
    x = torch.cat([gauss(n - 64, seed=n_works), rand_bits(64, seed=1)])
    n_8, det, esc, gc = _split_encode(x, base, n_works)
    n_8c, detc, escc, gcc = _split_encode(x.cpu(), base, n_works)
    assert torch.equal(gc.cpu(), gcc)
    assert torch.equal(det.cpu(), detc)
    off = 0
    for w in range(n_works):
        c = int(gcc[w])
        assert torch.equal(esc.cpu()[off:off + c], escc[off:off + c])
        off += codec.align128(c)
    per = int(n_8[0])
    out = torch.zeros(n_works * per, dtype=torch.bfloat16, device=DEV)
    hz.decompress_split_store(det, esc, n_8, gc, out, n_works)
    xp = torch.zeros(n_works * per, dtype=torch.bfloat16, device=DEV)
    xp[:n] = x
    assert torch.equal(bits(out), bits(xp))


def test_v1_gather_protocol_unpad_and_unpad_v():
    world, orig = 4, 5000 + 3
    per = codec.pad_to_block(orig)
    xs = [gauss(orig, seed=r) for r in range(world)]
    dets, escs, gcs = [], [], []
    for x in xs:
        _, det, esc, gc = _split_encode(x, 116)
        dets.append(det), escs.append(esc), gcs.append(int(gc[0]))
    stride = codec.align128(max(gcs))
    det_all = torch.cat(dets)
    esc_all = torch.cat([e[:stride] for e in escs])
    n_8 = torch.full((world,), per, dtype=torch.int32, device=DEV)
    nbytes = torch.full((world,), stride, dtype=torch.int32, device=DEV)
    out = torch.zeros(world * orig, dtype=torch.bfloat16, device=DEV)
    hz.decompress_split_store_unpad(det_all, esc_all, n_8, nbytes, out, orig, world)   # odd offsets: scalar stores
    assert torch.equal(bits(out), bits(torch.cat(xs)))
    out_off = torch.tensor([(world - 1 - r) * orig for r in range(world)], dtype=torch.int32, device=DEV)
    orig_n = torch.full((world,), orig, dtype=torch.int32, device=DEV)
    out2 = torch.zeros(world * orig, dtype=torch.bfloat16, device=DEV)
    hz.decompress_split_store_unpad_v(det_all, esc_all, n_8, nbytes, out_off, orig_n, out2, world * per, world)
    assert torch.equal(bits(out2), bits(torch.cat(xs[::-1])))


def test_v1_pad_variant_and_fused_layout():
    origs = [100, 4096, 7168, 1]
    xs = [rand_bits(o, seed=i) for i, o in enumerate(origs)]
    dense = torch.cat(xs)
    n_8 = torch.tensor([codec.pad_to_block(o) for o in origs], dtype=torch.int32, device=DEV)
    orig_n = torch.tensor(origs, dtype=torch.int32, device=DEV)
    total_pad = int(n_8.sum())
    bases = torch.full((256,), 120, dtype=torch.int32, device=DEV)
    det = torch.zeros(sum(codec.v1_det_bytes(int(p)) for p in n_8), dtype=torch.uint8, device=DEV)
    scratch = torch.zeros(total_pad, dtype=torch.uint8, device=DEV)
    esc = torch.zeros(total_pad + 128 * 4, dtype=torch.uint8, device=DEV)
    gc = torch.zeros(4, dtype=torch.int32, device=DEV)
    hz.compress_split_store_pad(dense, n_8, orig_n, bases, det, scratch, esc, gc, total_pad, 4)
    detc = torch.zeros_like(det, device="cpu"); escc = torch.zeros_like(esc, device="cpu"); gcc = torch.zeros(4, dtype=torch.int32)
    hz.compress_split_store_pad(dense.cpu(), n_8.cpu(), orig_n.cpu(), bases.cpu(), detc, scratch.cpu(), escc, gcc, total_pad, 4)
    assert torch.equal(det.cpu(), detc) and torch.equal(gc.cpu(), gcc)
    # fused layout, 3 works, GPU encode -> CPU decode and GPU decode
    per = 8192
    x = torch.cat([gauss(per, std=10.0 ** (-w), seed=w) for w in range(3)])
    n8 = torch.full((3,), per, dtype=torch.int32, device=DEV)
    nbytes = torch.zeros(3, dtype=torch.int32, device=DEV)
    sc = torch.zeros(4 * x.numel(), dtype=torch.uint8, device=DEV)
    fin = torch.zeros(4 * x.numel(), dtype=torch.uint8, device=DEV)
    g3 = torch.zeros(3, dtype=torch.int32, device=DEV)
    hz.compress_8(x, n8, nbytes, bases, sc, fin, g3, 3)
    out = torch.zeros_like(x)
    hz.decompress_8(fin, n8, nbytes, out, 3)
    assert torch.equal(bits(out), bits(x))
    outc = torch.zeros_like(x, device="cpu")
    hz.decompress_8(fin.cpu(), n8.cpu(), nbytes.cpu(), outc, 3)
    assert torch.equal(bits(outc), bits(x.cpu()))
    buf = hz.compress_8_padded(x[:9999], bases, 1)
    back = hz.decompress_8_padded(buf, 9999, torch.zeros(1, dtype=torch.int32, device=DEV), 1)
    assert torch.equal(bits(back), bits(x[:9999]))
    out2 = torch.zeros(3 * 5000, dtype=torch.bfloat16, device=DEV)
    hz.decompress_8_unpad(fin, n8, nbytes, out2, 5000, 3)
    for w in range(3):
        assert torch.equal(bits(out2[w * 5000:(w + 1) * 5000]), bits(x[w * per:w * per + 5000]))


def test_v1_base_statistic_kernel():
    x = gauss(1 << 20, 0.02, seed=1)
    bases = torch.zeros(256, dtype=torch.int32, device=DEV)
    codec.v1_base_from_std(x, bases)
    codec.v1_base_from_std(x * 0 + x, bases)   # second call reuses the zeroed accumulator
    assert int(bases[0]) == 116


# ------------------------------------------------------------------ elementwise
def test_rmsnorm_fwd_bwd():
    torch.manual_seed(0)
    for rows, cols in [(64, 4096), (33, 256), (8, 8192)]:
        x = torch.randn(rows, cols, device=DEV).bfloat16().requires_grad_()
        r = torch.randn(rows, cols, device=DEV).bfloat16().requires_grad_()
        w = (1 + 0.1 * torch.randn(cols, device=DEV)).bfloat16().requires_grad_()
        y, h = norm.add_rms_norm(x, r, w, 1e-5)
        g = torch.randn_like(y)
        (y.float() * g.float()).sum().backward()
        xf, rf, wf = (t.detach().float().requires_grad_() for t in (x, r, w))
        hf = (xf + rf).bfloat16().float()
        yf = F.rms_norm(xf + rf, (cols,), wf, 1e-5)
        (yf * g.float()).sum().backward()
        assert torch.equal(h.float(), hf)
        assert torch.allclose(y.float(), yf, atol=2e-2, rtol=2e-2)
        assert torch.allclose(x.grad.float(), xf.grad, atol=3e-2, rtol=3e-2)
        assert torch.allclose(w.grad.float(), wf.grad, atol=0.15, rtol=3e-2)
        y2 = norm.rms_norm(x.detach(), w.detach(), 1e-5)
        assert torch.allclose(y2.float(), F.rms_norm(x.detach().float(), (cols,), w.detach().float(), 1e-5), atol=2e-2, rtol=2e-2)


def test_swiglu_fwd_bwd():
    torch.manual_seed(1)
    gu = torch.randn(257, 2 * 1024, device=DEV).bfloat16().requires_grad_()
    out = swiglu.swiglu(gu)
    g = torch.randn_like(out)
    out.backward(g)
    gf = gu.detach().float().requires_grad_()
    ref = F.silu(gf[:, :1024]) * gf[:, 1024:]
    ref.backward(g.float())
    assert torch.allclose(out.float(), ref, atol=2e-2, rtol=2e-2)
    assert torch.allclose(gu.grad.float(), gf.grad, atol=3e-2, rtol=3e-2)


def test_rope_matches_cpu_path():
    torch.manual_seed(2)
    S, Hq, Hkv, D = 96, 4, 2, 128
    cos, sin = rope.rope_tables(S, D, 500000.0, DEV)
    x = torch.randn(2 * S, (Hq + 2 * Hkv) * D, device=DEV).bfloat16()
    ref = rope._rotate(x.cpu().float(), cos.cpu(), sin.cpu(), Hq + Hkv, D, S, 1.0)
    got = rope._rotate(x.clone(), cos, sin, Hq + Hkv, D, S, 1.0)
    assert torch.allclose(got.float().cpu(), ref, atol=2e-2, rtol=2e-2)
    back = rope._rotate(got.clone(), cos, sin, Hq + Hkv, D, S, -1.0)
    assert torch.allclose(back.float(), x.float(), atol=5e-2, rtol=5e-2)
    assert torch.equal(got[:, (Hq + Hkv) * D:], x[:, (Hq + Hkv) * D:])   # v heads untouched


@pytest.mark.parametrize("V", [8192, 50257, 128256])
def test_cross_entropy_fwd_bwd(V):
    torch.manual_seed(3)
    T = 64
    logits = (torch.randn(T, V, device=DEV) * 2).bfloat16()
    labels = torch.randint(0, V, (T,), device=DEV)
    labels[5] = -100
    lf = logits.float().requires_grad_()
    ref = F.cross_entropy(lf, labels, ignore_index=-100)
    ref.backward()
    work = logits.clone().requires_grad_()
    out = loss.cross_entropy(work * 1, labels)
    out.backward()
    assert abs(out.item() - ref.item()) < 2e-3
    assert torch.allclose(work.grad.float(), lf.grad, atol=2e-4, rtol=2e-2)


def test_int8_quant_kernels():
    torch.manual_seed(4)
    n, world = 100003, 3
    buf = torch.zeros(world, quant.packed_bytes(n), dtype=torch.uint8, device=DEV)
    xs = [(torch.randn(n, device=DEV) * 0.01 * (r + 1)).bfloat16() for r in range(world)]
    for r in range(world):
        quant.quantize_pack(xs[r], buf[r])
    out = torch.zeros(world * n, dtype=torch.bfloat16, device=DEV)
    quant.dequantize_unpack(buf, n, out)
    for r in range(world):
        scale = xs[r].float().abs().max() / 127
        assert torch.allclose(buf[r, :4].view(torch.float32), scale.reshape(1))
        assert (out[r * n:(r + 1) * n].float() - xs[r].float()).abs().max() <= scale * 1.01


@pytest.mark.parametrize("pdt,sdt", [(torch.bfloat16, torch.bfloat16), (torch.float32, torch.float32)])
def test_fused_adamw_kernel(pdt, sdt):
    torch.manual_seed(5)
    p0 = torch.randn(100003, device=DEV)
    p1 = torch.nn.Parameter(p0.to(pdt))
    p2 = torch.nn.Parameter(p0.to(pdt).float())
    o1 = adamw.FusedAdamW([p1], lr=1e-2, weight_decay=0.1)
    o2 = torch.optim.AdamW([p2], lr=1e-2, weight_decay=0.1)
    for _ in range(4):
        g = torch.randn(100003, device=DEV).to(pdt)
        p1.grad, p2.grad = g.clone(), g.float()
        o1.step(), o2.step()
    tol = 3e-2 if pdt == torch.bfloat16 else 1e-5
    assert torch.allclose(p1.float(), p2, atol=tol, rtol=tol)
    assert o1.kernel_launches == 4


# ------------------------------------------------------------------ tensor cores
@pytest.mark.parametrize("a_major,b_major", [(0, 0), (0, 1), (1, 0), (1, 1)])
def test_umma_descriptor_conventions(a_major, b_major):
    torch.manual_seed(6)
    ksteps = 3
    K = 64 * ksteps
    A = torch.randn(128, K, device=DEV).bfloat16()
    B = torch.randn(128, K, device=DEV).bfloat16()
    Ag = A if a_major == 0 else A.t().contiguous()
    Bg = B if b_major == 0 else B.t().contiguous()
    D = torch.zeros(128, 128, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    rc = _lib.cuda().zc_umma_selftest(Ag.data_ptr(), Bg.data_ptr(), D.data_ptr(), a_major, b_major, ksteps,
                                      status.data_ptr(), _lib.stream_ptr())
    assert rc == 0
    torch.cuda.synchronize()
    assert int(status[0]) == 0, "bounded wait expired"
    ref = A.float() @ B.float().t()
    assert torch.allclose(D, ref, atol=1e-2, rtol=1e-3), (D - ref).abs().max().item()


def _attn_ref(qkv, Hq, Hkv):
    q, k, v = qkv[:, :, :Hq], qkv[:, :, Hq:Hq + Hkv], qkv[:, :, Hq + Hkv:]
    g = Hq // Hkv
    q, k, v = (t.transpose(1, 2).float() for t in (q, k, v))
    k, v = k.repeat_interleave(g, 1), v.repeat_interleave(g, 1)
    return F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2)


@pytest.mark.parametrize("impl", ["2q+kt", "ws+ws", "simple+simple"])
@pytest.mark.parametrize("B,S,Hq,Hkv,D", [(1, 128, 1, 1, 128), (2, 384, 4, 2, 128), (1, 200, 2, 2, 64), (1, 512, 8, 2, 128),
                                          (1, 1000, 4, 1, 128), (2, 2048, 8, 2, 128)])
def test_attention_fwd_bwd(B, S, Hq, Hkv, D, impl, monkeypatch):
    fwd_impl, bwd_impl = impl.split("+")
    monkeypatch.setattr(attention, "_FWD_IMPL", fwd_impl)
    monkeypatch.setattr(attention, "_BWD_IMPL", bwd_impl)
    torch.manual_seed(7)
    qkv = (torch.randn(B, S, Hq + 2 * Hkv, D, device=DEV) * 0.5).bfloat16().requires_grad_()
    o = attention.causal_attention(qkv * 1, Hq, Hkv)
    g = (torch.randn_like(o) * 0.5)
    o.backward(g)
    torch.cuda.synchronize()
    assert attention.status_read_and_clear() == 0
    qf = qkv.detach().float().requires_grad_()
    ref = _attn_ref(qf, Hq, Hkv)
    ref.backward(g.float())
    assert torch.allclose(o.float(), ref, atol=2e-2, rtol=2e-2), (o.float() - ref).abs().max().item()
    err = (qkv.grad.float() - qf.grad).abs().max().item()
    assert torch.allclose(qkv.grad.float(), qf.grad, atol=3e-2, rtol=3e-2), err


@pytest.mark.parametrize("impl", ["2q+kt", "ws+ws"])
def test_attention_rising_scores_rescale_the_accumulator(impl, monkeypatch):
    """Keys whose scores grow along the sequence raise the running row maximum again and again, so
    the forward kernel must rescale the output it has accumulated so far (the two-tile kernel does
    that in TMEM, and only when the maximum rose by more than a factor of 2^8)."""
    fwd_impl, bwd_impl = impl.split("+")
    monkeypatch.setattr(attention, "_FWD_IMPL", fwd_impl)
    monkeypatch.setattr(attention, "_BWD_IMPL", bwd_impl)
    torch.manual_seed(11)
    B, S, Hq, Hkv, D = 1, 1024, 2, 1, 128
    qkv = torch.randn(B, S, Hq + 2 * Hkv, D, device=DEV) * 0.5
    # q = +1 everywhere, k ramps from -3 to +3: scores rise by ~70 (in log2 units ~100) over the row
    qkv[:, :, :Hq] = 1.0 + 0.05 * torch.randn(B, S, Hq, D, device=DEV)
    ramp = torch.linspace(-3.0, 3.0, S, device=DEV)[None, :, None, None]
    qkv[:, :, Hq:Hq + Hkv] = ramp + 0.05 * torch.randn(B, S, Hkv, D, device=DEV)
    qkv = qkv.bfloat16().requires_grad_()
    o = attention.causal_attention(qkv * 1, Hq, Hkv)
    g = torch.randn_like(o) * 0.5
    o.backward(g)
    torch.cuda.synchronize()
    assert attention.status_read_and_clear() == 0
    qf = qkv.detach().float().requires_grad_()
    ref = _attn_ref(qf, Hq, Hkv)
    ref.backward(g.float())
    assert torch.allclose(o.float(), ref, atol=3e-2, rtol=3e-2), (o.float() - ref).abs().max().item()
    assert torch.allclose(qkv.grad.float(), qf.grad, atol=5e-2, rtol=5e-2), (qkv.grad.float() - qf.grad).abs().max().item()


def test_attention_with_fused_rope_matches_unfused():
    torch.manual_seed(8)
    B, S, Hq, Hkv, D = 1, 256, 4, 2, 128
    cos, sin = rope.rope_tables(S, D, 10000.0, DEV)
    qkv = (torch.randn(B, S, Hq + 2 * Hkv, D, device=DEV) * 0.5).bfloat16().requires_grad_()
    o = attention.causal_attention((qkv * 1).contiguous(), Hq, Hkv, None, cos, sin)
    g = torch.randn_like(o) * 0.5
    o.backward(g)
    qf = qkv.detach().float().requires_grad_()
    half = D // 2
    rot = qf[:, :, :Hq + Hkv]
    c, s = cos[None, :, None, :], sin[None, :, None, :]
    a, b = rot[..., :half], rot[..., half:]
    rotated = torch.cat([torch.cat([a * c - b * s, b * c + a * s], -1), qf[:, :, Hq + Hkv:]], 2)
    ref = _attn_ref(rotated, Hq, Hkv)
    ref.backward(g.float())
    assert torch.allclose(o.float(), ref, atol=3e-2, rtol=3e-2)
    assert torch.allclose(qkv.grad.float(), qf.grad, atol=4e-2, rtol=4e-2)


# ------------------------------------------------------------------ GPT-2 family ops
@pytest.mark.parametrize("rows,cols", [(64, 1600), (300, 256), (17, 4096), (8, 8192)])
def test_layernorm_fwd_bwd(rows, cols):
    torch.manual_seed(21)
    x = (torch.randn(rows, cols, device=DEV) * 2 + 0.5).bfloat16().requires_grad_()
    w = (1 + 0.1 * torch.randn(cols, device=DEV)).bfloat16().requires_grad_()
    b = (0.1 * torch.randn(cols, device=DEV)).bfloat16().requires_grad_()
    y = gpt2_ops.layer_norm(x, w, b, 1e-5)
    g = torch.randn_like(y)
    y.backward(g)
    xf, wf, bf = (t.detach().float().requires_grad_() for t in (x, w, b))
    ref = F.layer_norm(xf, (cols,), wf, bf, 1e-5)
    ref.backward(g.float())
    assert torch.allclose(y.float(), ref, atol=3e-2, rtol=2e-2)
    assert torch.allclose(x.grad.float(), xf.grad, atol=3e-2, rtol=3e-2), (x.grad.float() - xf.grad).abs().max().item()
    assert torch.allclose(w.grad.float(), wf.grad, atol=0.02 * rows ** 0.5 + 0.05, rtol=3e-2)
    assert torch.allclose(b.grad.float(), bf.grad, atol=0.02 * rows ** 0.5 + 0.05, rtol=3e-2)


@pytest.mark.parametrize("rows,cols", [(128, 6400), (33, 1024)])
def test_bias_gelu_fwd_bwd(rows, cols):
    torch.manual_seed(22)
    x = (torch.randn(rows, cols, device=DEV) * 1.5).bfloat16().requires_grad_()
    b = (0.2 * torch.randn(cols, device=DEV)).bfloat16().requires_grad_()
    y = gpt2_ops.bias_gelu(x, b)
    g = torch.randn_like(y)
    y.backward(g)
    xf, bf = (t.detach().float().requires_grad_() for t in (x, b))
    ref = F.gelu(xf + bf, approximate="tanh")
    ref.backward(g.float())
    assert torch.allclose(y.float(), ref, atol=2e-2, rtol=2e-2)
    assert torch.allclose(x.grad.float(), xf.grad, atol=2e-2, rtol=2e-2)
    assert torch.allclose(b.grad.float(), bf.grad, atol=0.02 * rows ** 0.5 + 0.05, rtol=3e-2)


@pytest.mark.parametrize("rows,cols,main_grad", [(64, 1600, None), (300, 256, torch.bfloat16), (2048, 1600, torch.float32)])
def test_add_layernorm_and_direct_gradient_delivery(rows, cols, main_grad):
    """LayerNorm fused with the residual add in front of it, the gradient arriving through the sum added
    inside the backward kernel, and dw / db written (or accumulated) straight into ``main_grad``."""
    torch.manual_seed(23)
    x = (torch.randn(rows, cols, device=DEV) * 2).bfloat16().requires_grad_()
    r = (torch.randn(rows, cols, device=DEV)).bfloat16().requires_grad_()
    w = (1 + 0.1 * torch.randn(cols, device=DEV)).bfloat16().requires_grad_()
    b = (0.1 * torch.randn(cols, device=DEV)).bfloat16().requires_grad_()
    if main_grad is not None:
        for p_ in (w, b):
            p_.main_grad = torch.full((cols,), 0.5, dtype=main_grad, device=DEV)
            p_.main_grad_written = True            # accumulate on top of the 0.5
    y, h = gpt2_ops.add_layer_norm(x, r, w, b, 1e-5)
    g, gh = torch.randn_like(y), torch.randn_like(h)
    torch.autograd.backward([y, h], [g, gh])
    xf, rf, wf, bf = (t.detach().float().requires_grad_() for t in (x, r, w, b))
    hf = (xf + rf)
    hq = hf.bfloat16().float()                     # the kernel normalises the stored (rounded) sum
    ref = F.layer_norm(hf + (hq - hf).detach(), (cols,), wf, bf, 1e-5)
    torch.autograd.backward([ref, hf], [g.float(), gh.float()])
    assert torch.equal(h.float(), hq)
    assert torch.allclose(y.float(), ref, atol=3e-2, rtol=2e-2)
    assert torch.allclose(x.grad.float(), xf.grad, atol=4e-2, rtol=3e-2)
    assert torch.equal(x.grad, r.grad)
    tol = dict(atol=0.02 * rows ** 0.5 + 0.05, rtol=3e-2)
    if main_grad is None:
        assert torch.allclose(w.grad.float(), wf.grad, **tol) and torch.allclose(b.grad.float(), bf.grad, **tol)
    else:
        assert w.grad is None and b.grad is None
        assert torch.allclose(w.main_grad.float() - 0.5, wf.grad, **tol)
        assert torch.allclose(b.main_grad.float() - 0.5, bf.grad, **tol)


@pytest.mark.parametrize("T,K,N", [(2048, 1600, 4800), (300, 256, 1000)])
def test_linear_with_bias_in_the_gemm_epilogue(T, K, N):
    from fsdp_comm_opt_b200.ops import gemm

    torch.manual_seed(24)
    x = (torch.randn(T, K, device=DEV) * 0.5).bfloat16().requires_grad_()
    w = (torch.randn(N, K, device=DEV) * 0.05).bfloat16().requires_grad_()
    b = torch.randn(N, device=DEV).bfloat16().requires_grad_()
    b.main_grad = torch.zeros(N, dtype=torch.bfloat16, device=DEV)
    b.main_grad_written = False
    g = torch.randn(T, N, device=DEV).bfloat16()
    before = _lib.launch_count()
    y = gemm.linear(x, w, b)
    y.backward(g)
    torch.cuda.synchronize()
    assert _lib.launch_count() - before >= 4          # three GEMMs and the column-sum kernel pair
    xf, wf, bf = (t.detach().float().requires_grad_() for t in (x, w, b))
    ref = xf @ wf.t() + bf
    ref.backward(g.float())
    assert torch.allclose(y.float(), ref, atol=2e-2 * float(ref.abs().max()), rtol=2e-2)
    assert b.grad is None and b.main_grad_written
    assert torch.allclose(b.main_grad.float(), bf.grad, atol=0.02 * T ** 0.5 + 0.1, rtol=3e-2)
    assert torch.allclose(x.grad.float(), xf.grad, atol=2e-2 * float(xf.grad.abs().max()), rtol=3e-2)
    assert torch.allclose(w.grad.float(), wf.grad, atol=2e-2 * float(wf.grad.abs().max()), rtol=3e-2)


# ------------------------------------------------------------------ GEMM
@pytest.mark.parametrize("backend,M,N,K", [
    ("tcgen05", 128, 128, 128), ("tcgen05", 256, 512, 384), ("tcgen05", 4096, 1536, 1024), ("tcgen05", 384, 256, 4096),
    ("tcgen05", 128, 384, 128), ("tcgen05", 4096, 4096, 14336),
    # the two-SM kernel (the default backend): whole tiles, a split-K tail (4096 x 6144: 384 tiles on 74
    # clusters), and edge tiles in M, N and K
    ("tcgen05_2sm", 256, 256, 128), ("tcgen05_2sm", 512, 768, 256), ("tcgen05_2sm", 4096, 6144, 1024),
    ("tcgen05_2sm", 4096, 4096, 14336), ("tcgen05_2sm", 384, 640, 192), ("tcgen05_2sm", 2048, 1600, 1608),
    ("tcgen05_2sm", 136, 128, 136)])
def test_tcgen05_gemm_three_forms(backend, M, N, K):
    from fsdp_comm_opt_b200.ops import gemm

    torch.manual_seed(9)
    gemm.set_backend(backend)
    try:
        x = (torch.randn(M, K, device=DEV) * 0.5).bfloat16()
        w = (torch.randn(N, K, device=DEV) * 0.5).bfloat16()
        dy = (torch.randn(M, N, device=DEV) * 0.5).bfloat16()
        before = _lib.launch_count()
        y = gemm.gemm(x, w, False, True)            # forward
        dx = gemm.gemm(dy, w, False, False)         # dgrad:  [M,N] @ [N,K]
        dw = gemm.gemm(dy, x, True, False)          # wgrad:  [M,N]^T @ [M,K]  (needs N % 128 == 0 as "M")
        assert _lib.launch_count() - before == 3, "the hand-written kernel must have been taken"
        torch.cuda.synchronize()
        assert _lib.cuda().zc_gemm_status_read_and_clear() == 0
        for got, ref in ((y, x.float() @ w.float().t()), (dx, dy.float() @ w.float()), (dw, dy.float().t() @ x.float())):
            tol = 2e-2 * ref.abs().max().item()
            assert (got.float() - ref).abs().max().item() <= tol, (got.float() - ref).abs().max().item()
        acc = y.clone()
        gemm.gemm(x, w, False, True, out=acc, accumulate=True)
        assert torch.allclose(acc.float(), 2 * y.float(), atol=0.1, rtol=2e-2)
    finally:
        gemm.set_backend("auto")


def test_gemm_with_leading_dimensions_and_odd_sizes():
    """Operands and results that are slices of wider buffers, and M / N / K that are not multiples of 8
    (GPT-2's vocabulary): the two-SM kernel takes row strides, zero-fills what lies outside a slice and
    hands back a [:, :N] view of aligned rows whose padding columns are zero."""
    from fsdp_comm_opt_b200.ops import gemm

    torch.manual_seed(11)
    M, N, K = 300, 1001, 520
    xb = (torch.randn(M, K + 8, device=DEV) * 0.5).bfloat16()
    x = xb[:, :K - 5]                                # K = 515, rows 528 elements apart
    Ke = K - 5
    w = (torch.randn(N, K, device=DEV) * 0.5).bfloat16()[:, :Ke]
    before = _lib.launch_count()
    y = gemm.gemm(x, w, False, True)                 # [300, 1001] view of [300, 1008]
    assert y.shape == (M, N) and y.stride(0) == 1008
    dx = gemm.gemm(y, w, False, False)               # dgrad form: K = 1001, A strided, B rows = K
    dw = gemm.gemm(y, x, True, False)                # wgrad form: M = 1001 rows out, both operands strided
    assert _lib.launch_count() - before == 3, "the hand-written kernel must have been taken"
    torch.cuda.synchronize()
    assert _lib.cuda().zc_gemm_status_read_and_clear() == 0
    yf = y.float()
    for got, ref in ((y, x.float() @ w.float().t()), (dx, yf @ w.float()), (dw, yf.t() @ x.float())):
        assert got.shape == ref.shape
        tol = 2e-2 * ref.abs().max().item()
        assert (got.float() - ref).abs().max().item() <= tol, (got.float() - ref).abs().max().item()
    pad = torch.as_strided(y, (M, 1008 - N), (1008, 1), y.storage_offset() + N)
    assert int(pad.float().abs().max().item()) == 0
    # a column block of a wider result, accumulated into
    big = torch.zeros(M, 2048, dtype=torch.bfloat16, device=DEV)
    gemm.gemm(x, w, False, True, out=big[:, 1024:1024 + N])
    gemm.gemm(x, w, False, True, out=big[:, 1024:1024 + N], accumulate=True)
    torch.cuda.synchronize()
    assert torch.allclose(big[:, 1024:1024 + N].float(), 2 * yf, atol=0.1, rtol=2e-2)
    assert float(big[:, :1024].float().abs().max()) == 0.0


def test_linear_and_loss_over_a_vocabulary_that_is_not_a_multiple_of_8():
    """lm_head + cross-entropy at an odd vocabulary run on the hand-written GEMM and the strided loss
    kernel; gradients against fp32 PyTorch."""
    from fsdp_comm_opt_b200.ops import gemm

    torch.manual_seed(12)
    T, D, V = 256, 192, 1001
    x = (torch.randn(T, D, device=DEV) * 0.5).bfloat16().requires_grad_()
    w = (torch.randn(V, D, device=DEV) * 0.1).bfloat16().requires_grad_()
    labels = torch.randint(0, V, (T,), device=DEV)
    labels[7] = -100
    before = _lib.launch_count()
    out = loss.cross_entropy(gemm.linear(x, w), labels)
    out.backward()
    torch.cuda.synchronize()
    assert _lib.launch_count() - before >= 4        # three GEMMs and the loss kernel
    xf, wf = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    ref = F.cross_entropy((xf @ wf.t()).bfloat16().float(), labels, ignore_index=-100)
    ref2 = F.cross_entropy(xf @ wf.t(), labels, ignore_index=-100)
    ref2.backward()
    assert abs(out.item() - ref.item()) < 5e-3
    assert torch.allclose(x.grad.float(), xf.grad, atol=2e-2 * float(xf.grad.abs().max()), rtol=5e-2)
    assert torch.allclose(w.grad.float(), wf.grad, atol=2e-2 * float(wf.grad.abs().max()), rtol=5e-2)


def test_linear_autograd_on_tcgen05_matches_cublas():
    from fsdp_comm_opt_b200.ops import gemm

    torch.manual_seed(10)
    x = (torch.randn(2, 256, 512, device=DEV) * 0.5).bfloat16().requires_grad_()
    w = (torch.randn(768, 512, device=DEV) * 0.05).bfloat16().requires_grad_()
    g = torch.randn(2, 256, 768, device=DEV).bfloat16()
    gemm.set_backend("tcgen05")
    gemm.linear(x, w).backward(g)
    gx, gw = x.grad.clone(), w.grad.clone()
    x.grad = w.grad = None
    gemm.set_backend("cublas")
    gemm.linear(x, w).backward(g)
    gemm.set_backend("auto")
    assert torch.allclose(gx.float(), x.grad.float(), atol=3e-2, rtol=3e-2)
    assert torch.allclose(gw.float(), w.grad.float(), atol=0.3, rtol=3e-2)


# ------------------------------------------------------------------ whole models on the GPU
@pytest.mark.parametrize("shape", ["tiny", "gpt2-tiny"])
def test_model_forward_backward_matches_cpu(shape):
    """One forward + backward of a tiny model of each family on the GPU kernels against the same
    weights and tokens on the CPU reference paths of the ops."""
    from fsdp_comm_opt_b200.models import build_model, get_config

    cfg = get_config(shape)
    torch.manual_seed(3)
    ref = build_model(cfg).to(torch.bfloat16)
    ref.init_weights()
    gpu = build_model(cfg).to(torch.bfloat16)
    gpu.load_state_dict(ref.state_dict())
    gpu = gpu.to(DEV)
    ids = torch.randint(0, cfg.vocab_size, (2, 128))
    out_r = ref(input_ids=ids, labels=ids)
    out_r.loss.backward()
    out_g = gpu(input_ids=ids.to(DEV), labels=ids.to(DEV))
    out_g.loss.backward()
    torch.cuda.synchronize()
    assert abs(out_g.loss.item() - out_r.loss.item()) < 5e-2, (out_g.loss.item(), out_r.loss.item())
    checked = 0
    for (n, pr), (_, pg) in zip(ref.named_parameters(), gpu.named_parameters()):
        assert pg.grad is not None, n
        gr, gg = pr.grad.float(), pg.grad.float().cpu()
        assert torch.isfinite(gg).all(), n
        denom = gr.abs().max().item() + 1e-6
        assert (gg - gr).abs().max().item() / denom < 0.15, (n, (gg - gr).abs().max().item(), denom)
        checked += 1
    assert checked > 5


def test_device_status_check_is_clean_after_kernels():
    """The host-side health check reads every kernel family's status word; after normal launches it
    must find nothing (a wait that ran out would raise here instead of hanging the GPU)."""
    from fsdp_comm_opt_b200.utils.health import check_device_status

    qkv = (torch.randn(1, 256, 6, 128, device=DEV) * 0.5).bfloat16().requires_grad_()
    attention.causal_attention(qkv, 4, 1).sum().backward()
    torch.cuda.synchronize()
    check_device_status()


def test_adamw_is_skipped_while_the_health_word_is_set():
    """A step that follows a collective which gave up must not be applied: the guarded AdamW launch
    reads the library's health word on the device and leaves parameters and moments alone."""
    from fsdp_comm_opt_b200.ops.adamw import FusedAdamW

    lib = _lib.cuda()
    p = torch.nn.Parameter(torch.randn(1 << 16, device=DEV).bfloat16())
    p.grad = torch.randn_like(p)
    opt = FusedAdamW([p], lr=1e-2)
    before = p.detach().clone()
    assert lib.zc_health_set(2) == 0          # what an expired wait writes
    opt.step()
    torch.cuda.synchronize()
    assert torch.equal(p.detach(), before)
    assert float(opt.state[p]["exp_avg"].float().abs().sum()) == 0.0
    assert lib.zc_health_read_and_clear() == 2
    opt.step()
    torch.cuda.synchronize()
    assert not torch.equal(p.detach(), before)
    assert lib.zc_health_read_and_clear() == 0


def test_adamw_in_two_launches_equals_one():
    """``step(split_at=..., between=...)`` updates a prefix first, calls back, then updates the rest:
    same result as one launch (every element is independent)."""
    from fsdp_comm_opt_b200.ops.adamw import FusedAdamW

    torch.manual_seed(4)
    w = torch.randn(100_000, device=DEV).bfloat16()
    g = torch.randn_like(w)
    a, b = torch.nn.Parameter(w.clone()), torch.nn.Parameter(w.clone())
    a.grad, b.grad = g.clone(), g.clone()
    oa, ob = FusedAdamW([a], lr=1e-2), FusedAdamW([b], lr=1e-2)
    called = []
    for _ in range(3):
        oa.step()
        ob.step(split_at=33_333, between=lambda: called.append(1))
    torch.cuda.synchronize()
    assert len(called) == 3 and ob.kernel_launches == 6 and oa.kernel_launches == 3
    assert torch.equal(a.detach(), b.detach())
    assert torch.equal(oa.state[a]["exp_avg_sq"], ob.state[b]["exp_avg_sq"])


@pytest.mark.parametrize("N,K,M,slab_rows,ring", [(1024, 512, 256, 256, 3), (2048, 1024, 384, 512, 2), (512, 256, 128, 512, 2)])
def test_gemm_from_codec_records_matches_fp32_matmul(N, K, M, slab_rows, ring):
    """Decode fused with the consumer GEMM: the weight is given as v2 records, decoded slab by slab
    into an L2-resident ring beside the GEMM; same bits as decode-then-GEMM, close to fp32 matmul."""
    from fsdp_comm_opt_b200.ops.gemm_records import RecordLinear, linear_t_plain
    g = torch.Generator().manual_seed(N + K)
    w = (torch.randn(N, K, generator=g) * 0.02).bfloat16().cuda()
    w[::7, ::5] = 300.0                                   # escapes in most chunks
    x = torch.randn(M, K, generator=g).bfloat16().cuda()
    rec, hdr = codec.v2_encode(w.view(-1))
    rl = RecordLinear(N, K, "cuda", slab_rows=slab_rows, ring=ring)
    y1 = rl(x, rec, hdr).clone()
    y2 = rl(x, rec, hdr)                                  # second call runs over the first call's ring
    plain = linear_t_plain(x, rec, hdr, N, K)
    torch.cuda.synchronize()
    ref = w.float() @ x.float().t()
    assert torch.equal(y1, y2) and torch.equal(y1, plain)
    assert torch.allclose(y1.float(), ref, rtol=2e-2, atol=2e-2 * float(ref.abs().max()))
