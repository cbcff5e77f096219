"""CPU paths of the ops against plain PyTorch fp32 references (values and gradients)."""
import math

import pytest
import torch
import torch.nn.functional as F

from fsdp_comm_opt_b200.ops import adamw, attention, gemm, loss, norm, quant, rope, swiglu


def test_rms_norm_matches_torch():
    torch.manual_seed(0)
    x = torch.randn(6, 64, requires_grad=True)
    w = torch.randn(64, requires_grad=True)
    y = norm.rms_norm(x, w, 1e-5)
    ref = F.rms_norm(x.detach().requires_grad_(), (64,), w.detach().requires_grad_(), 1e-5)
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr = x.detach().clone().requires_grad_(), w.detach().clone().requires_grad_()
    F.rms_norm(xr, (64,), wr, 1e-5).backward(g)
    assert torch.allclose(y, ref, atol=1e-5)
    assert torch.allclose(x.grad, xr.grad, atol=1e-5) and torch.allclose(w.grad, wr.grad, atol=1e-4)


def test_add_rms_norm_matches_unfused():
    torch.manual_seed(1)
    a = torch.randn(5, 32, requires_grad=True)
    r = torch.randn(5, 32, requires_grad=True)
    w = torch.randn(32, requires_grad=True)
    y, h = norm.add_rms_norm(a, r, w, 1e-5)
    (y.sum() + (h * 0.5).sum()).backward()
    a2, r2, w2 = (t.detach().clone().requires_grad_() for t in (a, r, w))
    h2 = a2 + r2
    y2 = F.rms_norm(h2, (32,), w2, 1e-5)
    (y2.sum() + (h2 * 0.5).sum()).backward()
    assert torch.allclose(y, y2, atol=1e-5) and torch.allclose(h, h2)
    for p, q in ((a, a2), (r, r2), (w, w2)):
        assert torch.allclose(p.grad, q.grad, atol=1e-4)


def test_swiglu_matches_torch():
    torch.manual_seed(2)
    gu = torch.randn(7, 48, requires_grad=True)
    out = swiglu.swiglu(gu)
    g = torch.randn_like(out)
    out.backward(g)
    gu2 = gu.detach().clone().requires_grad_()
    ref = F.silu(gu2[:, :24]) * gu2[:, 24:]
    ref.backward(g)
    assert torch.allclose(out, ref, atol=1e-6) and torch.allclose(gu.grad, gu2.grad, atol=1e-5)


def test_cross_entropy_matches_torch_with_ignore():
    torch.manual_seed(3)
    logits = torch.randn(10, 50)
    labels = torch.randint(0, 50, (10,))
    labels[3] = -100
    l1 = logits.clone().requires_grad_()
    out = loss.cross_entropy(l1 * 1.0, labels)
    out.backward()
    l2 = logits.clone().requires_grad_()
    ref = F.cross_entropy(l2, labels, ignore_index=-100)
    ref.backward()
    assert torch.allclose(out, ref, atol=1e-5) and torch.allclose(l1.grad, l2.grad, atol=1e-6)


def _sdpa_ref(qkv, Hq, Hkv):
    q, k, v = qkv[:, :, :Hq], qkv[:, :, Hq:Hq + Hkv], qkv[:, :, Hq + Hkv:]
    g = Hq // Hkv
    q, k, v = (t.transpose(1, 2) for t in (q, k, v))
    k, v = k.repeat_interleave(g, 1), v.repeat_interleave(g, 1)
    return F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2)


def test_attention_gqa_matches_sdpa():
    torch.manual_seed(4)
    B, S, Hq, Hkv, D = 2, 17, 4, 2, 16
    qkv = torch.randn(B, S, Hq + 2 * Hkv, D, requires_grad=True)
    o = attention.causal_attention(qkv * 1.0, Hq, Hkv)
    g = torch.randn_like(o)
    o.backward(g)
    q2 = qkv.detach().clone().requires_grad_()
    _sdpa_ref(q2, Hq, Hkv).backward(g)
    assert torch.allclose(o, _sdpa_ref(q2, Hq, Hkv), atol=1e-5)
    assert torch.allclose(qkv.grad, q2.grad, atol=1e-4)


def test_rope_rotation_and_fused_attention_gradient():
    torch.manual_seed(5)
    B, S, Hq, Hkv, D = 1, 8, 2, 1, 8
    cos, sin = rope.rope_tables(S, D, 10000.0, "cpu")
    qkv = torch.randn(B, S, Hq + 2 * Hkv, D, requires_grad=True)
    # unfused reference: differentiable rope then attention
    flat = qkv.reshape(B * S, -1)
    rot = rope.apply_rope(flat, cos, sin, Hq + Hkv, D, S).view(B, S, -1, D)
    ref = attention.causal_attention(rot, Hq, Hkv)
    g = torch.randn_like(ref)
    ref.backward(g)
    gref = qkv.grad.clone()
    qkv.grad = None
    out = attention.causal_attention((qkv * 1.0).contiguous(), Hq, Hkv, None, cos, sin)
    out.backward(g)
    assert torch.allclose(out, ref, atol=1e-5) and torch.allclose(qkv.grad, gref, atol=1e-5)
    # rotation preserves norms and matches the closed form for one pair
    x = torch.randn(S, D)
    y = rope._rotate(x.clone(), cos, sin, 1, D, S, 1.0)
    assert torch.allclose(x.norm(dim=1), y.norm(dim=1), atol=1e-5)
    t, i = 3, 1
    a, b = x[t, i], x[t, i + D // 2]
    assert math.isclose(y[t, i].item(), (a * cos[t, i] - b * sin[t, i]).item(), abs_tol=1e-6)


def test_linear_matches_torch():
    torch.manual_seed(6)
    x = torch.randn(3, 5, 16, requires_grad=True)
    w = torch.randn(24, 16, requires_grad=True)
    y = gemm.linear(x, w)
    g = torch.randn_like(y)
    y.backward(g)
    x2, w2 = x.detach().clone().requires_grad_(), w.detach().clone().requires_grad_()
    F.linear(x2, w2).backward(g)
    assert torch.allclose(y, F.linear(x2, w2), atol=1e-5)
    assert torch.allclose(x.grad, x2.grad, atol=1e-5) and torch.allclose(w.grad, w2.grad, atol=1e-5)


def test_fused_adamw_matches_torch_adamw():
    torch.manual_seed(7)
    p1 = torch.nn.Parameter(torch.randn(100))
    p2 = torch.nn.Parameter(p1.detach().clone())
    o1 = adamw.FusedAdamW([p1], lr=1e-2, weight_decay=0.1)
    o2 = torch.optim.AdamW([p2], lr=1e-2, weight_decay=0.1)
    for _ in range(5):
        g = torch.randn(100)
        p1.grad, p2.grad = g.clone(), g.clone()
        o1.step(), o2.step()
    assert torch.allclose(p1, p2, atol=1e-6)
    sd = o1.state_dict()["state"][0]
    assert set(sd) == {"step", "exp_avg", "exp_avg_sq"}


def test_int8_quant_error_bound():
    torch.manual_seed(8)
    x = torch.randn(1000) * 0.02
    world = 3
    buf = torch.zeros(world, quant.packed_bytes(1000), dtype=torch.uint8)
    for r in range(world):
        quant.quantize_pack(x * (r + 1), buf[r])
    out = torch.zeros(world * 1000)
    quant.dequantize_unpack(buf, 1000, out)
    for r in range(world):
        scale = (x * (r + 1)).abs().max() / 127
        assert (out[r * 1000:(r + 1) * 1000] - x * (r + 1)).abs().max() <= scale / 2 + 1e-7


def test_gpt2_ops_cpu_paths_match_torch():
    """CPU paths of layer_norm and bias_gelu (the arithmetic the CUDA kernels implement)."""
    import torch.nn.functional as F

    from fsdp_comm_opt_b200.ops import gpt2_ops

    torch.manual_seed(5)
    x = torch.randn(12, 64, requires_grad=True)
    w = (1 + 0.1 * torch.randn(64)).requires_grad_()
    b = (0.1 * torch.randn(64)).requires_grad_()
    y = gpt2_ops.layer_norm(x, w, b, 1e-5)
    g = torch.randn_like(y)
    y.backward(g)
    x2, w2, b2 = (t.detach().clone().requires_grad_() for t in (x, w, b))
    ref = F.layer_norm(x2, (64,), w2, b2, 1e-5)
    ref.backward(g)
    for got, want in ((y, ref), (x.grad, x2.grad), (w.grad, w2.grad), (b.grad, b2.grad)):
        assert torch.allclose(got, want, atol=1e-5, rtol=1e-4)
    u = torch.randn(7, 32, requires_grad=True)
    c = torch.randn(32, requires_grad=True)
    z = gpt2_ops.bias_gelu(u, c)
    gz = torch.randn_like(z)
    z.backward(gz)
    u2, c2 = u.detach().clone().requires_grad_(), c.detach().clone().requires_grad_()
    zr = F.gelu(u2 + c2, approximate="tanh")
    zr.backward(gz)
    for got, want in ((z, zr), (u.grad, u2.grad), (c.grad, c2.grad)):
        assert torch.allclose(got, want, atol=1e-5, rtol=1e-4)


def test_gemm_from_codec_records_cpu():
    from fsdp_comm_opt_b200.ops import codec
    from fsdp_comm_opt_b200.ops.gemm_records import RecordLinear, linear_t_plain
    N, K, M = 512, 256, 48
    g = torch.Generator().manual_seed(5)
    w = (torch.randn(N, K, generator=g) * 0.02).bfloat16()
    x = torch.randn(M, K, generator=g).bfloat16()
    rec, hdr = codec.v2_encode(w.view(-1))
    y = RecordLinear(N, K, "cpu", slab_rows=128, ring=2)(x, rec, hdr)
    ref = (w.float() @ x.float().t()).to(torch.bfloat16)
    assert torch.equal(y, ref) and torch.equal(linear_t_plain(x, rec, hdr, N, K), ref)
    with pytest.raises(ValueError):
        RecordLinear(N, K, "cpu", slab_rows=100)
