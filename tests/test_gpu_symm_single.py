"""The fused collective kernels on ONE GPU: the ranks of a world of W are run one after the other
(every other rank's pusher half first, then rank 0's whole kernel), each on its own staging buffer
in this GPU's memory.  Pushers never wait for another launch and rank 0's decoders find every flag
already set, so no kernel waits for a kernel that has not run.  This checks the encode -> staging
layout -> flag -> pipelined decode (-> reduce) path bit for bit without a second device."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

from fsdp_comm_opt_b200 import _lib
from fsdp_comm_opt_b200.ops import codec

DEV = torch.device("cuda", 0)


GUARD, CANARY = 4096, 0xA5


class _World:
    def __init__(self, world: int, numel_per_source: int):
        lib = _lib.cuda()
        raw = lib._lib
        raw.zc_symm_buffer_bytes.restype = ctypes.c_int64
        raw.zc_symm_buffer_bytes.argtypes = [ctypes.c_int, ctypes.c_int64]
        self.lib, self.world = lib, world
        self.nc_max = max(1024, codec.v2_num_chunks(numel_per_source))
        nbytes = int(raw.zc_symm_buffer_bytes(world, self.nc_max))
        # every staging buffer sits between two canary regions that no kernel may touch
        self.raw = [torch.full((nbytes + 2 * GUARD,), CANARY, dtype=torch.uint8, device=DEV) for _ in range(world)]
        self.bufs = [r[GUARD:GUARD + nbytes] for r in self.raw]
        for b in self.bufs:
            b.zero_()
        self.ptrs = torch.tensor([b.data_ptr() for b in self.bufs], dtype=torch.int64, device=DEV)

    def canaries_intact(self):
        return all(bool((r[:GUARD] == CANARY).all()) and bool((r[-GUARD:] == CANARY).all()) for r in self.raw)

    def status(self, r):
        return self.bufs[r][:4096].view(torch.int32)[65:68].tolist()

    def all_gather(self, rank, x, out, push, dec, seq=1, wire=0):
        _lib.check(self.lib.zc_symm_all_gather(
            x.data_ptr(), out.data_ptr(), self.ptrs.data_ptr(), self.bufs[rank].data_ptr(), None, x.numel(), rank,
            self.world, self.nc_max, seq, push, dec, 1.0, wire, _lib.stream_ptr(DEV)), "zc_symm_all_gather")

    def reduce_scatter(self, rank, x, out, push, dec, seq=1, scale=1.0, wire=0):
        shard = x.numel() // self.world
        _lib.check(self.lib.zc_symm_reduce_scatter(
            x.data_ptr(), out.data_ptr(), None, self.ptrs.data_ptr(), self.bufs[rank].data_ptr(), shard, rank,
            self.world, self.nc_max, seq, int(x.dtype == torch.float32), int(out.dtype == torch.float32), scale,
            push, dec, 1.0, wire, _lib.stream_ptr(DEV)), "zc_symm_reduce_scatter")


def _params(n, seed, outliers=False):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(n, device=DEV, generator=g) * 0.02
    if outliers:
        m = torch.rand(n, device=DEV, generator=g) < 0.01
        x = torch.where(m, x * 100, x)
    return x.bfloat16()


@pytest.mark.parametrize("wire", [0, 2, 1], ids=["compressed", "nibble", "verbatim"])
@pytest.mark.parametrize("world,n", [(2, 1 << 20), (4, 300_001), (8, 1 << 18), (8, 5000)])
def test_fused_all_gather_ranks_in_sequence(world, n, wire):
    w = _World(world, n)
    shards = [_params(n, 10 + r, outliers=(r % 2 == 1)) for r in range(world)]
    scratch = torch.empty(world * n, dtype=torch.bfloat16, device=DEV)
    for r in range(1, world):                      # the other ranks: encode and push only
        w.all_gather(r, shards[r], scratch, push=32, dec=0, wire=wire)
    out = torch.zeros(world * n, dtype=torch.bfloat16, device=DEV)
    w.all_gather(0, shards[0], out, push=32, dec=64, wire=wire)   # rank 0: push, then decode what has arrived
    torch.cuda.synchronize()
    assert w.status(0) == [0, 0, 0] and w.canaries_intact()
    assert torch.equal(out.view(torch.int16), torch.cat(shards).view(torch.int16))


@pytest.mark.parametrize("wire", [0, 2], ids=["compressed", "nibble"])
def test_fused_all_gather_adversarial_bit_patterns(wire):
    """Inputs that reach every branch of the record coder: random bit patterns (exponents all over the range:
    the raw fallback), zeros (one exponent: width 0), exponent fields below 15 (window base 0), and a
    Gaussian body with a few huge values (escapes below the window of the nibble mode)."""
    world, n = 4, 96 * 1024 + 77
    g = torch.Generator(device="cuda").manual_seed(5)
    rnd = torch.randint(0, 65536, (n,), device=DEV, generator=g, dtype=torch.int32).to(torch.int16).view(torch.bfloat16)
    tiny = (torch.randint(0, 15 << 7, (n,), device=DEV, generator=g, dtype=torch.int32)
            | (torch.randint(0, 2, (n,), device=DEV, generator=g, dtype=torch.int32) << 15)).to(torch.int16).view(torch.bfloat16)
    body = (torch.randn(n, device=DEV, generator=g) * 1e-3).bfloat16()
    body[::1500] = 3.0e4
    shards = [rnd, torch.zeros(n, dtype=torch.bfloat16, device=DEV), tiny, body]
    w = _World(world, n)
    scratch = torch.empty(world * n, dtype=torch.bfloat16, device=DEV)
    for r in range(1, world):
        w.all_gather(r, shards[r], scratch, push=16, dec=0, wire=wire)
    out = torch.zeros(world * n, dtype=torch.bfloat16, device=DEV)
    w.all_gather(0, shards[0], out, push=16, dec=32, wire=wire)
    torch.cuda.synchronize()
    assert w.status(0) == [0, 0, 0] and w.canaries_intact()
    assert torch.equal(out.view(torch.int16), torch.cat(shards).view(torch.int16))


def _decode_staged_records_on_host(buf, world, nc_max, parity, src, n, nibble):
    """Second oracle for the staging format: rebuild a source's n bf16 values from the bytes the pusher
    left in a staging buffer, using only the layout rules written down in ``csrc/codec_format.h``
    (header word, sign+mantissa section in two 512-byte halves, bit planes or nibble-packed codes,
    escapes in element order, raw records)."""
    import numpy as np

    b = buf.cpu().numpy()
    align128 = lambda x: (x + 127) // 128 * 128
    max_groups = (nc_max + 63) // 64
    flag_bytes = align128(2 * world * max_groups * 4)
    hdr_bytes = align128(nc_max * 4)
    slot_bytes = hdr_bytes + nc_max * 2048
    slot = 4096 + flag_bytes + parity * world * slot_bytes + src * slot_bytes
    hdrs = b[slot:slot + hdr_bytes].view(np.uint32)
    out = np.zeros(((n + 1023) // 1024) * 1024, dtype=np.uint16)
    for c in range((n + 1023) // 1024):
        h = int(hdrs[c])
        base, width, n_esc = h & 0xFF, (h >> 8) & 0xF, h >> 16
        rec = b[slot + hdr_bytes + c * 2048: slot + hdr_bytes + (c + 1) * 2048]
        lane = np.arange(1024) // 32
        j = np.arange(1024) % 32
        sm = np.where(j < 16, rec[16 * lane + j], rec[512 + 16 * lane + (j - 16)]).astype(np.uint16)
        if width == 8:
            ex = rec[1024:2048].astype(np.uint16)
        elif width == 0:
            ex = np.full(1024, base, dtype=np.uint16)
        else:
            if nibble:
                assert width == 4
                k, jj = (j // 8), (j % 8)
                byte = rec[1024 + 16 * lane + 4 * k + (jj % 4)]
                code = np.where(jj < 4, byte & 0xF, byte >> 4).astype(np.int32)
                tail = 1024 + 512
            else:
                planes = rec[1024:1024 + 128 * width].view(np.uint32).reshape(width, 32)
                code = np.zeros(1024, dtype=np.int32)
                for p_ in range(width):
                    code |= ((planes[p_][lane] >> j) & 1).astype(np.int32) << p_
                tail = 1024 + 128 * width
            esc_pos = np.cumsum(code == 0) - 1
            assert int((code == 0).sum()) == n_esc
            esc = rec[tail:tail + max(n_esc, 1)].astype(np.int32)
            ex = np.where(code == 0, esc[np.clip(esc_pos, 0, max(n_esc, 1) - 1)], base + code - 1).astype(np.uint16)
        out[c * 1024:(c + 1) * 1024] = (sm & 0x7F) | (ex << 7) | ((sm >> 7) << 15)
    return torch.from_numpy(out[:n].view(np.int16))


@pytest.mark.parametrize("wire", [0, 2], ids=["compressed", "nibble"])
def test_staged_records_follow_the_documented_layout(wire):
    world, n = 2, 20 * 1024 + 300
    g = torch.Generator(device="cuda").manual_seed(9)
    x = (torch.randn(n, device=DEV, generator=g) * 0.02).bfloat16()
    x[::700] = 250.0                                  # escapes
    x[5 * 1024:6 * 1024] = 0.5                        # one exponent: width 0
    x[7 * 1024:8 * 1024] = torch.randint(0, 65536, (1024,), device=DEV, generator=g, dtype=torch.int32).to(
        torch.int16).view(torch.bfloat16)             # raw record
    w = _World(world, n)
    scratch = torch.empty(world * n, dtype=torch.bfloat16, device=DEV)
    w.all_gather(1, x, scratch, push=8, dec=0, wire=wire)        # rank 1 pushes into rank 0's buffer, parity of seq 1
    torch.cuda.synchronize()
    got = _decode_staged_records_on_host(w.bufs[0], world, w.nc_max, parity=1, src=1, n=n, nibble=(wire == 2))
    assert torch.equal(got, x.cpu().view(torch.int16))


@pytest.mark.parametrize("world,shard,dtype", [(2, 1 << 19, torch.bfloat16), (4, 70_000, torch.float32),
                                               (8, 1 << 16, torch.bfloat16), (8, 3000, torch.bfloat16)])
@pytest.mark.parametrize("wire", [0, 2, 1], ids=["compressed", "nibble", "verbatim"])
def test_fused_reduce_scatter_ranks_in_sequence(world, shard, dtype, wire):
    w = _World(world, shard)
    rows = [(_params(world * shard, 40 + r, outliers=True).float() * 0.05).bfloat16().to(dtype) for r in range(world)]
    dummy = torch.empty(shard, dtype=torch.float32, device=DEV)
    for r in range(1, world):
        w.reduce_scatter(r, rows[r], dummy, push=48, dec=0, wire=wire)
    out = torch.zeros(shard, dtype=torch.float32, device=DEV)
    w.reduce_scatter(0, rows[0], out, push=48, dec=64, scale=1.0 / world, wire=wire)
    torch.cuda.synchronize()
    assert w.status(0) == [0, 0, 0] and w.canaries_intact()
    # the kernel adds its own row first, then the sources by rank, in fp32
    ref = rows[0][:shard].float()
    for r in range(1, world):
        ref = ref + rows[r][:shard].float()
    ref = ref * (1.0 / world)
    assert torch.equal(out, ref)


def test_decoder_reports_a_flag_that_never_comes():
    """Nothing pushed for source 1: rank 0's decoders give up after the (1 s) limit, record which source
    and group they waited for, and the kernel returns normally."""
    w = _World(2, 1 << 14)
    x = _params(1 << 14, 3)
    out = torch.zeros(2 << 14, dtype=torch.bfloat16, device=DEV)
    w.all_gather(0, x, out, push=4, dec=4)
    torch.cuda.synchronize()
    code, peer, _group = w.status(0)
    assert code == 2 and peer == 1
    torch.cuda.synchronize()  # the context is still usable
    assert torch.equal(out[: 1 << 14].view(torch.int16), x.view(torch.int16))


def test_same_cases_on_the_bounds_checked_build():
    """The small cases above once more in a fresh process on ``libzc_cuda_dbg.so`` (every store into a
    staging slot checked against the slot's extent before it is issued; an offending store would be
    skipped and show up as status code 3)."""
    import os
    import subprocess
    import sys

    if os.environ.get("ZC_DEBUG_BOUNDS") == "1":
        assert _lib.cuda()._lib.zc_debug_bounds_build() == 1
        return
    env = dict(os.environ, ZC_DEBUG_BOUNDS="1")
    r = subprocess.run([sys.executable, "-m", "pytest", __file__, "-x", "-q", "-k", "sequence or bounds_checked"],
                       env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
