"""Wire compatibility with the reference's own codec kernels on the GPU: streams written by the
reference extension (built from its sources, ``baseline/_ref/zipccl``) are decoded by this
package's v1 decoder and the other way round, bit for bit.  Buffers are sized exactly as the
reference hook sizes them (reference: main/zipccl_comm.py:81-152) and every tensor is a multiple
of 4096 elements on an aligned pointer, the only inputs the reference encoder handles without
dropping tail elements (reference: zipccl/hopper_zip.cu:336-349).  Skipped when the reference
extension is not installed."""
import glob
import importlib.util
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

from fsdp_comm_opt_b200.ops import codec

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DEV = torch.device("cuda", 0)


def load_reference_extension():
    """The reference's compiled module, loaded by path (its package name collides with the drop-in
    ``zipccl`` package of this repository).  None when it is not installed."""
    hits = glob.glob(os.path.join(ROOT, "baseline", "_ref", "zipccl", "hopper_fastzip2*.so"))
    if not hits:
        return None
    spec = importlib.util.spec_from_file_location("hopper_fastzip2", hits[0])
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@pytest.fixture(scope="module")
def ref():
    mod = load_reference_extension()
    if mod is None:
        pytest.skip("reference extension not installed under baseline/_ref")
    return mod


def _inputs(n, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = (torch.randn(n, device=DEV, generator=g) * 0.02).bfloat16()
    # every class of bit pattern: zeros, denormals, infinities, NaNs, large values
    special = torch.tensor([0.0, -0.0, 1e-40, -1e-40, float("inf"), float("-inf"), float("nan"), 3e38, 1.0, -2.5],
                           device=DEV).bfloat16()
    x[: special.numel()] = special
    x[n // 2: n // 2 + special.numel()] = special
    return x


class _Buffers:
    """The allocations of the reference hook for one work of ``n`` (padded) elements."""

    def __init__(self, n, base):
        self.n = n
        self.n_8 = torch.full((1,), n, dtype=torch.int32, device=DEV)
        self.bases = torch.full((256,), base, dtype=torch.int32, device=DEV)
        self.det = torch.zeros(codec.v1_det_bytes(n), dtype=torch.uint8, device=DEV)
        cap = codec.align128(n)
        self.scratch = torch.zeros(cap, dtype=torch.uint8, device=DEV)
        self.esc = torch.zeros(cap, dtype=torch.uint8, device=DEV)
        self.gc = torch.zeros(1, dtype=torch.int32, device=DEV)

    def decode_args(self):
        count = int(self.gc[0])
        stride = codec.align128(count)
        return (self.det, self.esc[:stride].contiguous(), self.n_8.clone(),
                torch.full((1,), stride, dtype=torch.int32, device=DEV))


@pytest.mark.parametrize("n,base", [(4096, 116), (4096 * 64, 116), (4096 * 257, 118), (4096 * 16, 200)])
def test_reference_streams_are_read_by_this_decoder_and_back(ref, n, base):
    x = _inputs(n, n % 97)
    # reference encoder -> this decoder
    a = _Buffers(n, base)
    ref.compress_split_store(x, a.n_8, a.bases, a.det, a.scratch, a.esc, a.gc, 1)
    torch.cuda.synchronize()
    out = torch.zeros(n, dtype=torch.bfloat16, device=DEV)
    det, esc, n_8, nbytes = a.decode_args()
    codec.v1_decompress_split_store_unpad(det, esc, n_8, nbytes, out, n, 1)
    torch.cuda.synchronize()
    assert torch.equal(out.view(torch.int16), x.view(torch.int16))
    # this encoder -> reference decoder
    b = _Buffers(n, base)
    codec.v1_compress_split_store(x, b.n_8, b.bases, b.det, b.scratch, b.esc, b.gc, 1)
    torch.cuda.synchronize()
    assert int(b.gc[0]) == int(a.gc[0])            # same outliers under the same base
    out2 = torch.zeros(n, dtype=torch.bfloat16, device=DEV)
    det, esc, n_8, nbytes = b.decode_args()
    ref.decompress_split_store_unpad(det, esc, n_8, nbytes, out2, n, 1)
    torch.cuda.synchronize()
    assert torch.equal(out2.view(torch.int16), x.view(torch.int16))
    # sign+mantissa bytes, bit planes and the base word are byte-identical; only the placement of
    # the blocks' outlier runs may differ (the reference reserves them with an atomic, in arrival
    # order), and with a single block not even that
    fixed = n + n // 8 * 3
    assert torch.equal(a.det[:fixed], b.det[:fixed])
    assert torch.equal(a.det[fixed + 4 * (n // 4096): fixed + 4 * (n // 4096) + 4],
                       b.det[fixed + 4 * (n // 4096): fixed + 4 * (n // 4096) + 4])
    if n == 4096:
        assert torch.equal(a.det, b.det) and torch.equal(a.esc[: int(a.gc[0])], b.esc[: int(b.gc[0])])


def test_multi_work_streams_cross_decode(ref):
    """Eight works (one per peer of an all-gather), decoded by the other implementation in one call."""
    world, n = 8, 4096 * 24
    xs = [_inputs(n, 500 + r) for r in range(world)]
    enc = []
    for r, x in enumerate(xs):
        b = _Buffers(n, 116)
        (ref.compress_split_store if r % 2 == 0 else codec.v1_compress_split_store)(
            x, b.n_8, b.bases, b.det, b.scratch, b.esc, b.gc, 1)
        enc.append(b)
    torch.cuda.synchronize()
    stride = codec.align128(max(int(b.gc[0]) for b in enc))
    det = torch.stack([b.det for b in enc]).reshape(-1)
    esc = torch.stack([b.esc[:stride] for b in enc]).reshape(-1).contiguous()
    n_8 = torch.full((world,), n, dtype=torch.int32, device=DEV)
    nbytes = torch.full((world,), stride, dtype=torch.int32, device=DEV)
    want = torch.cat(xs).view(torch.int16)
    for decode in (ref.decompress_split_store_unpad, codec.v1_decompress_split_store_unpad):
        out = torch.zeros(world * n, dtype=torch.bfloat16, device=DEV)
        decode(det, esc, n_8, nbytes, out, n, world)
        torch.cuda.synchronize()
        assert torch.equal(out.view(torch.int16), want)
