"""The allocation-free encoder entry point, called through its exported C symbol.

Some users of the library cannot allocate device memory at call time (see
``fsdp_comm_opt_b200/csrc/zc_noalloc.h``: side-stream comm hooks under a full caching allocator,
loops that must avoid the device synchronisation of cudaMalloc).  For them
``zc_v1_encode_split_noalloc`` keeps its scratch in a static device array.  This test checks that
it writes exactly the bytes of the regular entry point, twice in a row (the second, smaller call
runs over the first call's leftovers), and that an oversized request is refused.

The file name sorts last on purpose: a failure here cannot hide another test's result in a run
that stops at the first failure.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

from fsdp_comm_opt_b200 import _lib
from fsdp_comm_opt_b200.ops import codec

MAX_ELEMS = 16 * 1024 * 1024


def _symbol():
    raw = _lib.cuda()._lib                      # the ctypes.CDLL itself: plain exported C symbol
    fn = raw.zc_v1_encode_split_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int,
                   ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_longlong,
                   ctypes.c_void_p]
    return fn


def _buffers(n, n_works, dev):
    per = codec.pad_to_block((n + n_works - 1) // n_works)
    n_8 = torch.full((n_works,), per, dtype=torch.int32, device=dev)
    det = torch.zeros(n_works * codec.v1_det_bytes(per), dtype=torch.uint8, device=dev)
    esc = torch.zeros(n_works * codec.align128(per), dtype=torch.uint8, device=dev)
    gc = torch.zeros(n_works, dtype=torch.int32, device=dev)
    return per, n_8, det, esc, gc


def _run_pair(fn, n, n_works, seed, base):
    dev = torch.device("cuda")
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn(n, generator=g) * 0.02).to(torch.bfloat16)
    x[::97] = 1000.0                                           # plenty of outliers
    x = x.to(dev)
    bases = torch.full((256,), base, dtype=torch.int32, device=dev)
    per, n_8, det_a, esc_a, gc_a = _buffers(n, n_works, dev)
    scratch = torch.zeros(n_works * per, dtype=torch.uint8, device=dev)
    codec.v1_compress_split_store(x, n_8, bases, det_a, scratch, esc_a, gc_a, n_works)   # existing entry point
    _, _, det_b, esc_b, gc_b = _buffers(n, n_works, dev)
    stream = torch.cuda.current_stream().cuda_stream
    rc = fn(x.data_ptr(), n, n_8.data_ptr(), None, n_works, bases.data_ptr(), det_b.data_ptr(), esc_b.data_ptr(),
            gc_b.data_ptr(), n_works * per // 4096, stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert torch.equal(gc_a, gc_b) and int(gc_b.sum()) > 0
    assert torch.equal(det_a, det_b)
    assert torch.equal(esc_a, esc_b)
    # and the stream decodes back to the input
    out = torch.zeros(n_works * per, dtype=torch.bfloat16, device=dev)
    codec.v1_decompress_split_store(det_b, esc_b, n_8, gc_b, out, n_works)
    assert torch.equal(out[:n].view(torch.int16), x.view(torch.int16))


def test_noalloc_encode_matches_regular_entry_point_twice():
    fn = _symbol()
    _run_pair(fn, 3 * (1 << 20) + 123, 1, seed=1, base=116)   # first call on this device does the set-up
    _run_pair(fn, 8 * 12288, 8, seed=2, base=118)             # smaller, multi-work, over stale scratch


def test_noalloc_at_exactly_the_size_of_its_scratch():
    """Two works that together fill the built-in scratch to the last byte (4096 blocks of 4096)."""
    _run_pair(_symbol(), MAX_ELEMS, 2, seed=3, base=116)


def test_noalloc_rejects_requests_beyond_its_scratch():
    fn = _symbol()
    dev = torch.device("cuda")
    dummy = torch.zeros(16, dtype=torch.int32, device=dev)
    blocks = MAX_ELEMS // 4096 + 1
    rc = fn(dummy.data_ptr(), 1, dummy.data_ptr(), None, 1, dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(),
            dummy.data_ptr(), blocks, torch.cuda.current_stream().cuda_stream)
    assert rc == -3
    torch.cuda.synchronize()
