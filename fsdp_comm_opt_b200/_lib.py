"""ctypes access to the in-tree native libraries.

``cpu()`` returns ``libzc_cpu.so`` (built on first use with g++ when missing).  ``cuda()`` returns
``libzc_cuda.so``; when a CUDA device is present and the library is missing it is built with nvcc
or the call fails loudly -- kernels never fall back to eager PyTorch on a GPU box.
"""
from __future__ import annotations

import ctypes
import threading
from ctypes import c_int, c_int64, c_void_p, c_float, c_double, c_uint64
from pathlib import Path

import torch

from . import _build

_LOCK = threading.Lock()
_CPU = None
_CUDA = None

P = c_void_p
I = c_int
L = c_int64
F = c_float


def _sig(fn, restype, *argtypes):
    fn.restype = restype
    fn.argtypes = list(argtypes)


def cpu() -> ctypes.CDLL:
    global _CPU
    if _CPU is None:
        with _LOCK:
            if _CPU is None:
                path = _build.LIB / "libzc_cpu.so"
                if not path.exists():
                    _build.build_cpu()
                lib = ctypes.CDLL(str(path))
                _sig(lib.zc_cpu_v1_det_bytes, L, L)
                _sig(lib.zc_cpu_v1_encode_split, None, P, L, P, P, I, I, P, P, P)
                _sig(lib.zc_cpu_v1_decode_split, None, P, P, P, P, I, L, P, P, P)
                _sig(lib.zc_cpu_v1_encode_fused, L, P, L, P, I, I, P, P, P)
                _sig(lib.zc_cpu_v1_decode_fused, None, P, P, P, I, L, P)
                _sig(lib.zc_cpu_v2_encode, L, P, L, P, P)
                _sig(lib.zc_cpu_v2_decode, None, P, P, L, P)
                _sig(lib.zc_cpu_v2_encode_nibble, L, P, L, P, P)
                _sig(lib.zc_cpu_v2_decode_nibble, None, P, P, L, P)
                _sig(lib.zc_cpu_v2_compact, L, P, P, L, P, P)
                _sig(lib.zc_cpu_v2_expand, None, P, P, L, P)
                _CPU = lib
    return _CPU


def cuda_available() -> bool:
    return torch.cuda.is_available()


def debug_bounds() -> bool:
    """``ZC_DEBUG_BOUNDS=1`` selects the bounds-checked build of the kernels."""
    import os

    return os.environ.get("ZC_DEBUG_BOUNDS", "0") == "1"


def cuda_lib_path() -> Path:
    return _build.LIB / ("libzc_cuda_dbg.so" if debug_bounds() else "libzc_cuda.so")


# kernels launched by one call of each C launcher (for the launch counter)
_KERNELS_PER_CALL = {
    "zc_v1_encode_split": 3, "zc_v1_encode_fused": 3, "zc_v1_base_from_std": 2, "zc_quant_int8": 2,
    "zc_health_word": 0, "zc_health_read_and_clear": 0, "zc_health_set": 0, "zc_attn_bwd": 3, "zc_attn_bwd_ws": 3, "zc_attn_bwd_ws_status_read_and_clear": 0, "zc_attn_status_read_and_clear": 0, "zc_attn_ws_status_read_and_clear": 0, "zc_gemm_status_read_and_clear": 0,
}
_LAUNCHES = 0


class _CountingLib:
    """Proxy over the CDLL that counts kernel launches made through the C launchers."""

    def __init__(self, lib):
        self._lib = lib
        self._cache = {}

    def __getattr__(self, name):
        fn = self._cache.get(name)
        if fn is None:
            raw = getattr(self._lib, name)
            n = _KERNELS_PER_CALL.get(name, 1)

            def fn(*args, _raw=raw, _n=n):
                global _LAUNCHES
                _LAUNCHES += _n
                return _raw(*args)

            self._cache[name] = fn
        return fn


def launch_count() -> int:
    """Kernels of this library launched since the last ``reset_launch_count``."""
    return _LAUNCHES


def reset_launch_count() -> None:
    global _LAUNCHES
    _LAUNCHES = 0


def cuda():
    """The CUDA kernel library.  Raises when it cannot be loaded."""
    global _CUDA
    if _CUDA is None:
        with _LOCK:
            if _CUDA is None:
                path = cuda_lib_path()
                if not path.exists():
                    built = _build.build_cuda(debug_bounds=debug_bounds())
                    if built is None:
                        raise RuntimeError(
                            "libzc_cuda.so is missing and nvcc was not found; run "
                            "`python -m fsdp_comm_opt_b200._build` on a host with the CUDA toolkit")
                lib = ctypes.CDLL(str(path))
                from . import _cuda_sigs

                _cuda_sigs.declare(lib)
                _CUDA = _CountingLib(lib)
    return _CUDA


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


_RAW_STREAM = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def stream_ptr(device=None) -> int:
    """``cudaStream_t`` of the current stream of ``device`` (default: the current device).  Every kernel
    launch asks for it, so it takes the direct query: building a ``torch.cuda.Stream`` object per
    launch cost 8 us, a fifth of the host time of a launch-bound step."""
    if _RAW_STREAM is not None:
        if device is None:
            idx = torch.cuda.current_device()
        elif isinstance(device, int):
            idx = device
        else:
            idx = device.index if getattr(device, "index", None) is not None else torch.cuda.current_device()
        return _RAW_STREAM(idx)
    return torch.cuda.current_stream(device).cuda_stream


def check(code: int, what: str) -> None:
    if code != 0:
        raise RuntimeError(f"{what} failed with native status {code}")
