"""Python front end of the BF16 exponent codec (v1 window-7 format and v2 per-chunk format).

Every function dispatches on the device of its tensors: CUDA tensors go to the sm_100a kernels in
``libzc_cuda.so`` (current stream, no host sync, no allocation inside the launchers), CPU tensors
go to the scalar C++ codec in ``libzc_cpu.so``.  The ten ``v1_*`` functions implement the surface
of the reference extension (reference: zipccl/hopper_fastzip.cpp:97-403 and
zipccl/hopper_fastzip2.pyi:13-128) with the same argument order and the same wire format.

Differences from the reference that callers can rely on:
  * sizes and dtypes are validated and raise ``ValueError``/``TypeError`` instead of reading out
    of bounds;
  * the outlier stream is laid out in element order (deterministic), not in atomic arrival order;
  * ``nbytes_8`` is always written by ``compress_8`` (the reference skips it for one work);
  * element counts that are not a multiple of 8 and unaligned base pointers are handled exactly.
"""
from __future__ import annotations

import torch

from .. import _lib

ELEMS_PER_BLOCK = 4096
V2_CHUNK = 1024
V2_SLOT = 2048


def align128(n: int) -> int:
    return (n + 127) // 128 * 128


def pad_to_block(n: int) -> int:
    return (n + ELEMS_PER_BLOCK - 1) // ELEMS_PER_BLOCK * ELEMS_PER_BLOCK


def v1_det_bytes(padded_numel: int) -> int:
    """Aligned size of the deterministic stream of one work (reference: main/zipccl_comm.py:42-46)."""
    nb = padded_numel // ELEMS_PER_BLOCK
    return align128(padded_numel + padded_numel // 8 * 3 + nb * 4 + 4)


# --------------------------------------------------------------------------------------------
# helpers
# --------------------------------------------------------------------------------------------

def _req(t: torch.Tensor, dtype, name: str, numel_min: int = 0) -> torch.Tensor:
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name} must be a tensor")
    if t.dtype != dtype:
        raise TypeError(f"{name} must be {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    if t.numel() < numel_min:
        raise ValueError(f"{name} has {t.numel()} elements, needs at least {numel_min}")
    return t


def _same_device(*ts: torch.Tensor) -> torch.device:
    dev = ts[0].device
    for t in ts:
        if t is not None and t.device != dev:
            raise ValueError(f"all tensors must be on {dev}, got one on {t.device}")
    return dev


def _host_sizes(t: torch.Tensor, n: int) -> list[int]:
    return [int(v) for v in t[:n].tolist()]


def _total_blocks_hint(n_8: torch.Tensor, n_works: int, total_padded: int | None) -> int:
    """Grid size.  On CUDA the per-work sizes stay on the device (no sync): the grid is derived
    from a host-known padded total, exactly as the reference launchers do."""
    if total_padded is not None:
        return total_padded // ELEMS_PER_BLOCK
    return sum(_host_sizes(n_8, n_works)) // ELEMS_PER_BLOCK


# --------------------------------------------------------------------------------------------
# v1 surface
# --------------------------------------------------------------------------------------------

def v1_compress_split_store(input, n_8, bases_in, output, output1, output_final,
                            global_zero_counter_8, n_works: int, *, _orig_n_8=None,
                            _padded_n_total: int | None = None) -> None:
    """Split-layout encode (reference: hopper_fastzip.cpp:254-285 -> hopper_zip.cu:311-467, 475-548).

    ``output`` receives the deterministic streams back to back, ``output_final`` the compacted
    outlier streams (stride align128(count)), ``global_zero_counter_8[i]`` the outlier count of
    work i.  ``output1`` is scratch of at least sum(n_8) bytes on CUDA and unused on CPU.
    """
    _req(input, torch.bfloat16, "input")
    _req(n_8, torch.int32, "n_8", n_works)
    _req(bases_in, torch.int32, "bases_in", 1)
    _req(output, torch.uint8, "output")
    _req(output1, torch.uint8, "output1")
    _req(output_final, torch.uint8, "output_final")
    _req(global_zero_counter_8, torch.int32, "global_zero_counter_8", n_works)
    dev = _same_device(input, n_8, bases_in, output, output1, output_final, global_zero_counter_8)
    if _orig_n_8 is not None:
        _req(_orig_n_8, torch.int32, "orig_n_8", n_works)
    total_n = input.numel()
    if dev.type == "cpu":
        sizes = _host_sizes(n_8, n_works)
        if any(s % ELEMS_PER_BLOCK for s in sizes):
            raise ValueError("every n_8[i] must be a multiple of 4096")
        need = sum(v1_det_bytes(s) for s in sizes if s)
        if output.numel() < need:
            raise ValueError(f"output holds {output.numel()} bytes, det streams need {need}")
        _lib.cpu().zc_cpu_v1_encode_split(
            input.data_ptr(), total_n, n_8.data_ptr(), _lib.ptr(_orig_n_8), n_works,
            int(bases_in[0]), output.data_ptr(), output_final.data_ptr(),
            global_zero_counter_8.data_ptr())
        return
    padded = _padded_n_total if _padded_n_total is not None else pad_to_block(total_n)
    if output1.numel() < padded:
        raise ValueError(f"output1 (scratch) holds {output1.numel()} bytes, needs {padded}")
    blocks = padded // ELEMS_PER_BLOCK
    if blocks == 0:
        return
    _lib.check(_lib.cuda().zc_v1_encode_split(
        input.data_ptr(), total_n, n_8.data_ptr(), _lib.ptr(_orig_n_8), n_works,
        bases_in.data_ptr(), output.data_ptr(), output1.data_ptr(), output_final.data_ptr(),
        global_zero_counter_8.data_ptr(), blocks, _lib.stream_ptr(dev)), "zc_v1_encode_split")


def v1_compress_split_store_pad(input, n_8, orig_n_8, bases_in, output, output1, output_final,
                                global_zero_counter_8, padded_n_total: int, n_works: int) -> None:
    """Split encode from a dense input whose works are packed back to back with ``orig_n_8[i]``
    valid elements each, producing the layout of works padded to ``n_8[i]``
    (reference: hopper_fastzip.cpp:374-403 -> hopper_zip.cu:561-724)."""
    v1_compress_split_store(input, n_8, bases_in, output, output1, output_final,
                            global_zero_counter_8, n_works, _orig_n_8=orig_n_8,
                            _padded_n_total=padded_n_total)


def _v1_decode_split(compressed_input, zero_input, n_8, nbytes_8, output, n_works, *, orig_each=-1,
                     out_off=None, orig_n_8=None, padded_n_total=None) -> None:
    _req(compressed_input, torch.uint8, "compressed_input")
    _req(zero_input, torch.uint8, "zero_input")
    _req(n_8, torch.int32, "n_8", n_works)
    _req(nbytes_8, torch.int32, "nbytes_8", n_works)
    _req(output, torch.bfloat16, "output")
    dev = _same_device(compressed_input, zero_input, n_8, nbytes_8, output)
    if out_off is not None:
        _req(out_off, torch.int32, "out_off", n_works)
        _req(orig_n_8, torch.int32, "orig_n_8", n_works)
    if dev.type == "cpu":
        _lib.cpu().zc_cpu_v1_decode_split(
            compressed_input.data_ptr(), zero_input.data_ptr(), n_8.data_ptr(), nbytes_8.data_ptr(),
            n_works, orig_each, _lib.ptr(out_off), _lib.ptr(orig_n_8), output.data_ptr())
        return
    if padded_n_total is None:
        padded_n_total = pad_to_block(output.numel())
    blocks = padded_n_total // ELEMS_PER_BLOCK
    if blocks == 0:
        return
    _lib.check(_lib.cuda().zc_v1_decode_split(
        compressed_input.data_ptr(), zero_input.data_ptr(), n_8.data_ptr(), nbytes_8.data_ptr(),
        n_works, orig_each, _lib.ptr(out_off), _lib.ptr(orig_n_8), output.data_ptr(), output.numel(),
        blocks, _lib.stream_ptr(dev)), "zc_v1_decode_split")


def v1_decompress_split_store(compressed_input, zero_input, n_8, nbytes_8, output, n_works: int) -> None:
    """reference: hopper_fastzip.cpp:287-307 -> hopper_zip.cu:1024-1163."""
    _v1_decode_split(compressed_input, zero_input, n_8, nbytes_8, output, n_works)


def v1_decompress_split_store_unpad(compressed_input, zero_input, n_8, nbytes_8, output,
                                    orig_ele_num: int, n_works: int) -> None:
    """Work i writes its first ``orig_ele_num`` elements at ``i * orig_ele_num``
    (reference: hopper_fastzip.cpp:312-336 -> hopper_zip.cu:1170-1322)."""
    if output.numel() < orig_ele_num * n_works:
        raise ValueError("output is smaller than orig_ele_num * n_works")
    _v1_decode_split(compressed_input, zero_input, n_8, nbytes_8, output, n_works,
                     orig_each=int(orig_ele_num),
                     padded_n_total=pad_to_block(int(orig_ele_num)) * n_works)


def v1_decompress_split_store_unpad_v(compressed_input, zero_input, n_8, nbytes_8, out_off, orig_n_8,
                                      output, padded_n_total: int, n_works: int) -> None:
    """Per-work valid counts and output offsets
    (reference: hopper_fastzip.cpp:344-367 -> hopper_zip.cu:1332-1487)."""
    _v1_decode_split(compressed_input, zero_input, n_8, nbytes_8, output, n_works, out_off=out_off,
                     orig_n_8=orig_n_8, padded_n_total=int(padded_n_total))


def v1_compress_8(input, n_8, nbytes_8, bases_in, output, output_final, global_zero_counter_8,
                  n_works: int) -> None:
    """Fused-layout encode (reference: hopper_fastzip.cpp:97-126 -> hopper_zip.cu:31-201, 210-293).

    The compacted streams land in ``output_final`` (works back to back, ``nbytes_8[i]`` bytes
    each).  ``output`` needs 4 bytes per padded element, as in the reference; for a single work
    the stream is also left at the start of ``output`` so that ``output`` and ``output_final``
    may be the same buffer.
    """
    _req(input, torch.bfloat16, "input")
    _req(n_8, torch.int32, "n_8", n_works)
    _req(nbytes_8, torch.int32, "nbytes_8", n_works)
    _req(bases_in, torch.int32, "bases_in", 1)
    _req(output, torch.uint8, "output")
    _req(output_final, torch.uint8, "output_final")
    _req(global_zero_counter_8, torch.int32, "global_zero_counter_8", n_works)
    dev = _same_device(input, n_8, nbytes_8, bases_in, output, output_final, global_zero_counter_8)
    total_n = input.numel()
    padded = pad_to_block(total_n)
    if output.numel() < 4 * padded:
        raise ValueError(f"output holds {output.numel()} bytes, needs 4 per padded element ({4 * padded})")
    if dev.type == "cpu":
        same = output.data_ptr() == output_final.data_ptr()
        dst = output_final if (n_works > 1 or same) else output
        _lib.cpu().zc_cpu_v1_encode_fused(
            input.data_ptr(), total_n, n_8.data_ptr(), n_works, int(bases_in[0]), dst.data_ptr(),
            nbytes_8.data_ptr(), global_zero_counter_8.data_ptr())
        if n_works == 1 and not same:
            nb = int(nbytes_8[0])
            if output_final.numel() >= nb:
                output_final[:nb].copy_(output[:nb])
        return
    blocks = padded // ELEMS_PER_BLOCK
    if blocks == 0:
        return
    _lib.check(_lib.cuda().zc_v1_encode_fused(
        input.data_ptr(), total_n, n_8.data_ptr(), n_works, bases_in.data_ptr(), output.data_ptr(),
        output_final.data_ptr(), output_final.numel(), nbytes_8.data_ptr(),
        global_zero_counter_8.data_ptr(), blocks, _lib.stream_ptr(dev)), "zc_v1_encode_fused")


def _v1_decode_fused(compressed_input, n_8, nbytes_8, output, n_works, orig_each=-1,
                     padded_n_total=None) -> None:
    _req(compressed_input, torch.uint8, "compressed_input")
    _req(n_8, torch.int32, "n_8", n_works)
    _req(nbytes_8, torch.int32, "nbytes_8", n_works)
    _req(output, torch.bfloat16, "output")
    dev = _same_device(compressed_input, n_8, nbytes_8, output)
    if dev.type == "cpu":
        _lib.cpu().zc_cpu_v1_decode_fused(compressed_input.data_ptr(), n_8.data_ptr(),
                                          nbytes_8.data_ptr(), n_works, orig_each, output.data_ptr())
        return
    if padded_n_total is None:
        padded_n_total = pad_to_block(output.numel())
    blocks = padded_n_total // ELEMS_PER_BLOCK
    if blocks == 0:
        return
    _lib.check(_lib.cuda().zc_v1_decode_fused(
        compressed_input.data_ptr(), n_8.data_ptr(), nbytes_8.data_ptr(), n_works, orig_each,
        output.data_ptr(), output.numel(), blocks, _lib.stream_ptr(dev)), "zc_v1_decode_fused")


def v1_decompress_8(compressed_input, n_8, nbytes_8, output, n_works: int) -> None:
    """reference: hopper_fastzip.cpp:128-146 -> hopper_zip.cu:733-866."""
    _v1_decode_fused(compressed_input, n_8, nbytes_8, output, n_works)


def v1_decompress_8_unpad(compressed_input, n_8, nbytes_8, output, orig_ele_num: int, n_works: int) -> None:
    """reference: hopper_fastzip.cpp:221-243 -> hopper_zip.cu:874-1013."""
    if output.numel() < orig_ele_num * n_works:
        raise ValueError("output is smaller than orig_ele_num * n_works")
    _v1_decode_fused(compressed_input, n_8, nbytes_8, output, n_works, orig_each=int(orig_ele_num),
                     padded_n_total=pad_to_block(int(orig_ele_num)) * n_works)


def v1_compress_8_padded(input: torch.Tensor, bases_in: torch.Tensor, n_works: int = 1) -> torch.Tensor:
    """Pads to a multiple of 4096 and encodes as one work; returns the whole 4 B/element buffer
    with the stream at its start (reference: hopper_fastzip.cpp:149-186).  The reference reads
    ``n_8`` out of bounds for ``n_works > 1``; only one work is accepted here."""
    if n_works != 1:
        raise ValueError("compress_8_padded encodes a single work (n_works must be 1)")
    _req(input, torch.bfloat16, "input")
    flat = input.reshape(-1)
    padded = pad_to_block(flat.numel())
    dev = flat.device
    n_8 = torch.tensor([padded], dtype=torch.int32, device=dev)
    nbytes_8 = torch.zeros(1, dtype=torch.int32, device=dev)
    gc = torch.zeros(1, dtype=torch.int32, device=dev)
    out = torch.empty(max(padded * 4, 128), dtype=torch.uint8, device=dev)
    if padded:
        v1_compress_8(flat, n_8, nbytes_8, bases_in, out, out, gc, 1)
    return out


def v1_decompress_8_padded(compressed_input: torch.Tensor, orig_numel: int, nbytes_8: torch.Tensor,
                           n_works: int = 1) -> torch.Tensor:
    """reference: hopper_fastzip.cpp:189-215."""
    if n_works != 1:
        raise ValueError("decompress_8_padded decodes a single work (n_works must be 1)")
    dev = compressed_input.device
    padded = pad_to_block(int(orig_numel))
    out = torch.empty(int(orig_numel), dtype=torch.bfloat16, device=dev)
    if padded == 0:
        return out
    n_8 = torch.tensor([padded], dtype=torch.int32, device=dev)
    nb = nbytes_8 if nbytes_8.numel() >= 1 and nbytes_8.dtype == torch.int32 else torch.zeros(
        1, dtype=torch.int32, device=dev)
    _v1_decode_fused(compressed_input, n_8, nb, out, 1, orig_each=int(orig_numel),
                     padded_n_total=padded)
    return out


def v1_base_from_std(x: torch.Tensor, bases_out: torch.Tensor) -> None:
    """bases_out[0] = clamp(floor(log2(max(std(x), 1e-30)) - 5.35 + 127), 0, 255) without a host
    sync (reference: main/zipccl_comm.py:56-64, which runs six ATen kernels for this)."""
    _req(bases_out, torch.int32, "bases_out", 1)
    if x.device.type == "cuda" and x.dtype == torch.bfloat16 and x.is_contiguous():
        _lib.check(_lib.cuda().zc_v1_base_from_std(x.data_ptr(), x.numel(), bases_out.data_ptr(),
                                                   _lib.stream_ptr(x.device)), "zc_v1_base_from_std")
        return
    std = x.float().std() if x.numel() > 1 else torch.zeros((), device=x.device)
    base = torch.floor(torch.log2(std.clamp_min(1e-30)) - 5.35 + 127.0)
    bases_out[:1].copy_(base.clamp_(0, 255).to(torch.int32).reshape(1))


# --------------------------------------------------------------------------------------------
# v2
# --------------------------------------------------------------------------------------------

def v2_num_chunks(numel: int) -> int:
    return (numel + V2_CHUNK - 1) // V2_CHUNK


def v2_encode(x: torch.Tensor, records: torch.Tensor | None = None,
              headers: torch.Tensor | None = None, *, nibble: bool = False):
    """Encode a contiguous bf16 tensor into fixed-stride v2 records plus one uint32 header each.
    ``nibble=True`` writes the records in nibble mode (fixed four code bits packed two per byte,
    window anchored at the chunk's largest exponent: about 7 % larger, much cheaper to code; the
    mode is a property of the stream and must be given to ``v2_decode`` again).

    Returns ``(records[uint8, nc*2048], headers[int32, nc])``.  The bytes that must travel are
    ``v2_wire_bytes(headers)``; the slot stride equals the raw bf16 size, so the staging buffer
    never exceeds the uncompressed tensor."""
    _req(x, torch.bfloat16, "x")
    n = x.numel()
    nc = v2_num_chunks(n)
    dev = x.device
    if records is None:
        records = torch.empty(nc * V2_SLOT, dtype=torch.uint8, device=dev)
    if headers is None:
        headers = torch.empty(nc, dtype=torch.int32, device=dev)
    _req(records, torch.uint8, "records", nc * V2_SLOT)
    _req(headers, torch.int32, "headers", nc)
    if nc == 0:
        return records, headers
    if dev.type == "cpu":
        fn = _lib.cpu().zc_cpu_v2_encode_nibble if nibble else _lib.cpu().zc_cpu_v2_encode
        fn(x.data_ptr(), n, records.data_ptr(), headers.data_ptr())
    else:
        fn = _lib.cuda().zc_v2_encode_nibble if nibble else _lib.cuda().zc_v2_encode
        _lib.check(fn(x.data_ptr(), n, records.data_ptr(), headers.data_ptr(), _lib.stream_ptr(dev)), "zc_v2_encode")
    return records, headers


def v2_decode(records: torch.Tensor, headers: torch.Tensor, numel: int,
              out: torch.Tensor | None = None, *, nibble: bool = False) -> torch.Tensor:
    nc = v2_num_chunks(numel)
    _req(records, torch.uint8, "records", nc * V2_SLOT)
    _req(headers, torch.int32, "headers", nc)
    dev = records.device
    if out is None:
        out = torch.empty(numel, dtype=torch.bfloat16, device=dev)
    _req(out, torch.bfloat16, "out", numel)
    if nc == 0:
        return out
    if dev.type == "cpu":
        fn = _lib.cpu().zc_cpu_v2_decode_nibble if nibble else _lib.cpu().zc_cpu_v2_decode
        fn(records.data_ptr(), headers.data_ptr(), numel, out.data_ptr())
    else:
        fn = _lib.cuda().zc_v2_decode_nibble if nibble else _lib.cuda().zc_v2_decode
        _lib.check(fn(records.data_ptr(), headers.data_ptr(), numel, out.data_ptr(), _lib.stream_ptr(dev)),
                   "zc_v2_decode")
    return out


def v2_record_bytes(headers: torch.Tensor) -> torch.Tensor:
    """Used bytes of every record (int64 tensor), computed from the headers."""
    h = headers.to(torch.int64) & 0xFFFFFFFF
    width = (h >> 8) & 0xF
    nesc = h >> 16
    return torch.where(width == 8, torch.full_like(h, 2048), 1024 + 128 * width + nesc)


def v2_wire_bytes(headers: torch.Tensor) -> int:
    """Bytes on the wire for a v2 stream: used record bytes plus 4 header bytes per chunk."""
    return int(v2_record_bytes(headers).sum().item()) + 4 * headers.numel()


def v2_compact(records: torch.Tensor, headers: torch.Tensor):
    """Dense form for storage or a byte-counted transport: (dense[uint8], offsets[int64, nc+1])."""
    nc = headers.numel()
    sizes = v2_record_bytes(headers)
    offsets = torch.zeros(nc + 1, dtype=torch.int64, device=headers.device)
    offsets[1:] = torch.cumsum(sizes, 0)
    total = int(offsets[-1].item())
    if records.device.type == "cpu":
        dense = torch.empty(total, dtype=torch.uint8)
        offs = torch.empty(nc + 1, dtype=torch.int64)
        _lib.cpu().zc_cpu_v2_compact(records.data_ptr(), headers.data_ptr(), nc, dense.data_ptr(),
                                     offs.data_ptr())
        return dense, offs
    slot = torch.arange(V2_SLOT, device=records.device)
    mask = slot[None, :] < sizes[:, None]
    dense = records.view(nc, V2_SLOT)[mask]
    return dense, offsets


def v2_expand(dense: torch.Tensor, headers: torch.Tensor) -> torch.Tensor:
    nc = headers.numel()
    records = torch.zeros(nc * V2_SLOT, dtype=torch.uint8, device=dense.device)
    if dense.device.type == "cpu":
        _lib.cpu().zc_cpu_v2_expand(dense.data_ptr(), headers.data_ptr(), nc, records.data_ptr())
        return records
    sizes = v2_record_bytes(headers)
    slot = torch.arange(V2_SLOT, device=dense.device)
    mask = slot[None, :] < sizes[:, None]
    records.view(nc, V2_SLOT)[mask] = dense
    return records
