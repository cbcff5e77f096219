"""Typing stubs for ``zipccl.hopper_fastzip2``: the ten functions of the reference extension
(reference: zipccl/hopper_fastzip.cpp, zipccl/hopper_fastzip2.pyi), implemented by
``fsdp_comm_opt_b200.ops.codec`` on CPU (scalar C++ codec) and CUDA (sm_100a kernels).

Conventions shared by all functions
    * values are ``bfloat16``; every stream / scratch buffer is ``uint8``; ``n_8``, ``nbytes_8``,
      ``orig_n_8``, ``out_off``, ``global_zero_counter_8`` and ``bases_in`` are ``int32`` tensors on the
      same device as the data.
    * a call handles ``n_works`` independent pieces ("works") laid out back to back; ``n_8[i]`` is the
      element count of work ``i`` and must be a multiple of 4096 (``ELEMS_PER_BLOCK``).
    * ``bases_in[0]`` is the base exponent of the 7-value window (elements whose exponent falls
      outside it are outliers and carry their exponent byte verbatim); the tensor has 256 entries
      for compatibility, only the first is read.
    * "deterministic part" of a work of ``n`` elements = sign+mantissa bytes (``n``), three bit planes
      (``3 n / 8``), one int32 offset per 4096-element block plus one word for the base:
      ``det_bytes(n) = n + 3 n / 8 + 4 (n / 4096) + 4``, rounded up to 128 bytes between works.
    * all functions write into caller-provided tensors, run on the current stream and return
      nothing unless stated otherwise; sizes are validated and a ``ValueError`` / ``TypeError`` is
      raised before any kernel is launched.
"""
from torch import Tensor

# --------------------------------------------------------------------------------------------
# fused layout: one stream per work holding the deterministic part followed by its outliers
# --------------------------------------------------------------------------------------------

def compress_8(input: Tensor, n_8: Tensor, nbytes_8: Tensor, bases_in: Tensor, output: Tensor, output_final: Tensor, global_zero_counter_8: Tensor, n_works: int) -> None:
    """Encode ``n_works`` works into one compact stream each (deterministic part, then outliers).

    input: bf16 [sum(n_8)]: the works' values back to back
    n_8: int32 [n_works]: elements per work (multiples of 4096)
    nbytes_8: int32 [n_works], OUT: bytes of each work's stream (128-aligned)
    bases_in: int32 [256]: window base in [0]
    output: uint8 scratch, at least 4 bytes per input element
    output_final: uint8, OUT: the streams, work i at the sum of nbytes_8[:i]
    global_zero_counter_8: int32 [n_works], OUT: outlier count of each work
    """
    ...

def decompress_8(compressed_input: Tensor, n_8: Tensor, nbytes_8: Tensor, output: Tensor, n_works: int) -> None:
    """Inverse of :func:`compress_8`.

    compressed_input: uint8: streams as written by compress_8
    n_8: int32 [n_works]
    nbytes_8: int32 [n_works]: stream sizes from compress_8
    output: bf16 [sum(n_8)], OUT
    """
    ...

def compress_8_padded(input: Tensor, bases_in: Tensor, n_works: int = ...) -> Tensor:
    """Convenience form for one work (``n_works`` must be 1: the reference indexes ``n_8`` out of
    bounds for more): pads ``input`` (any length) to a multiple of 4096 elements, encodes it and
    returns a new uint8 tensor of 4 bytes per padded element with the stream at its start."""
    ...

def decompress_8_padded(compressed_input: Tensor, orig_numel: int, nbytes_8: Tensor, n_works: int = ...) -> Tensor:
    """Inverse of :func:`compress_8_padded`: returns a new bf16 tensor of ``orig_numel`` elements.
    ``nbytes_8`` (int32 [1]) is accepted for signature compatibility; the stream carries its own
    block offsets, so its size is not needed to decode it."""
    ...

def decompress_8_unpad(compressed_input: Tensor, n_8: Tensor, nbytes_8: Tensor, output: Tensor, orig_ele_num: int, n_works: int) -> None:
    """Decode and drop each work's padding: work ``i`` lands at ``output[i * orig_ele_num]``.

    compressed_input: uint8: streams as written by compress_8
    n_8: int32 [n_works]: padded element counts
    nbytes_8: int32 [n_works]
    output: bf16 [n_works * orig_ele_num], OUT: works packed without padding
    orig_ele_num: elements to keep from the start of every work
    """
    ...

# --------------------------------------------------------------------------------------------
# split layout: fixed-size deterministic parts in one tensor, outlier bytes in another, so that
# a gather can move the fixed-size parts first and size the second transfer from the counts
# --------------------------------------------------------------------------------------------

def compress_split_store(input: Tensor, n_8: Tensor, bases_in: Tensor, output: Tensor, output1: Tensor, output_final: Tensor, global_zero_counter_8: Tensor, n_works: int) -> None:
    """Encode into the split layout.

    input: bf16 [sum(n_8)]
    n_8: int32 [n_works]
    bases_in: int32 [256]
    output: uint8, OUT: deterministic parts, work i at sum(align128(det_bytes(n_8[:i])))
    output1: uint8 scratch, one byte per input element
    output_final: uint8, OUT: outlier bytes, work i at sum(align128(count[:i]))
    global_zero_counter_8: int32 [n_works], OUT: outlier count of each work
    """
    ...

def decompress_split_store(compressed_input: Tensor, zero_input: Tensor, n_8: Tensor, nbytes_8: Tensor, output: Tensor, n_works: int) -> None:
    """Inverse of :func:`compress_split_store`.

    compressed_input: uint8: deterministic parts
    zero_input: uint8: outlier bytes, work i at sum(align128(nbytes_8[:i]))
    n_8: int32 [n_works]
    nbytes_8: int32 [n_works]: outlier bytes (or the stride) of each work
    output: bf16 [sum(n_8)], OUT
    """
    ...

def decompress_split_store_unpad(compressed_input: Tensor, zero_input: Tensor, n_8: Tensor, nbytes_8: Tensor, output: Tensor, orig_ele_num: int, n_works: int) -> None:
    """Split-layout decode that drops the padding of every work (the all-gather's receive side: work
    ``i`` is rank ``i``'s shard and lands at ``output[i * orig_ele_num]``; any alignment of the
    destination is accepted).

    output: bf16 [n_works * orig_ele_num], OUT
    orig_ele_num: elements to keep from the start of every work
    """
    ...

def decompress_split_store_unpad_v(compressed_input: Tensor, zero_input: Tensor, n_8: Tensor, nbytes_8: Tensor, out_off: Tensor, orig_n_8: Tensor, output: Tensor, padded_n_total: int, n_works: int) -> None:
    """Variable form of :func:`decompress_split_store_unpad`: every work has its own kept length and
    its own destination offset.

    out_off: int32 [n_works]: element offset of work i in `output`
    orig_n_8: int32 [n_works]: elements to keep from work i
    output: bf16, OUT
    padded_n_total: sum of n_8 (host-side copy, sizes the launch without a device read)
    """
    ...

def compress_split_store_pad(input: Tensor, n_8: Tensor, orig_n_8: Tensor, bases_in: Tensor, output: Tensor, output1: Tensor, output_final: Tensor, global_zero_counter_8: Tensor, padded_n_total: int, n_works: int) -> None:
    """Split-layout encode of works whose lengths are not multiples of 4096: the padding is supplied
    by the encoder instead of a padded copy of the input.

    input: bf16 [sum(orig_n_8)]: the works' unpadded values back to back
    n_8: int32 [n_works]: padded element counts (multiples of 4096)
    orig_n_8: int32 [n_works]: real element counts; the rest encodes as zeros
    padded_n_total: sum of n_8 (host-side copy)
    """
    ...
