"""Drop-in module with the ten functions of the reference's ``hopper_fastzip2`` extension
(reference: zipccl/hopper_fastzip.cpp:405-424, stubs zipccl/hopper_fastzip2.pyi:13-128).

Same names, argument order and wire format; backed by sm_100a kernels for CUDA tensors and by the
scalar C++ codec for CPU tensors.  ``from zipccl import hopper_fastzip2`` keeps working.
"""
from fsdp_comm_opt_b200.ops.codec import (
    v1_compress_8 as compress_8,
    v1_decompress_8 as decompress_8,
    v1_compress_8_padded as compress_8_padded,
    v1_decompress_8_padded as decompress_8_padded,
    v1_decompress_8_unpad as decompress_8_unpad,
    v1_compress_split_store as _compress_split_store,
    v1_decompress_split_store as decompress_split_store,
    v1_decompress_split_store_unpad as decompress_split_store_unpad,
    v1_decompress_split_store_unpad_v as decompress_split_store_unpad_v,
    v1_compress_split_store_pad as compress_split_store_pad,
)


def compress_split_store(input, n_8, bases_in, output, output1, output_final,
                         global_zero_counter_8, n_works):
    return _compress_split_store(input, n_8, bases_in, output, output1, output_final,
                                 global_zero_counter_8, n_works)


__all__ = [
    "compress_8", "decompress_8", "compress_8_padded", "decompress_8_padded", "decompress_8_unpad",
    "compress_split_store", "decompress_split_store", "decompress_split_store_unpad",
    "decompress_split_store_unpad_v", "compress_split_store_pad",
]
