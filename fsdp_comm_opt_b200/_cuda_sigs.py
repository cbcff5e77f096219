"""ctypes prototypes of the C launchers exported by ``libzc_cuda.so`` (see ``csrc/*.cu``).

Every launcher takes raw device pointers plus a CUDA stream and returns 0 on success, a negative
library code (-1 bad argument, -2 unsupported shape) or a positive ``cudaError_t``.
"""
from ctypes import c_float, c_int, c_int64, c_void_p

P, I, L, F = c_void_p, c_int, c_int64, c_float


def _sig(lib, name, *argtypes):
    fn = getattr(lib, name, None)
    if fn is None:
        return
    fn.restype = I
    fn.argtypes = list(argtypes)


def declare(lib) -> None:
    # codec
    _sig(lib, "zc_v2_encode", P, L, P, P, P)
    _sig(lib, "zc_v2_decode", P, P, L, P, P)
    _sig(lib, "zc_v2_encode_nibble", P, L, P, P, P)
    _sig(lib, "zc_v2_decode_nibble", P, P, L, P, P)
    _sig(lib, "zc_v2_decode_ctas", P, P, L, P, I, P)
    _sig(lib, "zc_v1_encode_split", P, L, P, P, I, P, P, P, P, P, L, P)
    _sig(lib, "zc_v1_encode_fused", P, L, P, I, P, P, P, L, P, P, L, P)
    _sig(lib, "zc_v1_decode_split", P, P, P, P, I, L, P, P, P, L, L, P)
    _sig(lib, "zc_v1_decode_fused", P, P, P, I, L, P, L, L, P)
    _sig(lib, "zc_v1_base_from_std", P, L, P, P)
    # elementwise / optimizer
    _sig(lib, "zc_rmsnorm_fwd", P, P, P, P, P, P, L, I, F, P)
    _sig(lib, "zc_rmsnorm_bwd", P, P, P, P, P, P, P, P, L, I, P)
    _sig(lib, "zc_rmsnorm_bwd_ctas", L)
    _sig(lib, "zc_layernorm_fwd", P, P, P, P, P, P, P, P, L, I, F, P)
    _sig(lib, "zc_layernorm_bwd_ctas", L)
    _sig(lib, "zc_layernorm_bwd", P, P, P, P, P, P, P, P, P, I, I, I, P, L, I, P)
    _sig(lib, "zc_bf16_column_sum_blocks", L)
    _sig(lib, "zc_bf16_column_sum", P, L, I, L, P, I, I, P, P)
    _sig(lib, "zc_bias_gelu_fwd", P, P, P, L, I, P)
    _sig(lib, "zc_bias_gelu_bwd", P, P, P, P, L, I, P)
    _sig(lib, "zc_rope_inplace", P, P, P, L, I, I, I, I, F, P)
    _sig(lib, "zc_swiglu_fwd", P, P, L, I, P)
    _sig(lib, "zc_swiglu_bwd", P, P, P, L, I, P)
    _sig(lib, "zc_ce_fwd_bwd", P, P, P, P, L, I, I, P)
    _sig(lib, "zc_ce_fwd_bwd_ld", P, P, P, P, L, I, L, I, P)
    _sig(lib, "zc_quant_int8", P, L, I, P, P)
    _sig(lib, "zc_dequant_int8", P, L, I, L, I, P, P)
    _sig(lib, "zc_adamw", P, P, P, P, L, I, I, I, F, F, F, F, F, F, F, I, P)
    _sig(lib, "zc_adamw_guarded", P, P, P, P, L, I, I, I, F, F, F, F, F, F, F, I, P, P)
    _sig(lib, "zc_health_read_and_clear")
    _sig(lib, "zc_health_set", I)
    if hasattr(lib, "zc_health_word"):
        lib.zc_health_word.restype = P
        lib.zc_health_word.argtypes = []
    # tensor cores
    _sig(lib, "zc_umma_selftest", P, P, P, I, I, I, P, P)
    _sig(lib, "zc_attn_fwd", P, P, P, P, P, I, I, I, I, I, L, L, L, L, L, L, L, L, L, F, P)
    _sig(lib, "zc_attn_bwd", P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, *([L] * 18), F, P)
    _sig(lib, "zc_attn_status_read_and_clear")
    _sig(lib, "zc_attn_fwd_ws", P, P, P, P, P, I, I, I, I, I, L, L, L, L, L, L, L, L, L, F, P)
    _sig(lib, "zc_attn_ws_status_read_and_clear")
    _sig(lib, "zc_attn_bwd_ws", P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, *([L] * 18), F, P)
    _sig(lib, "zc_attn_bwd_ws_status_read_and_clear")
    _sig(lib, "zc_attn_fwd_2q", P, P, P, P, P, I, I, I, I, I, L, L, L, L, L, L, L, L, L, F, P)
    _sig(lib, "zc_attn_fwd_2q_status_read_and_clear")
    _sig(lib, "zc_attn_bwd_kt", P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, *([L] * 18), F, P)
    _sig(lib, "zc_gemm_bf16", P, P, P, L, L, L, I, I, I, P)
    _sig(lib, "zc_gemm_bf16_2sm", P, P, P, L, L, L, I, I, I, P)
    _sig(lib, "zc_gemm_bf16_2sm_ld", P, P, P, L, L, L, L, L, L, I, I, I, P)
    _sig(lib, "zc_gemm_bf16_2sm_bias", P, P, P, P, L, L, L, L, L, L, I, I, I, P)
    _sig(lib, "zc_gemm_status_read_and_clear")
    # fused collectives
    from ctypes import c_double, c_uint

    _sig(lib, "zc_symm_all_gather", P, P, P, P, P, L, I, I, L, c_uint, I, I, c_double, I, P)
    _sig(lib, "zc_symm_all_gather_int8", P, P, P, P, P, L, I, I, L, c_uint, I, I, c_double, P)
    _sig(lib, "zc_symm_reduce_scatter", P, P, P, P, P, L, I, I, L, c_uint, I, I, F, I, I, c_double, I, P)
