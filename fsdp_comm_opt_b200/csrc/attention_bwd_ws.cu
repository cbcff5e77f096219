// Causal GQA attention backward for sm_100a.  Two kernels: the warp-specialised kernel below (head
// dimension 64, and 128 with ZC_ATTN_BWD=ws) and, further down, the key-row kernel that is the default
// for head dimension 128.
//
// One CTA (320 threads) per (128-key block, kv head, batch); it loops over the query heads of the
// group and over the query blocks at or below the diagonal, with dK and dV accumulating in TMEM.
//   warp 0      TMA producer: K, V once; then Q_i and dO_i per iteration (4-D tensor maps,
//               SWIZZLE_128B, zero fill past S).  The next iteration's loads start as soon as the
//               MMAs that read the buffers have completed, and overlap the dQ reduction below.
//   warp 1      MMA issuer: S = Q K^T and dP = dO V^T, then dV += P^T dO, dK += dS^T Q and
//               dQ_i = dS K (P / dS are read through MN-major descriptors: no transposes)
//   warps 2-9   256 compute threads: two threads share a query row and take 64 columns each;
//               P = exp2(S*c - lse), dS = P (dP - delta) scale, written to smem as bf16; then the
//               dQ_i tile is read from TMEM and reduced into the fp32 accumulator with red.add
// TMEM (512 columns): dK | dV | R0 (S, later dQ_i) | R1 (dP).  Shared memory: K V Q dO P dS, 32 KB
// each.  Every wait is bounded; a timed-out role raises a CTA-wide abort flag.
#include <cuda.h>
#include <cuda_bf16.h>
#include <math_constants.h>

#include <cstdio>
#include <type_traits>

#include "launch_util.h"
#include "umma.cuh"

namespace zc {
namespace bws {
using namespace umma;

constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2,
                                            int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}
// global[tile at (c0..c3)] += smem tile  (element-wise fp32 add done by the TMA unit; rows past the
// tensor's extent are clipped)
__device__ __forceinline__ void tma_reduce_add_4d(const CUtensorMap* map, const void* src, int c0, int c1, int c2,
                                                  int c3) {
  asm volatile(
      "cp.reduce.async.bulk.tensor.4d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
      ::"l"(map), "r"(smem_u32(src)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void bulk_commit_and_wait_read() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
__device__ __forceinline__ uint64_t desc_k(uint32_t base, int k) {
  return smem_desc(base + (k >> 2) * 16384 + (k & 3) * 32, 16, 1024);
}
__device__ __forceinline__ uint64_t desc_mn(uint32_t base, int k) { return smem_desc(base + k * 2048, 16384, 1024); }

__device__ __forceinline__ void store_chunk32(uint8_t* tile, int row, int col0, const float (&v)[32]) {
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const int col = col0 + q * 8;
    __nv_bfloat162 a = __floats2bfloat162_rn(v[q * 8 + 0], v[q * 8 + 1]);
    __nv_bfloat162 b = __floats2bfloat162_rn(v[q * 8 + 2], v[q * 8 + 3]);
    __nv_bfloat162 c = __floats2bfloat162_rn(v[q * 8 + 4], v[q * 8 + 5]);
    __nv_bfloat162 d = __floats2bfloat162_rn(v[q * 8 + 6], v[q * 8 + 7]);
    uint4 u;
    u.x = *reinterpret_cast<uint32_t*>(&a);
    u.y = *reinterpret_cast<uint32_t*>(&b);
    u.z = *reinterpret_cast<uint32_t*>(&c);
    u.w = *reinterpret_cast<uint32_t*>(&d);
    *reinterpret_cast<uint4*>(tile + (col >> 6) * 16384 + sw128_off(row, (col >> 3) & 7)) = u;
  }
}

struct BwdParams {
  const float *lse, *delta;
  float* dq_acc;
  __nv_bfloat16 *dk, *dv;
  int B, S, Hq, Hkv;
  int64_t dks0, dks1, dks2, dvs0, dvs1, dvs2;
  float scale;
  int* status;
  long long* trace;  // null, or [3][256][8] SM-clock stamps written by CTA 0 of the key-row kernel
};

template <int D>
__global__ void __launch_bounds__(320, 1) attn_bwd_ws_kernel(const __grid_constant__ CUtensorMap mapQ,
                                                             const __grid_constant__ CUtensorMap mapK,
                                                             const __grid_constant__ CUtensorMap mapV,
                                                             const __grid_constant__ CUtensorMap mapdO,
                                                             const __grid_constant__ CUtensorMap mapdQ,
                                                             const BwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int TILE = 128 * D * 2;
  constexpr int SLABS = D / 64;
  uint8_t* sK = smem;
  uint8_t* sV = smem + 1 * 32768;
  uint8_t* sQ = smem + 2 * 32768;
  uint8_t* sdO = smem + 3 * 32768;
  uint8_t* sP = smem + 4 * 32768;
  uint8_t* sdS = smem + 5 * 32768;
  __shared__ uint64_t kv_full, qdo_full, qdo_empty, sdp_full, pds_full, dq_full, dq_empty;
  __shared__ uint32_t tmem_base;
  __shared__ volatile int s_abort;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nkb = gridDim.x;
  const int jb = blockIdx.x;
  const int hk = blockIdx.y, b = blockIdx.z;
  const int group = p.Hq / p.Hkv;
  const int k0 = jb * 128;
  const int iters = group * (nkb - jb);
  if (tid == 0) {
    mbar_init(&kv_full, 1);
    mbar_init(&qdo_full, 1);
    mbar_init(&qdo_empty, 1);
    mbar_init(&sdp_full, 1);
    mbar_init(&pds_full, 1);
    mbar_init(&dq_full, 1);
    mbar_init(&dq_empty, 1);
    mbar_fence_init();
    s_abort = 0;
  }
  if (warp == 1) {
    tmem_alloc(&tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tm_dk = tmem_base, tm_dv = tmem_base + 128, tm_r0 = tmem_base + 256, tm_r1 = tmem_base + 384;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(&kv_full, 2 * TILE);
#pragma unroll
      for (int sl = 0; sl < SLABS; ++sl) {
        tma_load_4d(sK + sl * 16384, &mapK, &kv_full, sl * 64, hk, k0, b);
        tma_load_4d(sV + sl * 16384, &mapV, &kv_full, sl * 64, hk, k0, b);
      }
      for (int it = 0; it < iters; ++it) {
        const int h = hk * group + it / (nkb - jb);
        const int q0 = (jb + it % (nkb - jb)) * 128;
        if (!mbar_wait_relaxed(&qdo_empty, (it & 1) ^ 1)) { s_abort = 1; break; }
        mbar_expect_tx(&qdo_full, 2 * TILE);
#pragma unroll
        for (int sl = 0; sl < SLABS; ++sl) {
          tma_load_4d(sQ + sl * 16384, &mapQ, &qdo_full, sl * 64, h, q0, b);
          tma_load_4d(sdO + sl * 16384, &mapdO, &qdo_full, sl * 64, h, q0, b);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t id_s = idesc_bf16(128, 128, MAJOR_K, MAJOR_K);
      const uint32_t id_kv = idesc_bf16(128, D, MAJOR_MN, MAJOR_MN);
      const uint32_t id_dq = idesc_bf16(128, D, MAJOR_K, MAJOR_MN);
      const uint32_t aK = smem_u32(sK), aV = smem_u32(sV), aQ = smem_u32(sQ), adO = smem_u32(sdO), aP = smem_u32(sP),
                     adS = smem_u32(sdS);
      bool ok = mbar_wait_relaxed(&kv_full, 0);
      for (int it = 0; it < iters && ok; ++it) {
        if (!(ok = mbar_wait_relaxed(&qdo_full, it & 1))) break;
        if (!(ok = mbar_wait_relaxed(&dq_empty, (it & 1) ^ 1))) break;
        tc_fence_after_sync();
#pragma unroll
        for (int k = 0; k < D / 16; ++k) mma_bf16(tm_r0, desc_k(aQ, k), desc_k(aK, k), id_s, k != 0);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) mma_bf16(tm_r1, desc_k(adO, k), desc_k(aV, k), id_s, k != 0);
        mma_commit(&sdp_full);
        if (!(ok = mbar_wait_relaxed(&pds_full, it & 1))) break;
        tc_fence_after_sync();
#pragma unroll
        for (int k = 0; k < 8; ++k) mma_bf16(tm_dv, desc_mn(aP, k), desc_mn(adO, k), id_kv, (it | k) != 0);
#pragma unroll
        for (int k = 0; k < 8; ++k) mma_bf16(tm_dk, desc_mn(adS, k), desc_mn(aQ, k), id_kv, (it | k) != 0);
#pragma unroll
        for (int k = 0; k < 8; ++k) mma_bf16(tm_r0, desc_k(adS, k), desc_mn(aK, k), id_dq, k != 0);
        mma_commit(&dq_full);
        mma_commit(&qdo_empty);
      }
      if (!ok) s_abort = 1;
    }
  } else {
    const int cw = warp - 2;
    const int quarter = warp & 3;
    const int half = cw >> 2;
    const int r = quarter * 32 + lane;
    const uint32_t lane_base = (uint32_t)(quarter * 32);
    const float sl2 = p.scale * LOG2E;
    for (int it = 0; it < iters; ++it) {
      const int h = hk * group + it / (nkb - jb);
      const int ib = jb + it % (nkb - jb);
      const int q0 = ib * 128;
      const int row = q0 + r;
      float lse2 = 0.f, dl = 0.f;
      if (row < p.S) {
        lse2 = __ldg(p.lse + ((int64_t)b * p.Hq + h) * p.S + row) * LOG2E;
        dl = __ldg(p.delta + ((int64_t)b * p.Hq + h) * p.S + row);
      }
      if (!mbar_wait(&sdp_full, it & 1)) s_abort = 1;
      tc_fence_after_sync();
      const bool diag = (ib == jb) || (q0 + 128 > p.S) || (k0 + 128 > p.S);
#pragma unroll 1
      for (int c = half * 64; c < half * 64 + 64; c += 32) {
        uint32_t rs[32], rp[32];
        tmem_ld32(tmem_addr(tm_r0, lane_base, c), rs);
        tmem_ld32(tmem_addr(tm_r1, lane_base, c), rp);
        tmem_ld_wait();
        float pv[32], ds[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float e = exp2f(__uint_as_float(rs[i]) * sl2 - lse2);
          if (diag && (k0 + c + i > row || k0 + c + i >= p.S || row >= p.S)) e = 0.f;
          pv[i] = e;
          ds[i] = e * (__uint_as_float(rp[i]) - dl) * p.scale;
        }
        store_chunk32(sP, r, c, pv);
        store_chunk32(sdS, r, c, ds);
      }
      fence_proxy_async_smem();
      tc_fence_before_sync();
      named_bar_sync(1, 256);
      if (s_abort) break;
      if (tid == 64) mbar_arrive(&pds_full);
      // ---- dQ_i partial: this thread reduces its row's columns [half*D/2, half*D/2 + D/2) ---------
      if (!mbar_wait(&dq_full, it & 1)) s_abort = 1;
      tc_fence_after_sync();
      // The dV/dK/dQ MMAs have finished reading P and dS, so their 64 KB of shared memory are
      // free: stage the fp32 dQ_i tile there (32-column slabs, 128B swizzle) and let one thread add
      // it into the global accumulator with bulk tensor reductions instead of 4096 red.add per CTA.
#pragma unroll 1
      for (int c = half * (D / 2); c < half * (D / 2) + D / 2; c += 32) {
        uint32_t rr[32];
        tmem_ld32(tmem_addr(tm_r0, lane_base, c), rr);
        tmem_ld_wait();
        uint8_t* slab = sP + (c >> 5) * 16384;
#pragma unroll
        for (int i = 0; i < 8; ++i)
          *reinterpret_cast<uint4*>(slab + sw128_off(r, i)) =
              make_uint4(rr[4 * i], rr[4 * i + 1], rr[4 * i + 2], rr[4 * i + 3]);
      }
      fence_proxy_async_smem();
      tc_fence_before_sync();
      named_bar_sync(1, 256);
      if (s_abort) break;
      if (tid == 64) {
#pragma unroll
        for (int t = 0; t < D / 32; ++t) tma_reduce_add_4d(&mapdQ, sP + t * 16384, t * 32, h, q0, b);
        bulk_commit_and_wait_read();
        mbar_arrive(&dq_empty);
      }
    }
    if (!s_abort) {
      // all MMAs into dK / dV have completed (dq_full of the last iteration covers them)
      const int krow = k0 + r;
#pragma unroll 1
      for (int which = 0; which < 2; ++which) {
        const uint32_t tmx = which ? tm_dv : tm_dk;
        __nv_bfloat16* dst = which ? p.dv + b * p.dvs0 + (int64_t)krow * p.dvs1 + hk * p.dvs2
                                   : p.dk + b * p.dks0 + (int64_t)krow * p.dks1 + hk * p.dks2;
#pragma unroll 1
        for (int c = half * (D / 2); c < half * (D / 2) + D / 2; c += 32) {
          uint32_t rr[32];
          tmem_ld32(tmem_addr(tmx, lane_base, c), rr);
          tmem_ld_wait();
          if (krow < p.S) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              __nv_bfloat162 a0 = __floats2bfloat162_rn(__uint_as_float(rr[i]), __uint_as_float(rr[i + 1]));
              __nv_bfloat162 a1 = __floats2bfloat162_rn(__uint_as_float(rr[i + 2]), __uint_as_float(rr[i + 3]));
              __nv_bfloat162 a2 = __floats2bfloat162_rn(__uint_as_float(rr[i + 4]), __uint_as_float(rr[i + 5]));
              __nv_bfloat162 a3 = __floats2bfloat162_rn(__uint_as_float(rr[i + 6]), __uint_as_float(rr[i + 7]));
              uint4 u;
              u.x = *reinterpret_cast<uint32_t*>(&a0);
              u.y = *reinterpret_cast<uint32_t*>(&a1);
              u.z = *reinterpret_cast<uint32_t*>(&a2);
              u.w = *reinterpret_cast<uint32_t*>(&a3);
              *reinterpret_cast<uint4*>(dst + c + i) = u;
            }
          }
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (tid == 0 && s_abort) atomicExch(p.status, 5);
  if (warp == 1) tmem_dealloc(tmem_base, 512);
}

typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                             const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                             CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeFn encode_fn() {
  static EncodeFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeFn>(ptr);
  }
  return fn;
}
// bf16 [B, S, H, D] with element strides (s_b, s_s, s_h), viewed as (D, H, S, B); box = one 64-wide
// slab of `rows` sequence positions of one head
static bool make_map4(CUtensorMap* m, const void* base, int D, int H, int S, int B, int64_t s_b, int64_t s_s,
                      int64_t s_h, int rows = 128) {
  EncodeFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)H, (cuuint64_t)S, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)s_h * 2, (cuuint64_t)s_s * 2, (cuuint64_t)s_b * 2};
  cuuint32_t box[4] = {64, 1, (cuuint32_t)rows, 1};
  cuuint32_t el[4] = {1, 1, 1, 1};
  const CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, el,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    fprintf(stderr, "[zc_attn_bwd] cuTensorMapEncodeTiled failed (%d): base=%p D=%d H=%d S=%d B=%d\n", (int)r, base, D,
            H, S, B);
  return r == CUDA_SUCCESS;
}

// fp32 accumulator [B, S, Hq, D] viewed as (D, Hq, S, B); box = 32 columns x `rows` rows of one head
static bool make_map4_f32(CUtensorMap* m, const void* base, int D, int H, int S, int B, int rows = 128,
                          bool swizzle = true) {
  EncodeFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)H, (cuuint64_t)S, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)D * 4, (cuuint64_t)H * D * 4, (cuuint64_t)S * H * D * 4};
  cuuint32_t box[4] = {32, 1, (cuuint32_t)rows, 1};
  cuuint32_t el[4] = {1, 1, 1, 1};
  const CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<void*>(base), dims, strides, box, el,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                        CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) fprintf(stderr, "[zc_attn_bwd] fp32 tensor map failed (%d)\n", (int)r);
  return r == CUDA_SUCCESS;
}

struct Scratch {
  int* status = nullptr;
  float* dq_acc = nullptr;
  size_t dq_bytes = 0;
};
static Scratch g_scratch[64];
static long long* g_trace = nullptr;

__global__ void __launch_bounds__(256) delta_kernel(const __nv_bfloat16* __restrict__ o,
                                                    const __nv_bfloat16* __restrict__ dout, float* __restrict__ delta,
                                                    int B, int S, int Hq, int D) {
  const int64_t wid = ((int64_t)blockIdx.x * 256 + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int64_t total = (int64_t)B * S * Hq;
  if (wid >= total) return;
  const __nv_bfloat16* po = o + wid * D;
  const __nv_bfloat16* pd = dout + wid * D;
  float acc = 0.f;
  for (int i = lane * 2; i < D; i += 64) {
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(po + i));
    const float2 g = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(pd + i));
    acc += a.x * g.x + a.y * g.y;
  }
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
  if (lane == 0) {
    const int64_t bs = wid / Hq;
    const int hh = (int)(wid % Hq);
    delta[((bs / S) * Hq + hh) * S + bs % S] = acc;
  }
}

__global__ void __launch_bounds__(256) dq_convert_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dq,
                                                         int64_t rows, int Hq, int D, int64_t s_bs, int64_t s_h) {
  const int vpr = D / 4;
  const int64_t total = rows * Hq * vpr;
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < total; i += (int64_t)gridDim.x * 256) {
    const int v = (int)(i % vpr);
    const int h = (int)((i / vpr) % Hq);
    const int64_t r = i / ((int64_t)vpr * Hq);
    const float4 f = *reinterpret_cast<const float4*>(acc + (r * Hq + h) * D + v * 4);
    __nv_bfloat162 a = __floats2bfloat162_rn(f.x, f.y), c = __floats2bfloat162_rn(f.z, f.w);
    uint2 u;
    u.x = *reinterpret_cast<uint32_t*>(&a);
    u.y = *reinterpret_cast<uint32_t*>(&c);
    *reinterpret_cast<uint2*>(dq + r * s_bs + h * s_h + v * 4) = u;
  }
}

// fp32 accumulator kept transposed, [B, H, D, Sp] (queries contiguous, Sp = S rounded up to 4 so
// that every stride is a multiple of 16 bytes), viewed as (S, D, H, B); box = 32 queries x 128 dims
static bool make_map_dq_t(CUtensorMap* m, const void* base, int D, int H, int S, int Sp, int B) {
  EncodeFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[4] = {(cuuint64_t)S, (cuuint64_t)D, (cuuint64_t)H, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)Sp * 4, (cuuint64_t)D * Sp * 4, (cuuint64_t)H * D * Sp * 4};
  cuuint32_t box[4] = {32, (cuuint32_t)D, 1, 1};
  cuuint32_t el[4] = {1, 1, 1, 1};
  const CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<void*>(base), dims, strides, box, el,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) fprintf(stderr, "[zc_attn_bwd] transposed fp32 tensor map failed (%d)\n", (int)r);
  return r == CUDA_SUCCESS;
}

// acc [B, H, D, Sp] fp32 -> dq [B, S, H, D] bf16 (element strides s_b, s_s, s_h): tiles of 32 queries
// x 64 dims transposed through shared memory (128-byte rows on both sides);
// grid (ceil(S/32), D/64, B*H), block (32, 8)
__global__ void __launch_bounds__(256) dq_convert_t_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dq,
                                                           int S, int Sp, int H, int D, int64_t s_b, int64_t s_s,
                                                           int64_t s_h) {
  __shared__ float tile[64][33];
  const int q0 = blockIdx.x * 32, d0 = blockIdx.y * 64;
  const int b = blockIdx.z / H, h = blockIdx.z % H;
  const float* src = acc + ((int64_t)blockIdx.z * D + d0) * Sp + q0;
  const bool qok = q0 + (int)threadIdx.x < S;
#pragma unroll
  for (int dy = threadIdx.y; dy < 64; dy += 8) tile[dy][threadIdx.x] = qok ? src[(int64_t)dy * Sp + threadIdx.x] : 0.f;
  __syncthreads();
#pragma unroll
  for (int qy = threadIdx.y; qy < 32; qy += 8) {
    if (q0 + qy < S) {
      const __nv_bfloat162 v = __floats2bfloat162_rn(tile[2 * threadIdx.x][qy], tile[2 * threadIdx.x + 1][qy]);
      *reinterpret_cast<__nv_bfloat162*>(dq + b * s_b + (int64_t)(q0 + qy) * s_s + h * s_h + d0 + 2 * threadIdx.x) = v;
    }
  }
}

}  // namespace bws

// =================================================================================================
// Key-row ("transposed") backward for head dimension 128: the default.
//
// The kernel above keeps one Q/dO tile in flight and spends most of an iteration waiting (loads,
// then MMAs, then the element-wise pass, then the dQ drain, one after the other).  This one works on
// 64 queries per iteration and computes everything with the KEY index on the TMEM lane axis:
//   S^T  = K  Q^T   (128 keys x 64 queries)        dP^T = V dO^T
//   P^T  = exp2(S^T c - lse[q]),  dS^T = P^T (dP^T - delta[q]) scale      (bf16, K-major A tiles)
//   dV  += P^T dO,  dK += dS^T Q                   (accumulate in TMEM over all iterations)
//   dQ^T = K^T dS^T (128 dims x 64 queries)        -> staged in shared memory as it is and added by
//                                                     bulk tensor reductions to an fp32 accumulator
//                                                     that is kept transposed ([B, Hq, D, S])
// so a 64-query tile is half the size (two Q/dO stages, two P^T/dS^T stages and the dQ staging
// buffer fit beside K and V in 224 KB) and no operand needs a transpose.  The S^T/dP^T accumulators
// are read into registers at once and released before the arithmetic, so the tensor core computes
// iteration i+1's scores during iteration i's element-wise pass, and iteration i's dQ^T is drained
// while iteration i+1's MMAs run.
// TMEM (512 columns): dK 128 | dV 128 | S^T 64 | dP^T 64 | dQ^T 2 x 64.
// CTAs are numbered heaviest first (key block 0 has the most query blocks below the diagonal).
namespace bkt {
using namespace bws;

// Phase stamps for kernel development: compiled in only with -DZC_PHASE_TRACE
#ifdef ZC_PHASE_TRACE
#define ZC_BTRACE(slot, i, k)                                                                      \
  do {                                                                                             \
    if (p.trace && blockIdx.x == 0 && (i) < 256) p.trace[((slot) * 256 + (i)) * 8 + (k)] = clock64(); \
  } while (0)
#else
#define ZC_BTRACE(slot, i, k) \
  do {                        \
  } while (0)
#endif

constexpr int QB = 64;  // queries per iteration

// barrier over `nthreads` threads that also ORs a predicate: every participant gets the same answer,
// so all compute threads leave the loop at the same barrier when one of them timed out
__device__ __forceinline__ bool named_bar_or(int id, int nthreads, bool pred) {
  uint32_t r;
  asm volatile(
      "{\n"
      ".reg .pred p, q;\n"
      "setp.ne.u32 p, %3, 0;\n"
      "bar.red.or.pred q, %1, %2, p;\n"
      "selp.u32 %0, 1, 0, q;\n"
      "}\n"
      : "=r"(r)
      : "r"(id), "r"(nthreads), "r"((uint32_t)pred)
      : "memory");
  return r != 0;
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait0() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

__global__ void __launch_bounds__(352, 1) attn_bwd_kt_kernel(const __grid_constant__ CUtensorMap mapQ,
                                                             const __grid_constant__ CUtensorMap mapK,
                                                             const __grid_constant__ CUtensorMap mapV,
                                                             const __grid_constant__ CUtensorMap mapdO,
                                                             const __grid_constant__ CUtensorMap mapdQ,
                                                             const BwdParams p, const int nkb) {
  constexpr int D = 128;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;                 // [128 keys x 128] bf16, two 64-column slabs of 16 KB
  uint8_t* sV = smem + 32768;
  uint8_t* sQ = smem + 65536;         // 2 stages x [64 queries x 128], two slabs of 8 KB each
  uint8_t* sdO = smem + 98304;        // 2 stages
  uint8_t* sP = smem + 131072;        // 2 stages x [128 keys x 64 queries] bf16 (one slab)
  uint8_t* sdS = smem + 163840;       // 2 stages
  uint8_t* sStage = smem + 196608;    // dQ staging: per query half, [128 dims x 32 queries] fp32, swizzled
  __shared__ uint64_t kv_full, qdo_full[2], qdo_empty[2], sdp_full, sdp_empty, pds_full[2], pds_empty[2], dq_full[2],
      dq_empty[2];
  __shared__ uint32_t tmem_base;
  __shared__ volatile int s_abort;
  __shared__ __align__(16) float s_stat[2][128];  // per stage: lse * log2(e) of the 64 queries, then their delta * scale
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int per_jb = p.Hkv * p.B;
  const int jb = blockIdx.x / per_jb;
  const int hk = (blockIdx.x % per_jb) % p.Hkv, b = (blockIdx.x % per_jb) / p.Hkv;
  const int group = p.Hq / p.Hkv;
  const int k0 = jb * 128;
  const int nq64 = (p.S + QB - 1) / QB;
  const int nqi = nq64 - 2 * jb;  // query blocks at or below this key block's diagonal
  const int iters = group * nqi;
  (void)nkb;
  if (tid == 0) {
    mbar_init(&kv_full, 1);
    mbar_init(&sdp_full, 1);
    mbar_init(&sdp_empty, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&qdo_full[i], 1);
      mbar_init(&qdo_empty[i], 1);
      mbar_init(&pds_full[i], 1);
      mbar_init(&pds_empty[i], 1);
      mbar_init(&dq_full[i], 1);
      mbar_init(&dq_empty[i], 1);
    }
    mbar_fence_init();
    s_abort = 0;
  }
  if (warp == 1) {
    tmem_alloc(&tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tm_dk = tmem_base, tm_dv = tmem_base + 128, tm_st = tmem_base + 256, tm_dp = tmem_base + 320,
                 tm_dq = tmem_base + 384;

  // bounded wait of the single-thread roles: parked in hardware, woken when the phase completes,
  // given up after two seconds or when another role raised the abort flag
  auto role_wait = [&](uint64_t* bar, uint32_t parity) -> bool { return mbar_wait_parked(bar, parity, &s_abort); };

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(&kv_full, 2 * 32768);
#pragma unroll
      for (int sl = 0; sl < 2; ++sl) {
        tma_load_4d(sK + sl * 16384, &mapK, &kv_full, sl * 64, hk, k0, b);
        tma_load_4d(sV + sl * 16384, &mapV, &kv_full, sl * 64, hk, k0, b);
      }
      int h = hk * group, ib = 2 * jb;
      for (int i = 0; i < iters; ++i) {
        const int st = i & 1;
        const int q0 = ib * QB;
        if (!role_wait(&qdo_empty[st], ((i >> 1) & 1) ^ 1)) { s_abort = 1; break; }
        mbar_expect_tx(&qdo_full[st], 2 * 16384);
#pragma unroll
        for (int sl = 0; sl < 2; ++sl) {
          tma_load_4d(sQ + st * 16384 + sl * 8192, &mapQ, &qdo_full[st], sl * 64, h, q0, b);
          tma_load_4d(sdO + st * 16384 + sl * 8192, &mapdO, &qdo_full[st], sl * 64, h, q0, b);
        }
        if (++ib == nq64) { ib = 2 * jb; ++h; }
      }
    }
  } else if (warp == 1 || warp == 10) {
    if (lane == 0) {
      const uint32_t id_st = idesc_bf16(128, QB, MAJOR_K, MAJOR_K);     // S^T, dP^T
      const uint32_t id_kv = idesc_bf16(128, D, MAJOR_K, MAJOR_MN);     // dV, dK
      const uint32_t id_dq = idesc_bf16(128, QB, MAJOR_MN, MAJOR_MN);   // dQ^T
      const uint32_t aK = smem_u32(sK), aV = smem_u32(sV), aQ = smem_u32(sQ), adO = smem_u32(sdO), aP = smem_u32(sP),
                     adS = smem_u32(sdS);
      // Operand descriptors at offset 0, built once; an MMA adds (byte offset >> 4) to the start-address
      // field (shared memory is below 256 KB, the 14-bit field never carries).  The S^T / dP^T / dQ^T
      // MMAs are 32 clocks of tensor work each: the issuing thread cannot afford to build two
      // descriptors between them.
      const uint64_t dK_k = smem_desc(aK, 16, 1024), dV_k = smem_desc(aV, 16, 1024);       // K-major, 16 KB slabs
      const uint64_t dQ_k = smem_desc(aQ, 16, 1024), ddO_k = smem_desc(adO, 16, 1024);     // K-major, 8 KB slabs
      const uint64_t dP_k = smem_desc(aP, 16, 1024), ddS_k = smem_desc(adS, 16, 1024);     // K-major A operands
      const uint64_t ddO_mn = smem_desc(adO, 8192, 1024), dQ_mn = smem_desc(aQ, 8192, 1024);  // MN-major B operands
      const uint64_t dK_mn = smem_desc(aK, 16384, 1024), ddS_mn = smem_desc(adS, 8192, 1024);
      auto off128 = [](int k) { return (uint64_t)(((k >> 2) * 16384 + (k & 3) * 32) >> 4); };
      auto off64 = [](int k) { return (uint64_t)(((k >> 2) * 8192 + (k & 3) * 32) >> 4); };
      bool ok = role_wait(&kv_full, 0);
      // Two issuers: a tcgen05.mma takes about a hundred cycles to issue whatever its width, so the
      // 32 MMAs of an iteration are split between warp 1 (S^T, dP^T) and warp 10 (dV, dK, dQ^T).
      if (warp == 1) {
        for (int i = 0; i < iters && ok; ++i) {
          const int st = i & 1;
          ZC_BTRACE(1, i, 0);
          if (!(ok = role_wait(&qdo_full[st], (i >> 1) & 1))) break;
          ZC_BTRACE(1, i, 1);
          if (i > 0 && !(ok = role_wait(&sdp_empty, (i - 1) & 1))) break;
          tc_fence_after_sync();
          ZC_BTRACE(1, i, 2);
          const uint64_t stg = (uint64_t)(st * (16384 >> 4));
#pragma unroll
          for (int k = 0; k < D / 16; ++k) mma_bf16(tm_st, dK_k + off128(k), dQ_k + stg + off64(k), id_st, k != 0);
#pragma unroll
          for (int k = 0; k < D / 16; ++k) mma_bf16(tm_dp, dV_k + off128(k), ddO_k + stg + off64(k), id_st, k != 0);
          mma_commit(&sdp_full);
          ZC_BTRACE(1, i, 3);
        }
      } else {
        for (int i = 0; i < iters && ok; ++i) {
          const int st = i & 1, ph = (i >> 1) & 1;
          // pds_full(i) also tells that S^T(i) and dP^T(i) have completed (the compute threads read
          // them before writing P^T and dS^T), so this thread's commits cover every reader of Q/dO
          ZC_BTRACE(2, i, 0);
          if (!(ok = role_wait(&pds_full[st], ph))) break;
          ZC_BTRACE(2, i, 1);
          if (!(ok = role_wait(&dq_empty[st], ph ^ 1))) break;
          tc_fence_after_sync();
          ZC_BTRACE(2, i, 2);
          const uint64_t stg = (uint64_t)(st * (16384 >> 4));
          // dV += P^T dO and dK += dS^T Q: A = [128 keys x 64 queries] K-major, B = [64 queries x 128] MN-major
#pragma unroll
          for (int k = 0; k < QB / 16; ++k)
            mma_bf16(tm_dv, dP_k + stg + (uint64_t)((k * 32) >> 4), ddO_mn + stg + (uint64_t)((k * 2048) >> 4), id_kv,
                     (i | k) != 0);
#pragma unroll
          for (int k = 0; k < QB / 16; ++k)
            mma_bf16(tm_dk, ddS_k + stg + (uint64_t)((k * 32) >> 4), dQ_mn + stg + (uint64_t)((k * 2048) >> 4), id_kv,
                     (i | k) != 0);
          // dQ^T = K^T dS^T: A = K read MN-major (M = head dim), B = dS^T read MN-major (N = queries)
#pragma unroll
          for (int k = 0; k < 8; ++k)
            mma_bf16(tm_dq + st * QB, dK_mn + (uint64_t)((k * 2048) >> 4), ddS_mn + stg + (uint64_t)((k * 2048) >> 4),
                     id_dq, k != 0);
          mma_commit(&dq_full[st]);
          mma_commit(&pds_empty[st]);
          mma_commit(&qdo_empty[st]);
          ZC_BTRACE(2, i, 3);
        }
      }
      if (!ok) s_abort = 1;
    }
  } else {
    const int ct = tid - 64;               // 0..255
    const int quarter = warp & 3;          // TMEM lane quarter this warp may access
    const int half = (warp - 2) >> 2;      // which 32 of the 64 query columns
    const int r = quarter * 32 + lane;     // key row of the tile == TMEM lane (head dim index for dQ^T)
    const int key = k0 + r;
    const uint32_t lane_base = (uint32_t)(quarter * 32);
    const int c0 = half * 32;
    const float sl2 = p.scale * LOG2E;
    // threads 0..63 fetch lse, 64..127 fetch delta of the next iteration's queries (one value each)
    auto fetch = [&](int h, int ib, bool valid) -> float {
      if (ct >= 128 || !valid) return 0.f;
      const int q = ib * QB + (ct & 63);
      if (q >= p.S) return 0.f;
      const int64_t idx = ((int64_t)b * p.Hq + h) * p.S + q;
      return ct < 64 ? __ldg(p.lse + idx) * LOG2E : __ldg(p.delta + idx) * p.scale;
    };
    // (head, 64-query block) of the current and of the previous iteration, advanced without divisions
    int cur_h = hk * group, cur_ib = 2 * jb, prev_h = 0, prev_q0 = 0;
    float pre = fetch(cur_h, cur_ib, iters > 0);
    bool fail = false, aborted = false;
    for (int i = 0; i <= iters; ++i) {
      if (i < iters) {
        const int st = i & 1, ph = (i >> 1) & 1;
        // ---- A: scores and dP of this thread's key row into registers, then release the accumulators
        if (tid == 64) ZC_BTRACE(0, i, 0);
        if (!mbar_wait_parked(&sdp_full, i & 1, &s_abort)) fail = true;
        tc_fence_after_sync();
        if (tid == 64) ZC_BTRACE(0, i, 1);
        uint32_t rs[32], rp[32];
        tmem_ld32(tmem_addr(tm_st, lane_base, c0), rs);
        tmem_ld32(tmem_addr(tm_dp, lane_base, c0), rp);
        if (ct < 128) s_stat[st][ct] = pre;
        tmem_ld_wait();
        tc_fence_before_sync();
        if (named_bar_or(1, 256, fail || s_abort)) { aborted = true; break; }
        if (tid == 64) mbar_arrive(&sdp_empty);
        __syncwarp();
        if (tid == 64) ZC_BTRACE(0, i, 2);
        {
          int nh = cur_h, nib = cur_ib + 1;
          if (nib == nq64) { nib = 2 * jb; ++nh; }
          pre = fetch(nh, nib, i + 1 < iters);
        }
        // ---- B: P^T and dS^T ------------------------------------------------------------------
        const int q0 = cur_ib * QB;
        const bool diag = (q0 < k0 + 128) || (q0 + QB > p.S) || (k0 + 128 > p.S);
        const float4* st_l = reinterpret_cast<const float4*>(&s_stat[st][c0]);
        const float4* st_d = reinterpret_cast<const float4*>(&s_stat[st][64 + c0]);
        uint32_t pk[16], dk_[16];
        // two copies of the loop, so that blocks away from the diagonal carry no masking
        // instructions at all (predicated-off instructions still take issue slots)
        auto elementwise = [&](auto masked) {
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            const float4 l4 = st_l[g], d4 = st_d[g];
            const float ls[4] = {l4.x, l4.y, l4.z, l4.w};
            const float dl[4] = {d4.x, d4.y, d4.z, d4.w};
            float e[4], ds[4];
#pragma unroll
            for (int t = 0; t < 4; ++t) {
              const int c = g * 4 + t;
              float ev = exp2f(__uint_as_float(rs[c]) * sl2 - ls[t]);
              if (decltype(masked)::value) {
                const int q = q0 + c0 + c;
                if (key > q || key >= p.S || q >= p.S) ev = 0.f;
              }
              e[t] = ev;
              ds[t] = ev * fmaf(__uint_as_float(rp[c]), p.scale, -dl[t]);
            }
            pk[2 * g] = pack_bf16(e[0], e[1]);
            pk[2 * g + 1] = pack_bf16(e[2], e[3]);
            dk_[2 * g] = pack_bf16(ds[0], ds[1]);
            dk_[2 * g + 1] = pack_bf16(ds[2], ds[3]);
          }
        };
        if (diag) elementwise(std::true_type{});
        else elementwise(std::false_type{});
        if (tid == 64) ZC_BTRACE(0, i, 3);
        if (!mbar_wait_parked(&pds_empty[st], ph ^ 1, &s_abort)) fail = true;  // MMAs of iteration i-2 have read this stage
        if (tid == 64) ZC_BTRACE(0, i, 4);
        uint8_t* tp = sP + st * 16384;
        uint8_t* td = sdS + st * 16384;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          *reinterpret_cast<uint4*>(tp + sw128_off(r, half * 4 + j)) =
              make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
          *reinterpret_cast<uint4*>(td + sw128_off(r, half * 4 + j)) =
              make_uint4(dk_[4 * j], dk_[4 * j + 1], dk_[4 * j + 2], dk_[4 * j + 3]);
        }
        fence_proxy_async_smem();
        if (tid == 64) bulk_wait_read0();  // the previous dQ reduction has read the staging buffer
        __syncwarp();
        if (named_bar_or(2, 256, fail || s_abort)) { aborted = true; break; }
        if (tid == 64) mbar_arrive(&pds_full[st]);
        __syncwarp();
        if (tid == 64) ZC_BTRACE(0, i, 5);
      } else {
        if (tid == 64) bulk_wait_read0();
        __syncwarp();
        if (named_bar_or(1, 256, fail || s_abort)) { aborted = true; break; }
      }
      if (i > 0) {
        // ---- C: drain dQ^T of iteration i-1 (its MMAs ran during this iteration's phases A and B)
        const int j = i - 1, sj = j & 1;
        if (!mbar_wait_parked(&dq_full[sj], (j >> 1) & 1, &s_abort)) fail = true;
        tc_fence_after_sync();
        if (tid == 64) ZC_BTRACE(0, i, 6);
        uint32_t rr[32];
        tmem_ld32(tmem_addr(tm_dq + sj * QB, lane_base, c0), rr);
        tmem_ld_wait();
        // this thread holds dQ^T[dim r][query c0 .. c0+31]: 128 contiguous bytes of row r of the
        // staging slab of its query half ([128 dims x 32 queries] fp32, 128-byte swizzle), which is
        // also the layout of the accumulator ([B, Hq, D, S]: queries contiguous), so the drain is
        // eight 16-byte stores per thread and no transpose
        uint8_t* slab = sStage + half * 16384;
#pragma unroll
        for (int t = 0; t < 8; ++t)
          *reinterpret_cast<uint4*>(slab + sw128_off(r, t)) =
              make_uint4(rr[4 * t], rr[4 * t + 1], rr[4 * t + 2], rr[4 * t + 3]);
        fence_proxy_async_smem();
        tc_fence_before_sync();
        if (named_bar_or(3, 256, fail || s_abort)) { aborted = true; break; }
        if (tid == 64) {
#pragma unroll
          for (int t = 0; t < 2; ++t) tma_reduce_add_4d(&mapdQ, sStage + t * 16384, prev_q0 + t * 32, 0, prev_h, b);
          bulk_commit();
          mbar_arrive(&dq_empty[sj]);
          ZC_BTRACE(0, i, 7);
        }
        __syncwarp();
      }
      prev_h = cur_h;
      prev_q0 = cur_ib * QB;
      if (++cur_ib == nq64) { cur_ib = 2 * jb; ++cur_h; }
    }
    if (tid == 64) bulk_wait0();
    __syncwarp();
    if (aborted) s_abort = 1;
    if (!aborted) {
      // every MMA into dK / dV has completed: dq_full of the last iteration was committed after them
#pragma unroll 1
      for (int which = 0; which < 2; ++which) {
        const uint32_t tmx = which ? tm_dv : tm_dk;
        __nv_bfloat16* dst = which ? p.dv + b * p.dvs0 + (int64_t)key * p.dvs1 + hk * p.dvs2
                                   : p.dk + b * p.dks0 + (int64_t)key * p.dks1 + hk * p.dks2;
#pragma unroll 1
        for (int c = half * 64; c < half * 64 + 64; c += 32) {
          uint32_t rr[32];
          tmem_ld32(tmem_addr(tmx, lane_base, c), rr);
          tmem_ld_wait();
          if (key < p.S) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              uint4 u;
              u.x = pack_bf16(__uint_as_float(rr[i]), __uint_as_float(rr[i + 1]));
              u.y = pack_bf16(__uint_as_float(rr[i + 2]), __uint_as_float(rr[i + 3]));
              u.z = pack_bf16(__uint_as_float(rr[i + 4]), __uint_as_float(rr[i + 5]));
              u.w = pack_bf16(__uint_as_float(rr[i + 6]), __uint_as_float(rr[i + 7]));
              *reinterpret_cast<uint4*>(dst + c + i) = u;
            }
          }
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (tid == 0 && s_abort) atomicExch(p.status, 6);
  if (warp == 1) tmem_dealloc(tmem_base, 512);
}

}  // namespace bkt
}  // namespace zc

extern "C" {

int zc_attn_bwd_ws_status_read_and_clear() {
  int dev = 0;
  cudaGetDevice(&dev);
  zc::bws::Scratch& sc = zc::bws::g_scratch[dev];
  if (!sc.status) return 0;
  int v = 0;
  cudaMemcpy(&v, sc.status, sizeof(int), cudaMemcpyDeviceToHost);
  if (v) cudaMemset(sc.status, 0, sizeof(int));
  return v;
}

// Same argument list as zc_attn_bwd.
int zc_attn_bwd_ws(const void* q, const void* k, const void* v, const void* o, const void* dout, const float* lse,
                   float* delta, void* dq, void* dk, void* dv, int B, int S, int Hq, int Hkv, int D, int64_t qs0,
                   int64_t qs1, int64_t qs2, int64_t ks0, int64_t ks1, int64_t ks2, int64_t vs0, int64_t vs1,
                   int64_t vs2, int64_t dqs0, int64_t dqs1, int64_t dqs2, int64_t dks0, int64_t dks1, int64_t dks2,
                   int64_t dvs0, int64_t dvs1, int64_t dvs2, float scale, cudaStream_t st) {
  using namespace zc;
  using namespace zc::bws;
  if ((D != 64 && D != 128) || Hq % Hkv) return ERR_UNSUPPORTED;
  if ((qs1 | qs2 | ks1 | ks2 | vs1 | vs2 | qs0 | ks0 | vs0 | dqs1 | dqs2 | dks1 | dks2 | dvs1 | dvs2 | dqs0 | dks0 | dvs0) % 8)
    return ERR_UNSUPPORTED;
  if (dqs0 != (int64_t)S * dqs1) return ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
       reinterpret_cast<uintptr_t>(dout)) & 15)
    return ERR_UNSUPPORTED;
  int dev = 0;
  cudaGetDevice(&dev);
  cudaSetDevice(dev);
  Scratch& sc = g_scratch[dev];
  if (!sc.status) {
    if (cudaMalloc(&sc.status, sizeof(int)) != cudaSuccess) return ERR_BAD_ARG;
    cudaMemset(sc.status, 0, sizeof(int));
  }
  const size_t need = (size_t)B * S * Hq * D * sizeof(float);
  if (sc.dq_bytes < need) {
    if (sc.dq_acc) cudaFreeAsync(sc.dq_acc, st);
    if (cudaMallocAsync(&sc.dq_acc, need, st) != cudaSuccess) { sc.dq_acc = nullptr; sc.dq_bytes = 0; return (int)cudaGetLastError(); }
    sc.dq_bytes = need;
  }
  cudaMemsetAsync(sc.dq_acc, 0, need, st);
  CUtensorMap mq, mk, mv, mdo, mdq;
  if (!make_map4(&mq, q, D, Hq, S, B, qs0, qs1, qs2) || !make_map4(&mk, k, D, Hkv, S, B, ks0, ks1, ks2) ||
      !make_map4(&mv, v, D, Hkv, S, B, vs0, vs1, vs2) ||
      !make_map4(&mdo, dout, D, Hq, S, B, (int64_t)S * Hq * D, (int64_t)Hq * D, D) ||
      !make_map4_f32(&mdq, sc.dq_acc, D, Hq, S, B))
    return ERR_BAD_ARG;
  BwdParams p;
  p.lse = lse; p.delta = delta; p.dq_acc = sc.dq_acc; p.dk = (__nv_bfloat16*)dk; p.dv = (__nv_bfloat16*)dv;
  p.B = B; p.S = S; p.Hq = Hq; p.Hkv = Hkv;
  p.dks0 = dks0; p.dks1 = dks1; p.dks2 = dks2; p.dvs0 = dvs0; p.dvs1 = dvs1; p.dvs2 = dvs2;
  p.scale = scale; p.status = sc.status; p.trace = nullptr;
  const int64_t rows = (int64_t)B * S * Hq;
  delta_kernel<<<(unsigned)((rows * 32 + 255) / 256), 256, 0, st>>>((const __nv_bfloat16*)o, (const __nv_bfloat16*)dout,
                                                                   delta, B, S, Hq, D);
  const int smem = 6 * 32768 + 1024;
  static bool attr[2] = {false, false};
  const dim3 grid((S + 127) / 128, Hkv, B);
  if (D == 128) {
    if (!attr[0]) { cudaFuncSetAttribute(attn_bwd_ws_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); attr[0] = true; }
    attn_bwd_ws_kernel<128><<<grid, 320, smem, st>>>(mq, mk, mv, mdo, mdq, p);
  } else {
    if (!attr[1]) { cudaFuncSetAttribute(attn_bwd_ws_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); attr[1] = true; }
    attn_bwd_ws_kernel<64><<<grid, 320, smem, st>>>(mq, mk, mv, mdo, mdq, p);
  }
  const int cgrid = (int)std::min<int64_t>((rows * (D / 4) + 255) / 256, (int64_t)sm_count() * 16);
  dq_convert_kernel<<<cgrid, 256, 0, st>>>(sc.dq_acc, (__nv_bfloat16*)dq, (int64_t)B * S, Hq, D, dqs1, dqs2);
  return launch_status();
}

#ifdef ZC_PHASE_TRACE
// Development builds only: a device buffer of 3 * 256 * 8 int64 (or null) that CTA 0 of later key-row
// launches fills with SM-clock stamps of its phases.
void zc_attn_bwd_kt_set_trace(void* buf) { zc::bws::g_trace = (long long*)buf; }
#endif

// Same argument list as zc_attn_bwd.  Head dimension 128 runs the key-row kernel; 64 falls back to
// zc_attn_bwd_ws.
int zc_attn_bwd_kt(const void* q, const void* k, const void* v, const void* o, const void* dout, const float* lse,
                   float* delta, void* dq, void* dk, void* dv, int B, int S, int Hq, int Hkv, int D, int64_t qs0,
                   int64_t qs1, int64_t qs2, int64_t ks0, int64_t ks1, int64_t ks2, int64_t vs0, int64_t vs1,
                   int64_t vs2, int64_t dqs0, int64_t dqs1, int64_t dqs2, int64_t dks0, int64_t dks1, int64_t dks2,
                   int64_t dvs0, int64_t dvs1, int64_t dvs2, float scale, cudaStream_t st) {
  using namespace zc;
  using namespace zc::bws;
  if (D != 128)
    return zc_attn_bwd_ws(q, k, v, o, dout, lse, delta, dq, dk, dv, B, S, Hq, Hkv, D, qs0, qs1, qs2, ks0, ks1, ks2, vs0,
                          vs1, vs2, dqs0, dqs1, dqs2, dks0, dks1, dks2, dvs0, dvs1, dvs2, scale, st);
  if (Hq % Hkv) return ERR_UNSUPPORTED;
  if ((qs1 | qs2 | ks1 | ks2 | vs1 | vs2 | qs0 | ks0 | vs0 | dqs1 | dqs2 | dks1 | dks2 | dvs1 | dvs2 | dqs0 | dks0 | dvs0) % 8)
    return ERR_UNSUPPORTED;
  if (dqs0 != (int64_t)S * dqs1) return ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
       reinterpret_cast<uintptr_t>(dout)) & 15)
    return ERR_UNSUPPORTED;
  int dev = 0;
  cudaGetDevice(&dev);
  cudaSetDevice(dev);
  Scratch& sc = g_scratch[dev];
  if (!sc.status) {
    if (cudaMalloc(&sc.status, sizeof(int)) != cudaSuccess) return ERR_BAD_ARG;
    cudaMemset(sc.status, 0, sizeof(int));
  }
  const int Sp = (S + 3) & ~3;  // row stride of the transposed accumulator: a multiple of 16 bytes
  const size_t need = (size_t)B * Hq * D * Sp * sizeof(float);
  if (sc.dq_bytes < need) {
    if (sc.dq_acc) cudaFreeAsync(sc.dq_acc, st);
    if (cudaMallocAsync(&sc.dq_acc, need, st) != cudaSuccess) { sc.dq_acc = nullptr; sc.dq_bytes = 0; return (int)cudaGetLastError(); }
    sc.dq_bytes = need;
  }
  cudaMemsetAsync(sc.dq_acc, 0, need, st);
  CUtensorMap mq, mk, mv, mdo, mdq;
  if (!make_map4(&mq, q, D, Hq, S, B, qs0, qs1, qs2, bkt::QB) || !make_map4(&mk, k, D, Hkv, S, B, ks0, ks1, ks2) ||
      !make_map4(&mv, v, D, Hkv, S, B, vs0, vs1, vs2) ||
      !make_map4(&mdo, dout, D, Hq, S, B, (int64_t)S * Hq * D, (int64_t)Hq * D, D, bkt::QB) ||
      !make_map_dq_t(&mdq, sc.dq_acc, D, Hq, S, Sp, B))
    return ERR_BAD_ARG;
  BwdParams p;
  p.lse = lse; p.delta = delta; p.dq_acc = sc.dq_acc; p.dk = (__nv_bfloat16*)dk; p.dv = (__nv_bfloat16*)dv;
  p.B = B; p.S = S; p.Hq = Hq; p.Hkv = Hkv;
  p.dks0 = dks0; p.dks1 = dks1; p.dks2 = dks2; p.dvs0 = dvs0; p.dvs1 = dvs1; p.dvs2 = dvs2;
  p.scale = scale; p.status = sc.status; p.trace = g_trace;
  const int64_t rows = (int64_t)B * S * Hq;
  delta_kernel<<<(unsigned)((rows * 32 + 255) / 256), 256, 0, st>>>((const __nv_bfloat16*)o, (const __nv_bfloat16*)dout,
                                                                   delta, B, S, Hq, D);
  const int smem = 7 * 32768 + 1024;
  static bool attr = false;
  if (!attr) { cudaFuncSetAttribute(bkt::attn_bwd_kt_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); attr = true; }
  const int nkb = (S + 127) / 128;
  bkt::attn_bwd_kt_kernel<<<nkb * Hkv * B, 352, smem, st>>>(mq, mk, mv, mdo, mdq, p, nkb);
  dq_convert_t_kernel<<<dim3((S + 31) / 32, D / 64, B * Hq), dim3(32, 8), 0, st>>>(
      sc.dq_acc, (__nv_bfloat16*)dq, S, Sp, Hq, D, dqs0, dqs1, dqs2);
  return launch_status();
}

}  // extern "C"
