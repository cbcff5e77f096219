// Causal grouped-query flash attention for sm_100a on the tcgen05 tensor cores.
//
// Forward, one CTA (128 threads) per (128-query block, query head, batch):
//   for each 128-key block up to the diagonal:
//     S = Q K^T            tcgen05.mma, both operands K-major from swizzled smem, S in TMEM
//     softmax              thread t owns query row t: tcgen05.ld gives it the whole row, so the
//                          running max / sum need no shuffles; P is written to smem as bf16
//                          (it reuses the K buffer, which is dead once S is complete)
//     PV = P V             tcgen05.mma, A = P K-major, B = V MN-major (V is [key][d], d contiguous,
//                          so no transposed copy is made)
//     O = O * alpha + PV   in registers
//   96 KB of smem and 256 TMEM columns per CTA, so two CTAs share an SM and overlap each other's
//   load / MMA / softmax phases.
// Backward, one CTA per (128-key block, kv head, batch), looping over the query heads of the group
// and the query blocks at or below the diagonal; dK and dV accumulate in TMEM for the whole loop:
//     S = Q K^T, dP = dO V^T ; P = exp2(S - lse), dS = P * (dP - delta) * scale
//     dV += P^T dO, dK += dS^T Q   (A operands are the MN-major view of P / dS, no transposes)
//     dQ_i += dS K                 (fp32 red.add into an accumulator, converted afterwards)
// Every mbarrier wait is bounded; on expiry the status word is set and the CTA frees its TMEM.
#include <cuda_bf16.h>
#include <math_constants.h>

#include "launch_util.h"
#include "umma.cuh"

namespace zc {
using namespace umma;

constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;

// Stage a [128 x D] tile (row stride `ld` elements) into swizzled slabs of 64 columns.
template <int D>
__device__ __forceinline__ void stage_tile(uint8_t* dst, const __nv_bfloat16* src, int64_t ld, int rows_valid,
                                           int tid) {
  constexpr int CPR = D / 8;  // 16-byte chunks per row
  // all of this thread's loads are issued before the first store, so a whole tile is in flight
  uint4 v[CPR];
#pragma unroll
  for (int it = 0; it < CPR; ++it) {
    const int i = tid + it * 128;
    const int row = i / CPR, chunk = i % CPR;
    v[it] = make_uint4(0, 0, 0, 0);
    if (row < rows_valid) v[it] = __ldg(reinterpret_cast<const uint4*>(src + (int64_t)row * ld + chunk * 8));
  }
#pragma unroll
  for (int it = 0; it < CPR; ++it) {
    const int i = tid + it * 128;
    const int row = i / CPR, chunk = i % CPR;
    *reinterpret_cast<uint4*>(dst + (chunk >> 3) * 16384 + sw128_off(row, chunk & 7)) = v[it];
  }
}

// descriptors for a staged [128 x 64*slabs] tile
//   as K-major operand (rows = M/N index, columns = K): K-step k covers columns 16k..16k+15
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t base, int k) {
  return smem_desc(base + (k >> 2) * 16384 + (k & 3) * 32, 16, 1024);
}
//   as MN-major operand (rows = K index, columns = M/N): K-step k covers rows 16k..16k+15
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t base, int k) {
  return smem_desc(base + k * 2048, 16384, 1024);
}

// write 32 bf16 values (one TMEM chunk of this thread's row) into a K-major [128 x 128] smem tile
__device__ __forceinline__ void store_row_chunk(uint8_t* tile, int row, int col0, const float (&v)[32]) {
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const int col = col0 + q * 8;
    uint4 u;
    __nv_bfloat162 a = __floats2bfloat162_rn(v[q * 8 + 0], v[q * 8 + 1]);
    __nv_bfloat162 b = __floats2bfloat162_rn(v[q * 8 + 2], v[q * 8 + 3]);
    __nv_bfloat162 c = __floats2bfloat162_rn(v[q * 8 + 4], v[q * 8 + 5]);
    __nv_bfloat162 d = __floats2bfloat162_rn(v[q * 8 + 6], v[q * 8 + 7]);
    u.x = *reinterpret_cast<uint32_t*>(&a);
    u.y = *reinterpret_cast<uint32_t*>(&b);
    u.z = *reinterpret_cast<uint32_t*>(&c);
    u.w = *reinterpret_cast<uint32_t*>(&d);
    *reinterpret_cast<uint4*>(tile + (col >> 6) * 16384 + sw128_off(row, (col >> 3) & 7)) = u;
  }
}

struct AttnParams {
  const __nv_bfloat16 *q, *k, *v;
  __nv_bfloat16* o;
  float* lse;
  int B, S, Hq, Hkv;
  int64_t qs0, qs1, qs2, ks0, ks1, ks2, vs0, vs1, vs2;  // element strides of (batch, seq, head)
  float scale;
  int* status;
};

template <int D>
__global__ void __launch_bounds__(128) attn_fwd_kernel(const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int TILE = 128 * D * 2;  // bytes; D=128 -> 32 KB (two slabs), D=64 -> 16 KB
  uint8_t* sQ = smem;
  uint8_t* sK = smem + 32768;  // reused for P (always [128 x 128] bf16 = 32 KB)
  uint8_t* sV = smem + 65536;
  __shared__ uint64_t bar_s, bar_o;
  __shared__ uint32_t tmem_base;
  const int tid = threadIdx.x, warp = tid >> 5;
  const int qb = gridDim.x - 1 - blockIdx.x;  // heavy (late) query blocks first
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.Hq / p.Hkv);
  if (tid == 0) {
    mbar_init(&bar_s, 1);
    mbar_init(&bar_o, 1);
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc(&tmem_base, 256);
    tmem_relinquish();
  }
  const int q0 = qb * 128;
  stage_tile<D>(sQ, p.q + b * p.qs0 + (int64_t)q0 * p.qs1 + h * p.qs2, p.qs1, p.S - q0, tid);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmS = tmem_base, tmO = tmem_base + 128;
  const uint32_t idesc_s = idesc_bf16(128, 128, MAJOR_K, MAJOR_K);
  const uint32_t idesc_o = idesc_bf16(128, D, MAJOR_K, MAJOR_MN);
  const float sl2 = p.scale * LOG2E;
  const int row = q0 + tid;
  const uint32_t lane_base = (uint32_t)(warp * 32);
  float m = -CUDART_INF_F, l = 0.f;
  float o[D];
#pragma unroll
  for (int i = 0; i < D; ++i) o[i] = 0.f;
  bool ok = true;
  (void)TILE;
  for (int j = 0; j <= qb && ok; ++j) {
    const int k0 = j * 128;
    stage_tile<D>(sK, p.k + b * p.ks0 + (int64_t)k0 * p.ks1 + hk * p.ks2, p.ks1, p.S - k0, tid);
    stage_tile<D>(sV, p.v + b * p.vs0 + (int64_t)k0 * p.vs1 + hk * p.vs2, p.vs1, p.S - k0, tid);
    fence_proxy_async_smem();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after_sync();
#pragma unroll
      for (int k = 0; k < D / 16; ++k)
        mma_bf16(tmS, desc_kmajor(smem_u32(sQ), k), desc_kmajor(smem_u32(sK), k), idesc_s, k != 0);
      mma_commit(&bar_s);
    }
    ok = mbar_wait(&bar_s, j & 1);
    if (!ok) break;
    tc_fence_after_sync();
    // ---- softmax of this thread's row -----------------------------------------------------------
    const bool diag = (j == qb) || (k0 + 128 > p.S);
    float mx = -CUDART_INF_F;
#pragma unroll 1
    for (int c = 0; c < 128; c += 32) {
      uint32_t r[32];
      tmem_ld32(tmem_addr(tmS, lane_base, c), r);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        float s = __uint_as_float(r[i]);
        if (diag && (k0 + c + i > row || k0 + c + i >= p.S)) s = -CUDART_INF_F;
        mx = fmaxf(mx, s);
      }
    }
    const float m_new = fmaxf(m, mx * sl2);
    const float m_use = (m_new == -CUDART_INF_F) ? 0.f : m_new;
    const float alpha = exp2f(m - m_use);
    float rs = 0.f;
#pragma unroll 1
    for (int c = 0; c < 128; c += 32) {
      uint32_t r[32];
      tmem_ld32(tmem_addr(tmS, lane_base, c), r);
      tmem_ld_wait();
      float pv[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        float s = __uint_as_float(r[i]);
        float e = exp2f(s * sl2 - m_use);
        if (diag && (k0 + c + i > row || k0 + c + i >= p.S)) e = 0.f;
        pv[i] = e;
        rs += e;
      }
      store_row_chunk(sK, tid, c, pv);  // P overwrites K
    }
    l = l * alpha + rs;
    m = m_new;
    fence_proxy_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after_sync();
#pragma unroll
      for (int k = 0; k < 8; ++k)
        mma_bf16(tmO, desc_kmajor(smem_u32(sK), k), desc_mnmajor(smem_u32(sV), k), idesc_o, k != 0);
      mma_commit(&bar_o);
    }
    ok = mbar_wait(&bar_o, j & 1);
    if (!ok) break;
    tc_fence_after_sync();
#pragma unroll
    for (int c = 0; c < D; c += 32) {
      uint32_t r[32];
      tmem_ld32(tmem_addr(tmO, lane_base, c), r);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 32; ++i) o[c + i] = o[c + i] * alpha + __uint_as_float(r[i]);
    }
    tc_fence_before_sync();
    __syncthreads();  // P / V buffers are free for the next block's staging
  }
  if (ok) {
    if (row < p.S) {
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* dst = p.o + ((int64_t)(b * p.S + row) * p.Hq + h) * D;
#pragma unroll
      for (int c = 0; c < D; c += 8) {
        uint4 u;
        __nv_bfloat162 a0 = __floats2bfloat162_rn(o[c] * inv, o[c + 1] * inv);
        __nv_bfloat162 a1 = __floats2bfloat162_rn(o[c + 2] * inv, o[c + 3] * inv);
        __nv_bfloat162 a2 = __floats2bfloat162_rn(o[c + 4] * inv, o[c + 5] * inv);
        __nv_bfloat162 a3 = __floats2bfloat162_rn(o[c + 6] * inv, o[c + 7] * inv);
        u.x = *reinterpret_cast<uint32_t*>(&a0);
        u.y = *reinterpret_cast<uint32_t*>(&a1);
        u.z = *reinterpret_cast<uint32_t*>(&a2);
        u.w = *reinterpret_cast<uint32_t*>(&a3);
        *reinterpret_cast<uint4*>(dst + c) = u;
      }
      p.lse[((int64_t)b * p.Hq + h) * p.S + row] = (l > 0.f) ? (m + log2f(l)) * LN2 : -CUDART_INF_F;
    }
  } else if (tid == 0) {
    atomicExch(p.status, 1);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, 256);
}

// delta[b,h,s] = sum_d dO * O
template <int D>
__global__ void __launch_bounds__(256) attn_delta_kernel(const __nv_bfloat16* __restrict__ o,
                                                         const __nv_bfloat16* __restrict__ dout,
                                                         float* __restrict__ delta, int B, int S, int Hq) {
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
    const int64_t bb = bs / S, ss = bs % S;
    delta[(bb * Hq + hh) * S + ss] = acc;
  }
}

struct AttnBwdParams {
  const __nv_bfloat16 *q, *k, *v, *dout;
  const float *lse, *delta;
  float* dq_acc;  // fp32 [B, S, Hq, D], zeroed by the launcher
  __nv_bfloat16 *dk, *dv;
  int B, S, Hq, Hkv;
  int64_t qs0, qs1, qs2, ks0, ks1, ks2, vs0, vs1, vs2;
  int64_t dks0, dks1, dks2, dvs0, dvs1, dvs2;
  float scale;
  int* status;
};

template <int D>
__global__ void __launch_bounds__(128) attn_bwd_kernel(const AttnBwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = smem + 1 * 32768;
  uint8_t* sQ = smem + 2 * 32768;
  uint8_t* sdO = smem + 3 * 32768;
  uint8_t* sP = smem + 4 * 32768;
  uint8_t* sdS = smem + 5 * 32768;
  __shared__ uint64_t bar1, bar2;
  __shared__ uint32_t tmem_base;
  const int tid = threadIdx.x, warp = tid >> 5;
  const int nkb = gridDim.x;
  const int jb = blockIdx.x;  // key block; early key blocks have the most query blocks
  const int hk = blockIdx.y, b = blockIdx.z;
  const int group = p.Hq / p.Hkv;
  if (tid == 0) {
    mbar_init(&bar1, 1);
    mbar_init(&bar2, 1);
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc(&tmem_base, 512);
    tmem_relinquish();
  }
  const int k0 = jb * 128;
  stage_tile<D>(sK, p.k + b * p.ks0 + (int64_t)k0 * p.ks1 + hk * p.ks2, p.ks1, p.S - k0, tid);
  stage_tile<D>(sV, p.v + b * p.vs0 + (int64_t)k0 * p.vs1 + hk * p.vs2, p.vs1, p.S - k0, tid);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tm_dk = tmem_base, tm_dv = tmem_base + 128, tm_s = tmem_base + 256, tm_dp = tmem_base + 384;
  const uint32_t id_s = idesc_bf16(128, 128, MAJOR_K, MAJOR_K);     // S, dP
  const uint32_t id_kv = idesc_bf16(128, D, MAJOR_MN, MAJOR_MN);    // dV, dK
  const uint32_t id_dq = idesc_bf16(128, D, MAJOR_K, MAJOR_MN);     // dQ partial
  const float sl2 = p.scale * LOG2E;
  const uint32_t lane_base = (uint32_t)(warp * 32);
  bool ok = true;
  uint32_t it = 0;
  for (int hh = 0; hh < group && ok; ++hh) {
    const int h = hk * group + hh;
    for (int ib = jb; ib < nkb && ok; ++ib, ++it) {
      const int q0 = ib * 128;
      const int row = q0 + tid;
      stage_tile<D>(sQ, p.q + b * p.qs0 + (int64_t)q0 * p.qs1 + h * p.qs2, p.qs1, p.S - q0, tid);
      stage_tile<D>(sdO, p.dout + ((int64_t)(b * p.S + q0) * p.Hq + h) * D, (int64_t)p.Hq * D, p.S - q0, tid);
      float lse2 = 0.f, dl = 0.f;
      if (row < p.S) {
        lse2 = p.lse[((int64_t)b * p.Hq + h) * p.S + row] * LOG2E;
        dl = p.delta[((int64_t)b * p.Hq + h) * p.S + row];
      }
      fence_proxy_async_smem();
      __syncthreads();
      if (tid == 0) {
        tc_fence_after_sync();
#pragma unroll
        for (int k = 0; k < D / 16; ++k)
          mma_bf16(tm_s, desc_kmajor(smem_u32(sQ), k), desc_kmajor(smem_u32(sK), k), id_s, k != 0);
#pragma unroll
        for (int k = 0; k < D / 16; ++k)
          mma_bf16(tm_dp, desc_kmajor(smem_u32(sdO), k), desc_kmajor(smem_u32(sV), k), id_s, k != 0);
        mma_commit(&bar1);
      }
      ok = mbar_wait(&bar1, it & 1);
      if (!ok) break;
      tc_fence_after_sync();
      const bool diag = (ib == jb) || (q0 + 128 > p.S) || (k0 + 128 > p.S);
#pragma unroll 1
      for (int c = 0; c < 128; c += 32) {
        uint32_t rs[32], rp[32];
        tmem_ld32(tmem_addr(tm_s, lane_base, c), rs);
        tmem_ld32(tmem_addr(tm_dp, lane_base, c), rp);
        tmem_ld_wait();
        float pv[32], ds[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float e = exp2f(__uint_as_float(rs[i]) * sl2 - lse2);
          if (diag && (k0 + c + i > row || k0 + c + i >= p.S || row >= p.S)) e = 0.f;
          pv[i] = e;
          ds[i] = e * (__uint_as_float(rp[i]) - dl) * p.scale;
        }
        store_row_chunk(sP, tid, c, pv);
        store_row_chunk(sdS, tid, c, ds);
      }
      fence_proxy_async_smem();
      tc_fence_before_sync();
      __syncthreads();
      if (tid == 0) {
        tc_fence_after_sync();
#pragma unroll
        for (int k = 0; k < 8; ++k)  // dV += P^T dO
          mma_bf16(tm_dv, desc_mnmajor(smem_u32(sP), k), desc_mnmajor(smem_u32(sdO), k), id_kv, (it | k) != 0);
#pragma unroll
        for (int k = 0; k < 8; ++k)  // dK += dS^T Q
          mma_bf16(tm_dk, desc_mnmajor(smem_u32(sdS), k), desc_mnmajor(smem_u32(sQ), k), id_kv, (it | k) != 0);
#pragma unroll
        for (int k = 0; k < 8; ++k)  // dQ_i partial = dS K  (reuses the S columns)
          mma_bf16(tm_s, desc_kmajor(smem_u32(sdS), k), desc_mnmajor(smem_u32(sK), k), id_dq, k != 0);
        mma_commit(&bar2);
      }
      ok = mbar_wait(&bar2, it & 1);
      if (!ok) break;
      tc_fence_after_sync();
      float* dqrow = p.dq_acc + ((int64_t)(b * p.S + row) * p.Hq + h) * D;
#pragma unroll 1
      for (int c = 0; c < D; c += 32) {
        uint32_t r[32];
        tmem_ld32(tmem_addr(tm_s, lane_base, c), r);
        tmem_ld_wait();
        if (row < p.S) {
#pragma unroll
          for (int i = 0; i < 32; i += 4)
            atomicAdd(reinterpret_cast<float4*>(dqrow + c + i),
                      make_float4(__uint_as_float(r[i]), __uint_as_float(r[i + 1]), __uint_as_float(r[i + 2]),
                                  __uint_as_float(r[i + 3])));
        }
      }
      tc_fence_before_sync();
      __syncthreads();
    }
  }
  if (ok) {
    const int krow = k0 + tid;
#pragma unroll 1
    for (int which = 0; which < 2; ++which) {
      const uint32_t tm = which ? tm_dv : tm_dk;
      __nv_bfloat16* dst = which ? p.dv + b * p.dvs0 + (int64_t)krow * p.dvs1 + hk * p.dvs2
                                 : p.dk + b * p.dks0 + (int64_t)krow * p.dks1 + hk * p.dks2;
#pragma unroll 1
      for (int c = 0; c < D; c += 32) {
        uint32_t r[32];
        tmem_ld32(tmem_addr(tm, lane_base, c), r);
        tmem_ld_wait();
        if (krow < p.S) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 u;
            __nv_bfloat162 a0 = __floats2bfloat162_rn(__uint_as_float(r[i]), __uint_as_float(r[i + 1]));
            __nv_bfloat162 a1 = __floats2bfloat162_rn(__uint_as_float(r[i + 2]), __uint_as_float(r[i + 3]));
            __nv_bfloat162 a2 = __floats2bfloat162_rn(__uint_as_float(r[i + 4]), __uint_as_float(r[i + 5]));
            __nv_bfloat162 a3 = __floats2bfloat162_rn(__uint_as_float(r[i + 6]), __uint_as_float(r[i + 7]));
            u.x = *reinterpret_cast<uint32_t*>(&a0);
            u.y = *reinterpret_cast<uint32_t*>(&a1);
            u.z = *reinterpret_cast<uint32_t*>(&a2);
            u.w = *reinterpret_cast<uint32_t*>(&a3);
            *reinterpret_cast<uint4*>(dst + c + i) = u;
          }
        }
      }
    }
  } else if (tid == 0) {
    atomicExch(p.status, 2);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, 512);
}

// dq (bf16, strided) = dq_acc (fp32, contiguous [B,S,Hq,D])
__global__ void __launch_bounds__(256) attn_dq_convert_kernel(const float* __restrict__ acc,
                                                              __nv_bfloat16* __restrict__ dq, int64_t rows, int Hq,
                                                              int D, int64_t s_bs, int64_t s_h) {
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

// per-device scratch that persists across calls: status word and the fp32 dQ accumulator
struct AttnScratch {
  int* status = nullptr;
  float* dq_acc = nullptr;
  size_t dq_bytes = 0;
};
static AttnScratch g_scratch[64];

static int* attn_status(int dev) {
  AttnScratch& s = g_scratch[dev];
  if (!s.status) {
    if (cudaMalloc(&s.status, sizeof(int)) != cudaSuccess) return nullptr;
    cudaMemset(s.status, 0, sizeof(int));
  }
  return s.status;
}

}  // namespace zc

extern "C" {

// Reads the sticky status word (0 = no bounded wait expired since the last call); synchronises.
int zc_attn_status_read_and_clear() {
  int dev = 0;
  cudaGetDevice(&dev);
  int* st = zc::attn_status(dev);
  if (!st) return -1;
  int v = 0;
  cudaMemcpy(&v, st, sizeof(int), cudaMemcpyDeviceToHost);
  if (v) cudaMemset(st, 0, sizeof(int));
  return v;
}

int zc_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B, int S, int Hq, int Hkv, int D,
                int64_t qs0, int64_t qs1, int64_t qs2, int64_t ks0, int64_t ks1, int64_t ks2, int64_t vs0,
                int64_t vs1, int64_t vs2, float scale, cudaStream_t st) {
  using namespace zc;
  if ((D != 64 && D != 128) || Hq % Hkv) return ERR_UNSUPPORTED;
  if ((qs1 | qs2 | ks1 | ks2 | vs1 | vs2 | qs0 | ks0 | vs0) % 8) return ERR_UNSUPPORTED;  // 16-byte vector loads
  int dev = 0;
  cudaGetDevice(&dev);
  AttnParams p;
  p.q = (const __nv_bfloat16*)q; p.k = (const __nv_bfloat16*)k; p.v = (const __nv_bfloat16*)v;
  p.o = (__nv_bfloat16*)o; p.lse = lse;
  p.B = B; p.S = S; p.Hq = Hq; p.Hkv = Hkv;
  p.qs0 = qs0; p.qs1 = qs1; p.qs2 = qs2; p.ks0 = ks0; p.ks1 = ks1; p.ks2 = ks2; p.vs0 = vs0; p.vs1 = vs1; p.vs2 = vs2;
  p.scale = scale;
  p.status = attn_status(dev);
  if (!p.status) return ERR_BAD_ARG;
  const int smem = 3 * 32768 + 1024;
  static bool attr[2] = {false, false};
  const dim3 grid((S + 127) / 128, Hq, B);
  if (D == 128) {
    if (!attr[0]) { cudaFuncSetAttribute(attn_fwd_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); attr[0] = true; }
    attn_fwd_kernel<128><<<grid, 128, smem, st>>>(p);
  } else {
    if (!attr[1]) { cudaFuncSetAttribute(attn_fwd_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); attr[1] = true; }
    attn_fwd_kernel<64><<<grid, 128, smem, st>>>(p);
  }
  return launch_status();
}

int zc_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* dout, const float* lse,
                float* delta, void* dq, void* dk, void* dv, int B, int S, int Hq, int Hkv, int D, int64_t qs0,
                int64_t qs1, int64_t qs2, int64_t ks0, int64_t ks1, int64_t ks2, int64_t vs0, int64_t vs1,
                int64_t vs2, int64_t dqs0, int64_t dqs1, int64_t dqs2, int64_t dks0, int64_t dks1, int64_t dks2,
                int64_t dvs0, int64_t dvs1, int64_t dvs2, float scale, cudaStream_t st) {
  using namespace zc;
  if ((D != 64 && D != 128) || Hq % Hkv) return ERR_UNSUPPORTED;
  if ((qs1 | qs2 | ks1 | ks2 | vs1 | vs2 | qs0 | ks0 | vs0 | dqs1 | dqs2 | dks1 | dks2 | dvs1 | dvs2 | dqs0 | dks0 | dvs0) % 8)
    return ERR_UNSUPPORTED;
  if (dqs0 != (int64_t)S * dqs1) return ERR_UNSUPPORTED;  // (batch, seq) must flatten to one row index
  int dev = 0;
  cudaGetDevice(&dev);
  AttnScratch& sc = g_scratch[dev];
  const size_t need = (size_t)B * S * Hq * D * sizeof(float);
  if (sc.dq_bytes < need) {
    // grown only when a larger problem appears; stream-ordered so earlier launches keep their buffer
    if (sc.dq_acc) cudaFreeAsync(sc.dq_acc, st);
    if (cudaMallocAsync(&sc.dq_acc, need, st) != cudaSuccess) { sc.dq_acc = nullptr; sc.dq_bytes = 0; return (int)cudaGetLastError(); }
    sc.dq_bytes = need;
  }
  cudaMemsetAsync(sc.dq_acc, 0, need, st);
  AttnBwdParams p;
  p.q = (const __nv_bfloat16*)q; p.k = (const __nv_bfloat16*)k; p.v = (const __nv_bfloat16*)v;
  p.dout = (const __nv_bfloat16*)dout; p.lse = lse; p.delta = delta; p.dq_acc = sc.dq_acc;
  p.dk = (__nv_bfloat16*)dk; p.dv = (__nv_bfloat16*)dv;
  p.B = B; p.S = S; p.Hq = Hq; p.Hkv = Hkv;
  p.qs0 = qs0; p.qs1 = qs1; p.qs2 = qs2; p.ks0 = ks0; p.ks1 = ks1; p.ks2 = ks2; p.vs0 = vs0; p.vs1 = vs1; p.vs2 = vs2;
  p.dks0 = dks0; p.dks1 = dks1; p.dks2 = dks2; p.dvs0 = dvs0; p.dvs1 = dvs1; p.dvs2 = dvs2;
  p.scale = scale;
  p.status = attn_status(dev);
  if (!p.status) return ERR_BAD_ARG;
  const int64_t rows = (int64_t)B * S * Hq;
  const int smem = 6 * 32768 + 1024;
  static bool attr[2] = {false, false};
  const dim3 grid((S + 127) / 128, Hkv, B);
  const int cgrid = (int)std::min<int64_t>((rows * (D / 4) + 255) / 256, (int64_t)sm_count() * 16);
  if (D == 128) {
    attn_delta_kernel<128><<<(unsigned)((rows * 32 + 255) / 256), 256, 0, st>>>((const __nv_bfloat16*)o, (const __nv_bfloat16*)dout, delta, B, S, Hq);
    if (!attr[0]) { cudaFuncSetAttribute(attn_bwd_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); attr[0] = true; }
    attn_bwd_kernel<128><<<grid, 128, smem, st>>>(p);
  } else {
    attn_delta_kernel<64><<<(unsigned)((rows * 32 + 255) / 256), 256, 0, st>>>((const __nv_bfloat16*)o, (const __nv_bfloat16*)dout, delta, B, S, Hq);
    if (!attr[1]) { cudaFuncSetAttribute(attn_bwd_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); attr[1] = true; }
    attn_bwd_kernel<64><<<grid, 128, smem, st>>>(p);
  }
  attn_dq_convert_kernel<<<cgrid, 256, 0, st>>>(sc.dq_acc, (__nv_bfloat16*)dq, (int64_t)B * S, Hq, D, dqs1, dqs2);
  return launch_status();
}

}  // extern "C"
