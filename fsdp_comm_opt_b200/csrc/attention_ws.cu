// Warp-specialised causal GQA attention forward for sm_100a: the path for head dimension 64 (and for
// 128 with ZC_ATTN_FWD=ws; attention_fwd_2q.cu is the default there).
//
// One CTA (320 threads) per (128-query block, query head, batch):
//   warp 0      TMA producer: Q once, then K/V tiles of 128 keys into a two-stage ring (4-D tensor
//               maps over the packed [B, S, H, D] projection, SWIZZLE_128B, zero fill past S)
//   warp 1      MMA issuer: S_j = Q K_j^T into one of two TMEM S buffers, issued one block ahead so
//               the tensor core works on S_{j+1} while the softmax warps are busy with S_j;
//               then O_j = P_j V_j (V read as an MN-major operand, no transpose)
//   warps 2-9   softmax: two threads per query row, 64 score columns and D/2 output columns each.
//               A thread reads its half row of S from TMEM once (kept in registers), the pair
//               exchanges its partial row maximum through shared memory, each thread writes its
//               half of P_j (bf16) to shared memory and accumulates its half of
//               O = O * alpha + P_j V_j in registers once that MMA has completed.
// Hand-offs are mbarriers (TMA complete_tx, tcgen05.commit, thread arrivals); every wait is
// bounded and a timed-out role raises a CTA-wide abort flag that all roles honour at their next
// synchronisation point, so the CTA always reaches its teardown and frees its TMEM.
#include <cuda.h>
#include <cuda_bf16.h>
#include <math_constants.h>

#include <cstdio>

#include "launch_util.h"
#include "umma.cuh"

namespace zc {
namespace ws {
using namespace umma;

constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;
constexpr int THREADS = 320;
constexpr int SM_THREADS = 256;  // softmax threads

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
__device__ __forceinline__ uint64_t desc_k(uint32_t base, int k) {   // K-major tile, K step k
  return smem_desc(base + (k >> 2) * 16384 + (k & 3) * 32, 16, 1024);
}
__device__ __forceinline__ uint64_t desc_mn(uint32_t base, int k) {  // MN-major tile, K step k
  return smem_desc(base + k * 2048, 16384, 1024);
}
// 32 consecutive P values of row `row`, columns col0..col0+31, into the K-major [128 x 128] tile
__device__ __forceinline__ void store_p32(uint8_t* tile, int row, int col0, const float* v) {
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

struct FwdParams {
  __nv_bfloat16* o;
  float* lse;
  int B, S, Hq, Hkv;
  float scale;
  int* status;
};

template <int D>
// Ten warps put three warps on two of the four SM sub-partitions, each of which owns 16384
// registers: 3 x 32 x R <= 16384 caps a thread at 168 registers (a launch with more fails).
__global__ void __launch_bounds__(THREADS, 1) attn_fwd_ws_kernel(const __grid_constant__ CUtensorMap mapQ,
                                                                 const __grid_constant__ CUtensorMap mapK,
                                                                 const __grid_constant__ CUtensorMap mapV,
                                                                 const FwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int TILE = 128 * D * 2;  // bytes of one [128 x D] tile
  constexpr int SLABS = D / 64;
  constexpr int DH = D / 2;          // output columns per softmax thread
  uint8_t* sQ = smem;
  uint8_t* sP = smem + 32768;
  uint8_t* sKV = smem + 65536;  // stage s: K at s*65536, V at s*65536 + 32768
  __shared__ uint64_t q_full, kv_full[2], kv_empty[2], s_full[2], s_empty[2], p_full, o_full;
  __shared__ uint32_t tmem_base;
  __shared__ volatile int s_abort;
  __shared__ float s_xchg[2][128];  // partial row max (per block) / partial row sum (at the end)
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int qb = gridDim.x - 1 - blockIdx.x;
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.Hq / p.Hkv);
  const int q0 = qb * 128;
  const int nb = qb + 1;
  if (tid == 0) {
    mbar_init(&q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_empty[i], 1);
    }
    mbar_init(&p_full, 1);
    mbar_init(&o_full, 1);
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
  const uint32_t tm = tmem_base;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(&q_full, TILE);
#pragma unroll
      for (int sl = 0; sl < SLABS; ++sl) tma_load_4d(sQ + sl * 16384, &mapQ, &q_full, sl * 64, h, q0, b);
      for (int j = 0; j < nb; ++j) {
        const int s = j & 1;
        if (!mbar_wait_relaxed(&kv_empty[s], ((j >> 1) & 1) ^ 1)) { s_abort = 1; break; }
        uint8_t* sk = sKV + s * 65536;
        mbar_expect_tx(&kv_full[s], 2 * TILE);
#pragma unroll
        for (int sl = 0; sl < SLABS; ++sl) {
          tma_load_4d(sk + sl * 16384, &mapK, &kv_full[s], sl * 64, hk, j * 128, b);
          tma_load_4d(sk + 32768 + sl * 16384, &mapV, &kv_full[s], sl * 64, hk, j * 128, b);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t id_s = idesc_bf16(128, 128, MAJOR_K, MAJOR_K);
      const uint32_t id_o = idesc_bf16(128, D, MAJOR_K, MAJOR_MN);
      bool ok = mbar_wait_relaxed(&q_full, 0);
      auto issue_s = [&](int i) -> bool {
        const int s = i & 1;
        if (!mbar_wait_relaxed(&kv_full[s], (i >> 1) & 1)) return false;
        if (!mbar_wait_relaxed(&s_empty[s], ((i >> 1) & 1) ^ 1)) return false;
        tc_fence_after_sync();
        const uint32_t kq = smem_u32(sQ), kk = smem_u32(sKV + s * 65536);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) mma_bf16(tm + s * 128, desc_k(kq, k), desc_k(kk, k), id_s, k != 0);
        mma_commit(&s_full[s]);
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int j = 0; j < nb && ok; ++j) {
        if (j + 1 < nb) ok = issue_s(j + 1);
        if (!ok) break;
        if (!(ok = mbar_wait_relaxed(&p_full, j & 1))) break;
        tc_fence_after_sync();
        const uint32_t pp = smem_u32(sP), vv = smem_u32(sKV + (j & 1) * 65536 + 32768);
#pragma unroll
        for (int k = 0; k < 8; ++k) mma_bf16(tm + 256, desc_k(pp, k), desc_mn(vv, k), id_o, k != 0);
        mma_commit(&o_full);
        mma_commit(&kv_empty[j & 1]);
      }
      if (!ok) s_abort = 1;
    }
  } else {
    const int cw = warp - 2;
    const int quarter = warp & 3;          // TMEM lane quarter this warp may access
    const int half = cw >> 2;              // which 64 score columns / D/2 output columns
    const int r = quarter * 32 + lane;     // query row inside the tile == TMEM lane
    const int row = q0 + r;
    const uint32_t lane_base = (uint32_t)(quarter * 32);
    const int sc0 = half * 64;             // first score column of this thread
    const int oc0 = half * DH;             // first output column of this thread
    const float sl2 = p.scale * LOG2E;
    float m = -CUDART_INF_F, l = 0.f, alpha_prev = 1.f;
    float o[DH];
#pragma unroll
    for (int i = 0; i < DH; ++i) o[i] = 0.f;
    for (int j = 0; j < nb; ++j) {
      const int sb = j & 1;
      if (!mbar_wait(&s_full[sb], (j >> 1) & 1)) s_abort = 1;
      tc_fence_after_sync();
      const int k0 = j * 128;
      const bool diag = (j == qb) || (k0 + 128 > p.S);
      // pass 1: row maximum over this thread's 64 columns (both loads in flight, one wait)
      float mx = -CUDART_INF_F;
      {
        uint32_t sa[32], sbv[32];
        tmem_ld32(tmem_addr(tm + sb * 128, lane_base, sc0), sa);
        tmem_ld32(tmem_addr(tm + sb * 128, lane_base, sc0 + 32), sbv);
        tmem_ld_wait();
        if (diag) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int c0 = k0 + sc0 + i, c1 = c0 + 32;
            if (c0 <= row && c0 < p.S) mx = fmaxf(mx, __uint_as_float(sa[i]));
            if (c1 <= row && c1 < p.S) mx = fmaxf(mx, __uint_as_float(sbv[i]));
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) mx = fmaxf(mx, fmaxf(__uint_as_float(sa[i]), __uint_as_float(sbv[i])));
        }
      }
      s_xchg[half][r] = mx;
      named_bar_sync(1, SM_THREADS);
      mx = fmaxf(mx, s_xchg[half ^ 1][r]);
      const float m_new = fmaxf(m, mx * sl2);
      const float m_use = (m_new == -CUDART_INF_F) ? 0.f : m_new;
      const float alpha = exp2f(m - m_use);
      if (j > 0) {
        // fold in the previous block's P V (its MMA ran while this block's scores were read)
        if (!mbar_wait(&o_full, (j - 1) & 1)) s_abort = 1;
        tc_fence_after_sync();
#pragma unroll
        for (int c = 0; c < DH; c += 32) {
          uint32_t rr[32];
          tmem_ld32(tmem_addr(tm + 256, lane_base, oc0 + c), rr);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[c + i] = o[c + i] * alpha_prev + __uint_as_float(rr[i]);
        }
      }
      // pass 2: re-read the scores 32 columns at a time, exponentiate, write P
      float rs = 0.f;
#pragma unroll 1
      for (int c = 0; c < 64; c += 32) {
        uint32_t rr[32];
        tmem_ld32(tmem_addr(tm + sb * 128, lane_base, sc0 + c), rr);
        tmem_ld_wait();
        float pv[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float e = exp2f(__uint_as_float(rr[i]) * sl2 - m_use);
          const int col = k0 + sc0 + c + i;
          if (diag && (col > row || col >= p.S)) e = 0.f;
          pv[i] = e;
          rs += e;
        }
        store_p32(sP, r, sc0 + c, pv);
      }
      l = l * alpha + rs;
      m = m_new;
      alpha_prev = alpha;
      fence_proxy_async_smem();
      tc_fence_before_sync();
      named_bar_sync(2, SM_THREADS);
      if (s_abort) break;
      if (tid == 64) {
        mbar_arrive(&p_full);
        mbar_arrive(&s_empty[sb]);
      }
    }
    if (!s_abort) {
      if (!mbar_wait(&o_full, (nb - 1) & 1)) s_abort = 1;
      tc_fence_after_sync();
#pragma unroll
      for (int c = 0; c < DH; c += 32) {
        uint32_t rr[32];
        tmem_ld32(tmem_addr(tm + 256, lane_base, oc0 + c), rr);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) o[c + i] = o[c + i] * alpha_prev + __uint_as_float(rr[i]);
      }
    }
    // combine the two partial row sums
    s_xchg[half][r] = l;
    named_bar_sync(1, SM_THREADS);
    l += s_xchg[half ^ 1][r];
    if (!s_abort && row < p.S) {
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* dst = p.o + ((int64_t)(b * p.S + row) * p.Hq + h) * D + oc0;
#pragma unroll
      for (int c = 0; c < DH; c += 8) {
        __nv_bfloat162 a0 = __floats2bfloat162_rn(o[c] * inv, o[c + 1] * inv);
        __nv_bfloat162 a1 = __floats2bfloat162_rn(o[c + 2] * inv, o[c + 3] * inv);
        __nv_bfloat162 a2 = __floats2bfloat162_rn(o[c + 4] * inv, o[c + 5] * inv);
        __nv_bfloat162 a3 = __floats2bfloat162_rn(o[c + 6] * inv, o[c + 7] * inv);
        uint4 u;
        u.x = *reinterpret_cast<uint32_t*>(&a0);
        u.y = *reinterpret_cast<uint32_t*>(&a1);
        u.z = *reinterpret_cast<uint32_t*>(&a2);
        u.w = *reinterpret_cast<uint32_t*>(&a3);
        *reinterpret_cast<uint4*>(dst + c) = u;
      }
      if (half == 0)
        p.lse[((int64_t)b * p.Hq + h) * p.S + row] = (l > 0.f) ? (m + log2f(l)) * LN2 : -CUDART_INF_F;
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (tid == 0 && s_abort) atomicExch(p.status, 4);
  if (warp == 1) tmem_dealloc(tm, 512);
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

// 4-D view (D, H, S, B) of a packed bf16 projection with element strides (s_b, s_s, s_h); box = one
// 64-wide slab of 128 sequence positions of one head
static bool make_map4(CUtensorMap* m, const void* base, int D, int H, int S, int B, int64_t s_b, int64_t s_s,
                      int64_t s_h) {
  EncodeFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)H, (cuuint64_t)S, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)s_h * 2, (cuuint64_t)s_s * 2, (cuuint64_t)s_b * 2};
  cuuint32_t box[4] = {64, 1, 128, 1};
  cuuint32_t el[4] = {1, 1, 1, 1};
  const CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, el,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    fprintf(stderr, "[zc_attn] cuTensorMapEncodeTiled failed (%d): base=%p D=%d H=%d S=%d B=%d strides=%lld,%lld,%lld\n",
            (int)r, base, D, H, S, B, (long long)s_b, (long long)s_s, (long long)s_h);
  return r == CUDA_SUCCESS;
}

static int* ws_status(int dev) {
  static int* st[64] = {nullptr};
  if (!st[dev]) {
    if (cudaMalloc(&st[dev], sizeof(int)) != cudaSuccess) return nullptr;
    cudaMemset(st[dev], 0, sizeof(int));
  }
  return st[dev];
}

}  // namespace ws
}  // namespace zc

extern "C" {

int zc_attn_ws_status_read_and_clear() {
  int dev = 0;
  cudaGetDevice(&dev);
  int* st = zc::ws::ws_status(dev);
  if (!st) return -1;
  int v = 0;
  cudaMemcpy(&v, st, sizeof(int), cudaMemcpyDeviceToHost);
  if (v) cudaMemset(st, 0, sizeof(int));
  return v;
}

// q/k/v: base pointers of the head-0 slices; element strides of (batch, seq, head); heads hold D
// contiguous elements.  o: contiguous [B, S, Hq, D]; lse: [B, Hq, S] fp32.
int zc_attn_fwd_ws(const void* q, const void* k, const void* v, void* o, float* lse, int B, int S, int Hq, int Hkv,
                   int D, int64_t qs0, int64_t qs1, int64_t qs2, int64_t ks0, int64_t ks1, int64_t ks2, int64_t vs0,
                   int64_t vs1, int64_t vs2, float scale, cudaStream_t st) {
  using namespace zc;
  using namespace zc::ws;
  if ((D != 64 && D != 128) || Hq % Hkv) return ERR_UNSUPPORTED;
  if ((qs0 | qs1 | qs2 | ks0 | ks1 | ks2 | vs0 | vs1 | vs2) % 8) return ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v)) & 15)
    return ERR_UNSUPPORTED;
  int dev = 0;
  cudaGetDevice(&dev);
  cudaSetDevice(dev);  // binds the primary context on autograd worker threads (tensor-map encoder needs it)
  CUtensorMap mq, mk, mv;
  if (!make_map4(&mq, q, D, Hq, S, B, qs0, qs1, qs2) || !make_map4(&mk, k, D, Hkv, S, B, ks0, ks1, ks2) ||
      !make_map4(&mv, v, D, Hkv, S, B, vs0, vs1, vs2))
    return ERR_BAD_ARG;
  FwdParams p;
  p.o = (__nv_bfloat16*)o; p.lse = lse; p.B = B; p.S = S; p.Hq = Hq; p.Hkv = Hkv; p.scale = scale;
  p.status = ws_status(dev);
  if (!p.status) return ERR_BAD_ARG;
  const int smem = 65536 + 2 * 65536 + 1024;
  static bool attr[2] = {false, false};
  const dim3 grid((S + 127) / 128, Hq, B);
  if (D == 128) {
    if (!attr[0]) { cudaFuncSetAttribute(attn_fwd_ws_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); attr[0] = true; }
    attn_fwd_ws_kernel<128><<<grid, THREADS, smem, st>>>(mq, mk, mv, p);
  } else {
    if (!attr[1]) { cudaFuncSetAttribute(attn_fwd_ws_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); attr[1] = true; }
    attn_fwd_ws_kernel<64><<<grid, THREADS, smem, st>>>(mq, mk, mv, p);
  }
  return launch_status();
}

}  // extern "C"
