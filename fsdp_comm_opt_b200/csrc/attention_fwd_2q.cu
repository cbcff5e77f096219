// Causal GQA attention forward for sm_100a, head dimension 128: two query tiles per CTA (the
// default forward path).
//
// One CTA (352 threads) owns 256 consecutive queries of one head as two 128-row tiles that share
// every K/V block it loads.  Key blocks hold 64 keys, so a softmax thread owns a whole score row
// of a block (64 fp32 registers): no partner thread, no exchange through shared memory, and the
// row maximum, the exponentials and the row sum come from one read of TMEM.
//   warp 0      TMA producer: both Q tiles once, then K/V blocks into a four-stage ring
//   warps 1,10  MMA issuers, one per tile: S_t = Q_t K_j^T (128 x 64, fp32 in TMEM) and
//               O_t += P_t V_j with the output accumulating in TMEM for the whole row of blocks
//   warps 2-5   softmax of tile 0, warps 6-9 softmax of tile 1, one thread per query row.  A
//               thread copies its row of S_t to registers and releases the TMEM buffer at once, so
//               the next block's scores are computed while this block is exponentiated; the two
//               tiles' warps share the SM's schedulers and hide each other's latencies.
// The running maximum is only raised when the new block's maximum exceeds it by more than 2^8
// (exponentials stay below 256, exact enough in bf16 and fp32); raising it rescales the row of O in
// TMEM (tcgen05.ld, multiply, tcgen05.st), which after the first few blocks almost never happens.
// The probabilities never touch shared memory: a softmax thread writes its row of P_t as bf16 pairs
// into tensor memory (tcgen05.st) and O_t += P_t V_j takes its A operand from there, so that MMA
// fetches only V from shared memory.
// TMEM (512 columns allocated): S_0 64 | S_1 64 | O_0 128 | O_1 128 | P: tile t, block parity u at
// 384 + (2 t + u) * 32 (64 keys as 32 columns).
// Shared memory: Q 2 x 32 KB, K/V ring 4 x (16 + 16) KB.
// CTAs are numbered heaviest first (the last 256 queries see the most keys).  Every wait is
// bounded; a timed-out role raises a CTA-wide abort flag, the CTA frees its TMEM and returns, and the
// launcher's status word reports it.
#include <cuda.h>
#include <cuda_bf16.h>
#include <math_constants.h>

#include "attn_common.cuh"
#include "launch_util.h"

extern "C" int zc_attn_fwd_ws(const void* q, const void* k, const void* v, void* o, float* lse, int B, int S, int Hq,
                              int Hkv, int D, int64_t qs0, int64_t qs1, int64_t qs2, int64_t ks0, int64_t ks1,
                              int64_t ks2, int64_t vs0, int64_t vs1, int64_t vs2, float scale, cudaStream_t st);

namespace zc {
namespace fwd2q {
using namespace attn;

constexpr int THREADS = 352;
constexpr int KB = 64;          // keys per block
constexpr int STAGES = 4;       // K/V ring
constexpr float RAISE = 8.f;    // log2 of the factor by which a row maximum may lag behind

struct Params {
  __nv_bfloat16* o;
  float* lse;
  int B, S, Hq, Hkv;
  float scale;
  int* status;
  int ncb;  // number of 256-query blocks
  long long* trace;  // null, or [2][blocks][8] SM-clock stamps written by CTA 0 (softmax warp 2, MMA thread)
};
// Phase stamps for kernel development: compiled in only with -DZC_PHASE_TRACE
#ifdef ZC_PHASE_TRACE
#define ZC_TRACE(slot, j, k)                                                          \
  do {                                                                                \
    if (p.trace && blockIdx.x == 0 && (j) < 128) p.trace[((slot) * 128 + (j)) * 8 + (k)] = clock64(); \
  } while (0)
#else
#define ZC_TRACE(slot, j, k) \
  do {                       \
  } while (0)
#endif

__global__ void __launch_bounds__(THREADS, 1) attn_fwd_2q_kernel(const __grid_constant__ CUtensorMap mapQ,
                                                                 const __grid_constant__ CUtensorMap mapK,
                                                                 const __grid_constant__ CUtensorMap mapV,
                                                                 const Params p) {
  constexpr int D = 128;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;              // tile t at t * 32 KB: two 64-column slabs of [128 x 128 B]
  uint8_t* sKV = smem + 65536;     // stage s at s * 32 KB: K (two slabs of [64 x 128 B]), then V
  __shared__ uint64_t q_full, kv_full[STAGES], kv_empty[STAGES], s_full[2], s_empty[2], p_full[2], o_full[4];  // o_full[2 t + (j & 1)]
  __shared__ uint32_t tmem_base;
  __shared__ volatile int s_abort;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int per_c = p.Hq * p.B;
  const int cb = p.ncb - 1 - (int)blockIdx.x / per_c;
  const int h = ((int)blockIdx.x % per_c) % p.Hq, b = ((int)blockIdx.x % per_c) / p.Hq;
  const int hk = h / (p.Hq / p.Hkv);
  const int q0 = cb * 256;
  int nb[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int qt0 = q0 + 128 * t;
    nb[t] = qt0 >= p.S ? 0 : (min(qt0 + 128, p.S) + KB - 1) / KB;
  }
  const int nbmax = max(nb[0], nb[1]);
  if (tid == 0) {
    mbar_init(&q_full, 1);
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 2);  // one arrival per MMA issuer
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&s_empty[i], 4);  // one arrival per softmax warp of the tile
      mbar_init(&p_full[i], 4);
    }
    for (int i = 0; i < 4; ++i) mbar_init(&o_full[i], 1);
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
      mbar_expect_tx(&q_full, (nb[1] > 0 ? 2 : 1) * 32768);
#pragma unroll
      for (int t = 0; t < 2; ++t)
        if (nb[t] > 0)
#pragma unroll
          for (int sl = 0; sl < 2; ++sl)
            tma_load_4d(sQ + t * 32768 + sl * 16384, &mapQ, &q_full, sl * 64, h, q0 + 128 * t, b);
      for (int j = 0; j < nbmax; ++j) {
        const int s = j % STAGES;
        if (!role_wait(&kv_empty[s], ((j / STAGES) & 1) ^ 1, &s_abort)) { s_abort = 1; break; }
        uint8_t* stage = sKV + s * 32768;
        mbar_expect_tx(&kv_full[s], 32768);
#pragma unroll
        for (int sl = 0; sl < 2; ++sl) {
          tma_load_4d(stage + sl * 8192, &mapK, &kv_full[s], sl * 64, hk, j * KB, b);
          tma_load_4d(stage + 16384 + sl * 8192, &mapV, &kv_full[s], sl * 64, hk, j * KB, b);
        }
      }
    }
  } else if (warp == 1 || warp == 10) {
    // one MMA issuer per query tile (warp 1: tile 0, warp 10: tile 1).  The S MMAs are 32 clocks of
    // tensor work each, so the issuing thread must not spend more than that between two of them:
    // the operand descriptors are built once and an MMA adds a constant to their address field.
    if (lane == 0) {
      const int t = warp == 1 ? 0 : 1;
      const uint32_t id_s = idesc_bf16(128, KB, MAJOR_K, MAJOR_K);
      const uint32_t id_o = idesc_bf16(128, D, MAJOR_K, MAJOR_MN);
      const uint32_t aQ = smem_u32(sQ) + t * 32768, aKV = smem_u32(sKV);
      const uint32_t tm_s = tm + t * 64, tm_o = tm + 128 + t * 128, tm_p = tm + 384 + t * 64;
      const int nbt = nb[t];
      // descriptors at offset 0 of each operand; byte offsets are added to the start-address field as
      // offset >> 4 (shared memory is below 256 KB, the 14-bit field never carries)
      const uint64_t dQ0 = smem_desc(aQ, 16, 1024);               // Q tile, K-major, 16 KB slabs
      const uint64_t dK0 = smem_desc(aKV, 16, 1024);              // K block of stage 0, K-major, 8 KB slabs
      const uint64_t dV0 = smem_desc(aKV + 16384, 8192, 1024);    // V block of stage 0, MN-major
      bool ok = role_wait(&q_full, 0, &s_abort);
      // S_t(j) = Q_t K_j^T: A = Q tile (K-major, 16 KB slabs), B = K block (K-major, 8 KB slabs)
      auto issue_s = [&](int j) -> bool {
        const int s = j % STAGES;
        if (!role_wait(&kv_full[s], (j / STAGES) & 1, &s_abort)) return false;
        if (j > 0 && !role_wait(&s_empty[t], (j - 1) & 1, &s_abort)) return false;
        tc_fence_after_sync();
        const uint64_t dK = dK0 + (uint64_t)(s * (32768 >> 4));
#pragma unroll
        for (int k = 0; k < D / 16; ++k)
          mma_bf16(tm_s, dQ0 + (uint64_t)(((k >> 2) * 16384 + (k & 3) * 32) >> 4),
                   dK + (uint64_t)(((k >> 2) * 8192 + (k & 3) * 32) >> 4), id_s, k != 0);
        mma_commit(&s_full[t]);
        return true;
      };
      if (ok && nbt > 0) ok = issue_s(0);
      for (int j = 0; j < nbmax && ok; ++j) {
        if (t == 0) ZC_TRACE(1, j, 0);
        if (j >= nbt) {
          // this tile has no such block: only hand the stage back, and only once it has been
          // filled, so that each phase of kv_empty gets exactly one arrival from each issuer
          if (!(ok = role_wait(&kv_full[j % STAGES], (j / STAGES) & 1, &s_abort))) break;
          mbar_arrive(&kv_empty[j % STAGES]);
          continue;
        }
        if (j + 1 < nbt && !(ok = issue_s(j + 1))) break;
        if (t == 0) ZC_TRACE(1, j, 1);
        if (!(ok = role_wait(&p_full[t], j & 1, &s_abort))) break;
        tc_fence_after_sync();
        if (t == 0) ZC_TRACE(1, j, 2);
        // O_t += P_t V_j: A = P tile [128 x 64 keys] in tensor memory, B = V block [64 keys x 128] MN-major
        const uint64_t dV = dV0 + (uint64_t)((j % STAGES) * (32768 >> 4));
        const uint32_t tP = tm_p + (uint32_t)((j & 1) * 32);
#pragma unroll
        for (int k = 0; k < KB / 16; ++k)
          mma_bf16_tmem_a(tm_o, tP + (uint32_t)(k * 8), dV + (uint64_t)((k * 2048) >> 4), id_o, (j | k) != 0);
        mma_commit(&o_full[2 * t + (j & 1)]);
        mma_commit(&kv_empty[j % STAGES]);  // this tile's readers of the stage have been issued
        if (t == 0) ZC_TRACE(1, j, 3);
      }
      if (!ok) s_abort = 1;
    }
  } else {
    const int t = (warp - 2) >> 2;         // query tile of this warp
    const int quarter = warp & 3;          // TMEM lane quarter this warp may access
    const int r = quarter * 32 + lane;     // query row inside the tile == TMEM lane
    const int qt0 = q0 + 128 * t;
    const int row = qt0 + r;
    const int nbt = nb[t];
    const uint32_t lane_base = (uint32_t)(quarter * 32);
    const uint32_t tm_s = tm + t * 64, tm_o = tm + 128 + t * 128, tm_p = tm + 384 + t * 64;
    const float sl2 = p.scale * LOG2E;
    float m_ref = -CUDART_INF_F, l = 0.f;
    bool fail = false;
    const bool tr = (warp == 2 && lane == 0);
    for (int j = 0; j < nbt; ++j) {
      if (tr) ZC_TRACE(0, j, 0);
      fail = !mbar_wait_parked(&s_full[t], j & 1, &s_abort);
      if (__any_sync(0xffffffffu, fail || s_abort)) { fail = true; break; }
      tc_fence_after_sync();
      if (tr) ZC_TRACE(0, j, 1);
      uint32_t sa[32], sb[32];
      tmem_ld32(tmem_addr(tm_s, lane_base, 0), sa);
      tmem_ld32(tmem_addr(tm_s, lane_base, 32), sb);
      tmem_ld_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_empty[t]);  // the next block's scores may overwrite S_t now
      __syncwarp();
      if (tr) ZC_TRACE(0, j, 2);
      const int k0 = j * KB;
      if ((k0 + KB - 1 > qt0) || (k0 + KB > p.S)) {  // block touches the diagonal or the end of the sequence
        const uint32_t ninf = __float_as_uint(-CUDART_INF_F);
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int c = k0 + i;
          if (c > row || c >= p.S) sa[i] = ninf;
          if (c + 32 > row || c + 32 >= p.S) sb[i] = ninf;
        }
      }
      // four independent chains: a single running maximum would serialise 64 dependent operations
      float mx4[4] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
      for (int i = 0; i < 32; ++i)
        mx4[i & 3] = fmaxf(mx4[i & 3], fmaxf(__uint_as_float(sa[i]), __uint_as_float(sb[i])));
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      const float m_cand = mx * sl2;
      const bool raise = m_cand > m_ref + RAISE;  // also true for the first unmasked block (m_ref = -inf)
      float alpha = 1.f;
      if (raise) {
        alpha = exp2f(m_ref - m_cand);
        m_ref = m_cand;
        l *= alpha;
      }
      const float m_use = (m_ref == -CUDART_INF_F) ? 0.f : m_ref;
      if (tr) ZC_TRACE(0, j, 3);
      // P_t is double-buffered by block parity: block j's buffer was last read by P_t V of block
      // j-2, which has long completed (the wait returns at once for j < 2)
      fail = !mbar_wait_parked(&o_full[2 * t + (j & 1)], ((j >> 1) & 1) ^ 1, &s_abort);
      if (__any_sync(0xffffffffu, fail || s_abort)) { fail = true; break; }
      if (j > 0 && __any_sync(0xffffffffu, raise)) {
        // rescaling O_t has to wait for the P_t V of the previous block as well
        fail = !mbar_wait_parked(&o_full[2 * t + ((j - 1) & 1)], ((j - 1) >> 1) & 1, &s_abort);
        if (__any_sync(0xffffffffu, fail || s_abort)) { fail = true; break; }
        tc_fence_after_sync();
        {
#pragma unroll 1
          for (int c = 0; c < D; c += 32) {
            uint32_t rr[32];
            tmem_ld32(tmem_addr(tm_o, lane_base, c), rr);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) rr[i] = __float_as_uint(__uint_as_float(rr[i]) * alpha);
            tmem_st32(tmem_addr(tm_o, lane_base, c), rr);
          }
          tmem_st_wait();
        }
      }
      if (tr) ZC_TRACE(0, j, 4);
      float rs4[4] = {0.f, 0.f, 0.f, 0.f};
      uint32_t pk[32];  // the row of P as bf16 pairs: column c holds keys 2 c (low half) and 2 c + 1
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        const uint32_t* src = q < 4 ? &sa[q * 8] : &sb[(q - 4) * 8];
        float e[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          e[i] = exp2f(__uint_as_float(src[i]) * sl2 - m_use);
          rs4[i & 3] += e[i];
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) pk[q * 4 + i] = pack_bf16(e[2 * i], e[2 * i + 1]);
      }
      tmem_st32(tmem_addr(tm_p + (uint32_t)((j & 1) * 32), lane_base, 0), pk);
      l += (rs4[0] + rs4[1]) + (rs4[2] + rs4[3]);
      tmem_st_wait();
      if (tr) ZC_TRACE(0, j, 5);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[t]);
      __syncwarp();
      if (tr) ZC_TRACE(0, j, 6);
    }
    if (fail) s_abort = 1;
    if (!fail && nbt > 0) {
      fail = !mbar_wait_parked(&o_full[2 * t + ((nbt - 1) & 1)], ((nbt - 1) >> 1) & 1, &s_abort);
      if (__any_sync(0xffffffffu, fail)) {
        s_abort = 1;
      } else {
        tc_fence_after_sync();
        const float inv = l > 0.f ? 1.f / l : 0.f;
        __nv_bfloat16* dst = p.o + ((int64_t)(b * p.S + row) * p.Hq + h) * D;
#pragma unroll 1
        for (int c = 0; c < D; c += 32) {
          uint32_t rr[32];
          tmem_ld32(tmem_addr(tm_o, lane_base, c), rr);
          tmem_ld_wait();
          if (row < p.S) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              uint4 u;
              u.x = pack_bf16(__uint_as_float(rr[i]) * inv, __uint_as_float(rr[i + 1]) * inv);
              u.y = pack_bf16(__uint_as_float(rr[i + 2]) * inv, __uint_as_float(rr[i + 3]) * inv);
              u.z = pack_bf16(__uint_as_float(rr[i + 4]) * inv, __uint_as_float(rr[i + 5]) * inv);
              u.w = pack_bf16(__uint_as_float(rr[i + 6]) * inv, __uint_as_float(rr[i + 7]) * inv);
              *reinterpret_cast<uint4*>(dst + c + i) = u;
            }
          }
        }
        if (row < p.S)
          p.lse[((int64_t)b * p.Hq + h) * p.S + row] = (l > 0.f) ? (m_ref + log2f(l)) * LN2 : -CUDART_INF_F;
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (tid == 0 && s_abort) atomicExch(p.status, 7);
  if (warp == 1) tmem_dealloc(tm, 512);
}

static long long* g_trace = nullptr;

static int* status_word(int dev) {
  static int* st[64] = {nullptr};
  if (!st[dev]) {
    if (cudaMalloc(&st[dev], sizeof(int)) != cudaSuccess) return nullptr;
    cudaMemset(st[dev], 0, sizeof(int));
  }
  return st[dev];
}

}  // namespace fwd2q
}  // namespace zc

extern "C" {

int zc_attn_fwd_2q_status_read_and_clear() {
  int dev = 0;
  cudaGetDevice(&dev);
  int* st = zc::fwd2q::status_word(dev);
  if (!st) return -1;
  int v = 0;
  cudaMemcpy(&v, st, sizeof(int), cudaMemcpyDeviceToHost);
  if (v) cudaMemset(st, 0, sizeof(int));
  return v;
}

#ifdef ZC_PHASE_TRACE
// Development builds only: a device buffer of 2 * 128 * 8 int64 (or null) that CTA 0 of later launches
// fills with SM-clock stamps of its phases.
void zc_attn_fwd_2q_set_trace(void* buf) { zc::fwd2q::g_trace = (long long*)buf; }
#endif

// Same argument list as zc_attn_fwd_ws.  Head dimension 128 runs the two-tile kernel; 64 falls back
// to zc_attn_fwd_ws.
int zc_attn_fwd_2q(const void* q, const void* k, const void* v, void* o, float* lse, int B, int S, int Hq, int Hkv,
                   int D, int64_t qs0, int64_t qs1, int64_t qs2, int64_t ks0, int64_t ks1, int64_t ks2, int64_t vs0,
                   int64_t vs1, int64_t vs2, float scale, cudaStream_t st) {
  using namespace zc;
  using namespace zc::fwd2q;
  if (D != 128)
    return zc_attn_fwd_ws(q, k, v, o, lse, B, S, Hq, Hkv, D, qs0, qs1, qs2, ks0, ks1, ks2, vs0, vs1, vs2, scale, st);
  if (Hq % Hkv) return ERR_UNSUPPORTED;
  if ((qs0 | qs1 | qs2 | ks0 | ks1 | ks2 | vs0 | vs1 | vs2) % 8) return ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v)) & 15)
    return ERR_UNSUPPORTED;
  int dev = 0;
  cudaGetDevice(&dev);
  cudaSetDevice(dev);  // binds the primary context on autograd worker threads (tensor-map encoder needs it)
  CUtensorMap mq, mk, mv;
  if (!make_map_bshd(&mq, q, D, Hq, S, B, qs0, qs1, qs2, 128) || !make_map_bshd(&mk, k, D, Hkv, S, B, ks0, ks1, ks2, KB) ||
      !make_map_bshd(&mv, v, D, Hkv, S, B, vs0, vs1, vs2, KB))
    return ERR_BAD_ARG;
  Params p;
  p.o = (__nv_bfloat16*)o; p.lse = lse; p.B = B; p.S = S; p.Hq = Hq; p.Hkv = Hkv; p.scale = scale;
  p.status = status_word(dev);
  p.ncb = (S + 255) / 256;
  p.trace = g_trace;
  if (!p.status) return ERR_BAD_ARG;
  const int smem = 65536 + STAGES * 32768 + 1024;
  static bool attr = false;
  if (!attr) { cudaFuncSetAttribute(attn_fwd_2q_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); attr = true; }
  attn_fwd_2q_kernel<<<p.ncb * Hq * B, THREADS, smem, st>>>(mq, mk, mv, p);
  return launch_status();
}

}  // extern "C"
