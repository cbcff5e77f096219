// Two-SM (cta_group::2) variant of the persistent bf16 GEMM: a cluster of two CTAs owns a 256 x 256
// output tile.  Each CTA stages its own 128 rows of A and its own 128 of the tile's 256 columns of
// B; one thread of the even CTA issues tcgen05.mma.cta_group::2 (M = 256, N = 256, K = 16), which
// reads both CTAs' shared memory and accumulates each CTA's 128 rows into that CTA's TMEM.
//
// Why: a tcgen05.mma fetches its shared-memory operands at about 68 B per clock per SM (measured
// with the 1-SM kernel and the attention kernels), so the 1-SM 128 x 256 tile (12 KB per K = 16
// step) is operand-bound at ~190 clocks against 128 of tensor work.  With the B operand split
// between the pair an SM fetches 8 KB per step (~118 clocks): the tile becomes tensor-bound.
//
//   warp 0      TMA producer (both CTAs): cp.async.bulk.tensor...cta_group::2 loads into the CTA's
//               own stage buffers, transaction bytes counted on the even CTA's `full` barrier
//   warp 1      even CTA: MMA issuer; commits arrive on the `empty` / `acc_full` barriers of both CTAs
//   warps 2-5   epilogue (both CTAs): tcgen05.ld the CTA's 128 x 256 accumulator, convert, store;
//               arrivals of both CTAs' epilogue warps free the accumulator on the even CTA
// Every CTA fetches its own tiles with plain per-CTA TMA loads; no load is shared between CTAs.
// Every wait is bounded; on expiry the status word is set and both CTAs reach the teardown.
//
// State: written against the 1-SM kernel and compiled for sm_100a; selected only by
// ZC_GEMM_BACKEND=tcgen05_2sm (never by "auto").
#include <cuda.h>
#include <cuda_bf16.h>

#include <algorithm>
#include <cstdio>

#include "launch_util.h"
#include "umma.cuh"

namespace zc {
namespace g2 {
using namespace umma;

constexpr int BM_CTA = 128;   // rows of A per CTA (256 per cluster)
constexpr int BN_CTA = 128;   // columns of B staged per CTA (256 per cluster)
constexpr int BN = 256;       // accumulator columns
constexpr int BK = 64;
constexpr int STAGES = 6;
constexpr int THREADS = 192;
constexpr int A_BYTES = BM_CTA * BK * 2;  // 16 KB
constexpr int B_BYTES = BN_CTA * BK * 2;  // 16 KB
constexpr int STAGE = A_BYTES + B_BYTES;

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `local_addr` (a shared::cta address) in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA load into this CTA's shared memory; the bytes are counted on the barrier at `bar_cluster_addr`
// (the even CTA's `full` barrier)
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, uint32_t bar_cluster_addr,
                                                 int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void mma_bf16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrive on the barrier at `cluster_addr` (either CTA of the pair) when all MMAs issued so far by this
// thread have completed
__device__ __forceinline__ void mma_commit_pair(uint32_t cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_addr)
               : "memory");
}

struct Params {
  __nv_bfloat16* C;
  int64_t M, N, K;
  int a_major, b_major, accumulate;
  int m_fast;
  int* status;
};

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
    gemm_2sm_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t full[STAGES], empty[STAGES], acc_full[2], acc_empty[2];
  __shared__ uint32_t tmem_base;
  __shared__ volatile int s_abort;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t rank = cluster_ctarank();  // 0: even CTA (issues the MMAs), 1: odd CTA
  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);    // used on the even CTA: its producer's arrive.expect_tx
      mbar_init(&empty[s], 1);   // one commit per use, on both CTAs
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);   // one commit per tile, on both CTAs
      mbar_init(&acc_empty[a], 8);  // used on the even CTA: four epilogue warps of each CTA
    }
    mbar_fence_init();
    s_abort = 0;
  }
  if (warp == 1) {
    tmem_alloc_pair(&tmem_base, 2 * BN);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers are initialised before any remote arrival
  tc_fence_after_sync();
  const uint32_t tm = tmem_base;
  const int64_t m_tiles = p.M / (2 * BM_CTA), n_tiles = p.N / BN, k_blocks = p.K / BK;
  const int64_t tiles = m_tiles * n_tiles;
  const int64_t cluster_id = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;
  bool ok = true;

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;
      for (int64_t t = cluster_id; t < tiles && ok; t += n_clusters) {
        const int m0 = (int)(p.m_fast ? t % m_tiles : t / n_tiles) * (2 * BM_CTA) + (int)rank * BM_CTA;
        const int n0 = (int)(p.m_fast ? t / m_tiles : t % n_tiles) * BN + (int)rank * BN_CTA;
        for (int64_t kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!(ok = mbar_wait_parked(&empty[s], ph ^ 1, &s_abort))) break;
          uint8_t* sa = smem + s * STAGE;
          uint8_t* sb = sa + A_BYTES;
          const uint32_t full0 = map_to_cta(smem_u32(&full[s]), 0);
          if (rank == 0) mbar_expect_tx(&full[s], 2 * STAGE);  // both CTAs' bytes land on this barrier
          const int k0 = (int)kb * BK;
          if (p.a_major == MAJOR_K) {
            tma_load_2d_pair(sa, &mapA, full0, k0, m0);
          } else {
#pragma unroll
            for (int sl = 0; sl < BM_CTA / 64; ++sl) tma_load_2d_pair(sa + sl * 8192, &mapA, full0, m0 + sl * 64, k0);
          }
          if (p.b_major == MAJOR_K) {
            tma_load_2d_pair(sb, &mapB, full0, k0, n0);
          } else {
#pragma unroll
            for (int sl = 0; sl < BN_CTA / 64; ++sl) tma_load_2d_pair(sb + sl * 8192, &mapB, full0, n0 + sl * 64, k0);
          }
        }
      }
      if (!ok) s_abort = 1;
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = idesc_bf16(2 * BM_CTA, BN, p.a_major, p.b_major);
      uint32_t it = 0, tile_it = 0;
      for (int64_t t = cluster_id; t < tiles && ok; t += n_clusters, ++tile_it) {
        const int acc = tile_it & 1;
        const uint32_t acc_ph = (tile_it >> 1) & 1;
        if (!(ok = mbar_wait_parked(&acc_empty[acc], acc_ph ^ 1, &s_abort))) break;
        tc_fence_after_sync();
        const uint32_t d = tm + acc * BN;
        for (int64_t kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!(ok = mbar_wait_parked(&full[s], ph, &s_abort))) break;
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + s * STAGE), sb = sa + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t da = (p.a_major == MAJOR_K) ? smem_desc(sa + k * 32, 16, 1024)
                                                       : smem_desc(sa + k * 2048, 8192, 1024);
            const uint64_t db = (p.b_major == MAJOR_K) ? smem_desc(sb + k * 32, 16, 1024)
                                                       : smem_desc(sb + k * 2048, 8192, 1024);
            mma_bf16_pair(d, da, db, idesc, (kb | k) != 0);
          }
          // the stage is reusable in both CTAs once these MMAs have read it
          mma_commit_pair(map_to_cta(smem_u32(&empty[s]), 0));
          mma_commit_pair(map_to_cta(smem_u32(&empty[s]), 1));
        }
        if (ok) {
          mma_commit_pair(map_to_cta(smem_u32(&acc_full[acc]), 0));
          mma_commit_pair(map_to_cta(smem_u32(&acc_full[acc]), 1));
        }
      }
      if (!ok) s_abort = 1;
    }
  } else {
    const int quarter = warp & 3;
    uint32_t tile_it = 0;
    for (int64_t t = cluster_id; t < tiles && ok; t += n_clusters, ++tile_it) {
      const int acc = tile_it & 1;
      const uint32_t acc_ph = (tile_it >> 1) & 1;
      const int64_t m0 = (p.m_fast ? t % m_tiles : t / n_tiles) * (2 * BM_CTA) + (int64_t)rank * BM_CTA;
      const int64_t n0 = (p.m_fast ? t / m_tiles : t % n_tiles) * BN;
      ok = mbar_wait_parked(&acc_full[acc], acc_ph, &s_abort);
      if (__any_sync(0xffffffffu, !ok)) { ok = false; break; }
      tc_fence_after_sync();
      const int64_t row = m0 + quarter * 32 + lane;
      __nv_bfloat16* crow = p.C + row * p.N + n0;
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        uint32_t r[32];
        tmem_ld32(tmem_addr(tm + acc * BN, quarter * 32, c), r);
        tmem_ld_wait();
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          float f[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(r[q * 8 + j]);
          uint4* dst = reinterpret_cast<uint4*>(crow + c + q * 8);
          if (p.accumulate) {
            const uint4 old = *dst;
            const __nv_bfloat162* ob = reinterpret_cast<const __nv_bfloat162*>(&old);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float2 o2 = __bfloat1622float2(ob[j]);
              f[2 * j] += o2.x;
              f[2 * j + 1] += o2.y;
            }
          }
          uint4 u;
          __nv_bfloat162 a0 = __floats2bfloat162_rn(f[0], f[1]), a1 = __floats2bfloat162_rn(f[2], f[3]);
          __nv_bfloat162 a2 = __floats2bfloat162_rn(f[4], f[5]), a3 = __floats2bfloat162_rn(f[6], f[7]);
          u.x = *reinterpret_cast<uint32_t*>(&a0);
          u.y = *reinterpret_cast<uint32_t*>(&a1);
          u.z = *reinterpret_cast<uint32_t*>(&a2);
          u.w = *reinterpret_cast<uint32_t*>(&a3);
          *dst = u;
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty[acc]), 0));
    }
    if (!ok) s_abort = 1;
  }
  tc_fence_before_sync();
  __syncthreads();
  if (tid == 0 && s_abort) atomicExch(p.status, 8);
  // neither CTA may leave (or free its TMEM) while the pair's MMAs can still touch its memory
  cluster_sync_all();
  if (warp == 1) tmem_dealloc_pair(tm, 2 * BN);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}
// 2-D bf16 row-major tensor [rows][cols]; box = (box_cols inner, box_rows), 128B swizzle
static bool make_map(CUtensorMap* m, const void* ptr, int64_t rows, int64_t cols, int box_cols, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
  cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
  cuuint32_t el[2] = {1, 1};
  const CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, el,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    fprintf(stderr, "[zc_gemm_2sm] cuTensorMapEncodeTiled failed (%d): ptr=%p rows=%lld cols=%lld box=(%d,%d)\n",
            (int)r, ptr, (long long)rows, (long long)cols, box_cols, box_rows);
  return r == CUDA_SUCCESS;
}

}  // namespace g2
}  // namespace zc

extern "C" {

int* zc_gemm_status_word();  // gemm_tcgen05.cu: the current device's GEMM status word

// Same contract as zc_gemm_bf16, for M % 256 == 0, N % 256 == 0, K % 64 == 0; shares its status word
// (zc_gemm_status_read_and_clear; code 8 = a bounded wait of this kernel expired).
int zc_gemm_bf16_2sm(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K, int trans_a, int trans_b,
                     int accumulate, cudaStream_t st) {
  using namespace zc;
  using namespace zc::g2;
  if (M <= 0 || N <= 0 || K <= 0 || M % (2 * BM_CTA) || N % BN || K % BK) return ERR_UNSUPPORTED;
  int* status = zc_gemm_status_word();
  if (!status) return ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) & 15)
    return ERR_UNSUPPORTED;
  int dev = 0;
  cudaGetDevice(&dev);
  cudaSetDevice(dev);
  const int a_major = trans_a ? MAJOR_MN : MAJOR_K;
  const int b_major = trans_b ? MAJOR_K : MAJOR_MN;
  CUtensorMap mapA, mapB;
  bool ok;
  if (a_major == MAJOR_K) ok = make_map(&mapA, A, M, K, BK, BM_CTA);
  else ok = make_map(&mapA, A, K, M, 64, BK);
  if (b_major == MAJOR_K) ok = ok && make_map(&mapB, B, N, K, BK, BN_CTA);
  else ok = ok && make_map(&mapB, B, K, N, 64, BK);
  if (!ok) return ERR_BAD_ARG;
  Params p;
  p.C = (__nv_bfloat16*)C; p.M = M; p.N = N; p.K = K;
  p.a_major = a_major; p.b_major = b_major; p.accumulate = accumulate;
  p.m_fast = (M <= N) ? 1 : 0;
  p.status = status;
  const int64_t tiles = (M / (2 * BM_CTA)) * (N / BN);
  const int clusters = (int)std::min<int64_t>(tiles, sm_count() / 2);
  const int smem = STAGES * STAGE + 1024;
  static bool attr = false;
  if (!attr) { cudaFuncSetAttribute(gemm_2sm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); attr = true; }
  gemm_2sm_kernel<<<2 * clusters, THREADS, smem, st>>>(mapA, mapB, p);
  return launch_status();
}

}  // extern "C"
