// Two-SM (cta_group::2) persistent bf16 GEMM for sm_100a: C[M,N] (+)= op(A) * op(B), fp32 accumulate.
//
// A cluster of two CTAs owns a 256 x 256 output tile.  Each CTA stages its own 128 rows of A and its
// own 128 of the tile's 256 columns of B; one thread of the even CTA issues
// tcgen05.mma.cta_group::2 (M = 256, N = 256, K = 16), which reads both CTAs' shared memory and
// accumulates each CTA's 128 rows into that CTA's TMEM.
//
//   warp 0      TMA producer (both CTAs): cp.async.bulk.tensor ... cta_group::2 loads into the CTA's
//               own stage buffers, transaction bytes counted on the even CTA's `full` barrier
//   warp 1      even CTA: MMA issuer; commits arrive on the `empty` / `acc_full` barriers of both CTAs
//   warps 2-5   epilogue (both CTAs): tcgen05.ld the CTA's 128 x 256 accumulator, convert, store;
//               arrivals of both CTAs' epilogue warps free the accumulator on the even CTA
// Every CTA fetches its own tiles with plain per-CTA TMA loads; no load is shared between CTAs.
//
// The issuing thread is the scarce resource: one thread has to launch a 128-clock MMA every 128
// clocks, so everything that can be is precomputed (stage-0 descriptors, remote barrier addresses)
// and the operand layouts are template parameters; per MMA the loop adds a constant to the
// descriptors and nothing else.
//
// Work is handed out dynamically.  The clusters take units from a global counter (the even CTA's
// producer thread fetches the next index and publishes it to every role of both CTAs through a small
// ring in shared memory), so a cluster that starts late, or not at all for a while, because another
// kernel (a collective running beside the GEMM) holds its SMs simply takes fewer units; with a
// static round-robin the whole GEMM would wait for that cluster's share.
// Units: whole tiles first, then the tiles of the last, partial wave are split
// along K into `split` slices each, so that all clusters stay busy to the end.  A slice writes its
// fp32 partial sums to a workspace and a small second kernel adds the slices and rounds to bf16.
// Every wait is bounded; on expiry the status word is set and both CTAs reach the teardown.
#include <cuda.h>
#include <cuda_bf16.h>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <mutex>

#include "launch_util.h"
#include "nvtx_util.h"
#include "umma.cuh"

namespace zc {
namespace g2 {
using namespace umma;

constexpr int BM_CTA = 128;   // rows of A per CTA (256 per cluster)
constexpr int BN_CTA = 128;   // columns of B staged per CTA (256 per cluster)
constexpr int BM = 256;
constexpr int BN = 256;       // accumulator columns
constexpr int BK = 64;
constexpr int STAGES = 6;
constexpr int THREADS = 192;
constexpr int A_BYTES = BM_CTA * BK * 2;  // 16 KB
constexpr int B_BYTES = BN_CTA * BK * 2;  // 16 KB
constexpr int STAGE = A_BYTES + B_BYTES;
constexpr int MAX_SPLIT = 4;
constexpr int SCHED = 4;       // slots of the unit-index ring
constexpr int COUNTER_SLOTS = 256;

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
__device__ __forceinline__ void tma_load_2d_pair(uint32_t smem_dst, const CUtensorMap* map, uint32_t bar_cluster_addr,
                                                 int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_dst), "l"(map), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
      : "memory");
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
__device__ __forceinline__ uint32_t mbar_addr_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}
__device__ __forceinline__ uint32_t mbar_addr_try_wait_cluster(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}
// the same wait with cluster-scope acquire: the arrival (and the data it publishes) came from the other CTA
__device__ __forceinline__ bool wait_bar_cluster(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_addr_try_wait_cluster(bar, parity)) return true;
  const unsigned long long t0 = globaltimer_ns();
  for (uint32_t it = 0;; ++it) {
    if (mbar_addr_try_wait_cluster(bar, parity)) return true;
    if ((it & 255u) == 255u && (*abort_flag || globaltimer_ns() - t0 > 2000000000ull)) return false;
  }
}
__device__ __forceinline__ void st_shared_cluster_u32(uint32_t cluster_addr, uint32_t v) {
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}
// bounded spin on a barrier given by its shared::cta address; the limit is only looked at on the slow path
__device__ __forceinline__ bool wait_bar(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_addr_try_wait(bar, parity)) return true;
  const unsigned long long t0 = globaltimer_ns();
  for (uint32_t it = 0;; ++it) {
    if (mbar_addr_try_wait(bar, parity)) return true;
    if ((it & 255u) == 255u && (*abort_flag || globaltimer_ns() - t0 > 2000000000ull)) return false;
  }
}

struct Params {
  __nv_bfloat16* C;
  float* partial;      // [tail tiles][split][256][256] fp32, or null when split == 1
  int64_t M, N, K;
  int64_t ldc;         // elements between rows of C (>= N rounded up to 8: whole 8-column groups are stored)
  const __nv_bfloat16* bias;  // [N] added to every row before rounding, or null
  int accumulate;
  int group_m;         // tiles are walked in bands of `group_m` m-tiles, n-major inside a band
  int full_tiles;      // tiles computed whole; the remaining tiles are split along K
  int split;           // K slices per tail tile (1: no tile is split)
  int* status;
  unsigned* counter;   // [0] units handed out beyond the first round, [1] clusters finished; both 0 at launch
};

// Tile order.  The clusters running at one time work on consecutive tile indices; walking bands of
// `group_m` m-tiles keeps that set a compact block of the output, so the A rows and B columns it
// needs together stay in L2 however large K is (a full column of m-tiles does not once M * K
// outgrows the cache).
// (32-bit arithmetic: the issuing thread pays for every instruction between two tiles.)
__device__ __forceinline__ void tile_coords(int t, int m_tiles, int n_tiles, int group_m, int& mi, int& ni) {
  const int per_band = group_m * n_tiles;
  const int band = t / per_band, r = t - band * per_band;
  const int rows = min(group_m, m_tiles - band * group_m);
  ni = r / rows;
  mi = band * group_m + (r - ni * rows);
}

// One unit of work: a tile and a range of its K blocks.
struct Unit {
  int mi, ni;
  int kb0, kb1;
  int slice;  // index of the fp32 partial slab, or -1 for a whole tile
};
__device__ __forceinline__ Unit unit_of(int u, const Params& p, int m_tiles, int n_tiles, int k_blocks) {
  Unit w;
  int t = u;
  w.kb0 = 0;
  w.kb1 = k_blocks;
  w.slice = -1;
  if (u >= p.full_tiles) {
    const int r = u - p.full_tiles;
    t = p.full_tiles + r / p.split;
    const int s = r % p.split;
    const int per = (k_blocks + p.split - 1) / p.split;
    w.kb0 = s * per;
    w.kb1 = min(k_blocks, w.kb0 + per);
    w.slice = r;
  }
  tile_coords(t, m_tiles, n_tiles, p.group_m, w.mi, w.ni);
  return w;
}

// f[j] += bias[col + j], j = 0..7 (col is a multiple of 8; the last group of a ragged N is read element-wise)
__device__ __forceinline__ void add_bias8(const __nv_bfloat16* bias, int64_t col, int64_t N, float (&f)[8]) {
  if (col + 8 <= N) {
    const uint4 b = __ldg(reinterpret_cast<const uint4*>(bias + col));
    const __nv_bfloat162* bb = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 t = __bfloat1622float2(bb[j]);
      f[2 * j] += t.x;
      f[2 * j + 1] += t.y;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (col + j < N) f[j] += __bfloat162float(bias[col + j]);
  }
}

template <int A_MAJOR, int B_MAJOR>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
    gemm_2sm_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t full[STAGES], empty[STAGES], acc_full[2], acc_empty[2];
  __shared__ uint64_t sched_full[SCHED], sched_empty[SCHED];
  __shared__ int sched_u[SCHED];
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
      mbar_init(&acc_full[a], 1);   // one commit per unit, on both CTAs
      mbar_init(&acc_empty[a], 8);  // used on the even CTA: four epilogue warps of each CTA
    }
    for (int q = 0; q < SCHED; ++q) {
      mbar_init(&sched_full[q], 1);    // the even CTA's producer publishes a unit index (in both CTAs)
      mbar_init(&sched_empty[q], 10);  // used on the even CTA: every other role of both CTAs has read it
    }
    mbar_fence_init();
    s_abort = 0;
    asm volatile("prefetch.tensormap [%0];" ::"l"(&mapA) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&mapB) : "memory");
  }
  if (warp == 1) {
    // each CTA allocates its own SM's whole TMEM (512 columns, so the base is column 0 in both)
    tmem_alloc(&tmem_base, 2 * BN);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers are initialised before any remote arrival
  tc_fence_after_sync();
  const uint32_t tm = tmem_base;
  // edge tiles: rows / columns / K blocks past the matrix read as zeros (TMA fill) and are not stored
  const int m_tiles = (int)((p.M + BM - 1) / BM), n_tiles = (int)((p.N + BN - 1) / BN);
  const int k_blocks = (int)((p.K + BK - 1) / BK);
  const int tiles = m_tiles * n_tiles;
  const int units = p.full_tiles + (tiles - p.full_tiles) * p.split;
  const int cluster_id = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t full_base = smem_u32(&full[0]), empty_base = smem_u32(&empty[0]);
  const uint32_t sfull_base = smem_u32(&sched_full[0]);
  const uint32_t sempty_c0 = map_to_cta(smem_u32(&sched_empty[0]), 0);  // the even CTA's sched_empty[0]
  bool ok = true;
  // Every role walks the same sequence of units, i = 0, 1, ...: slot i % SCHED of the ring holds the
  // i-th unit of this cluster (an index >= units ends the sequence).
  auto next_unit = [&](uint32_t i, bool& good) -> int {
    const uint32_t slot = i & (SCHED - 1), sph = (i / SCHED) & 1;
    good = rank == 0 ? wait_bar(sfull_base + 8 * slot, sph, &s_abort)
                     : wait_bar_cluster(sfull_base + 8 * slot, sph, &s_abort);
    return good ? sched_u[slot] : 0x7fffffff;
  };
  auto release_unit = [&](uint32_t i) { mbar_arrive_cluster(sempty_c0 + 8 * (i & (SCHED - 1))); };

  if (warp == 0) {
    if (lane == 0) {
      const uint32_t full0 = map_to_cta(full_base, 0);  // the even CTA's full[0]; full[s] is 8 s bytes on
      const uint32_t sfull_c1 = map_to_cta(sfull_base, 1);
      const uint32_t su_c1 = map_to_cta(smem_u32(&sched_u[0]), 1);
      uint32_t s = 0, ph = 0;
      for (uint32_t i = 0; ok; ++i) {
        int u;
        if (rank == 0) {
          // fetch the i-th unit and publish it to both CTAs
          const uint32_t slot = i & (SCHED - 1), sph = (i / SCHED) & 1;
          if (!(ok = wait_bar_cluster(smem_u32(&sched_empty[slot]), sph ^ 1, &s_abort))) break;
          u = (i == 0) ? cluster_id : n_clusters + (int)atomicAdd(p.counter, 1u);
          sched_u[slot] = u;
          st_shared_cluster_u32(su_c1 + 4 * slot, (uint32_t)u);
          mbar_arrive(&sched_full[slot]);
          mbar_arrive_cluster(sfull_c1 + 8 * slot);  // release.cluster: orders the store above
        } else {
          u = next_unit(i, ok);
          if (!ok) break;
          release_unit(i);
        }
        if (u >= units) break;
        const Unit w = unit_of(u, p, m_tiles, n_tiles, k_blocks);
        const int m0 = w.mi * BM + (int)rank * BM_CTA;
        const int n0 = w.ni * BN + (int)rank * BN_CTA;
        for (int kb = w.kb0; kb < w.kb1; ++kb) {
          if (!(ok = wait_bar(empty_base + 8 * s, ph ^ 1, &s_abort))) break;
          const uint32_t sa = smem_base + s * STAGE, sb = sa + A_BYTES;
          const uint32_t fb = full0 + 8 * s;
          if (rank == 0) mbar_expect_tx(&full[s], 2 * STAGE);  // both CTAs' bytes land on this barrier
          const int k0 = kb * BK;
          if (A_MAJOR == MAJOR_K) {
            tma_load_2d_pair(sa, &mapA, fb, k0, m0);
          } else {
#pragma unroll
            for (int sl = 0; sl < BM_CTA / 64; ++sl) tma_load_2d_pair(sa + sl * 8192, &mapA, fb, m0 + sl * 64, k0);
          }
          if (B_MAJOR == MAJOR_K) {
            tma_load_2d_pair(sb, &mapB, fb, k0, n0);
          } else {
#pragma unroll
            for (int sl = 0; sl < BN_CTA / 64; ++sl) tma_load_2d_pair(sb + sl * 8192, &mapB, fb, n0 + sl * 64, k0);
          }
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
      }
      if (!ok) s_abort = 1;
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = idesc_bf16(BM, BN, A_MAJOR, B_MAJOR);
      // descriptors of stage 0, K step 0; a stage adds STAGE >> 4, a K = 16 step adds KSTEP >> 4 to the
      // start-address field (shared memory is below 256 KB, so the 14-bit field never carries)
      const uint64_t a0 = (A_MAJOR == MAJOR_K) ? smem_desc(smem_base, 16, 1024) : smem_desc(smem_base, 8192, 1024);
      const uint64_t b0 = (B_MAJOR == MAJOR_K) ? smem_desc(smem_base + A_BYTES, 16, 1024)
                                               : smem_desc(smem_base + A_BYTES, 8192, 1024);
      constexpr uint64_t A_KSTEP = ((A_MAJOR == MAJOR_K) ? 32 : 2048) >> 4;
      constexpr uint64_t B_KSTEP = ((B_MAJOR == MAJOR_K) ? 32 : 2048) >> 4;
      constexpr uint64_t STAGE_STEP = STAGE >> 4;
      const uint32_t empty_c0 = map_to_cta(empty_base, 0), empty_c1 = map_to_cta(empty_base, 1);
      const uint32_t accf_c0 = map_to_cta(smem_u32(&acc_full[0]), 0), accf_c1 = map_to_cta(smem_u32(&acc_full[0]), 1);
      const uint32_t acce = smem_u32(&acc_empty[0]);
      uint32_t s = 0, ph = 0;
      for (uint32_t unit_it = 0; ok; ++unit_it) {
        const int u = next_unit(unit_it, ok);
        if (!ok) break;
        release_unit(unit_it);
        if (u >= units) break;
        const Unit w = unit_of(u, p, m_tiles, n_tiles, k_blocks);
        const uint32_t acc = unit_it & 1, acc_ph = (unit_it >> 1) & 1;
        if (!(ok = wait_bar_cluster(acce + 8 * acc, acc_ph ^ 1, &s_abort))) break;
        tc_fence_after_sync();
        const uint32_t d = tm + acc * BN;
        uint32_t accum = 0;
        for (int kb = w.kb0; kb < w.kb1; ++kb) {
          if (!(ok = wait_bar(full_base + 8 * s, ph, &s_abort))) break;
          const uint64_t da = a0 + s * STAGE_STEP, db = b0 + s * STAGE_STEP;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            mma_bf16_pair(d, da + k * A_KSTEP, db + k * B_KSTEP, idesc, accum);
            accum = 1;
          }
          // the stage is reusable in both CTAs once these MMAs have read it
          mma_commit_pair(empty_c0 + 8 * s);
          mma_commit_pair(empty_c1 + 8 * s);
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
        if (ok) {
          mma_commit_pair(accf_c0 + 8 * acc);
          mma_commit_pair(accf_c1 + 8 * acc);
        }
      }
      if (!ok) s_abort = 1;
    }
  } else {
    const int quarter = warp & 3;
    const uint32_t accf = smem_u32(&acc_full[0]);
    const uint32_t acce_c0 = map_to_cta(smem_u32(&acc_empty[0]), 0);
    for (uint32_t unit_it = 0; ok; ++unit_it) {
      const int u = next_unit(unit_it, ok);
      if (__any_sync(0xffffffffu, !ok)) { ok = false; break; }
      __syncwarp();
      if (lane == 0) release_unit(unit_it);
      if (u >= units) break;
      const Unit w = unit_of(u, p, m_tiles, n_tiles, k_blocks);
      const uint32_t acc = unit_it & 1, acc_ph = (unit_it >> 1) & 1;
      ok = wait_bar_cluster(accf + 8 * acc, acc_ph, &s_abort);
      if (__any_sync(0xffffffffu, !ok)) { ok = false; break; }
      tc_fence_after_sync();
      const int row_in_tile = (int)rank * BM_CTA + quarter * 32 + lane;
      if (w.slice < 0) {
        const int64_t row = (int64_t)w.mi * BM + row_in_tile;
        const int64_t col0 = (int64_t)w.ni * BN;
        __nv_bfloat16* crow = p.C + row * p.ldc + col0;
        const bool row_ok = row < p.M;
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
          uint32_t r[32];
          tmem_ld32(tmem_addr(tm + acc * BN, quarter * 32, c), r);
          tmem_ld_wait();
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            if (!row_ok || col0 + c + q * 8 >= p.N) continue;
            float f[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(r[q * 8 + j]);
            if (p.bias) add_bias8(p.bias, col0 + c + q * 8, p.N, f);
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
            uint4 v;
            __nv_bfloat162 a0 = __floats2bfloat162_rn(f[0], f[1]), a1 = __floats2bfloat162_rn(f[2], f[3]);
            __nv_bfloat162 a2 = __floats2bfloat162_rn(f[4], f[5]), a3 = __floats2bfloat162_rn(f[6], f[7]);
            v.x = *reinterpret_cast<uint32_t*>(&a0);
            v.y = *reinterpret_cast<uint32_t*>(&a1);
            v.z = *reinterpret_cast<uint32_t*>(&a2);
            v.w = *reinterpret_cast<uint32_t*>(&a3);
            *dst = v;
          }
        }
      } else {
        // K slice of a tail tile: fp32 partial sums, added up by gemm_2sm_fixup_kernel
        float* prow = p.partial + ((int64_t)w.slice * BM + row_in_tile) * BN;
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
          uint32_t r[32];
          tmem_ld32(tmem_addr(tm + acc * BN, quarter * 32, c), r);
          tmem_ld_wait();
#pragma unroll
          for (int q = 0; q < 8; ++q)
            reinterpret_cast<uint4*>(prow + c)[q] = make_uint4(r[4 * q], r[4 * q + 1], r[4 * q + 2], r[4 * q + 3]);
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(acce_c0 + 8 * acc);
    }
    if (!ok) s_abort = 1;
  }
  tc_fence_before_sync();
  __syncthreads();
  if (tid == 0 && s_abort) atomicExch(p.status, 8);
  // neither CTA may leave (or free its TMEM) while the pair's MMAs can still touch its memory
  cluster_sync_all();
  if (warp == 1) tmem_dealloc(tm, 2 * BN);
  if (tid == 0 && rank == 0) {
    // the last cluster to finish puts the counters back to zero for the next launch that uses this slot
    if (atomicAdd(p.counter + 1, 1u) == (unsigned)n_clusters - 1u) {
      p.counter[0] = 0u;
      p.counter[1] = 0u;
    }
  }
}

// C tile (+)= sum over the K slices of its fp32 partials, rounded once to bf16.
__global__ void __launch_bounds__(256) gemm_2sm_fixup_kernel(const Params p, int m_tiles, int n_tiles) {
  const int tail = blockIdx.y;  // index among the split tiles
  int mi, ni;
  tile_coords(p.full_tiles + tail, m_tiles, n_tiles, p.group_m, mi, ni);
  const float* base = p.partial + (int64_t)tail * p.split * (BM * BN);
  for (int i = blockIdx.x * 256 + threadIdx.x; i < BM * BN / 8; i += gridDim.x * 256) {
    const int row = i / (BN / 8), c8 = i % (BN / 8);
    if ((int64_t)mi * BM + row >= p.M || (int64_t)ni * BN + c8 * 8 >= p.N) continue;
    float f[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int s = 0; s < p.split; ++s) {
      const float4* src = reinterpret_cast<const float4*>(base + (int64_t)s * (BM * BN) + row * BN + c8 * 8);
      const float4 x = src[0], y = src[1];
      f[0] += x.x; f[1] += x.y; f[2] += x.z; f[3] += x.w;
      f[4] += y.x; f[5] += y.y; f[6] += y.z; f[7] += y.w;
    }
    if (p.bias) add_bias8(p.bias, (int64_t)ni * BN + c8 * 8, p.N, f);
    uint4* dst = reinterpret_cast<uint4*>(p.C + ((int64_t)mi * BM + row) * p.ldc + (int64_t)ni * BN + c8 * 8);
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
    uint4 v;
    __nv_bfloat162 a0 = __floats2bfloat162_rn(f[0], f[1]), a1 = __floats2bfloat162_rn(f[2], f[3]);
    __nv_bfloat162 a2 = __floats2bfloat162_rn(f[4], f[5]), a3 = __floats2bfloat162_rn(f[6], f[7]);
    v.x = *reinterpret_cast<uint32_t*>(&a0);
    v.y = *reinterpret_cast<uint32_t*>(&a1);
    v.z = *reinterpret_cast<uint32_t*>(&a2);
    v.w = *reinterpret_cast<uint32_t*>(&a3);
    *dst = v;
  }
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
// 2-D bf16 row-major tensor [rows][cols] with rows `ld` elements apart; box = (box_cols inner, box_rows),
// 128B swizzle.  Elements past `cols` in a row (padding up to ld) are outside the map and read as zeros.
static bool make_map(CUtensorMap* m, const void* ptr, int64_t rows, int64_t cols, int64_t ld, int box_cols, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
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

// Per-device launch state: how many clusters of two the device runs at once, and the fp32 workspace
// of the split tail (grown on demand, never shrunk; growing it is the only allocation this file
// makes and it happens before the launch that needs it).
struct DeviceState {
  bool ready = false;
  int clusters = 0;
  float* partial = nullptr;
  size_t partial_elems = 0;
  unsigned* counters = nullptr;  // COUNTER_SLOTS pairs, all zero between launches; launches take slots in turn
  unsigned next_slot = 0;
};
static DeviceState g_state[64];
static std::mutex g_mutex;

template <int A_MAJOR, int B_MAJOR>
static int max_clusters(int smem) {
  cudaFuncSetAttribute(gemm_2sm_kernel<A_MAJOR, B_MAJOR>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * (sm_count() / 2));
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = smem;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = 2;
  at[0].val.clusterDim.y = 1;
  at[0].val.clusterDim.z = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, gemm_2sm_kernel<A_MAJOR, B_MAJOR>, &cfg) != cudaSuccess || n <= 0) {
    cudaGetLastError();
    n = sm_count() / 2;
  }
  return std::min(n, sm_count() / 2);
}

}  // namespace g2
}  // namespace zc

extern "C" {

int* zc_gemm_status_word();  // gemm_tcgen05.cu: the current device's GEMM status word

// Same contract as zc_gemm_bf16 with explicit leading dimensions: lda / ldb / ldc are the distances in
// elements between consecutive rows of the STORED A, B and C ([M,K] or [K,M]; [N,K] or [K,N]; [M,N]).
// M, N and K are free; every leading dimension must be a multiple of 8 (16 bytes) and ldc at least N
// rounded up to 8, because C is stored in whole 8-column groups (the up to 7 padding columns after
// column N of a row are written too: with zeros, since the operand columns they multiply are outside the
// tensor map and load as zeros).  Edge tiles are zero-filled on load and masked on store.  Shares zc_gemm_bf16's status word
// (zc_gemm_status_read_and_clear; code 8 = a bounded wait of this kernel expired).
// `bias`: null, or N bf16 values (16-byte aligned) added to every row of the product before it is rounded
// (and before the old C is added when `accumulate` is set).
int zc_gemm_bf16_2sm_bias(const void* A, const void* B, void* C, const void* bias, int64_t M, int64_t N, int64_t K,
                          int64_t lda, int64_t ldb, int64_t ldc, int trans_a, int trans_b, int accumulate,
                          cudaStream_t st) {
  ZC_NVTX_RANGE("zc_gemm_bf16_2sm");
  if (reinterpret_cast<uintptr_t>(bias) & 15) return zc::ERR_UNSUPPORTED;
  using namespace zc;
  using namespace zc::g2;
  if (M <= 0 || N <= 0 || K <= 0) return ERR_UNSUPPORTED;
  if (lda % 8 || ldb % 8 || ldc % 8 || ldc < ((N + 7) / 8) * 8) return ERR_UNSUPPORTED;
  if (lda < (trans_a ? M : K) || ldb < (trans_b ? K : N)) return ERR_BAD_ARG;
  const int64_t m_tiles = (M + BM - 1) / BM, n_tiles = (N + BN - 1) / BN;
  if (m_tiles * n_tiles > (1 << 28)) return ERR_UNSUPPORTED;
  int* status = zc_gemm_status_word();
  if (!status) return ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) & 15)
    return ERR_UNSUPPORTED;
  int dev = 0;
  cudaGetDevice(&dev);
  cudaSetDevice(dev);
  if (dev < 0 || dev >= 64) return ERR_BAD_ARG;
  const int a_major = trans_a ? MAJOR_MN : MAJOR_K;
  const int b_major = trans_b ? MAJOR_K : MAJOR_MN;
  if (a_major == MAJOR_MN && b_major == MAJOR_K) return ERR_UNSUPPORTED;  // no layer GEMM has this form
  CUtensorMap mapA, mapB;
  bool ok;
  if (a_major == MAJOR_K) ok = make_map(&mapA, A, M, K, lda, BK, BM_CTA);
  else ok = make_map(&mapA, A, K, M, lda, 64, BK);
  if (b_major == MAJOR_K) ok = ok && make_map(&mapB, B, N, K, ldb, BK, BN_CTA);
  else ok = ok && make_map(&mapB, B, K, N, ldb, 64, BK);
  if (!ok) return ERR_BAD_ARG;
  const int smem = STAGES * STAGE + 1024;
  DeviceState& ds = g_state[dev];
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    if (!ds.ready) {
      int c = max_clusters<MAJOR_K, MAJOR_K>(smem);
      c = std::min(c, max_clusters<MAJOR_K, MAJOR_MN>(smem));
      c = std::min(c, max_clusters<MAJOR_MN, MAJOR_MN>(smem));
      ds.clusters = c;
      if (cudaMalloc(&ds.counters, 2 * COUNTER_SLOTS * sizeof(unsigned)) != cudaSuccess) return ERR_BAD_ARG;
      cudaMemset(ds.counters, 0, 2 * COUNTER_SLOTS * sizeof(unsigned));
      ds.ready = true;
    }
  }
  Params p;
  p.C = (__nv_bfloat16*)C; p.M = M; p.N = N; p.K = K; p.ldc = ldc;
  p.bias = (const __nv_bfloat16*)bias;
  p.accumulate = accumulate;
  static const int forced_gm = getenv("ZC_GEMM_GROUP_M") ? atoi(getenv("ZC_GEMM_GROUP_M")) : 0;
  static const int forced_split = getenv("ZC_GEMM_SPLIT") ? atoi(getenv("ZC_GEMM_SPLIT")) : -1;
  p.group_m = forced_gm > 0 ? forced_gm : 8;
  p.status = status;
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    p.counter = ds.counters + 2 * (ds.next_slot++ % COUNTER_SLOTS);
  }
  const int64_t tiles = m_tiles * n_tiles;
  const int64_t k_blocks = (K + BK - 1) / BK;
  const int clusters = (int)std::min<int64_t>(tiles, ds.clusters);
  // Tail: the tiles of the last, partial wave are cut into K slices so that every cluster has one
  // unit of about the same length to finish with.
  const int64_t rem = tiles % clusters;
  int split = 1;
  if (rem > 0 && tiles > clusters) {
    split = (int)std::min<int64_t>(std::min<int64_t>(clusters / rem, MAX_SPLIT), k_blocks / 8);
    if (forced_split >= 0) split = std::min(forced_split, MAX_SPLIT);
    if (split < 2 || rem * 10 > (int64_t)clusters * 8) split = 1;  // a nearly full last wave is left alone
  }
  p.split = split;
  p.full_tiles = (int)(split > 1 ? tiles - rem : tiles);
  p.partial = nullptr;
  if (split > 1) {
    const size_t need = (size_t)rem * split * BM * BN;
    std::lock_guard<std::mutex> lock(g_mutex);
    if (ds.partial_elems < need) {
      // earlier launches may still read the old buffer: drain the device before replacing it
      if (ds.partial) { cudaDeviceSynchronize(); cudaFree(ds.partial); ds.partial = nullptr; ds.partial_elems = 0; }
      const size_t want = std::max(need, (size_t)ds.clusters * BM * BN);
      if (cudaMalloc(&ds.partial, want * sizeof(float)) != cudaSuccess) {
        cudaGetLastError();
        p.split = 1;
        p.full_tiles = (int)tiles;
      } else {
        ds.partial_elems = want;
      }
    }
    p.partial = ds.partial;
  }
  const dim3 grid(2 * clusters);
  if (a_major == MAJOR_K && b_major == MAJOR_K) gemm_2sm_kernel<MAJOR_K, MAJOR_K><<<grid, THREADS, smem, st>>>(mapA, mapB, p);
  else if (a_major == MAJOR_K) gemm_2sm_kernel<MAJOR_K, MAJOR_MN><<<grid, THREADS, smem, st>>>(mapA, mapB, p);
  else gemm_2sm_kernel<MAJOR_MN, MAJOR_MN><<<grid, THREADS, smem, st>>>(mapA, mapB, p);
  int rc = launch_status();
  if (rc == 0 && p.split > 1) {
    gemm_2sm_fixup_kernel<<<dim3(16, (unsigned)rem), 256, 0, st>>>(p, (int)m_tiles, (int)n_tiles);
    rc = launch_status();
  }
  return rc;
}

int zc_gemm_bf16_2sm_ld(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K, int64_t lda,
                        int64_t ldb, int64_t ldc, int trans_a, int trans_b, int accumulate, cudaStream_t st) {
  return zc_gemm_bf16_2sm_bias(A, B, C, nullptr, M, N, K, lda, ldb, ldc, trans_a, trans_b, accumulate, st);
}

// Contiguous operands: M, N and K multiples of 8.
int zc_gemm_bf16_2sm(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K, int trans_a, int trans_b,
                     int accumulate, cudaStream_t st) {
  if (M % 8 || N % 8 || K % 8) return zc::ERR_UNSUPPORTED;
  return zc_gemm_bf16_2sm_ld(A, B, C, M, N, K, trans_a ? M : K, trans_b ? K : N, N, trans_a, trans_b, accumulate, st);
}

}  // extern "C"
