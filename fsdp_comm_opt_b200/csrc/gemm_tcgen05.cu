// Persistent, warp-specialised bf16 GEMM for sm_100a:  C[M,N] (+)= op(A) * op(B), fp32 accumulate.
//
//   warp 0      TMA producer: cp.async.bulk.tensor loads of A and B tiles into a 4-stage ring of
//               128B-swizzled shared-memory buffers, completion on mbarriers; every CTA loads
//               its own tiles (plain per-CTA TMA, nothing is shared across CTAs)
//   warp 1      MMA issuer: one elected thread issues tcgen05.mma (M=128, N=BN, K=16) into one of
//               two TMEM accumulators; tcgen05.commit releases smem stages and publishes tiles
//   warps 2-5   epilogue: tcgen05.ld the finished accumulator (while the next tile's MMAs run into
//               the other accumulator), convert to bf16, 16-byte stores to C
// One CTA per SM loops over output tiles (m fastest, so a B tile is reused from L2 by all m-tiles).
//
// The three GEMMs of a linear layer map to operand "major" flags instead of transposed copies:
//   forward  y  = x  w^T   A = x  [M,K] K-major            B = w [N,K] K-major
//   dgrad    dx = dy w     A = dy [M,K] K-major            B = w [K,N] MN-major
//   wgrad    dw = dy^T x   A = dy [K,M] MN-major           B = x [K,N] MN-major
// Every wait is bounded; on expiry the status word is set and the CTA tears down normally.
#include <cuda.h>
#include <cuda_bf16.h>

#include <cstdio>
#include <cstdlib>

#include "launch_util.h"
#include "nvtx_util.h"
#include "umma.cuh"

namespace zc {
using namespace umma;

constexpr int G_BM = 128;
constexpr int G_BK = 64;
constexpr int G_STAGES = 4;
constexpr int G_THREADS = 192;

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void prefetch_tmap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

struct GemmParams {
  __nv_bfloat16* C;
  int64_t M, N, K;
  int a_major, b_major, accumulate;
  int group_m;  // tiles are walked in bands of `group_m` m-tiles, n-major inside a band
  int* status;
};

// Tile order: bands of `group_m` m-tiles keep the tiles in flight a compact block of the output, so
// the A rows and B columns they share stay in L2 however large K is.
__device__ __forceinline__ void tile_coords(int64_t t, int64_t m_tiles, int64_t n_tiles, int group_m, int64_t& mi,
                                            int64_t& ni) {
  const int64_t per_band = (int64_t)group_m * n_tiles;
  const int64_t band = t / per_band, r = t - band * per_band;
  const int64_t rows = min((int64_t)group_m, m_tiles - band * group_m);
  mi = band * group_m + r % rows;
  ni = r / rows;
}

template <int BN>
__global__ void __launch_bounds__(G_THREADS, 1) gemm_kernel(const __grid_constant__ CUtensorMap mapA,
                                                            const __grid_constant__ CUtensorMap mapB,
                                                            const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int A_BYTES = G_BM * G_BK * 2;  // 16 KB
  constexpr int B_BYTES = BN * G_BK * 2;    // 32 KB (BN=256) / 16 KB (BN=128)
  constexpr int STAGE = A_BYTES + B_BYTES;
  __shared__ uint64_t full[G_STAGES], empty[G_STAGES], acc_full[2], acc_empty[2];
  __shared__ uint32_t tmem_base;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    for (int s = 0; s < G_STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 4);  // one arrival per epilogue warp
    }
    mbar_fence_init();
    prefetch_tmap(&mapA);
    prefetch_tmap(&mapB);
  }
  if (warp == 1) {
    tmem_alloc(&tmem_base, 2 * BN);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tm = tmem_base;
  const int64_t m_tiles = p.M / G_BM, n_tiles = p.N / BN, k_blocks = p.K / G_BK;
  const int64_t tiles = m_tiles * n_tiles;
  bool ok = true;

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;
      for (int64_t t = blockIdx.x; t < tiles && ok; t += gridDim.x) {
        int64_t mi, ni;
        tile_coords(t, m_tiles, n_tiles, p.group_m, mi, ni);
        const int m0 = (int)mi * G_BM, n0 = (int)ni * BN;
        for (int64_t kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % G_STAGES;
          const uint32_t ph = (it / G_STAGES) & 1;
          if (!(ok = mbar_wait(&empty[s], ph ^ 1))) break;
          uint8_t* sa = smem + s * STAGE;
          uint8_t* sb = sa + A_BYTES;
          mbar_expect_tx(&full[s], STAGE);
          const int k0 = (int)kb * G_BK;
          if (p.a_major == MAJOR_K) {
            tma_load_2d(sa, &mapA, &full[s], k0, m0);
          } else {
#pragma unroll
            for (int sl = 0; sl < G_BM / 64; ++sl) tma_load_2d(sa + sl * 8192, &mapA, &full[s], m0 + sl * 64, k0);
          }
          if (p.b_major == MAJOR_K) {
            tma_load_2d(sb, &mapB, &full[s], k0, n0);
          } else {
#pragma unroll
            for (int sl = 0; sl < BN / 64; ++sl) tma_load_2d(sb + sl * 8192, &mapB, &full[s], n0 + sl * 64, k0);
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = idesc_bf16(G_BM, BN, p.a_major, p.b_major);
      uint32_t it = 0, tile_it = 0;
      for (int64_t t = blockIdx.x; t < tiles && ok; t += gridDim.x, ++tile_it) {
        const int acc = tile_it & 1;
        const uint32_t acc_ph = (tile_it >> 1) & 1;
        if (!(ok = mbar_wait(&acc_empty[acc], acc_ph ^ 1))) break;
        tc_fence_after_sync();
        const uint32_t d = tm + acc * BN;
        for (int64_t kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % G_STAGES;
          const uint32_t ph = (it / G_STAGES) & 1;
          if (!(ok = mbar_wait(&full[s], ph))) break;
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + s * STAGE), sb = sa + A_BYTES;
#pragma unroll
          for (int k = 0; k < G_BK / 16; ++k) {
            const uint64_t da = (p.a_major == MAJOR_K) ? smem_desc(sa + k * 32, 16, 1024)
                                                       : smem_desc(sa + k * 2048, 8192, 1024);
            const uint64_t db = (p.b_major == MAJOR_K) ? smem_desc(sb + k * 32, 16, 1024)
                                                       : smem_desc(sb + k * 2048, 8192, 1024);
            mma_bf16(d, da, db, idesc, (kb | k) != 0);
          }
          mma_commit(&empty[s]);  // stage reusable once these MMAs have read it
        }
        if (ok) mma_commit(&acc_full[acc]);
      }
    }
  } else {
    // epilogue warps 2..5; TMEM lane quarter is fixed by warp id modulo 4
    const int quarter = warp & 3;
    uint32_t tile_it = 0;
    for (int64_t t = blockIdx.x; t < tiles && ok; t += gridDim.x, ++tile_it) {
      const int acc = tile_it & 1;
      const uint32_t acc_ph = (tile_it >> 1) & 1;
      int64_t mi, ni;
      tile_coords(t, m_tiles, n_tiles, p.group_m, mi, ni);
      const int64_t m0 = mi * G_BM, n0 = ni * BN;
      if (!(ok = mbar_wait(&acc_full[acc], acc_ph))) break;
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
      if (lane == 0) mbar_arrive(&acc_empty[acc]);
    }
  }
  if (!ok) atomicExch(p.status, 3);
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tm, 2 * BN);
}

// ---- host side ----------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
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
    fprintf(stderr, "[zc_gemm] cuTensorMapEncodeTiled failed (%d): ptr=%p rows=%lld cols=%lld box=(%d,%d)\n", (int)r,
            ptr, (long long)rows, (long long)cols, box_cols, box_rows);
  return r == CUDA_SUCCESS;
}

static int* gemm_status(int dev) {
  static int* st[64] = {nullptr};
  if (!st[dev]) {
    if (cudaMalloc(&st[dev], sizeof(int)) != cudaSuccess) return nullptr;
    cudaMemset(st[dev], 0, sizeof(int));
  }
  return st[dev];
}

}  // namespace zc

extern "C" {

// device pointer of the current device's GEMM status word (shared with the two-SM kernel)
int* zc_gemm_status_word() {
  int dev = 0;
  cudaGetDevice(&dev);
  return zc::gemm_status(dev);
}

int zc_gemm_status_read_and_clear() {
  int dev = 0;
  cudaGetDevice(&dev);
  int* st = zc::gemm_status(dev);
  if (!st) return -1;
  int v = 0;
  cudaMemcpy(&v, st, sizeof(int), cudaMemcpyDeviceToHost);
  if (v) cudaMemset(st, 0, sizeof(int));
  return v;
}

// C[M,N] (+)= op(A) op(B).  trans_a: A stored [K,M]; trans_b: B stored [N,K] (the nn.Linear weight).
int zc_gemm_bf16(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K, int trans_a, int trans_b,
                 int accumulate, cudaStream_t st) {
  ZC_NVTX_RANGE("zc_gemm_bf16");
  using namespace zc;
  if (M <= 0 || N <= 0 || K <= 0 || M % G_BM || N % 128 || K % G_BK) return ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) & 15)
    return ERR_UNSUPPORTED;
  int dev = 0;
  cudaGetDevice(&dev);
  // autograd worker threads may not have the primary context bound yet; the driver-API tensor-map
  // encoder needs a current context on the calling thread
  cudaSetDevice(dev);
  const int a_major = trans_a ? MAJOR_MN : MAJOR_K;   // A stored [K,M] -> M contiguous
  const int b_major = trans_b ? MAJOR_K : MAJOR_MN;   // B stored [N,K] -> K contiguous
  // Tile width 256 whenever N allows it.  128x128 tiles need 128 B/clk of operand traffic per SM,
  // which is more than the L2 can feed (measured: 865 TFLOP/s on 4096x4096x14336 against 1295
  // with 128x256 tiles), so a better wave count does not pay for the narrower tile.
  int BN = (N % 256 == 0) ? 256 : 128;
  {
    static const int force = getenv("ZC_GEMM_BN") ? atoi(getenv("ZC_GEMM_BN")) : 0;
    if (force == 128) BN = 128;
  }
  CUtensorMap mapA, mapB;
  bool ok;
  if (a_major == MAJOR_K) ok = make_map(&mapA, A, M, K, G_BK, G_BM);
  else ok = make_map(&mapA, A, K, M, 64, G_BK);
  if (b_major == MAJOR_K) ok = ok && make_map(&mapB, B, N, K, G_BK, BN);
  else ok = ok && make_map(&mapB, B, K, N, 64, G_BK);
  if (!ok) return ERR_BAD_ARG;
  GemmParams p;
  p.C = (__nv_bfloat16*)C; p.M = M; p.N = N; p.K = K;
  p.a_major = a_major; p.b_major = b_major; p.accumulate = accumulate;
  {
    static const int forced = getenv("ZC_GEMM_GROUP_M") ? atoi(getenv("ZC_GEMM_GROUP_M")) : 0;
    p.group_m = forced > 0 ? forced : 16;
  }
  p.status = gemm_status(dev);
  if (!p.status) {
    fprintf(stderr, "[zc_gemm] could not allocate the status word on device %d\n", dev);
    return ERR_BAD_ARG;
  }
  const int64_t tiles = (M / G_BM) * (N / BN);
  const int grid = (int)std::min<int64_t>(tiles, sm_count());
  static bool attr_all[64][2] = {{false, false}};  // per device
  bool* attr = attr_all[dev & 63];
  if (BN == 256) {
    const int smem = G_STAGES * (16384 + 32768) + 1024;
    if (!attr[0]) { cudaFuncSetAttribute(gemm_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); attr[0] = true; }
    gemm_kernel<256><<<grid, G_THREADS, smem, st>>>(mapA, mapB, p);
  } else {
    const int smem = G_STAGES * (16384 + 16384) + 1024;
    if (!attr[1]) { cudaFuncSetAttribute(gemm_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); attr[1] = true; }
    gemm_kernel<128><<<grid, G_THREADS, smem, st>>>(mapA, mapB, p);
  }
  return launch_status();
}

}  // extern "C"
