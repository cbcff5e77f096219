// One-CTA tcgen05 GEMM used to validate the operand descriptor conventions of umma.cuh.
//
// D[128,128] (fp32) = A[128,K] * B[128,K]^T for K = 64*ksteps, with each operand given either
// K-major (row-major [128][K]) or MN-major ([K][128]) in global memory.  Operands are staged by the
// threads into the 128B-swizzled layouts described in umma.cuh (the layouts a TMA load with
// SWIZZLE_128B produces), the MMAs are issued by one thread, and the accumulator is read back from
// TMEM.  Every wait is bounded; on expiry `status[0]` is set and the kernel leaves normally.
#include <cuda_bf16.h>

#include "launch_util.h"
#include "umma.cuh"

namespace zc {
using namespace umma;

// Stage one 64-wide K block of an operand with 128 M/N rows.
//   K-major : dst slab [128 rows x 128 B];  src row-major [128][ld], columns k0..k0+63
//   MN-major: two slabs (rows 0..63, 64..127), each [64 k-rows x 128 B]; src [K][128], rows k0..
__device__ void stage_operand(uint8_t* dst, const __nv_bfloat16* src, int major, int ld, int k0, int tid,
                              int nthr) {
  if (major == MAJOR_K) {
    for (int i = tid; i < 128 * 8; i += nthr) {
      const int row = i >> 3, chunk = i & 7;
      const uint4 v = *reinterpret_cast<const uint4*>(src + (size_t)row * ld + k0 + chunk * 8);
      *reinterpret_cast<uint4*>(dst + sw128_off(row, chunk)) = v;
    }
  } else {
    for (int i = tid; i < 2 * 64 * 8; i += nthr) {
      const int slab = i >> 9, krow = (i >> 3) & 63, chunk = i & 7;
      const uint4 v = *reinterpret_cast<const uint4*>(src + (size_t)(k0 + krow) * ld + slab * 64 + chunk * 8);
      *reinterpret_cast<uint4*>(dst + slab * 8192 + sw128_off(krow, chunk)) = v;
    }
  }
}

__global__ void __launch_bounds__(128) umma_selftest_kernel(const __nv_bfloat16* __restrict__ A,
                                                            const __nv_bfloat16* __restrict__ B,
                                                            float* __restrict__ D, int a_major, int b_major,
                                                            int ksteps, int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;           // 16 KB
  uint8_t* sB = smem + 16384;   // 16 KB
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_base;
  const int tid = threadIdx.x, warp = tid >> 5;
  const int K = 64 * ksteps;
  if (tid == 0) {
    mbar_init(&bar, 1);
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc(&tmem_base, 128);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tm = tmem_base;
  const uint32_t idesc = idesc_bf16(128, 128, a_major, b_major);
  bool ok = true;
  for (int ks = 0; ks < ksteps; ++ks) {
    stage_operand(sA, A, a_major, a_major == MAJOR_K ? K : 128, ks * 64, tid, 128);
    stage_operand(sB, B, b_major, b_major == MAJOR_K ? K : 128, ks * 64, tid, 128);
    fence_proxy_async_smem();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after_sync();
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const uint64_t da = (a_major == MAJOR_K) ? smem_desc(smem_u32(sA) + k * 32, 16, 1024)
                                                 : smem_desc(smem_u32(sA) + k * 2048, 8192, 1024);
        const uint64_t db = (b_major == MAJOR_K) ? smem_desc(smem_u32(sB) + k * 32, 16, 1024)
                                                 : smem_desc(smem_u32(sB) + k * 2048, 8192, 1024);
        mma_bf16(tm, da, db, idesc, (ks | k) != 0);
      }
      mma_commit(&bar);
    }
    // the staging buffers are reused next step: wait until the MMAs have read them
    ok = mbar_wait(&bar, ks & 1);
    if (!ok) break;
    tc_fence_after_sync();
  }
  if (ok) {
    // warp w reads TMEM lanes 32w..32w+31; thread t of the warp holds accumulator row 32w+t
#pragma unroll 1
    for (int c = 0; c < 128; c += 32) {
      uint32_t r[32];
      tmem_ld32(tmem_addr(tm, warp * 32, c), r);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; ++j) D[(size_t)tid * 128 + c + j] = __uint_as_float(r[j]);
    }
  } else if (tid == 0) {
    status[0] = 1;
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tm, 128);
}

}  // namespace zc

extern "C" int zc_umma_selftest(const void* A, const void* B, float* D, int a_major, int b_major, int ksteps,
                                int* status, cudaStream_t st) {
  static bool attr_set = false;
  const int smem = 32768 + 1024;
  if (!attr_set) {
    cudaFuncSetAttribute(zc::umma_selftest_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    attr_set = true;
  }
  zc::umma_selftest_kernel<<<1, 128, smem, st>>>((const __nv_bfloat16*)A, (const __nv_bfloat16*)B, D, a_major,
                                                 b_major, ksteps, status);
  return zc::launch_status();
}
