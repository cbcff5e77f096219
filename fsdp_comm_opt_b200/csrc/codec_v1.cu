// v1 (window-7) codec kernels for sm_100a: the wire format of the reference's hopper_fastzip2
// streams (reference: zipccl/hopper_zip.cu), produced and consumed by new kernels.
//
// Differences in how the work is done (the bytes on the wire are the same fields):
//   * bit planes, codes and sign/mantissa bytes are built four elements at a time on packed bytes
//     (codec_dev.cuh) instead of 32-iteration scalar loops, straight from registers;
//   * outliers are first stored block-locally (fixed 4096-byte stride, no atomics); a one-CTA-per-
//     work scan turns the per-block counts into offsets and a compaction pass packs the bytes, so
//     the outlier stream is in element order and the result is deterministic;
//   * one decode kernel serves the fused/split x plain/unpad/unpad_v variants;
//   * sizes and offsets are 64-bit; ragged tails and unaligned outputs take a scalar path.
//
// Encode = 3 launches (encode, scan, compact); decode = 1 launch.  No host sync, no allocation.
#include "codec_dev.cuh"
#include "launch_util.h"

namespace zc {

struct V1Where {
  int work;          // -1: block past the last work
  int blk;           // block index inside the work
  long long n;       // padded elements of the work
  long long det_off; // byte offset of the work's stream (split: det stream, fused: scratch/final)
  long long aux_off; // split: offset into the outlier scratch / compacted stream; fused: unused
  long long in_off;  // element offset of the work in the dense input
  long long valid;   // valid elements of the work
  long long pad_off; // sum of padded sizes of the previous works
};

enum : int { LAYOUT_SPLIT = 0, LAYOUT_FUSED = 1 };

// Fused scratch layout of one work (stride 4*n): [0, det) det fields, [S, S+n) staged outliers.
__device__ __host__ inline long long fused_stage_off(long long n) { return align128(v1_det_bytes(n) + n); }

// Locate block `b`.  Thread 0 scans the (few) works; result is broadcast through shared memory.
// aux_stride: 0 -> aux advances by n (encode scratch); else -> by align128(nbytes_8[i]) (decode).
__device__ __forceinline__ void v1_locate(long long b, const int* n_8, const int* orig_n, const int* nbytes_8,
                                          int n_works, int layout, bool decode, long long total_n,
                                          V1Where& w) {
  long long blk0 = 0, det = 0, aux = 0, in_off = 0, pad = 0;
  w.work = -1;
  for (int i = 0; i < n_works; ++i) {
    const long long n = n_8[i];
    const long long nb = n / V1_BLOCK_ELEMS;
    if (b >= blk0 && b < blk0 + nb) {
      w.work = i; w.blk = (int)(b - blk0); w.n = n; w.det_off = det; w.aux_off = aux;
      w.in_off = in_off; w.pad_off = pad;
      if (orig_n) w.valid = orig_n[i];
      else {
        long long v = total_n - in_off;
        w.valid = v < 0 ? 0 : (v > n ? n : v);
      }
      return;
    }
    blk0 += nb;
    pad += n;
    in_off += orig_n ? (long long)orig_n[i] : n;
    if (layout == LAYOUT_SPLIT) {
      det += n ? align128(v1_det_bytes(n)) : 0;
      aux += decode ? align128((long long)nbytes_8[i]) : n;
    } else {
      det += decode ? (long long)nbytes_8[i] : 4 * n;
    }
  }
}

struct V1Fields {
  uint8_t* sm;
  uint32_t* b0;
  uint32_t* b1;
  uint32_t* b2;
  int* boff;
};

__device__ __forceinline__ V1Fields v1_fields(uint8_t* stream, long long n) {
  V1Fields f;
  f.sm = stream;
  f.b0 = reinterpret_cast<uint32_t*>(stream + n);
  f.b1 = f.b0 + n / 32;
  f.b2 = f.b1 + n / 32;
  f.boff = reinterpret_cast<int*>(f.b2 + n / 32);
  return f;
}

// ---------------------------------------------------------------------------------------------
// encode: one CTA of 128 threads per 4096-element block
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128) v1_encode_kernel(
    const uint16_t* __restrict__ in, long long total_n, const int* __restrict__ n_8,
    const int* __restrict__ orig_n, int n_works, const int* __restrict__ bases, int layout,
    uint8_t* __restrict__ stream, uint8_t* __restrict__ stage) {
  __shared__ V1Where sw;
  __shared__ int warp_tot[4];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) v1_locate(blockIdx.x, n_8, orig_n, nullptr, n_works, layout, false, total_n, sw);
  __syncthreads();
  const V1Where w = sw;
  if (w.work < 0) return;
  const int base = bases[0];
  const long long e0 = (long long)w.blk * V1_BLOCK_ELEMS + tid * 32;
  const uint16_t* src = in + w.in_off + e0;
  LaneIn li;
  load_lane(src, w.valid - e0, (reinterpret_cast<uintptr_t>(src) & 15) == 0, li);
  LaneSplit s;
  split_lane(li, s);
  uint32_t code[8];
  codes_lane(s, base, 7u, code);
  if (base > 249) {
    // window would wrap past exponent 255: codes above 256-base do not exist
    const uint32_t lim = 256u - (uint32_t)base;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      uint32_t c = code[k], r = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t v = (c >> (8 * j)) & 0xFFu;
        r |= (v <= lim ? v : 0u) << (8 * j);
      }
      code[k] = r;
    }
  }
  const uint32_t zm = zero_mask(code);
  int wtot;
  const int pos_in_warp = warp_excl_scan(__popc(zm), lane, wtot);
  if (lane == 0) warp_tot[warp] = wtot;
  __syncthreads();
  int before = 0, total = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    before += (i < warp) ? warp_tot[i] : 0;
    total += warp_tot[i];
  }
  uint8_t* wstream = stream + w.det_off;
  const V1Fields f = v1_fields(wstream, w.n);
  uint4* smp = reinterpret_cast<uint4*>(f.sm + e0);
  smp[0] = make_uint4(s.sm[0], s.sm[1], s.sm[2], s.sm[3]);
  smp[1] = make_uint4(s.sm[4], s.sm[5], s.sm[6], s.sm[7]);
  const long long widx = (long long)w.blk * V1_THREADS + tid;
  f.b0[widx] = plane_word<0>(code);
  f.b1[widx] = plane_word<1>(code);
  f.b2[widx] = plane_word<2>(code);
  const long long nb = w.n / V1_BLOCK_ELEMS;
  if (tid == 0) {
    f.boff[w.blk] = total;  // count for now; the scan kernel turns it into the offset
    if (w.blk == 0) f.boff[nb] = base;
  }
  uint8_t* st = (layout == LAYOUT_SPLIT) ? stage + w.aux_off : wstream + fused_stage_off(w.n);
  scatter_escapes(st + (long long)w.blk * V1_BLOCK_ELEMS + before + pos_in_warp, s, zm);
}

// ---------------------------------------------------------------------------------------------
// scan: one CTA per work turns per-block counts into exclusive offsets, writes totals / sizes
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(1024) v1_scan_kernel(const int* __restrict__ n_8, int n_works, int layout,
                                                       uint8_t* __restrict__ stream, int* __restrict__ counts,
                                                       int* __restrict__ nbytes_8) {
  __shared__ int wsum[32];
  __shared__ long long s_off;
  __shared__ int s_carry, s_chunk;
  const int i = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) {
    long long det = 0;
    for (int j = 0; j < i; ++j) {
      const long long n = n_8[j];
      det += (layout == LAYOUT_SPLIT) ? (n ? align128(v1_det_bytes(n)) : 0) : 4 * n;
    }
    s_off = det;
    s_carry = 0;
  }
  __syncthreads();
  const long long n = n_8[i];
  const long long nb = n / V1_BLOCK_ELEMS;
  if (n == 0) {
    if (tid == 0) { counts[i] = 0; if (nbytes_8) nbytes_8[i] = 0; }
    return;
  }
  int* boff = v1_fields(stream + s_off, n).boff;
  for (long long start = 0; start < nb; start += 1024) {
    const long long b = start + tid;
    const int v = b < nb ? boff[b] : 0;
    int tot;
    const int ex = warp_excl_scan(v, lane, tot);
    if (lane == 0) wsum[warp] = tot;
    __syncthreads();
    if (warp == 0) {
      int t2;
      const int e2 = warp_excl_scan(wsum[lane], lane, t2);
      wsum[lane] = e2;
      if (lane == 0) s_chunk = t2;
    }
    __syncthreads();
    const int carry = s_carry;
    if (b < nb) boff[b] = carry + wsum[warp] + ex;
    __syncthreads();
    if (tid == 0) s_carry = carry + s_chunk;
    __syncthreads();
  }
  if (tid == 0) {
    const int total = s_carry;
    counts[i] = total;
    if (nbytes_8) nbytes_8[i] = (int)align128(v1_det_bytes(n) + total);
  }
}

// ---------------------------------------------------------------------------------------------
// compact: block-local outliers (and, for the fused layout, the det fields) -> final streams
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void copy_bytes(uint8_t* dst, const uint8_t* src, long long nbytes, int tid, int nthr) {
  if (dst == src || nbytes <= 0) return;
  if (((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) & 15) == 0) {
    const long long nv = nbytes / 16;
    for (long long k = tid; k < nv; k += nthr)
      reinterpret_cast<uint4*>(dst)[k] = reinterpret_cast<const uint4*>(src)[k];
    for (long long k = nv * 16 + tid; k < nbytes; k += nthr) dst[k] = src[k];
  } else {
    for (long long k = tid; k < nbytes; k += nthr) dst[k] = src[k];
  }
}

__global__ void __launch_bounds__(128) v1_compact_kernel(
    const int* __restrict__ n_8, int n_works, int layout, const int* __restrict__ counts,
    const int* __restrict__ nbytes_8, uint8_t* __restrict__ stream, const uint8_t* __restrict__ stage,
    uint8_t* __restrict__ final_out) {
  __shared__ V1Where sw;
  __shared__ long long s_final;
  const int tid = threadIdx.x;
  if (tid == 0) {
    v1_locate(blockIdx.x, n_8, nullptr, nullptr, n_works, layout, false, 0x7fffffffffffffffLL, sw);
    long long fo = 0;
    for (int j = 0; j < sw.work; ++j)
      fo += (layout == LAYOUT_SPLIT) ? align128((long long)counts[j]) : (long long)nbytes_8[j];
    s_final = fo;
  }
  __syncthreads();
  const V1Where w = sw;
  if (w.work < 0) return;
  const long long nb = w.n / V1_BLOCK_ELEMS;
  uint8_t* wstream = stream + w.det_off;
  const V1Fields f = v1_fields(wstream, w.n);
  const int off = f.boff[w.blk];
  const int end = (w.blk + 1 < nb) ? f.boff[w.blk + 1] : counts[w.work];
  const uint8_t* st = (layout == LAYOUT_SPLIT) ? stage + w.aux_off : wstream + fused_stage_off(w.n);
  st += (long long)w.blk * V1_BLOCK_ELEMS;
  if (layout == LAYOUT_SPLIT) {
    uint8_t* dst = final_out + s_final + off;
    for (int k = tid; k < end - off; k += 128) dst[k] = st[k];
    return;
  }
  uint8_t* fstream = final_out + s_final;
  const V1Fields g = v1_fields(fstream, w.n);
  uint8_t* dst = reinterpret_cast<uint8_t*>(g.boff + nb + 1) + off;
  for (int k = tid; k < end - off; k += 128) dst[k] = st[k];
  if (fstream != wstream) {
    const long long e0 = (long long)w.blk * V1_BLOCK_ELEMS;
    copy_bytes(g.sm + e0, f.sm + e0, V1_BLOCK_ELEMS, tid, 128);
    g.b0[(long long)w.blk * 128 + tid] = f.b0[(long long)w.blk * 128 + tid];
    g.b1[(long long)w.blk * 128 + tid] = f.b1[(long long)w.blk * 128 + tid];
    g.b2[(long long)w.blk * 128 + tid] = f.b2[(long long)w.blk * 128 + tid];
    if (tid == 0) {
      g.boff[w.blk] = off;
      if (w.blk == 0) g.boff[nb] = f.boff[nb];
    }
  }
}

// ---------------------------------------------------------------------------------------------
// decode: one CTA per block, every variant
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128) v1_decode_kernel(
    const uint8_t* __restrict__ stream, const uint8_t* __restrict__ esc_stream, const int* __restrict__ n_8,
    const int* __restrict__ nbytes_8, int n_works, int layout, long long orig_each,
    const int* __restrict__ out_off, const int* __restrict__ orig_n, uint16_t* __restrict__ out,
    long long out_numel) {
  __shared__ V1Where sw;
  __shared__ int warp_tot[4];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) v1_locate(blockIdx.x, n_8, nullptr, nbytes_8, n_works, layout, true, 0x7fffffffffffffffLL, sw);
  __syncthreads();
  const V1Where w = sw;
  if (w.work < 0) return;
  const long long nb = w.n / V1_BLOCK_ELEMS;
  const V1Fields f = v1_fields(const_cast<uint8_t*>(stream) + w.det_off, w.n);
  const uint8_t* esc = (layout == LAYOUT_SPLIT) ? esc_stream + w.aux_off
                                                : reinterpret_cast<const uint8_t*>(f.boff + nb + 1);
  const int base = f.boff[nb];
  const long long e0 = (long long)w.blk * V1_BLOCK_ELEMS + tid * 32;
  const long long widx = (long long)w.blk * V1_THREADS + tid;
  uint32_t planes[4] = {f.b0[widx], f.b1[widx], f.b2[widx], 0};
  const uint32_t zm = ~(planes[0] | planes[1] | planes[2]);
  int wtot;
  const int pos_in_warp = warp_excl_scan(__popc(zm), lane, wtot);
  if (lane == 0) warp_tot[warp] = wtot;
  __syncthreads();
  int before = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) before += (i < warp) ? warp_tot[i] : 0;
  const long long valid_work = orig_n ? (long long)orig_n[w.work] : (orig_each >= 0 ? orig_each : w.n);
  const long long valid = valid_work - e0;
  if (valid <= 0) return;
  LaneSplit s;
  const uint4* smp = reinterpret_cast<const uint4*>(f.sm + e0);
  const uint4 a = smp[0], b = smp[1];
  s.sm[0] = a.x; s.sm[1] = a.y; s.sm[2] = a.z; s.sm[3] = a.w;
  s.sm[4] = b.x; s.sm[5] = b.y; s.sm[6] = b.z; s.sm[7] = b.w;
  decode_lane<3>(planes, base, esc + f.boff[w.blk] + before + pos_in_warp, s.ex);
  LaneIn o;
  join_lane(s, o);
  const long long ooff = out_off ? (long long)out_off[w.work]
                                 : (orig_each >= 0 ? (long long)w.work * orig_each : w.pad_off);
  long long lim = out_numel - (ooff + e0);
  if (lim > valid) lim = valid;
  if (lim <= 0) return;
  uint16_t* dst = out + ooff + e0;
  store_lane(dst, lim, (reinterpret_cast<uintptr_t>(dst) & 15) == 0, o);
}

// ---------------------------------------------------------------------------------------------
// base statistic: bases[0] = clamp(floor(log2(max(std,1e-30)) - 5.35 + 127), 0, 255)
// (reference rule: main/zipccl_comm.py:56-64).  Two launches, no host sync.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) v1_moments_kernel(const uint16_t* __restrict__ x, long long n,
                                                         double* __restrict__ acc) {
  double s = 0.0, q = 0.0;
  for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < n; i += (long long)gridDim.x * 256) {
    const float v = __uint_as_float((uint32_t)__ldg(x + i) << 16);
    s += v;
    q += (double)v * v;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    s += __shfl_xor_sync(FULL, s, o);
    q += __shfl_xor_sync(FULL, q, o);
  }
  __shared__ double ss[8], sq[8];
  if ((threadIdx.x & 31) == 0) { ss[threadIdx.x >> 5] = s; sq[threadIdx.x >> 5] = q; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < 8; ++i) { s += ss[i]; q += sq[i]; }
    atomicAdd(acc, s);
    atomicAdd(acc + 1, q);
  }
}

__global__ void v1_base_kernel(double* acc, long long n, int* bases) {
  const double mean = acc[0] / (double)n;
  double var = n > 1 ? (acc[1] - (double)n * mean * mean) / (double)(n - 1) : 0.0;
  if (!(var > 0.0)) var = 0.0;
  double sd = sqrt(var);
  if (sd < 1e-30) sd = 1e-30;
  double b = floor(log2(sd) - 5.35 + 127.0);
  b = b < 0.0 ? 0.0 : (b > 255.0 ? 255.0 : b);
  bases[0] = (int)b;
  acc[0] = 0.0;
  acc[1] = 0.0;
}

}  // namespace zc

extern "C" {

int zc_v1_encode_split(const void* in, long long total_n, const int* n_8, const int* orig_n, int n_works,
                       const int* bases, void* det, void* scratch, void* esc_final, int* counts,
                       long long total_blocks, cudaStream_t st) {
  using namespace zc;
  if (total_blocks <= 0) return 0;
  if (n_works <= 0) return ERR_BAD_ARG;
  v1_encode_kernel<<<(unsigned)total_blocks, 128, 0, st>>>((const uint16_t*)in, total_n, n_8, orig_n, n_works,
                                                           bases, LAYOUT_SPLIT, (uint8_t*)det, (uint8_t*)scratch);
  v1_scan_kernel<<<n_works, 1024, 0, st>>>(n_8, n_works, LAYOUT_SPLIT, (uint8_t*)det, counts, nullptr);
  v1_compact_kernel<<<(unsigned)total_blocks, 128, 0, st>>>(n_8, n_works, LAYOUT_SPLIT, counts, nullptr,
                                                            (uint8_t*)det, (const uint8_t*)scratch,
                                                            (uint8_t*)esc_final);
  return launch_status();
}

int zc_v1_encode_fused(const void* in, long long total_n, const int* n_8, int n_works, const int* bases,
                       void* scratch, void* out_final, long long out_final_bytes, int* nbytes_8, int* counts,
                       long long total_blocks, cudaStream_t st) {
  using namespace zc;
  (void)out_final_bytes;
  if (total_blocks <= 0) return 0;
  if (n_works <= 0) return ERR_BAD_ARG;
  v1_encode_kernel<<<(unsigned)total_blocks, 128, 0, st>>>((const uint16_t*)in, total_n, n_8, nullptr, n_works,
                                                           bases, LAYOUT_FUSED, (uint8_t*)scratch, nullptr);
  v1_scan_kernel<<<n_works, 1024, 0, st>>>(n_8, n_works, LAYOUT_FUSED, (uint8_t*)scratch, counts, nbytes_8);
  v1_compact_kernel<<<(unsigned)total_blocks, 128, 0, st>>>(n_8, n_works, LAYOUT_FUSED, counts, nbytes_8,
                                                            (uint8_t*)scratch, nullptr, (uint8_t*)out_final);
  return launch_status();
}

int zc_v1_decode_split(const void* det, const void* esc, const int* n_8, const int* nbytes_8, int n_works,
                       long long orig_each, const int* out_off, const int* orig_n, void* out,
                       long long out_numel, long long total_blocks, cudaStream_t st) {
  using namespace zc;
  if (total_blocks <= 0) return 0;
  v1_decode_kernel<<<(unsigned)total_blocks, 128, 0, st>>>((const uint8_t*)det, (const uint8_t*)esc, n_8,
                                                           nbytes_8, n_works, LAYOUT_SPLIT, orig_each, out_off,
                                                           orig_n, (uint16_t*)out, out_numel);
  return launch_status();
}

int zc_v1_decode_fused(const void* comp, const int* n_8, const int* nbytes_8, int n_works, long long orig_each,
                       void* out, long long out_numel, long long total_blocks, cudaStream_t st) {
  using namespace zc;
  if (total_blocks <= 0) return 0;
  v1_decode_kernel<<<(unsigned)total_blocks, 128, 0, st>>>((const uint8_t*)comp, nullptr, n_8, nbytes_8, n_works,
                                                           LAYOUT_FUSED, orig_each, nullptr, nullptr,
                                                           (uint16_t*)out, out_numel);
  return launch_status();
}

// `acc` scratch: two doubles per device, zeroed once and re-zeroed by the base kernel.
int zc_v1_base_from_std(const void* x, long long n, int* bases, cudaStream_t st) {
  using namespace zc;
  static double* acc[64] = {nullptr};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return ERR_BAD_ARG;
  if (!acc[dev]) {
    if (cudaMalloc(&acc[dev], 2 * sizeof(double)) != cudaSuccess) return (int)cudaGetLastError();
    cudaMemsetAsync(acc[dev], 0, 2 * sizeof(double), st);
  }
  if (n <= 0) return 0;
  const int grid = (int)std::min<long long>((n + 255) / 256, (long long)sm_count() * 8);
  v1_moments_kernel<<<grid, 256, 0, st>>>((const uint16_t*)x, n, acc[dev]);
  v1_base_kernel<<<1, 1, 0, st>>>(acc[dev], n, bases);
  return launch_status();
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------
// Allocation-free variant (see zc_noalloc.h): the outlier staging area is a static device array.
// ---------------------------------------------------------------------------------------------
#include <cstdio>
#include <mutex>

#include "zc_noalloc.h"

static __device__ __align__(256) unsigned char g_noalloc_scratch[ZC_NOALLOC_MAX_ELEMS];

namespace {
std::mutex g_noalloc_mutex;
unsigned char* g_noalloc_ptr[64] = {nullptr};  // device address of the array, per device

// In host code `g_noalloc_scratch` is only a handle for the runtime, not a device address; the
// address is looked up once per device, with that device current.
int noalloc_scratch(unsigned char** out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return ZC_ERR_SYMBOL;
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  if (!g_noalloc_ptr[dev]) {
    unsigned char* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress((void**)&p, g_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr) {
      fprintf(stderr, "[zc_noalloc] cudaGetSymbolAddress failed on device %d: %s\n", dev, cudaGetErrorString(e));
      return ZC_ERR_SYMBOL;
    }
    g_noalloc_ptr[dev] = p;
  }
  *out = g_noalloc_ptr[dev];
  return 0;
}
}  // namespace

extern "C" int zc_v1_encode_split_noalloc(const void* in, long long total_n, const int* n_8, const int* orig_n,
                                          int n_works, const int* bases, void* det, void* esc_final, int* counts,
                                          long long total_blocks, cudaStream_t st) {
  using namespace zc;
  if (total_blocks <= 0) return 0;
  if (n_works <= 0) return ERR_BAD_ARG;
  if (total_blocks * V1_BLOCK_ELEMS > ZC_NOALLOC_MAX_ELEMS) {
    fprintf(stderr,
            "[zc_noalloc] request of %lld padded elements exceeds the built-in scratch of %lld; "
            "use zc_v1_encode_split with your own scratch buffer\n",
            total_blocks * V1_BLOCK_ELEMS, (long long)ZC_NOALLOC_MAX_ELEMS);
    return ZC_ERR_TOO_LARGE;
  }
  unsigned char* scratch = nullptr;
  const int rc = noalloc_scratch(&scratch);
  if (rc != 0) return rc;
  v1_encode_kernel<<<(unsigned)total_blocks, 128, 0, st>>>((const uint16_t*)in, total_n, n_8, orig_n, n_works,
                                                           bases, LAYOUT_SPLIT, (uint8_t*)det, scratch);
  v1_scan_kernel<<<n_works, 1024, 0, st>>>(n_8, n_works, LAYOUT_SPLIT, (uint8_t*)det, counts, nullptr);
  v1_compact_kernel<<<(unsigned)total_blocks, 128, 0, st>>>(n_8, n_works, LAYOUT_SPLIT, counts, nullptr,
                                                            (uint8_t*)det, scratch, (uint8_t*)esc_final);
  return launch_status();
}
