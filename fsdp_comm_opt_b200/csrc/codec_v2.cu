// v2 codec kernels (per-chunk base and width) for sm_100a: standalone encode and decode.
//
// One warp per 1024-element chunk, eight warps per CTA, persistent grid-stride loop sized to the
// SM count.  No shared memory, no atomics, no cross-chunk dependency: chunk c lives at the fixed
// offset c*2048 of the record buffer, so encode and decode are embarrassingly parallel and the
// same device functions are reused inside the fused collective kernels.
#include "codec_v2_dev.cuh"
#include "launch_util.h"
#include "nvtx_util.h"

namespace zc {


// NIBBLE: records in nibble mode (codec_format.h): fixed four code bits, codes packed two per byte
template <bool NIBBLE>
__global__ void __launch_bounds__(256) v2_encode_kernel(const uint16_t* __restrict__ in, int64_t n,
                                                        uint8_t* __restrict__ records,
                                                        uint32_t* __restrict__ headers, int64_t nc) {
  const int lane = threadIdx.x & 31;
  const int64_t warp0 = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  const int64_t stride = (int64_t)gridDim.x * 8;
  const bool al = (reinterpret_cast<uintptr_t>(in) & 15) == 0;
  for (int64_t c = warp0; c < nc; c += stride) {
    const int64_t e0 = c * V2_CHUNK_ELEMS + lane * 32;
    LaneIn li;
    load_lane(in + e0, n - e0, al, li);
    LaneSplit s;
    split_lane(li, s);
    uint32_t hdr;
    if (NIBBLE) {
      uint8_t* rec = records + c * V2_SLOT_BYTES;
      uint4* smp = reinterpret_cast<uint4*>(rec + lane * 32);
      smp[0] = make_uint4(s.sm[0], s.sm[1], s.sm[2], s.sm[3]);
      smp[1] = make_uint4(s.sm[4], s.sm[5], s.sm[6], s.sm[7]);
      hdr = v2_encode_chunk_nibble(s, rec, lane);
    } else {
      hdr = v2_encode_chunk(s, records + c * V2_SLOT_BYTES, lane);
    }
    if (lane == 0) headers[c] = hdr;
  }
}

template <bool NIBBLE>
__global__ void __launch_bounds__(256) v2_decode_kernel(const uint8_t* __restrict__ records,
                                                        const uint32_t* __restrict__ headers, int64_t n,
                                                        uint16_t* __restrict__ out, int64_t nc) {
  __shared__ __align__(16) uint8_t esc[8][1024];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t warp0 = (int64_t)blockIdx.x * 8 + warp;
  const int64_t stride = (int64_t)gridDim.x * 8;
  const bool al = (reinterpret_cast<uintptr_t>(out) & 15) == 0;
  // software pipeline: record c + stride is in flight while record c is decoded and stored
  RecRegs cur, nxt;
  int64_t c = warp0;
  if (c < nc) v2_prefetch<false, NIBBLE>(records + c * V2_SLOT_BYTES, __ldcg(headers + c), lane, cur);
  uint32_t hdr_next = (c + stride < nc) ? __ldcg(headers + c + stride) : 0u;
  for (; c < nc; c += stride) {
    const int64_t cn = c + stride;
    if (cn < nc) {
      v2_prefetch<false, NIBBLE>(records + cn * V2_SLOT_BYTES, hdr_next, lane, nxt);
      if (cn + stride < nc) hdr_next = __ldcg(headers + cn + stride);
    }
    LaneSplit s;
    v2_decode_regs<NIBBLE>(cur, esc[warp], lane, s);
    LaneIn o;
    join_lane(s, o);
    const int64_t e0 = c * V2_CHUNK_ELEMS + lane * 32;
    store_lane(out + e0, n - e0, al, o);
    cur = nxt;
  }
}

}  // namespace zc

extern "C" {

int zc_v2_encode(const void* in, int64_t n, void* records, void* headers, cudaStream_t stream) {
  ZC_NVTX_RANGE("zc_v2_encode");
  const int64_t nc = (n + zc::V2_CHUNK_ELEMS - 1) / zc::V2_CHUNK_ELEMS;
  if (nc == 0) return 0;
  const int grid = (int)std::min<int64_t>((nc + 7) / 8, (int64_t)zc::sm_count() * 8);
  zc::v2_encode_kernel<false><<<grid, 256, 0, stream>>>((const uint16_t*)in, n, (uint8_t*)records,
                                                        (uint32_t*)headers, nc);
  return zc::launch_status();
}

// `max_ctas` > 0 caps the grid (how the decoder behaves with the SM budget it has inside a fused
// collective); 0 sizes it to the device.
int zc_v2_decode_ctas(const void* records, const void* headers, int64_t n, void* out, int max_ctas,
                      cudaStream_t stream) {
  const int64_t nc = (n + zc::V2_CHUNK_ELEMS - 1) / zc::V2_CHUNK_ELEMS;
  if (nc == 0) return 0;
  int grid = (int)std::min<int64_t>((nc + 7) / 8, (int64_t)zc::sm_count() * 8);
  if (max_ctas > 0) grid = std::min(grid, max_ctas);
  zc::v2_decode_kernel<false><<<grid, 256, 0, stream>>>((const uint8_t*)records, (const uint32_t*)headers, n,
                                                        (uint16_t*)out, nc);
  return zc::launch_status();
}

int zc_v2_decode(const void* records, const void* headers, int64_t n, void* out, cudaStream_t stream) {
  ZC_NVTX_RANGE("zc_v2_decode");
  const int64_t nc = (n + zc::V2_CHUNK_ELEMS - 1) / zc::V2_CHUNK_ELEMS;
  if (nc == 0) return 0;
  const int grid = (int)std::min<int64_t>((nc + 7) / 8, (int64_t)zc::sm_count() * 8);
  zc::v2_decode_kernel<false><<<grid, 256, 0, stream>>>((const uint8_t*)records, (const uint32_t*)headers, n,
                                                        (uint16_t*)out, nc);
  return zc::launch_status();
}

// The same two entry points for records in nibble mode (the records the fused collectives stage by
// default, here with the documented 32-consecutive-bytes-per-lane sign+mantissa section).
int zc_v2_encode_nibble(const void* in, int64_t n, void* records, void* headers, cudaStream_t stream) {
  ZC_NVTX_RANGE("zc_v2_encode_nibble");
  const int64_t nc = (n + zc::V2_CHUNK_ELEMS - 1) / zc::V2_CHUNK_ELEMS;
  if (nc == 0) return 0;
  const int grid = (int)std::min<int64_t>((nc + 7) / 8, (int64_t)zc::sm_count() * 8);
  zc::v2_encode_kernel<true><<<grid, 256, 0, stream>>>((const uint16_t*)in, n, (uint8_t*)records,
                                                       (uint32_t*)headers, nc);
  return zc::launch_status();
}

int zc_v2_decode_nibble(const void* records, const void* headers, int64_t n, void* out, cudaStream_t stream) {
  ZC_NVTX_RANGE("zc_v2_decode_nibble");
  const int64_t nc = (n + zc::V2_CHUNK_ELEMS - 1) / zc::V2_CHUNK_ELEMS;
  if (nc == 0) return 0;
  const int grid = (int)std::min<int64_t>((nc + 7) / 8, (int64_t)zc::sm_count() * 8);
  zc::v2_decode_kernel<true><<<grid, 256, 0, stream>>>((const uint8_t*)records, (const uint32_t*)headers, n,
                                                       (uint16_t*)out, nc);
  return zc::launch_status();
}

}  // extern "C"
