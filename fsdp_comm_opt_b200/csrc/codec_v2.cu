// v2 codec kernels (per-chunk base and width) for sm_100a: standalone encode and decode.
//
// One warp per 1024-element chunk, eight warps per CTA, persistent grid-stride loop sized to the
// SM count.  No shared memory, no atomics, no cross-chunk dependency: chunk c lives at the fixed
// offset c*2048 of the record buffer, so encode and decode are embarrassingly parallel and the
// same device functions are reused inside the fused collective kernels.
#include "codec_v2_dev.cuh"
#include "launch_util.h"

namespace zc {


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
    const uint32_t hdr = v2_encode_chunk(s, records + c * V2_SLOT_BYTES, lane);
    if (lane == 0) headers[c] = hdr;
  }
}

__global__ void __launch_bounds__(256) v2_decode_kernel(const uint8_t* __restrict__ records,
                                                        const uint32_t* __restrict__ headers, int64_t n,
                                                        uint16_t* __restrict__ out, int64_t nc) {
  const int lane = threadIdx.x & 31;
  const int64_t warp0 = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  const int64_t stride = (int64_t)gridDim.x * 8;
  const bool al = (reinterpret_cast<uintptr_t>(out) & 15) == 0;
  for (int64_t c = warp0; c < nc; c += stride) {
    LaneSplit s;
    v2_decode_chunk(records + c * V2_SLOT_BYTES, __ldg(headers + c), lane, s);
    LaneIn o;
    join_lane(s, o);
    const int64_t e0 = c * V2_CHUNK_ELEMS + lane * 32;
    store_lane(out + e0, n - e0, al, o);
  }
}

}  // namespace zc

extern "C" {

int zc_v2_encode(const void* in, int64_t n, void* records, void* headers, cudaStream_t stream) {
  const int64_t nc = (n + zc::V2_CHUNK_ELEMS - 1) / zc::V2_CHUNK_ELEMS;
  if (nc == 0) return 0;
  const int grid = (int)std::min<int64_t>((nc + 7) / 8, (int64_t)zc::sm_count() * 8);
  zc::v2_encode_kernel<<<grid, 256, 0, stream>>>((const uint16_t*)in, n, (uint8_t*)records,
                                                 (uint32_t*)headers, nc);
  return zc::launch_status();
}

int zc_v2_decode(const void* records, const void* headers, int64_t n, void* out, cudaStream_t stream) {
  const int64_t nc = (n + zc::V2_CHUNK_ELEMS - 1) / zc::V2_CHUNK_ELEMS;
  if (nc == 0) return 0;
  const int grid = (int)std::min<int64_t>((nc + 7) / 8, (int64_t)zc::sm_count() * 8);
  zc::v2_decode_kernel<<<grid, 256, 0, stream>>>((const uint8_t*)records, (const uint32_t*)headers, n,
                                                 (uint16_t*)out, nc);
  return zc::launch_status();
}

}  // extern "C"
