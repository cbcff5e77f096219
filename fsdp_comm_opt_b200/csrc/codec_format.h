// Wire formats of the BF16 exponent codec, shared by the CPU scalar codec and the sm_100a kernels.
//
// A bf16 value v is split into a "sign+mantissa" byte  sm = ((v >> 8) & 0x80) | (v & 0x7F)
// and its 8-bit exponent  e = (v >> 7) & 0xFF.  Both formats store sm verbatim (1 B/elem) and
// differ in how the exponent is coded.
//
// ---------------------------------------------------------------------------------------------
// v1 ("window-7", wire compatible with the reference's hopper_fastzip2 streams;
//     reference: zipccl/hopper_zip.cu:82-100 encode, :826-853 decode, :409-410 sizes)
//
//   block  = 4096 elements = 128 threads x 32 elements; thread t of block b owns elements
//            b*4096 + t*32 + j (j = 0..31) and bit j of bit-plane word b*128 + t.
//   code   = e - base + 1 (1..7) when base <= e < base+7, else 0 (outlier, raw e goes to the
//            outlier byte stream in element order inside a block).
//   "work" = independently decodable segment of N elements (N % 4096 == 0), nb = N/4096 blocks.
//
//   fused layout, one work:            split layout, one work:
//     [0, N)        sm bytes             det stream (stride align128(det_bytes(N))):
//     3 x N/8       planes b0|b1|b2        sm | b0|b1|b2 | block_off[nb] | base
//     int32[nb]     block outlier start  outlier stream: compacted, stride align128(count)
//     int32         base
//     count bytes   outlier exponents
//
// ---------------------------------------------------------------------------------------------
// v2 ("per-chunk base and width"; no counterpart in the reference)
//
//   chunk  = 1024 elements = 32 lanes x 32 elements; lane l owns elements l*32 + j and bit j of
//            word l of every plane.  Elements past the end of the tensor count as 0x0000.
//   header = one uint32 per chunk:  base | width << 8 | n_esc << 16
//            width in {0,1,2,3,4}: codes of `width` bits, code 0 = escape,
//                                  code c>0 means e = base + c - 1;
//            width 0: every element has e == base (no planes, no escapes);
//            width 8: raw mode, the 1024 exponents follow the sm bytes verbatim.
//   record = [sm: 1024 B][planes: width x 128 B][escapes: n_esc B in element order]
//            never longer than 2048 B, so a record slot has the size of the raw bf16 chunk and
//            every chunk is encodable and decodable on its own at a fixed offset.
//   window choice (identical on CPU and GPU, so streams are byte-identical):
//            emin, emax = exact min / max exponent of the chunk; emin == emax gives width 0.
//            anchor a = max(emax-15, 0); h[d] = #{sampled e - a == d}, d = 0..15, where the
//            sample is every 4th element (index % 4 == 0, 256 samples);
//            candidates (width w, first bin d0) with span s = 2^w - 1, d0 = 0..16-s:
//            estimated cost = 128*w + 4*(256 - sum(h[d0..d0+s-1])).  Smallest estimate wins; ties
//            go to the smaller width, then the smaller d0; an estimate above 1024 selects raw.
//            The escapes are then counted exactly; if 128*w + n_esc > 1024 the chunk is stored
//            raw after all, so a record never exceeds its slot.
//   nibble mode (streams staged by the fused collectives when the caller asks for it; a property of
//   the stream, not marked in the record): only widths 0, 4 and 8 occur; a width-4 record is
//            [sm: 1024 B][codes: 512 B][escapes: n_esc B]
//            with base = max(emax - 14, 0) and lane l's sixteen code bytes at 1024 + 16 l, byte 4 k + j
//            of them holding the code of element 32 l + 8 k + j in its low nibble and of element
//            32 l + 8 k + 4 + j in its high nibble (k = 0..3, j = 0..3); escapes and the raw fallback
//            (512 + n_esc > 1024) as above.  In the staging buffers of the fused collectives the sm
//            section of every record is stored as two 512-byte halves (lane l's bytes 0..15 at 16 l,
//            bytes 16..31 at 512 + 16 l).
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define ZC_HD __host__ __device__ __forceinline__
#else
#define ZC_HD inline
#endif

namespace zc {

constexpr int V1_BLOCK_ELEMS = 4096;
constexpr int V1_THREADS = 128;
constexpr int V1_WINDOW = 7;

constexpr int V2_CHUNK_ELEMS = 1024;
constexpr int V2_SLOT_BYTES = 2048;
constexpr int V2_RAW_WIDTH = 8;

ZC_HD int64_t align128(int64_t x) { return (x + 127) / 128 * 128; }

// Bytes of the deterministic part of one v1 work of n padded elements (before align128).
ZC_HD int64_t v1_det_bytes(int64_t n) { return n + n / 8 * 3 + (n / V1_BLOCK_ELEMS) * 4 + 4; }

ZC_HD uint8_t bf16_sm(uint16_t v) { return (uint8_t)(((v >> 8) & 0x80) | (v & 0x7F)); }
ZC_HD uint8_t bf16_exp(uint16_t v) { return (uint8_t)((v >> 7) & 0xFF); }
ZC_HD uint16_t bf16_join(uint8_t sm, uint8_t e) {
  return (uint16_t)((sm & 0x7F) | ((uint16_t)e << 7) | ((uint16_t)(sm >> 7) << 15));
}

ZC_HD uint32_t v2_header(int base, int width, int n_esc) {
  return (uint32_t)base | ((uint32_t)width << 8) | ((uint32_t)n_esc << 16);
}
ZC_HD int v2_hdr_base(uint32_t h) { return (int)(h & 0xFF); }
ZC_HD int v2_hdr_width(uint32_t h) { return (int)((h >> 8) & 0xF); }
ZC_HD int v2_hdr_nesc(uint32_t h) { return (int)(h >> 16); }
ZC_HD int v2_record_bytes(uint32_t h) {
  int w = v2_hdr_width(h);
  if (w == V2_RAW_WIDTH) return 2048;
  return 1024 + 128 * w + v2_hdr_nesc(h);
}

// Candidate table of the v2 window choice: index -> (width, first bin).  Ordered so that a
// smaller index wins ties (smaller width first, then smaller d0).  42 candidates.
constexpr int V2_NUM_CAND = 42;
ZC_HD void v2_candidate(int idx, int& w, int& d0) {
  if (idx < 16) { w = 1; d0 = idx; }
  else if (idx < 30) { w = 2; d0 = idx - 16; }
  else if (idx < 40) { w = 3; d0 = idx - 30; }
  else { w = 4; d0 = idx - 40; }
}

// Given the 16-bin sample histogram (256 samples) anchored at `anchor`, pick (base, width).
// prefix[k] = sum of h[0..k-1], k = 0..16.  Returns the header with n_esc = 0 (the exact escape
// count is filled in by the encoder) or a raw header.
ZC_HD uint32_t v2_choose(const int* prefix, int anchor) {
  int best_key = 0x7fffffff;
  for (int idx = 0; idx < V2_NUM_CAND; ++idx) {
    int w, d0;
    v2_candidate(idx, w, d0);
    const int s = (1 << w) - 1;
    const int cost = 128 * w + 4 * (256 - (prefix[d0 + s] - prefix[d0]));
    const int key = (cost << 6) | idx;
    if (key < best_key) best_key = key;
  }
  if ((best_key >> 6) > V2_CHUNK_ELEMS) return v2_header(0, V2_RAW_WIDTH, 0);
  int w, d0;
  v2_candidate(best_key & 63, w, d0);
  return v2_header(anchor + d0, w, 0);
}

}  // namespace zc
