// Warp-level building blocks of the BF16 exponent codec for sm_100a.
//
// One warp handles 1024 consecutive elements; lane l owns elements l*32 .. l*32+31 (64 bytes),
// which is the ownership both wire formats prescribe (v1: thread t of a 128-thread block, v2: lane
// l of a chunk).  Everything is done four elements at a time on packed bytes (SWAR), with no
// shared memory and no per-element branches:
//   split      16 u32 (32 bf16) -> 8 u32 of sign+mantissa bytes, 8 u32 of exponent bytes
//   codes      per-byte  c = e - (base-1);  code = (1 <= c <= span) ? c : 0
//   planes     bit p of every code gathered into one 32-bit word per plane
//   escapes    exponent bytes whose code is 0, compacted in element order
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "codec_format.h"

namespace zc {

constexpr unsigned FULL = 0xffffffffu;
constexpr uint32_t H4 = 0x80808080u;
constexpr uint32_t L4 = 0x7f7f7f7fu;

__device__ __forceinline__ uint32_t rep4(uint32_t b) { return (b & 0xFFu) * 0x01010101u; }

// per-byte x - y (mod 256), y given as  yl = y & 0x7f7f7f7f  and  yn = ~y & 0x80808080
__device__ __forceinline__ uint32_t sub4(uint32_t x, uint32_t yl, uint32_t yn) {
  return ((x | H4) - yl) ^ ((x & H4) ^ yn);
}

// 0xFF in every byte of m that is non-zero, 0x00 elsewhere
__device__ __forceinline__ uint32_t nzmask4(uint32_t m) {
  uint32_t hb = (((m & L4) + L4) | m) & H4;
  return (hb - (hb >> 7)) | hb;
}

// 32 bf16 values of one lane, as loaded (two elements per word, low half first)
struct LaneIn {
  uint32_t w[16];
};

// sign+mantissa bytes and exponent bytes of one lane, four elements per word
struct LaneSplit {
  uint32_t sm[8];
  uint32_t ex[8];
};

__device__ __forceinline__ void split_lane(const LaneIn& in, LaneSplit& s) {
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const uint32_t a = in.w[2 * k], b = in.w[2 * k + 1];
    uint32_t xa = a & 0x807F807Fu, xb = b & 0x807F807Fu;
    xa |= xa >> 8;
    xb |= xb >> 8;
    s.sm[k] = __byte_perm(xa, xb, 0x6420);
    s.ex[k] = __byte_perm(a >> 7, b >> 7, 0x6420);
  }
}

__device__ __forceinline__ void join_lane(const LaneSplit& s, LaneIn& out) {
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    // element i: (sm & 0x7F) | e << 7 | (sm >> 7) << 15
    const uint32_t sm = s.sm[k], ex = s.ex[k];
    const uint32_t m01 = __byte_perm(sm, 0, 0x4140);  // bytes: sm0,0,sm1,0
    const uint32_t m23 = __byte_perm(sm, 0, 0x4342);
    const uint32_t e01 = __byte_perm(ex, 0, 0x4140);
    const uint32_t e23 = __byte_perm(ex, 0, 0x4342);
    out.w[2 * k] = (m01 & 0x007F007Fu) | ((m01 & 0x00800080u) << 8) | (e01 << 7);
    out.w[2 * k + 1] = (m23 & 0x007F007Fu) | ((m23 & 0x00800080u) << 8) | (e23 << 7);
  }
}

// Loads.  `aligned`: pointer is 16-byte aligned and all 32 elements are in range.
__device__ __forceinline__ void load_lane(const uint16_t* p, int64_t valid, bool aligned, LaneIn& in) {
  if (aligned && valid >= 32) {
    const uint4* q = reinterpret_cast<const uint4*>(p);
    uint4 a = __ldg(q), b = __ldg(q + 1), c = __ldg(q + 2), d = __ldg(q + 3);
    in.w[0] = a.x; in.w[1] = a.y; in.w[2] = a.z; in.w[3] = a.w;
    in.w[4] = b.x; in.w[5] = b.y; in.w[6] = b.z; in.w[7] = b.w;
    in.w[8] = c.x; in.w[9] = c.y; in.w[10] = c.z; in.w[11] = c.w;
    in.w[12] = d.x; in.w[13] = d.y; in.w[14] = d.z; in.w[15] = d.w;
  } else {
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      const uint32_t lo = (2 * k < valid) ? (uint32_t)__ldg(p + 2 * k) : 0u;
      const uint32_t hi = (2 * k + 1 < valid) ? (uint32_t)__ldg(p + 2 * k + 1) : 0u;
      in.w[k] = lo | (hi << 16);
    }
  }
}

__device__ __forceinline__ void store_lane(uint16_t* p, int64_t valid, bool aligned, const LaneIn& o) {
  if (aligned && valid >= 32) {
    uint4* q = reinterpret_cast<uint4*>(p);
    q[0] = make_uint4(o.w[0], o.w[1], o.w[2], o.w[3]);
    q[1] = make_uint4(o.w[4], o.w[5], o.w[6], o.w[7]);
    q[2] = make_uint4(o.w[8], o.w[9], o.w[10], o.w[11]);
    q[3] = make_uint4(o.w[12], o.w[13], o.w[14], o.w[15]);
  } else {
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      if (2 * k < valid) p[2 * k] = (uint16_t)(o.w[k] & 0xFFFFu);
      if (2 * k + 1 < valid) p[2 * k + 1] = (uint16_t)(o.w[k] >> 16);
    }
  }
}

// codes for a window [base, base+span): returns per-byte codes (0 = escape), four per word
__device__ __forceinline__ void codes_lane(const LaneSplit& s, int base, uint32_t span, uint32_t (&code)[8]) {
  const uint32_t y = rep4((uint32_t)(base - 1));
  const uint32_t yl = y & L4, yn = ~y & H4;
  const uint32_t ns = rep4(~span);
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const uint32_t c = sub4(s.ex[k], yl, yn);
    code[k] = c & ~nzmask4(c & ns);
  }
}

// bit p of the 32 codes -> one word (bit j = element j)
template <int P>
__device__ __forceinline__ uint32_t plane_word(const uint32_t (&code)[8]) {
  uint32_t w = 0;
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const uint32_t bits = (code[k] >> P) & 0x01010101u;
    w |= ((bits * 0x01020408u) >> 24 & 0xFu) << (4 * k);
  }
  return w;
}

// bit j set when element j's code is zero
__device__ __forceinline__ uint32_t zero_mask(const uint32_t (&code)[8]) {
  uint32_t w = 0;
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const uint32_t nz = nzmask4(code[k]) & 0x01010101u;
    w |= ((nz * 0x01020408u) >> 24 & 0xFu) << (4 * k);
  }
  return ~w;
}

__device__ __forceinline__ uint32_t byte_of(const uint32_t (&a)[8], int j) {
  return (a[j >> 2] >> ((j & 3) * 8)) & 0xFFu;
}

// exclusive prefix of v over the warp; total returned through `total`
__device__ __forceinline__ int warp_excl_scan(int v, int lane, int& total) {
  int x = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int t = __shfl_up_sync(FULL, x, o);
    if (lane >= o) x += t;
  }
  total = __shfl_sync(FULL, x, 31);
  return x - v;
}

// write this lane's escapes (exponents of zero-coded elements) at dst[0..popc(zmask))
__device__ __forceinline__ void scatter_escapes(uint8_t* dst, const LaneSplit& s, uint32_t zmask) {
  if (zmask == 0) return;
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    uint32_t m = (zmask >> (4 * k)) & 0xFu;
    while (m) {
      const int j = __ffs(m) - 1;
      *dst++ = (uint8_t)((s.ex[k] >> (j * 8)) & 0xFFu);
      m &= m - 1;
    }
  }
}

// Rebuild exponent bytes from planes (W planes) and the escape stream.
//   planes[p] = this lane's word of plane p; esc = this lane's first escape byte.
template <int W>
__device__ __forceinline__ void decode_lane(const uint32_t (&planes)[4], int base, const uint8_t* esc,
                                            uint32_t (&ex)[8]) {
  uint32_t zm = ~0u;
#pragma unroll
  for (int p = 0; p < W; ++p) zm &= ~planes[p];
  const uint32_t b4 = rep4((uint32_t)base);
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    // spread 4 bits of every plane into the low bits of 4 bytes
    uint32_t c = 0;
#pragma unroll
    for (int p = 0; p < W; ++p) {
      const uint32_t nib = (planes[p] >> (4 * k)) & 0xFu;
      // nibble bits b0..b3 -> bytes: (nib * 0x00204081) & 0x01010101 places bit i at byte i
      c |= ((nib * 0x00204081u) & 0x01010101u) << p;
    }
    // e = base + (code - 1) for coded elements: code >= 1 so the subtraction never borrows, and
    // base + code - 1 <= 255 so the addition never carries into the next byte
    const uint32_t nz = nzmask4(c);
    ex[k] = (c - (nz & 0x01010101u)) + (b4 & nz);
  }
  // escapes overwrite the zero-coded bytes
  if (zm == 0) return;
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    uint32_t m = (zm >> (4 * k)) & 0xFu;
    while (m) {
      const int j = __ffs(m) - 1;
      ex[k] |= (uint32_t)(*esc++) << (j * 8);
      m &= m - 1;
    }
  }
}

}  // namespace zc
