// v2 codec device functions shared by the standalone kernels (codec_v2.cu) and the fused
// collective kernels (symm_collectives.cu): window choice, chunk encode, chunk decode.
// `rec` may point to global or shared memory (generic address).
#pragma once
#include "codec_dev.cuh"

namespace zc {


// Window choice for one chunk.  Every lane passes its 8 exponent words; the result (header with
// n_esc = 0, or a raw header) is uniform across the warp.
__device__ __forceinline__ uint32_t v2_choose_warp(const LaneSplit& s, int lane) {
  // exact min / max of the 1024 exponents
  uint32_t mx = s.ex[0], mn = s.ex[0];
#pragma unroll
  for (int k = 1; k < 8; ++k) {
    mx = __vmaxu4(mx, s.ex[k]);
    mn = __vminu4(mn, s.ex[k]);
  }
  uint32_t mxb = max(max(mx & 0xFF, (mx >> 8) & 0xFF), max((mx >> 16) & 0xFF, mx >> 24));
  uint32_t mnb = min(min(mn & 0xFF, (mn >> 8) & 0xFF), min((mn >> 16) & 0xFF, mn >> 24));
  const int emax = (int)__reduce_max_sync(FULL, mxb);
  const int emin = (int)__reduce_min_sync(FULL, mnb);
  if (emin == emax) return v2_header(emax, 0, 0);
  const int anchor = emax > 15 ? emax - 15 : 0;
  // sample histogram: byte 0 of every word (elements with index % 4 == 0), 16 bins x 4 bit
  unsigned long long h = 0;
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const int d = (int)(s.ex[k] & 0xFFu) - anchor;
    if (d >= 0) h += 1ull << (4 * d);
  }
  // widen to 16-bit fields (two bins per word) and sum over the warp
  int tot[16];
#pragma unroll
  for (int q = 0; q < 8; ++q) {
    const uint32_t pair = (uint32_t)((h >> (8 * q)) & 0xFull) | ((uint32_t)((h >> (8 * q + 4)) & 0xFull) << 16);
    const uint32_t sum = __reduce_add_sync(FULL, pair);
    tot[2 * q] = (int)(sum & 0xFFFFu);
    tot[2 * q + 1] = (int)(sum >> 16);
  }
  // lane k keeps prefix[k] (k = 0..16); candidates fetch their two prefixes by shuffle
  int mine = 0;
#pragma unroll
  for (int d = 0; d < 16; ++d) mine += (d < lane) ? tot[d] : 0;
  int best = 0x7fffffff;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int idx = lane + 32 * r;
    int w = 1, d0 = 0;
    if (idx < V2_NUM_CAND) v2_candidate(idx, w, d0);
    const int sp = (1 << w) - 1;
    const int hi = __shfl_sync(FULL, mine, d0 + sp);
    const int lo = __shfl_sync(FULL, mine, d0);
    const int cost = 128 * w + 4 * (256 - (hi - lo));
    if (idx < V2_NUM_CAND) best = min(best, (cost << 6) | idx);
  }
  best = __reduce_min_sync(FULL, best);
  if ((best >> 6) > V2_CHUNK_ELEMS) return v2_header(0, V2_RAW_WIDTH, 0);
  int w, d0;
  v2_candidate(best & 63, w, d0);
  return v2_header(anchor + d0, w, 0);
}

// Encode the chunk whose split fields are in `s` into `rec`; returns the final header.
// STORE_SM = false leaves out the first 1024 bytes of the record (the sign+mantissa bytes, which a
// caller that pushes them straight from registers does not need staged): only rec[1024 ...) is
// written, so `rec` may then point 1024 bytes before a buffer that holds just the record's tail.
template <bool STORE_SM = true>
__device__ __forceinline__ uint32_t v2_encode_chunk(const LaneSplit& s, uint8_t* rec, int lane) {
  uint32_t hdr = v2_choose_warp(s, lane);
  int w = v2_hdr_width(hdr);
  const int base = v2_hdr_base(hdr);
  if (STORE_SM) {
    uint4* smp = reinterpret_cast<uint4*>(rec + lane * 32);
    smp[0] = make_uint4(s.sm[0], s.sm[1], s.sm[2], s.sm[3]);
    smp[1] = make_uint4(s.sm[4], s.sm[5], s.sm[6], s.sm[7]);
  }
  if (w != V2_RAW_WIDTH && w > 0) {
    uint32_t code[8];
    codes_lane(s, base, (1u << w) - 1u, code);
    const uint32_t zm = zero_mask(code);
    int n_esc;
    const int pos = warp_excl_scan(__popc(zm), lane, n_esc);
    if (128 * w + n_esc > V2_CHUNK_ELEMS) {
      w = V2_RAW_WIDTH;
      hdr = v2_header(0, V2_RAW_WIDTH, 0);
    } else {
      hdr = v2_header(base, w, n_esc);
      uint32_t* pl = reinterpret_cast<uint32_t*>(rec + 1024) + lane;
      pl[0] = plane_word<0>(code);
      if (w > 1) pl[32] = plane_word<1>(code);
      if (w > 2) pl[64] = plane_word<2>(code);
      if (w > 3) pl[96] = plane_word<3>(code);
      scatter_escapes(rec + 1024 + 128 * w + pos, s, zm);
    }
  }
  if (w == V2_RAW_WIDTH) {
    uint4* ep = reinterpret_cast<uint4*>(rec + 1024 + lane * 32);
    ep[0] = make_uint4(s.ex[0], s.ex[1], s.ex[2], s.ex[3]);
    ep[1] = make_uint4(s.ex[4], s.ex[5], s.ex[6], s.ex[7]);
  }
  return hdr;
}

// Encode with a window carried over from the previous chunk of the same stream ("hint", a header
// with width 1..4, or 0xFFFFFFFF for none).  The hint is kept while its exact escape count stays
// close to the count it had when it was chosen; otherwise the window is chosen afresh.  Any valid
// choice decodes correctly, so this only trades a little compression for skipping the histogram.
// Returns the header; `hint` / `hint_esc` are updated for the next chunk.
template <bool STORE_SM = true>
__device__ __forceinline__ uint32_t v2_encode_chunk_hint(const LaneSplit& s, uint8_t* rec, int lane, uint32_t& hint,
                                                         int& hint_esc) {
  if (hint != 0xFFFFFFFFu) {
    const int w = v2_hdr_width(hint), base = v2_hdr_base(hint);
    uint32_t code[8];
    codes_lane(s, base, (1u << w) - 1u, code);
    const uint32_t zm = zero_mask(code);
    int n_esc;
    const int pos = warp_excl_scan(__popc(zm), lane, n_esc);
    if (n_esc <= hint_esc + (hint_esc >> 1) + 16 && 128 * w + n_esc <= V2_CHUNK_ELEMS) {
      if (STORE_SM) {
        uint4* smp = reinterpret_cast<uint4*>(rec + lane * 32);
        smp[0] = make_uint4(s.sm[0], s.sm[1], s.sm[2], s.sm[3]);
        smp[1] = make_uint4(s.sm[4], s.sm[5], s.sm[6], s.sm[7]);
      }
      uint32_t* pl = reinterpret_cast<uint32_t*>(rec + 1024) + lane;
      pl[0] = plane_word<0>(code);
      if (w > 1) pl[32] = plane_word<1>(code);
      if (w > 2) pl[64] = plane_word<2>(code);
      if (w > 3) pl[96] = plane_word<3>(code);
      scatter_escapes(rec + 1024 + 128 * w + pos, s, zm);
      return v2_header(base, w, n_esc);
    }
  }
  const uint32_t hdr = v2_encode_chunk<STORE_SM>(s, rec, lane);
  const int w = v2_hdr_width(hdr);
  if (w >= 1 && w <= 4) {
    hint = hdr & 0xFFFFu;
    hint_esc = v2_hdr_nesc(hdr);
  } else {
    hint = 0xFFFFFFFFu;
  }
  return hdr;
}

// ---------------------------------------------------------------------------------------------
// Nibble mode: the cheap variant of the same idea, used by the fused collectives when the links are
// not the bottleneck.  Always four code bits with the window anchored at the chunk's largest
// exponent (base = max(emax - 14, 0): no histogram, no candidate search), and the 4-bit codes
// packed two per byte instead of sliced into four bit planes: byte 4 k + j of a lane's 16 code bytes
// holds element 8 k + j in its low nibble and element 8 k + 4 + j in its high one, so that encode is
// one shift-or per eight elements and decode two masks.  Same header word (base | 4 << 8 |
// n_esc << 16), same record size (1024 + 512 + n_esc bytes), same escape rule and raw fallback as
// width 4 of the plane format; which of the two layouts a width-4 record has is a property of the
// stream (the caller's choice), not of the record.  About 1.50 bytes per element on weights and
// gradients against 1.40 for the plane format, for roughly half the instructions.
// Writes only rec[1024 ...) (the sign+mantissa bytes are the caller's).  Returns the header.
__device__ __forceinline__ uint32_t v2_encode_chunk_nibble(const LaneSplit& s, uint8_t* rec, int lane) {
  uint32_t mx = s.ex[0], mn = s.ex[0];
#pragma unroll
  for (int k = 1; k < 8; ++k) {
    mx = __vmaxu4(mx, s.ex[k]);
    mn = __vminu4(mn, s.ex[k]);
  }
  const uint32_t mxb = max(max(mx & 0xFF, (mx >> 8) & 0xFF), max((mx >> 16) & 0xFF, mx >> 24));
  const uint32_t mnb = min(min(mn & 0xFF, (mn >> 8) & 0xFF), min((mn >> 16) & 0xFF, mn >> 24));
  const int emax = (int)__reduce_max_sync(FULL, mxb);
  const int emin = (int)__reduce_min_sync(FULL, mnb);
  if (emin == emax) return v2_header(emax, 0, 0);
  const int base = emax > 14 ? emax - 14 : 0;
  uint32_t code[8];
  codes_lane(s, base, 15u, code);
  int n_esc = 0, pos = 0;
  uint32_t zm = 0;
  if (emin < base) {  // warp-uniform: only then can an element fall below the window
    zm = zero_mask(code);
    pos = warp_excl_scan(__popc(zm), lane, n_esc);
    if (512 + n_esc > V2_CHUNK_ELEMS) {
      uint4* ep = reinterpret_cast<uint4*>(rec + 1024 + lane * 32);
      ep[0] = make_uint4(s.ex[0], s.ex[1], s.ex[2], s.ex[3]);
      ep[1] = make_uint4(s.ex[4], s.ex[5], s.ex[6], s.ex[7]);
      return v2_header(0, V2_RAW_WIDTH, 0);
    }
  }
  reinterpret_cast<uint4*>(rec + 1024)[lane] = make_uint4(code[0] | (code[1] << 4), code[2] | (code[3] << 4),
                                                          code[4] | (code[5] << 4), code[6] | (code[7] << 4));
  if (n_esc > 0) scatter_escapes(rec + 1024 + 512 + pos, s, zm);
  return v2_header(base, 4, n_esc);
}

// Decode one chunk record into split fields.
__device__ __forceinline__ void v2_decode_chunk(const uint8_t* rec, uint32_t hdr, int lane, LaneSplit& s) {
  const int w = v2_hdr_width(hdr);
  const int base = v2_hdr_base(hdr);
  const uint4* smp = reinterpret_cast<const uint4*>(rec + lane * 32);
  const uint4 a = smp[0], b = smp[1];
  s.sm[0] = a.x; s.sm[1] = a.y; s.sm[2] = a.z; s.sm[3] = a.w;
  s.sm[4] = b.x; s.sm[5] = b.y; s.sm[6] = b.z; s.sm[7] = b.w;
  if (w == V2_RAW_WIDTH) {
    const uint4* ep = reinterpret_cast<const uint4*>(rec + 1024 + lane * 32);
    const uint4 c = ep[0], d = ep[1];
    s.ex[0] = c.x; s.ex[1] = c.y; s.ex[2] = c.z; s.ex[3] = c.w;
    s.ex[4] = d.x; s.ex[5] = d.y; s.ex[6] = d.z; s.ex[7] = d.w;
    return;
  }
  if (w == 0) {
    const uint32_t e4 = rep4((uint32_t)base);
#pragma unroll
    for (int k = 0; k < 8; ++k) s.ex[k] = e4;
    return;
  }
  uint32_t planes[4] = {0, 0, 0, 0};
  const uint32_t* pl = reinterpret_cast<const uint32_t*>(rec + 1024) + lane;
  planes[0] = pl[0];
  if (w > 1) planes[1] = pl[32];
  if (w > 2) planes[2] = pl[64];
  if (w > 3) planes[3] = pl[96];
  uint32_t zm = ~planes[0];
  if (w > 1) zm &= ~planes[1];
  if (w > 2) zm &= ~planes[2];
  if (w > 3) zm &= ~planes[3];
  int total;
  const int pos = warp_excl_scan(__popc(zm), lane, total);
  const uint8_t* esc = rec + 1024 + 128 * w + pos;
  switch (w) {
    case 1: decode_lane<1>(planes, base, esc, s.ex); break;
    case 2: decode_lane<2>(planes, base, esc, s.ex); break;
    case 3: decode_lane<3>(planes, base, esc, s.ex); break;
    default: decode_lane<4>(planes, base, esc, s.ex); break;
  }
}

// ---------------------------------------------------------------------------------------------
// Two-phase decode: `v2_prefetch` issues every global load a lane needs of one record (32 sign +
// mantissa bytes, its word of up to four planes, its share of the escape bytes) without using the
// values, `v2_decode_regs` turns them into exponents later.  A decoder that prefetches record i+1
// before it decodes record i keeps one record's loads in flight per warp at all times, which is what
// hides the memory latency when few warps per SM are available (inside the fused collectives, next
// to a GEMM).  Escapes go through 1 KB of shared memory per warp: the lanes store the 16-byte pieces
// they fetched, then every lane picks its own bytes by prefix position (no serial global loads).
// Loads use ld.global.cg: records may have been written by another GPU.
// ---------------------------------------------------------------------------------------------
struct RecRegs {
  uint32_t hdr;
  uint4 sm0, sm1;   // sign+mantissa bytes of this lane (raw mode: e0/e1 hold its exponent bytes)
  uint32_t pl[4];
  uint4 e0, e1;     // bytes [16 lane, 16 lane + 16) and [512 + 16 lane, ...) of the escape area
};

// SM_SPLIT: the sign+mantissa section is stored as two 512-byte halves (lane l's bytes 0..15 at 16 l,
// bytes 16..31 at 512 + 16 l) instead of 32 consecutive bytes per lane.  The fused collectives stage
// their records that way: each of a warp's two stores then covers 512 contiguous bytes of the peer's
// memory instead of 32 half-used 32-byte sectors.  Records in the documented format use SM_SPLIT = false.
// NIBBLE: width-4 records of this stream carry nibble-packed codes (v2_encode_chunk_nibble): a lane's
// 16 code bytes are one load and land in pl[0..3].
template <bool SM_SPLIT = false, bool NIBBLE = false>
__device__ __forceinline__ void v2_prefetch(const uint8_t* rec, uint32_t hdr, int lane, RecRegs& r) {
  r.hdr = hdr;
  if (SM_SPLIT) {
    const uint4* smp = reinterpret_cast<const uint4*>(rec) + lane;
    r.sm0 = __ldcg(smp);
    r.sm1 = __ldcg(smp + 32);
  } else {
    const uint4* smp = reinterpret_cast<const uint4*>(rec + lane * 32);
    r.sm0 = __ldcg(smp);
    r.sm1 = __ldcg(smp + 1);
  }
  const int w = v2_hdr_width(hdr);
  if (w == V2_RAW_WIDTH) {
    const uint4* ep = reinterpret_cast<const uint4*>(rec + 1024 + lane * 32);
    r.e0 = __ldcg(ep);
    r.e1 = __ldcg(ep + 1);
    return;
  }
  if (w == 0) return;
  if (NIBBLE) {
    const uint4 nb = __ldcg(reinterpret_cast<const uint4*>(rec + 1024) + lane);
    r.pl[0] = nb.x; r.pl[1] = nb.y; r.pl[2] = nb.z; r.pl[3] = nb.w;
  } else {
    const uint32_t* pl = reinterpret_cast<const uint32_t*>(rec + 1024) + lane;
    r.pl[0] = __ldcg(pl);
    r.pl[1] = w > 1 ? __ldcg(pl + 32) : 0u;
    r.pl[2] = w > 2 ? __ldcg(pl + 64) : 0u;
    r.pl[3] = w > 3 ? __ldcg(pl + 96) : 0u;
  }
  const int n_esc = v2_hdr_nesc(hdr);
  const uint4* eb = reinterpret_cast<const uint4*>(rec + 1024 + 128 * w);
  if (16 * lane < n_esc) r.e0 = __ldcg(eb + lane);
  if (512 + 16 * lane < n_esc) r.e1 = __ldcg(eb + 32 + lane);
}

// `esc_smem`: 1024 bytes of shared memory owned by this warp (16-byte aligned).
template <bool NIBBLE = false>
__device__ __forceinline__ void v2_decode_regs(const RecRegs& r, uint8_t* esc_smem, int lane, LaneSplit& s) {
  s.sm[0] = r.sm0.x; s.sm[1] = r.sm0.y; s.sm[2] = r.sm0.z; s.sm[3] = r.sm0.w;
  s.sm[4] = r.sm1.x; s.sm[5] = r.sm1.y; s.sm[6] = r.sm1.z; s.sm[7] = r.sm1.w;
  const int w = v2_hdr_width(r.hdr);
  const int base = v2_hdr_base(r.hdr);
  if (w == V2_RAW_WIDTH) {
    s.ex[0] = r.e0.x; s.ex[1] = r.e0.y; s.ex[2] = r.e0.z; s.ex[3] = r.e0.w;
    s.ex[4] = r.e1.x; s.ex[5] = r.e1.y; s.ex[6] = r.e1.z; s.ex[7] = r.e1.w;
    return;
  }
  if (w == 0) {
    const uint32_t e4 = rep4((uint32_t)base);
#pragma unroll
    for (int k = 0; k < 8; ++k) s.ex[k] = e4;
    return;
  }
  const int n_esc = v2_hdr_nesc(r.hdr);
  if (NIBBLE) {
    // codes: four per word after two masks; e = base + code - 1 for code >= 1
    uint32_t code[8];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      code[2 * k] = r.pl[k] & 0x0F0F0F0Fu;
      code[2 * k + 1] = (r.pl[k] >> 4) & 0x0F0F0F0Fu;
    }
    if (n_esc == 0) {  // warp-uniform: no code is zero, so base - 1 is added to every byte (base >= 1 here,
                       // or base == 0 where the sum wraps to code - 1 per byte without carrying out: code >= 1)
      const uint32_t y = rep4((uint32_t)(base - 1));
      const uint32_t yl = y & L4, yh = y & H4;
#pragma unroll
      for (int k = 0; k < 8; ++k) s.ex[k] = ((code[k] & L4) + yl) ^ ((code[k] & H4) ^ yh);   // per-byte add mod 256
      return;
    }
    uint4* es = reinterpret_cast<uint4*>(esc_smem);
    if (16 * lane < n_esc) es[lane] = r.e0;
    if (512 + 16 * lane < n_esc) es[32 + lane] = r.e1;
    const uint32_t zmn = zero_mask(code);
    int total;
    const int posn = warp_excl_scan(__popc(zmn), lane, total);
    __syncwarp();
    const uint8_t* escn = esc_smem + posn;
    const uint32_t b4 = rep4((uint32_t)base);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const uint32_t nz = nzmask4(code[k]);
      s.ex[k] = (code[k] - (nz & 0x01010101u)) + (b4 & nz);
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      uint32_t m = (zmn >> (4 * k)) & 0xFu;
      while (m) {
        const int j = __ffs(m) - 1;
        s.ex[k] |= (uint32_t)(*escn++) << (j * 8);
        m &= m - 1;
      }
    }
    __syncwarp();  // the next record's escapes overwrite esc_smem
    return;
  }
  uint32_t planes[4] = {r.pl[0], r.pl[1], r.pl[2], r.pl[3]};
  uint32_t zm = ~planes[0];
  if (w > 1) zm &= ~planes[1];
  if (w > 2) zm &= ~planes[2];
  if (w > 3) zm &= ~planes[3];
  int pos = 0;
  if (n_esc > 0) {  // warp-uniform
    uint4* es = reinterpret_cast<uint4*>(esc_smem);
    if (16 * lane < n_esc) es[lane] = r.e0;
    if (512 + 16 * lane < n_esc) es[32 + lane] = r.e1;
    int total;
    pos = warp_excl_scan(__popc(zm), lane, total);
    __syncwarp();
  }
  const uint8_t* esc = esc_smem + pos;
  switch (w) {
    case 1: decode_lane<1>(planes, base, esc, s.ex); break;
    case 2: decode_lane<2>(planes, base, esc, s.ex); break;
    case 3: decode_lane<3>(planes, base, esc, s.ex); break;
    default: decode_lane<4>(planes, base, esc, s.ex); break;
  }
  if (n_esc > 0) __syncwarp();  // the next record's escapes overwrite esc_smem
}
}  // namespace zc
