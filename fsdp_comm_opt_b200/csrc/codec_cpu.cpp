// Scalar C++ implementation of the v1 and v2 BF16 exponent codecs.
//
// Three jobs: (1) the oracle the sm_100a kernels are tested against, (2) the codec that CPU/gloo
// ranks use behind the comm hooks, (3) the timed CPU baseline.  The reference has no CPU path;
// the v1 functions here restate the math of its kernels (zipccl/hopper_zip.cu:82-100, 162-200,
// 409-461, 826-853) with deterministic, in-order outlier placement.
//
// Plain C ABI, loaded with ctypes.  All sizes are int64; offsets never narrow to 32 bit.
#include <cstring>
#include <vector>

#include "codec_format.h"

using namespace zc;

namespace {

// Encode one 4096-element block.  `src` may be null past `valid` elements (zero padding).
// Returns the number of outliers appended at `esc` (in element order).
int v1_encode_block(const uint16_t* src, int64_t valid, int base, uint8_t* sm, uint32_t* b0,
                    uint32_t* b1, uint32_t* b2, uint8_t* esc) {
  int n_esc = 0;
  for (int t = 0; t < V1_THREADS; ++t) {
    uint32_t w0 = 0, w1 = 0, w2 = 0;
    for (int j = 0; j < 32; ++j) {
      const int64_t i = (int64_t)t * 32 + j;
      const uint16_t v = i < valid ? src[i] : (uint16_t)0;
      sm[i] = bf16_sm(v);
      const int e = bf16_exp(v);
      const unsigned code = (e >= base && e < base + V1_WINDOW) ? (unsigned)(e - base + 1) : 0u;
      w0 |= ((code >> 0) & 1u) << j;
      w1 |= ((code >> 1) & 1u) << j;
      w2 |= ((code >> 2) & 1u) << j;
      if (code == 0) esc[n_esc++] = (uint8_t)e;
    }
    b0[t] = w0; b1[t] = w1; b2[t] = w2;
  }
  return n_esc;
}

void v1_decode_block(const uint8_t* sm, const uint32_t* b0, const uint32_t* b1, const uint32_t* b2,
                     const uint8_t* esc, int base, uint16_t* dst, int64_t valid) {
  int k = 0;
  for (int t = 0; t < V1_THREADS; ++t) {
    const uint32_t w0 = b0[t], w1 = b1[t], w2 = b2[t];
    for (int j = 0; j < 32; ++j) {
      const int64_t i = (int64_t)t * 32 + j;
      const unsigned code = ((w0 >> j) & 1u) | (((w1 >> j) & 1u) << 1) | (((w2 >> j) & 1u) << 2);
      const uint8_t e = code ? (uint8_t)(base + code - 1) : esc[k++];
      if (i < valid) dst[i] = bf16_join(sm[i], e);
    }
  }
}

}  // namespace

extern "C" {

int64_t zc_cpu_v1_det_bytes(int64_t n_padded) { return align128(v1_det_bytes(n_padded)); }

// Split-layout encode of `n_works` works.
//   in        dense input; work i reads orig_n[i] elements starting where work i-1 ended when
//             orig_n != null (the "pad" variant), else reads n_8[i] elements at the padded
//             offset and zero-fills past total_n.
//   det       det streams back to back (stride align128(det_bytes(n_8[i])))
//   esc_final compacted outliers, stride align128(count[i])
//   counts    out: outliers per work
void zc_cpu_v1_encode_split(const uint16_t* in, int64_t total_n, const int32_t* n_8,
                            const int32_t* orig_n, int n_works, int base, uint8_t* det,
                            uint8_t* esc_final, int32_t* counts) {
  int64_t in_off = 0, det_off = 0, esc_off = 0;
  std::vector<uint8_t> esc;
  for (int w = 0; w < n_works; ++w) {
    const int64_t n = n_8[w];
    const int64_t nb = n / V1_BLOCK_ELEMS;
    if (n == 0) { counts[w] = 0; continue; }
    uint8_t* sm = det + det_off;
    uint32_t* b0 = reinterpret_cast<uint32_t*>(sm + n);
    uint32_t* b1 = b0 + n / 32;
    uint32_t* b2 = b1 + n / 32;
    int32_t* boff = reinterpret_cast<int32_t*>(b2 + n / 32);
    esc.assign((size_t)n, 0);
    int64_t cnt = 0;
    const int64_t valid_work = orig_n ? (int64_t)orig_n[w]
                                      : (total_n - in_off < n ? (total_n - in_off > 0 ? total_n - in_off : 0) : n);
    for (int64_t b = 0; b < nb; ++b) {
      const int64_t e0 = b * V1_BLOCK_ELEMS;
      int64_t valid = valid_work - e0;
      if (valid < 0) valid = 0;
      if (valid > V1_BLOCK_ELEMS) valid = V1_BLOCK_ELEMS;
      boff[b] = (int32_t)cnt;
      cnt += v1_encode_block(in + in_off + e0, valid, base, sm + e0, b0 + b * V1_THREADS,
                             b1 + b * V1_THREADS, b2 + b * V1_THREADS, esc.data() + cnt);
    }
    boff[nb] = base;
    counts[w] = (int32_t)cnt;
    std::memcpy(esc_final + esc_off, esc.data(), (size_t)cnt);
    in_off += orig_n ? (int64_t)orig_n[w] : n;
    det_off += align128(v1_det_bytes(n));
    esc_off += align128(cnt);
  }
}

// Split-layout decode.  Work i writes min(valid_i, n_8[i]) elements at out + out_off_i where
//   valid_i  = orig_n[i] if orig_n else (orig_each >= 0 ? orig_each : n_8[i])
//   out_off_i= out_off[i] if out_off else i * (orig_each >= 0 ? orig_each : padded prefix)
void zc_cpu_v1_decode_split(const uint8_t* det, const uint8_t* esc, const int32_t* n_8,
                            const int32_t* nbytes_8, int n_works, int64_t orig_each,
                            const int32_t* out_off, const int32_t* orig_n, uint16_t* out) {
  int64_t det_off = 0, esc_off = 0, pad_prefix = 0;
  for (int w = 0; w < n_works; ++w) {
    const int64_t n = n_8[w];
    const int64_t nb = n / V1_BLOCK_ELEMS;
    if (n > 0) {
      const uint8_t* sm = det + det_off;
      const uint32_t* b0 = reinterpret_cast<const uint32_t*>(sm + n);
      const uint32_t* b1 = b0 + n / 32;
      const uint32_t* b2 = b1 + n / 32;
      const int32_t* boff = reinterpret_cast<const int32_t*>(b2 + n / 32);
      const int base = boff[nb];
      const int64_t valid_work = orig_n ? (int64_t)orig_n[w] : (orig_each >= 0 ? orig_each : n);
      const int64_t o = out_off ? (int64_t)out_off[w] : (orig_each >= 0 ? w * orig_each : pad_prefix);
      for (int64_t b = 0; b < nb; ++b) {
        const int64_t e0 = b * V1_BLOCK_ELEMS;
        int64_t valid = valid_work - e0;
        if (valid <= 0) break;
        if (valid > V1_BLOCK_ELEMS) valid = V1_BLOCK_ELEMS;
        v1_decode_block(sm + e0, b0 + b * V1_THREADS, b1 + b * V1_THREADS, b2 + b * V1_THREADS,
                        esc + esc_off + boff[b], base, out + o + e0, valid);
      }
    }
    pad_prefix += n;
    det_off += align128(v1_det_bytes(n));
    esc_off += align128((int64_t)nbytes_8[w]);
  }
}

// Fused-layout encode: work i occupies nbytes_8[i] = align128(det_bytes + count) bytes of `out`,
// works back to back.  Returns total bytes written.
int64_t zc_cpu_v1_encode_fused(const uint16_t* in, int64_t total_n, const int32_t* n_8, int n_works,
                               int base, uint8_t* out, int32_t* nbytes_8, int32_t* counts) {
  int64_t in_off = 0, out_off = 0;
  for (int w = 0; w < n_works; ++w) {
    const int64_t n = n_8[w];
    const int64_t nb = n / V1_BLOCK_ELEMS;
    if (n == 0) { nbytes_8[w] = 0; counts[w] = 0; continue; }
    uint8_t* sm = out + out_off;
    uint32_t* b0 = reinterpret_cast<uint32_t*>(sm + n);
    uint32_t* b1 = b0 + n / 32;
    uint32_t* b2 = b1 + n / 32;
    int32_t* boff = reinterpret_cast<int32_t*>(b2 + n / 32);
    uint8_t* esc = reinterpret_cast<uint8_t*>(boff + nb + 1);
    int64_t cnt = 0;
    for (int64_t b = 0; b < nb; ++b) {
      const int64_t e0 = b * V1_BLOCK_ELEMS;
      int64_t valid = total_n - (in_off + e0);
      if (valid < 0) valid = 0;
      if (valid > V1_BLOCK_ELEMS) valid = V1_BLOCK_ELEMS;
      boff[b] = (int32_t)cnt;
      cnt += v1_encode_block(in + in_off + e0, valid, base, sm + e0, b0 + b * V1_THREADS,
                             b1 + b * V1_THREADS, b2 + b * V1_THREADS, esc + cnt);
    }
    boff[nb] = base;
    counts[w] = (int32_t)cnt;
    const int64_t bytes = align128(v1_det_bytes(n) + cnt);
    nbytes_8[w] = (int32_t)bytes;
    in_off += n;
    out_off += bytes;
  }
  return out_off;
}

// Fused-layout decode; same output addressing rules as zc_cpu_v1_decode_split.
void zc_cpu_v1_decode_fused(const uint8_t* comp, const int32_t* n_8, const int32_t* nbytes_8,
                            int n_works, int64_t orig_each, uint16_t* out) {
  int64_t off = 0, pad_prefix = 0;
  for (int w = 0; w < n_works; ++w) {
    const int64_t n = n_8[w];
    const int64_t nb = n / V1_BLOCK_ELEMS;
    if (n > 0) {
      const uint8_t* sm = comp + off;
      const uint32_t* b0 = reinterpret_cast<const uint32_t*>(sm + n);
      const uint32_t* b1 = b0 + n / 32;
      const uint32_t* b2 = b1 + n / 32;
      const int32_t* boff = reinterpret_cast<const int32_t*>(b2 + n / 32);
      const uint8_t* esc = reinterpret_cast<const uint8_t*>(boff + nb + 1);
      const int base = boff[nb];
      const int64_t valid_work = orig_each >= 0 ? orig_each : n;
      const int64_t o = orig_each >= 0 ? w * orig_each : pad_prefix;
      for (int64_t b = 0; b < nb; ++b) {
        const int64_t e0 = b * V1_BLOCK_ELEMS;
        int64_t valid = valid_work - e0;
        if (valid <= 0) break;
        if (valid > V1_BLOCK_ELEMS) valid = V1_BLOCK_ELEMS;
        v1_decode_block(sm + e0, b0 + b * V1_THREADS, b1 + b * V1_THREADS, b2 + b * V1_THREADS,
                        esc + boff[b], base, out + o + e0, valid);
      }
    }
    pad_prefix += n;
    off += nbytes_8[w];
  }
}

// ------------------------------------------------------------------------------------------
// v2
// ------------------------------------------------------------------------------------------

// Encode n elements into ceil(n/1024) records at fixed stride 2048 B plus one header each.
// Returns the sum of used record bytes (the bytes that would cross the wire, headers excluded).
int64_t zc_cpu_v2_encode(const uint16_t* in, int64_t n, uint8_t* records, uint32_t* headers) {
  const int64_t nc = (n + V2_CHUNK_ELEMS - 1) / V2_CHUNK_ELEMS;
  int64_t used = 0;
  for (int64_t c = 0; c < nc; ++c) {
    uint8_t* rec = records + c * V2_SLOT_BYTES;
    uint8_t ex[V2_CHUNK_ELEMS];
    int emax = 0, emin = 255;
    for (int i = 0; i < V2_CHUNK_ELEMS; ++i) {
      const int64_t g = c * V2_CHUNK_ELEMS + i;
      const uint16_t v = g < n ? in[g] : (uint16_t)0;
      rec[i] = bf16_sm(v);
      ex[i] = bf16_exp(v);
      if (ex[i] > emax) emax = ex[i];
      if (ex[i] < emin) emin = ex[i];
    }
    uint32_t hdr;
    if (emin == emax) {
      hdr = v2_header(emax, 0, 0);
    } else {
      const int anchor = emax > 15 ? emax - 15 : 0;
      int prefix[17] = {0};
      int h[16] = {0};
      for (int i = 0; i < V2_CHUNK_ELEMS; i += 4) {
        const int d = (int)ex[i] - anchor;
        if (d >= 0) h[d]++;
      }
      for (int k = 0; k < 16; ++k) prefix[k + 1] = prefix[k] + h[k];
      hdr = v2_choose(prefix, anchor);
    }
    int w = v2_hdr_width(hdr);
    const int base = v2_hdr_base(hdr);
    if (w != V2_RAW_WIDTH && w > 0) {
      const unsigned span = (1u << w) - 1u;
      int n_esc = 0;
      for (int i = 0; i < V2_CHUNK_ELEMS; ++i) n_esc += ((unsigned)((int)ex[i] - base) < span) ? 0 : 1;
      if (128 * w + n_esc > V2_CHUNK_ELEMS) { hdr = v2_header(0, V2_RAW_WIDTH, 0); w = V2_RAW_WIDTH; }
      else hdr = v2_header(base, w, n_esc);
    }
    headers[c] = hdr;
    if (w == V2_RAW_WIDTH) {
      std::memcpy(rec + 1024, ex, 1024);
    } else if (w > 0) {
      uint32_t* planes = reinterpret_cast<uint32_t*>(rec + 1024);
      uint8_t* esc = rec + 1024 + 128 * w;
      const unsigned span = (1u << w) - 1u;
      int n_esc = 0;
      for (int l = 0; l < 32; ++l) {
        uint32_t pw[4] = {0, 0, 0, 0};
        for (int j = 0; j < 32; ++j) {
          const int e = ex[l * 32 + j];
          const unsigned d = (unsigned)(e - base);
          const unsigned code = d < span ? d + 1 : 0u;
          for (int p = 0; p < w; ++p) pw[p] |= ((code >> p) & 1u) << j;
          if (code == 0) esc[n_esc++] = (uint8_t)e;
        }
        for (int p = 0; p < w; ++p) planes[p * 32 + l] = pw[p];
      }
    }
    used += v2_record_bytes(hdr);
  }
  return used;
}

void zc_cpu_v2_decode(const uint8_t* records, const uint32_t* headers, int64_t n, uint16_t* out) {
  const int64_t nc = (n + V2_CHUNK_ELEMS - 1) / V2_CHUNK_ELEMS;
  for (int64_t c = 0; c < nc; ++c) {
    const uint8_t* rec = records + c * V2_SLOT_BYTES;
    const uint32_t hdr = headers[c];
    const int w = v2_hdr_width(hdr), base = v2_hdr_base(hdr);
    const uint32_t* planes = reinterpret_cast<const uint32_t*>(rec + 1024);
    const uint8_t* esc = rec + 1024 + 128 * (w == V2_RAW_WIDTH ? 0 : w);
    int k = 0;
    for (int i = 0; i < V2_CHUNK_ELEMS; ++i) {
      const int64_t g = c * V2_CHUNK_ELEMS + i;
      uint8_t e;
      if (w == V2_RAW_WIDTH) {
        e = rec[1024 + i];
      } else if (w == 0) {
        e = (uint8_t)base;
      } else {
        const int l = i >> 5, j = i & 31;
        unsigned code = 0;
        for (int p = 0; p < w; ++p) code |= ((planes[p * 32 + l] >> j) & 1u) << p;
        e = code ? (uint8_t)(base + code - 1) : esc[k++];
      }
      if (g < n) out[g] = bf16_join(rec[i], e);
    }
  }
}

// Nibble mode (codec_format.h): fixed four code bits, base = max(emax - 14, 0), lane l's sixteen code
// bytes at 1024 + 16 l, byte 4 k + j holding element 32 l + 8 k + j (low nibble) and 32 l + 8 k + 4 + j
// (high nibble); width 0, escapes and the raw fallback as in the plane format.
int64_t zc_cpu_v2_encode_nibble(const uint16_t* in, int64_t n, uint8_t* records, uint32_t* headers) {
  const int64_t nc = (n + V2_CHUNK_ELEMS - 1) / V2_CHUNK_ELEMS;
  int64_t used = 0;
  for (int64_t c = 0; c < nc; ++c) {
    uint8_t* rec = records + c * V2_SLOT_BYTES;
    uint8_t ex[V2_CHUNK_ELEMS];
    int emax = 0, emin = 255;
    for (int i = 0; i < V2_CHUNK_ELEMS; ++i) {
      const int64_t g = c * V2_CHUNK_ELEMS + i;
      const uint16_t v = g < n ? in[g] : (uint16_t)0;
      rec[i] = bf16_sm(v);
      ex[i] = bf16_exp(v);
      if (ex[i] > emax) emax = ex[i];
      if (ex[i] < emin) emin = ex[i];
    }
    uint32_t hdr;
    if (emin == emax) {
      hdr = v2_header(emax, 0, 0);
    } else {
      const int base = emax > 14 ? emax - 14 : 0;
      int n_esc = 0;
      for (int i = 0; i < V2_CHUNK_ELEMS; ++i) n_esc += ((unsigned)((int)ex[i] - base) < 15u) ? 0 : 1;
      if (512 + n_esc > V2_CHUNK_ELEMS) {
        hdr = v2_header(0, V2_RAW_WIDTH, 0);
        std::memcpy(rec + 1024, ex, 1024);
      } else {
        hdr = v2_header(base, 4, n_esc);
        uint8_t* codes = rec + 1024;
        uint8_t* esc = rec + 1024 + 512;
        std::memset(codes, 0, 512);
        int k = 0;
        for (int i = 0; i < V2_CHUNK_ELEMS; ++i) {
          const unsigned d = (unsigned)((int)ex[i] - base);
          const unsigned code = d < 15u ? d + 1 : 0u;
          const int l = i >> 5, j = i & 31, kk = j >> 3, jj = j & 7;
          codes[16 * l + 4 * kk + (jj & 3)] |= (uint8_t)(jj < 4 ? code : code << 4);
          if (code == 0) esc[k++] = ex[i];
        }
      }
    }
    headers[c] = hdr;
    used += v2_record_bytes(hdr);
  }
  return used;
}

void zc_cpu_v2_decode_nibble(const uint8_t* records, const uint32_t* headers, int64_t n, uint16_t* out) {
  const int64_t nc = (n + V2_CHUNK_ELEMS - 1) / V2_CHUNK_ELEMS;
  for (int64_t c = 0; c < nc; ++c) {
    const uint8_t* rec = records + c * V2_SLOT_BYTES;
    const uint32_t hdr = headers[c];
    const int w = v2_hdr_width(hdr), base = v2_hdr_base(hdr);
    const uint8_t* codes = rec + 1024;
    const uint8_t* esc = rec + 1024 + 512;
    int k = 0;
    for (int i = 0; i < V2_CHUNK_ELEMS; ++i) {
      const int64_t g = c * V2_CHUNK_ELEMS + i;
      uint8_t e;
      if (w == V2_RAW_WIDTH) {
        e = rec[1024 + i];
      } else if (w == 0) {
        e = (uint8_t)base;
      } else {
        const int l = i >> 5, j = i & 31, kk = j >> 3, jj = j & 7;
        const uint8_t b = codes[16 * l + 4 * kk + (jj & 3)];
        const unsigned code = jj < 4 ? (b & 0xFu) : (unsigned)(b >> 4);
        e = code ? (uint8_t)(base + code - 1) : esc[k++];
      }
      if (g < n) out[g] = bf16_join(rec[i], e);
    }
  }
}

// Gather the used bytes of every record into one dense stream.  offsets[c] (int64) receives the
// start of record c; offsets[nc] the total.  Returns the total.
int64_t zc_cpu_v2_compact(const uint8_t* records, const uint32_t* headers, int64_t nc, uint8_t* dense,
                          int64_t* offsets) {
  int64_t off = 0;
  for (int64_t c = 0; c < nc; ++c) {
    offsets[c] = off;
    const int b = v2_record_bytes(headers[c]);
    if (dense) std::memcpy(dense + off, records + c * V2_SLOT_BYTES, (size_t)b);
    off += b;
  }
  offsets[nc] = off;
  return off;
}

void zc_cpu_v2_expand(const uint8_t* dense, const uint32_t* headers, int64_t nc, uint8_t* records) {
  int64_t off = 0;
  for (int64_t c = 0; c < nc; ++c) {
    const int b = v2_record_bytes(headers[c]);
    std::memcpy(records + c * V2_SLOT_BYTES, dense + off, (size_t)b);
    off += b;
  }
}

}  // extern "C"
