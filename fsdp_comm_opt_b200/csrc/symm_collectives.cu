// Fused compressed collectives over NVLink peer memory (sm_100a): one kernel per collective does
// encode -> push into the peers' symmetric staging buffers -> signal -> bounded wait -> decode
// (-> fp32 reduce).  No NCCL call, no host sync, no allocation; sizes travel in band (one uint32
// header per chunk), so only the used bytes of each v2 record cross the wire.
//
// Symmetric buffer layout (identical on every rank; `peers[q]` is rank q's buffer in this rank's
// address space, obtained from the symmetric-memory rendezvous):
//   [0, 4096)                 control: done[world] (uint32), local counters
//   [4096, 4096 + flag_bytes) flags[2 parities][world sources][max_groups] (uint32)
//   data                      2 parities x world source slots; slot = header table + records
// A "group" is 8 to 64 chunks (the launcher picks the size so that small messages still spread over
// many CTAs; the flag area is sized for groups of 64).  The pusher CTAs encode group after group and,
// after a system-scope fence, release-store flag[parity][me][group] = seq on the receivers.  The
// decoder warps (each on its own slice of eight chunks) acquire-load their local flags and decode as
// groups arrive, so push, transfer and decode overlap inside one launch.  A decoder warp keeps the
// next record's loads in flight while it decodes the current one (v2_prefetch / v2_decode_regs):
// beside a GEMM only a few warps per SM are available, and it is the loads in flight that set the
// decode rate.  Buffers alternate by call parity; before pushing call `seq` a rank
// waits until every peer has reported done >= seq - 2 (it finished reading that parity).
// Waits are bounded by wall time; on expiry the kernel records {code, peer, group} in the status
// words of its own control block and returns normally, leaving the context usable.
//
// Peer memory is only touched with plain ld/st (st.release.sys for flags) and, for the all-gather
// payload where the buffer has an NVSwitch multicast mapping, multimem.st; no bulk-tensor copies.
#include <cuda_bf16.h>

#include "codec_v2_dev.cuh"
#include "launch_util.h"
#include "nvtx_util.h"

namespace zc {

constexpr int GROUP_CHUNKS = 64;
constexpr int CTRL_BYTES = 4096;
// control block word indices (uint32)
constexpr int CW_DONE = 0;        // done[q], q < 64
constexpr int CW_COUNTER = 64;    // decoder CTAs finished in this call
constexpr int CW_STATUS = 65;     // 0 ok, else code
constexpr int CW_STATUS_PEER = 66;
constexpr int CW_STATUS_GROUP = 67;
constexpr int CW_WIRE_LO = 68;    // 64-bit count of record bytes pushed (all calls)

struct SymmLayout {
  int world, rank;
  long long nc_max;      // chunks per source slot
  int max_groups;
  long long flag_bytes, hdr_bytes, slot_bytes, parity_bytes;
};

__device__ __forceinline__ uint32_t* ctrl(uint8_t* buf) { return reinterpret_cast<uint32_t*>(buf); }
__device__ __forceinline__ uint32_t* flag_ptr(uint8_t* buf, const SymmLayout& L, int parity, int src, long long g) {
  return reinterpret_cast<uint32_t*>(buf + CTRL_BYTES) + ((long long)parity * L.world + src) * L.max_groups + g;
}
__device__ __forceinline__ uint8_t* slot_ptr(uint8_t* buf, const SymmLayout& L, int parity, int src) {
  return buf + CTRL_BYTES + L.flag_bytes + parity * L.parity_bytes + src * L.slot_bytes;
}

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// spin until *p >= want (sequence numbers only grow); false on timeout
__device__ __forceinline__ bool wait_ge(const uint32_t* p, uint32_t want, unsigned long long limit_ns) {
  if ((int)(ld_acquire_sys(p) - want) >= 0) return true;
  const unsigned long long t0 = now_ns();
  for (uint32_t it = 0;; ++it) {
    if ((int)(ld_acquire_sys(p) - want) >= 0) return true;
    if ((it & 31u) == 31u && now_ns() - t0 > limit_ns) return false;
    __nanosleep(64);
  }
}
// (the last control word holds the device pointer of the library's health word, written by the launcher)
constexpr int CW_HEALTH_PTR = 72;  // two words: 64-bit device address or 0
__device__ __forceinline__ void set_status(uint8_t* local, int code, int peer, long long group) {
  uint32_t* c = ctrl(local);
  int* health = *reinterpret_cast<int**>(c + CW_HEALTH_PTR);
  if (health) atomicCAS(health, 0, code);
  if (atomicCAS(c + CW_STATUS, 0u, (uint32_t)code) == 0u) {
    c[CW_STATUS_PEER] = (uint32_t)peer;
    c[CW_STATUS_GROUP] = (uint32_t)group;
  }
}

// Debug-bounds build (-DZC_DEBUG_BOUNDS; compute-sanitizer's stand-in for stores into peer memory):
// every record store is checked against the extent of the destination slot and every header store
// against the header table before it is issued.  A store that would leave its slot is skipped and
// recorded in the status words as code 3 with the peer and the chunk; nothing traps.
#ifdef ZC_DEBUG_BOUNDS
#define ZC_SLOT_OK(L, c, used, local, peer)                                                            \
  (((c) >= 0 && (c) < (L).nc_max && (L).hdr_bytes + ((c) + 1) * (long long)V2_SLOT_BYTES <= (L).slot_bytes && \
    (used) >= 0 && (used) <= V2_SLOT_BYTES)                                                             \
       ? true                                                                                          \
       : (set_status((local), 3, (peer), (c)), false))
#else
#define ZC_SLOT_OK(L, c, used, local, peer) true
#endif

// copy `bytes` (rounded up to 16) from shared memory to global/peer memory, warp-cooperative
__device__ __forceinline__ void warp_copy16(uint8_t* dst, const uint8_t* src, int bytes, int lane) {
  const int nv = (bytes + 15) >> 4;
  for (int i = lane; i < nv; i += 32)
    reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
}

// the 32 sign+mantissa bytes of one lane, straight from registers to (peer) memory, as two halves 512
// bytes apart (v2_prefetch<true> reads them back): each store instruction of the warp covers 512
// contiguous bytes, so the data crosses NVLink in full lines
__device__ __forceinline__ void store_sm32(uint8_t* rec, int lane, const LaneSplit& s) {
  uint4* p = reinterpret_cast<uint4*>(rec) + lane;
  p[0] = make_uint4(s.sm[0], s.sm[1], s.sm[2], s.sm[3]);
  p[32] = make_uint4(s.sm[4], s.sm[5], s.sm[6], s.sm[7]);
}

// NVSwitch multicast stores: one store to the multicast mapping of the symmetric buffer lands at the
// same offset in every rank's copy (this rank's included), so an all-gather leaves the GPU once
// instead of once per peer.  Values are moved as raw bits.
__device__ __forceinline__ void mc_st128(void* mc_addr, const uint4& v) {
  asm volatile("multimem.st.weak.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "f"(__uint_as_float(v.x)),
               "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w))
               : "memory");
}
__device__ __forceinline__ void mc_st32(void* mc_addr, uint32_t v) {
  asm volatile("multimem.st.weak.global.f32 [%0], %1;" ::"l"(mc_addr), "f"(__uint_as_float(v)) : "memory");
}
__device__ __forceinline__ void warp_copy16_mc(uint8_t* mc_dst, const uint8_t* src, int bytes, int lane) {
  const int nv = (bytes + 15) >> 4;
  for (int i = lane; i < nv; i += 32) mc_st128(mc_dst + 16 * i, reinterpret_cast<const uint4*>(src)[i]);
}

// Verbatim wire: a record is the chunk's 2048 bf16 bytes with no codec work, interleaved so that every
// store and load instruction of a warp covers 512 contiguous bytes (lane l's k-th 16 bytes sit at
// byte (k * 32 + l) * 16): remote stores leave the GPU as full lines.  Same slots, flags and parity
// protocol as the compressed records, no header words.  For links with bandwidth to spare, where the
// codec's instructions cost the kernels running beside the collective more than the bytes saved.
// Chosen per call; every rank must make the same choice.
__device__ __forceinline__ void store_verbatim(uint8_t* rec, int lane, const LaneIn& li) {
  uint4* p = reinterpret_cast<uint4*>(rec);
#pragma unroll
  for (int k = 0; k < 4; ++k)
    p[k * 32 + lane] = make_uint4(li.w[4 * k], li.w[4 * k + 1], li.w[4 * k + 2], li.w[4 * k + 3]);
}
__device__ __forceinline__ void load_verbatim(const uint8_t* rec, int lane, LaneIn& li) {
  const uint4* p = reinterpret_cast<const uint4*>(rec);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const uint4 v = __ldcg(p + k * 32 + lane);
    li.w[4 * k] = v.x; li.w[4 * k + 1] = v.y; li.w[4 * k + 2] = v.z; li.w[4 * k + 3] = v.w;
  }
}

struct AgArgs {
  const uint16_t* in;     // this rank's shard, n elements
  uint16_t* out;          // world * n elements
  uint8_t* const* peers;  // device array of world buffer pointers
  uint8_t* local;         // == peers[rank]
  uint8_t* mc;            // multicast mapping of the same buffer on all ranks, or null (per-peer stores)
  long long n;
  uint32_t seq;
  int push_ctas;
  int gc;                 // chunks per group in this call: 8, 16, 32 or 64
  int verbatim;           // 1: records are the chunks' bf16 bytes as they are (no codec work, 2048 B per chunk)
  unsigned long long timeout_ns;
  SymmLayout L;
};

// lane 0 waits for *fl >= want; every lane learns the outcome and is ordered after the flag
__device__ __forceinline__ bool warp_wait_flag(const uint32_t* fl, uint32_t want, unsigned long long limit_ns,
                                               int lane) {
  int ok = 1;
  if (lane == 0) ok = wait_ge(fl, want, limit_ns) ? 1 : 0;
  ok = __shfl_sync(FULL, ok, 0);
  __syncwarp();
  return ok != 0;
}

// WIRE: 0 = v2 records (bit planes), 1 = verbatim bf16, 2 = v2 records in nibble mode
// (three CTAs per SM by registers: two of them still fit beside a resident GEMM CTA and a
// reduce-scatter CTA, which is what the CTA budgets assume)
template <int WIRE>
__global__ void __launch_bounds__(256, 3) symm_all_gather_kernel(const AgArgs a) {
  // pushers: the record's tail (planes, escapes, raw exponents), its first 1024 bytes go out straight
  // from registers; decoders: escape staging.  8 KB, so that two collective CTAs fit beside a GEMM CTA.
  __shared__ __align__(16) uint8_t srec[8][V2_SLOT_BYTES / 2];
  __shared__ int s_ok;
  const SymmLayout& L = a.L;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int parity = a.seq & 1;
  const long long nc = (a.n + V2_CHUNK_ELEMS - 1) / V2_CHUNK_ELEMS;
  const int gc = a.gc;
  const long long ngroups = (nc + gc - 1) / gc;
  if (tid == 0) s_ok = 1;
  __syncthreads();

  if ((int)blockIdx.x < a.push_ctas) {
    // ---- pusher --------------------------------------------------------------------------------
    if (tid < L.world && tid != L.rank && a.seq >= 3) {
      if (!wait_ge(ctrl(a.local) + CW_DONE + tid, a.seq - 2, a.timeout_ns)) {
        set_status(a.local, 1, tid, -1);
        s_ok = 0;
      }
    }
    __syncthreads();
    if (!s_ok) return;
    const bool in_al = (reinterpret_cast<uintptr_t>(a.in) & 15) == 0;
    uint16_t* own = a.out + (long long)L.rank * a.n;
    const bool copy_own = own != a.in;
    const bool own_al = (reinterpret_cast<uintptr_t>(own) & 15) == 0;
    unsigned long long pushed = 0;
    uint32_t hint = 0xFFFFFFFFu;  // window of the previous chunk this warp encoded
    int hint_esc = 0;
    for (long long g = blockIdx.x; g < ngroups; g += a.push_ctas) {
      for (int it = 0; it < gc / 8; ++it) {
        const long long c = g * gc + it * 8 + warp;
        if (c >= nc) break;
        const long long e0 = c * V2_CHUNK_ELEMS + lane * 32;
        LaneIn li;
        load_lane(a.in + e0, a.n - e0, in_al, li);
        if (copy_own) store_lane(own + e0, a.n - e0, own_al, li);
        if constexpr (WIRE == 1) {
          if (!ZC_SLOT_OK(L, c, V2_SLOT_BYTES, a.local, L.rank)) continue;
          if (a.mc) {
            uint8_t* rec = slot_ptr(a.mc, L, parity, L.rank) + L.hdr_bytes + c * V2_SLOT_BYTES;
#pragma unroll
            for (int k = 0; k < 4; ++k)
              mc_st128(rec + 16 * (k * 32 + lane),
                       make_uint4(li.w[4 * k], li.w[4 * k + 1], li.w[4 * k + 2], li.w[4 * k + 3]));
          } else {
            for (int q = 0; q < L.world; ++q)
              if (q != L.rank)
                store_verbatim(slot_ptr(a.peers[q], L, parity, L.rank) + L.hdr_bytes + c * V2_SLOT_BYTES, lane, li);
          }
          if (lane == 0) pushed += (unsigned long long)V2_SLOT_BYTES * (L.world - 1);
          continue;
        }
        LaneSplit s;
        split_lane(li, s);
        const uint32_t hdr = WIRE == 2 ? v2_encode_chunk_nibble(s, srec[warp] - 1024, lane)
                                       : v2_encode_chunk_hint<false>(s, srec[warp] - 1024, lane, hint, hint_esc);
        __syncwarp();
        const int used = v2_record_bytes(hdr);
        if (!ZC_SLOT_OK(L, c, used, a.local, L.rank)) {
          __syncwarp();
          continue;
        }
        if (a.mc) {
          uint8_t* rec = slot_ptr(a.mc, L, parity, L.rank) + L.hdr_bytes + c * V2_SLOT_BYTES;
          mc_st128(rec + lane * 16, make_uint4(s.sm[0], s.sm[1], s.sm[2], s.sm[3]));
          mc_st128(rec + 512 + lane * 16, make_uint4(s.sm[4], s.sm[5], s.sm[6], s.sm[7]));
          warp_copy16_mc(rec + 1024, srec[warp], used - 1024, lane);
          if (lane == 0) mc_st32(reinterpret_cast<uint32_t*>(slot_ptr(a.mc, L, parity, L.rank)) + c, hdr);
        } else {
          for (int q = 0; q < L.world; ++q) {
            if (q == L.rank) continue;
            uint8_t* slot = slot_ptr(a.peers[q], L, parity, L.rank);
            uint8_t* rec = slot + L.hdr_bytes + c * V2_SLOT_BYTES;
            store_sm32(rec, lane, s);
            warp_copy16(rec + 1024, srec[warp], used - 1024, lane);
            if (lane == 0) reinterpret_cast<uint32_t*>(slot)[c] = hdr;
          }
        }
        if (lane == 0) pushed += (unsigned long long)(used + 4) * (L.world - 1);
        __syncwarp();
      }
      __threadfence_system();
      __syncthreads();
      if (tid < L.world && tid != L.rank) st_release_sys(flag_ptr(a.peers[tid], L, parity, L.rank, g), a.seq);
    }
    if (lane == 0 && pushed) atomicAdd(reinterpret_cast<unsigned long long*>(ctrl(a.local) + CW_WIRE_LO), pushed);
    return;
  }
  // ---- decoder: each warp takes items (group, source, slice of eight chunks) -----------------------
  const int dec_ctas = gridDim.x - a.push_ctas;
  const int subs = gc / 8;
  const long long items = ngroups * (L.world - 1) * subs;
  const long long wstride = (long long)dec_ctas * 8;
  volatile int* okp = &s_ok;
  uint8_t* esc = srec[warp];
  for (long long i = ((long long)blockIdx.x - a.push_ctas) * 8 + warp; i < items && *okp; i += wstride) {
    const int sub = (int)(i % subs);
    const long long gi = i / subs;
    int src = (int)(gi % (L.world - 1));
    const long long g = gi / (L.world - 1);
    if (src >= L.rank) ++src;
    const long long c0 = g * gc + sub * 8;
    if (c0 >= nc) continue;
    const int cnt = (int)min((long long)8, nc - c0);
    if (!warp_wait_flag(flag_ptr(a.local, L, parity, src, g), a.seq, a.timeout_ns, lane)) {
      if (lane == 0) {
        set_status(a.local, 2, src, g);
        *okp = 0;
      }
      break;
    }
    const uint8_t* slot = slot_ptr(a.local, L, parity, src);
    const uint8_t* recs = slot + L.hdr_bytes + c0 * V2_SLOT_BYTES;
    uint16_t* dst = a.out + (long long)src * a.n;
    const bool al = (reinterpret_cast<uintptr_t>(dst) & 15) == 0;
    if constexpr (WIRE == 1) {
      // a copy: all loads of the slice first, then the stores
      for (int k0 = 0; k0 < cnt; k0 += 2) {
        LaneIn v[2];
#pragma unroll
        for (int k = 0; k < 2; ++k)
          if (k0 + k < cnt) load_verbatim(recs + (long long)(k0 + k) * V2_SLOT_BYTES, lane, v[k]);
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          if (k0 + k >= cnt) continue;
          const long long e0 = (c0 + k0 + k) * V2_CHUNK_ELEMS + lane * 32;
          store_lane(dst + e0, a.n - e0, al, v[k]);
        }
      }
      continue;
    }
    // the item's eight headers in one load, then record k+1 in flight while record k is decoded
    // (two records ahead was measured and is slower: with eight warps per SM the decoder is bound by
    // its own instruction stream, and the extra registers cost a resident CTA)
    const uint32_t myhdr = lane < cnt ? __ldcg(reinterpret_cast<const uint32_t*>(slot) + c0 + lane) : 0u;
    RecRegs cur, nxt;
    v2_prefetch<true, WIRE == 2>(recs, __shfl_sync(FULL, myhdr, 0), lane, cur);
    for (int k = 0; k < cnt; ++k) {
      const uint32_t hn = __shfl_sync(FULL, myhdr, (k + 1) & 7);
      if (k + 1 < cnt) v2_prefetch<true, WIRE == 2>(recs + (long long)(k + 1) * V2_SLOT_BYTES, hn, lane, nxt);
      LaneSplit s;
      v2_decode_regs<WIRE == 2>(cur, esc, lane, s);
      LaneIn o;
      join_lane(s, o);
      const long long e0 = (c0 + k) * V2_CHUNK_ELEMS + lane * 32;
      store_lane(dst + e0, a.n - e0, al, o);
      cur = nxt;
    }
  }
  // last decoder CTA of this call tells every peer that this rank is done with the parity buffer
  __syncthreads();
  if (tid == 0) {
    uint32_t* c = ctrl(a.local);
    __threadfence();
    const uint32_t prev = atomicAdd(c + CW_COUNTER, 1u);
    if (prev + 1 == (uint32_t)dec_ctas) {
      c[CW_COUNTER] = 0;
      __threadfence_system();
      for (int q = 0; q < L.world; ++q)
        if (q != L.rank) st_release_sys(ctrl(a.peers[q]) + CW_DONE + L.rank, a.seq);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// reduce-scatter
// ---------------------------------------------------------------------------------------------
struct RsArgs {
  const void* in;         // [world, shard] fp32 or bf16
  void* out;              // [shard] fp32 or bf16
  uint16_t* residual;     // [world * shard] bf16 or null
  uint8_t* const* peers;
  uint8_t* local;
  long long shard;
  uint32_t seq;
  int push_ctas, in_fp32, out_fp32;
  int gc;                 // chunks per group in this call: 8, 16, 32 or 64
  int verbatim;           // 1: records are the chunks' bf16 bytes as they are
  float scale;
  unsigned long long timeout_ns;
  SymmLayout L;
};

__device__ __forceinline__ float bf16_bits_to_f(uint32_t b) { return __uint_as_float(b << 16); }
__device__ __forceinline__ uint32_t f_to_bf16_bits(float f) {
  return (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(f));
}

// load 32 values of one lane as fp32 (zero past `valid`)
__device__ __forceinline__ void load_lane_f32(const void* base, bool fp32, long long e0, long long valid, float (&v)[32]) {
  if (fp32) {
    const float* p = reinterpret_cast<const float*>(base) + e0;
    if (valid >= 32 && (reinterpret_cast<uintptr_t>(p) & 15) == 0) {
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float4 f = __ldg(reinterpret_cast<const float4*>(p) + k);
        v[4 * k] = f.x; v[4 * k + 1] = f.y; v[4 * k + 2] = f.z; v[4 * k + 3] = f.w;
      }
    } else {
#pragma unroll
      for (int k = 0; k < 32; ++k) v[k] = k < valid ? __ldg(p + k) : 0.f;
    }
  } else {
    LaneIn li;
    const uint16_t* p = reinterpret_cast<const uint16_t*>(base) + e0;
    load_lane(p, valid, (reinterpret_cast<uintptr_t>(p) & 15) == 0, li);
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      v[2 * k] = bf16_bits_to_f(li.w[k] & 0xFFFFu);
      v[2 * k + 1] = bf16_bits_to_f(li.w[k] >> 16);
    }
  }
}

// the 32 sums of one lane, times `scale`, to the fp32 or bf16 output
__device__ __forceinline__ void store_lane_scaled(void* out, int out_fp32, long long e0, long long valid, float scale,
                                                  const float (&acc)[32]) {
  if (out_fp32) {
    float* dst = reinterpret_cast<float*>(out) + e0;
    if (valid >= 32 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
      for (int j = 0; j < 8; ++j)
        reinterpret_cast<float4*>(dst)[j] = make_float4(acc[4 * j] * scale, acc[4 * j + 1] * scale,
                                                        acc[4 * j + 2] * scale, acc[4 * j + 3] * scale);
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (j < valid) dst[j] = acc[j] * scale;
    }
  } else {
    LaneIn o;
#pragma unroll
    for (int j = 0; j < 16; ++j)
      o.w[j] = f_to_bf16_bits(acc[2 * j] * scale) | (f_to_bf16_bits(acc[2 * j + 1] * scale) << 16);
    uint16_t* dst = reinterpret_cast<uint16_t*>(out) + e0;
    store_lane(dst, valid, (reinterpret_cast<uintptr_t>(dst) & 15) == 0, o);
  }
}

// WIRE: 0 = v2 records (bit planes), 1 = verbatim bf16, 2 = v2 records in nibble mode
template <int WIRE>
__global__ void __launch_bounds__(256, 2) symm_reduce_scatter_kernel(const RsArgs a) {
  // pushers: the record's tail (planes, escapes, raw exponents), its first 1024 bytes go out straight
  // from registers; decoders: escape staging.  8 KB, so that two collective CTAs fit beside a GEMM CTA.
  __shared__ __align__(16) uint8_t srec[8][V2_SLOT_BYTES / 2];
  __shared__ int s_ok;
  const SymmLayout& L = a.L;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int parity = a.seq & 1;
  const long long nc = (a.shard + V2_CHUNK_ELEMS - 1) / V2_CHUNK_ELEMS;
  const int gc = a.gc;
  const long long ngroups = (nc + gc - 1) / gc;
  if (tid == 0) s_ok = 1;
  __syncthreads();

  if ((int)blockIdx.x < a.push_ctas) {
    if (tid < L.world && tid != L.rank && a.seq >= 3) {
      if (!wait_ge(ctrl(a.local) + CW_DONE + tid, a.seq - 2, a.timeout_ns)) {
        set_status(a.local, 1, tid, -1);
        s_ok = 0;
      }
    }
    __syncthreads();
    if (!s_ok) return;
    unsigned long long pushed = 0;
    uint32_t hint = 0xFFFFFFFFu;
    int hint_esc = 0;
    // work item = (destination, group); destinations interleaved so all links are busy
    const long long items = ngroups * (L.world - 1);
    for (long long i = blockIdx.x; i < items; i += a.push_ctas) {
      const long long g = i / (L.world - 1);
      int q = (int)(i % (L.world - 1));
      q = (L.rank + 1 + q) % L.world;  // start with the next rank: spreads traffic over peers
      uint8_t* slot = slot_ptr(a.peers[q], L, parity, L.rank);
      for (int it = 0; it < gc / 8; ++it) {
        const long long c = g * gc + it * 8 + warp;
        if (c >= nc) break;
        const long long e0 = c * V2_CHUNK_ELEMS + lane * 32;
        const long long valid = a.shard - e0;
        LaneIn li;
        if (!a.in_fp32) {
          // bf16 rows go out as they are: no detour through fp32
          const uint16_t* ip = reinterpret_cast<const uint16_t*>(a.in) + (long long)q * a.shard + e0;
          load_lane(ip, valid, (reinterpret_cast<uintptr_t>(ip) & 15) == 0, li);
        } else {
          float v[32];
          load_lane_f32(a.in, 1, (long long)q * a.shard + e0, valid, v);
          if (a.residual) {
            uint16_t* rp = a.residual + (long long)q * a.shard + e0;
            LaneIn r;
            const bool ral = (reinterpret_cast<uintptr_t>(rp) & 15) == 0;
            load_lane(rp, valid, ral, r);
#pragma unroll
            for (int k = 0; k < 16; ++k) {
              const float x0 = v[2 * k] + bf16_bits_to_f(r.w[k] & 0xFFFFu);
              const float x1 = v[2 * k + 1] + bf16_bits_to_f(r.w[k] >> 16);
              const uint32_t b0 = f_to_bf16_bits(x0), b1 = f_to_bf16_bits(x1);
              li.w[k] = b0 | (b1 << 16);
              r.w[k] = f_to_bf16_bits(x0 - bf16_bits_to_f(b0)) | (f_to_bf16_bits(x1 - bf16_bits_to_f(b1)) << 16);
            }
            store_lane(rp, valid, ral, r);
          } else {
#pragma unroll
            for (int k = 0; k < 16; ++k) li.w[k] = f_to_bf16_bits(v[2 * k]) | (f_to_bf16_bits(v[2 * k + 1]) << 16);
          }
        }
        if constexpr (WIRE == 1) {
          if (!ZC_SLOT_OK(L, c, V2_SLOT_BYTES, a.local, q)) continue;
          store_verbatim(slot + L.hdr_bytes + c * V2_SLOT_BYTES, lane, li);
          if (lane == 0) pushed += (unsigned long long)V2_SLOT_BYTES;
          continue;
        }
        LaneSplit s;
        split_lane(li, s);
        const uint32_t hdr = WIRE == 2 ? v2_encode_chunk_nibble(s, srec[warp] - 1024, lane)
                                       : v2_encode_chunk_hint<false>(s, srec[warp] - 1024, lane, hint, hint_esc);
        __syncwarp();
        const int used = v2_record_bytes(hdr);
        if (!ZC_SLOT_OK(L, c, used, a.local, q)) {
          __syncwarp();
          continue;
        }
        store_sm32(slot + L.hdr_bytes + c * V2_SLOT_BYTES, lane, s);
        warp_copy16(slot + L.hdr_bytes + c * V2_SLOT_BYTES + 1024, srec[warp], used - 1024, lane);
        if (lane == 0) {
          reinterpret_cast<uint32_t*>(slot)[c] = hdr;
          pushed += (unsigned long long)(used + 4);
        }
        __syncwarp();
      }
      __threadfence_system();
      __syncthreads();
      if (tid == 0) st_release_sys(flag_ptr(a.peers[q], L, parity, L.rank, g), a.seq);
    }
    if (lane == 0 && pushed) atomicAdd(reinterpret_cast<unsigned long long*>(ctrl(a.local) + CW_WIRE_LO), pushed);
    return;
  }
  // ---- decoder + reduce: each warp takes items (group, slice of eight chunks) -----------------------
  const int dec_ctas = gridDim.x - a.push_ctas;
  const int subs = gc / 8;
  const long long items = ngroups * subs;
  const long long wstride = (long long)dec_ctas * 8;
  volatile int* okp = &s_ok;
  uint8_t* esc = srec[warp];
  const bool is_src = lane < L.world && lane != L.rank;   // lane l looks after source rank l
  const int p0 = L.rank == 0 ? 1 : 0;                     // first source in rank order
  for (long long i = ((long long)blockIdx.x - a.push_ctas) * 8 + warp; i < items && *okp; i += wstride) {
    const int sub = (int)(i % subs);
    const long long g = i / subs;
    const long long c0 = g * gc + sub * 8;
    if (c0 >= nc) continue;
    const int cnt = (int)min((long long)8, nc - c0);
    int ok = 1;
    if (is_src && !wait_ge(flag_ptr(a.local, L, parity, lane, g), a.seq, a.timeout_ns)) {
      set_status(a.local, 2, lane, g);
      ok = 0;
    }
    ok = __all_sync(FULL, ok);
    __syncwarp();
    if (!ok) {
      if (lane == 0) *okp = 0;
      break;
    }
    if constexpr (WIRE == 1) {
      for (int k = 0; k < cnt; ++k) {
        const long long c = c0 + k;
        const long long e0 = c * V2_CHUNK_ELEMS + lane * 32;
        const long long valid = a.shard - e0;
        // fixed order (this rank's own row, then the sources by rank): a deterministic sum
        float acc[32];
        load_lane_f32(a.in, a.in_fp32, (long long)L.rank * a.shard + e0, valid, acc);
        for (int p = 0; p < L.world; ++p) {
          if (p == L.rank) continue;
          LaneIn o;
          load_verbatim(slot_ptr(a.local, L, parity, p) + L.hdr_bytes + c * V2_SLOT_BYTES, lane, o);
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            acc[2 * j] += bf16_bits_to_f(o.w[j] & 0xFFFFu);
            acc[2 * j + 1] += bf16_bits_to_f(o.w[j] >> 16);
          }
        }
        if (valid > 0) store_lane_scaled(a.out, a.out_fp32, e0, valid, a.scale, acc);
      }
      continue;
    }
    const uint8_t* myslot = slot_ptr(a.local, L, parity, is_src ? lane : p0);
    uint32_t myhdr = is_src ? __ldcg(reinterpret_cast<const uint32_t*>(myslot) + c0) : 0u;
    RecRegs cur, nxt;
    v2_prefetch<true, WIRE == 2>(slot_ptr(a.local, L, parity, p0) + L.hdr_bytes + c0 * V2_SLOT_BYTES, __shfl_sync(FULL, myhdr, p0), lane,
                cur);
    for (int k = 0; k < cnt; ++k) {
      const long long c = c0 + k;
      const long long e0 = c * V2_CHUNK_ELEMS + lane * 32;
      const long long valid = a.shard - e0;
      const uint32_t nexthdr = (is_src && k + 1 < cnt) ? __ldcg(reinterpret_cast<const uint32_t*>(myslot) + c + 1) : 0u;
      // fixed order (this rank's own row, then the sources by rank): a deterministic sum
      float acc[32];
      load_lane_f32(a.in, a.in_fp32, (long long)L.rank * a.shard + e0, valid, acc);
      for (int p = 0; p < L.world; ++p) {
        if (p == L.rank) continue;
        // the record decoded after this one: the next source of this chunk, else the first source of the next
        int pn = p + 1;
        if (pn == L.rank) ++pn;
        if (pn < L.world) {
          v2_prefetch<true, WIRE == 2>(slot_ptr(a.local, L, parity, pn) + L.hdr_bytes + c * V2_SLOT_BYTES, __shfl_sync(FULL, myhdr, pn),
                      lane, nxt);
        } else if (k + 1 < cnt) {
          v2_prefetch<true, WIRE == 2>(slot_ptr(a.local, L, parity, p0) + L.hdr_bytes + (c + 1) * V2_SLOT_BYTES,
                      __shfl_sync(FULL, nexthdr, p0), lane, nxt);
        }
        LaneSplit s;
        v2_decode_regs<WIRE == 2>(cur, esc, lane, s);
        LaneIn o;
        join_lane(s, o);
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          acc[2 * j] += bf16_bits_to_f(o.w[j] & 0xFFFFu);
          acc[2 * j + 1] += bf16_bits_to_f(o.w[j] >> 16);
        }
        cur = nxt;
      }
      myhdr = nexthdr;
      if (valid <= 0) continue;
      store_lane_scaled(a.out, a.out_fp32, e0, valid, a.scale, acc);
    }
  }
  __syncthreads();
  if (tid == 0) {
    uint32_t* c = ctrl(a.local);
    __threadfence();
    const uint32_t prev = atomicAdd(c + CW_COUNTER, 1u);
    if (prev + 1 == (uint32_t)dec_ctas) {
      c[CW_COUNTER] = 0;
      __threadfence_system();
      for (int q = 0; q < L.world; ++q)
        if (q != L.rank) st_release_sys(ctrl(a.peers[q]) + CW_DONE + L.rank, a.seq);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// int8 all-gather: the arithmetic of the int8 hook (per-shard absmax scale = max(absmax/127, 1e-8),
// q = clamp(round(x / scale), -127, 127)) on the same staging protocol.  A chunk's record is its
// 1024 int8 values at the start of its slot (lane l's bytes 0..15 at 16 l, 16..31 at 512 + 16 l);
// the header word carries the source's scale, so the wire cost is 1028 bytes per 1024 elements.  Every rank, the source included, ends up with the
// dequantised values, so all ranks see identical parameters.
// ---------------------------------------------------------------------------------------------
constexpr int CW_ABSMAX = 70;  // bits of max|x| over the shard being gathered (set by absmax_bf16_kernel)

__global__ void __launch_bounds__(256) absmax_bf16_kernel(const uint16_t* __restrict__ x, long long n,
                                                          uint32_t* __restrict__ word) {
  uint32_t m = 0;  // |bf16| bit patterns order like the values
  const long long nv = ((reinterpret_cast<uintptr_t>(x) & 15) == 0) ? n / 8 : 0;
  for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < nv; i += (long long)gridDim.x * 256) {
    const uint4 v = __ldg(reinterpret_cast<const uint4*>(x) + i);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) m = max(m, max(w[k] & 0x7FFFu, (w[k] >> 16) & 0x7FFFu));
  }
  for (long long i = nv * 8 + (long long)blockIdx.x * 256 + threadIdx.x; i < n; i += (long long)gridDim.x * 256)
    m = max(m, (uint32_t)x[i] & 0x7FFFu);
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, s));
  if ((threadIdx.x & 31) == 0 && m) atomicMax(word, m << 16);  // fp32 bits of the bf16 magnitude
}

// one value -> its int8 byte; `dq` receives the value every rank will reconstruct
__device__ __forceinline__ uint32_t quant_byte(float x, float scale, float& dq) {
  const float r = fminf(fmaxf(rintf(x / scale), -127.f), 127.f);
  dq = r * scale;
  return (uint32_t)((int)r) & 0xFFu;
}

__global__ void __launch_bounds__(256) symm_all_gather_int8_kernel(const AgArgs a) {
  __shared__ int s_ok;
  const SymmLayout& L = a.L;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int parity = a.seq & 1;
  const long long nc = (a.n + V2_CHUNK_ELEMS - 1) / V2_CHUNK_ELEMS;
  const long long ngroups = (nc + GROUP_CHUNKS - 1) / GROUP_CHUNKS;
  if (tid == 0) s_ok = 1;
  __syncthreads();

  if ((int)blockIdx.x < a.push_ctas) {
    if (tid < L.world && tid != L.rank && a.seq >= 3) {
      if (!wait_ge(ctrl(a.local) + CW_DONE + tid, a.seq - 2, a.timeout_ns)) {
        set_status(a.local, 1, tid, -1);
        s_ok = 0;
      }
    }
    __syncthreads();
    if (!s_ok) return;
    const float absmax = __uint_as_float(ctrl(a.local)[CW_ABSMAX]);
    const float scale = fmaxf(absmax / 127.f, 1e-8f);
    const bool in_al = (reinterpret_cast<uintptr_t>(a.in) & 15) == 0;
    uint16_t* own = a.out + (long long)L.rank * a.n;
    const bool own_al = (reinterpret_cast<uintptr_t>(own) & 15) == 0;
    unsigned long long pushed = 0;
    for (long long g = blockIdx.x; g < ngroups; g += a.push_ctas) {
      for (int it = 0; it < GROUP_CHUNKS / 8; ++it) {
        const long long c = g * GROUP_CHUNKS + it * 8 + warp;
        if (c >= nc) break;
        const long long e0 = c * V2_CHUNK_ELEMS + lane * 32;
        LaneIn li, dq;
        load_lane(a.in + e0, a.n - e0, in_al, li);
        uint32_t qw[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          float d0, d1, d2, d3;
          const uint32_t b0 = quant_byte(bf16_bits_to_f(li.w[2 * k] & 0xFFFFu), scale, d0);
          const uint32_t b1 = quant_byte(bf16_bits_to_f(li.w[2 * k] >> 16), scale, d1);
          const uint32_t b2 = quant_byte(bf16_bits_to_f(li.w[2 * k + 1] & 0xFFFFu), scale, d2);
          const uint32_t b3 = quant_byte(bf16_bits_to_f(li.w[2 * k + 1] >> 16), scale, d3);
          qw[k] = b0 | (b1 << 8) | (b2 << 16) | (b3 << 24);
          dq.w[2 * k] = f_to_bf16_bits(d0) | (f_to_bf16_bits(d1) << 16);
          dq.w[2 * k + 1] = f_to_bf16_bits(d2) | (f_to_bf16_bits(d3) << 16);
        }
        store_lane(own + e0, a.n - e0, own_al, dq);  // the source keeps what the others will see
        const uint4 q0 = make_uint4(qw[0], qw[1], qw[2], qw[3]), q1 = make_uint4(qw[4], qw[5], qw[6], qw[7]);
        if (a.mc) {
          uint8_t* slot = slot_ptr(a.mc, L, parity, L.rank);
          uint8_t* dst = slot + L.hdr_bytes + c * V2_SLOT_BYTES + lane * 16;  // two 512-byte halves, as store_sm32
          mc_st128(dst, q0);
          mc_st128(dst + 512, q1);
          if (lane == 0) mc_st32(reinterpret_cast<uint32_t*>(slot) + c, __float_as_uint(scale));
        } else {
          for (int q = 0; q < L.world; ++q) {
            if (q == L.rank) continue;
            uint8_t* slot = slot_ptr(a.peers[q], L, parity, L.rank);
            uint4* dst = reinterpret_cast<uint4*>(slot + L.hdr_bytes + c * V2_SLOT_BYTES) + lane;
            dst[0] = q0;
            dst[32] = q1;
            if (lane == 0) reinterpret_cast<uint32_t*>(slot)[c] = __float_as_uint(scale);
          }
        }
        if (lane == 0) pushed += (unsigned long long)(V2_CHUNK_ELEMS + 4) * (L.world - 1);
      }
      __threadfence_system();
      __syncthreads();
      if (tid < L.world && tid != L.rank) st_release_sys(flag_ptr(a.peers[tid], L, parity, L.rank, g), a.seq);
    }
    if (lane == 0 && pushed) atomicAdd(reinterpret_cast<unsigned long long*>(ctrl(a.local) + CW_WIRE_LO), pushed);
    return;
  }
  const int dec_ctas = gridDim.x - a.push_ctas;
  const long long items = ngroups * (L.world - 1);
  for (long long i = (long long)blockIdx.x - a.push_ctas; i < items; i += dec_ctas) {
    const long long g = i / (L.world - 1);
    int src = (int)(i % (L.world - 1));
    if (src >= L.rank) ++src;
    uint32_t* fl = flag_ptr(a.local, L, parity, src, g);
    if (tid == 0 && !wait_ge(fl, a.seq, a.timeout_ns)) {
      set_status(a.local, 2, src, g);
      s_ok = 0;
    }
    __syncthreads();
    if (!s_ok) break;
    (void)ld_acquire_sys(fl);
    const uint8_t* slot = slot_ptr(a.local, L, parity, src);
    uint16_t* dst = a.out + (long long)src * a.n;
    const bool al = (reinterpret_cast<uintptr_t>(dst) & 15) == 0;
    for (int it = 0; it < GROUP_CHUNKS / 8; ++it) {
      const long long c = g * GROUP_CHUNKS + it * 8 + warp;
      if (c >= nc) break;
      const float scale = __uint_as_float(__ldcg(reinterpret_cast<const uint32_t*>(slot) + c));
      const uint4* rec = reinterpret_cast<const uint4*>(slot + L.hdr_bytes + c * V2_SLOT_BYTES) + lane;
      const uint4 q0 = __ldcg(rec), q1 = __ldcg(rec + 32);
      const uint32_t qw[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
      LaneIn o;
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float d0 = (float)(int8_t)(qw[k] & 0xFFu) * scale, d1 = (float)(int8_t)((qw[k] >> 8) & 0xFFu) * scale;
        const float d2 = (float)(int8_t)((qw[k] >> 16) & 0xFFu) * scale, d3 = (float)(int8_t)(qw[k] >> 24) * scale;
        o.w[2 * k] = f_to_bf16_bits(d0) | (f_to_bf16_bits(d1) << 16);
        o.w[2 * k + 1] = f_to_bf16_bits(d2) | (f_to_bf16_bits(d3) << 16);
      }
      const long long e0 = c * V2_CHUNK_ELEMS + lane * 32;
      store_lane(dst + e0, a.n - e0, al, o);
    }
  }
  __syncthreads();
  if (tid == 0) {
    uint32_t* c = ctrl(a.local);
    __threadfence();
    const uint32_t prev = atomicAdd(c + CW_COUNTER, 1u);
    if (prev + 1 == (uint32_t)dec_ctas) {
      c[CW_COUNTER] = 0;
      __threadfence_system();
      for (int q = 0; q < L.world; ++q)
        if (q != L.rank) st_release_sys(ctrl(a.peers[q]) + CW_DONE + L.rank, a.seq);
    }
  }
}

// Chunks per group for a message of `nc` chunks per source: the largest of 64, 32, 16, 8 that still
// gives every pusher CTA about two groups, subject to the flag area (one flag per 64 chunks of nc_max).
// Every rank must arrive at the same value, so it depends on the message and the device only
// (`push_ctas` is the SM count here, not the caller's CTA budget).
static int pick_group_chunks(long long nc, int push_ctas, int max_groups) {
  int gc = 64;
  while (gc > 8 && (nc + gc - 1) / gc < 2LL * push_ctas && (nc + gc / 2 - 1) / (gc / 2) <= max_groups) gc >>= 1;
  return gc;
}

static SymmLayout make_layout(int world, int rank, long long nc_max) {
  SymmLayout L;
  L.world = world;
  L.rank = rank;
  L.nc_max = nc_max;
  L.max_groups = (int)((nc_max + GROUP_CHUNKS - 1) / GROUP_CHUNKS);
  L.flag_bytes = align128(2LL * world * L.max_groups * 4);
  L.hdr_bytes = align128(nc_max * 4);
  L.slot_bytes = L.hdr_bytes + nc_max * V2_SLOT_BYTES;
  L.parity_bytes = (long long)world * L.slot_bytes;
  return L;
}

}  // namespace zc

extern "C" {

// bytes of symmetric memory a channel needs for messages of up to nc_max chunks per source
long long zc_symm_buffer_bytes(int world, long long nc_max) {
  const zc::SymmLayout L = zc::make_layout(world, 0, nc_max);
  return zc::CTRL_BYTES + L.flag_bytes + 2 * L.parity_bytes;
}

// in: n bf16 elements; out: world*n; peers: device array of `world` buffer pointers
// mc: multicast mapping of the symmetric buffer (NVSwitch), or null to push with per-peer stores
// wire: 0 = v2 records (bit planes, about 1.40 bytes per element), 1 = the bf16 bytes as they are,
// 2 = v2 records in nibble mode (about 1.50 bytes per element, roughly half the codec instructions)
int zc_symm_all_gather(const void* in, void* out, void* const* peers, void* local, void* mc, long long n, int rank,
                       int world, long long nc_max, unsigned seq, int push_ctas, int dec_ctas, double timeout_s,
                       int wire, cudaStream_t st) {
  ZC_NVTX_RANGE("zc_symm_all_gather");
  using namespace zc;
  const long long nc = (n + V2_CHUNK_ELEMS - 1) / V2_CHUNK_ELEMS;
  // push_ctas == 0 (decode what has already arrived) or dec_ctas == 0 (encode and push only) run one
  // half of the collective: the halves of different ranks can then be run one after the other on a
  // single GPU, pushers first, without any kernel waiting for another launch
  if (world < 2 || world > 64 || nc > nc_max || nc == 0 || push_ctas < 0 || dec_ctas < 0 || push_ctas + dec_ctas < 1)
    return ERR_BAD_ARG;
  AgArgs a;
  a.in = (const uint16_t*)in; a.out = (uint16_t*)out; a.peers = (uint8_t* const*)peers; a.local = (uint8_t*)local;
  a.mc = (uint8_t*)mc; a.n = n; a.seq = seq; a.verbatim = wire == 1;
  a.timeout_ns = (unsigned long long)(timeout_s * 1e9);
  a.L = make_layout(world, rank, nc_max);
  a.gc = pick_group_chunks(nc, sm_count(), a.L.max_groups);
  // no more CTAs than there is work: small messages pay for the launch, not for idle CTAs
  const long long ngroups = (nc + a.gc - 1) / a.gc;
  a.push_ctas = (int)std::min<long long>(push_ctas, ngroups);
  const long long dec_items = ngroups * (world - 1) * (a.gc / 8);
  const int dec = (int)std::min<long long>(dec_ctas, (dec_items + 7) / 8);
  if (wire == 1) symm_all_gather_kernel<1><<<a.push_ctas + dec, 256, 0, st>>>(a);
  else if (wire == 2) symm_all_gather_kernel<2><<<a.push_ctas + dec, 256, 0, st>>>(a);
  else symm_all_gather_kernel<0><<<a.push_ctas + dec, 256, 0, st>>>(a);
  return launch_status();
}

int zc_symm_reduce_scatter(const void* in, void* out, void* residual, void* const* peers, void* local,
                           long long shard, int rank, int world, long long nc_max, unsigned seq, int in_fp32,
                           int out_fp32, float scale, int push_ctas, int dec_ctas, double timeout_s,
                           int wire, cudaStream_t st) {
  ZC_NVTX_RANGE("zc_symm_reduce_scatter");
  using namespace zc;
  const long long nc = (shard + V2_CHUNK_ELEMS - 1) / V2_CHUNK_ELEMS;
  if (world < 2 || world > 32 || nc > nc_max || nc == 0 || push_ctas < 0 || dec_ctas < 0 || push_ctas + dec_ctas < 1)
    return ERR_BAD_ARG;
  RsArgs a;
  a.in = in; a.out = out; a.residual = (uint16_t*)residual; a.peers = (uint8_t* const*)peers;
  a.local = (uint8_t*)local; a.shard = shard; a.seq = seq; a.in_fp32 = in_fp32;
  a.out_fp32 = out_fp32; a.scale = scale; a.verbatim = wire == 1;
  a.timeout_ns = (unsigned long long)(timeout_s * 1e9);
  a.L = make_layout(world, rank, nc_max);
  // a pusher item is (destination, group): world - 1 times as many items as groups
  a.gc = pick_group_chunks(nc * (world - 1), sm_count(), a.L.max_groups * (world - 1));
  while (a.gc < 64 && (nc + a.gc - 1) / a.gc > a.L.max_groups) a.gc <<= 1;
  const long long ngroups = (nc + a.gc - 1) / a.gc;
  a.push_ctas = (int)std::min<long long>(push_ctas, ngroups * (world - 1));
  const long long dec_items = ngroups * (a.gc / 8);
  const int dec = (int)std::min<long long>(dec_ctas, (dec_items + 7) / 8);
  if (wire == 1) symm_reduce_scatter_kernel<1><<<a.push_ctas + dec, 256, 0, st>>>(a);
  else if (wire == 2) symm_reduce_scatter_kernel<2><<<a.push_ctas + dec, 256, 0, st>>>(a);
  else symm_reduce_scatter_kernel<0><<<a.push_ctas + dec, 256, 0, st>>>(a);
  return launch_status();
}

// int8 variant of zc_symm_all_gather: three stream-ordered operations (clear the absmax word,
// reduce max|x| over the shard, then the fused quantise/push/dequantise kernel)
int zc_symm_all_gather_int8(const void* in, void* out, void* const* peers, void* local, void* mc, long long n,
                            int rank, int world, long long nc_max, unsigned seq, int push_ctas, int dec_ctas,
                            double timeout_s, cudaStream_t st) {
  ZC_NVTX_RANGE("zc_symm_all_gather_int8");
  using namespace zc;
  const long long nc = (n + V2_CHUNK_ELEMS - 1) / V2_CHUNK_ELEMS;
  if (world < 2 || world > 64 || nc > nc_max || nc == 0 || push_ctas < 1 || dec_ctas < 1) return ERR_BAD_ARG;
  AgArgs a;
  a.in = (const uint16_t*)in; a.out = (uint16_t*)out; a.peers = (uint8_t* const*)peers; a.local = (uint8_t*)local;
  a.mc = (uint8_t*)mc; a.n = n; a.seq = seq; a.push_ctas = push_ctas; a.gc = GROUP_CHUNKS; a.verbatim = 0;
  a.timeout_ns = (unsigned long long)(timeout_s * 1e9);
  a.L = make_layout(world, rank, nc_max);
  uint32_t* word = reinterpret_cast<uint32_t*>(local) + CW_ABSMAX;
  cudaMemsetAsync(word, 0, sizeof(uint32_t), st);
  const int grid = (int)std::min<long long>((n / 8 + 255) / 256 + 1, (long long)sm_count() * 8);
  absmax_bf16_kernel<<<grid, 256, 0, st>>>((const uint16_t*)in, n, word);
  symm_all_gather_int8_kernel<<<push_ctas + dec_ctas, 256, 0, st>>>(a);
  return launch_status();
}

// 1 when this library was compiled with -DZC_DEBUG_BOUNDS
int zc_debug_bounds_build() {
#ifdef ZC_DEBUG_BOUNDS
  return 1;
#else
  return 0;
#endif
}

}  // extern "C"
