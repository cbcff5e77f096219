// Memory-bound training ops for sm_100a: RMSNorm (+ residual add) forward/backward, RoPE, SwiGLU
// forward/backward, cross-entropy with in-place gradient, int8 absmax quantise/dequantise and
// fused AdamW.  Every kernel moves 16-byte vectors, keeps fp32 math in registers and touches each
// HBM byte once per pass.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

#include "launch_util.h"

namespace zc {

constexpr unsigned FULLM = 0xffffffffu;

struct alignas(16) BF8 {
  __nv_bfloat162 v[4];
};

__device__ __forceinline__ void unpack8(const BF8& p, float (&f)[8]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(p.v[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ BF8 pack8(const float (&f)[8]) {
  BF8 p;
#pragma unroll
  for (int i = 0; i < 4; ++i) p.v[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return p;
}
__device__ __forceinline__ BF8 ld8(const __nv_bfloat16* p) { return *reinterpret_cast<const BF8*>(p); }
__device__ __forceinline__ void st8(__nv_bfloat16* p, const BF8& v) { *reinterpret_cast<BF8*>(p) = v; }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(FULLM, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(FULLM, v, o));
  return v;
}

// block-wide sum for up to 1024 threads; every thread gets the result
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : 0.f;
  return warp_sum(t);
}
__device__ __forceinline__ float block_max(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : -CUDART_INF_F;
  return warp_max(t);
}

// ---------------------------------------------------------------------------------------------
// RMSNorm.  One CTA (256 threads) per row, row cached in registers (cols <= 8192, cols % 8 == 0).
//   h = x (+ residual, rounded to bf16);  rstd = rsqrt(mean(h^2) + eps);  y = h * rstd * w
// ---------------------------------------------------------------------------------------------
constexpr int RN_THREADS = 256;
constexpr int RN_MAX_COLS = RN_THREADS * 4 * 8;  // MAXV (vectors of 8 per thread) is 1, 2 or 4

template <int MAXV>
__global__ void __launch_bounds__(RN_THREADS) rmsnorm_fwd_kernel(
    const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
    const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y, __nv_bfloat16* __restrict__ h_out,
    float* __restrict__ rstd_out, int cols, float eps) {
  __shared__ float red[32];
  const int64_t row = blockIdx.x;
  const int nvec = cols / 8;
  float h[MAXV][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int v = threadIdx.x + i * RN_THREADS;
    if (v < nvec) {
      unpack8(ld8(x + row * cols + v * 8), h[i]);
      if (res) {
        float r[8];
        unpack8(ld8(res + row * cols + v * 8), r);
#pragma unroll
        for (int j = 0; j < 8; ++j) h[i][j] += r[j];
        const BF8 hb = pack8(h[i]);
        st8(h_out + row * cols + v * 8, hb);
        unpack8(hb, h[i]);  // normalise the rounded sum, as the unfused op order would
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += h[i][j] * h[i][j];
    }
  }
  ss = block_sum(ss, red);
  const float rstd = rsqrtf(ss / (float)cols + eps);
  if (threadIdx.x == 0) rstd_out[row] = rstd;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int v = threadIdx.x + i * RN_THREADS;
    if (v < nvec) {
      float wv[8], o[8];
      unpack8(ld8(w + v * 8), wv);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = h[i][j] * rstd * wv[j];
      st8(y + row * cols + v * 8, pack8(o));
    }
  }
}

// The same forward with one WARP per row (cols <= NV * 256): no block-wide synchronisation, all of a
// row's loads issued before the first use, and the row kept packed (bf16) in registers between the
// sum of squares and the scaling.  One row per CTA leaves the kernel waiting on two barriers per row
// with a single load batch in flight (0.44 of the copy bandwidth); independent warps keep many rows'
// loads in flight per SM.
template <int NV>
__global__ void __launch_bounds__(128) rmsnorm_fwd_warp_kernel(
    const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
    const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y, __nv_bfloat16* __restrict__ h_out,
    float* __restrict__ rstd_out, int64_t rows, int cols, float eps) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int nvec = cols / 8;
  const __nv_bfloat16* xr = x + row * cols;
  BF8 hv[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int v = lane + 32 * i;
    if (v < nvec) hv[i] = ld8(xr + v * 8);
  }
  if (res) {
    const __nv_bfloat16* rr = res + row * cols;
    BF8 rv[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = lane + 32 * i;
      if (v < nvec) rv[i] = ld8(rr + v * 8);
    }
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = lane + 32 * i;
      if (v < nvec) {
        float a[8], b[8];
        unpack8(hv[i], a);
        unpack8(rv[i], b);
#pragma unroll
        for (int j = 0; j < 8; ++j) a[j] += b[j];
        hv[i] = pack8(a);  // the rounded sum is what gets normalised, as the unfused op order would
        st8(h_out + row * cols + v * 8, hv[i]);
      }
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    if (lane + 32 * i < nvec) {
      float a[8];
      unpack8(hv[i], a);
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += a[j] * a[j];
    }
  }
  ss = warp_sum(ss);
  const float rstd = rsqrtf(ss / (float)cols + eps);
  if (lane == 0) rstd_out[row] = rstd;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int v = lane + 32 * i;
    if (v < nvec) {
      float a[8], wv[8], o[8];
      unpack8(hv[i], a);
      unpack8(ld8(w + v * 8), wv);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = a[j] * rstd * wv[j];
      st8(y + row * cols + v * 8, pack8(o));
    }
  }
}

// dx = rstd * (g - xhat * mean(g * xhat)) (+ dh),  g = dy * w,  xhat = h * rstd
// dw = sum_rows dy * xhat: every CTA keeps partial sums in registers over its rows and writes them
// to its row of `partials` ([gridDim.x, cols] fp32), which rmsnorm_dw_reduce_kernel then sums
// (one fp32 atomic per column and CTA instead was 2.4 M atomics on 4096 addresses per call and
// took most of the kernel's time); with partials == nullptr the atomics into dw32 remain
template <int MAXV>
__global__ void __launch_bounds__(RN_THREADS) rmsnorm_bwd_kernel(
    const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ h,
    const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd_in,
    const __nv_bfloat16* __restrict__ dh, __nv_bfloat16* __restrict__ dx, float* __restrict__ dw32,
    float* __restrict__ partials, int64_t rows, int cols) {
  __shared__ float red[32];
  const int nvec = cols / 8;
  float wv[MAXV][8], dwacc[MAXV][8];
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int v = threadIdx.x + i * RN_THREADS;
#pragma unroll
    for (int j = 0; j < 8; ++j) dwacc[i][j] = 0.f;
    if (v < nvec) unpack8(ld8(w + v * 8), wv[i]);
  }
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const float rstd = rstd_in[row];
    float g[MAXV][8], xh[MAXV][8];
    BF8 eh[MAXV];  // the residual-path gradient, fetched with the other operands: one memory round trip per row
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int v = threadIdx.x + i * RN_THREADS;
      if (v < nvec) {
        float d[8];
        unpack8(ld8(dy + row * cols + v * 8), d);
        unpack8(ld8(h + row * cols + v * 8), xh[i]);
        if (dh) eh[i] = ld8(dh + row * cols + v * 8);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[i][j] *= rstd;
          g[i][j] = d[j] * wv[i][j];
          dot += g[i][j] * xh[i][j];
          dwacc[i][j] += d[j] * xh[i][j];
        }
      }
    }
    dot = block_sum(dot, red) / (float)cols;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int v = threadIdx.x + i * RN_THREADS;
      if (v < nvec) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rstd * (g[i][j] - xh[i][j] * dot);
        if (dh) {
          float e[8];
          unpack8(eh[i], e);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += e[j];
        }
        st8(dx + row * cols + v * 8, pack8(o));
      }
    }
  }
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int v = threadIdx.x + i * RN_THREADS;
    if (v < nvec) {
      if (partials) {
        float4* dst = reinterpret_cast<float4*>(partials + (int64_t)blockIdx.x * cols + v * 8);
        dst[0] = make_float4(dwacc[i][0], dwacc[i][1], dwacc[i][2], dwacc[i][3]);
        dst[1] = make_float4(dwacc[i][4], dwacc[i][5], dwacc[i][6], dwacc[i][7]);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) atomicAdd(dw32 + v * 8 + j, dwacc[i][j]);
      }
    }
  }
}

// dw[c] = sum over the CTAs' partial rows; block (32, 32): 32 float4 columns x 32 row groups
__global__ void __launch_bounds__(1024) rmsnorm_dw_reduce_kernel(const float* __restrict__ partials, int nblocks,
                                                                int cols, float* __restrict__ dw) {
  __shared__ float4 acc[32][32];
  const int c4 = blockIdx.x * 32 + threadIdx.x;  // float4 column
  float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
  if (c4 * 4 < cols) {
    for (int r = threadIdx.y; r < nblocks; r += 32) {
      const float4 v = __ldg(reinterpret_cast<const float4*>(partials + (int64_t)r * cols) + c4);
      s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
    }
  }
  acc[threadIdx.y][threadIdx.x] = s;
  __syncthreads();
  if (threadIdx.y == 0 && c4 * 4 < cols) {
#pragma unroll
    for (int k = 1; k < 32; ++k) {
      const float4 v = acc[k][threadIdx.x];
      s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
    }
    reinterpret_cast<float4*>(dw)[c4] = s;
  }
}

// ---------------------------------------------------------------------------------------------
// RoPE in place on the first n_rot heads of a packed [T, total_heads * D] tensor
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) rope_kernel(__nv_bfloat16* __restrict__ qkv, const float* __restrict__ cosT,
                                                   const float* __restrict__ sinT, int64_t T, int S, int n_rot,
                                                   int total_heads, int D, float sign) {
  const int vph = D / 16;  // 8-element vectors per half head
  const int64_t total = T * n_rot * vph;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int v = (int)(idx % vph);
    const int hd = (int)((idx / vph) % n_rot);
    const int64_t t = idx / ((int64_t)vph * n_rot);
    const int pos = (int)(t % S);
    __nv_bfloat16* p = qkv + (t * total_heads + hd) * D + v * 8;
    float a[8], b[8], oa[8], ob[8];
    unpack8(ld8(p), a);
    unpack8(ld8(p + D / 2), b);
    const float4* c4 = reinterpret_cast<const float4*>(cosT + (int64_t)pos * (D / 2) + v * 8);
    const float4* s4 = reinterpret_cast<const float4*>(sinT + (int64_t)pos * (D / 2) + v * 8);
    const float4 c0 = c4[0], c1 = c4[1], s0 = s4[0], s1 = s4[1];
    const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    const float s[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float sj = s[j] * sign;
      oa[j] = a[j] * c[j] - b[j] * sj;
      ob[j] = b[j] * c[j] + a[j] * sj;
    }
    st8(p, pack8(oa));
    st8(p + D / 2, pack8(ob));
  }
}

// ---------------------------------------------------------------------------------------------
// SwiGLU on packed [T, 2F] = [gate | up]
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu,
                                                         __nv_bfloat16* __restrict__ out, int64_t T, int F) {
  const int vpr = F / 8;
  const int64_t total = T * vpr;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = idx / vpr;
    const int v = (int)(idx % vpr);
    float g[8], u[8], o[8];
    unpack8(ld8(gu + t * 2 * F + v * 8), g);
    unpack8(ld8(gu + t * 2 * F + F + v * 8), u);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = g[j] / (1.f + __expf(-g[j])) * u[j];
    st8(out + t * F + v * 8, pack8(o));
  }
}

__global__ void __launch_bounds__(256) swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ gu,
                                                         const __nv_bfloat16* __restrict__ dy,
                                                         __nv_bfloat16* __restrict__ dgu, int64_t T, int F) {
  const int vpr = F / 8;
  const int64_t total = T * vpr;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = idx / vpr;
    const int v = (int)(idx % vpr);
    float g[8], u[8], d[8], dg[8], du[8];
    unpack8(ld8(gu + t * 2 * F + v * 8), g);
    unpack8(ld8(gu + t * 2 * F + F + v * 8), u);
    unpack8(ld8(dy + t * F + v * 8), d);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float s = 1.f / (1.f + __expf(-g[j]));
      dg[j] = d[j] * u[j] * s * (1.f + g[j] * (1.f - s));
      du[j] = d[j] * g[j] * s;
    }
    st8(dgu + t * 2 * F + v * 8, pack8(dg));
    st8(dgu + t * 2 * F + F + v * 8, pack8(du));
  }
}

// ---------------------------------------------------------------------------------------------
// Cross-entropy: one CTA per row; pass 1 online max / sum-exp, pass 2 writes the gradient over the
// logits.  row_loss = lse - logit[label];  grad = (softmax - onehot) * inv_count
// Rows are `ld` elements apart (ld >= V; ld > V for a vocabulary that is not a multiple of 8, whose
// logits the GEMM writes into rows padded to an aligned stride); the pad columns come out as zeros.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(1024) ce_kernel(__nv_bfloat16* __restrict__ logits,
                                                  const int64_t* __restrict__ labels,
                                                  float* __restrict__ row_loss, const float* __restrict__ inv_count,
                                                  int V, int64_t ld, int ignore_index) {
  __shared__ float red[32];
  const int64_t row = blockIdx.x;
  __nv_bfloat16* lr = logits + row * ld;
  const int64_t label = labels[row];
  // whole 8-element vectors when the row starts on 16 bytes; the last V % 8 columns one by one
  const int nvec = ((ld % 8 == 0) && ((reinterpret_cast<uintptr_t>(logits) & 15) == 0)) ? V / 8 : 0;
  const int tail0 = nvec * 8;
  const __nv_bfloat16 zero = __float2bfloat16(0.f);
  if (label == ignore_index) {
    BF8 z;
#pragma unroll
    for (int i = 0; i < 4; ++i) z.v[i] = __floats2bfloat162_rn(0.f, 0.f);
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) st8(lr + v * 8, z);
    for (int64_t i = tail0 + threadIdx.x; i < ld; i += blockDim.x) lr[i] = zero;
    if (threadIdx.x == 0) row_loss[row] = 0.f;
    return;
  }
  float m = -CUDART_INF_F, s = 0.f;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    float f[8];
    unpack8(ld8(lr + v * 8), f);
    float lm = f[0];
#pragma unroll
    for (int j = 1; j < 8; ++j) lm = fmaxf(lm, f[j]);
    if (lm > m) { s *= __expf(m - lm); m = lm; }
#pragma unroll
    for (int j = 0; j < 8; ++j) s += __expf(f[j] - m);
  }
  for (int i = tail0 + threadIdx.x; i < V; i += blockDim.x) {
    const float f = __bfloat162float(lr[i]);
    if (f > m) { s *= __expf(m - f); m = f; }
    s += __expf(f - m);
  }
  const float gm = block_max(m, red);
  s = (m == -CUDART_INF_F) ? 0.f : s * __expf(m - gm);
  const float gs = block_sum(s, red);
  const float lse = gm + __logf(gs);
  const float scale = inv_count[0];
  const float picked = __bfloat162float(lr[label]);
  __syncthreads();  // everyone has read lr[label] before it is overwritten
  if (threadIdx.x == 0) row_loss[row] = lse - picked;
  const float inv_s = 1.f / gs;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    float f[8];
    unpack8(ld8(lr + v * 8), f);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float p = __expf(f[j] - gm) * inv_s;
      if (v * 8 + j == label) p -= 1.f;
      f[j] = p * scale;
    }
    st8(lr + v * 8, pack8(f));
  }
  for (int64_t i = tail0 + threadIdx.x; i < ld; i += blockDim.x) {
    if (i < V) {
      float p = __expf(__bfloat162float(lr[i]) - gm) * inv_s;
      if (i == label) p -= 1.f;
      lr[i] = __float2bfloat16(p * scale);
    } else {
      lr[i] = zero;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// int8 absmax quantisation.  Packed buffer: word0 = fp32 scale, word1 = absmax bits (scratch),
// bytes [16, 16+n) = int8 payload.
// ---------------------------------------------------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16(v); }
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f<__half>(float v) { return __float2half(v); }

template <typename T>
__global__ void __launch_bounds__(256) absmax_kernel(const T* __restrict__ x, int64_t n, uint32_t* __restrict__ hdr) {
  float m = 0.f;
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < n; i += (int64_t)gridDim.x * 256)
    m = fmaxf(m, fabsf(to_f<T>(x[i])));
  m = warp_max(m);
  __shared__ float red[8];
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < 8; ++i) m = fmaxf(m, red[i]);
    atomicMax(hdr + 1, __float_as_uint(m));  // non-negative floats order like their bit patterns
  }
}

template <typename T>
__global__ void __launch_bounds__(256) quant_kernel(const T* __restrict__ x, int64_t n, uint8_t* __restrict__ out) {
  const float absmax = __uint_as_float(reinterpret_cast<const uint32_t*>(out)[1]);
  const float scale = fmaxf(absmax / 127.f, 1e-8f);
  if (blockIdx.x == 0 && threadIdx.x == 0) reinterpret_cast<float*>(out)[0] = scale;
  int8_t* q = reinterpret_cast<int8_t*>(out + 16);
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < n; i += (int64_t)gridDim.x * 256) {
    const float r = rintf(to_f<T>(x[i]) / scale);
    q[i] = (int8_t)fminf(fmaxf(r, -127.f), 127.f);
  }
}

template <typename T>
__global__ void __launch_bounds__(256) dequant_kernel(const uint8_t* __restrict__ gathered, int64_t stride,
                                                      int world, int64_t n, T* __restrict__ out) {
  const int64_t total = (int64_t)world * n;
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < total; i += (int64_t)gridDim.x * 256) {
    const int r = (int)(i / n);
    const int64_t k = i - (int64_t)r * n;
    const uint8_t* slot = gathered + r * stride;
    const float scale = reinterpret_cast<const float*>(slot)[0];
    out[i] = from_f<T>((float)reinterpret_cast<const int8_t*>(slot + 16)[k] * scale);
  }
}

// ---------------------------------------------------------------------------------------------
// AdamW (decoupled weight decay), one launch per shard
// ---------------------------------------------------------------------------------------------
template <typename TP, typename TG, typename TS>
__global__ void __launch_bounds__(256) adamw_kernel(TP* __restrict__ p, TG* __restrict__ g, TS* __restrict__ m,
                                                    TS* __restrict__ v, int64_t n, float lr, float b1, float b2,
                                                    float eps, float wd, float bc1, float rsqrt_bc2, int zero_grad, const int* __restrict__ guard) {
  if (guard && *guard) return;
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < n; i += (int64_t)gridDim.x * 256) {
    const float gf = to_f<TG>(g[i]);
    float pf = to_f<TP>(p[i]);
    float mf = to_f<TS>(m[i]) * b1 + (1.f - b1) * gf;
    float vf = to_f<TS>(v[i]) * b2 + (1.f - b2) * gf * gf;
    pf *= 1.f - lr * wd;
    const float denom = sqrtf(vf) * rsqrt_bc2 + eps;
    pf -= (lr / bc1) * mf / denom;
    p[i] = from_f<TP>(pf);
    m[i] = from_f<TS>(mf);
    v[i] = from_f<TS>(vf);
    if (zero_grad) g[i] = from_f<TG>(0.f);
  }
}

// eight elements per thread, 16-byte accesses (pointers 16-byte aligned, n % 8 == 0)
template <typename T> __device__ __forceinline__ void load8(const T* p, float (&f)[8]);
template <> __device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&f)[8]) {
  unpack8(ld8(p), f);
}
template <> __device__ __forceinline__ void load8<float>(const float* p, float (&f)[8]) {
  const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}
template <typename T> __device__ __forceinline__ void store8(T* p, const float (&f)[8]);
template <> __device__ __forceinline__ void store8<__nv_bfloat16>(__nv_bfloat16* p, const float (&f)[8]) {
  st8(p, pack8(f));
}
template <> __device__ __forceinline__ void store8<float>(float* p, const float (&f)[8]) {
  reinterpret_cast<float4*>(p)[0] = make_float4(f[0], f[1], f[2], f[3]);
  reinterpret_cast<float4*>(p)[1] = make_float4(f[4], f[5], f[6], f[7]);
}

template <typename TP, typename TG, typename TS>
__global__ void __launch_bounds__(256) adamw_vec_kernel(TP* __restrict__ p, TG* __restrict__ g, TS* __restrict__ m,
                                                        TS* __restrict__ v, int64_t nvec, float lr, float b1, float b2,
                                                        float eps, float wd, float bc1, float rsqrt_bc2,
                                                        int zero_grad, const int* __restrict__ guard) {
  if (guard && *guard) return;  // a collective of this step gave up: leave parameters and moments alone
  const float decay = 1.f - lr * wd, step = lr / bc1;
  auto update = [&](float (&pf)[8], const float (&gf)[8], float (&mf)[8], float (&vf)[8]) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      mf[j] = mf[j] * b1 + (1.f - b1) * gf[j];
      vf[j] = vf[j] * b2 + (1.f - b2) * gf[j] * gf[j];
      pf[j] = pf[j] * decay - step * mf[j] / (sqrtf(vf[j]) * rsqrt_bc2 + eps);
    }
  };
  const float z[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  const int64_t stride = (int64_t)gridDim.x * 256;
  int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
  // two vectors per thread and trip: eight 16-byte loads in flight before the first use
  for (; i + stride < nvec; i += 2 * stride) {
    const int64_t k = i + stride;
    float pf[8], gf[8], mf[8], vf[8], pf2[8], gf2[8], mf2[8], vf2[8];
    load8<TP>(p + i * 8, pf);
    load8<TG>(g + i * 8, gf);
    load8<TS>(m + i * 8, mf);
    load8<TS>(v + i * 8, vf);
    load8<TP>(p + k * 8, pf2);
    load8<TG>(g + k * 8, gf2);
    load8<TS>(m + k * 8, mf2);
    load8<TS>(v + k * 8, vf2);
    update(pf, gf, mf, vf);
    update(pf2, gf2, mf2, vf2);
    store8<TP>(p + i * 8, pf);
    store8<TS>(m + i * 8, mf);
    store8<TS>(v + i * 8, vf);
    store8<TP>(p + k * 8, pf2);
    store8<TS>(m + k * 8, mf2);
    store8<TS>(v + k * 8, vf2);
    if (zero_grad) {
      store8<TG>(g + i * 8, z);
      store8<TG>(g + k * 8, z);
    }
  }
  for (; i < nvec; i += stride) {
    float pf[8], gf[8], mf[8], vf[8];
    load8<TP>(p + i * 8, pf);
    load8<TG>(g + i * 8, gf);
    load8<TS>(m + i * 8, mf);
    load8<TS>(v + i * 8, vf);
    update(pf, gf, mf, vf);
    store8<TP>(p + i * 8, pf);
    store8<TS>(m + i * 8, mf);
    store8<TS>(v + i * 8, vf);
    if (zero_grad) store8<TG>(g + i * 8, z);
  }
}

template <typename TP, typename TG, typename TS>
int adamw_launch(void* p, void* g, void* m, void* v, int64_t n, float lr, float b1, float b2, float eps, float wd,
                 float bc1, float rs, int zg, const int* guard, cudaStream_t st) {
  const bool vec = (n % 8 == 0) && (((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(g) |
                                      reinterpret_cast<uintptr_t>(m) | reinterpret_cast<uintptr_t>(v)) & 15) == 0);
  if (vec) {
    const int64_t nvec = n / 8;
    const int grid = (int)std::min<int64_t>((nvec + 255) / 256, (int64_t)sm_count() * 8);
    adamw_vec_kernel<TP, TG, TS><<<grid, 256, 0, st>>>((TP*)p, (TG*)g, (TS*)m, (TS*)v, nvec, lr, b1, b2, eps, wd,
                                                        bc1, rs, zg, guard);
  } else {
    const int grid = (int)std::min<int64_t>((n + 255) / 256, (int64_t)sm_count() * 16);
    adamw_kernel<TP, TG, TS><<<grid, 256, 0, st>>>((TP*)p, (TG*)g, (TS*)m, (TS*)v, n, lr, b1, b2, eps, wd, bc1, rs,
                                                    zg, guard);
  }
  return launch_status();
}

template <typename TP, typename TG>
int adamw_dispatch_s(void* p, void* g, void* m, void* v, int64_t n, int sdt, float lr, float b1, float b2, float eps,
                     float wd, float bc1, float bc2, int zg, const int* guard, cudaStream_t st) {
  const float rs = 1.f / sqrtf(bc2);
  if (sdt == 0) return adamw_launch<TP, TG, __nv_bfloat16>(p, g, m, v, n, lr, b1, b2, eps, wd, bc1, rs, zg, guard, st);
  if (sdt == 1) return adamw_launch<TP, TG, float>(p, g, m, v, n, lr, b1, b2, eps, wd, bc1, rs, zg, guard, st);
  return ERR_UNSUPPORTED;
}

}  // namespace zc

extern "C" {

using zc::ERR_BAD_ARG;
using zc::ERR_UNSUPPORTED;
typedef __nv_bfloat16 bf16;

int zc_rmsnorm_fwd(const void* x, const void* res, const void* w, void* y, void* h_out, float* rstd, int64_t rows,
                   int cols, float eps, cudaStream_t st) {
  if (cols % 8 || cols > zc::RN_MAX_COLS) return ERR_UNSUPPORTED;
  if (rows == 0) return 0;
  const int nvec = cols / 8;
  if (nvec <= 32 * 20) {  // one warp per row (wider rows do not fit a warp's registers)
    const unsigned grid = (unsigned)((rows + 3) / 4);
#define ZC_RN_FWDW(V)                                                                                             \
  zc::rmsnorm_fwd_warp_kernel<V><<<grid, 128, 0, st>>>((const bf16*)x, (const bf16*)res, (const bf16*)w, (bf16*)y, \
                                                       (bf16*)h_out, rstd, rows, cols, eps)
    if (nvec <= 32 * 4) ZC_RN_FWDW(4);
    else if (nvec <= 32 * 16) ZC_RN_FWDW(16);
    else ZC_RN_FWDW(20);
#undef ZC_RN_FWDW
    return zc::launch_status();
  }
#define ZC_RN_FWD(V)                                                                                              \
  zc::rmsnorm_fwd_kernel<V><<<(unsigned)rows, zc::RN_THREADS, 0, st>>>((const bf16*)x, (const bf16*)res,          \
                                                                       (const bf16*)w, (bf16*)y, (bf16*)h_out,    \
                                                                       rstd, cols, eps)
  if (nvec <= zc::RN_THREADS) ZC_RN_FWD(1);
  else if (nvec <= 2 * zc::RN_THREADS) ZC_RN_FWD(2);
  else ZC_RN_FWD(4);
#undef ZC_RN_FWD
  return zc::launch_status();
}

// CTAs the backward launches for `rows` rows: the number of rows `partials` must have
int zc_rmsnorm_bwd_ctas(int64_t rows) { return (int)std::min<int64_t>(rows, (int64_t)zc::sm_count() * 4); }

// dw32: [cols] fp32.  With partials ([zc_rmsnorm_bwd_ctas(rows), cols] fp32) it is overwritten with
// the column sums; with partials == nullptr it must be zero on entry and is accumulated with atomics.
int zc_rmsnorm_bwd(const void* dy, const void* h, const void* w, const float* rstd, const void* dh, void* dx,
                   float* dw32, float* partials, int64_t rows, int cols, cudaStream_t st) {
  if (cols % 8 || cols > zc::RN_MAX_COLS) return ERR_UNSUPPORTED;
  if (rows == 0) return 0;
  const int grid = zc_rmsnorm_bwd_ctas(rows);
  const int nvec = cols / 8;
#define ZC_RN_BWD(V)                                                                                             \
  zc::rmsnorm_bwd_kernel<V><<<grid, zc::RN_THREADS, 0, st>>>((const bf16*)dy, (const bf16*)h, (const bf16*)w,    \
                                                             rstd, (const bf16*)dh, (bf16*)dx, dw32, partials,   \
                                                             rows, cols)
  if (nvec <= zc::RN_THREADS) ZC_RN_BWD(1);
  else if (nvec <= 2 * zc::RN_THREADS) ZC_RN_BWD(2);
  else ZC_RN_BWD(4);
#undef ZC_RN_BWD
  if (partials)
    zc::rmsnorm_dw_reduce_kernel<<<(cols / 4 + 31) / 32, dim3(32, 32), 0, st>>>(partials, grid, cols, dw32);
  return zc::launch_status();
}

int zc_rope_inplace(void* qkv, const float* cosT, const float* sinT, int64_t T, int S, int n_rot, int total_heads,
                    int D, float sign, cudaStream_t st) {
  if (D % 16 || n_rot > total_heads) return ERR_UNSUPPORTED;
  const int64_t total = T * n_rot * (D / 16);
  if (total == 0) return 0;
  const int grid = (int)std::min<int64_t>((total + 255) / 256, (int64_t)zc::sm_count() * 16);
  zc::rope_kernel<<<grid, 256, 0, st>>>((bf16*)qkv, cosT, sinT, T, S, n_rot, total_heads, D, sign);
  return zc::launch_status();
}

int zc_swiglu_fwd(const void* gu, void* out, int64_t T, int F, cudaStream_t st) {
  if (F % 8) return ERR_UNSUPPORTED;
  const int64_t total = T * (F / 8);
  if (total == 0) return 0;
  const int grid = (int)std::min<int64_t>((total + 255) / 256, (int64_t)zc::sm_count() * 16);
  zc::swiglu_fwd_kernel<<<grid, 256, 0, st>>>((const bf16*)gu, (bf16*)out, T, F);
  return zc::launch_status();
}

int zc_swiglu_bwd(const void* gu, const void* dy, void* dgu, int64_t T, int F, cudaStream_t st) {
  if (F % 8) return ERR_UNSUPPORTED;
  const int64_t total = T * (F / 8);
  if (total == 0) return 0;
  const int grid = (int)std::min<int64_t>((total + 255) / 256, (int64_t)zc::sm_count() * 16);
  zc::swiglu_bwd_kernel<<<grid, 256, 0, st>>>((const bf16*)gu, (const bf16*)dy, (bf16*)dgu, T, F);
  return zc::launch_status();
}

int zc_ce_fwd_bwd_ld(void* logits, const int64_t* labels, float* row_loss, const float* inv_count, int64_t T, int V,
                     int64_t ld, int ignore_index, cudaStream_t st) {
  if (T == 0) return 0;
  if (V <= 0 || ld < V) return ERR_BAD_ARG;
  zc::ce_kernel<<<(unsigned)T, 1024, 0, st>>>((bf16*)logits, labels, row_loss, inv_count, V, ld, ignore_index);
  return zc::launch_status();
}

int zc_ce_fwd_bwd(void* logits, const int64_t* labels, float* row_loss, const float* inv_count, int64_t T, int V,
                  int ignore_index, cudaStream_t st) {
  return zc_ce_fwd_bwd_ld(logits, labels, row_loss, inv_count, T, V, V, ignore_index, st);
}

int zc_quant_int8(const void* x, int64_t n, int dtype, void* out, cudaStream_t st) {
  cudaMemsetAsync(out, 0, 16, st);
  if (n == 0) return zc::launch_status();
  const int grid = (int)std::min<int64_t>((n + 255) / 256, (int64_t)zc::sm_count() * 16);
  if (dtype == 0) {
    zc::absmax_kernel<bf16><<<grid, 256, 0, st>>>((const bf16*)x, n, (uint32_t*)out);
    zc::quant_kernel<bf16><<<grid, 256, 0, st>>>((const bf16*)x, n, (uint8_t*)out);
  } else if (dtype == 1) {
    zc::absmax_kernel<float><<<grid, 256, 0, st>>>((const float*)x, n, (uint32_t*)out);
    zc::quant_kernel<float><<<grid, 256, 0, st>>>((const float*)x, n, (uint8_t*)out);
  } else if (dtype == 2) {
    zc::absmax_kernel<__half><<<grid, 256, 0, st>>>((const __half*)x, n, (uint32_t*)out);
    zc::quant_kernel<__half><<<grid, 256, 0, st>>>((const __half*)x, n, (uint8_t*)out);
  } else {
    return ERR_UNSUPPORTED;
  }
  return zc::launch_status();
}

int zc_dequant_int8(const void* gathered, int64_t stride, int world, int64_t n, int dtype, void* out,
                    cudaStream_t st) {
  const int64_t total = (int64_t)world * n;
  if (total == 0) return 0;
  const int grid = (int)std::min<int64_t>((total + 255) / 256, (int64_t)zc::sm_count() * 16);
  if (dtype == 0)
    zc::dequant_kernel<bf16><<<grid, 256, 0, st>>>((const uint8_t*)gathered, stride, world, n, (bf16*)out);
  else if (dtype == 1)
    zc::dequant_kernel<float><<<grid, 256, 0, st>>>((const uint8_t*)gathered, stride, world, n, (float*)out);
  else if (dtype == 2)
    zc::dequant_kernel<__half><<<grid, 256, 0, st>>>((const uint8_t*)gathered, stride, world, n, (__half*)out);
  else
    return ERR_UNSUPPORTED;
  return zc::launch_status();
}

// The library's health word of the current device (0 = healthy): set by a fused collective whose
// bounded wait ran out, read on the device by zc_adamw_guarded, read and cleared on the host by
// zc_health_read_and_clear.  Allocated on first use.
int* zc_health_word() {
  static int* words[64] = {nullptr};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return nullptr;
  if (!words[dev]) {
    if (cudaMalloc(&words[dev], sizeof(int)) != cudaSuccess) return nullptr;
    cudaMemset(words[dev], 0, sizeof(int));
  }
  return words[dev];
}

int zc_health_read_and_clear() {
  int* w = zc_health_word();
  if (!w) return -1;
  int v = 0;
  cudaMemcpy(&v, w, sizeof(int), cudaMemcpyDeviceToHost);
  if (v) cudaMemset(w, 0, sizeof(int));
  return v;
}

// Host-side injection of a failure (tests, drills): what a collective that gave up would have written.
int zc_health_set(int value) {
  int* w = zc_health_word();
  if (!w) return -1;
  return cudaMemcpy(w, &value, sizeof(int), cudaMemcpyHostToDevice) == cudaSuccess ? 0 : -1;
}

// `guard`: device pointer to a word that must be 0 for the update to happen (null: unconditional).
// With the health word there, an optimizer step that follows a collective which gave up leaves
// parameters and moments untouched, with no host synchronisation between the two.
int zc_adamw_guarded(void* p, void* g, void* m, void* v, int64_t n, int pdt, int gdt, int sdt, float lr, float b1,
                     float b2, float eps, float wd, float bc1, float bc2, int zero_grad, const int* guard,
                     cudaStream_t st) {
  if (n == 0) return 0;
  if (pdt == 0 && gdt == 0)
    return zc::adamw_dispatch_s<bf16, bf16>(p, g, m, v, n, sdt, lr, b1, b2, eps, wd, bc1, bc2, zero_grad, guard, st);
  if (pdt == 1 && gdt == 1)
    return zc::adamw_dispatch_s<float, float>(p, g, m, v, n, sdt, lr, b1, b2, eps, wd, bc1, bc2, zero_grad, guard, st);
  if (pdt == 0 && gdt == 1)
    return zc::adamw_dispatch_s<bf16, float>(p, g, m, v, n, sdt, lr, b1, b2, eps, wd, bc1, bc2, zero_grad, guard, st);
  if (pdt == 1 && gdt == 0)
    return zc::adamw_dispatch_s<float, bf16>(p, g, m, v, n, sdt, lr, b1, b2, eps, wd, bc1, bc2, zero_grad, guard, st);
  return ERR_UNSUPPORTED;
}

int zc_adamw(void* p, void* g, void* m, void* v, int64_t n, int pdt, int gdt, int sdt, float lr, float b1, float b2,
             float eps, float wd, float bc1, float bc2, int zero_grad, cudaStream_t st) {
  return zc_adamw_guarded(p, g, m, v, n, pdt, gdt, sdt, lr, b1, b2, eps, wd, bc1, bc2, zero_grad, nullptr, st);
}

}  // extern "C"
