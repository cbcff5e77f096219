// Memory-bound ops of the GPT-2 decoder family for sm_100a: LayerNorm forward/backward (weight and
// bias) and the fused bias + tanh-GELU of the MLP, forward and backward.  Same conventions as the
// RMSNorm / SwiGLU kernels: bf16 tensors, 16-byte vectors, fp32 arithmetic in registers, one pass
// over HBM per kernel.  The reference gets these from HF GPT-2 modules (ATen LayerNorm, `NewGELU`,
// separate bias adds).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <algorithm>

#include "launch_util.h"

namespace zc {
namespace gpt2 {

constexpr unsigned FULLM = 0xffffffffu;
constexpr int LN_THREADS = 256;
constexpr int LN_MAX_COLS = LN_THREADS * 4 * 8;  // vectors of 8 per thread: 1, 2 or 4

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
// block-wide sums of two values at once (one pair of barriers); every thread gets both results
__device__ __forceinline__ float2 block_sum2(float a, float b, float2* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  a = warp_sum(a);
  b = warp_sum(b);
  __syncthreads();
  if (lane == 0) red[warp] = make_float2(a, b);
  __syncthreads();
  const float2 t = (lane < nw) ? red[lane] : make_float2(0.f, 0.f);
  return make_float2(warp_sum(t.x), warp_sum(t.y));
}

// ---------------------------------------------------------------------------------------------
// LayerNorm.  One CTA per row, row cached in registers (cols <= 8192, cols % 8 == 0).
//   mean = E[h], rstd = rsqrt(E[(h - mean)^2] + eps), y = (h - mean) * rstd * w + b
// h = x, or with `res` the residual sum x + res rounded to bf16, which is also written to `h_out`
// (the residual add of the block before, done here instead of in a kernel of its own).
// ---------------------------------------------------------------------------------------------
template <int MAXV>
__global__ void __launch_bounds__(LN_THREADS) layernorm_fwd_kernel(
    const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res, const __nv_bfloat16* __restrict__ w,
    const __nv_bfloat16* __restrict__ b, __nv_bfloat16* __restrict__ y, __nv_bfloat16* __restrict__ h_out,
    float* __restrict__ mean_out, float* __restrict__ rstd_out, int cols, float eps) {
  __shared__ float2 red[32];
  const int64_t row = blockIdx.x;
  const int nvec = cols / 8;
  float h[MAXV][8];
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int v = threadIdx.x + i * LN_THREADS;
    if (v < nvec) {
      unpack8(ld8(x + row * cols + v * 8), h[i]);
      if (res) {
        float r[8];
        unpack8(ld8(res + row * cols + v * 8), r);
#pragma unroll
        for (int j = 0; j < 8; ++j) h[i][j] += r[j];
        const BF8 hb = pack8(h[i]);
        st8(h_out + row * cols + v * 8, hb);
        unpack8(hb, h[i]);  // normalise what was stored: the backward pass reads it back
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) s += h[i][j];
    }
  }
  const float mean = block_sum2(s, 0.f, red).x / (float)cols;
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int v = threadIdx.x + i * LN_THREADS;
    if (v < nvec) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        h[i][j] -= mean;
        ss += h[i][j] * h[i][j];
      }
    }
  }
  const float rstd = rsqrtf(block_sum2(ss, 0.f, red).x / (float)cols + eps);
  if (threadIdx.x == 0) {
    mean_out[row] = mean;
    rstd_out[row] = rstd;
  }
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int v = threadIdx.x + i * LN_THREADS;
    if (v < nvec) {
      float wv[8], bv[8], o[8];
      unpack8(ld8(w + v * 8), wv);
      unpack8(ld8(b + v * 8), bv);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = h[i][j] * rstd * wv[j] + bv[j];
      st8(y + row * cols + v * 8, pack8(o));
    }
  }
}

// dx = rstd * (g - mean(g) - xhat * mean(g * xhat)) (+ dh),  g = dy * w,  xhat = (x - mean) * rstd
// dw = sum_rows dy * xhat, db = sum_rows dy: per-CTA partial sums in registers, written to
// partials[cta][0 | 1][cols] and summed by column_sum_deliver_kernel (no atomics)
template <int MAXV>
__global__ void __launch_bounds__(LN_THREADS) layernorm_bwd_kernel(
    const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
    const float* __restrict__ mean_in, const float* __restrict__ rstd_in, const __nv_bfloat16* __restrict__ dh,
    __nv_bfloat16* __restrict__ dx, float* __restrict__ partials, int64_t rows, int cols) {
  __shared__ float2 red[32];
  const int nvec = cols / 8;
  float wv[MAXV][8], dwacc[MAXV][8], dbacc[MAXV][8];
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int v = threadIdx.x + i * LN_THREADS;
#pragma unroll
    for (int j = 0; j < 8; ++j) dwacc[i][j] = dbacc[i][j] = 0.f;
    if (v < nvec) unpack8(ld8(w + v * 8), wv[i]);
  }
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const float mean = mean_in[row], rstd = rstd_in[row];
    float g[MAXV][8], xh[MAXV][8];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int v = threadIdx.x + i * LN_THREADS;
      if (v < nvec) {
        float d[8];
        unpack8(ld8(dy + row * cols + v * 8), d);
        unpack8(ld8(x + row * cols + v * 8), xh[i]);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[i][j] = (xh[i][j] - mean) * rstd;
          g[i][j] = d[j] * wv[i][j];
          s1 += g[i][j];
          s2 += g[i][j] * xh[i][j];
          dwacc[i][j] += d[j] * xh[i][j];
          dbacc[i][j] += d[j];
        }
      }
    }
    const float2 t = block_sum2(s1, s2, red);
    const float m1 = t.x / (float)cols, m2 = t.y / (float)cols;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int v = threadIdx.x + i * LN_THREADS;
      if (v < nvec) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rstd * (g[i][j] - m1 - xh[i][j] * m2);
        if (dh) {  // gradient arriving through the residual path of the same tensor
          float e[8];
          unpack8(ld8(dh + row * cols + v * 8), e);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += e[j];
        }
        st8(dx + row * cols + v * 8, pack8(o));
      }
    }
  }
  float* pw = partials + (int64_t)blockIdx.x * 2 * cols;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int v = threadIdx.x + i * LN_THREADS;
    if (v < nvec) {
      float4* dst = reinterpret_cast<float4*>(pw + v * 8);
      dst[0] = make_float4(dwacc[i][0], dwacc[i][1], dwacc[i][2], dwacc[i][3]);
      dst[1] = make_float4(dwacc[i][4], dwacc[i][5], dwacc[i][6], dwacc[i][7]);
      dst = reinterpret_cast<float4*>(pw + cols + v * 8);
      dst[0] = make_float4(dbacc[i][0], dbacc[i][1], dbacc[i][2], dbacc[i][3]);
      dst[1] = make_float4(dbacc[i][4], dbacc[i][5], dbacc[i][6], dbacc[i][7]);
    }
  }
}

// out[c] = sum_r in[r][c] for an [nrows, ncols] fp32 matrix (ncols % 4 == 0); block (32, 32): 32 float4
// columns x 32 row groups.  The result is delivered where the optimizer reads it: columns [0, seg) go to outA,
// [seg, 2 seg) to outB (null: a single segment), as fp32 or bf16, overwriting or adding to what is
// there.  Used for LayerNorm's weight / bias gradients and the linear layers' bias gradients, which
// can then be written straight into the flat gradient buffer of a sharded engine.
__global__ void __launch_bounds__(1024) column_sum_deliver_kernel(const float* __restrict__ in, int nrows, int ncols,
                                                                  int seg, void* __restrict__ outA,
                                                                  void* __restrict__ outB, int out_bf16, int accA,
                                                                  int accB) {
  __shared__ float4 acc[32][32];
  const int c4 = blockIdx.x * 32 + threadIdx.x;
  float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
  if (c4 * 4 < ncols) {
    for (int r = threadIdx.y; r < nrows; r += 32) {
      const float4 v = __ldg(reinterpret_cast<const float4*>(in + (int64_t)r * ncols) + c4);
      s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
    }
  }
  acc[threadIdx.y][threadIdx.x] = s;
  __syncthreads();
  if (threadIdx.y == 0 && c4 * 4 < ncols) {
#pragma unroll
    for (int k = 1; k < 32; ++k) {
      const float4 v = acc[k][threadIdx.x];
      s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
    }
    const float f[4] = {s.x, s.y, s.z, s.w};
    const int col = c4 * 4;                       // seg % 4 == 0: a float4 never straddles the segments
    const bool second = outB != nullptr && col >= seg;
    void* out = second ? outB : outA;
    const int oc = second ? col - seg : col;
    const int accumulate = second ? accB : accA;
    if (out_bf16) {
      __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(out) + oc;
#pragma unroll
      for (int j = 0; j < 4; ++j) o[j] = __float2bfloat16_rn(f[j] + (accumulate ? __bfloat162float(o[j]) : 0.f));
    } else {
      float* o = reinterpret_cast<float*>(out) + oc;
#pragma unroll
      for (int j = 0; j < 4; ++j) o[j] = f[j] + (accumulate ? o[j] : 0.f);
    }
  }
}

// partial column sums of a bf16 matrix [rows, cols] (rows `ld` elements apart): block (32, 8) covers
// 256 columns; blockIdx.y strides over the rows; partials[blockIdx.y][cols] fp32
__global__ void __launch_bounds__(256) bf16_column_partials_kernel(const __nv_bfloat16* __restrict__ in, int64_t rows,
                                                                   int cols, int64_t ld, float* __restrict__ partials) {
  __shared__ float red[8][32][8];
  const int v = blockIdx.x * 32 + threadIdx.x;  // 8-column vector
  float a[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (v * 8 < cols) {
    for (int64_t r = (int64_t)blockIdx.y * 8 + threadIdx.y; r < rows; r += (int64_t)gridDim.y * 8) {
      float f[8];
      unpack8(ld8(in + r * ld + v * 8), f);
#pragma unroll
      for (int j = 0; j < 8; ++j) a[j] += f[j];
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) red[threadIdx.y][threadIdx.x][j] = a[j];
  __syncthreads();
  if (threadIdx.y == 0 && v * 8 < cols) {
#pragma unroll
    for (int k = 1; k < 8; ++k)
#pragma unroll
      for (int j = 0; j < 8; ++j) a[j] += red[k][threadIdx.x][j];
    float4* dst = reinterpret_cast<float4*>(partials + (int64_t)blockIdx.y * cols + v * 8);
    dst[0] = make_float4(a[0], a[1], a[2], a[3]);
    dst[1] = make_float4(a[4], a[5], a[6], a[7]);
  }
}

// ---------------------------------------------------------------------------------------------
// y = gelu_tanh(x + bias):  0.5 u (1 + tanh(k (u + 0.044715 u^3))),  k = sqrt(2 / pi)
// backward: dx = dy * gelu'(x + bias); the bias gradient is the column sum of dx
// ---------------------------------------------------------------------------------------------
constexpr float GELU_K = 0.7978845608028654f;
constexpr float GELU_C = 0.044715f;

__global__ void __launch_bounds__(256) bias_gelu_fwd_kernel(const __nv_bfloat16* __restrict__ x,
                                                            const __nv_bfloat16* __restrict__ bias,
                                                            __nv_bfloat16* __restrict__ y, int64_t rows, int cols) {
  const int vpr = cols / 8;
  const int64_t total = rows * vpr;
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < total; i += (int64_t)gridDim.x * 256) {
    const int v = (int)(i % vpr);
    float u[8], bv[8], o[8];
    unpack8(ld8(x + i * 8), u);
    unpack8(ld8(bias + v * 8), bv);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float a = u[j] + bv[j];
      const float t = tanhf(GELU_K * (a + GELU_C * a * a * a));
      o[j] = 0.5f * a * (1.f + t);
    }
    st8(y + i * 8, pack8(o));
  }
}

__global__ void __launch_bounds__(256) bias_gelu_bwd_kernel(const __nv_bfloat16* __restrict__ x,
                                                            const __nv_bfloat16* __restrict__ bias,
                                                            const __nv_bfloat16* __restrict__ dy,
                                                            __nv_bfloat16* __restrict__ dx, int64_t rows, int cols) {
  const int vpr = cols / 8;
  const int64_t total = rows * vpr;
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < total; i += (int64_t)gridDim.x * 256) {
    const int v = (int)(i % vpr);
    float u[8], bv[8], g[8], o[8];
    unpack8(ld8(x + i * 8), u);
    unpack8(ld8(bias + v * 8), bv);
    unpack8(ld8(dy + i * 8), g);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float a = u[j] + bv[j];
      const float t = tanhf(GELU_K * (a + GELU_C * a * a * a));
      const float dt = (1.f - t * t) * GELU_K * (1.f + 3.f * GELU_C * a * a);
      o[j] = g[j] * (0.5f * (1.f + t) + 0.5f * a * dt);
    }
    st8(dx + i * 8, pack8(o));
  }
}

}  // namespace gpt2
}  // namespace zc

extern "C" {

using zc::ERR_UNSUPPORTED;
typedef __nv_bfloat16 bf16;

// res / h_out: both null, or the residual to add to x first and where to write the sum
int zc_layernorm_fwd(const void* x, const void* res, const void* w, const void* b, void* y, void* h_out, float* mean,
                     float* rstd, int64_t rows, int cols, float eps, cudaStream_t st) {
  using namespace zc::gpt2;
  if (cols % 8 || cols > LN_MAX_COLS || ((res == nullptr) != (h_out == nullptr))) return ERR_UNSUPPORTED;
  if (rows == 0) return 0;
  const int nvec = cols / 8;
#define ZC_LN_FWD(V)                                                                                              \
  layernorm_fwd_kernel<V><<<(unsigned)rows, LN_THREADS, 0, st>>>((const bf16*)x, (const bf16*)res, (const bf16*)w,  \
                                                                 (const bf16*)b, (bf16*)y, (bf16*)h_out, mean, rstd, \
                                                                 cols, eps)
  if (nvec <= LN_THREADS) ZC_LN_FWD(1);
  else if (nvec <= 2 * LN_THREADS) ZC_LN_FWD(2);
  else ZC_LN_FWD(4);
#undef ZC_LN_FWD
  return zc::launch_status();
}

// CTAs the backward launches for `rows` rows: `partials` must hold [that many, 2, cols] fp32
int zc_layernorm_bwd_ctas(int64_t rows) { return (int)std::min<int64_t>(rows, (int64_t)zc::sm_count() * 4); }

// dh: null, or a gradient of the same shape added to dx.  dw / db: [cols] each, fp32 or (out_bf16) bf16,
// overwritten or (acc_w / acc_b) added to.
int zc_layernorm_bwd(const void* dy, const void* x, const void* w, const float* mean, const float* rstd,
                     const void* dh, void* dx, void* dw, void* db, int out_bf16, int acc_w, int acc_b,
                     float* partials, int64_t rows, int cols, cudaStream_t st) {
  using namespace zc::gpt2;
  if (cols % 8 || cols > LN_MAX_COLS) return ERR_UNSUPPORTED;
  if (rows == 0) return 0;
  const int grid = zc_layernorm_bwd_ctas(rows);
  const int nvec = cols / 8;
#define ZC_LN_BWD(V)                                                                                          \
  layernorm_bwd_kernel<V><<<grid, LN_THREADS, 0, st>>>((const bf16*)dy, (const bf16*)x, (const bf16*)w, mean, rstd, \
                                                       (const bf16*)dh, (bf16*)dx, partials, rows, cols)
  if (nvec <= LN_THREADS) ZC_LN_BWD(1);
  else if (nvec <= 2 * LN_THREADS) ZC_LN_BWD(2);
  else ZC_LN_BWD(4);
#undef ZC_LN_BWD
  column_sum_deliver_kernel<<<(2 * cols / 4 + 31) / 32, dim3(32, 32), 0, st>>>(partials, grid, 2 * cols, cols, dw, db,
                                                                                out_bf16, acc_w, acc_b);
  return zc::launch_status();
}

// Row blocks of zc_bf16_column_sum for `rows` rows: `partials` must hold [that many, cols] fp32
int zc_bf16_column_sum_blocks(int64_t rows) { return (int)std::max<int64_t>(1, std::min<int64_t>(rows / 64, 32)); }

// out[c] (+)= sum over rows of in[r][c] for a bf16 matrix whose rows are `ld` elements apart
// (cols % 8 == 0, ld % 8 == 0): the bias gradient of a linear layer from its output gradient.
int zc_bf16_column_sum(const void* in, int64_t rows, int cols, int64_t ld, void* out, int out_bf16, int accumulate,
                       float* partials, cudaStream_t st) {
  using namespace zc::gpt2;
  if (cols % 8 || ld % 8 || (reinterpret_cast<uintptr_t>(in) & 15)) return ERR_UNSUPPORTED;
  if (rows == 0 || cols == 0) return 0;
  const int rb = zc_bf16_column_sum_blocks(rows);
  bf16_column_partials_kernel<<<dim3((cols / 8 + 31) / 32, rb), dim3(32, 8), 0, st>>>((const bf16*)in, rows, cols, ld,
                                                                                       partials);
  column_sum_deliver_kernel<<<(cols / 4 + 31) / 32, dim3(32, 32), 0, st>>>(partials, rb, cols, cols, out, nullptr,
                                                                            out_bf16, accumulate, 0);
  return zc::launch_status();
}

int zc_bias_gelu_fwd(const void* x, const void* bias, void* y, int64_t rows, int cols, cudaStream_t st) {
  if (cols % 8) return ERR_UNSUPPORTED;
  const int64_t total = rows * (cols / 8);
  if (total == 0) return 0;
  const int grid = (int)std::min<int64_t>((total + 255) / 256, (int64_t)zc::sm_count() * 16);
  zc::gpt2::bias_gelu_fwd_kernel<<<grid, 256, 0, st>>>((const bf16*)x, (const bf16*)bias, (bf16*)y, rows, cols);
  return zc::launch_status();
}

int zc_bias_gelu_bwd(const void* x, const void* bias, const void* dy, void* dx, int64_t rows, int cols,
                     cudaStream_t st) {
  if (cols % 8) return ERR_UNSUPPORTED;
  const int64_t total = rows * (cols / 8);
  if (total == 0) return 0;
  const int grid = (int)std::min<int64_t>((total + 255) / 256, (int64_t)zc::sm_count() * 16);
  zc::gpt2::bias_gelu_bwd_kernel<<<grid, 256, 0, st>>>((const bf16*)x, (const bf16*)bias, (const bf16*)dy, (bf16*)dx,
                                                        rows, cols);
  return zc::launch_status();
}

}  // extern "C"
