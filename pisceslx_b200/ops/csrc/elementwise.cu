// Memory-bound kernels: RMSNorm forward/backward (with fused residual add and FiLM epilogue), rotary
// embeddings (1-D / partial and 3-D video), SwiGLU forward/backward, FiLM, add, and an L2 flush.
// All of them move 16-byte vectors and keep a row in registers so that each element crosses HBM once.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "yv_ops.h"

namespace yv {

namespace {

struct alignas(16) BF8 {
  __nv_bfloat162 v[4];
};

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&f)[8]) {
  BF8 r = *reinterpret_cast<const BF8*>(p);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(r.v[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&f)[8]) {
  BF8 r;
#pragma unroll
  for (int i = 0; i < 4; ++i) r.v[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  *reinterpret_cast<BF8*>(p) = r;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
  return v;
}

__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum(v);
  if (lane == 0) red[warp] = v;
  __syncthreads();
  const int nw = (blockDim.x + 31) >> 5;
  float t = (threadIdx.x < nw) ? red[threadIdx.x] : 0.f;
  if (warp == 0) {
    t = warp_sum(t);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  const float out = red[32];
  __syncthreads();
  return out;
}

// ---------------------------------------------------------------------------------------------
// RMSNorm forward.  One block per row; VPT 16-byte vectors per thread stay in registers.
// ---------------------------------------------------------------------------------------------
template <int VPT>
__global__ void rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ residual,
                                   const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ fscale,
                                   const __nv_bfloat16* __restrict__ fshift, int64_t film_rows,
                                   __nv_bfloat16* __restrict__ y, __nv_bfloat16* __restrict__ res_out,
                                   float* __restrict__ rstd_out, int cols, float eps) {
  __shared__ float red[33];
  const int64_t row = blockIdx.x;
  const int nvec = cols >> 3;
  float v[VPT][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int vec = threadIdx.x + i * blockDim.x;
    if (vec < nvec) {
      load8(x + row * cols + vec * 8, v[i]);
      if (residual != nullptr) {
        float r[8];
        load8(residual + row * cols + vec * 8, r);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[i][j] += r[j];
        if (res_out != nullptr) {
          store8(res_out + row * cols + vec * 8, v[i]);
          // normalise what was stored: the bf16-rounded sum
#pragma unroll
          for (int j = 0; j < 8; ++j) v[i][j] = __bfloat162float(__float2bfloat16(v[i][j]));
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += v[i][j] * v[i][j];
    }
  }
  ss = block_sum(ss, red);
  const float rstd = rsqrtf(ss / static_cast<float>(cols) + eps);
  if (threadIdx.x == 0 && rstd_out != nullptr) rstd_out[row] = rstd;
  const int64_t g = (fscale != nullptr) ? row / film_rows : 0;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int vec = threadIdx.x + i * blockDim.x;
    if (vec < nvec) {
      float wv[8], o[8];
      load8(w + vec * 8, wv);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = v[i][j] * rstd * wv[j];
      if (fscale != nullptr) {
        float s[8], b[8];
        load8(fscale + g * cols + vec * 8, s);
        load8(fshift + g * cols + vec * 8, b);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = o[j] * (1.f + s[j]) + b[j];
      }
      store8(y + row * cols + vec * 8, o);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// RMSNorm backward.  Each block walks a strip of rows, keeps its dw partial sums in registers and
// writes them once; dx is written per row.
//   xhat = x * rstd;  g = dy * w;  dx = rstd * (g - xhat * mean(g * xhat)) (+ dres_in);  dw = sum dy * xhat
// ---------------------------------------------------------------------------------------------
template <int VPT>
__global__ void rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                   const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd,
                                   const __nv_bfloat16* __restrict__ dres_in, __nv_bfloat16* __restrict__ dx,
                                   float* __restrict__ dw_partial, int64_t rows, int cols) {
  __shared__ float red[33];
  const int nvec = cols >> 3;
  float dwacc[VPT][8];
  float wv[VPT][8];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int vec = threadIdx.x + i * blockDim.x;
#pragma unroll
    for (int j = 0; j < 8; ++j) dwacc[i][j] = 0.f;
    if (vec < nvec) load8(w + vec * 8, wv[i]);
  }
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const float rs = rstd[row];
    float xh[VPT][8], g[VPT][8];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vec = threadIdx.x + i * blockDim.x;
      if (vec < nvec) {
        float dyv[8];
        load8(dy + row * cols + vec * 8, dyv);
        load8(x + row * cols + vec * 8, xh[i]);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[i][j] *= rs;
          g[i][j] = dyv[j] * wv[i][j];
          dot += g[i][j] * xh[i][j];
          dwacc[i][j] += dyv[j] * xh[i][j];
        }
      }
    }
    dot = block_sum(dot, red) / static_cast<float>(cols);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vec = threadIdx.x + i * blockDim.x;
      if (vec < nvec) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rs * (g[i][j] - xh[i][j] * dot);
        if (dres_in != nullptr) {
          float r[8];
          load8(dres_in + row * cols + vec * 8, r);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += r[j];
        }
        store8(dx + row * cols + vec * 8, o);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int vec = threadIdx.x + i * blockDim.x;
    if (vec < nvec) {
      float* dst = dw_partial + static_cast<int64_t>(blockIdx.x) * cols + vec * 8;
#pragma unroll
      for (int j = 0; j < 8; ++j) dst[j] = dwacc[i][j];
    }
  }
}

__global__ void colsum_kernel(const float* __restrict__ partial, int blocks, int cols, void* out, int out_fp32,
                              int accumulate) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  float s = 0.f;
  for (int b = 0; b < blocks; ++b) s += partial[static_cast<int64_t>(b) * cols + c];
  if (out_fp32) {
    float* o = reinterpret_cast<float*>(out);
    o[c] = accumulate ? o[c] + s : s;
  } else {
    __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(out);
    o[c] = __float2bfloat16(accumulate ? __bfloat162float(o[c]) + s : s);
  }
}

// ---------------------------------------------------------------------------------------------
// Rotary embedding, rotate-half layout: pairs (i, i + rot/2) of the first rot_dim dims of each head.
// cos/sin tables are fp32 [max_pos, rot/2].  One block per token, threads over (head, pair).
// ---------------------------------------------------------------------------------------------
__global__ void rope_kernel(__nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ k,
                            const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                            const int* __restrict__ positions, int hq, int hk, int head_dim, int rot_dim,
                            int inverse, int64_t q_stride, int64_t k_stride) {
  const int64_t t = blockIdx.x;
  const int half = rot_dim >> 1;
  const int pos = positions[t];
  const int total = (hq + hk) * half;
  for (int i = threadIdx.x; i < total; i += blockDim.x) {
    const int h = i / half, p = i - h * half;
    __nv_bfloat16* base = (h < hq) ? (q + t * q_stride + static_cast<int64_t>(h) * head_dim)
                                   : (k + t * k_stride + static_cast<int64_t>(h - hq) * head_dim);
    const float c = cos_t[static_cast<int64_t>(pos) * half + p];
    float s = sin_t[static_cast<int64_t>(pos) * half + p];
    if (inverse) s = -s;
    const float a = __bfloat162float(base[p]);
    const float b = __bfloat162float(base[p + half]);
    base[p] = __float2bfloat16(a * c - b * s);
    base[p + half] = __float2bfloat16(b * c + a * s);
  }
}

// 3-D rotary embedding: the head dimension is split into (d_t, d_h, d_w) sections; section s rotates
// with position pos[s] and frequencies theta^(-2i/d_s), rotate-half inside the section.
__global__ void rope3d_kernel(__nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ k,
                              const int* __restrict__ pos_thw, int hq, int hk, int head_dim, int d_t, int d_h,
                              int d_w, float theta, int inverse) {
  const int64_t t = blockIdx.x;
  const int halves = (d_t + d_h + d_w) >> 1;
  const int total = (hq + hk) * halves;
  const float log2_theta = log2f(theta);
  for (int i = threadIdx.x; i < total; i += blockDim.x) {
    const int h = i / halves;
    int p = i - h * halves;
    int sec_off, sec_dim, pos;
    if (p < (d_t >> 1)) {
      sec_off = 0; sec_dim = d_t; pos = pos_thw[t * 3 + 0];
    } else if (p < ((d_t + d_h) >> 1)) {
      p -= d_t >> 1; sec_off = d_t; sec_dim = d_h; pos = pos_thw[t * 3 + 1];
    } else {
      p -= (d_t + d_h) >> 1; sec_off = d_t + d_h; sec_dim = d_w; pos = pos_thw[t * 3 + 2];
    }
    const int half = sec_dim >> 1;
    const float inv_freq = exp2f(-log2_theta * (2.f * p) / static_cast<float>(sec_dim));
    float s, c;
    sincosf(static_cast<float>(pos) * inv_freq, &s, &c);
    if (inverse) s = -s;
    __nv_bfloat16* base = (h < hq) ? (q + (t * hq + h) * head_dim) : (k + (t * hk + (h - hq)) * head_dim);
    base += sec_off;
    const float a = __bfloat162float(base[p]);
    const float b = __bfloat162float(base[p + half]);
    base[p] = __float2bfloat16(a * c - b * s);
    base[p + half] = __float2bfloat16(b * c + a * s);
  }
}

// ---------------------------------------------------------------------------------------------
// SwiGLU
// ---------------------------------------------------------------------------------------------
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out,
                                  int64_t rows, int F) {
  const int fv = F >> 3;
  const int64_t total = rows * fv;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / fv;
    const int c = static_cast<int>(i - r * fv) * 8;
    float g[8], u[8], o[8];
    load8(in + r * 2 * F + c, g);
    load8(in + r * 2 * F + F + c, u);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = g[j] / (1.f + __expf(-g[j])) * u[j];
    store8(out + r * F + c, o);
  }
}

__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ in, const __nv_bfloat16* __restrict__ dout,
                                  __nv_bfloat16* __restrict__ din, int64_t rows, int F) {
  const int fv = F >> 3;
  const int64_t total = rows * fv;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / fv;
    const int c = static_cast<int>(i - r * fv) * 8;
    float g[8], u[8], d[8], dg[8], du[8];
    load8(in + r * 2 * F + c, g);
    load8(in + r * 2 * F + F + c, u);
    load8(dout + r * F + c, d);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float sg = 1.f / (1.f + __expf(-g[j]));
      const float silu = g[j] * sg;
      du[j] = d[j] * silu;
      dg[j] = d[j] * u[j] * (sg + silu * (1.f - sg));
    }
    store8(din + r * 2 * F + c, dg);
    store8(din + r * 2 * F + F + c, du);
  }
}

// SwiGLU backward for expert rows when neither the activation nor the expert outputs were kept: one warp per row.
//   in [rows, 2F] (gate | up pre-activations), dact [rows, F] = UNWEIGHTED gradient of the activation,
//   row_w [rows] = combine weight of the row (0 on pad rows and dropped assignments)
//   din  [rows, 2F] = row_w * dSwiGLU(in, dact)          (gradient of the up projection's output)
//   actw [rows, F]  = row_w * SwiGLU(in)                 (B operand of the down projection's weight gradient)
//   rowdot [rows]   = sum_f SwiGLU(in)[f] * dact[f]      (gradient of the row's combine weight)
__global__ void swiglu_bwd_rows_kernel(const __nv_bfloat16* __restrict__ in, const __nv_bfloat16* __restrict__ dact,
                                       const float* __restrict__ row_w, __nv_bfloat16* __restrict__ din,
                                       __nv_bfloat16* __restrict__ actw, float* __restrict__ rowdot, int64_t rows, int F) {
  const int lane = threadIdx.x & 31;
  const int fv = F >> 3;
  const int64_t warp0 = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5;
  const int64_t nwarps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  for (int64_t r = warp0; r < rows; r += nwarps) {
    const float w = row_w[r];
    float dot = 0.f;
    for (int cv = lane; cv < fv; cv += 32) {
      const int c = cv * 8;
      float g[8], u[8], d[8], dg[8], du[8], a[8];
      load8(in + r * 2 * F + c, g);
      load8(in + r * 2 * F + F + c, u);
      load8(dact + r * F + c, d);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float sg = 1.f / (1.f + __expf(-g[j]));
        const float silu = g[j] * sg;
        const float act = silu * u[j];
        dot += act * d[j];
        a[j] = w * act;
        du[j] = w * d[j] * silu;
        dg[j] = w * d[j] * u[j] * (sg + silu * (1.f - sg));
      }
      store8(din + r * 2 * F + c, dg);
      store8(din + r * 2 * F + F + c, du);
      store8(actw + r * F + c, a);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
    if (lane == 0) rowdot[r] = dot;
  }
}

__global__ void film_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ scale,
                            const __nv_bfloat16* __restrict__ shift, __nv_bfloat16* __restrict__ y, int64_t rows,
                            int cols, int64_t rows_per_group) {
  const int cv = cols >> 3;
  const int64_t total = rows * cv;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / cv;
    const int c = static_cast<int>(i - r * cv) * 8;
    const int64_t g = r / rows_per_group;
    float a[8], s[8], b[8];
    load8(x + r * cols + c, a);
    load8(scale + g * cols + c, s);
    load8(shift + g * cols + c, b);
#pragma unroll
    for (int j = 0; j < 8; ++j) a[j] = a[j] * (1.f + s[j]) + b[j];
    store8(y + r * cols + c, a);
  }
}

__global__ void add_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                           __nv_bfloat16* __restrict__ out, int64_t nvec) {
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    float x[8], y[8];
    load8(a + i * 8, x);
    load8(b + i * 8, y);
#pragma unroll
    for (int j = 0; j < 8; ++j) x[j] += y[j];
    store8(out + i * 8, x);
  }
}

__global__ void l2_flush_kernel(uint4* buf, int64_t n) {
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    buf[i] = make_uint4(static_cast<uint32_t>(i), 0u, 0u, 0u);
  }
}

inline int grid_for(int64_t work, int block, int cap = 148 * 16) {
  int64_t g = (work + block - 1) / block;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  return static_cast<int>(g);
}

inline int norm_block(int cols, int* vpt) {
  const int nvec = cols >> 3;
  int block = 256;
  if (nvec <= 128) block = 128;
  int v = (nvec + block - 1) / block;
  if (v <= 1) v = 1; else if (v <= 2) v = 2; else if (v <= 4) v = 4; else v = 8;
  *vpt = v;
  return block;
}

}  // namespace

#define YV_BF(p) reinterpret_cast<const __nv_bfloat16*>(p)
#define YV_BFM(p) reinterpret_cast<__nv_bfloat16*>(p)

int launch_rmsnorm_fwd(const void* x, const void* residual, const void* w, const void* film_scale,
                       const void* film_shift, int64_t film_rows_per_group, void* y, void* res_out, float* rstd,
                       int64_t rows, int cols, float eps, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if ((cols & 7) != 0 || cols > 16384) return -1;
  int vpt;
  const int block = norm_block(cols, &vpt);
  const unsigned grid = static_cast<unsigned>(rows);
#define YV_LAUNCH(V)                                                                                          \
  rmsnorm_fwd_kernel<V><<<grid, block, 0, stream>>>(YV_BF(x), YV_BF(residual), YV_BF(w), YV_BF(film_scale),   \
                                                     YV_BF(film_shift), film_rows_per_group, YV_BFM(y),       \
                                                     YV_BFM(res_out), rstd, cols, eps)
  switch (vpt) {
    case 1: YV_LAUNCH(1); break;
    case 2: YV_LAUNCH(2); break;
    case 4: YV_LAUNCH(4); break;
    default: YV_LAUNCH(8); break;
  }
#undef YV_LAUNCH
  return static_cast<int>(cudaGetLastError());
}

int launch_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const void* dres_in,
                       void* dx, float* dw_partial, int dw_blocks, int64_t rows, int cols, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if ((cols & 7) != 0 || cols > 16384 || dw_blocks <= 0) return -1;
  int vpt;
  const int block = norm_block(cols, &vpt);
#define YV_LAUNCH(V)                                                                                         \
  rmsnorm_bwd_kernel<V><<<dw_blocks, block, 0, stream>>>(YV_BF(dy), YV_BF(x), YV_BF(w), rstd, YV_BF(dres_in), \
                                                          YV_BFM(dx), dw_partial, rows, cols)
  switch (vpt) {
    case 1: YV_LAUNCH(1); break;
    case 2: YV_LAUNCH(2); break;
    case 4: YV_LAUNCH(4); break;
    default: YV_LAUNCH(8); break;
  }
#undef YV_LAUNCH
  return static_cast<int>(cudaGetLastError());
}

int launch_colsum(const float* partial, int blocks, int cols, void* out, int out_fp32, int accumulate,
                  cudaStream_t stream) {
  colsum_kernel<<<(cols + 255) / 256, 256, 0, stream>>>(partial, blocks, cols, out, out_fp32, accumulate);
  return static_cast<int>(cudaGetLastError());
}

int launch_rope_tables(void* q, void* k, const float* cos_t, const float* sin_t, const int* positions,
                       int64_t tokens, int hq, int hk, int head_dim, int rot_dim, int inverse, int64_t q_stride,
                       int64_t k_stride, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if ((rot_dim & 1) != 0 || rot_dim > head_dim) return -1;
  const int total = (hq + hk) * (rot_dim >> 1);
  const int block = total >= 256 ? 256 : ((total + 31) / 32) * 32;
  rope_kernel<<<static_cast<unsigned>(tokens), block, 0, stream>>>(YV_BFM(q), YV_BFM(k), cos_t, sin_t, positions,
                                                                   hq, hk, head_dim, rot_dim, inverse, q_stride,
                                                                   k_stride);
  return static_cast<int>(cudaGetLastError());
}

int launch_rope3d(void* q, void* k, const int* pos_thw, int64_t tokens, int hq, int hk, int head_dim, int d_t,
                  int d_h, int d_w, float theta, int inverse, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (((d_t | d_h | d_w) & 1) != 0 || d_t + d_h + d_w > head_dim) return -1;
  rope3d_kernel<<<static_cast<unsigned>(tokens), 256, 0, stream>>>(YV_BFM(q), YV_BFM(k), pos_thw, hq, hk, head_dim,
                                                                   d_t, d_h, d_w, theta, inverse);
  return static_cast<int>(cudaGetLastError());
}

int launch_swiglu_fwd(const void* in, void* out, int64_t rows, int F, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if ((F & 7) != 0) return -1;
  swiglu_fwd_kernel<<<grid_for(rows * (F >> 3), 256), 256, 0, stream>>>(YV_BF(in), YV_BFM(out), rows, F);
  return static_cast<int>(cudaGetLastError());
}

int launch_swiglu_bwd_rows(const void* in, const void* dact, const float* row_w, void* din, void* actw, float* rowdot,
                           int64_t rows, int F, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if ((F & 7) != 0) return -1;
  swiglu_bwd_rows_kernel<<<grid_for(rows * 32, 256), 256, 0, stream>>>(YV_BF(in), YV_BF(dact), row_w, YV_BFM(din),
                                                                      YV_BFM(actw), rowdot, rows, F);
  return static_cast<int>(cudaGetLastError());
}

int launch_swiglu_bwd(const void* in, const void* dout, void* din, int64_t rows, int F, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if ((F & 7) != 0) return -1;
  swiglu_bwd_kernel<<<grid_for(rows * (F >> 3), 256), 256, 0, stream>>>(YV_BF(in), YV_BF(dout), YV_BFM(din), rows,
                                                                        F);
  return static_cast<int>(cudaGetLastError());
}

int launch_film(const void* x, const void* scale, const void* shift, void* y, int64_t rows, int cols,
                int64_t rows_per_group, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if ((cols & 7) != 0 || rows_per_group <= 0) return -1;
  film_kernel<<<grid_for(rows * (cols >> 3), 256), 256, 0, stream>>>(YV_BF(x), YV_BF(scale), YV_BF(shift),
                                                                     YV_BFM(y), rows, cols, rows_per_group);
  return static_cast<int>(cudaGetLastError());
}

int launch_add(const void* a, const void* b, void* out, int64_t n, cudaStream_t stream) {
  if (n <= 0) return 0;
  if ((n & 7) != 0) return -1;
  add_kernel<<<grid_for(n >> 3, 256), 256, 0, stream>>>(YV_BF(a), YV_BF(b), YV_BFM(out), n >> 3);
  return static_cast<int>(cudaGetLastError());
}

namespace {
// out[m, n] = sum_s ws[s][m, n] (+ bias[n]); ws is fp32 [slices][m_pad, N]; four columns per thread
__global__ void splitk_reduce_kernel(const float* __restrict__ ws, const __nv_bfloat16* __restrict__ bias,
                                     __nv_bfloat16* __restrict__ out, int slices, int M, int m_pad, int N) {
  const int64_t quads = static_cast<int64_t>(M) * (N >> 2);
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < quads;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t m = i / (N >> 2);
    const int n = static_cast<int>(i - m * (N >> 2)) << 2;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s = 0; s < slices; ++s) {
      const float4 v = *reinterpret_cast<const float4*>(ws + (static_cast<int64_t>(s) * m_pad + m) * N + n);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    if (bias != nullptr) {
      acc.x += __bfloat162float(bias[n]); acc.y += __bfloat162float(bias[n + 1]);
      acc.z += __bfloat162float(bias[n + 2]); acc.w += __bfloat162float(bias[n + 3]);
    }
    __nv_bfloat162* o = reinterpret_cast<__nv_bfloat162*>(out + m * N + n);
    o[0] = __floats2bfloat162_rn(acc.x, acc.y);
    o[1] = __floats2bfloat162_rn(acc.z, acc.w);
  }
}
}  // namespace

int launch_splitk_reduce(const float* ws, const void* bias, void* out, int slices, int M, int m_pad, int N,
                         cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if ((N & 3) != 0 || slices <= 0 || m_pad < M) return -1;
  splitk_reduce_kernel<<<grid_for(static_cast<int64_t>(M) * (N >> 2), 256), 256, 0, stream>>>(
      ws, YV_BF(bias), YV_BFM(out), slices, M, m_pad, N);
  return static_cast<int>(cudaGetLastError());
}

namespace {
// eight bf16 values per thread -> eight e4m3 bytes; |x| maximum reduced per warp, one atomic per warp
__global__ void fp8_quantize_kernel(const uint4* __restrict__ x, const float* __restrict__ scale,
                                    uint2* __restrict__ q, float* __restrict__ amax, int64_t n8) {
  const float sc = *scale;
  float mx = 0.f;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n8;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const uint4 v = x[i];
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
    uint32_t out[2];
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const float2 a = __bfloat1622float2(h[2 * k]), b = __bfloat1622float2(h[2 * k + 1]);
      mx = fmaxf(mx, fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(b.x), fabsf(b.y))));
      uint16_t lo, hi;
      asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(lo) : "f"(a.y * sc), "f"(a.x * sc));
      asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(hi) : "f"(b.y * sc), "f"(b.x * sc));
      out[k] = static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
    }
    q[i] = make_uint2(out[0], out[1]);
  }
  if (amax != nullptr) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
    if ((threadIdx.x & 31) == 0) atomicMax(reinterpret_cast<int*>(amax), __float_as_int(mx));   // mx >= 0
  }
}

// Running attention partial <- merged with another partial over a disjoint key set (ring / context parallel attention):
// lse = log(exp(lse_a) + exp(lse_b)), o = o_a * exp(lse_a - lse) + o_b * exp(lse_b - lse); rows with no keys on
// either side (lse = -inf) keep zeros.  One warp per (token, head) row of d floats.
__global__ void attn_merge_kernel(float* __restrict__ o_acc, float* __restrict__ lse_acc, const float* __restrict__ o_b,
                                  const float* __restrict__ lse_b, int64_t rows, int d) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5;
  if (row >= rows) return;
  const float la = lse_acc[row], lb = lse_b[row];
  const float m = fmaxf(la, lb);
  float wa = 0.f, wb = 0.f, l = m;
  if (m > -INFINITY) {
    const float ea = __expf(la - m), eb = __expf(lb - m);
    l = m + __logf(ea + eb);
    wa = ea / (ea + eb);
    wb = eb / (ea + eb);
  }
  for (int c = lane; c < d; c += 32) {
    const int64_t i = row * d + c;
    o_acc[i] = o_acc[i] * wa + o_b[i] * wb;
  }
  __syncwarp();
  if (lane == 0) lse_acc[row] = l;
}

// Block-scaled (MX) quantisation: four lanes share one 32-element block (8 elements each).
__global__ void mx_quantize_kernel(const uint4* __restrict__ x, uint2* __restrict__ q, uint8_t* __restrict__ sf,
                                   int64_t n8, int K) {
  const int kchunks = K >> 7;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;           // a multiple of 32
  const int64_t n8_up = (n8 + 31) & ~static_cast<int64_t>(31);                    // whole warps take the shuffles
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n8_up; i += stride) {
    const bool in = i < n8;
    const uint4 v = in ? x[i] : make_uint4(0u, 0u, 0u, 0u);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
    float f[8];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 a = __bfloat1622float2(h[k]);
      f[2 * k] = a.x; f[2 * k + 1] = a.y;
    }
    float mx = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) mx = fmaxf(mx, fabsf(f[k]));
    mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 2));
    // smallest power-of-two scale that brings the block's largest magnitude to at most 448 = 1.75 * 2^8:
    // amax = m * 2^x with 1 <= m < 2 gives exponent x - 8, one more when m > 1.75.  Stored as a biased exponent byte,
    // 127 (= 1.0) for an all-zero block.
    const uint32_t mbits = __float_as_uint(mx);
    int eb = static_cast<int>((mbits >> 23) & 0xFFu) - 8 + ((mbits & 0x7FFFFFu) > 0x600000u ? 1 : 0);
    if (!(mx > 0.f)) eb = 127;
    eb = eb < 0 ? 0 : (eb > 253 ? 253 : eb);
    const float inv = __uint_as_float(static_cast<uint32_t>(254 - eb) << 23);
    if (!in) continue;
    uint32_t out[2];
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      uint16_t lo, hi;
      asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(lo) : "f"(f[4 * k + 1] * inv), "f"(f[4 * k] * inv));
      asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(hi) : "f"(f[4 * k + 3] * inv), "f"(f[4 * k + 2] * inv));
      out[k] = static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
    }
    q[i] = make_uint2(out[0], out[1]);
    if ((threadIdx.x & 3) == 0) {
      const int64_t e0 = i << 3;
      const int64_t row = e0 / K;
      const int col = static_cast<int>(e0 - row * K);
      const int r = static_cast<int>(row & 127);
      sf[((row >> 7) * kchunks + (col >> 7)) * 512 + (r & 31) * 16 + (r >> 5) * 4 + ((col & 127) >> 5)] =
          static_cast<uint8_t>(eb);
    }
  }
}
}  // namespace

int launch_attn_merge(float* o_acc, float* lse_acc, const float* o_b, const float* lse_b, int64_t rows, int d,
                      cudaStream_t stream) {
  if (rows <= 0) return 0;
  const int64_t threads = rows * 32;
  attn_merge_kernel<<<static_cast<unsigned>((threads + 255) / 256), 256, 0, stream>>>(o_acc, lse_acc, o_b, lse_b, rows, d);
  return static_cast<int>(cudaGetLastError());
}

int launch_mx_quantize(const void* x_bf16, void* q_e4m3, void* sf, int64_t rows, int K, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (K <= 0 || (K & 127) != 0) return -1;
  const int64_t n8 = rows * K / 8;
  mx_quantize_kernel<<<grid_for(n8, 256), 256, 0, stream>>>(reinterpret_cast<const uint4*>(x_bf16),
                                                            reinterpret_cast<uint2*>(q_e4m3),
                                                            reinterpret_cast<uint8_t*>(sf), n8, K);
  return static_cast<int>(cudaGetLastError());
}

int launch_fp8_quantize(const void* x_bf16, const float* scale, void* q_e4m3, float* amax, int64_t n,
                        cudaStream_t stream) {
  if (n <= 0) return 0;
  if ((n & 7) != 0) return -1;
  fp8_quantize_kernel<<<grid_for(n >> 3, 256), 256, 0, stream>>>(reinterpret_cast<const uint4*>(x_bf16), scale,
                                                                 reinterpret_cast<uint2*>(q_e4m3), amax, n >> 3);
  return static_cast<int>(cudaGetLastError());
}

int launch_l2_flush(void* buf, int64_t bytes, cudaStream_t stream) {
  l2_flush_kernel<<<148 * 8, 256, 0, stream>>>(reinterpret_cast<uint4*>(buf), bytes / 16);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace yv
