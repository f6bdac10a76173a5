// Loss, optimizer and miscellaneous streaming kernels: row-wise softmax cross-entropy that emits the
// logit gradient in the same pass, AdamW (mixed dtypes), Muon helpers (momentum fold, Frobenius
// normalisation, axpby, apply), sum of squares / scale (gradient clipping), patch extraction for the
// vision patch-embed GEMM, product-quantised codebook gather / scatter, and grouped argmax.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <float.h>
#include <stdint.h>

#include "yv_ops.h"

namespace yv {

namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
  return v;
}

__device__ __forceinline__ float ld_any(const void* p, int dtype, int64_t i) {
  return dtype == 1 ? reinterpret_cast<const float*>(p)[i]
                    : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}

__device__ __forceinline__ void st_any(void* p, int dtype, int64_t i, float v) {
  if (dtype == 1) reinterpret_cast<float*>(p)[i] = v;
  else reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16(v);
}

// ---------------------------------------------------------------------------------------------
// Cross-entropy: one block per row.  Pass 1: online max / sum-exp.  Pass 2: gradient.
// ---------------------------------------------------------------------------------------------
__global__ void ce_kernel(const float* __restrict__ logits, const int64_t* __restrict__ labels,
                          float* __restrict__ loss, __nv_bfloat16* __restrict__ dlogits, int V, int64_t ld,
                          int ignore_index, float grad_scale) {
  __shared__ float s_m[32], s_s[32];
  __shared__ float s_max, s_lse;
  const int64_t row = blockIdx.x;
  const float* lr = logits + row * ld;
  const int64_t label = labels[row];
  const bool valid = (label != ignore_index) && label >= 0 && label < V;
  float m = -FLT_MAX, s = 0.f;
  const int V4 = V >> 2;
  for (int i = threadIdx.x; i < V4; i += blockDim.x) {
    const float4 v = reinterpret_cast<const float4*>(lr)[i];
    const float mm = fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w));
    if (mm > m) { s *= __expf(m - mm); m = mm; }
    s += __expf(v.x - m) + __expf(v.y - m) + __expf(v.z - m) + __expf(v.w - m);
  }
  for (int i = (V4 << 2) + threadIdx.x; i < V; i += blockDim.x) {
    const float v = lr[i];
    if (v > m) { s *= __expf(m - v); m = v; }
    s += __expf(v - m);
  }
  // combine (m, s) pairs
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float om = __shfl_xor_sync(0xFFFFFFFFu, m, o);
    const float os = __shfl_xor_sync(0xFFFFFFFFu, s, o);
    const float nm = fmaxf(m, om);
    s = s * __expf(m - nm) + os * __expf(om - nm);
    m = nm;
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { s_m[warp] = m; s_s[warp] = s; }
  __syncthreads();
  if (warp == 0) {
    const int nw = blockDim.x >> 5;
    m = lane < nw ? s_m[lane] : -FLT_MAX;
    s = lane < nw ? s_s[lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float om = __shfl_xor_sync(0xFFFFFFFFu, m, o);
      const float os = __shfl_xor_sync(0xFFFFFFFFu, s, o);
      const float nm = fmaxf(m, om);
      s = s * __expf(m - nm) + os * __expf(om - nm);
      m = nm;
    }
    if (lane == 0) { s_max = m; s_lse = m + logf(s); }
  }
  __syncthreads();
  const float lse = s_lse;
  if (threadIdx.x == 0) loss[row] = valid ? (lse - lr[label]) : 0.f;
  if (dlogits == nullptr) return;
  __nv_bfloat16* dr = dlogits + row * static_cast<int64_t>(V);
  const float gs = valid ? grad_scale : 0.f;
  const int V2 = V >> 1;
  for (int i = threadIdx.x; i < V2; i += blockDim.x) {
    const float2 v = reinterpret_cast<const float2*>(lr)[i];
    float a = __expf(v.x - lse), b = __expf(v.y - lse);
    if (2 * i == label) a -= 1.f;
    if (2 * i + 1 == label) b -= 1.f;
    reinterpret_cast<__nv_bfloat162*>(dr)[i] = __floats2bfloat162_rn(a * gs, b * gs);
  }
  if ((V & 1) && threadIdx.x == 0) {
    float a = __expf(lr[V - 1] - lse);
    if (V - 1 == label) a -= 1.f;
    dr[V - 1] = __float2bfloat16(a * gs);
  }
}

// ---------------------------------------------------------------------------------------------
// AdamW with the decay applied to the pre-update parameter:
//   p <- p - lr * ( m_hat / (sqrt(v_hat) + eps) + wd * p )
// ---------------------------------------------------------------------------------------------
__global__ void adamw_kernel(AdamWArgs a) {
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < a.n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const float g = ld_any(a.g, a.g_dtype, i) * a.grad_scale;
    const float p = ld_any(a.p, a.p_dtype, i);
    float m = ld_any(a.m, a.s_dtype, i);
    float v = ld_any(a.v, a.s_dtype, i);
    m = a.beta1 * m + (1.f - a.beta1) * g;
    v = a.beta2 * v + (1.f - a.beta2) * g * g;
    const float mh = m / a.bc1;
    const float vh = v / a.bc2;
    const float np = p - a.lr * (mh / (sqrtf(vh) + a.eps) + a.wd * p);
    st_any(a.p, a.p_dtype, i, np);
    st_any(a.m, a.s_dtype, i, m);
    st_any(a.v, a.s_dtype, i, v);
  }
}

// Eight bf16 values per 16-byte access: the optimizer's streaming kernels below move tens of GB per step and are
// bound by memory, which 2-byte accesses per thread do not saturate.  Rounding is the same as in the scalar kernels.
__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 t = __bfloat1622float2(h[j]);
    f[2 * j] = t.x;
    f[2 * j + 1] = t.y;
  }
}

__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 u;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(f[2 * j], f[2 * j + 1]);
  return u;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// vector form of momentum_kernel over nvec = n / 8 vectors (the launcher runs the scalar kernel on the tail)
__global__ void momentum_vec_kernel(uint4* __restrict__ m, const uint4* __restrict__ g, uint4* __restrict__ out,
                                    int64_t nvec, float mu, float gscale, int nesterov, int first_fold) {
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    float gv[8], mv[8], ov[8];
    unpack8(g[i], gv);
    unpack8(m[i], mv);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      gv[j] *= gscale;
      if (first_fold) mv[j] *= mu;
      mv[j] += gv[j];
    }
    const uint4 packed = pack8(mv);
    m[i] = packed;
    if (out != nullptr) {
      if (nesterov) {
#pragma unroll
        for (int j = 0; j < 8; ++j) ov[j] = gv[j] + mu * mv[j];      // unrounded momentum, as in the scalar kernel
        out[i] = pack8(ov);
      } else {
        out[i] = packed;
      }
    }
  }
}

__global__ void muon_apply_vec_kernel(uint4* __restrict__ p, const uint4* __restrict__ u, int64_t nvec, float lr,
                                      float wd, float scale) {
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    float pv[8], uv[8];
    unpack8(p[i], pv);
    unpack8(u[i], uv);
#pragma unroll
    for (int j = 0; j < 8; ++j) pv[j] = pv[j] * (1.f - lr * wd) - lr * scale * uv[j];
    p[i] = pack8(pv);
  }
}

// ---- block-quantised momentum: int8 values with one fp32 scale per 128 consecutive elements ----------------------
// 32-bit mix of an element index and a per-call seed (the finaliser of MurmurHash3): the uniform variate of the
// stochastic rounding.  The same (seed, index) always rounds the same way, so a run is reproducible.
__device__ __forceinline__ uint32_t hash_u32(uint32_t x) {
  x ^= x >> 16; x *= 0x85ebca6bu; x ^= x >> 13; x *= 0xc2b2ae35u; x ^= x >> 16;
  return x;
}

// m <- (first_fold ? mu * m : m) + gscale * g on a quantised m.  Sixteen lanes own one 128-element block (8 elements
// each: one 8-byte load of q, one 16-byte load of g); the block's new absolute maximum is reduced over the half-warp
// and the values are re-quantised with stochastic rounding, which keeps the accumulated momentum unbiased over the
// many folds of a step (round-to-nearest would drop every contribution below half a quantisation step).
__global__ void momentum_q8_kernel(int8_t* __restrict__ q, float* __restrict__ scale, const __nv_bfloat16* __restrict__ g,
                                   int64_t nblocks, float mu, float gscale, int first_fold, uint32_t seed) {
  const int lane16 = threadIdx.x & 15;
  const int64_t hw = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 4;     // half-warp index
  const int64_t nhw = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 4;
  // every lane of a warp runs the same number of iterations (the shuffles below need all 32 lanes)
  const int64_t iters = (nblocks + nhw - 1) / nhw;
  for (int64_t it = 0; it < iters; ++it) {
    const int64_t b = hw + it * nhw;
    const bool live = b < nblocks;
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = 0.f;
    const int64_t e0 = b * 128 + lane16 * 8;
    if (live) {
      const float sc = scale[b] * (first_fold ? mu : 1.f);
      const uint2 qraw = *reinterpret_cast<const uint2*>(q + e0);
      const int8_t* qb = reinterpret_cast<const int8_t*>(&qraw);
      float gv[8];
      unpack8(*reinterpret_cast<const uint4*>(g + e0), gv);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = static_cast<float>(qb[j]) * sc + gv[j] * gscale;
    }
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[j]));
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if (live) {
      const float ns = amax > 0.f ? amax * (1.f / 127.f) : 1.f;
      const float inv256 = 256.f / ns;
      // Stochastic rounding in fixed point: t = round(v / ns * 256) carries 8 fractional bits, a uniform byte is
      // added and the arithmetic shift by 8 is the floor.  Two hashes per thread supply the eight bytes (1/256
      // resolution bounds the rounding bias at 1/512 of a quantisation step).  |v / ns| <= 127, so the result is
      // within [-127, 127] without clamping.
      const uint32_t key = static_cast<uint32_t>(e0 >> 3) * 0x9e3779b9u ^ static_cast<uint32_t>(e0 >> 35) ^ seed;
      const uint32_t r0 = hash_u32(key), r1 = hash_u32(key ^ 0x68bc21ebu);
      uint32_t lo = 0u, hi = 0u;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int a = (__float2int_rn(v[j] * inv256) + static_cast<int>((r0 >> (8 * j)) & 0xffu)) >> 8;
        const int b = (__float2int_rn(v[j + 4] * inv256) + static_cast<int>((r1 >> (8 * j)) & 0xffu)) >> 8;
        lo |= (static_cast<uint32_t>(a) & 0xffu) << (8 * j);
        hi |= (static_cast<uint32_t>(b) & 0xffu) << (8 * j);
      }
      const uint2 out = make_uint2(lo, hi);
      *reinterpret_cast<uint2*>(q + e0) = out;
      if (lane16 == 0) scale[b] = ns;
    }
  }
}

// out (bf16) <- q * scale, eight elements per thread
__global__ void dequant_q8_kernel(const int8_t* __restrict__ q, const float* __restrict__ scale,
                                  __nv_bfloat16* __restrict__ out, int64_t nvec) {
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const float sc = scale[i >> 4];
    const uint2 qraw = *reinterpret_cast<const uint2*>(q + i * 8);
    const int8_t* qb = reinterpret_cast<const int8_t*>(&qraw);
    float f[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = static_cast<float>(qb[j]) * sc;
    reinterpret_cast<uint4*>(out)[i] = pack8(f);
  }
}

// m <- (first_fold ? mu * m : m) + gscale * g ;   out <- nesterov ? gscale*g + mu*m : m   (out optional)
__global__ void momentum_kernel(__nv_bfloat16* __restrict__ m, const __nv_bfloat16* __restrict__ g,
                                __nv_bfloat16* __restrict__ out, int64_t n, float mu, float gscale, int nesterov,
                                int first_fold) {
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const float gv = __bfloat162float(g[i]) * gscale;
    float mv = __bfloat162float(m[i]);
    if (first_fold) mv *= mu;
    mv += gv;
    m[i] = __float2bfloat16(mv);
    if (out != nullptr) out[i] = __float2bfloat16(nesterov ? gv + mu * mv : mv);
  }
}

__global__ void muon_apply_kernel(__nv_bfloat16* __restrict__ p, const __nv_bfloat16* __restrict__ u, int64_t n,
                                  float lr, float wd, float scale) {
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const float pv = __bfloat162float(p[i]);
    p[i] = __float2bfloat16(pv * (1.f - lr * wd) - lr * scale * __bfloat162float(u[i]));
  }
}

// grid (chunks, batch): partial sums of squares per matrix accumulated with atomics into norms[batch]
__global__ void frob_sumsq_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ norms,
                                  int64_t per_matrix) {
  const __nv_bfloat16* xm = x + static_cast<int64_t>(blockIdx.y) * per_matrix;
  float s = 0.f;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < per_matrix;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const float v = __bfloat162float(xm[i]);
    s += v * v;
  }
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) atomicAdd(&norms[blockIdx.y], s);
}

__global__ void frob_scale_kernel(__nv_bfloat16* __restrict__ x, const float* __restrict__ norms,
                                  int64_t per_matrix, float eps) {
  __nv_bfloat16* xm = x + static_cast<int64_t>(blockIdx.y) * per_matrix;
  const float inv = 1.f / fmaxf(sqrtf(norms[blockIdx.y]), eps);
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < per_matrix;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    xm[i] = __float2bfloat16(__bfloat162float(xm[i]) * inv);
  }
}

// vector forms of the two Frobenius kernels (per_matrix a multiple of 8, x 16-byte aligned)
__global__ void frob_sumsq_vec_kernel(const uint4* __restrict__ x, float* __restrict__ norms, int64_t vec_per_matrix) {
  const uint4* xm = x + static_cast<int64_t>(blockIdx.y) * vec_per_matrix;
  float s = 0.f;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < vec_per_matrix;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    float v[8];
    unpack8(xm[i], v);
#pragma unroll
    for (int j = 0; j < 8; ++j) s += v[j] * v[j];
  }
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) atomicAdd(&norms[blockIdx.y], s);
}

__global__ void frob_scale_vec_kernel(uint4* __restrict__ x, const float* __restrict__ norms, int64_t vec_per_matrix,
                                      float eps) {
  uint4* xm = x + static_cast<int64_t>(blockIdx.y) * vec_per_matrix;
  const float inv = 1.f / fmaxf(sqrtf(norms[blockIdx.y]), eps);
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < vec_per_matrix;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    float v[8];
    unpack8(xm[i], v);
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] *= inv;
    xm[i] = pack8(v);
  }
}

__global__ void axpby_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ y,
                             __nv_bfloat16* __restrict__ out, int64_t n, float a, float b) {
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    out[i] = __float2bfloat16(a * __bfloat162float(x[i]) + b * __bfloat162float(y[i]));
  }
}

// out[g] = a * I + b * A[g] + c * A2[g] for a batch of n x n matrices (Newton-Schulz polynomial on the Gram side)
__global__ void ns_poly_kernel(const __nv_bfloat16* __restrict__ A, const __nv_bfloat16* __restrict__ A2,
                               __nv_bfloat16* __restrict__ out, int64_t total, int n, float a, float b, float c) {
  const int64_t nn = static_cast<int64_t>(n) * n;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i % nn;
    const float diag = (r / n == r % n) ? a : 0.f;
    out[i] = __float2bfloat16(diag + b * __bfloat162float(A[i]) + c * __bfloat162float(A2[i]));
  }
}

__global__ void sumsq_kernel(const void* __restrict__ x, int dtype, int64_t n, float* __restrict__ out) {
  float s = 0.f;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const float v = ld_any(x, dtype, i);
    s += v * v;
  }
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) atomicAdd(out, s);
}

__global__ void scale_kernel(void* __restrict__ x, int dtype, int64_t n, const float* __restrict__ scale_dev,
                             float scale_host) {
  const float sc = scale_host * (scale_dev != nullptr ? *scale_dev : 1.f);
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    st_any(x, dtype, i, ld_any(x, dtype, i) * sc);
  }
}

// ---------------------------------------------------------------------------------------------
// Patch extraction: img [B, C, H, W] -> rows [B * gh * gw, Kpad] bf16, column = c*P*P + py*P + px,
// normalised per channel, zero padded to Kpad (a multiple of 64 so the GEMM K loop is whole).
// ---------------------------------------------------------------------------------------------
__global__ void patchify_kernel(const void* __restrict__ img, int img_fp32, __nv_bfloat16* __restrict__ out, int C,
                                int H, int W, int P, int Kpad, const float* __restrict__ mean,
                                const float* __restrict__ stdv) {
  const int gw = W / P, gh = H / P;
  const int64_t patch = blockIdx.x;
  const int b = static_cast<int>(patch / (gh * gw));
  const int r = static_cast<int>(patch % (gh * gw));
  const int py0 = (r / gw) * P, px0 = (r % gw) * P;
  const int K = C * P * P;
  for (int c = threadIdx.x; c < Kpad; c += blockDim.x) {
    float v = 0.f;
    if (c < K) {
      const int ch = c / (P * P), rem = c % (P * P);
      const int y = py0 + rem / P, x = px0 + rem % P;
      const int64_t off = ((static_cast<int64_t>(b) * C + ch) * H + y) * W + x;
      v = img_fp32 ? reinterpret_cast<const float*>(img)[off]
                   : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(img)[off]);
      if (mean != nullptr) v = (v - mean[ch]) / stdv[ch];
    }
    out[patch * Kpad + c] = __float2bfloat16(v);
  }
}

// ---------------------------------------------------------------------------------------------
// Product-quantised field: out[t] = sum_c table[c][idx[t,c]]   (one warp per token, D <= 256)
// ---------------------------------------------------------------------------------------------
__global__ void pq_gather_sum_kernel(const __nv_bfloat16* __restrict__ table, const int* __restrict__ idx,
                                     __nv_bfloat16* __restrict__ out, int64_t tokens, int C, int64_t N, int D,
                                     uint32_t* status) {
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  for (int64_t t = static_cast<int64_t>(blockIdx.x) * wpb + (threadIdx.x >> 5); t < tokens;
       t += static_cast<int64_t>(gridDim.x) * wpb) {
    for (int d = lane * 2; d < D; d += 64) {
      float a0 = 0.f, a1 = 0.f;
      for (int c = 0; c < C; ++c) {
        int64_t e = idx[t * C + c];
        if (e < 0 || e >= N) {
          if (status != nullptr) atomicOr(status, 8u);
          continue;
        }
        const __nv_bfloat162 v =
            *reinterpret_cast<const __nv_bfloat162*>(table + (static_cast<int64_t>(c) * N + e) * D + d);
        a0 += __low2float(v);
        a1 += __high2float(v);
      }
      *reinterpret_cast<__nv_bfloat162*>(out + t * D + d) = __floats2bfloat162_rn(a0, a1);
    }
  }
}

__global__ void pq_scatter_grad_kernel(const __nv_bfloat16* __restrict__ dout, const int* __restrict__ idx,
                                       float* __restrict__ dtable, int64_t tokens, int C, int64_t N, int D) {
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  for (int64_t t = static_cast<int64_t>(blockIdx.x) * wpb + (threadIdx.x >> 5); t < tokens;
       t += static_cast<int64_t>(gridDim.x) * wpb) {
    for (int d = lane; d < D; d += 32) {
      const float g = __bfloat162float(dout[t * D + d]);
      for (int c = 0; c < C; ++c) {
        const int64_t e = idx[t * C + c];
        if (e >= 0 && e < N) atomicAdd(&dtable[(static_cast<int64_t>(c) * N + e) * D + d], g);
      }
    }
  }
}

// argmax over `per_group` entries for each of `groups` groups of a row (one warp per (row, group))
__global__ void argmax_rows_kernel(const void* __restrict__ logits, int dtype, int* __restrict__ out, int64_t rows,
                                   int groups, int per_group) {
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  const int64_t total = rows * groups;
  for (int64_t w = static_cast<int64_t>(blockIdx.x) * wpb + (threadIdx.x >> 5); w < total;
       w += static_cast<int64_t>(gridDim.x) * wpb) {
    const int64_t base = w * per_group;
    float best = -FLT_MAX;
    int bi = 0x7FFFFFFF;
    for (int i = lane; i < per_group; i += 32) {
      const float v = ld_any(logits, dtype, base + i);
      if (v > best) { best = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xFFFFFFFFu, best, o);
      const int oi = __shfl_xor_sync(0xFFFFFFFFu, bi, o);
      if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    }
    if (lane == 0) out[w] = bi;
  }
}

inline int grid_for(int64_t work, int block, int cap = 148 * 16) {
  int64_t g = (work + block - 1) / block;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  return static_cast<int>(g);
}

}  // namespace

#define YV_BF(p) reinterpret_cast<const __nv_bfloat16*>(p)
#define YV_BFM(p) reinterpret_cast<__nv_bfloat16*>(p)

int launch_ce_fwd_bwd(const float* logits, const int64_t* labels, float* loss, void* dlogits_bf16, int64_t rows,
                      int V, int64_t ld, int ignore_index, float grad_scale, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if ((ld & 3) != 0 || (reinterpret_cast<uintptr_t>(logits) & 15u) != 0) return -1;
  ce_kernel<<<static_cast<unsigned>(rows), 1024, 0, stream>>>(logits, labels, loss, YV_BFM(dlogits_bf16), V, ld,
                                                              ignore_index, grad_scale);
  return static_cast<int>(cudaGetLastError());
}

int launch_adamw(const AdamWArgs& a, cudaStream_t stream) {
  if (a.n <= 0) return 0;
  adamw_kernel<<<grid_for(a.n, 256), 256, 0, stream>>>(a);
  return static_cast<int>(cudaGetLastError());
}

int launch_momentum(void* m, const void* g, void* out, int64_t n, float mu, float gscale, int nesterov,
                    int first_fold, cudaStream_t stream) {
  if (n <= 0) return 0;
  int64_t done = 0;
  if (n >= 8 && aligned16(m) && aligned16(g) && aligned16(out)) {
    const int64_t nvec = n / 8;
    momentum_vec_kernel<<<grid_for(nvec, 256), 256, 0, stream>>>(
        static_cast<uint4*>(m), static_cast<const uint4*>(g), static_cast<uint4*>(out), nvec, mu, gscale, nesterov,
        first_fold);
    done = nvec * 8;
  }
  if (done < n) {
    momentum_kernel<<<grid_for(n - done, 256), 256, 0, stream>>>(
        YV_BFM(m) + done, YV_BF(g) + done, out != nullptr ? YV_BFM(out) + done : nullptr, n - done, mu, gscale,
        nesterov, first_fold);
  }
  return static_cast<int>(cudaGetLastError());
}

int launch_momentum_q8(void* q, float* scale, const void* g, int64_t n, float mu, float gscale, int first_fold,
                       uint32_t seed, cudaStream_t stream) {
  if (n <= 0) return 0;
  if ((n & 127) != 0 || !aligned16(g) || (reinterpret_cast<uintptr_t>(q) & 7u) != 0) return -1;
  const int64_t nblocks = n >> 7;
  momentum_q8_kernel<<<grid_for(nblocks * 16, 256), 256, 0, stream>>>(
      static_cast<int8_t*>(q), scale, YV_BF(g), nblocks, mu, gscale, first_fold, seed);
  return static_cast<int>(cudaGetLastError());
}

int launch_dequant_q8(const void* q, const float* scale, void* out, int64_t n, cudaStream_t stream) {
  if (n <= 0) return 0;
  if ((n & 127) != 0 || !aligned16(out) || (reinterpret_cast<uintptr_t>(q) & 7u) != 0) return -1;
  dequant_q8_kernel<<<grid_for(n >> 3, 256), 256, 0, stream>>>(static_cast<const int8_t*>(q), scale, YV_BFM(out), n >> 3);
  return static_cast<int>(cudaGetLastError());
}

int launch_muon_apply(void* p, const void* u, int64_t n, float lr, float wd, float scale, cudaStream_t stream) {
  if (n <= 0) return 0;
  int64_t done = 0;
  if (n >= 8 && aligned16(p) && aligned16(u)) {
    const int64_t nvec = n / 8;
    muon_apply_vec_kernel<<<grid_for(nvec, 256), 256, 0, stream>>>(static_cast<uint4*>(p),
                                                                   static_cast<const uint4*>(u), nvec, lr, wd, scale);
    done = nvec * 8;
  }
  if (done < n)
    muon_apply_kernel<<<grid_for(n - done, 256), 256, 0, stream>>>(YV_BFM(p) + done, YV_BF(u) + done, n - done, lr, wd,
                                                                   scale);
  return static_cast<int>(cudaGetLastError());
}

int launch_frob_normalize(void* x, float* norms, int batch, int64_t per_matrix, float eps, cudaStream_t stream) {
  if (batch <= 0 || per_matrix <= 0) return 0;
  cudaMemsetAsync(norms, 0, sizeof(float) * batch, stream);
  if ((per_matrix & 7) == 0 && aligned16(x)) {
    const int64_t vpm = per_matrix / 8;
    // enough CTAs in total to fill the machine a few times over, whatever the batch
    int gx = grid_for(vpm, 256, batch >= 64 ? 32 : (148 * 8 + batch - 1) / batch);
    frob_sumsq_vec_kernel<<<dim3(gx, batch), 256, 0, stream>>>(static_cast<const uint4*>(x), norms, vpm);
    frob_scale_vec_kernel<<<dim3(gx, batch), 256, 0, stream>>>(static_cast<uint4*>(x), norms, vpm, eps);
    return static_cast<int>(cudaGetLastError());
  }
  int gx = grid_for(per_matrix, 256, 64);
  frob_sumsq_kernel<<<dim3(gx, batch), 256, 0, stream>>>(YV_BF(x), norms, per_matrix);
  frob_scale_kernel<<<dim3(gx, batch), 256, 0, stream>>>(YV_BFM(x), norms, per_matrix, eps);
  return static_cast<int>(cudaGetLastError());
}

int launch_axpby(const void* x, const void* y, void* out, int64_t n, float a, float b, cudaStream_t stream) {
  if (n <= 0) return 0;
  axpby_kernel<<<grid_for(n, 256), 256, 0, stream>>>(YV_BF(x), YV_BF(y), YV_BFM(out), n, a, b);
  return static_cast<int>(cudaGetLastError());
}

int launch_ns_poly(const void* A, const void* A2, void* out, int64_t batch, int n, float a, float b, float c,
                   cudaStream_t stream) {
  const int64_t total = batch * static_cast<int64_t>(n) * n;
  if (total <= 0) return 0;
  ns_poly_kernel<<<grid_for(total, 256), 256, 0, stream>>>(YV_BF(A), YV_BF(A2), YV_BFM(out), total, n, a, b, c);
  return static_cast<int>(cudaGetLastError());
}

int launch_sumsq(const void* x, int dtype, int64_t n, float* out_accum, cudaStream_t stream) {
  if (n <= 0) return 0;
  sumsq_kernel<<<grid_for(n, 256, 148 * 4), 256, 0, stream>>>(x, dtype, n, out_accum);
  return static_cast<int>(cudaGetLastError());
}

int launch_scale(void* x, int dtype, int64_t n, const float* scale_dev, float scale_host, cudaStream_t stream) {
  if (n <= 0) return 0;
  scale_kernel<<<grid_for(n, 256), 256, 0, stream>>>(x, dtype, n, scale_dev, scale_host);
  return static_cast<int>(cudaGetLastError());
}

int launch_patchify(const void* img, int img_fp32, void* out, int B, int C, int H, int W, int P, int Kpad,
                    const float* mean, const float* stdv, cudaStream_t stream) {
  if (H % P != 0 || W % P != 0 || Kpad < C * P * P) return -1;
  const int64_t patches = static_cast<int64_t>(B) * (H / P) * (W / P);
  if (patches <= 0) return 0;
  patchify_kernel<<<static_cast<unsigned>(patches), 128, 0, stream>>>(img, img_fp32, YV_BFM(out), C, H, W, P, Kpad,
                                                                      mean, stdv);
  return static_cast<int>(cudaGetLastError());
}

int launch_pq_gather_sum(const void* table, const int* idx, void* out, int64_t tokens, int C, int64_t N, int D,
                         uint32_t* status, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if ((D & 1) != 0) return -1;
  pq_gather_sum_kernel<<<grid_for(tokens, 8), 256, 0, stream>>>(YV_BF(table), idx, YV_BFM(out), tokens, C, N, D,
                                                                status);
  return static_cast<int>(cudaGetLastError());
}

int launch_pq_scatter_grad(const void* dout, const int* idx, float* dtable, int64_t tokens, int C, int64_t N, int D,
                           cudaStream_t stream) {
  if (tokens <= 0) return 0;
  pq_scatter_grad_kernel<<<grid_for(tokens, 8), 256, 0, stream>>>(YV_BF(dout), idx, dtable, tokens, C, N, D);
  return static_cast<int>(cudaGetLastError());
}

int launch_argmax_rows(const void* logits, int dtype, int* out, int64_t rows, int groups, int per_group,
                       cudaStream_t stream) {
  if (rows <= 0) return 0;
  argmax_rows_kernel<<<grid_for(rows * groups, 8), 256, 0, stream>>>(logits, dtype, out, rows, groups, per_group);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace yv
