// Mixture-of-experts routing kernels: gate (bias + softmax + top-k + renormalise + histogram), the
// dispatch plan (padded expert segments and the tile -> expert table the grouped GEMM reads), token
// permutation, weighted combine and their backward passes.  Nothing here synchronises with the host:
// every size the host needs is an upper bound known before launch.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <float.h>
#include <stdint.h>

#include "yv_ops.h"

namespace yv {

namespace {

constexpr int kMaxExpertsPerLane = 8;   // E <= 256
constexpr int kMaxTopK = 16;

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

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
  return v;
}

// ---------------------------------------------------------------------------------------------
// Gate: one warp per token.
//   sel = logits + bias                      (selection key)
//   p   = softmax(bias_in_combine ? sel : logits)
//   top-k of sel (ties -> lower expert id);  w = p_sel / sum(p_sel)   (renorm_mode 0)
//                                            w = softmax(p_sel)       (renorm_mode 1)
// ---------------------------------------------------------------------------------------------
__global__ void gate_topk_kernel(const float* __restrict__ logits, const float* __restrict__ bias,
                                 float* __restrict__ weights, int* __restrict__ idx, float* __restrict__ probs,
                                 int* __restrict__ counts, int64_t tokens, int E, int k, int bias_in_combine,
                                 int renorm_mode) {
  extern __shared__ int hist[];
  for (int e = threadIdx.x; e < E; e += blockDim.x) hist[e] = 0;
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  const int npl = (E + 31) >> 5;
  for (int64_t t = static_cast<int64_t>(blockIdx.x) * warps_per_block + (threadIdx.x >> 5); t < tokens;
       t += static_cast<int64_t>(gridDim.x) * warps_per_block) {
    float sel[kMaxExpertsPerLane], p[kMaxExpertsPerLane];
    float mx = -FLT_MAX;
#pragma unroll
    for (int i = 0; i < kMaxExpertsPerLane; ++i) {
      const int e = lane + 32 * i;
      sel[i] = -FLT_MAX;
      p[i] = -FLT_MAX;
      if (i < npl && e < E) {
        const float l = logits[t * E + e];
        const float b = (bias != nullptr) ? bias[e] : 0.f;
        sel[i] = l + b;
        p[i] = bias_in_combine ? sel[i] : l;
        mx = fmaxf(mx, p[i]);
      }
    }
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxExpertsPerLane; ++i) {
      const int e = lane + 32 * i;
      if (i < npl && e < E) {
        p[i] = __expf(p[i] - mx);
        sum += p[i];
      } else {
        p[i] = 0.f;
      }
    }
    sum = warp_sum(sum);
    const float inv = 1.f / sum;
#pragma unroll
    for (int i = 0; i < kMaxExpertsPerLane; ++i) {
      const int e = lane + 32 * i;
      p[i] *= inv;
      if (probs != nullptr && i < npl && e < E) probs[t * E + e] = p[i];
    }
    float wsel[kMaxTopK];
    int isel[kMaxTopK];
    float psum = 0.f, pmax = 0.f;
    for (int j = 0; j < k; ++j) {
      float best = -FLT_MAX;
      int best_e = 0x7FFFFFFF;
#pragma unroll
      for (int i = 0; i < kMaxExpertsPerLane; ++i) {
        const int e = lane + 32 * i;
        if (i < npl && e < E && (sel[i] > best)) { best = sel[i]; best_e = e; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xFFFFFFFFu, best, o);
        const int oe = __shfl_xor_sync(0xFFFFFFFFu, best_e, o);
        if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
      }
      // owner lane publishes the probability and retires the expert
      float pv = 0.f;
#pragma unroll
      for (int i = 0; i < kMaxExpertsPerLane; ++i) {
        if (lane + 32 * i == best_e) { pv = p[i]; sel[i] = -FLT_MAX; }
      }
      pv = __shfl_sync(0xFFFFFFFFu, pv, best_e & 31);
      isel[j] = best_e;
      wsel[j] = pv;
      psum += pv;
      pmax = fmaxf(pmax, pv);
    }
    if (renorm_mode == 1) {
      float s = 0.f;
      for (int j = 0; j < k; ++j) { wsel[j] = __expf(wsel[j] - pmax); s += wsel[j]; }
      for (int j = 0; j < k; ++j) wsel[j] /= s;
    } else {
      const float r = 1.f / fmaxf(psum, 1e-20f);
      for (int j = 0; j < k; ++j) wsel[j] *= r;
    }
    if (lane == 0) {
      for (int j = 0; j < k; ++j) {
        weights[t * k + j] = wsel[j];
        idx[t * k + j] = isel[j];
        atomicAdd(&hist[isel[j]], 1);
      }
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x)
    if (hist[e] != 0) atomicAdd(&counts[e], hist[e]);
}

// Backward of the gate for renorm_mode 0/1: dweights[T,k] -> dlogits[T,E].
__global__ void gate_topk_bwd_kernel(const float* __restrict__ dweights, const float* __restrict__ probs,
                                     const int* __restrict__ idx, const float* __restrict__ weights,
                                     float* __restrict__ dlogits, int64_t tokens, int E, int k, int renorm_mode) {
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  for (int64_t t = static_cast<int64_t>(blockIdx.x) * warps_per_block + (threadIdx.x >> 5); t < tokens;
       t += static_cast<int64_t>(gridDim.x) * warps_per_block) {
    // dp for the selected experts
    float dot = 0.f, psum = 0.f;
    for (int j = 0; j < k; ++j) {
      dot += dweights[t * k + j] * weights[t * k + j];
      psum += probs[t * E + idx[t * k + j]];
    }
    float inner = 0.f;   // sum_e dp_e * p_e
    for (int j = 0; j < k; ++j) {
      const int e = idx[t * k + j];
      const float w = weights[t * k + j];
      const float dp = (renorm_mode == 1) ? w * (dweights[t * k + j] - dot)
                                          : (dweights[t * k + j] - dot) / fmaxf(psum, 1e-20f);
      inner += dp * probs[t * E + e];
    }
    for (int e = lane; e < E; e += 32) {
      float dp = 0.f;
      for (int j = 0; j < k; ++j) {
        if (idx[t * k + j] == e) {
          const float w = weights[t * k + j];
          dp = (renorm_mode == 1) ? w * (dweights[t * k + j] - dot)
                                  : (dweights[t * k + j] - dot) / fmaxf(psum, 1e-20f);
        }
      }
      dlogits[t * E + e] = probs[t * E + e] * (dp - inner);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Dispatch plan (single block): pad every expert segment to a multiple of 128 rows.
// ---------------------------------------------------------------------------------------------
__global__ void moe_plan_kernel(const int* __restrict__ counts, int* __restrict__ seg_offsets,
                                int* __restrict__ tile_expert, int* __restrict__ num_m_tiles,
                                int* __restrict__ cursor, int E, int max_tiles) {
  // launched with 256 threads and E <= 256: thread e owns expert e; the padded sizes are scanned in shared memory
  __shared__ int s_off[257];
  __shared__ int s_scan[256];
  const int tid = threadIdx.x;
  s_scan[tid] = tid < E ? ((counts[tid] + 127) / 128) * 128 : 0;
  __syncthreads();
  for (int d = 1; d < 256; d <<= 1) {
    const int v = tid >= d ? s_scan[tid - d] : 0;
    __syncthreads();
    s_scan[tid] += v;
    __syncthreads();
  }
  if (tid == 0) s_off[0] = 0;
  if (tid < E) s_off[tid + 1] = s_scan[tid];
  __syncthreads();
  if (tid == 0) {
    const int tiles = s_off[E] / 128;
    *num_m_tiles = tiles < max_tiles ? tiles : max_tiles;
  }
  for (int e = tid; e <= E; e += blockDim.x) {
    seg_offsets[e] = s_off[e];
    if (e < E) cursor[e] = s_off[e];
  }
  if (tid < E) {
    const int t0 = s_off[tid] / 128, t1 = s_off[tid + 1] / 128;
    for (int t = t0; t < t1 && t < max_tiles; ++t) tile_expert[t] = tid;
  }
}

// One block per token: reserve a row in each selected expert's segment and copy the token row there.
__global__ void moe_permute_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ idx,
                                   int* __restrict__ cursor, int* __restrict__ row_map,
                                   __nv_bfloat16* __restrict__ xp, int k, int cols) {
  __shared__ int dest[kMaxTopK];
  const int64_t t = blockIdx.x;
  if (threadIdx.x < k) {
    const int e = idx[t * k + threadIdx.x];
    const int r = atomicAdd(&cursor[e], 1);
    dest[threadIdx.x] = r;
    row_map[t * k + threadIdx.x] = r;
  }
  __syncthreads();
  const int nvec = cols >> 3;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    const uint4 val = *reinterpret_cast<const uint4*>(x + t * cols + v * 8);
    for (int j = 0; j < k; ++j) *reinterpret_cast<uint4*>(xp + static_cast<int64_t>(dest[j]) * cols + v * 8) = val;
  }
}

// Deterministic variant of the row reservation: row_map is given (computed by a stable sort on the host
// framework side); only copies rows.
__global__ void moe_permute_mapped_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ row_map,
                                          __nv_bfloat16* __restrict__ xp, int k, int cols) {
  const int64_t t = blockIdx.x;
  const int nvec = cols >> 3;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    const uint4 val = *reinterpret_cast<const uint4*>(x + t * cols + v * 8);
    for (int j = 0; j < k; ++j)
      *reinterpret_cast<uint4*>(xp + static_cast<int64_t>(row_map[t * k + j]) * cols + v * 8) = val;
  }
}

// grid (E, chunks): zero the pad rows [seg + count, next seg) of expert e.
__global__ void moe_zero_pad_kernel(__nv_bfloat16* __restrict__ xp, const int* __restrict__ seg_offsets,
                                    const int* __restrict__ counts, int cols) {
  const int e = blockIdx.x;
  const int r0 = seg_offsets[e] + counts[e], r1 = seg_offsets[e + 1];
  const int nvec = cols >> 3;
  const int64_t total = static_cast<int64_t>(r1 - r0) * nvec;
  for (int64_t i = blockIdx.y * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.y) * blockDim.x) {
    const int64_t r = r0 + i / nvec;
    const int v = static_cast<int>(i % nvec);
    *reinterpret_cast<uint4*>(xp + r * cols + v * 8) = make_uint4(0u, 0u, 0u, 0u);
  }
}

__global__ void moe_combine_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ row_map,
                                   const float* __restrict__ weights, const __nv_bfloat16* __restrict__ add,
                                   __nv_bfloat16* __restrict__ out, int k, int cols) {
  const int64_t t = blockIdx.x;
  const int nvec = cols >> 3;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    float acc[8];
    if (add != nullptr) {
      load8(add + t * cols + v * 8, acc);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    }
    for (int j = 0; j < k; ++j) {
      const float w = weights[t * k + j];
      if (w != 0.f) {
        float r[8];
        load8(y + static_cast<int64_t>(row_map[t * k + j]) * cols + v * 8, r);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] += w * r[i];
      }
    }
    store8(out + t * cols + v * 8, acc);
  }
}

__global__ void moe_combine_bwd_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ y,
                                       const int* __restrict__ row_map, const float* __restrict__ weights,
                                       __nv_bfloat16* __restrict__ dy, float* __restrict__ dweights, int k,
                                       int cols) {
  __shared__ float red[kMaxTopK][33];
  const int64_t t = blockIdx.x;
  const int nvec = cols >> 3;
  float dots[kMaxTopK];
#pragma unroll
  for (int j = 0; j < kMaxTopK; ++j) dots[j] = 0.f;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    float g[8];
    load8(dout + t * cols + v * 8, g);
    for (int j = 0; j < k; ++j) {
      const int64_t r = row_map[t * k + j];
      const float w = weights[t * k + j];
      float yv[8], o[8];
      load8(y + r * cols + v * 8, yv);
      float d = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) { d += g[i] * yv[i]; o[i] = w * g[i]; }
      dots[j] += d;
      store8(dy + r * cols + v * 8, o);
    }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int j = 0; j < k; ++j) {
    const float s = warp_sum(dots[j]);
    if (lane == 0) red[j][warp] = s;
  }
  __syncthreads();
  if (threadIdx.x < k) {
    float s = 0.f;
    const int nw = blockDim.x >> 5;
    for (int w = 0; w < nw; ++w) s += red[threadIdx.x][w];
    dweights[t * k + threadIdx.x] = s;
  }
}

__global__ void moe_unpermute_sum_kernel(const __nv_bfloat16* __restrict__ dxp, const int* __restrict__ row_map,
                                         __nv_bfloat16* __restrict__ dx, int k, int cols) {
  const int64_t t = blockIdx.x;
  const int nvec = cols >> 3;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    for (int j = 0; j < k; ++j) {
      float r[8];
      load8(dxp + static_cast<int64_t>(row_map[t * k + j]) * cols + v * 8, r);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += r[i];
    }
    store8(dx + t * cols + v * 8, acc);
  }
}

__global__ void gate_bias_update_kernel(float* __restrict__ bias, const int* __restrict__ counts, int E, float rate,
                                        float clampv) {
  __shared__ float total;
  if (threadIdx.x == 0) {
    long long s = 0;
    for (int e = 0; e < E; ++e) s += counts[e];
    total = static_cast<float>(s > 0 ? s : 1);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    const float usage = static_cast<float>(counts[e]) / total;
    float b = bias[e] + rate * (1.f / static_cast<float>(E) - usage);
    bias[e] = fminf(fmaxf(b, -clampv), clampv);
  }
}

// ---------------------------------------------------------------------------------------------
// deterministic row map and capacity mask: one CTA per expert walks all assignments in order
// ---------------------------------------------------------------------------------------------
// Exclusive prefix of `flag` over the 256 threads of the CTA in thread order, and the CTA's total.
__device__ __forceinline__ int block_scan_flags(bool flag, int* s_warp, int& total) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const unsigned m = __ballot_sync(0xFFFFFFFFu, flag);
  if (lane == 0) s_warp[w] = __popc(m);
  __syncthreads();
  int before = 0, all = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int c = s_warp[i];
    before += i < w ? c : 0;
    all += c;
  }
  __syncthreads();
  total = all;
  return before + __popc(m & ((1u << lane) - 1u));
}

// row_map[a] = seg_offsets[e] + (number of earlier assignments of expert e), a = t * k + j in token order: the
// stable order a sort by expert would give, without the sort.  grid = E, block = 256.
__global__ void moe_rank_kernel(const int* __restrict__ idx, const int* __restrict__ seg_offsets,
                                int* __restrict__ row_map, int64_t n) {
  __shared__ int s_warp[8];
  const int e = blockIdx.x;
  int running = seg_offsets[e];
  for (int64_t base = 0; base < n; base += 256) {
    const int64_t a = base + threadIdx.x;
    const bool mine = a < n && idx[a] == e;
    int total;
    const int before = block_scan_flags(mine, s_warp, total);
    if (mine) row_map[a] = running + before;
    running += total;
  }
}

// keep[a] = 1 when assignment a is among the `capacity` highest routing probabilities of its expert (ties broken
// by token order), else 0.  An exact radix select over the probabilities' bit patterns (non-negative floats order
// like their bits) finds the threshold in four passes; a last ordered pass settles the ties.  grid = E, block = 256.
__global__ void moe_capacity_keep_kernel(const int* __restrict__ idx, const float* __restrict__ probs,
                                         const int* __restrict__ counts, uint8_t* __restrict__ keep, int64_t n, int k,
                                         int E, int capacity) {
  __shared__ int s_warp[8];
  __shared__ int s_hist[256];
  __shared__ unsigned s_prefix;
  __shared__ int s_remaining;
  const int e = blockIdx.x;
  const bool all_fit = counts[e] <= capacity;
  unsigned thr = 0u;
  int ties_kept = 0;
  if (!all_fit) {
    if (threadIdx.x == 0) { s_prefix = 0u; s_remaining = capacity; }
    __syncthreads();
    for (int pass = 3; pass >= 0; --pass) {
      s_hist[threadIdx.x] = 0;
      __syncthreads();
      const unsigned prefix = s_prefix;
      const unsigned hi_mask = pass == 3 ? 0u : (0xFFFFFFFFu << (8 * (pass + 1)));
      for (int64_t a = threadIdx.x; a < n; a += 256) {
        if (idx[a] != e) continue;
        const unsigned key = __float_as_uint(fmaxf(probs[(a / k) * E + e], 0.f));
        if ((key & hi_mask) == (prefix & hi_mask)) atomicAdd(&s_hist[(key >> (8 * pass)) & 0xFFu], 1);
      }
      __syncthreads();
      if (threadIdx.x == 0) {
        int rem = s_remaining, b = 255;
        for (; b > 0; --b) {
          if (s_hist[b] >= rem) break;
          rem -= s_hist[b];
        }
        s_remaining = rem;                       // how many of the chosen byte's group are still to be kept
        s_prefix = prefix | (static_cast<unsigned>(b) << (8 * pass));
      }
      __syncthreads();
    }
    thr = s_prefix;
    ties_kept = s_remaining;
  }
  int tie_running = 0;
  for (int64_t base = 0; base < n; base += 256) {
    const int64_t a = base + threadIdx.x;
    const bool mine = a < n && idx[a] == e;
    unsigned key = 0u;
    if (mine && !all_fit) key = __float_as_uint(fmaxf(probs[(a / k) * E + e], 0.f));
    const bool tie = mine && !all_fit && key == thr;
    int total;
    const int before = block_scan_flags(tie, s_warp, total);
    if (mine) keep[a] = (all_fit || key > thr || (tie && tie_running + before < ties_kept)) ? 1 : 0;
    tie_running += total;
  }
}

// weights[t, :] <- weights * keep, renormalised to sum 1 (all zero when every assignment of the token was dropped)
__global__ void moe_capacity_renorm_kernel(const float* __restrict__ w, const uint8_t* __restrict__ keep,
                                           float* __restrict__ out, int64_t tokens, int k) {
  const int64_t t = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  if (t >= tokens) return;
  float s = 0.f;
  for (int j = 0; j < k; ++j) s += keep[t * k + j] ? w[t * k + j] : 0.f;
  const float inv = s > 0.f ? 1.f / fmaxf(s, 1e-20f) : 0.f;
  for (int j = 0; j < k; ++j) out[t * k + j] = keep[t * k + j] ? w[t * k + j] * inv : 0.f;
}

}  // namespace

#define YV_BF(p) reinterpret_cast<const __nv_bfloat16*>(p)
#define YV_BFM(p) reinterpret_cast<__nv_bfloat16*>(p)

int launch_gate_topk(const float* logits, const float* bias, float* weights, int* idx, float* probs, int* counts,
                     int64_t tokens, int E, int k, int bias_in_combine, int renorm_mode, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (E > 32 * kMaxExpertsPerLane || k > kMaxTopK || k > E) return -1;
  const int block = 256;
  int64_t grid = (tokens + 7) / 8;
  if (grid > 148 * 8) grid = 148 * 8;
  gate_topk_kernel<<<static_cast<unsigned>(grid), block, E * sizeof(int), stream>>>(
      logits, bias, weights, idx, probs, counts, tokens, E, k, bias_in_combine, renorm_mode);
  return static_cast<int>(cudaGetLastError());
}

int launch_gate_topk_bwd(const float* dweights, const float* probs, const int* idx, const float* weights,
                         float* dlogits, int64_t tokens, int E, int k, int renorm_mode, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  int64_t grid = (tokens + 7) / 8;
  if (grid > 148 * 8) grid = 148 * 8;
  gate_topk_bwd_kernel<<<static_cast<unsigned>(grid), 256, 0, stream>>>(dweights, probs, idx, weights, dlogits,
                                                                        tokens, E, k, renorm_mode);
  return static_cast<int>(cudaGetLastError());
}

int launch_moe_plan(const int* counts, int* seg_offsets, int* tile_expert, int* num_m_tiles, int* cursor, int E,
                    int max_tiles, cudaStream_t stream) {
  if (E > 256) return -1;
  moe_plan_kernel<<<1, 256, 0, stream>>>(counts, seg_offsets, tile_expert, num_m_tiles, cursor, E, max_tiles);
  return static_cast<int>(cudaGetLastError());
}

int launch_moe_rank(const int* idx, const int* seg_offsets, int* row_map, int64_t n, int E, cudaStream_t stream) {
  if (n <= 0 || E <= 0) return 0;
  moe_rank_kernel<<<E, 256, 0, stream>>>(idx, seg_offsets, row_map, n);
  return static_cast<int>(cudaGetLastError());
}

int launch_moe_capacity_mask(const float* weights, const int* idx, const float* probs, const int* counts, uint8_t* keep,
                             float* out, int64_t tokens, int k, int E, int capacity, cudaStream_t stream) {
  if (tokens <= 0 || E <= 0) return 0;
  moe_capacity_keep_kernel<<<E, 256, 0, stream>>>(idx, probs, counts, keep, tokens * k, k, E, capacity);
  moe_capacity_renorm_kernel<<<static_cast<unsigned>((tokens + 255) / 256), 256, 0, stream>>>(weights, keep, out, tokens, k);
  return static_cast<int>(cudaGetLastError());
}

int launch_moe_permute(const void* x, const int* idx, int* cursor, int* row_map, void* xp, int64_t tokens, int k,
                       int cols, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if ((cols & 7) != 0 || k > kMaxTopK) return -1;
  const int block = (cols >> 3) >= 256 ? 256 : 128;
  if (cursor != nullptr) {
    moe_permute_kernel<<<static_cast<unsigned>(tokens), block, 0, stream>>>(YV_BF(x), idx, cursor, row_map,
                                                                            YV_BFM(xp), k, cols);
  } else {
    moe_permute_mapped_kernel<<<static_cast<unsigned>(tokens), block, 0, stream>>>(YV_BF(x), row_map, YV_BFM(xp), k,
                                                                                   cols);
  }
  return static_cast<int>(cudaGetLastError());
}

int launch_moe_zero_pad(void* xp, const int* seg_offsets, const int* counts, int E, int cols, cudaStream_t stream) {
  if ((cols & 7) != 0) return -1;
  moe_zero_pad_kernel<<<dim3(E, 4), 256, 0, stream>>>(YV_BFM(xp), seg_offsets, counts, cols);
  return static_cast<int>(cudaGetLastError());
}

int launch_moe_combine(const void* y, const int* row_map, const float* weights, const void* add, void* out,
                       int64_t tokens, int k, int cols, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if ((cols & 7) != 0) return -1;
  const int block = (cols >> 3) >= 256 ? 256 : 128;
  moe_combine_kernel<<<static_cast<unsigned>(tokens), block, 0, stream>>>(YV_BF(y), row_map, weights, YV_BF(add),
                                                                          YV_BFM(out), k, cols);
  return static_cast<int>(cudaGetLastError());
}

int launch_moe_combine_bwd(const void* dout, const void* y, const int* row_map, const float* weights, void* dy,
                           float* dweights, int64_t tokens, int k, int cols, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if ((cols & 7) != 0 || k > kMaxTopK) return -1;
  const int block = (cols >> 3) >= 256 ? 256 : 128;
  moe_combine_bwd_kernel<<<static_cast<unsigned>(tokens), block, 0, stream>>>(YV_BF(dout), YV_BF(y), row_map,
                                                                              weights, YV_BFM(dy), dweights, k,
                                                                              cols);
  return static_cast<int>(cudaGetLastError());
}

int launch_moe_unpermute_sum(const void* dxp, const int* row_map, void* dx, int64_t tokens, int k, int cols,
                             cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if ((cols & 7) != 0) return -1;
  const int block = (cols >> 3) >= 256 ? 256 : 128;
  moe_unpermute_sum_kernel<<<static_cast<unsigned>(tokens), block, 0, stream>>>(YV_BF(dxp), row_map, YV_BFM(dx), k,
                                                                                cols);
  return static_cast<int>(cudaGetLastError());
}

int launch_gate_bias_update(float* bias, const int* counts, int E, float rate, float clampv, cudaStream_t stream) {
  gate_bias_update_kernel<<<1, 256, 0, stream>>>(bias, counts, E, rate, clampv);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace yv
