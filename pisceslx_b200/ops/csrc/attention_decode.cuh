// Paged-KV decode attention (one new query token per sequence) and the KV-cache append kernel.
//
// Decode is bandwidth bound: every key/value byte is read once and used by the G query heads that share
// the KV head, so the math runs on the CUDA cores.  grid = (kv heads, sequences, splits); 128 threads =
// 16 groups of 8 lanes; a group owns one key per step, a lane owns D/8 contiguous dims of it.  Each CTA
// writes an unnormalised partial (max, sum, out) per query head to scratch; a second kernel merges splits.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "sm100.cuh"

namespace yv {

struct PagedDecodeParams {
  const __nv_bfloat16* q;          // [B, hq, D]
  const __nv_bfloat16* k_cache;    // [num_blocks, block, hk, D]
  const __nv_bfloat16* v_cache;
  const int* block_table;          // [B, max_blocks_per_seq]
  const int* seq_lens;             // [B]
  __nv_bfloat16* o;                // [B, hq, D]
  float* partial_o;                // [B, hq, splits, D]
  float* partial_ml;               // [B, hq, splits, 2]
  int hq, hk, block, max_blocks_per_seq, splits, num_blocks;
  float scale_log2;
  uint32_t* status;
};

// Sequence length of batch row b, clamped to what its block-table row can describe.  A longer length would walk past
// the row (into the next sequence's table or out of the tensor): it is cut to the row's capacity and reported.
__device__ __forceinline__ int decode_seq_len(const PagedDecodeParams& p, int b) {
  int n = p.seq_lens[b];
  const int64_t cap = static_cast<int64_t>(p.max_blocks_per_seq) * p.block;
  if (n < 0 || n > cap) {
    if (p.status != nullptr && threadIdx.x == 0) atomicOr(p.status, kStatusIndexOutOfRange);
    n = n < 0 ? 0 : static_cast<int>(cap);
  }
  return n;
}

// Merge of the 16 key groups of a CTA (each group holds a running max / sum / accumulator for its keys) into the
// split's partial result in scratch.  Shared by the direct-load and the TMA-fed kernels; every thread of the CTA
// calls it (it synchronises the CTA).
template <int D, int G>
__device__ __forceinline__ void decode_merge_groups(const PagedDecodeParams& p, const float (&m)[G], const float (&l)[G],
                                                    const float (&acc)[G][D / 8], int b, int kvh, int split,
                                                    float (*s_red_o)[G][D / 8 + 1], float (*s_m)[G], float (*s_l)[G]) {
  constexpr int EPL = D / 8;
  const int tid = threadIdx.x;
  const int grp = tid >> 3, sub = tid & 7;
  // merge the 16 key groups of the CTA
  if (sub == 0) {
#pragma unroll
    for (int g = 0; g < G; ++g) { s_m[grp][g] = m[g]; s_l[grp][g] = l[g]; }
  }
  __syncthreads();
  float mg[G], scale_me[G];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    float mm = -1.0e29f;
    for (int r = 0; r < 16; ++r) mm = fmaxf(mm, s_m[r][g]);
    mg[g] = mm;
    scale_me[g] = exp2f(m[g] - mm);
  }
  // each lane slice (sub) is reduced over groups through shared memory, one slice at a time
  for (int s = 0; s < 8; ++s) {
    if (sub == s) {
#pragma unroll
      for (int g = 0; g < G; ++g)
#pragma unroll
        for (int e = 0; e < EPL; ++e) s_red_o[grp][g][e] = acc[g][e] * scale_me[g];
    }
    __syncthreads();
    for (int i = tid; i < G * EPL; i += 128) {
      const int g = i / EPL, e = i % EPL;
      float t = 0.f;
      for (int r = 0; r < 16; ++r) t += s_red_o[r][g][e];
      const int64_t base = ((static_cast<int64_t>(b) * p.hq + kvh * G + g) * p.splits + split);
      p.partial_o[base * D + s * EPL + e] = t;
    }
    __syncthreads();
  }
  if (tid < G) {
    const int g = tid;
    float lt = 0.f;
    for (int r = 0; r < 16; ++r) lt += s_l[r][g] * exp2f(s_m[r][g] - mg[g]);
    const int64_t base = ((static_cast<int64_t>(b) * p.hq + kvh * G + g) * p.splits + split);
    p.partial_ml[base * 2] = mg[g];
    p.partial_ml[base * 2 + 1] = lt;
  }
}

template <int D, int G>
__global__ void __launch_bounds__(128) paged_decode_kernel(const PagedDecodeParams p) {
  constexpr int EPL = D / 8;                       // elements per lane
  __shared__ float s_q[G][D];
  __shared__ float s_red_o[16][G][D / 8 + 1];      // reused per d-slice pass (see merge below)
  __shared__ float s_m[16][G], s_l[16][G];
  const int kvh = blockIdx.x, b = blockIdx.y, split = blockIdx.z;
  const int tid = threadIdx.x;
  const int grp = tid >> 3, sub = tid & 7;
  const int seq_len = decode_seq_len(p, b);
  // keys of this split: whole cache blocks
  const int n_blocks = (seq_len + p.block - 1) / p.block;
  const int blocks_per_split = (n_blocks + p.splits - 1) / p.splits;
  const int blk0 = split * blocks_per_split;
  const int blk1 = min(n_blocks, blk0 + blocks_per_split);

  for (int i = tid; i < G * D; i += 128) {
    const int g = i / D, d = i % D;
    s_q[g][d] = __bfloat162float(p.q[(static_cast<int64_t>(b) * p.hq + kvh * G + g) * D + d]) * p.scale_log2;
  }
  __syncthreads();

  float m[G], l[G], acc[G][EPL];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m[g] = -1.0e29f;
    l[g] = 0.f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) acc[g][e] = 0.f;
  }

  for (int blk = blk0; blk < blk1; ++blk) {
    const int phys = p.block_table[static_cast<int64_t>(b) * p.max_blocks_per_seq + blk];
    if (phys < 0 || phys >= p.num_blocks) {
      if (p.status != nullptr && tid == 0) atomicOr(p.status, kStatusIndexOutOfRange);
      continue;
    }
    const int in_blk = min(p.block, seq_len - blk * p.block);
    for (int t0 = 0; t0 < in_blk; t0 += 16) {
      const int t = t0 + grp;
      const bool live = t < in_blk;
      float kf[EPL], vf[EPL];
      if (live) {
        const int64_t off = ((static_cast<int64_t>(phys) * p.block + t) * p.hk + kvh) * D + sub * EPL;
#pragma unroll
        for (int e = 0; e < EPL; e += 8) {
          const uint4 kr = *reinterpret_cast<const uint4*>(p.k_cache + off + e);
          const uint4 vr = *reinterpret_cast<const uint4*>(p.v_cache + off + e);
          const __nv_bfloat162* k2 = reinterpret_cast<const __nv_bfloat162*>(&kr);
          const __nv_bfloat162* v2 = reinterpret_cast<const __nv_bfloat162*>(&vr);
#pragma unroll
          for (int x = 0; x < 4; ++x) {
            const float2 a = __bfloat1622float2(k2[x]);
            const float2 c = __bfloat1622float2(v2[x]);
            kf[e + 2 * x] = a.x; kf[e + 2 * x + 1] = a.y;
            vf[e + 2 * x] = c.x; vf[e + 2 * x + 1] = c.y;
          }
        }
      }
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float s = 0.f;
        if (live) {
#pragma unroll
          for (int e = 0; e < EPL; ++e) s += kf[e] * s_q[g][sub * EPL + e];
        }
        s += __shfl_xor_sync(0xFFFFFFFFu, s, 1);
        s += __shfl_xor_sync(0xFFFFFFFFu, s, 2);
        s += __shfl_xor_sync(0xFFFFFFFFu, s, 4);
        if (live) {
          const float mn = fmaxf(m[g], s);
          const float alpha = exp2f(m[g] - mn);
          const float pr = exp2f(s - mn);
          l[g] = l[g] * alpha + pr;
#pragma unroll
          for (int e = 0; e < EPL; ++e) acc[g][e] = acc[g][e] * alpha + pr * vf[e];
          m[g] = mn;
        }
      }
    }
  }

  decode_merge_groups<D, G>(p, m, l, acc, b, kvh, split, s_red_o, s_m, s_l);
}

// merge splits: one warp per (sequence, query head)
template <int D>
__global__ void paged_decode_merge_kernel(const float* __restrict__ partial_o, const float* __restrict__ partial_ml,
                                          __nv_bfloat16* __restrict__ o, int64_t heads_total, int splits) {
  const int lane = threadIdx.x & 31;
  const int64_t w = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (w >= heads_total) return;
  float mm = -1.0e29f;
  for (int s = 0; s < splits; ++s) mm = fmaxf(mm, partial_ml[(w * splits + s) * 2]);
  float lt = 0.f;
  for (int s = 0; s < splits; ++s) lt += partial_ml[(w * splits + s) * 2 + 1] * exp2f(partial_ml[(w * splits + s) * 2] - mm);
  const float inv = lt > 0.f ? 1.f / lt : 0.f;
  for (int d = lane; d < D; d += 32) {
    float t = 0.f;
    for (int s = 0; s < splits; ++s)
      t += partial_o[(w * splits + s) * D + d] * exp2f(partial_ml[(w * splits + s) * 2] - mm);
    o[w * D + d] = __float2bfloat16(t * inv);
  }
}

// Append new K/V rows into the paged cache: slot = block_id * block + offset.
__global__ void kv_cache_write_kernel(const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
                                      __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache,
                                      const int* __restrict__ slot_map, int row_elems, int64_t k_stride,
                                      int64_t v_stride, int64_t num_slots, uint32_t* status) {
  const int64_t t = blockIdx.x;
  const int64_t slot = slot_map[t];
  if (slot < 0) return;                       // padding token
  if (slot >= num_slots) {
    if (status != nullptr && threadIdx.x == 0) atomicOr(status, kStatusIndexOutOfRange);
    return;
  }
  const int nvec = row_elems >> 3;
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    reinterpret_cast<uint4*>(k_cache + slot * row_elems)[i] = reinterpret_cast<const uint4*>(k + t * k_stride)[i];
    reinterpret_cast<uint4*>(v_cache + slot * row_elems)[i] = reinterpret_cast<const uint4*>(v + t * v_stride)[i];
  }
}

}  // namespace yv
