// Paged-KV decode attention fed by TMA.
//
// Same work split as paged_decode_kernel (grid = kv heads x sequences x splits, 128 threads = 16 key groups of 8
// lanes, one partial (max, sum, out) per query head and split), but the key/value bytes do not go through the
// threads' registers on their way from HBM: one thread issues a tiled bulk copy of a whole cache block (all `block`
// tokens of this KV head, K and V) into a ring of shared-memory stages, several blocks ahead of the block being
// consumed.  The copies of the next blocks are in flight while the current one is reduced, so the loop is no longer
// bound by the latency of dependent global loads.
//
// Shared memory per stage: K tile [block][D] and V tile [block][D], bf16, un-swizzled (a lane reads 16-byte pieces
// at a 32-byte stride inside a row: the eight lanes of a key cover all 32 banks once).
#pragma once
#include "attention_decode.cuh"

namespace yv {

struct PagedDecodeTmaParams {
  CUtensorMap tma_k;   // 3-D (d, kv head, token slot), box (D, 1, block), no swizzle
  CUtensorMap tma_v;
  PagedDecodeParams p;
};

constexpr int kDecodeStages = 3;

template <int D, int G>
__global__ void __launch_bounds__(128) paged_decode_tma_kernel(const __grid_constant__ PagedDecodeTmaParams pp) {
  const PagedDecodeParams& p = pp.p;
  constexpr int EPL = D / 8;                       // elements per lane
  constexpr int VEC = EPL / 8;                     // 16-byte pieces per lane per row
  constexpr int KPI = 4;                           // keys per group per step
  extern __shared__ uint8_t dsm_raw[];
  uint8_t* dsm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(dsm_raw) + 127) & ~uintptr_t(127));
  __shared__ float s_q[G][D];
  __shared__ float s_red_o[16][G][D / 8 + 1];
  __shared__ float s_m[16][G], s_l[16][G];
  __shared__ uint64_t full_bar[kDecodeStages];
  const int kvh = blockIdx.x, b = blockIdx.y, split = blockIdx.z;
  const int tid = threadIdx.x;
  const int grp = tid >> 3, sub = tid & 7;
  const int seq_len = decode_seq_len(p, b);
  const int n_blocks = (seq_len + p.block - 1) / p.block;
  const int blocks_per_split = (n_blocks + p.splits - 1) / p.splits;
  const int blk0 = split * blocks_per_split;
  const int blk1 = min(n_blocks, blk0 + blocks_per_split);
  const int n_tiles = blk1 > blk0 ? blk1 - blk0 : 0;
  const uint32_t tile_bytes = static_cast<uint32_t>(p.block) * D * 2;          // one K (or V) tile
  const int* table = p.block_table + static_cast<int64_t>(b) * p.max_blocks_per_seq;

  if (tid == 0) {
    tma_prefetch_desc(&pp.tma_k);
    tma_prefetch_desc(&pp.tma_v);
    for (int s = 0; s < kDecodeStages; ++s) mbar_init(&full_bar[s], 1);
    fence_barrier_init();
  }
  for (int i = tid; i < G * D; i += 128) {
    const int g = i / D, d = i % D;
    s_q[g][d] = __bfloat162float(p.q[(static_cast<int64_t>(b) * p.hq + kvh * G + g) * D + d]) * p.scale_log2;
  }
  __syncthreads();

  // one thread feeds the ring; a block whose table entry is out of range is reported and skipped by everybody
  auto issue = [&](int j) {
    const int s = j % kDecodeStages;
    const int phys = table[blk0 + j];
    if (phys < 0 || phys >= p.num_blocks) {
      if (p.status != nullptr) atomicOr(p.status, kStatusIndexOutOfRange);
      mbar_arrive(&full_bar[s]);
      return;
    }
    uint8_t* sk = dsm + static_cast<size_t>(s) * 2 * tile_bytes;
    mbar_expect_tx(&full_bar[s], 2 * tile_bytes);
    tma_load_3d(sk, &pp.tma_k, &full_bar[s], 0, kvh, phys * p.block);
    tma_load_3d(sk + tile_bytes, &pp.tma_v, &full_bar[s], 0, kvh, phys * p.block);
  };
  if (tid == 0) {
    const int pre = n_tiles < kDecodeStages ? n_tiles : kDecodeStages;
    for (int j = 0; j < pre; ++j) issue(j);
  }

  float m[G], l[G], acc[G][EPL];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m[g] = -1.0e29f;
    l[g] = 0.f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) acc[g][e] = 0.f;
  }

  for (int j = 0; j < n_tiles; ++j) {
    const int s = j % kDecodeStages;
    bool ok = mbar_wait(&full_bar[s], (j / kDecodeStages) & 1u, p.status);
    ok = __all_sync(0xFFFFFFFFu, ok);              // warp-uniform: the shuffles below run under `valid`
    const int phys = table[blk0 + j];
    const bool valid = ok && phys >= 0 && phys < p.num_blocks;
    if (valid) {
      const uint8_t* sk = dsm + static_cast<size_t>(s) * 2 * tile_bytes;
      const uint8_t* sv = sk + tile_bytes;
      const int in_blk = min(p.block, seq_len - (blk0 + j) * p.block);
      // trip count depends on the block size only: the full-mask shuffles below need warp-uniform control flow
      for (int t0 = 0; t0 < p.block; t0 += 16 * KPI) {
        bool live[KPI];
        float sc[KPI][G];
#pragma unroll
        for (int u = 0; u < KPI; ++u) {
          const int t = t0 + 16 * u + grp;
          live[u] = t < in_blk;
          float kf[EPL];
          const uint4* krow = reinterpret_cast<const uint4*>(sk + (static_cast<size_t>(t) * D + sub * EPL) * 2);
          if (live[u]) {
#pragma unroll
            for (int e = 0; e < VEC; ++e) {
              const uint4 kr = krow[e];
              const __nv_bfloat162* k2 = reinterpret_cast<const __nv_bfloat162*>(&kr);
#pragma unroll
              for (int x = 0; x < 4; ++x) {
                const float2 a = __bfloat1622float2(k2[x]);
                kf[e * 8 + 2 * x] = a.x;
                kf[e * 8 + 2 * x + 1] = a.y;
              }
            }
          }
#pragma unroll
          for (int g = 0; g < G; ++g) {
            float sdot = 0.f;
            if (live[u]) {
#pragma unroll
              for (int e = 0; e < EPL; ++e) sdot += kf[e] * s_q[g][sub * EPL + e];
            }
            sdot += __shfl_xor_sync(0xFFFFFFFFu, sdot, 1);
            sdot += __shfl_xor_sync(0xFFFFFFFFu, sdot, 2);
            sdot += __shfl_xor_sync(0xFFFFFFFFu, sdot, 4);
            sc[u][g] = live[u] ? sdot : -1.0e30f;
          }
        }
        float pr[KPI][G];
#pragma unroll
        for (int g = 0; g < G; ++g) {
          float mn = m[g];
#pragma unroll
          for (int u = 0; u < KPI; ++u) mn = fmaxf(mn, sc[u][g]);
          const float alpha = exp2f(m[g] - mn);
          float ps = 0.f;
#pragma unroll
          for (int u = 0; u < KPI; ++u) {
            pr[u][g] = live[u] ? exp2f(sc[u][g] - mn) : 0.f;
            ps += pr[u][g];
          }
          l[g] = l[g] * alpha + ps;
          m[g] = mn;
#pragma unroll
          for (int e = 0; e < EPL; ++e) acc[g][e] *= alpha;
        }
#pragma unroll
        for (int u = 0; u < KPI; ++u) {
          if (live[u]) {
            const int t = t0 + 16 * u + grp;
            const uint4* vrow = reinterpret_cast<const uint4*>(sv + (static_cast<size_t>(t) * D + sub * EPL) * 2);
#pragma unroll
            for (int e = 0; e < VEC; ++e) {
              const uint4 vr = vrow[e];
              const __nv_bfloat162* v2 = reinterpret_cast<const __nv_bfloat162*>(&vr);
#pragma unroll
              for (int x = 0; x < 4; ++x) {
                const float2 c = __bfloat1622float2(v2[x]);
#pragma unroll
                for (int g = 0; g < G; ++g) {
                  acc[g][e * 8 + 2 * x] += pr[u][g] * c.x;
                  acc[g][e * 8 + 2 * x + 1] += pr[u][g] * c.y;
                }
              }
            }
          }
        }
      }
    }
    // every thread is done with stage s (and agrees on whether a wait ran out) before it is refilled
    const int all_ok = __syncthreads_and(ok ? 1 : 0);
    if (!all_ok) {
      // a wait ran out: give the copies that may still be in flight time to land before this CTA's shared
      // memory can be handed to another CTA
      const uint64_t t0 = globaltimer_ns();
      while (globaltimer_ns() - t0 < 200000ull) { __nanosleep(1000); }
      break;
    }
    if (tid == 0 && j + kDecodeStages < n_tiles) issue(j + kDecodeStages);
  }
  decode_merge_groups<D, G>(p, m, l, acc, b, kvh, split, s_red_o, s_m, s_l);
}

}  // namespace yv
