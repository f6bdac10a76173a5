// Paged-KV decode attention on the tensor cores (head_dim 128, up to 16 query heads per KV head).
//
// A decode step has G = hq / hk real query rows per KV head, far below the 128-row UMMA tile, but the op is bound by
// the K/V bytes, not by FLOPs: padding the query-head dimension to N = 16 costs tensor-core time that stays well
// under the time the bytes take to arrive, and it removes the 2 * G * D fp32 FMAs per key that bound the CUDA-core
// kernels.  Keys are the M dimension:
//
//   S^T[128 keys, 16 heads]  = K_tile[128 keys, D] * Qpad[16, D]^T          (SS, K-major operands)
//   O^T[D = 128,  16 heads] += V_tile^T[D, 128 keys] * P[16 heads, 128 keys]^T   (SS, A MN-major = V as stored)
//
// grid = (kv heads, sequences, splits), 160 threads, one CTA per SM (three 64 KB K/V stages):
//   warps 0..3  softmax: thread t owns key t of the tile (TMEM lane t of S^T) and output dimension t (lane t of O^T);
//               the running max per head is kept identically by every thread, the running sum per warp
//   warp 4      one lane issues everything asynchronous: the TMA copies of the K/V ring (a tile is two cache blocks of
//               64 tokens, 128B swizzle), S^T one tile ahead into one of two TMEM buffers, and the P V product
// Hand-offs are mbarriers (TMA -> issuer, S^T done -> softmax, P ready -> issuer, P V done -> both); the softmax warps
// meet at ONE named barrier per tile (the exchange of the per-warp maxima).
// Output: unnormalised partial (max, sum, out) per query head and split, merged by paged_decode_merge_kernel.
#pragma once
#include "attention_decode.cuh"

namespace yv {

struct PagedDecodeMmaParams {
  CUtensorMap tma_k;   // 3-D (d, kv head, token slot), box (64, 1, 64), 128B swizzle
  CUtensorMap tma_v;
  PagedDecodeParams p;
};

constexpr int kDmStages = 3;
constexpr int kDmTileKeys = 128;
constexpr int kDmD = 128;
constexpr int kDmThreads = 160;
constexpr int kDmHalfBytes = kDmTileKeys * 128;             // [128 keys][64 d] bf16
constexpr int kDmTileBytes = 2 * kDmHalfBytes;              // K (or V) tile
constexpr int kDmStageBytes = 2 * kDmTileBytes;             // K + V
constexpr int kDmQBytes = 2 * 16 * 128;                     // Qpad [16][128 d] as two 64-d slabs
constexpr int kDmPBytes = 2 * 16 * 128;                     // P [16 heads][128 keys] as two 64-key slabs
constexpr int kDmSmem = kDmStages * kDmStageBytes + kDmQBytes + kDmPBytes + 1024;

// byte offset of element (row, col) in a K-major 128B-swizzled slab of 64 columns (rows of 128 bytes)
__device__ __forceinline__ uint32_t sw128_off(int row, int col) {
  return static_cast<uint32_t>(row * 128 + ((((col >> 3) ^ (row & 7)) << 4) | ((col & 7) << 1)));
}

// barrier over the 128 softmax threads with an AND reduction of `ok`
__device__ __forceinline__ bool softmax_barrier_and(bool ok) {
  uint32_t all_ok;
  asm volatile(
      "{\n"
      ".reg .pred pin, pout;\n"
      "setp.ne.u32 pin, %1, 0;\n"
      "bar.red.and.pred pout, 1, 128, pin;\n"
      "selp.u32 %0, 1, 0, pout;\n"
      "}\n"
      : "=r"(all_ok)
      : "r"(static_cast<uint32_t>(ok))
      : "memory");
  return all_ok != 0u;
}

template <int G>
__global__ void __launch_bounds__(kDmThreads, 1) paged_decode_mma_kernel(const __grid_constant__ PagedDecodeMmaParams pp) {
  const PagedDecodeParams& p = pp.p;
  constexpr uint32_t kIdescQK = make_idesc_bf16(128, 16, false, false);
  constexpr uint32_t kIdescPV = make_idesc_bf16(128, 16, true, false);
  constexpr int kTableCap = 2048;
  extern __shared__ uint8_t dsm_raw[];
  uint8_t* dsm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(dsm_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = dsm + kDmStages * kDmStageBytes;
  uint8_t* sP = sQ + kDmQBytes;
  __shared__ uint64_t full_bar[kDmStages];
  __shared__ uint64_t s_bar[2], pv_bar, p_bar;
  __shared__ uint32_t tmem_slot;
  __shared__ float s_wmax[4][G], s_wsum[4][G];
  __shared__ int s_table[kTableCap];

  const int kvh = blockIdx.x, b = blockIdx.y, split = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int seq_len = decode_seq_len(p, b);
  const int n_blocks = (seq_len + p.block - 1) / p.block;                 // p.block == 64
  const int blocks_per_split = (n_blocks + p.splits - 1) / p.splits;
  const int blk0 = split * blocks_per_split;
  const int blk1 = min(n_blocks, blk0 + blocks_per_split);
  const int n_tiles = blk1 > blk0 ? (blk1 - blk0 + 1) / 2 : 0;
  // The block-table entries of this split are staged in shared memory once: the per-tile look-ups would otherwise be
  // dependent global loads on the tile chain.
  const int* gtable = p.block_table + static_cast<int64_t>(b) * p.max_blocks_per_seq;
  const bool staged = (blk1 - blk0) <= kTableCap;
  if (staged)
    for (int i = tid; i < blk1 - blk0; i += kDmThreads) s_table[i] = gtable[blk0 + i];
  const int* table = staged ? (s_table - blk0) : gtable;          // indexed by absolute block number either way

  if (tid == 0) {
    tma_prefetch_desc(&pp.tma_k);
    tma_prefetch_desc(&pp.tma_v);
    for (int s = 0; s < kDmStages; ++s) mbar_init(&full_bar[s], 1);
    mbar_init(&s_bar[0], 1);
    mbar_init(&s_bar[1], 1);
    mbar_init(&pv_bar, 1);
    mbar_init(&p_bar, 128);
    fence_barrier_init();
  }
  if (warp == 0) {
    tmem_alloc(&tmem_slot, 64);
    tmem_relinquish();
  }
  // Qpad (rows >= G are zero), P (rows >= G stay zero for the whole kernel) and the V halves of every stage are
  // cleared once: rows that a short last tile does not fill must hold finite values, because 0 * NaN is NaN
  for (int i = tid; i < (kDmQBytes + kDmPBytes) / 16; i += kDmThreads) reinterpret_cast<uint4*>(sQ)[i] = make_uint4(0, 0, 0, 0);
  for (int s = 0; s < kDmStages; ++s)
    for (int i = tid; i < kDmTileBytes / 16; i += kDmThreads)
      reinterpret_cast<uint4*>(dsm + s * kDmStageBytes + kDmTileBytes)[i] = make_uint4(0, 0, 0, 0);
  __syncthreads();
  for (int i = tid; i < G * kDmD; i += kDmThreads) {
    const int g = i / kDmD, d = i % kDmD;
    const __nv_bfloat16 v = p.q[(static_cast<int64_t>(b) * p.hq + kvh * G + g) * kDmD + d];
    *reinterpret_cast<__nv_bfloat16*>(sQ + (d >> 6) * 2048 + sw128_off(g, d & 63)) = v;
  }
  fence_proxy_async_smem();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_slot;
  const uint32_t tS = tmem_base, tO = tmem_base + 32u;      // S^T buffers at columns 0 and 16, O^T at 32

  // tile j = cache blocks blk0 + 2j (and + 1 when it exists); an out-of-range table entry is reported and its
  // half of the tile is treated as empty
  auto block_ok = [&](int blk) { const int ph = table[blk]; return ph >= 0 && ph < p.num_blocks; };

  if (warp == 4) {
    // ------------------------------------ issuer ---------------------------------------------
    if (lane == 0 && n_tiles > 0) {
      auto issue_tma = [&](int j) {
        const int s = j % kDmStages;
        uint8_t* sk = dsm + static_cast<size_t>(s) * kDmStageBytes;
        uint8_t* sv = sk + kDmTileBytes;
        uint32_t bytes = 0;
        for (int h = 0; h < 2; ++h) {
          const int blk = blk0 + 2 * j + h;
          if (blk < blk1 && block_ok(blk)) bytes += 4u * 64u * 128u;
        }
        if (bytes == 0) { mbar_arrive(&full_bar[s]); return; }
        mbar_expect_tx(&full_bar[s], bytes);
        for (int h = 0; h < 2; ++h) {
          const int blk = blk0 + 2 * j + h;
          if (blk >= blk1) continue;
          if (!block_ok(blk)) { if (p.status != nullptr) atomicOr(p.status, kStatusIndexOutOfRange); continue; }
          const int slot = table[blk] * 64;
          for (int c = 0; c < 2; ++c) {
            tma_load_3d(sk + c * kDmHalfBytes + h * 8192, &pp.tma_k, &full_bar[s], c * 64, kvh, slot);
            tma_load_3d(sv + c * kDmHalfBytes + h * 8192, &pp.tma_v, &full_bar[s], c * 64, kvh, slot);
          }
        }
      };
      // S^T(j) = K_j Qpad^T into buffer j & 1
      auto issue_qk = [&](int j) -> bool {
        const int s = j % kDmStages;
        if (!mbar_wait(&full_bar[s], (j / kDmStages) & 1u, p.status)) return false;
        tc_fence_after_sync();
        const uint32_t aK = smem_u32(dsm + static_cast<size_t>(s) * kDmStageBytes), aQ = smem_u32(sQ);
        const uint32_t dS = tS + static_cast<uint32_t>((j & 1) * 16);
#pragma unroll
        for (int kk = 0; kk < kDmD / 16; ++kk) {
          tc_mma_f16_ss(dS, make_smem_desc(aK + (kk / 4) * kDmHalfBytes + (kk % 4) * 32, 16, 1024),
                        make_smem_desc(aQ + (kk / 4) * 2048 + (kk % 4) * 32, 16, 1024), kIdescQK, kk != 0 ? 1u : 0u);
        }
        tc_commit(&s_bar[j & 1]);
        return true;
      };
      const int pre = n_tiles < kDmStages ? n_tiles : kDmStages;
      for (int j = 0; j < pre; ++j) issue_tma(j);
      bool iok = issue_qk(0);
      for (int j = 0; j < n_tiles && iok; ++j) {
        // S^T of the next tile runs under this tile's softmax; its buffer was last read for tile j - 1, whose
        // "P ready" this thread has already waited for
        if (j + 1 < n_tiles) iok = issue_qk(j + 1);
        if (!iok) break;
        iok = mbar_wait(&p_bar, j & 1u, p.status);                 // P(j), the V fix-ups and all reads of S^T(j) are done
        if (!iok) break;
        tc_fence_after_sync();
        const uint32_t aV = smem_u32(dsm + static_cast<size_t>(j % kDmStages) * kDmStageBytes + kDmTileBytes);
        const uint32_t aP = smem_u32(sP);
#pragma unroll
        for (int kk = 0; kk < kDmTileKeys / 16; ++kk) {
          tc_mma_f16_ss(tO, make_smem_desc(aV + kk * 2048, kDmHalfBytes, 1024),
                        make_smem_desc(aP + (kk / 4) * 2048 + (kk % 4) * 32, 16, 1024), kIdescPV,
                        (j | kk) != 0 ? 1u : 0u);
        }
        tc_commit(&pv_bar);
        if (j + kDmStages < n_tiles) {                             // the stage is free once P V has read it
          iok = mbar_wait(&pv_bar, j & 1u, p.status);
          if (iok) issue_tma(j + kDmStages);
        }
      }
    }
  } else {
    // ------------------------------------ softmax --------------------------------------------
    const uint32_t lane_off = static_cast<uint32_t>(warp * 32) << 16;
    float m_run[G], l_warp[G];
#pragma unroll
    for (int g = 0; g < G; ++g) { m_run[g] = -1.0e29f; l_warp[g] = 0.f; }
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      uint8_t* sv = dsm + static_cast<size_t>(j % kDmStages) * kDmStageBytes + kDmTileBytes;
      // keys of this tile that exist: whole blocks except the last one of the sequence
      int n_keys = 0;
      for (int h = 0; h < 2; ++h) {
        const int blk = blk0 + 2 * j + h;
        if (blk < blk1) n_keys = h * 64 + (block_ok(blk) ? min(64, seq_len - blk * 64) : 0);
      }
      const bool first_half_ok = block_ok(blk0 + 2 * j);
      ok = ok && mbar_wait(&s_bar[j & 1], (j >> 1) & 1u, p.status);
      ok = __all_sync(0xFFFFFFFFu, ok);              // the aligned tcgen05 instructions below need warp-uniform flow
      // scores of my key for the G heads (log2 domain); keys that do not exist are masked
      float sc[G];
      if (ok) {
        tc_fence_after_sync();
        uint32_t r[16];
        tmem_ld16(tS + static_cast<uint32_t>((j & 1) * 16) + lane_off, r);
        tc_wait_ld();
        const bool exists = tid < n_keys && (tid >= 64 || first_half_ok);
#pragma unroll
        for (int g = 0; g < G; ++g) sc[g] = exists ? __uint_as_float(r[g]) * p.scale_log2 : -1.0e30f;
      } else {
#pragma unroll
        for (int g = 0; g < G; ++g) sc[g] = -1.0e30f;
      }
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float v = sc[g];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
        if (lane == 0) s_wmax[warp][g] = v;
      }
      tc_fence_before_sync();
      ok = softmax_barrier_and(ok);                  // the per-warp maxima are visible; every thread agrees on `ok`
      if (!ok) break;
      // the previous tile's P V product must be complete before O is rescaled and P is overwritten
      if (j > 0) {
        ok = ok && mbar_wait(&pv_bar, (j - 1) & 1u, p.status);
        ok = __all_sync(0xFFFFFFFFu, ok);
      }
      float alpha[G], pj[G];
      bool any_rescale = false;
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const float mt = fmaxf(fmaxf(s_wmax[0][g], s_wmax[1][g]), fmaxf(s_wmax[2][g], s_wmax[3][g]));
        // lazy: the reference max moves only when the tile's max exceeds it by more than 2^8, so most tiles leave
        // the accumulator alone (p <= 256 stays exact enough in bf16; the final division uses the same reference)
        const float mn = (mt > m_run[g] + 8.f) ? mt : m_run[g];
        alpha[g] = exp2f(m_run[g] - mn);
        any_rescale |= (mn != m_run[g]) && j > 0;
        m_run[g] = mn;
        pj[g] = exp2f(sc[g] - mn);                                      // masked keys: exp2(-1e30 - m) = 0
      }
      if (ok && any_rescale) {
        tc_fence_after_sync();
        uint32_t o[16];
        tmem_ld16(tO + lane_off, o);
        tc_wait_ld();
#pragma unroll
        for (int g = 0; g < G; ++g) o[g] = __float_as_uint(__uint_as_float(o[g]) * alpha[g]);
        tmem_st16(tO + lane_off, o);
        tc_wait_st();
      }
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const __nv_bfloat16 pb = __float2bfloat16(pj[g]);
        *reinterpret_cast<__nv_bfloat16*>(sP + (tid >> 6) * 2048 + sw128_off(g, tid & 63)) = pb;
        float v = __bfloat162float(pb);              // the sum uses the rounded value that the tensor core multiplies
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
        l_warp[g] = l_warp[g] * alpha[g] + v;        // per-warp running sum (identical in all lanes of the warp)
      }
      // rows of V that this tile did not fill: key t's row in both 64-d halves
      if (tid >= n_keys || (tid < 64 && !first_half_ok)) {
        for (int c = 0; c < 2; ++c)
          for (int i = 0; i < 8; ++i) reinterpret_cast<uint4*>(sv + c * kDmHalfBytes + tid * 128)[i] = make_uint4(0, 0, 0, 0);
      }
      // After a wait that ran out P is not reported as ready; the warp keeps walking the loop (without waiting) so
      // that every warp meets the named barrier the same number of times, and all leave together through its AND.
      if (ok) {
        fence_proxy_async_smem();
        tc_fence_before_sync();
        mbar_arrive(&p_bar);
      }
    }
    if (ok && n_tiles > 0) ok = mbar_wait(&pv_bar, (n_tiles - 1) & 1u, p.status);
    if (lane == 0) {
#pragma unroll
      for (int g = 0; g < G; ++g) s_wsum[warp][g] = l_warp[g];
    }
    ok = softmax_barrier_and(ok);
    if (ok) {
      tc_fence_after_sync();
      uint32_t o[16];
      if (n_tiles > 0) {
        tmem_ld16(tO + lane_off, o);
        tc_wait_ld();
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) o[i] = 0u;
      }
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const int64_t base = (static_cast<int64_t>(b) * p.hq + kvh * G + g) * p.splits + split;
        p.partial_o[base * kDmD + tid] = __uint_as_float(o[g]);           // output dimension tid of head g
        if (tid == 0) {
          p.partial_ml[base * 2] = m_run[g];
          p.partial_ml[base * 2 + 1] = s_wsum[0][g] + s_wsum[1][g] + s_wsum[2][g] + s_wsum[3][g];
        }
      }
    } else {
      // A wait ran out (status bit set).  The split's slots in the scratch are still written, as an empty partial
      // (max = -1e29, sum = 0, zeros): the merge kernel then never reads what an earlier launch left there.
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const int64_t base = (static_cast<int64_t>(b) * p.hq + kvh * G + g) * p.splits + split;
        p.partial_o[base * kDmD + tid] = 0.f;
        if (tid == 0) {
          p.partial_ml[base * 2] = -1.0e29f;
          p.partial_ml[base * 2 + 1] = 0.f;
        }
      }
      // let copies that may still be in flight land before shared memory and TMEM are released
      const uint64_t t0 = globaltimer_ns();
      while (globaltimer_ns() - t0 < 200000ull) { __nanosleep(1000); }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 64);
  }
}

}  // namespace yv
