// Flash attention backward for sm_100a, as two tcgen05 kernels that recompute the probabilities from
// the saved log-sum-exp (natural log of the scaled scores) and delta = rowsum(dO * O):
//
//   attn_bwd_dq_kernel   one CTA per (128-query block, query head, sequence), loops over key blocks:
//        S = Q K^T, dP = dO V^T            (SS MMAs into TMEM)
//        dS = P * (dP - delta)              (softmax warps: thread r = query row r; bf16 dS over S in TMEM)
//        dQ += dS K                         (TS MMA; K tile read MN-major from the same shared tile)
//   attn_bwd_dkv_kernel  one CTA per (128-key block, KV head, sequence), loops over the G query heads
//        of the group and the query blocks that see this key block:
//        S^T = K Q^T, dP^T = V dO^T         (lanes = keys, columns = queries)
//        P^T, dS^T -> bf16 in TMEM
//        dV += P^T dO,  dK += dS^T Q        (TS MMAs; dO and Q tiles read MN-major)
//   Both scale by the softmax scale in the epilogue.  No atomics: every output row has one writer.
#pragma once
#include "sm100.cuh"

namespace yv {

struct AttnBwdParams {
  CUtensorMap tma_q, tma_k, tma_v, tma_do;   // 3-D (d, head, token), box (64, 1, 128)
  __nv_bfloat16* dq;
  __nv_bfloat16* dk;
  __nv_bfloat16* dv;
  const float* lse;      // [hq, total_q] natural log
  const float* delta;    // [hq, total_q]
  const int* cu_q;
  const int* cu_k;
  int hq, hk;
  int64_t dq_stride, dk_stride, dv_stride;
  int64_t total_q;
  int causal;
  float scale;           // softmax scale
  float scale_log2;      // scale * log2(e)
  uint32_t* status;
};

constexpr float kLog2e = 1.4426950408889634f;
// Backward CTAs: TMA warp, MMA warp and eight softmax warps (two per TMEM lane quarter, each converting half of the
// columns of a 64-wide half-block).
constexpr int kAttnBwdSoftmaxThreads = 256;
constexpr int kAttnBwdThreads = 64 + kAttnBwdSoftmaxThreads;

template <int D>
struct AttnBwdSmem {
  static constexpr int kTile = 128 * D * 2;
  static constexpr int kStages = 2;
  static constexpr int kTotal = kTile * (2 + 2 * kStages) + 2 * 2 * 128 * 4 + 256 + 1024;
};

// --------------------------------------------------------------------------------------------------
// dQ kernel
// --------------------------------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(kAttnBwdThreads, 1) attn_bwd_dq_kernel(const __grid_constant__ AttnBwdParams p) {
  using S = AttnBwdSmem<D>;
  constexpr int kStages = S::kStages;
  constexpr int kDBoxes = D / 64;
  constexpr uint32_t kBoxBytes = 128 * 128;
  // A 128-key block is processed as two 64-key halves: TMEM stage s in {0,1} holds S at [128 s, 128 s + 64) and dP at
  // [128 s + 64, 128 s + 128) (dS as bf16 over the first 32 columns of S), so the scores of half h + 1 are computed
  // while the softmax threads work on half h; dQ accumulates at [256, 256 + D).
  constexpr uint32_t kIdescNT = make_idesc_bf16(128, 64, false, false);    // S, dP: 128 queries x 64 keys
  constexpr uint32_t kIdescDQ = make_idesc_bf16(128, D, false, true);      // dS (TMEM) x K (MN-major)
  constexpr uint32_t kTmemCols = 512;
  constexpr uint32_t kColDQ = 256;
  constexpr uint32_t kHalfRows = 64 * 128;            // byte offset of key rows 64.. inside a 64-column box

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sDO = sQ + S::kTile;
  uint8_t* sK = sDO + S::kTile;
  uint8_t* sV = sK + kStages * S::kTile;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + kStages * S::kTile + 2 * 2 * 128 * 4);
  uint64_t* qdo_full = bars;            // [1]
  uint64_t* k_full = bars + 1;          // [2]
  uint64_t* v_full = bars + 3;          // [2]
  uint64_t* k_empty = bars + 5;         // [2]  released after dQ MMA (last reader of K_j)
  uint64_t* v_empty = bars + 7;         // [2]  released after dP MMA
  uint64_t* sdp_full = bars + 9;        // [2]  S and dP of a TMEM stage ready
  uint64_t* ds_full = bars + 11;        // [2]  128 arrivals: dS written
  uint64_t* dq_done = bars + 13;        // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.z, h = blockIdx.y;
  const int hkv = h / (p.hq / p.hk);
  const int q_begin = p.cu_q[b], q_len = p.cu_q[b + 1] - q_begin;
  const int k_begin = p.cu_k[b], k_len = p.cu_k[b + 1] - k_begin;
  const int n_qblk = (q_len + 127) / 128;
  const int q_blk = n_qblk - 1 - static_cast<int>(blockIdx.x);
  if (q_blk < 0) return;
  const int q0 = q_blk * 128;
  const int causal_shift = k_len - q_len;
  int n_kv = (k_len + 127) / 128;
  if (p.causal) {
    const int last_key = q0 + 127 + causal_shift;
    const int lim = last_key / 128 + 1;
    n_kv = last_key < 0 ? 0 : (lim < n_kv ? lim : n_kv);
  }

  if (threadIdx.x == 0) {
    mbar_init(qdo_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&k_full[s], 1); mbar_init(&v_full[s], 1);
      mbar_init(&k_empty[s], 1); mbar_init(&v_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) { mbar_init(&sdp_full[s], 1); mbar_init(&ds_full[s], kAttnBwdSoftmaxThreads); }
    mbar_init(dq_done, 1);
    fence_barrier_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, kTmemCols); tmem_relinquish(); }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (elect_one() && n_kv > 0) {
      mbar_expect_tx(qdo_full, 2 * S::kTile);
#pragma unroll
      for (int c = 0; c < kDBoxes; ++c) {
        tma_load_3d(sQ + c * kBoxBytes, &p.tma_q, qdo_full, c * 64, h, q_begin + q0);
        tma_load_3d(sDO + c * kBoxBytes, &p.tma_do, qdo_full, c * 64, h, q_begin + q0);
      }
      bool ok = true;
      for (int j = 0; j < n_kv && ok; ++j) {
        const int s = j % kStages;
        const uint32_t ph = (j / kStages) & 1u;
        ok = mbar_wait(&k_empty[s], ph ^ 1u, p.status);
        if (!ok) break;
        mbar_expect_tx(&k_full[s], S::kTile);
#pragma unroll
        for (int c = 0; c < kDBoxes; ++c)
          tma_load_3d(sK + s * S::kTile + c * kBoxBytes, &p.tma_k, &k_full[s], c * 64, hkv, k_begin + j * 128);
        ok = mbar_wait(&v_empty[s], ph ^ 1u, p.status);
        if (!ok) break;
        mbar_expect_tx(&v_full[s], S::kTile);
#pragma unroll
        for (int c = 0; c < kDBoxes; ++c)
          tma_load_3d(sV + s * S::kTile + c * kBoxBytes, &p.tma_v, &v_full[s], c * 64, hkv, k_begin + j * 128);
      }
    }
  } else if (warp == 1) {
    if (elect_one() && n_kv > 0) {
      bool ok = mbar_wait(qdo_full, 0, p.status);
      const uint32_t aQ = smem_u32(sQ), aDO = smem_u32(sDO);
      const int n_half = 2 * n_kv;
      // S = Q K^T and dP = dO V^T of key half `hf` (block hf / 2, key rows 64 (hf % 2) ..) into TMEM stage hf % 2
      auto issue_sdp = [&](int hf) -> bool {
        const int j = hf >> 1, half = hf & 1;
        const int s = j % kStages;
        if (half == 0) {
          const uint32_t ph = (j / kStages) & 1u;
          if (!mbar_wait(&k_full[s], ph, p.status)) return false;
          if (!mbar_wait(&v_full[s], ph, p.status)) return false;
          tc_fence_after_sync();
        }
        const uint32_t aK = smem_u32(sK + s * S::kTile) + half * kHalfRows;
        const uint32_t aV = smem_u32(sV + s * S::kTile) + half * kHalfRows;
        const uint32_t tS = tmem_base + static_cast<uint32_t>((hf & 1) * 128);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk / 4) * kBoxBytes + (kk % 4) * 32;
          tc_mma_f16_ss(tS, make_smem_desc(aQ + off, 16, 1024), make_smem_desc(aK + off, 16, 1024), kIdescNT,
                        kk != 0 ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk / 4) * kBoxBytes + (kk % 4) * 32;
          tc_mma_f16_ss(tS + 64, make_smem_desc(aDO + off, 16, 1024), make_smem_desc(aV + off, 16, 1024), kIdescNT,
                        kk != 0 ? 1u : 0u);
        }
        if (half == 1) tc_commit(&v_empty[s]);          // V_j is read by the dP products only
        tc_commit(&sdp_full[hf & 1]);
        return true;
      };
      if (ok) ok = issue_sdp(0);
      for (int hf = 0; hf < n_half && ok; ++hf) {
        if (hf + 1 < n_half) {                           // next half's scores are queued before this half's dQ product
          ok = issue_sdp(hf + 1);
          if (!ok) break;
        }
        ok = mbar_wait(&ds_full[hf & 1], (hf >> 1) & 1u, p.status);
        if (!ok) break;
        tc_fence_after_sync();
        const int j = hf >> 1, half = hf & 1;
        const int s = j % kStages;
        const uint32_t aK = smem_u32(sK + s * S::kTile);
        const uint32_t tS = tmem_base + static_cast<uint32_t>((hf & 1) * 128);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {                 // 64 keys = 4 K-steps of 16
          tc_mma_f16_ts(tmem_base + kColDQ, tS + kk * 8, make_smem_desc(aK + (half * 4 + kk) * 2048, kBoxBytes, 1024),
                        kIdescDQ, (hf | kk) != 0 ? 1u : 0u);
        }
        if (half == 1) tc_commit(&k_empty[s]);
        if (hf == n_half - 1) tc_commit(dq_done);        // one completion, after the last product
      }
    }
  } else {
    const int quarter = warp & 3;
    const int colhalf = (warp - 2) >> 2;                 // two warps per TMEM lane quarter split the columns
    const int row = quarter * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    const int q_pos = q0 + row;
    const bool q_valid = q_pos < q_len;
    const int key_limit = p.causal ? (q_pos + causal_shift) : (k_len - 1);
    const int64_t stat_idx = static_cast<int64_t>(h) * p.total_q + q_begin + q_pos;
    const float lse2 = q_valid ? p.lse[stat_idx] * kLog2e : 0.f;
    const float delta = q_valid ? p.delta[stat_idx] : 0.f;
    bool ok = true;
    const int n_half = 2 * n_kv;
    for (int hf = 0; hf < n_half && ok; ++hf) {
      ok = mbar_wait(&sdp_full[hf & 1], (hf >> 1) & 1u, p.status);
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t tS = tmem_base + lane_off + static_cast<uint32_t>((hf & 1) * 128), tDP = tS + 64;
      const int kbase = (hf >> 1) * 128 + (hf & 1) * 64;
      // the select per element is only needed on halves that touch the causal diagonal, the end of the keys or a
      // query row past the end (uniform over the warp except for q_valid, which is folded in)
      const bool need_mask = !q_valid || (kbase + 63 > key_limit) || (kbase + 64 > k_len);
      const float2 sc2 = make_float2(p.scale_log2, p.scale_log2);
      const float2 nl2 = make_float2(-lse2, -lse2), nd2 = make_float2(-delta, -delta);
      uint32_t pk[16];
      {
        const int c = colhalf;
        uint32_t sv[32], dv[32];
        tmem_ld32(tS + c * 32, sv);
        tmem_ld32(tDP + c * 32, dv);
        tc_wait_ld();
        // two keys per step: packed FMA -> bf16x2 -> one ex2 on the pair; dS = P * (dP - delta) in packed fp32
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const int kidx = kbase + c * 32 + 2 * i;
          float2 x = __ffma2_rn(make_float2(__uint_as_float(sv[2 * i]), __uint_as_float(sv[2 * i + 1])), sc2, nl2);
          if (need_mask) {
            if (!(q_valid && kidx <= key_limit && kidx < k_len)) x.x = -INFINITY;
            if (!(q_valid && kidx + 1 <= key_limit && kidx + 1 < k_len)) x.y = -INFINITY;
          }
          const __nv_bfloat162 e = h2exp2(__float22bfloat162_rn(x));
          const uint32_t bits = *reinterpret_cast<const uint32_t*>(&e);
          const float2 pf = make_float2(__uint_as_float(bits << 16), __uint_as_float(bits & 0xFFFF0000u));
          const float2 dd = __fadd2_rn(make_float2(__uint_as_float(dv[2 * i]), __uint_as_float(dv[2 * i + 1])), nd2);
          const float2 r = __fmul2_rn(pf, dd);
          pk[i] = pack_bf16(r.x, r.y);
        }
      }
      tmem_st16(tS + colhalf * 16, pk);
      tc_wait_st();
      tc_fence_before_sync();
      mbar_arrive(&ds_full[hf & 1]);
    }
    if (ok && n_kv > 0) {
      ok = mbar_wait(dq_done, 0u, p.status);
      ok = __all_sync(0xFFFFFFFFu, ok);
    }
    if (ok) {
      tc_fence_after_sync();
      __nv_bfloat16* orow = p.dq + static_cast<int64_t>(q_begin + q_pos) * p.dq_stride + static_cast<int64_t>(h) * D;
#pragma unroll
      for (int c = colhalf * (D / 64); c < (colhalf + 1) * (D / 64); ++c) {      // each warp of a quarter writes half of D
        uint32_t ov[32];
        if (n_kv > 0) {
          tmem_ld32(tmem_base + lane_off + kColDQ + c * 32, ov);
          tc_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) ov[i] = 0u;
        }
        if (q_valid) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 v;
            v.x = pack_bf16(__uint_as_float(ov[8 * i + 0]) * p.scale, __uint_as_float(ov[8 * i + 1]) * p.scale);
            v.y = pack_bf16(__uint_as_float(ov[8 * i + 2]) * p.scale, __uint_as_float(ov[8 * i + 3]) * p.scale);
            v.z = pack_bf16(__uint_as_float(ov[8 * i + 4]) * p.scale, __uint_as_float(ov[8 * i + 5]) * p.scale);
            v.w = pack_bf16(__uint_as_float(ov[8 * i + 6]) * p.scale, __uint_as_float(ov[8 * i + 7]) * p.scale);
            *reinterpret_cast<uint4*>(orow + c * 32 + i * 8) = v;
          }
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (p.status != nullptr && *reinterpret_cast<volatile uint32_t*>(p.status) != 0u) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) { __nanosleep(1000); }
    __syncthreads();
  }
  if (warp == 1) { tc_fence_after_sync(); tmem_dealloc(tmem_base, kTmemCols); }
}

}  // namespace yv

#include "attention_bwd_dkv.cuh"
