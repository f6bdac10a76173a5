// Flash attention forward for sm_100a: GQA, causal or full, packed variable-length sequences.
//
// One CTA per (128-query block, query head, sequence); 192 threads:
//   warp 0      TMA producer: Q once, then K_j / V_j tiles through two-stage rings
//   warp 1      MMA issuer:  S_j = Q K_j^T (SS) into one of two TMEM S buffers, O += P_j V_j (TS: P read
//               from TMEM where the softmax warps wrote it over S_j)
//   warps 2..5  softmax: thread r owns query row r (= TMEM lane r): tcgen05.ld the 128 scores, online
//               softmax with lazy rescaling of the O accumulator, pack P to bf16, tcgen05.st
// TMEM columns: [0,128) S0/P0, [128,256) S1/P1, [256,256+D) O.
#pragma once
#include "sm100.cuh"

namespace yv {

struct AttnFwdParams {
  CUtensorMap tma_q;   // 3-D (d, head, token), box (64, 1, 128)
  CUtensorMap tma_k;
  CUtensorMap tma_v;
  __nv_bfloat16* o;
  float* lse;          // [hq, total_q]
  const int* cu_q;     // [B+1]
  const int* cu_k;     // [B+1]
  int hq, hk;
  int64_t o_stride;    // elements between consecutive tokens of o
  int64_t total_q;
  int causal;
  float scale_log2;    // softmax scale * log2(e)
  uint32_t* status;
};

constexpr int kAttnThreads = 192;
constexpr int kAttnBlock = 128;     // query rows and key rows per tile
constexpr float kMaskValue = -1.0e30f;
constexpr float kRescaleThreshold = 8.0f;   // log2 units: O is rescaled only when the row max grew by more

template <int D>
struct AttnFwdSmem {
  static constexpr int kTile = kAttnBlock * D * 2;       // bytes of one Q/K/V tile
  static constexpr int kStages = 2;
  static constexpr int kTotal = kTile * (1 + 2 * kStages) + 256 + 1024;
};

template <int D>
__global__ void __launch_bounds__(kAttnThreads, 1) attn_fwd_kernel(const __grid_constant__ AttnFwdParams p) {
  using S = AttnFwdSmem<D>;
  constexpr int kStages = S::kStages;
  constexpr int kDBoxes = D / 64;
  constexpr uint32_t kBoxBytes = kAttnBlock * 128;     // one (128 rows x 64 cols) box
  constexpr uint32_t kIdescQK = make_idesc_bf16(128, 128, false, false);
  constexpr uint32_t kIdescPV = make_idesc_bf16(128, D, false, true);
  constexpr uint32_t kTmemCols = 512;
  constexpr uint32_t kOCol = 256;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + S::kTile;
  uint8_t* sV = sK + kStages * S::kTile;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + kStages * S::kTile);
  uint64_t* q_full = bars;                 // [1]
  uint64_t* k_full = bars + 1;             // [2]
  uint64_t* k_empty = bars + 3;            // [2]
  uint64_t* v_full = bars + 5;             // [2]
  uint64_t* v_empty = bars + 7;            // [2]
  uint64_t* s_full = bars + 9;             // [2]
  uint64_t* p_full = bars + 11;            // [2]
  uint64_t* o_done = bars + 13;            // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int b = blockIdx.z;
  const int h = blockIdx.y;
  const int hkv = h / (p.hq / p.hk);
  const int q_begin = p.cu_q[b], q_len = p.cu_q[b + 1] - q_begin;
  const int k_begin = p.cu_k[b], k_len = p.cu_k[b + 1] - k_begin;
  const int n_qblk = (q_len + kAttnBlock - 1) / kAttnBlock;
  // heavy (late) query blocks first for causal load balance
  const int q_blk = n_qblk - 1 - static_cast<int>(blockIdx.x);
  if (q_blk < 0) return;
  const int q0 = q_blk * kAttnBlock;
  int n_kv = (k_len + kAttnBlock - 1) / kAttnBlock;
  // causal: query i (bottom-right aligned when k_len != q_len) sees keys <= i + (k_len - q_len)
  const int causal_shift = k_len - q_len;
  if (p.causal) {
    const int last_key = q0 + kAttnBlock - 1 + causal_shift;
    const int lim = last_key / kAttnBlock + 1;
    n_kv = last_key < 0 ? 0 : (lim < n_kv ? lim : n_kv);
  }

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&p.tma_q);
    tma_prefetch_desc(&p.tma_k);
    tma_prefetch_desc(&p.tma_v);
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
      mbar_init(&s_full[s], 1);
      mbar_init(&p_full[s], 128);
    }
    mbar_init(o_done, 1);
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------ producer ------------------------------------------
    if (elect_one() && n_kv > 0) {
      mbar_expect_tx(q_full, S::kTile);
#pragma unroll
      for (int c = 0; c < kDBoxes; ++c) tma_load_3d(sQ + c * kBoxBytes, &p.tma_q, q_full, c * 64, h, q_begin + q0);
      bool ok = true;
      for (int j = 0; j < n_kv && ok; ++j) {
        const int s = j % kStages;
        const uint32_t ph = (j / kStages) & 1u;
        ok = mbar_wait(&k_empty[s], ph ^ 1u, p.status);
        if (!ok) break;
        mbar_expect_tx(&k_full[s], S::kTile);
#pragma unroll
        for (int c = 0; c < kDBoxes; ++c)
          tma_load_3d(sK + s * S::kTile + c * kBoxBytes, &p.tma_k, &k_full[s], c * 64, hkv,
                      k_begin + j * kAttnBlock);
        ok = mbar_wait(&v_empty[s], ph ^ 1u, p.status);
        if (!ok) break;
        mbar_expect_tx(&v_full[s], S::kTile);
#pragma unroll
        for (int c = 0; c < kDBoxes; ++c)
          tma_load_3d(sV + s * S::kTile + c * kBoxBytes, &p.tma_v, &v_full[s], c * 64, hkv,
                      k_begin + j * kAttnBlock);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------ MMA issuer ----------------------------------------
    if (elect_one() && n_kv > 0) {
      bool ok = mbar_wait(q_full, 0, p.status);
      const uint32_t aQ = smem_u32(sQ);
      auto issue_qk = [&](int j) -> bool {
        const int s = j % kStages;
        if (!mbar_wait(&k_full[s], (j / kStages) & 1u, p.status)) return false;
        tc_fence_after_sync();
        const uint32_t aK = smem_u32(sK + s * S::kTile);
        const uint32_t tS = tmem_base + static_cast<uint32_t>((j & 1) * 128);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk / 4) * kBoxBytes + (kk % 4) * 32;
          tc_mma_f16_ss(tS, make_smem_desc(aQ + off, 16, 1024), make_smem_desc(aK + off, 16, 1024), kIdescQK,
                        kk != 0 ? 1u : 0u);
        }
        tc_commit(&k_empty[s]);
        tc_commit(&s_full[j & 1]);
        return true;
      };
      if (ok) ok = issue_qk(0);
      for (int j = 0; j < n_kv && ok; ++j) {
        if (j + 1 < n_kv) {
          ok = issue_qk(j + 1);
          if (!ok) break;
        }
        const int s = j % kStages;
        ok = mbar_wait(&p_full[j & 1], (j >> 1) & 1u, p.status);
        if (!ok) break;
        ok = mbar_wait(&v_full[s], (j / kStages) & 1u, p.status);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t aV = smem_u32(sV + s * S::kTile);
        const uint32_t tP = tmem_base + static_cast<uint32_t>((j & 1) * 128);
        const uint32_t tO = tmem_base + kOCol;
#pragma unroll
        for (int kk = 0; kk < kAttnBlock / 16; ++kk) {
          // 16 keys per step: 8 packed bf16x2 columns of P; 16 key rows (2048 B) of the V tile
          tc_mma_f16_ts(tO, tP + kk * 8, make_smem_desc(aV + kk * 2048, kBoxBytes, 1024), kIdescPV,
                        (j | kk) != 0 ? 1u : 0u);
        }
        tc_commit(&v_empty[s]);
        tc_commit(o_done);
      }
    }
  } else {
    // ------------------------------------ softmax / epilogue --------------------------------
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;              // query row inside the tile
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    const int q_pos = q0 + row;                       // position inside the sequence
    const int key_limit = p.causal ? (q_pos + causal_shift) : (k_len - 1);   // last visible key
    float m_used = -1.0e29f;                          // running max (log2 domain); above kMaskValue so masked scores give 0
    float l_sum = 0.f;
    bool ok = true;
    for (int j = 0; j < n_kv && ok; ++j) {
      ok = mbar_wait(&s_full[j & 1], (j >> 1) & 1u, p.status);
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t tS = tmem_base + lane_off + static_cast<uint32_t>((j & 1) * 128);
      uint32_t sreg[128];
      {
        uint32_t(&c0)[32] = *reinterpret_cast<uint32_t(*)[32]>(&sreg[0]);
        uint32_t(&c1)[32] = *reinterpret_cast<uint32_t(*)[32]>(&sreg[32]);
        uint32_t(&c2)[32] = *reinterpret_cast<uint32_t(*)[32]>(&sreg[64]);
        uint32_t(&c3)[32] = *reinterpret_cast<uint32_t(*)[32]>(&sreg[96]);
        tmem_ld32(tS, c0);
        tmem_ld32(tS + 32, c1);
        tmem_ld32(tS + 64, c2);
        tmem_ld32(tS + 96, c3);
        tc_wait_ld();
      }
      const int kbase = j * kAttnBlock;
      const bool need_mask = (kbase + kAttnBlock - 1 > key_limit) || (kbase + kAttnBlock > k_len);
      // The row maximum is taken over the raw scores (the scale is positive); scaling and the subtraction of the
      // reference maximum are one fused multiply-add per pair of scores further down.
      float mx = kMaskValue;
      if (need_mask) {
#pragma unroll
        for (int i = 0; i < 128; ++i) {
          if (kbase + i > key_limit || kbase + i >= k_len) sreg[i] = 0xFF800000u;      // -inf: 2^(-inf) = 0
          mx = fmaxf(mx, __uint_as_float(sreg[i]));
        }
      } else {
#pragma unroll
        for (int i = 0; i < 128; i += 2)
          mx = fmaxf(mx, fmaxf(__uint_as_float(sreg[i]), __uint_as_float(sreg[i + 1])));
      }
      mx = (mx > 0.5f * kMaskValue) ? mx * p.scale_log2 : kMaskValue;
      // lazy rescale: keep the old reference max unless the new one is much larger
      float alpha = 1.f;
      bool rescale = false;
      if (mx > m_used + kRescaleThreshold) {
        alpha = exp2f(m_used - mx);
        m_used = mx;
        rescale = (j > 0);
      }
      // p = 2^(s * scale - m) two scores at a time: one packed fp32 FMA, one conversion to bf16x2 and ONE
      // special-function instruction (ex2 on a bf16 pair) whose result already is the packed P operand.  The row sum
      // adds the rounded values that the tensor core will multiply, unpacked with two logic ops and a packed add.
      float2 rs2 = make_float2(0.f, 0.f);
      uint32_t pk[64];
      const float2 sc2 = make_float2(p.scale_log2, p.scale_log2);
      const float2 nm2 = make_float2(-m_used, -m_used);
#pragma unroll
      for (int i = 0; i < 64; ++i) {
        const float2 x = __ffma2_rn(make_float2(__uint_as_float(sreg[2 * i]), __uint_as_float(sreg[2 * i + 1])), sc2, nm2);
        const __nv_bfloat162 e = h2exp2(__float22bfloat162_rn(x));
        const uint32_t bits = *reinterpret_cast<const uint32_t*>(&e);
        pk[i] = bits;
        rs2 = __fadd2_rn(rs2, make_float2(__uint_as_float(bits << 16), __uint_as_float(bits & 0xFFFF0000u)));
      }
      const float rs = rs2.x + rs2.y;
      l_sum = l_sum * alpha + rs;
      if (__any_sync(0xFFFFFFFFu, rescale)) {
        // O holds sums relative to the old max: wait for the previous P V product, then scale the row
        ok = mbar_wait(o_done, (j - 1) & 1u, p.status);
        ok = __all_sync(0xFFFFFFFFu, ok);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t tO = tmem_base + lane_off + kOCol;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t ov[32];
          tmem_ld32(tO + c * 32, ov);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * alpha);
          tmem_st32(tO + c * 32, ov);
        }
      }
      {
        uint32_t(&h0)[32] = *reinterpret_cast<uint32_t(*)[32]>(&pk[0]);
        uint32_t(&h1)[32] = *reinterpret_cast<uint32_t(*)[32]>(&pk[32]);
        tmem_st32(tS, h0);
        tmem_st32(tS + 32, h1);
      }
      tc_wait_st();
      tc_fence_before_sync();
      mbar_arrive(&p_full[j & 1]);
    }
    // ---- epilogue: O / l, LSE ----
    if (ok && n_kv > 0) {
      ok = mbar_wait(o_done, (n_kv - 1) & 1u, p.status);
      ok = __all_sync(0xFFFFFFFFu, ok);
    }
    if (ok) {
      tc_fence_after_sync();
      const bool valid = q_pos < q_len;
      const float inv_l = (l_sum > 0.f) ? 1.f / l_sum : 0.f;
      __nv_bfloat16* orow = p.o + (static_cast<int64_t>(q_begin + q_pos) * p.o_stride) + static_cast<int64_t>(h) * D;
      const uint32_t tO = tmem_base + lane_off + kOCol;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t ov[32];
        if (n_kv > 0) {
          tmem_ld32(tO + c * 32, ov);
          tc_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) ov[i] = 0u;
        }
        if (valid) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 v;
            v.x = pack_bf16(__uint_as_float(ov[8 * i + 0]) * inv_l, __uint_as_float(ov[8 * i + 1]) * inv_l);
            v.y = pack_bf16(__uint_as_float(ov[8 * i + 2]) * inv_l, __uint_as_float(ov[8 * i + 3]) * inv_l);
            v.z = pack_bf16(__uint_as_float(ov[8 * i + 4]) * inv_l, __uint_as_float(ov[8 * i + 5]) * inv_l);
            v.w = pack_bf16(__uint_as_float(ov[8 * i + 6]) * inv_l, __uint_as_float(ov[8 * i + 7]) * inv_l);
            *reinterpret_cast<uint4*>(orow + c * 32 + i * 8) = v;
          }
        }
      }
      if (valid && p.lse != nullptr) {
        // natural-log LSE of the scaled scores
        p.lse[static_cast<int64_t>(h) * p.total_q + q_begin + q_pos] =
            (l_sum > 0.f) ? (m_used + log2f(l_sum)) * 0.6931471805599453f : -INFINITY;
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
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace yv
