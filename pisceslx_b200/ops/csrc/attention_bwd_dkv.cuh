// dK / dV kernel of the flash attention backward (see attention_bwd.cuh for the scheme).
// A 128-query block is processed as two 64-query halves so that S^T / dP^T double-buffer inside the 512 TMEM columns:
// while the softmax threads turn half h into P^T / dS^T, the tensor core already computes S^T / dP^T of half h + 1,
// and the dV / dK products of half h are queued behind them.
// TMEM columns: stage s in {0,1}: [128 s, 128 s + 64) S^T then P^T (bf16, 32 columns),
//               [128 s + 64, 128 s + 128) dP^T then dS^T (bf16, 32 columns); [256,256+D) dV, [384,384+D) dK.
#pragma once

namespace yv {

template <int D>
__global__ void __launch_bounds__(kAttnBwdThreads, 1) attn_bwd_dkv_kernel(const __grid_constant__ AttnBwdParams p) {
  using S = AttnBwdSmem<D>;
  constexpr int kStages = S::kStages;
  constexpr int kDBoxes = D / 64;
  constexpr uint32_t kBoxBytes = 128 * 128;
  constexpr uint32_t kIdescNT = make_idesc_bf16(128, 64, false, false);     // 128 keys x 64 queries
  constexpr uint32_t kIdescAcc = make_idesc_bf16(128, D, false, true);
  constexpr uint32_t kTmemCols = 512;
  constexpr uint32_t kColDV = 256, kColDK = 384;
  constexpr uint32_t kHalfRows = 64 * 128;            // byte offset of query rows 64.. inside a 64-column box

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + S::kTile;
  uint8_t* sQ = sV + S::kTile;
  uint8_t* sDO = sQ + kStages * S::kTile;
  float* s_lse = reinterpret_cast<float*>(sDO + kStages * S::kTile);   // [2][128]
  float* s_delta = s_lse + 2 * 128;                                     // [2][128]
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_delta + 2 * 128);
  uint64_t* kv_full = bars;             // [1]
  uint64_t* q_full = bars + 1;          // [2]
  uint64_t* do_full = bars + 3;         // [2]
  uint64_t* q_empty = bars + 5;         // [2]
  uint64_t* do_empty = bars + 7;        // [2]
  uint64_t* sdp_full = bars + 9;        // [2] per TMEM stage
  uint64_t* pds_full = bars + 11;       // [2] 128 arrivals each
  uint64_t* acc_done = bars + 13;       // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.z, hkv = blockIdx.y;
  const int G = p.hq / p.hk;
  const int q_begin = p.cu_q[b], q_len = p.cu_q[b + 1] - q_begin;
  const int k_begin = p.cu_k[b], k_len = p.cu_k[b + 1] - k_begin;
  const int n_kblk = (k_len + 127) / 128;
  const int k_blk = static_cast<int>(blockIdx.x);
  if (k_blk >= n_kblk) return;
  const int k0 = k_blk * 128;
  const int causal_shift = k_len - q_len;
  const int n_qblk = (q_len + 127) / 128;
  int i_start = 0;
  if (p.causal) {
    const int first_q = k0 - causal_shift;          // first query position that sees key k0
    i_start = first_q > 0 ? first_q / 128 : 0;
  }
  const int n_i = n_qblk > i_start ? n_qblk - i_start : 0;
  const int n_it = n_i * G;
  const int n_half = 2 * n_it;                      // 64-query halves

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&q_full[s], 1); mbar_init(&do_full[s], 1);
      mbar_init(&q_empty[s], 1); mbar_init(&do_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) { mbar_init(&sdp_full[s], 1); mbar_init(&pds_full[s], kAttnBwdSoftmaxThreads); }
    mbar_init(acc_done, 1);
    fence_barrier_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, kTmemCols); tmem_relinquish(); }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (elect_one() && n_it > 0) {
      mbar_expect_tx(kv_full, 2 * S::kTile);
#pragma unroll
      for (int c = 0; c < kDBoxes; ++c) {
        tma_load_3d(sK + c * kBoxBytes, &p.tma_k, kv_full, c * 64, hkv, k_begin + k0);
        tma_load_3d(sV + c * kBoxBytes, &p.tma_v, kv_full, c * 64, hkv, k_begin + k0);
      }
      bool ok = true;
      for (int it = 0; it < n_it && ok; ++it) {
        const int g = it / n_i, i = i_start + it % n_i;
        const int h = hkv * G + g;
        const int s = it % kStages;
        const uint32_t ph = (it / kStages) & 1u;
        ok = mbar_wait(&q_empty[s], ph ^ 1u, p.status);
        if (!ok) break;
        mbar_expect_tx(&q_full[s], S::kTile);
#pragma unroll
        for (int c = 0; c < kDBoxes; ++c)
          tma_load_3d(sQ + s * S::kTile + c * kBoxBytes, &p.tma_q, &q_full[s], c * 64, h, q_begin + i * 128);
        ok = mbar_wait(&do_empty[s], ph ^ 1u, p.status);
        if (!ok) break;
        mbar_expect_tx(&do_full[s], S::kTile);
#pragma unroll
        for (int c = 0; c < kDBoxes; ++c)
          tma_load_3d(sDO + s * S::kTile + c * kBoxBytes, &p.tma_do, &do_full[s], c * 64, h, q_begin + i * 128);
      }
    }
  } else if (warp == 1) {
    if (elect_one() && n_it > 0) {
      bool ok = mbar_wait(kv_full, 0, p.status);
      const uint32_t aK = smem_u32(sK), aV = smem_u32(sV);
      // S^T and dP^T of half `hf` (block hf / 2, rows 64 (hf % 2) .. of its Q / dO tiles) into TMEM stage hf % 2
      auto issue_sdp = [&](int hf) -> bool {
        const int it = hf >> 1, half = hf & 1;
        const int s = it % kStages;
        if (half == 0) {
          const uint32_t ph = (it / kStages) & 1u;
          if (!mbar_wait(&q_full[s], ph, p.status)) return false;
          if (!mbar_wait(&do_full[s], ph, p.status)) return false;
          tc_fence_after_sync();
        }
        const uint32_t aQ = smem_u32(sQ + s * S::kTile) + half * kHalfRows;
        const uint32_t aDO = smem_u32(sDO + s * S::kTile) + half * kHalfRows;
        const uint32_t tS = tmem_base + static_cast<uint32_t>((hf & 1) * 128);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk / 4) * kBoxBytes + (kk % 4) * 32;
          tc_mma_f16_ss(tS, make_smem_desc(aK + off, 16, 1024), make_smem_desc(aQ + off, 16, 1024), kIdescNT,
                        kk != 0 ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk / 4) * kBoxBytes + (kk % 4) * 32;
          tc_mma_f16_ss(tS + 64, make_smem_desc(aV + off, 16, 1024), make_smem_desc(aDO + off, 16, 1024), kIdescNT,
                        kk != 0 ? 1u : 0u);
        }
        tc_commit(&sdp_full[hf & 1]);
        return true;
      };
      if (ok) ok = issue_sdp(0);
      for (int hf = 0; hf < n_half && ok; ++hf) {
        // keep the tensor core busy while the softmax threads work on half hf: queue the next half's scores first
        if (hf + 1 < n_half) {
          ok = issue_sdp(hf + 1);
          if (!ok) break;
        }
        ok = mbar_wait(&pds_full[hf & 1], (hf >> 1) & 1u, p.status);
        if (!ok) break;
        tc_fence_after_sync();
        const int it = hf >> 1, half = hf & 1;
        const int s = it % kStages;
        const uint32_t aQ = smem_u32(sQ + s * S::kTile), aDO = smem_u32(sDO + s * S::kTile);
        const uint32_t tS = tmem_base + static_cast<uint32_t>((hf & 1) * 128);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {                 // 64 queries = 4 K-steps of 16
          tc_mma_f16_ts(tmem_base + kColDV, tS + kk * 8,
                        make_smem_desc(aDO + (half * 4 + kk) * 2048, kBoxBytes, 1024), kIdescAcc, (hf | kk) != 0 ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          tc_mma_f16_ts(tmem_base + kColDK, tS + 64 + kk * 8,
                        make_smem_desc(aQ + (half * 4 + kk) * 2048, kBoxBytes, 1024), kIdescAcc, (hf | kk) != 0 ? 1u : 0u);
        }
        if (half == 1) {
          tc_commit(&q_empty[s]);
          tc_commit(&do_empty[s]);
        }
        // one completion only, after the very last products: the scores of half hf + 1 are issued ahead of the
        // accumulator products of half hf, so a barrier that flipped every half could be observed one phase early
        if (hf == n_half - 1) tc_commit(acc_done);
      }
    }
  } else {
    // Eight softmax warps: two warps share each TMEM lane quarter (a warp may only touch lanes 32 (warp % 4) ..) and
    // split the 64 query columns of a half between them, 32 each.
    const int quarter = warp & 3;
    const int colhalf = (warp - 2) >> 2;                 // which 32 of the 64 columns of a half this warp converts
    const int row = quarter * 32 + lane;                 // key row of the tile
    const int tix = threadIdx.x - 64;                    // 0..255 among the softmax threads
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    const int key = k0 + row;
    const bool key_valid = key < k_len;
    bool ok = true;
    for (int hf = 0; hf < n_half && ok; ++hf) {
      const int it = hf >> 1, half = hf & 1;
      const int g = it / n_i, i = i_start + it % n_i;
      const int h = hkv * G + g;
      const int qb = i * 128;
      float* lse_b = s_lse + (it & 1) * 128;
      float* del_b = s_delta + (it & 1) * 128;
      if (half == 0) {
        if (tix < 128) {
          const int qpos = qb + tix;
          const bool v = qpos < q_len;
          const int64_t idx = static_cast<int64_t>(h) * p.total_q + q_begin + qpos;
          // stored negated so that the consumers fold them into packed fused multiply-adds
          lse_b[tix] = v ? -p.lse[idx] * kLog2e : -INFINITY;   // -inf -> probability 0 for rows past the end
          del_b[tix] = v ? -p.delta[idx] : 0.f;
        }
        asm volatile("bar.sync 1, 256;" ::: "memory");
      }
      ok = mbar_wait(&sdp_full[hf & 1], (hf >> 1) & 1u, p.status);
      {
        uint32_t all_ok;
        asm volatile(
            "{\n"
            ".reg .pred pin, pout;\n"
            "setp.ne.u32 pin, %1, 0;\n"
            "bar.red.and.pred pout, 1, 256, pin;\n"
            "selp.u32 %0, 1, 0, pout;\n"
            "}\n"
            : "=r"(all_ok)
            : "r"(static_cast<uint32_t>(ok))
            : "memory");
        ok = all_ok != 0u;
      }
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t tST = tmem_base + lane_off + static_cast<uint32_t>((hf & 1) * 128), tDPT = tST + 64;
      // a query column c is visible to this key iff key <= (qb + c) + shift
      const int first_vis_c = p.causal ? (key - causal_shift - qb) : 0;
      // every (key, query) pair of this block is visible: no per-element selects (uniform over the CTA)
      const bool full_vis = (!p.causal || qb >= k0 + 127 - causal_shift) && (k0 + 127 < k_len);
      const float2 sc2 = make_float2(p.scale_log2, p.scale_log2);
      uint32_t pp[16], ds[16];
      {
        const int c = colhalf;
        uint32_t sv[32], dv[32];
        tmem_ld32(tST + c * 32, sv);
        tmem_ld32(tDPT + c * 32, dv);
        tc_wait_ld();
        // Two queries per step: P = 2^(s * scale - lse) through one packed FMA, one bf16x2 conversion and one
        // special-function instruction whose result is the packed P operand; dS = P * (dP - delta) in packed fp32.
#pragma unroll
        for (int i2 = 0; i2 < 16; ++i2) {
          const int col = half * 64 + c * 32 + 2 * i2;           // query column inside the 128-query block
          const float2 nl = *reinterpret_cast<const float2*>(lse_b + col);
          const float2 nd = *reinterpret_cast<const float2*>(del_b + col);
          float2 x = __ffma2_rn(make_float2(__uint_as_float(sv[2 * i2]), __uint_as_float(sv[2 * i2 + 1])), sc2, nl);
          if (!full_vis) {
            if (!(key_valid && col >= first_vis_c)) x.x = -INFINITY;
            if (!(key_valid && col + 1 >= first_vis_c)) x.y = -INFINITY;
          }
          const __nv_bfloat162 e = h2exp2(__float22bfloat162_rn(x));
          const uint32_t bits = *reinterpret_cast<const uint32_t*>(&e);
          pp[i2] = bits;
          const float2 pf = make_float2(__uint_as_float(bits << 16), __uint_as_float(bits & 0xFFFF0000u));
          const float2 dd = __fadd2_rn(make_float2(__uint_as_float(dv[2 * i2]), __uint_as_float(dv[2 * i2 + 1])), nd);
          const float2 dsf = __fmul2_rn(pf, dd);
          ds[i2] = pack_bf16(dsf.x, dsf.y);
        }
      }
      // 32 queries as bf16 = 16 packed columns, behind the 16 columns of the other warp of this lane quarter
      tmem_st16(tST + colhalf * 16, pp);
      tmem_st16(tDPT + colhalf * 16, ds);
      tc_wait_st();
      tc_fence_before_sync();
      mbar_arrive(&pds_full[hf & 1]);
    }
    if (ok && n_it > 0) {
      ok = mbar_wait(acc_done, 0u, p.status);
      ok = __all_sync(0xFFFFFFFFu, ok);
    }
    if (ok) {
      tc_fence_after_sync();
      const int64_t tok = k_begin + key;
      __nv_bfloat16* dkrow = p.dk + tok * p.dk_stride + static_cast<int64_t>(hkv) * D;
      __nv_bfloat16* dvrow = p.dv + tok * p.dv_stride + static_cast<int64_t>(hkv) * D;
      {
        const int which = colhalf;                         // one warp of the quarter writes dV, the other dK
        const uint32_t col = which == 0 ? kColDV : kColDK;
        const float sc = which == 0 ? 1.f : p.scale;
        __nv_bfloat16* orow = which == 0 ? dvrow : dkrow;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t ov[32];
          if (n_it > 0) {
            tmem_ld32(tmem_base + lane_off + col + c * 32, ov);
            tc_wait_ld();
          } else {
#pragma unroll
            for (int i2 = 0; i2 < 32; ++i2) ov[i2] = 0u;
          }
          if (key_valid) {
#pragma unroll
            for (int i2 = 0; i2 < 4; ++i2) {
              uint4 v;
              v.x = pack_bf16(__uint_as_float(ov[8 * i2 + 0]) * sc, __uint_as_float(ov[8 * i2 + 1]) * sc);
              v.y = pack_bf16(__uint_as_float(ov[8 * i2 + 2]) * sc, __uint_as_float(ov[8 * i2 + 3]) * sc);
              v.z = pack_bf16(__uint_as_float(ov[8 * i2 + 4]) * sc, __uint_as_float(ov[8 * i2 + 5]) * sc);
              v.w = pack_bf16(__uint_as_float(ov[8 * i2 + 6]) * sc, __uint_as_float(ov[8 * i2 + 7]) * sc);
              *reinterpret_cast<uint4*>(orow + c * 32 + i2 * 8) = v;
            }
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

// delta[h, t] = sum_d dO[t,h,d] * O[t,h,d]   (one warp per (token, head))
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ dout,
                                  float* __restrict__ delta, int64_t total_q, int hq, int D, int64_t o_stride,
                                  int64_t do_stride) {
  const int lane = threadIdx.x & 31;
  const int64_t w = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (w >= total_q * hq) return;
  const int64_t t = w / hq;
  const int h = static_cast<int>(w % hq);
  const __nv_bfloat16* orow = o + t * o_stride + static_cast<int64_t>(h) * D;
  const __nv_bfloat16* drow = dout + t * do_stride + static_cast<int64_t>(h) * D;
  float s = 0.f;
  for (int d = lane * 2; d < D; d += 64) {
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(orow + d));
    const float2 c = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(drow + d));
    s += a.x * c.x + a.y * c.y;
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, off);
  if (lane == 0) delta[static_cast<int64_t>(h) * total_q + t] = s;
}

}  // namespace yv
