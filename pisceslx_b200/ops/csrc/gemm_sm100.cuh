// Persistent, warp-specialised bf16 GEMM for sm_100a: TMA -> 128B-swizzled shared memory ->
// tcgen05.mma (UMMA 128 x BN x 16, fp32 accumulators in TMEM, double buffered) -> tcgen05.ld ->
// shared staging -> TMA store (or TMA reduce-add when accumulating into C).
//
// One CTA per SM, 192 threads:
//   warp 0      TMA producer (one elected lane)
//   warp 1      TMEM allocation + MMA issue (one elected lane)
//   warps 2..5  epilogue (each owns the 32 TMEM lanes  32*(warp%4) .. +31)
//
// Three problem modes share the main loop:
//   kDense     C[M,N]          = A[M,K] * B
//   kGroupedM  C[rows,N]       = A[rows,K] * B[expert(tile)]      rows are expert-sorted and each
//                                 expert's segment is padded to a multiple of 128 rows
//   kGroupedK  C[e][M,N]       = A[:, seg(e)] * B[seg(e), :]       the reduction runs over expert e's
//                                 row segment (weight gradients of the grouped expert GEMMs)
//   kBatched   C[g][M,N]       = A[g] * B[g]                        equal-shaped problems stacked along the
//                                 outer dimension of every operand (Muon's Newton-Schulz iterations)
// Operand layouts are template flags: K-major ("row-major [rows, K]") or MN-major ("row-major [K, rows]").
#pragma once
#include "sm100.cuh"

namespace yv {

enum GemmMode : int { kDense = 0, kGroupedM = 1, kGroupedK = 2, kBatched = 3 };

struct GemmParams {
  CUtensorMap tma_a;
  CUtensorMap tma_b;
  CUtensorMap tma_c;
  int M, N, K;                 // per-problem extents (kGroupedM: M = max rows; kGroupedK: K unused)
  int mode;
  int accumulate;              // 1: C += result through TMA reduce-add
  int num_groups;              // experts (grouped modes)
  int b_group_stride;          // kGroupedM: outer-dim rows of B per expert
  int c_group_stride;          // kGroupedK / kBatched: rows of C per group
  int a_group_stride;          // kBatched: outer-dim rows of A per batch entry
  const int* tile_expert;      // kGroupedM: expert id of every 128-row tile
  const int* tile_rows;        // kGroupedM (optional): index of the 128-row tile in A / C for every listed tile
  int tile_rows_c_only;        // 1: the list addresses C only, A is compact (listed tile j = rows 128 j .. of A)
  const int* num_m_tiles;      // kGroupedM: number of valid 128-row tiles (device scalar)
  const int* seg_offsets;      // kGroupedK: [E+1] row offsets of the expert segments (multiples of 128)
  uint32_t* status;            // device status word (0 = ok)
  // ---- fused tensor-parallel collectives (template parameter COMM != 0; dense mode, K-major A, bf16 C) ----
  // COMM 1, all-gather -> GEMM: A = the local gathered buffer [world * rows_per_rank, K]; extra warps in every CTA
  //   pull the peers' shards into it and count the vectors landed per 128-row block in comm_flags; the
  //   TMA producer waits for a block's count before it loads tiles of that block.  Own rows come first.
  // COMM 2, GEMM -> reduce-scatter: tiles whose rows another rank owns are stored straight into that rank's inbox
  //   [source rank][rows_per_rank, N] as 128-byte row segments; own rows go to C as usual and come last.
  int comm_world, comm_rank;
  int comm_blocks_per_rank;    // 128-row blocks per rank
  void* comm_peer[8];          // COMM 1: peers' published shards; COMM 2: peers' inboxes
  uint8_t* comm_local;         // COMM 1: base of the local gathered A
  uint32_t* comm_flags;        // COMM 1: one counter per 128-row block, zeroed before the launch
  uint32_t comm_flag_target;   // COMM 1: count that marks a block complete (= 16-byte vectors per block)
  long long comm_row_bytes;    // COMM 1: bytes per row of A; COMM 2: bytes per row of an inbox
  // ---- fp8 inputs (template parameter FP8): e4m3 operands, K-major, 128 elements per shared-memory row; the
  // epilogue multiplies the fp32 accumulator by *out_scale (= scale_a * scale_b of per-tensor scaling) ----
  const float* out_scale;
  // ---- block-scaled fp8 (template parameter FP8 == 2, "MX"): one e8m0 scale per 32 elements of K of every row of A
  // and of B.  Scales are stored in 512-byte chunks, one per (128 rows, 128 elements of K): byte
  // (r % 32) * 16 + (r / 32) * 4 + j holds row r, 32-element block j; chunk (row tile i, K chunk c) sits at
  // (i * sf_kchunks + c) * 512.  sf_b_tiles = 128-row tiles of B that have scales ----
  const uint8_t* sfa;
  const uint8_t* sfb;
  int sf_kchunks;
  int sf_b_tiles;
  // ---- affine epilogue (bf16 output, no fused collective): C = epi_c * (A B) + epi_b * epi_cin + epi_a * I, with
  // epi_cin laid out like C; the identity is per group in the batched mode ----
  const __nv_bfloat16* epi_cin;
  float epi_a, epi_b, epi_c;
  // ---- symmetric output (batched mode, M == N, bf16): tiles entirely below the diagonal are skipped and filled by
  // the mirrored stores of the computed tiles; sym_tiles = computed tiles per group, sym_c = C as a plain pointer ----
  int symmetric;
  int sym_tiles;
  __nv_bfloat16* sym_c;
};

constexpr int kBM = 128;
constexpr int kBK = 64;
constexpr int kGemmThreads = 192;
constexpr int kCopierWarps = 4;              // warps per CTA that pull the peers' shards (all-gather mode)
constexpr int kGemmThreadsAllGather = kGemmThreads + 32 * kCopierWarps;
constexpr int kGroupBand = 16;   // m-tiles per rasterisation band

template <int BN, bool MX = false>
struct GemmSmem {
  static constexpr int kStages = ((BN == 256) ? 4 : 6) - (MX ? 1 : 0);
  static constexpr int kSfBytes = MX ? 512 * (1 + BN / 128) : 0;     // scale factors of one stage: A, then B
  static constexpr int kABytes = kBM * kBK * 2;
  static constexpr int kBBytes = BN * kBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kEpiBytes = kBM * 128;            // 128 rows x 128 B per staging buffer
  static constexpr int kEpiBufs = 2;
  static constexpr int kBarrierBytes = 256;
  static constexpr int kTotal = kStages * (kStageBytes + kSfBytes) + kEpiBufs * kEpiBytes + kBarrierBytes + 1024;
};

struct TileCoord {
  int a_x, a_y;      // TMA coordinates of the first A box (x = inner)
  int b_x, b_y;
  int c_x, c_y;
  int k_iters;
  int m_blk;         // 128-row block of A / C this tile covers
};

// Decode linear tile index -> coordinates.  Returns false when idx is past the end.
template <int BN, bool A_MN, bool B_MN, int COMM = 0, int FP8 = 0>
__device__ __forceinline__ bool decode_tile(const GemmParams& p, int idx, int tiles_m, int tiles_n, TileCoord& t) {
  int m_blk, n_blk, group = 0;
  if (p.mode == kBatched && p.symmetric) {
    // column tile j keeps the row tiles that start above the column tile's last column: i * 128 < (j + 1) * BN
    group = idx / p.sym_tiles;
    if (group >= p.num_groups) return false;
    int r = idx - group * p.sym_tiles;
    int j = 0;
    for (;; ++j) {
      const int kept = min(tiles_m, (j + 1) * (BN / kBM));
      if (r < kept) break;
      r -= kept;
    }
    n_blk = j;
    m_blk = r;
  } else if (p.mode == kGroupedK || p.mode == kBatched) {
    const int per_group = tiles_m * tiles_n;
    group = idx / per_group;
    if (group >= p.num_groups) return false;
    const int r = idx - group * per_group;
    n_blk = r / tiles_m;
    m_blk = r - n_blk * tiles_m;
  } else {
    if (idx >= tiles_m * tiles_n) return false;
    const int band_tiles = kGroupBand * tiles_n;
    const int band = idx / band_tiles;
    const int r = idx - band * band_tiles;
    const int band_m = min(kGroupBand, tiles_m - band * kGroupBand);
    n_blk = r / band_m;
    m_blk = band * kGroupBand + (r - n_blk * band_m);
    if (COMM != 0) {
      // rotate the row blocks: all-gather starts with the rows this rank already holds, reduce-scatter ends with them
      const int shift = (COMM == 1 ? p.comm_rank : p.comm_rank + 1) * p.comm_blocks_per_rank;
      m_blk = (m_blk + shift) % tiles_m;
    }
  }
  // grouped-M problems may list their 128-row tiles explicitly (receive regions of several sources)
  const int row_tile = (p.mode == kGroupedM && p.tile_rows != nullptr) ? p.tile_rows[m_blk] : m_blk;
  const int m0 = row_tile * kBM, n0 = n_blk * BN;
  const int m0_a = (p.mode == kGroupedM && p.tile_rows_c_only) ? m_blk * kBM : m0;
  int k_begin = 0, k_len = p.K;
  int a_outer_off = 0, b_outer_off = 0, c_row_off = 0;
  if (p.mode == kBatched) {
    a_outer_off = group * p.a_group_stride;
    b_outer_off = group * p.b_group_stride;
    c_row_off = group * p.c_group_stride;
  } else if (p.mode == kGroupedM) {
    const int e = p.tile_expert[m_blk];
    b_outer_off = e * p.b_group_stride;
  } else if (p.mode == kGroupedK) {
    k_begin = p.seg_offsets[group];
    k_len = p.seg_offsets[group + 1] - k_begin;
    c_row_off = group * p.c_group_stride;
  }
  constexpr int kBKe = FP8 ? 2 * kBK : kBK;          // elements of K per pipeline stage (128 bytes per row)
  t.k_iters = (k_len + kBKe - 1) / kBKe;
  if (A_MN) { t.a_x = m0_a; t.a_y = a_outer_off + k_begin; } else { t.a_x = k_begin; t.a_y = a_outer_off + m0_a; }
  if (B_MN) { t.b_x = n0; t.b_y = b_outer_off + k_begin; } else { t.b_x = k_begin; t.b_y = b_outer_off + n0; }
  t.c_x = n0;
  t.c_y = c_row_off + m0;
  t.m_blk = row_tile;
  return true;
}

template <int BN, bool A_MN, bool B_MN, typename OutT, int COMM = 0, int FP8 = 0>
__global__ void __launch_bounds__(kGemmThreadsAllGather, 1) gemm_sm100_kernel(const __grid_constant__ GemmParams p) {
  constexpr bool MX = (FP8 == 2);
  using S = GemmSmem<BN, MX>;
  constexpr int kStages = S::kStages;
  constexpr int kColsPerChunk = 128 / sizeof(OutT);       // columns covered by one 128-byte staging row
  constexpr int kChunks = BN / kColsPerChunk;
  // block-scaled mode keeps the scale factors in tensor memory behind the accumulators: 4 columns for A's 128 rows
  // and 4 per 128 columns of B; with 256-wide tiles that leaves room for one accumulator instead of two
  constexpr int kAccBufs = (MX && BN == 256) ? 1 : 2;
  constexpr uint32_t kTmemCols = MX ? 512 : ((2 * BN <= 512) ? 2 * BN : 512);
  constexpr uint32_t kSfaCol = kAccBufs * BN;
  constexpr uint32_t kSfbCol = kSfaCol + 4;
  static_assert(!FP8 || (!A_MN && !B_MN), "fp8 operands are K-major");
  constexpr int kBKe = FP8 ? 2 * kBK : kBK;
  constexpr uint32_t kIdesc = MX ? make_idesc_mxf8(kBM, BN)
                                 : (FP8 ? make_idesc_e4m3(kBM, BN) : make_idesc_bf16(kBM, BN, A_MN, B_MN));

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_epi = smem + kStages * S::kStageBytes;
  uint8_t* smem_sf = smem_epi + S::kEpiBufs * S::kEpiBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_sf + kStages * S::kSfBytes);
  uint64_t* full_bar = bars;                       // [kStages]
  uint64_t* empty_bar = bars + kStages;            // [kStages]
  uint64_t* acc_full = bars + 2 * kStages;         // [2]
  uint64_t* acc_empty = bars + 2 * kStages + 2;    // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  int tiles_m, tiles_n;
  tiles_n = (p.N + BN - 1) / BN;
  if (p.mode == kGroupedM) {
    tiles_m = *p.num_m_tiles;
  } else {
    tiles_m = (p.M + kBM - 1) / kBM;
  }

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&p.tma_a);
    tma_prefetch_desc(&p.tma_b);
    tma_prefetch_desc(&p.tma_c);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&acc_full[s], 1);
      mbar_init(&acc_empty[s], 1);
    }
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
    // ------------------------------- TMA producer -------------------------------------------
    if (elect_one()) {
      uint32_t it = 0;
      bool ok = true;
      for (int idx = blockIdx.x; ok; idx += gridDim.x) {
        TileCoord t;
        if (!decode_tile<BN, A_MN, B_MN, COMM, FP8>(p, idx, tiles_m, tiles_n, t)) break;
        if (COMM == 1 && t.m_blk / p.comm_blocks_per_rank != p.comm_rank) {
          // rows of another rank: the copier warps of all CTAs must have landed this block in local memory
          const volatile uint32_t* flag = p.comm_flags + t.m_blk;
          const uint64_t t0 = globaltimer_ns();
          uint32_t spins = 0;
          while (ld_acquire_gpu(const_cast<const uint32_t*>(flag)) < p.comm_flag_target) {
            if ((++spins & 0x3Fu) == 0u) {
              if (globaltimer_ns() - t0 > YV_WAIT_LIMIT_NS) {
                if (p.status != nullptr) atomicOr(p.status, kStatusPeerTimeout);
                ok = false;
                break;
              }
              __nanosleep(100);
            }
          }
          if (!ok) break;
          fence_proxy_async_all();      // the block was written by generic-proxy stores; TMA reads it next
        }
        for (int k = 0; k < t.k_iters && ok; ++k, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1u;
          ok = mbar_wait(&empty_bar[s], ph ^ 1u, p.status);
          if (!ok) break;
          uint8_t* sa = smem + s * S::kStageBytes;
          uint8_t* sb = sa + S::kABytes;
          if (MX) {
            // scale factors of this stage: one 512-byte chunk for A's rows and one per 128 columns of B
            const int b_tile = t.b_y / kBM;
            const int nb = min(BN / kBM, p.sf_b_tiles - b_tile);
            mbar_expect_tx(&full_bar[s], S::kStageBytes + 512u * static_cast<uint32_t>(1 + nb));
            uint8_t* ssf = smem_sf + s * S::kSfBytes;
            bulk_load_1d(ssf, p.sfa + (static_cast<int64_t>(t.a_y / kBM) * p.sf_kchunks + k) * 512, 512, &full_bar[s]);
            for (int j = 0; j < nb; ++j)
              bulk_load_1d(ssf + 512 * (1 + j), p.sfb + (static_cast<int64_t>(b_tile + j) * p.sf_kchunks + k) * 512, 512,
                           &full_bar[s]);
          } else {
            mbar_expect_tx(&full_bar[s], S::kStageBytes);
          }
          if (A_MN) {
#pragma unroll
            for (int j = 0; j < kBM / 64; ++j)
              tma_load_2d(sa + j * (kBK * 128), &p.tma_a, &full_bar[s], t.a_x + j * 64, t.a_y + k * kBK);
          } else {
            tma_load_2d(sa, &p.tma_a, &full_bar[s], t.a_x + k * kBKe, t.a_y);
          }
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(sb + j * (kBK * 128), &p.tma_b, &full_bar[s], t.b_x + j * 64, t.b_y + k * kBK);
          } else {
            tma_load_2d(sb, &p.tma_b, &full_bar[s], t.b_x + k * kBKe, t.b_y);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer ---------------------------------------------
    if (elect_one()) {
      uint32_t it = 0, tile_it = 0;
      bool ok = true;
      for (int idx = blockIdx.x; ok; idx += gridDim.x, ++tile_it) {
        TileCoord t;
        if (!decode_tile<BN, A_MN, B_MN, COMM, FP8>(p, idx, tiles_m, tiles_n, t)) break;
        const int acc = tile_it % kAccBufs;
        const uint32_t acc_ph = (tile_it / kAccBufs) & 1u;
        ok = mbar_wait(&acc_empty[acc], acc_ph ^ 1u, p.status);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(acc * BN);
        for (int k = 0; k < t.k_iters && ok; ++k, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1u;
          ok = mbar_wait(&full_bar[s], ph, p.status);
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + s * S::kStageBytes);
          const uint32_t sb = sa + S::kABytes;
          if (MX) {
            const uint32_t ssf = smem_u32(smem_sf + s * S::kSfBytes);
            tc_cp_32x128b_warpx4(tmem_base + kSfaCol, make_smem_desc_rows16(ssf));
#pragma unroll
            for (int j = 0; j < BN / kBM; ++j)
              tc_cp_32x128b_warpx4(tmem_base + kSfbCol + 4 * j, make_smem_desc_rows16(ssf + 512 * (1 + j)));
          }
#pragma unroll
          for (int kk = 0; kk < kBK / 16; ++kk) {
            const uint64_t da = A_MN ? make_smem_desc(sa + kk * 2048, kBK * 128, 1024)
                                     : make_smem_desc(sa + kk * 32, 16, 1024);
            const uint64_t db = B_MN ? make_smem_desc(sb + kk * 2048, kBK * 128, 1024)
                                     : make_smem_desc(sb + kk * 32, 16, 1024);
            if (MX) {
              // 32-element block kk of this stage: byte kk of the scale-factor columns
              tc_mma_mxf8_ss(tmem_d, da, db, kIdesc | (static_cast<uint32_t>(kk) << 29) | (static_cast<uint32_t>(kk) << 4),
                             tmem_base + kSfaCol, tmem_base + kSfbCol, (k | kk) != 0 ? 1u : 0u);
            } else if (FP8) {
              tc_mma_f8_ss(tmem_d, da, db, kIdesc, (k | kk) != 0 ? 1u : 0u);
            } else {
              tc_mma_f16_ss(tmem_d, da, db, kIdesc, (k | kk) != 0 ? 1u : 0u);
            }
          }
          tc_commit(&empty_bar[s]);     // releases the stage once these MMAs have read it
        }
        if (!ok) break;
        if (t.k_iters > 0) {
          tc_commit(&acc_full[acc]);
        } else {
          mbar_arrive(&acc_full[acc]);  // empty reduction: the epilogue writes zeros
        }
      }
    }
  } else if (COMM == 1 && warp >= 6) {
    // ------------------------------- all-gather copiers ---------------------------------------
    // The remote rows, taken in the order in which the tiles need their 128-row blocks, form one sequence of
    // 16-byte vectors.  All copier lanes of the grid walk it in rounds of kRound vectors per lane: every load of a
    // round is issued before the first store, so a round keeps several MB in flight over NVLink.  After its stores
    // a warp adds, for each block the round touched, the number of vectors it landed to that block's counter; a
    // block is complete when its counter reaches the number of vectors in a block.
    constexpr int kRound = 16;
    const int bpr = p.comm_blocks_per_rank;
    const int64_t vpb = (static_cast<int64_t>(kBM) * p.comm_row_bytes) >> 4;          // vectors per block
    const int64_t total = static_cast<int64_t>(tiles_m - bpr) * vpb;
    const int64_t lanes = static_cast<int64_t>(gridDim.x) * kCopierWarps * 32;
    const int64_t me = (static_cast<int64_t>(blockIdx.x) * kCopierWarps + (warp - 6)) * 32 + lane;
    // 64-bit divisions cost a few hundred instructions each on this machine: the block index of a vector is taken
    // with a shift when the block holds a power-of-two number of vectors (K a power of two), and is computed once
    // per vector and kept in registers for the store and the counting below.
    const int vshift = (vpb & (vpb - 1)) == 0 ? 63 - __clzll(vpb) : -1;
    const int rot = bpr + p.comm_rank * bpr;               // < tiles_m: one conditional subtraction wraps lb + rot
    for (int64_t base = 0; base < total; base += lanes * kRound) {
      uint4 v[kRound];
      int lbv[kRound];                                     // block of vector u in copy order, -1 past the end
      int64_t dst[kRound];                                 // its offset (in vectors) in the local gathered matrix
#pragma unroll
      for (int u = 0; u < kRound; ++u) {
        const int64_t g = base + static_cast<int64_t>(u) * lanes + me;
        lbv[u] = -1;
        if (g < total) {
          const int lb = vshift >= 0 ? static_cast<int>(g >> vshift) : static_cast<int>(g / vpb);
          const int64_t within = g - static_cast<int64_t>(lb) * vpb;
          int phys = lb + rot;
          if (phys >= tiles_m) phys -= tiles_m;
          const int owner = phys / bpr;
          lbv[u] = lb;
          dst[u] = static_cast<int64_t>(phys) * vpb + within;
          v[u] = ld_peer_v4(reinterpret_cast<const uint4*>(p.comm_peer[owner]) +
                            (static_cast<int64_t>(phys - owner * bpr) * vpb + within));
        }
      }
#pragma unroll
      for (int u = 0; u < kRound; ++u)
        if (lbv[u] >= 0) reinterpret_cast<uint4*>(p.comm_local)[dst[u]] = v[u];
      __threadfence();
      // blocks touched by this round (identical for every lane of the grid)
      const int64_t round_end = (base + lanes * kRound < total ? base + lanes * kRound : total) - 1;
      const int lb_first = vshift >= 0 ? static_cast<int>(base >> vshift) : static_cast<int>(base / vpb);
      const int lb_last = vshift >= 0 ? static_cast<int>(round_end >> vshift) : static_cast<int>(round_end / vpb);
      for (int lb = lb_first; lb <= lb_last; ++lb) {
        int mine = 0;
#pragma unroll
        for (int u = 0; u < kRound; ++u) mine += (lbv[u] == lb) ? 1 : 0;
        const int cnt = __reduce_add_sync(0xFFFFFFFFu, mine);
        int phys = lb + rot;
        if (phys >= tiles_m) phys -= tiles_m;
        if (lane == 0 && cnt > 0) atomicAdd(p.comm_flags + phys, static_cast<uint32_t>(cnt));
      }
    }
  } else if (warp >= 6) {
    // no role (the kernel was launched with the all-gather block size without the all-gather mode)
  } else {
    // ------------------------------- epilogue -------------------------------------------------
    const int quarter = warp & 3;                      // TMEM lane quarter this warp may access
    const int row = quarter * 32 + lane;               // row of the tile owned by this thread
    const bool issuer = (threadIdx.x == 64);           // first epilogue thread issues the TMA stores
    uint32_t tile_it = 0, chunk_it = 0;
    bool ok = true;
    for (int idx = blockIdx.x; ok; idx += gridDim.x, ++tile_it) {
      TileCoord t;
      if (!decode_tile<BN, A_MN, B_MN, COMM, FP8>(p, idx, tiles_m, tiles_n, t)) break;
      const int acc = tile_it % kAccBufs;
      const uint32_t acc_ph = (tile_it / kAccBufs) & 1u;
      ok = mbar_wait(&acc_full[acc], acc_ph, p.status);
      // all 128 epilogue threads must take the same branch: barrier with an AND reduction
      {
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
        ok = all_ok != 0u;
      }
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + static_cast<uint32_t>(acc * BN) + (static_cast<uint32_t>(quarter * 32) << 16);
      // reduce-scatter push: tiles of rows that another rank owns leave through the staging buffer as 128-byte
      // row segments written into the owner's inbox, inbox[source = this rank][row inside the owner's shard][column]
      bool remote_tile = false;
      uint8_t* remote_base = nullptr;
      if (COMM == 2 && sizeof(OutT) == 2) {
        const int owner = t.m_blk / p.comm_blocks_per_rank;
        remote_tile = owner != p.comm_rank;
        const int64_t rows_per_rank = static_cast<int64_t>(p.comm_blocks_per_rank) * kBM;
        const int64_t in_row0 = static_cast<int64_t>(t.m_blk - owner * p.comm_blocks_per_rank) * kBM;
        remote_base = static_cast<uint8_t*>(p.comm_peer[owner]) +
                      (static_cast<int64_t>(p.comm_rank) * rows_per_rank + in_row0) * p.comm_row_bytes;
      }
#pragma unroll 1
      for (int c = 0; c < kChunks; ++c, ++chunk_it) {
        uint8_t* buf = smem_epi + (chunk_it & 1) * S::kEpiBytes;
        // the store that last used this buffer (two chunks ago) must have finished reading it
        if (issuer) tma_store_wait_read<1>();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        uint32_t packed[32];
        if (sizeof(OutT) == 2) {
          uint32_t v0[32], v1[32];
          if (t.k_iters > 0) {
            tmem_ld32(taddr + c * 64, v0);
            tmem_ld32(taddr + c * 64 + 32, v1);
            tc_wait_ld();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) { v0[i] = 0u; v1[i] = 0u; }
          }
          const float osc = (FP8 == 1 && p.out_scale != nullptr) ? *p.out_scale : 1.f;
          if (!FP8 && COMM == 0 && p.epi_cin != nullptr) {
            // out = epi_c * acc + epi_b * Cin + epi_a * I: the Newton-Schulz polynomial b A + c A^2 (+ a I) formed in
            // the epilogue of the A * A product, Cin = A in the layout of C (N a multiple of 64)
            const int col0 = t.c_x + c * kColsPerChunk;
            const bool in = col0 + kColsPerChunk <= p.N;
            const uint4* src = reinterpret_cast<const uint4*>(p.epi_cin + static_cast<int64_t>(t.c_y + row) * p.N + col0);
            uint4 cin[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) cin[j] = in ? src[j] : make_uint4(0u, 0u, 0u, 0u);
            const __nv_bfloat16* cb = reinterpret_cast<const __nv_bfloat16*>(cin);
            const int lrow = (p.c_group_stride > 0 ? t.c_y % p.c_group_stride : t.c_y) + row;
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const int ca = col0 + 2 * i, cbk = col0 + 32 + 2 * i;
              const float a0 = p.epi_c * __uint_as_float(v0[2 * i]) + p.epi_b * __bfloat162float(cb[2 * i]) + (lrow == ca ? p.epi_a : 0.f);
              const float a1 = p.epi_c * __uint_as_float(v0[2 * i + 1]) + p.epi_b * __bfloat162float(cb[2 * i + 1]) + (lrow == ca + 1 ? p.epi_a : 0.f);
              const float b0 = p.epi_c * __uint_as_float(v1[2 * i]) + p.epi_b * __bfloat162float(cb[32 + 2 * i]) + (lrow == cbk ? p.epi_a : 0.f);
              const float b1 = p.epi_c * __uint_as_float(v1[2 * i + 1]) + p.epi_b * __bfloat162float(cb[33 + 2 * i]) + (lrow == cbk + 1 ? p.epi_a : 0.f);
              packed[i] = pack_bf16(a0, a1);
              packed[16 + i] = pack_bf16(b0, b1);
            }
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              packed[i] = pack_bf16(__uint_as_float(v0[2 * i]) * osc, __uint_as_float(v0[2 * i + 1]) * osc);
              packed[16 + i] = pack_bf16(__uint_as_float(v1[2 * i]) * osc, __uint_as_float(v1[2 * i + 1]) * osc);
            }
          }
        } else {
          if (t.k_iters > 0) {
            tmem_ld32(taddr + c * 32, packed);
            tc_wait_ld();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) packed[i] = 0u;
          }
        }
        if (sizeof(OutT) == 2 && COMM == 0 && !FP8 && p.symmetric) {
          // mirrored elements C[col][row] = C[row][col] for the positions whose own tile was skipped.  For a fixed
          // column the 32 lanes of a warp hold 32 consecutive rows: every store instruction writes 64 contiguous bytes.
          const int grp_rows = p.c_group_stride;
          const int lrow = t.c_y % grp_rows + row;                       // row inside the matrix
          __nv_bfloat16* cbase = p.sym_c + static_cast<int64_t>(t.c_y - t.c_y % grp_rows) * p.N;
          const int row_tile_end = (lrow / BN + 1) * BN;                 // end of the column tile that holds `lrow` as a column
          const int col0 = t.c_x + c * kColsPerChunk;
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            // packed[i] (i < 16) holds columns 2i, 2i+1 of the chunk; packed[16 + i] holds columns 32 + 2i, 33 + 2i
            const int cc = col0 + (i < 16 ? 2 * i : 32 + 2 * (i - 16));
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const int gcol = cc + h;
              // the mirror position (gcol, lrow) lies in row tile gcol / 128 and column tile lrow / BN: skipped iff
              // that column tile ends at or before the row tile starts
              if (gcol < p.N && row_tile_end <= (gcol / kBM) * kBM && lrow < p.N) {
                const uint16_t bits = static_cast<uint16_t>(h == 0 ? (packed[i] & 0xffffu) : (packed[i] >> 16));
                reinterpret_cast<uint16_t*>(cbase)[static_cast<int64_t>(gcol) * p.N + lrow] = bits;
              }
            }
          }
        }
        // 128-byte row, eight 16-byte pieces, XOR-swizzled with the row index (TMA SWIZZLE_128B)
        uint4* rowp = reinterpret_cast<uint4*>(buf + row * 128);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          uint4 v = make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
          rowp[j ^ (row & 7)] = v;
        }
        fence_proxy_async_smem();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (COMM == 2 && remote_tile) {
          const int col0 = t.c_x + c * kColsPerChunk;
          if (col0 < p.N) {
            const int tid = threadIdx.x - 64;             // 0..127 over the epilogue warps
            const int piece = tid & 7;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int r = i * 16 + (tid >> 3);
              const uint4 v = *reinterpret_cast<const uint4*>(buf + r * 128 + ((piece ^ (r & 7)) << 4));
              *reinterpret_cast<uint4*>(remote_base + static_cast<int64_t>(r) * p.comm_row_bytes +
                                        static_cast<int64_t>(col0) * 2 + (piece << 4)) = v;
            }
          }
        } else if (issuer) {
          if (p.accumulate) {
            tma_reduce_add_2d(&p.tma_c, buf, t.c_x + c * kColsPerChunk, t.c_y);
          } else {
            tma_store_2d(&p.tma_c, buf, t.c_x + c * kColsPerChunk, t.c_y);
          }
          tma_store_commit();
        }
      }
      // all TMEM reads of this accumulator are done: hand it back to the MMA warp
      tc_fence_before_sync();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (issuer) mbar_arrive(&acc_empty[acc]);
    }
    if (issuer) tma_store_wait_all<0>();
  }

  // ------------------------------- teardown ---------------------------------------------------
  tc_fence_before_sync();
  __syncthreads();
  if (p.status != nullptr && *reinterpret_cast<volatile uint32_t*>(p.status) != 0u) {
    // A wait ran out somewhere: give copies that may still be in flight time to land before the
    // shared memory and TMEM of this CTA are released.
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
