// Product-quantised knowledge field -> FiLM modulation of the residual stream, one kernel:
//
//   e[t]    = sum_c table[c][idx[t][c]]                     (16 entries of 128 dims per token; the table is sharded by
//                                                            rows over the ranks of a group, entries are read from the
//                                                            owner's memory with 16-byte peer loads)
//   s | b   = e[t] @ W^T                                    (W [2H, 128]: rows 0..H-1 scale, H..2H-1 shift)
//   out[t]  = h[t] * (1 + s) + b
//
// A CTA owns 128 tokens.  Nine of its warps first gather and sum the tokens' entries into shared memory (meanwhile
// the producer warp already prefetches h tiles), already in
// the 128-byte-swizzled K-major layout the tensor cores read (the "A" operand, 128 x 128 bf16, written once).  Then
// the CTA walks the H / 64 column tiles: a producer thread streams the tile's 64 scale rows and 64 shift rows of W
// (one 128-wide "B" operand, three buffers) and the matching 128 x 64 tile of h (five buffers, so that loads run four
// tiles ahead of the stores: a memory-bound kernel needs about 100 KB in flight per SM) with TMA, one thread issues eight tcgen05 MMAs into one of two 128-column accumulators
// in tensor memory, and eight epilogue warps read scale and shift from tensor memory, modulate the h tile in shared
// memory and send it out with a TMA store.  Neither e, nor scale, nor shift touches
// device memory (e is written out only when the caller asks for it, for the backward pass).
#include "per_device.h"
#include "sm100.cuh"
#include "tensormap.h"
#include "yv_comm.h"
#include "yv_ops.h"

namespace yv {

namespace {

constexpr int kPqD = 128;                 // entry dimension = reduction length of the projection
constexpr int kPqTile = 128;              // tokens per CTA tile
constexpr int kPqCols = 64;               // output columns per column tile (the MMA is 2 * kPqCols wide)
constexpr int kPqHBufs = 5;               // h tile buffers: four tiles of loads in flight per SM
constexpr int kPqBStages = 3;             // W tile buffers: the W stream (2 MB per CTA out of L2) is as latency-bound as h
constexpr int kPqThreads = 320;           // warp 0: TMA producer, warp 1: MMA issuer, warps 2-9: epilogue
constexpr int kPqMaxC = 16;

struct PqFilmParams {
  CUtensorMap tma_w;                      // W [2H, 128] bf16, box 64 (K) x 64 rows
  CUtensorMap tma_h;                      // h [T, H] bf16, box 64 columns x 128 rows
  CUtensorMap tma_out;                    // out [T, H] bf16, box 64 columns x 128 rows
  const void* table[8];                   // per rank: [C, rows_per_rank, 128] bf16
  const int* idx;                         // [T, C] global entry ids
  __nv_bfloat16* e_out;                   // [T, 128] or null
  long long tokens;
  long long rows_per_rank;
  int C, world, H;
  uint32_t* status;
};

struct PqSmem {
  static constexpr int kABytes = kPqTile * kPqD * 2;            // 32 KB: two 64-wide K halves of 16 KB
  static constexpr int kBBytes = 2 * kPqCols * kPqD * 2;        // 32 KB per stage: two K halves of 16 KB (128 rows each)
  static constexpr int kHBytes = kPqTile * kPqCols * 2;         // 16 KB: 128 rows of 128 bytes
  static constexpr int kStages = kPqBStages;
  static constexpr int kIdxBytes = kPqTile * kPqMaxC * 4;       // 8 KB: the tile's entry ids
  static constexpr int kTotal = kABytes + kStages * kBBytes + kPqHBufs * kHBytes + kIdxBytes + 256 + 1024;
};

// Bounded wait that also records WHICH wait of the pipeline gave up (bits 8..14 of the status word).
__device__ __forceinline__ bool pq_wait(uint64_t* bar, uint32_t parity, uint32_t* status, uint32_t where) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++spins & 0xFFu) == 0u) {
      if (status != nullptr && *reinterpret_cast<volatile uint32_t*>(status) != 0u) return false;
      if (globaltimer_ns() - t0 > YV_WAIT_LIMIT_NS) {
        if (status != nullptr) atomicOr(status, kStatusWaitTimeout | (0x100u << where));
        return false;
      }
    }
  }
}

__global__ void __launch_bounds__(kPqThreads, 1) pq_film_kernel(const __grid_constant__ PqFilmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem_a + PqSmem::kABytes;
  uint8_t* smem_h = smem_b + PqSmem::kStages * PqSmem::kBBytes;
  int* s_idx = reinterpret_cast<int*>(smem_h + kPqHBufs * PqSmem::kHBytes);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_h + kPqHBufs * PqSmem::kHBytes + PqSmem::kIdxBytes);
  uint64_t* acc_full = bars;                      // [2]
  uint64_t* acc_empty = bars + 2;                 // [2]
  uint64_t* b_full = bars + 4;                    // [kPqBStages] W tile landed
  uint64_t* b_empty = b_full + kPqBStages;        // [kPqBStages] MMAs that read the W tile are done
  uint64_t* h_full = b_empty + kPqBStages;        // [kPqHBufs] h tile landed
  uint64_t* h_empty = h_full + kPqHBufs;          // [kPqHBufs] the store that read the h buffer is done
  uint64_t* a_free = h_empty + kPqHBufs;          // MMAs of the current token tile are done with the A operand
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(a_free + 1);
  static_assert((4 + 2 * kPqBStages + 2 * kPqHBufs + 2) * 8 <= 256, "barrier area");

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tiles_m = static_cast<int>((p.tokens + kPqTile - 1) / kPqTile);
  const int tiles_n = p.H / kPqCols;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&p.tma_w);
    tma_prefetch_desc(&p.tma_h);
    tma_prefetch_desc(&p.tma_out);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&acc_full[s], 1);
      mbar_init(&acc_empty[s], 1);
    }
    for (int s = 0; s < kPqBStages; ++s) {
      mbar_init(&b_full[s], 1);
      mbar_init(&b_empty[s], 1);
    }
    for (int s = 0; s < kPqHBufs; ++s) {
      mbar_init(&h_full[s], 1);
      mbar_init(&h_empty[s], 1);
    }
    mbar_init(a_free, 1);
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  constexpr uint32_t kIdesc = make_idesc_bf16(kPqTile, 2 * kPqCols, false, false);

  uint32_t it = 0;          // column-tile iterations done by this CTA (all roles count alike)
  uint32_t m_it = 0;        // token tiles done by this CTA
  bool ok = true;
  for (int m = blockIdx.x; m < tiles_m; m += gridDim.x, ++m_it) {
    // ---------------------------- gather + sum: warps 1-9, 16 lanes per token ----------------------------
    // Random 256-byte rows of a table far larger than L2 and than the reach of an SM's address-translation cache:
    // the loop runs over the CODEBOOKS on the outside (two at a time) and over the half-warp's tokens inside, so that
    // at any moment the whole grid reads from two 32 MB codebooks (a few dozen 2 MB pages) instead of from all of
    // them.  The tile's ids are staged in shared memory with one coalesced pass first; every lane keeps 16
    // independent 16-byte loads in flight.
    if (warp != 0) {
      constexpr int kGatherThreads = kPqThreads - 32;                   // 288
      constexpr int kHalfWarps = kGatherThreads / 16;                   // 18
      constexpr int kRowsPerHw = (kPqTile + kHalfWarps - 1) / kHalfWarps;   // 8
      const int gt = threadIdx.x - 32;
      const long long t0 = static_cast<long long>(m) * kPqTile;
      const long long n_ids = (p.tokens - t0 < kPqTile ? p.tokens - t0 : kPqTile) * p.C;
      for (int i = gt; i < kPqTile * p.C; i += kGatherThreads) s_idx[i] = i < n_ids ? p.idx[t0 * p.C + i] : -1;
      asm volatile("bar.sync 2, 288;" ::: "memory");
      const int hw = gt >> 4;                                           // half-warp 0..17: rows hw, hw + 18, ...
      const int piece = lane & 15;                                      // 16-byte piece (8 dims) of the 256-byte entry
      const unsigned rpr = static_cast<unsigned>(p.rows_per_rank);
      float acc[kRowsPerHw][8];
#pragma unroll
      for (int i = 0; i < kRowsPerHw; ++i)
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[i][k] = 0.f;
      for (int c0 = 0; c0 < p.C; c0 += 2) {
        uint4 v[2][kRowsPerHw];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
#pragma unroll
          for (int i = 0; i < kRowsPerHw; ++i) {
            v[u][i] = make_uint4(0u, 0u, 0u, 0u);
            const int r = hw + kHalfWarps * i, c = c0 + u;
            if (r < kPqTile && c < p.C) {
              const int e = s_idx[r * p.C + c];
              if (e >= 0) {
                const unsigned owner = static_cast<unsigned>(e) / rpr;
                if (owner >= static_cast<unsigned>(p.world)) {
                  if (p.status != nullptr) atomicOr(p.status, kStatusIndexOutOfRange);
                } else {
                  const uint4* row = reinterpret_cast<const uint4*>(p.table[owner]) +
                                     (static_cast<long long>(c) * p.rows_per_rank + (static_cast<unsigned>(e) - owner * rpr)) * (kPqD / 8);
                  v[u][i] = ld_peer_v4(row + piece);
                }
              } else if (t0 + r < p.tokens && p.status != nullptr) {
                atomicOr(p.status, kStatusIndexOutOfRange);              // a negative id of a real token
              }
            }
          }
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
#pragma unroll
          for (int i = 0; i < kRowsPerHw; ++i) {
            const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&v[u][i]);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const float2 f = __bfloat1622float2(h2[k]);
              acc[i][2 * k] += f.x;
              acc[i][2 * k + 1] += f.y;
            }
          }
        }
      }
#pragma unroll
      for (int i = 0; i < kRowsPerHw; ++i) {
        const int r = hw + kHalfWarps * i;
        if (r < kPqTile) {
          uint4 o;
          o.x = pack_bf16(acc[i][0], acc[i][1]); o.y = pack_bf16(acc[i][2], acc[i][3]);
          o.z = pack_bf16(acc[i][4], acc[i][5]); o.w = pack_bf16(acc[i][6], acc[i][7]);
          // K half (piece >> 3), 16-byte slot (piece & 7) XOR-swizzled with the row: the layout TMA SWIZZLE_128B produces
          *reinterpret_cast<uint4*>(smem_a + (piece >> 3) * (kPqTile * 128) + r * 128 + (((piece & 7) ^ (r & 7)) << 4)) = o;
          if (p.e_out != nullptr && t0 + r < p.tokens) reinterpret_cast<uint4*>(p.e_out + (t0 + r) * kPqD)[piece] = o;
        }
      }
      fence_proxy_async_smem();        // generic-proxy writes of A before the tensor cores read it
      asm volatile("bar.sync 2, 288;" ::: "memory");      // the gathering warps; the producer does not wait
    }

    if (warp == 0) {
      // ---------------------------- TMA producer ----------------------------
      if (elect_one()) {
        uint32_t j = it;
        for (int n = 0; n < tiles_n && ok; ++n, ++j) {
          const int s = j % kPqBStages;
          const uint32_t ph = (j / kPqBStages) & 1u;
          ok = pq_wait(&b_empty[s], ph ^ 1u, p.status, 0);
          if (!ok) break;
          uint8_t* sb = smem_b + s * PqSmem::kBBytes;
          mbar_expect_tx(&b_full[s], PqSmem::kBBytes);
#pragma unroll
          for (int kh = 0; kh < 2; ++kh) {
            tma_load_2d(sb + kh * (2 * kPqCols * 128), &p.tma_w, &b_full[s], kh * 64, n * kPqCols);
            tma_load_2d(sb + kh * (2 * kPqCols * 128) + kPqCols * 128, &p.tma_w, &b_full[s], kh * 64, p.H + n * kPqCols);
          }
          const int hb = j % kPqHBufs;
          ok = pq_wait(&h_empty[hb], ((j / kPqHBufs) & 1u) ^ 1u, p.status, 1);
          if (!ok) break;
          mbar_expect_tx(&h_full[hb], PqSmem::kHBytes);
          tma_load_2d(smem_h + hb * PqSmem::kHBytes, &p.tma_h, &h_full[hb], n * kPqCols, m * kPqTile);
        }
      }
    } else if (warp == 1) {
      // ---------------------------- MMA issuer ----------------------------
      if (elect_one()) {
        uint32_t j = it;
        const uint32_t sa = smem_u32(smem_a);
        for (int n = 0; n < tiles_n && ok; ++n, ++j) {
          const int s = j & 1;                                  // accumulator
          const uint32_t ph = (j >> 1) & 1u;
          const int bs = j % kPqBStages;                        // W buffer
          ok = pq_wait(&acc_empty[s], ph ^ 1u, p.status, 2);
          if (!ok) break;
          ok = pq_wait(&b_full[bs], (j / kPqBStages) & 1u, p.status, 3);
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t sb = smem_u32(smem_b + bs * PqSmem::kBBytes);
          const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(s * 2 * kPqCols);
#pragma unroll
          for (int kk = 0; kk < kPqD / 16; ++kk) {
            const uint64_t da = make_smem_desc(sa + (kk >> 2) * (kPqTile * 128) + (kk & 3) * 32, 16, 1024);
            const uint64_t db = make_smem_desc(sb + (kk >> 2) * (2 * kPqCols * 128) + (kk & 3) * 32, 16, 1024);
            tc_mma_f16_ss(tmem_d, da, db, kIdesc, kk != 0 ? 1u : 0u);
          }
          tc_commit(&b_empty[bs]);
          tc_commit(&acc_full[s]);
        }
        if (ok) {
          tc_commit(a_free);
          ok = pq_wait(a_free, m_it & 1u, p.status, 4);     // A may be overwritten by the next token tile
        }
      }
    } else {
      // ---------------------------- epilogue: 8 warps, one token row and 32 of the 64 columns per thread -----------
      const int quarter = warp & 3;                  // tensor-memory lane quarter this warp may read
      const int colhalf = (warp - 2) >> 2;           // warps 2-5: columns 0-31, warps 6-9: columns 32-63
      const int row = quarter * 32 + lane;
      const bool issuer = (threadIdx.x == 64);
      uint32_t j = it;
      for (int n = 0; n < tiles_n; ++n, ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1u;
        const int hb = j % kPqHBufs;
        bool w = pq_wait(&acc_full[s], ph, p.status, 5);
        w = pq_wait(&h_full[hb], (j / kPqHBufs) & 1u, p.status, 6) && w;
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
              : "r"(static_cast<uint32_t>(w && ok))
              : "memory");
          ok = all_ok != 0u;
        }
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t taddr = tmem_base + static_cast<uint32_t>(s * 2 * kPqCols) + (static_cast<uint32_t>(quarter * 32) << 16);
        uint8_t* sh = smem_h + hb * PqSmem::kHBytes;
        {
          const int c = colhalf;
          uint32_t sc[32], sf[32];
          tmem_ld32(taddr + c * 32, sc);
          tmem_ld32(taddr + kPqCols + c * 32, sf);
          tc_wait_ld();
          uint8_t* hrow = sh + row * 128;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4* slot = reinterpret_cast<uint4*>(hrow + (((c * 4 + q) ^ (row & 7)) << 4));
            uint4 hv = *slot;
            __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&hv);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float2 f = __bfloat1622float2(h2[i]);
              const int k = q * 8 + 2 * i;
              const float o0 = f.x * (1.f + __uint_as_float(sc[k])) + __uint_as_float(sf[k]);
              const float o1 = f.y * (1.f + __uint_as_float(sc[k + 1])) + __uint_as_float(sf[k + 1]);
              h2[i] = __floats2bfloat162_rn(o0, o1);
            }
            *slot = hv;
          }
        }
        tc_fence_before_sync();
        fence_proxy_async_smem();
        asm volatile("bar.sync 1, 256;" ::: "memory");
        if (issuer) {
          mbar_arrive(&acc_empty[s]);
          tma_store_2d(&p.tma_out, sh, n * kPqCols, m * kPqTile);
          tma_store_commit();
          // the previous store has finished reading its buffer: hand that buffer back to the producer
          if (j > 0) {
            tma_store_wait_read<1>();
            mbar_arrive(&h_empty[(j - 1) % kPqHBufs]);
          }
        }
      }
    }
    it += static_cast<uint32_t>(tiles_n);
    __syncthreads();
    if (p.status != nullptr && *reinterpret_cast<volatile uint32_t*>(p.status) != 0u) break;
  }
  if (threadIdx.x == 64) tma_store_wait_all<0>();

  tc_fence_before_sync();
  __syncthreads();
  if (p.status != nullptr && *reinterpret_cast<volatile uint32_t*>(p.status) != 0u) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) { __nanosleep(1000); }
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 256);
  }
}

}  // namespace

int launch_pq_film(void* const* table_ptrs, int world, const int* idx, const void* w, const void* h, void* out,
                   void* e_out, int64_t tokens, int C, int64_t rows_per_rank, int D, int H, uint32_t* status,
                   cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (D != kPqD || C < 1 || C > kPqMaxC || world < 1 || world > 8 || H <= 0 || (H % kPqCols) != 0) return -1;
  PqFilmParams p;
  for (int i = 0; i < 8; ++i) p.table[i] = i < world ? table_ptrs[i] : nullptr;
  p.idx = idx;
  p.e_out = reinterpret_cast<__nv_bfloat16*>(e_out);
  p.tokens = tokens; p.rows_per_rank = rows_per_rank; p.C = C; p.world = world; p.H = H;
  p.status = status;
  int r = make_tmap_2d(&p.tma_w, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, w, kPqD, 2ull * H, kPqD, 64, kPqCols);
  if (r != 0) return -20 + r;
  r = make_tmap_2d(&p.tma_h, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, h, H, tokens, H, 64, kPqTile);
  if (r != 0) return -30 + r;
  r = make_tmap_2d(&p.tma_out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, out, H, tokens, H, 64, kPqTile);
  if (r != 0) return -40 + r;
  static PerDeviceInt configured;
  if (!configured.cur()) {
    cudaError_t e = cudaFuncSetAttribute(pq_film_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PqSmem::kTotal);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured.cur() = 1;
  }
  int sms = 0, dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (sms <= 0) sms = 148;
  const int64_t tiles_m = (tokens + kPqTile - 1) / kPqTile;
  const int grid = static_cast<int>(tiles_m < sms ? tiles_m : sms);
  pq_film_kernel<<<grid, kPqThreads, PqSmem::kTotal, stream>>>(p);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace yv
