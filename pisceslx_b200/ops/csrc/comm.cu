// Peer-memory communication kernels (NVLink 5 / NVSwitch): every rank maps the other ranks' symmetric
// buffers (CUDA IPC) and the kernels below read and write them directly.
//
//   peer_barrier            bounded flag barrier across the ranks of a group (one small block)
//   ep_put_counts           publish this rank's per-expert row counts into every peer's table, then barrier
//   ep_recv_plan            receiver side: tile -> (row, expert) tables over the per-source receive regions
//   ep_dispatch             the MoE permutation with the destination rows living in the owner's memory:
//                           token rows are stored straight into the peer's receive region (dispatch all-to-all)
//   ep_combine              weighted un-permute that loads expert outputs from the owners' memory (combine)
//   ep_combine_bwd / ep_unpermute_sum    the two backward directions of the same traffic
//   zero_reduce_fold        ZeRO: owner pulls the peers' gradient shards, sums, scales and folds into the
//                           momentum buffer (Muon) or applies AdamW in the same pass
//   peer_copy               plain pull copy (parameter all-gather, staging of remote tiles)
//   pq_gather_sum_peer      row-sharded codebook gather over peers + sum
//
// Rules followed here: no TMA multicast anywhere; every wait on a peer is bounded and reports through the
// status word; plain (generic-proxy) loads and stores with system-scope release/acquire on the flags.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "sm100.cuh"
#include "yv_comm.h"

namespace yv {

namespace {

constexpr int kMaxRanks = 8;
constexpr int kMaxTopK = 16;

struct PeerPtrs {
  void* p[kMaxRanks];
};

__device__ __forceinline__ void st_release_sys(uint32_t* addr, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* addr) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}

// flags layout on every rank: uint32 flags[kMaxRanks]; rank r writes its epoch into flags[r] of every peer.
__device__ __forceinline__ bool barrier_device(const PeerPtrs& flag_ptrs, int my_rank, int world, uint32_t epoch,
                                               uint32_t* status) {
  __threadfence_system();
  __syncthreads();
  bool ok = true;
  if (threadIdx.x < world) {
    uint32_t* remote = reinterpret_cast<uint32_t*>(flag_ptrs.p[threadIdx.x]) + my_rank;
    st_release_sys(remote, epoch);
    const uint32_t* mine = reinterpret_cast<const uint32_t*>(flag_ptrs.p[my_rank]) + threadIdx.x;
    const uint64_t t0 = globaltimer_ns();
    uint32_t spins = 0;
    // epochs only grow; a peer that is already one barrier ahead also satisfies the wait
    while (static_cast<int32_t>(ld_acquire_sys(mine) - epoch) < 0) {
      if ((++spins & 0x3Fu) == 0u) {
        if (globaltimer_ns() - t0 > YV_WAIT_LIMIT_NS) {
          if (status != nullptr) atomicOr(status, kStatusPeerTimeout);
          ok = false;
          break;
        }
        __nanosleep(200);
      }
    }
  }
  __syncthreads();
  return ok;
}

__global__ void peer_barrier_kernel(PeerPtrs flag_ptrs, int my_rank, int world, uint32_t epoch, uint32_t* status) {
  barrier_device(flag_ptrs, my_rank, world, epoch, status);
}

// counts [E] = padded rows per global expert on this rank.  Peer d receives counts[d*E_local .. +E_local) into
// its table[my_rank][*].  One block; ends with a barrier so that all tables are complete on return.
__global__ void ep_put_counts_kernel(const int* __restrict__ seg_offsets, PeerPtrs table_ptrs, PeerPtrs flag_ptrs,
                                     int my_rank, int world, int e_local, uint32_t epoch, uint32_t* status) {
  const int E = world * e_local;
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    const int d = e / e_local;
    int* table = reinterpret_cast<int*>(table_ptrs.p[d]);
    table[my_rank * e_local + (e - d * e_local)] = seg_offsets[e + 1] - seg_offsets[e];
  }
  barrier_device(flag_ptrs, my_rank, world, epoch, status);
}

// counts_all [world][e_local] (rows sent by each source per local expert; multiples of 128).
// Source s's rows live at rows [s*cap, s*cap + sum_e counts_all[s][e]).  Emits one flat tile list.
//   source-major (expert_major = 0): tiles ordered (source, expert); seg_src [world][e_local + 1] = row offsets of the
//     expert segments inside each source's block.
//   expert-major (expert_major = 1): tiles ordered (expert, source), so that a COMPACT buffer holding the listed tiles
//     back to back has every expert's rows contiguous; seg_src [e_local + 1] = offsets of the experts in that buffer.
__global__ void ep_recv_plan_kernel(const int* __restrict__ counts_all, int world, int e_local, int cap_rows,
                                    int* __restrict__ tile_rows, int* __restrict__ tile_expert,
                                    int* __restrict__ num_tiles, int* __restrict__ seg_src, int max_tiles,
                                    int expert_major) {
  __shared__ int s_base[kMaxRanks + 1];
  if (expert_major) {
    // one thread walks the (expert, source) grid: e_local * world <= a few hundred entries
    if (threadIdx.x == 0) {
      int t = 0;
      for (int e = 0; e < e_local; ++e) {
        seg_src[e] = t * 128;
        for (int s = 0; s < world; ++s) {
          int row = 0;                                        // offset of expert e inside source s's block
          for (int e2 = 0; e2 < e; ++e2) row += counts_all[s * e_local + e2];
          const int n = counts_all[s * e_local + e] / 128;
          for (int i = 0; i < n; ++i, ++t) {
            if (t < max_tiles) {
              tile_rows[t] = (s * cap_rows + row) / 128 + i;
              tile_expert[t] = e;
            }
          }
        }
      }
      seg_src[e_local] = (t < max_tiles ? t : max_tiles) * 128;
      *num_tiles = t < max_tiles ? t : max_tiles;
    }
    return;
  }
  if (threadIdx.x == 0) {
    int t = 0;
    for (int s = 0; s < world; ++s) {
      s_base[s] = t;
      int rows = 0;
      for (int e = 0; e < e_local; ++e) rows += counts_all[s * e_local + e];
      t += rows / 128;
    }
    s_base[world] = t;
    *num_tiles = t < max_tiles ? t : max_tiles;
  }
  __syncthreads();
  for (int s = 0; s < world; ++s) {
    int row = 0;
    for (int e = 0; e < e_local; ++e) {
      const int c = counts_all[s * e_local + e];
      if (threadIdx.x == 0) seg_src[s * (e_local + 1) + e] = row;
      const int t0 = s_base[s] + row / 128;
      for (int t = threadIdx.x; t < c / 128; t += blockDim.x) {
        if (t0 + t < max_tiles) {
          tile_rows[t0 + t] = (s * cap_rows + row) / 128 + t;
          tile_expert[t0 + t] = e;
        }
      }
      row += c;
    }
    if (threadIdx.x == 0) seg_src[s * (e_local + 1) + e_local] = row;
  }
}

// dst tile j = src tile tile_rows[j] (128 rows of `cols` bf16 each); one CTA per tile, 16-byte copies.
__global__ void tile_gather_kernel(const uint4* __restrict__ src, const int* __restrict__ tile_rows, uint4* __restrict__ dst,
                                   int vec_per_tile, int src_tiles, uint32_t* status) {
  const int j = blockIdx.x;
  const int t = tile_rows[j];
  const bool ok = t >= 0 && t < src_tiles;
  if (!ok && status != nullptr && threadIdx.x == 0) atomicOr(status, kStatusIndexOutOfRange);
  const uint4* s = src + static_cast<int64_t>(ok ? t : 0) * vec_per_tile;
  uint4* d = dst + static_cast<int64_t>(j) * vec_per_tile;
  for (int i = threadIdx.x; i < vec_per_tile; i += blockDim.x) d[i] = ok ? s[i] : make_uint4(0u, 0u, 0u, 0u);
}

// Encoded destination of assignment (t, j): g = dest_rank * region + my_rank * cap + row_in_my_block,
// region = world * cap rows (one receive buffer).
__global__ void ep_dispatch_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ idx,
                                   int* __restrict__ cursor, const int* __restrict__ seg_offsets,
                                   int64_t* __restrict__ row_map, PeerPtrs recv_ptrs, int my_rank, int e_local,
                                   int cap_rows, int world, int k, int cols, uint32_t* status) {
  __shared__ long long dest[kMaxTopK];
  const int64_t t = blockIdx.x;
  if (threadIdx.x < k) {
    const int e = idx[t * k + threadIdx.x];
    const int d = e / e_local;
    const int r = atomicAdd(&cursor[e], 1) - seg_offsets[d * e_local];    // row inside my block at rank d
    long long g = -1;
    if (r >= 0 && r < cap_rows && d < world) {
      g = (static_cast<long long>(d) * world + my_rank) * cap_rows + r;
    } else if (status != nullptr) {
      atomicOr(status, kStatusIndexOutOfRange);
    }
    dest[threadIdx.x] = g;
    row_map[t * k + threadIdx.x] = g;
  }
  __syncthreads();
  const int nvec = cols >> 3;
  const long long region = static_cast<long long>(world) * cap_rows;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    const uint4 val = *reinterpret_cast<const uint4*>(x + t * cols + v * 8);
    for (int j = 0; j < k; ++j) {
      const long long g = dest[j];
      if (g < 0) continue;
      __nv_bfloat16* base = reinterpret_cast<__nv_bfloat16*>(recv_ptrs.p[g / region]);
      *reinterpret_cast<uint4*>(base + (g % region) * cols + v * 8) = val;
    }
  }
}

// zero the pad rows of my segments inside the owners' receive regions: grid (E, chunks)
__global__ void ep_zero_pad_kernel(const int* __restrict__ seg_offsets, const int* __restrict__ counts,
                                   PeerPtrs recv_ptrs, int my_rank, int e_local, int cap_rows, int world, int cols) {
  const int e = blockIdx.x;
  const int d = e / e_local;
  const int base_row = seg_offsets[e] - seg_offsets[d * e_local];
  const int r0 = base_row + counts[e];
  const int r1 = base_row + (seg_offsets[e + 1] - seg_offsets[e]);
  if (r1 > cap_rows) return;
  __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(recv_ptrs.p[d]) +
                       (static_cast<int64_t>(my_rank) * cap_rows) * cols;
  const int nvec = cols >> 3;
  const int64_t total = static_cast<int64_t>(r1 - r0) * nvec;
  for (int64_t i = blockIdx.y * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.y) * blockDim.x) {
    const int64_t r = r0 + i / nvec;
    const int v = static_cast<int>(i % nvec);
    *reinterpret_cast<uint4*>(dst + r * cols + v * 8) = make_uint4(0u, 0u, 0u, 0u);
  }
}

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

// out[t] = sum_j w[t,j] * Y[g(t,j)] with Y rows read from the owners' memory
__global__ void ep_combine_kernel(PeerPtrs y_ptrs, const int64_t* __restrict__ row_map,
                                  const float* __restrict__ weights, __nv_bfloat16* __restrict__ out, int k, int cols,
                                  long long region) {
  const int64_t t = blockIdx.x;
  const int nvec = cols >> 3;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    for (int j = 0; j < k; ++j) {
      const float w = weights[t * k + j];
      const long long g = row_map[t * k + j];
      if (w != 0.f && g >= 0) {
        const __nv_bfloat16* base = reinterpret_cast<const __nv_bfloat16*>(y_ptrs.p[g / region]);
        float r[8];
        load8(base + (g % region) * cols + v * 8, r);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] += w * r[i];
      }
    }
    store8(out + t * cols + v * 8, acc);
  }
}

// dY[g(t,j)] = w * dout[t] (peer store), dweights[t,j] = <dout[t], Y[g]> (peer load)
__global__ void ep_combine_bwd_kernel(const __nv_bfloat16* __restrict__ dout, PeerPtrs y_ptrs, PeerPtrs dy_ptrs,
                                      const int64_t* __restrict__ row_map, const float* __restrict__ weights,
                                      float* __restrict__ dweights, int k, int cols, long long region) {
  __shared__ float red[kMaxTopK][33];
  const int64_t t = blockIdx.x;
  const int nvec = cols >> 3;
  float dots[kMaxTopK];
#pragma unroll
  for (int j = 0; j < kMaxTopK; ++j) dots[j] = 0.f;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    float g8[8];
    load8(dout + t * cols + v * 8, g8);
    for (int j = 0; j < k; ++j) {
      const long long g = row_map[t * k + j];
      if (g < 0) continue;
      const float w = weights[t * k + j];
      const int64_t off = (g % region) * cols + v * 8;
      float yv[8], o[8];
      load8(reinterpret_cast<const __nv_bfloat16*>(y_ptrs.p[g / region]) + off, yv);
      float d = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) { d += g8[i] * yv[i]; o[i] = w * g8[i]; }
      dots[j] += d;
      store8(reinterpret_cast<__nv_bfloat16*>(dy_ptrs.p[g / region]) + off, o);
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

// dx[t] = sum_j dXp[g(t,j)] read from the owners
__global__ void ep_unpermute_sum_kernel(PeerPtrs dx_ptrs, const int64_t* __restrict__ row_map,
                                        __nv_bfloat16* __restrict__ dx, int k, int cols, long long region) {
  const int64_t t = blockIdx.x;
  const int nvec = cols >> 3;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    for (int j = 0; j < k; ++j) {
      const long long g = row_map[t * k + j];
      if (g < 0) continue;
      float r[8];
      load8(reinterpret_cast<const __nv_bfloat16*>(dx_ptrs.p[g / region]) + (g % region) * cols + v * 8, r);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += r[i];
    }
    store8(dx + t * cols + v * 8, acc);
  }
}

}  // namespace

}  // namespace yv

#include "comm_part2.inc"
