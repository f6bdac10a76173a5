// Host launchers for the attention kernels: tensor-map construction, grid sizing, template dispatch.
#include "per_device.h"
#include "attention_bwd.cuh"
#include "attention_decode.cuh"
#include "attention_decode_mma.cuh"
#include "attention_decode_tma.cuh"
#include "attention_fwd.cuh"
#include "tensormap.h"
#include "yv_ops.h"

namespace yv {

namespace {

// 3-D view (d, head, token) of a [tokens, heads, d] tensor whose token pitch is `stride` elements.
int make_head_map(CUtensorMap* m, const void* base, int d, int heads, int64_t tokens, int64_t stride) {
  return make_tmap_3d(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, static_cast<uint64_t>(d),
                      static_cast<uint64_t>(heads), static_cast<uint64_t>(tokens), static_cast<uint64_t>(d) * 2,
                      static_cast<uint64_t>(stride) * 2, 64, 1, 128);
}

template <typename K>
int set_smem(K kern, int bytes) {
  return static_cast<int>(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
}

constexpr float kLog2eHost = 1.4426950408889634f;

}  // namespace

int launch_attn_fwd(const AttnArgs& a, cudaStream_t stream) {
  if (a.batch <= 0 || a.total_q <= 0) return 0;
  if (a.d != 64 && a.d != 128) return -1;
  if (a.hk <= 0 || a.hq % a.hk != 0) return -2;
  AttnFwdParams p;
  int r = make_head_map(&p.tma_q, a.q, a.d, a.hq, a.total_q, a.q_stride);
  if (r != 0) return -10 + r;
  r = make_head_map(&p.tma_k, a.k, a.d, a.hk, a.total_k, a.k_stride);
  if (r != 0) return -20 + r;
  r = make_head_map(&p.tma_v, a.v, a.d, a.hk, a.total_k, a.v_stride);
  if (r != 0) return -30 + r;
  p.o = reinterpret_cast<__nv_bfloat16*>(a.o);
  p.lse = a.lse;
  p.cu_q = a.cu_q;
  p.cu_k = a.cu_k ? a.cu_k : a.cu_q;
  p.hq = a.hq; p.hk = a.hk;
  p.o_stride = a.o_stride;
  p.total_q = a.total_q;
  p.causal = a.causal;
  p.scale_log2 = a.scale * kLog2eHost;
  p.status = a.status;
  dim3 grid((a.max_q + 127) / 128, a.hq, a.batch);
  if (a.d == 128) {
    static PerDeviceInt cfg;
    if (!cfg.cur()) { r = set_smem(attn_fwd_kernel<128>, AttnFwdSmem<128>::kTotal); if (r) return r; cfg.cur() = 1; }
    attn_fwd_kernel<128><<<grid, kAttnThreads, AttnFwdSmem<128>::kTotal, stream>>>(p);
  } else {
    static PerDeviceInt cfg;
    if (!cfg.cur()) { r = set_smem(attn_fwd_kernel<64>, AttnFwdSmem<64>::kTotal); if (r) return r; cfg.cur() = 1; }
    attn_fwd_kernel<64><<<grid, kAttnThreads, AttnFwdSmem<64>::kTotal, stream>>>(p);
  }
  return static_cast<int>(cudaGetLastError());
}

int launch_attn_bwd(const AttnBwdArgs& b, cudaStream_t stream) {
  const AttnArgs& a = b.f;
  if (a.batch <= 0 || a.total_q <= 0) return 0;
  if (a.d != 64 && a.d != 128) return -1;
  if (a.hk <= 0 || a.hq % a.hk != 0) return -2;
  if (b.delta == nullptr || a.lse == nullptr) return -3;
  AttnBwdParams p;
  int r = make_head_map(&p.tma_q, a.q, a.d, a.hq, a.total_q, a.q_stride);
  if (r != 0) return -10 + r;
  r = make_head_map(&p.tma_k, a.k, a.d, a.hk, a.total_k, a.k_stride);
  if (r != 0) return -20 + r;
  r = make_head_map(&p.tma_v, a.v, a.d, a.hk, a.total_k, a.v_stride);
  if (r != 0) return -30 + r;
  r = make_head_map(&p.tma_do, b.dout, a.d, a.hq, a.total_q, b.do_stride);
  if (r != 0) return -40 + r;
  p.dq = reinterpret_cast<__nv_bfloat16*>(b.dq);
  p.dk = reinterpret_cast<__nv_bfloat16*>(b.dk);
  p.dv = reinterpret_cast<__nv_bfloat16*>(b.dv);
  p.lse = a.lse;
  p.delta = b.delta;
  p.cu_q = a.cu_q;
  p.cu_k = a.cu_k ? a.cu_k : a.cu_q;
  p.hq = a.hq; p.hk = a.hk;
  p.dq_stride = b.dq_stride; p.dk_stride = b.dk_stride; p.dv_stride = b.dv_stride;
  p.total_q = a.total_q;
  p.causal = a.causal;
  p.scale = a.scale;
  p.scale_log2 = a.scale * kLog2eHost;
  p.status = a.status;

  const int64_t warps = a.total_q * a.hq;
  attn_delta_kernel<<<static_cast<unsigned>((warps + 7) / 8), 256, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(a.o), reinterpret_cast<const __nv_bfloat16*>(b.dout), b.delta,
      a.total_q, a.hq, a.d, a.o_stride, b.do_stride);

  dim3 grid_q((a.max_q + 127) / 128, a.hq, a.batch);
  dim3 grid_k((a.max_k + 127) / 128, a.hk, a.batch);
  if (a.d == 128) {
    static PerDeviceInt cfg;
    if (!cfg.cur()) {
      r = set_smem(attn_bwd_dq_kernel<128>, AttnBwdSmem<128>::kTotal); if (r) return r;
      r = set_smem(attn_bwd_dkv_kernel<128>, AttnBwdSmem<128>::kTotal); if (r) return r;
      cfg.cur() = 1;
    }
    attn_bwd_dkv_kernel<128><<<grid_k, kAttnBwdThreads, AttnBwdSmem<128>::kTotal, stream>>>(p);
    attn_bwd_dq_kernel<128><<<grid_q, kAttnBwdThreads, AttnBwdSmem<128>::kTotal, stream>>>(p);
  } else {
    static PerDeviceInt cfg;
    if (!cfg.cur()) {
      r = set_smem(attn_bwd_dq_kernel<64>, AttnBwdSmem<64>::kTotal); if (r) return r;
      r = set_smem(attn_bwd_dkv_kernel<64>, AttnBwdSmem<64>::kTotal); if (r) return r;
      cfg.cur() = 1;
    }
    attn_bwd_dkv_kernel<64><<<grid_k, kAttnBwdThreads, AttnBwdSmem<64>::kTotal, stream>>>(p);
    attn_bwd_dq_kernel<64><<<grid_q, kAttnBwdThreads, AttnBwdSmem<64>::kTotal, stream>>>(p);
  }
  return static_cast<int>(cudaGetLastError());
}

namespace {
template <int D>
int decode_dispatch(const PagedDecodeParams& p, int G, dim3 grid, cudaStream_t stream) {
  switch (G) {
    case 1: paged_decode_kernel<D, 1><<<grid, 128, 0, stream>>>(p); break;
    case 2: paged_decode_kernel<D, 2><<<grid, 128, 0, stream>>>(p); break;
    case 4: paged_decode_kernel<D, 4><<<grid, 128, 0, stream>>>(p); break;
    case 8: paged_decode_kernel<D, 8><<<grid, 128, 0, stream>>>(p); break;
    default: return -4;
  }
  return 0;
}
}  // namespace

namespace {
template <int D, int G>
int decode_tma_launch(const PagedDecodeTmaParams& pp, dim3 grid, int smem, cudaStream_t stream) {
  static PerDeviceInt configured;
  if (configured.cur() < smem) {
    int r = set_smem(paged_decode_tma_kernel<D, G>, smem);
    if (r != 0) return r;
    configured.cur() = smem;
  }
  paged_decode_tma_kernel<D, G><<<grid, 128, smem, stream>>>(pp);
  return 0;
}

template <int D>
int decode_tma_dispatch(const PagedDecodeTmaParams& pp, int G, dim3 grid, int smem, cudaStream_t stream) {
  switch (G) {
    case 1: return decode_tma_launch<D, 1>(pp, grid, smem, stream);
    case 2: return decode_tma_launch<D, 2>(pp, grid, smem, stream);
    case 4: return decode_tma_launch<D, 4>(pp, grid, smem, stream);
    case 8: return decode_tma_launch<D, 8>(pp, grid, smem, stream);
    default: return -4;
  }
}
}  // namespace

int launch_paged_decode(const PagedDecodeArgs& a, cudaStream_t stream) {
  if (a.batch <= 0) return 0;
  if (a.d != 64 && a.d != 128) return -1;
  if (a.hk <= 0 || a.hq % a.hk != 0 || a.splits <= 0) return -2;
  if (a.partial_o == nullptr || a.partial_ml == nullptr) return -3;
  PagedDecodeParams p;
  p.q = reinterpret_cast<const __nv_bfloat16*>(a.q);
  p.k_cache = reinterpret_cast<const __nv_bfloat16*>(a.k_cache);
  p.v_cache = reinterpret_cast<const __nv_bfloat16*>(a.v_cache);
  p.block_table = a.block_table;
  p.seq_lens = a.seq_lens;
  p.o = reinterpret_cast<__nv_bfloat16*>(a.o);
  p.partial_o = a.partial_o;
  p.partial_ml = a.partial_ml;
  p.hq = a.hq; p.hk = a.hk; p.block = a.block; p.max_blocks_per_seq = a.max_blocks_per_seq;
  p.splits = a.splits; p.num_blocks = a.num_blocks;
  p.scale_log2 = a.scale * kLog2eHost;
  p.status = a.status;
  dim3 grid(a.hk, a.batch, a.splits);
  const int G = a.hq / a.hk;
  int r;
  // TMA-fed kernel: whole cache blocks of up to 128 tokens travel as one bulk copy each
  const int64_t slots = static_cast<int64_t>(a.num_blocks) * a.block;
  const bool use_tma = a.block >= 16 && a.block <= 128 && a.block % 16 == 0 && slots < (1ll << 31) && !a.force_direct;
  const bool use_mma = use_tma && a.d == 128 && a.block == 64 && (G == 1 || G == 2 || G == 4 || G == 8);
  if (use_mma) {
    // tensor-core kernel: keys are the M dimension, the query heads of the group are padded to N = 16
    PagedDecodeMmaParams pm;
    pm.p = p;
    r = make_tmap_3d(&pm.tma_k, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.k_cache, 128, static_cast<uint64_t>(a.hk),
                     static_cast<uint64_t>(slots), 256, static_cast<uint64_t>(a.hk) * 256, 64, 1, 64);
    if (r != 0) return -40 + r;
    r = make_tmap_3d(&pm.tma_v, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.v_cache, 128, static_cast<uint64_t>(a.hk),
                     static_cast<uint64_t>(slots), 256, static_cast<uint64_t>(a.hk) * 256, 64, 1, 64);
    if (r != 0) return -50 + r;
    static PerDeviceInt cfg;
    if (!cfg.cur()) {
      r = set_smem(paged_decode_mma_kernel<1>, kDmSmem); if (r) return r;
      r = set_smem(paged_decode_mma_kernel<2>, kDmSmem); if (r) return r;
      r = set_smem(paged_decode_mma_kernel<4>, kDmSmem); if (r) return r;
      r = set_smem(paged_decode_mma_kernel<8>, kDmSmem); if (r) return r;
      cfg.cur() = 1;
    }
    switch (G) {
      case 1: paged_decode_mma_kernel<1><<<grid, kDmThreads, kDmSmem, stream>>>(pm); break;
      case 2: paged_decode_mma_kernel<2><<<grid, kDmThreads, kDmSmem, stream>>>(pm); break;
      case 4: paged_decode_mma_kernel<4><<<grid, kDmThreads, kDmSmem, stream>>>(pm); break;
      default: paged_decode_mma_kernel<8><<<grid, kDmThreads, kDmSmem, stream>>>(pm); break;
    }
    r = 0;
  } else if (use_tma) {
    PagedDecodeTmaParams pp;
    pp.p = p;
    r = make_tmap_3d(&pp.tma_k, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.k_cache, static_cast<uint64_t>(a.d),
                     static_cast<uint64_t>(a.hk), static_cast<uint64_t>(slots), static_cast<uint64_t>(a.d) * 2,
                     static_cast<uint64_t>(a.hk) * a.d * 2, static_cast<uint32_t>(a.d), 1,
                     static_cast<uint32_t>(a.block), CU_TENSOR_MAP_SWIZZLE_NONE);
    if (r != 0) return -20 + r;
    r = make_tmap_3d(&pp.tma_v, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.v_cache, static_cast<uint64_t>(a.d),
                     static_cast<uint64_t>(a.hk), static_cast<uint64_t>(slots), static_cast<uint64_t>(a.d) * 2,
                     static_cast<uint64_t>(a.hk) * a.d * 2, static_cast<uint32_t>(a.d), 1,
                     static_cast<uint32_t>(a.block), CU_TENSOR_MAP_SWIZZLE_NONE);
    if (r != 0) return -30 + r;
    const int smem = kDecodeStages * 2 * a.block * a.d * 2 + 128;
    r = (a.d == 128) ? decode_tma_dispatch<128>(pp, G, grid, smem, stream)
                     : decode_tma_dispatch<64>(pp, G, grid, smem, stream);
  } else {
    r = (a.d == 128) ? decode_dispatch<128>(p, G, grid, stream) : decode_dispatch<64>(p, G, grid, stream);
  }
  if (r != 0) return r;
  const int64_t heads_total = static_cast<int64_t>(a.batch) * a.hq;
  const unsigned mgrid = static_cast<unsigned>((heads_total + 3) / 4);
  if (a.d == 128) {
    paged_decode_merge_kernel<128><<<mgrid, 128, 0, stream>>>(a.partial_o, a.partial_ml, p.o, heads_total, a.splits);
  } else {
    paged_decode_merge_kernel<64><<<mgrid, 128, 0, stream>>>(a.partial_o, a.partial_ml, p.o, heads_total, a.splits);
  }
  return static_cast<int>(cudaGetLastError());
}

int launch_kv_cache_write(const void* k, const void* v, void* k_cache, void* v_cache, const int* slot_map,
                          int64_t tokens, int row_elems, int64_t k_stride, int64_t v_stride, int64_t num_slots,
                          uint32_t* status, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if ((row_elems & 7) != 0) return -1;
  kv_cache_write_kernel<<<static_cast<unsigned>(tokens), 128, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(k), reinterpret_cast<const __nv_bfloat16*>(v),
      reinterpret_cast<__nv_bfloat16*>(k_cache), reinterpret_cast<__nv_bfloat16*>(v_cache), slot_map, row_elems,
      k_stride, v_stride, num_slots, status);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace yv
