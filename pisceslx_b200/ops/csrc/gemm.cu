// Host launcher of the tcgen05 GEMM: builds the three tensor maps, picks the template instance and
// launches one persistent CTA per SM.
#include "per_device.h"
#include "gemm_sm100.cuh"
#include "tensormap.h"
#include "yv_ops.h"

namespace yv {

namespace {

int g_sm_count = 0;

int sm_count() {
  if (g_sm_count == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (g_sm_count <= 0) g_sm_count = 148;
  }
  return g_sm_count;
}

template <int BN, bool A_MN, bool B_MN, typename OutT, int COMM = 0, int FP8 = 0>
int launch_instance(const GemmParams& p, int grid, cudaStream_t stream) {
  auto kern = gemm_sm100_kernel<BN, A_MN, B_MN, OutT, COMM, FP8>;
  static PerDeviceInt configured;
  if (!configured.cur()) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmSmem<BN, FP8 == 2>::kTotal);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured.cur() = 1;
  }
  kern<<<grid, COMM == 1 ? kGemmThreadsAllGather : kGemmThreads, GemmSmem<BN, FP8 == 2>::kTotal, stream>>>(p);
  return static_cast<int>(cudaGetLastError());
}

// The fused tensor-parallel variants exist for A stored [M,K] and bf16 output only.
template <int BN, int COMM>
int dispatch_comm(const GemmArgs& a, const GemmParams& p, int grid, cudaStream_t stream) {
  if (a.b_mn) return launch_instance<BN, false, true, __nv_bfloat16, COMM>(p, grid, stream);
  return launch_instance<BN, false, false, __nv_bfloat16, COMM>(p, grid, stream);
}

template <int BN, typename OutT>
int dispatch_layout(const GemmArgs& a, const GemmParams& p, int grid, cudaStream_t stream) {
  if (!a.a_mn && !a.b_mn) return launch_instance<BN, false, false, OutT>(p, grid, stream);
  if (!a.a_mn && a.b_mn) return launch_instance<BN, false, true, OutT>(p, grid, stream);
  if (a.a_mn && a.b_mn) return launch_instance<BN, true, true, OutT>(p, grid, stream);
  return launch_instance<BN, true, false, OutT>(p, grid, stream);
}

}  // namespace

int launch_gemm(const GemmArgs& a, cudaStream_t stream) {
  if (a.M <= 0 || a.N <= 0) return 0;
  if (a.a == nullptr || a.b == nullptr || a.c == nullptr) return -10;
  const int out_bytes = a.out_fp32 ? 4 : 2;
  int bn = a.bn;
  if (bn == 0) {
    // Estimated cost in waves of one CTA per SM.  A 128-wide tile takes about 0.6 of the time of a 256-wide one
    // (it re-reads A twice as often per output column): measured on N = 1408, K = 4096 at 49152 rows, 256-wide
    // tiles with a half-empty last column (1375 TFLOP/s) beat 128-wide ones without waste (1274 TFLOP/s), while
    // at 4096 rows the narrower tiles win by filling the last wave.
    const int64_t groups_est = (a.mode == kGroupedK || a.mode == kBatched) ? (a.num_groups > 0 ? a.num_groups : 1) : 1;
    const int64_t tm = (static_cast<int64_t>(a.M) + kBM - 1) / kBM * groups_est;
    const int64_t sms = sm_count();
    const int64_t waves256 = (tm * ((a.N + 255) / 256) + sms - 1) / sms;
    const int64_t waves128 = (tm * ((a.N + 127) / 128) + sms - 1) / sms;
    bn = (a.N <= 128 || 6 * waves128 <= 10 * waves256) ? 128 : 256;
  }
  if (bn != 128 && bn != 256) return -11;

  GemmParams p;
  p.M = a.M; p.N = a.N; p.K = a.K;
  p.mode = a.mode;
  p.accumulate = a.accumulate;
  p.num_groups = a.num_groups;
  p.tile_expert = a.tile_expert;
  p.tile_rows = a.tile_rows;
  p.tile_rows_c_only = (a.tile_rows != nullptr && a.tile_rows_c_only) ? 1 : 0;
  p.num_m_tiles = a.num_m_tiles;
  p.seg_offsets = a.seg_offsets;
  p.status = a.status;
  p.b_group_stride = 0;
  p.c_group_stride = 0;
  p.a_group_stride = 0;

  // extents of the stored operands
  uint64_t a_inner, a_outer, b_inner, b_outer, c_outer;
  const uint64_t groups = static_cast<uint64_t>(a.num_groups);
  if (a.mode == kDense) {
    a_inner = a.a_mn ? a.M : a.K;  a_outer = a.a_mn ? a.K : a.M;
    b_inner = a.b_mn ? a.N : a.K;  b_outer = a.b_mn ? a.K : a.N;
    c_outer = a.M;
  } else if (a.mode == kGroupedM) {
    if (a.a_mn || a.tile_expert == nullptr || a.num_m_tiles == nullptr) return -12;
    if (a.rows_total % kBM != 0) return -13;
    p.M = static_cast<int>(a.rows_total);
    a_inner = a.K;  a_outer = a.rows_total;
    b_inner = a.b_mn ? a.N : a.K;
    p.b_group_stride = a.b_mn ? a.K : a.N;
    b_outer = groups * static_cast<uint64_t>(p.b_group_stride);
    if (a.b_mn && (a.K % kBK) != 0) return -14;   // a K tile must not run into the next expert's rows
    c_outer = a.c_rows_total > 0 ? static_cast<uint64_t>(a.c_rows_total) : a.rows_total;
  } else if (a.mode == kGroupedK) {
    if (!a.a_mn || !a.b_mn || a.seg_offsets == nullptr) return -15;
    if (a.M % kBM != 0) return -16;               // C tiles must not cross expert boundaries
    a_inner = a.M;  a_outer = a.rows_total;
    b_inner = a.N;  b_outer = a.rows_total;
    p.c_group_stride = a.M;
    c_outer = groups * static_cast<uint64_t>(a.M);
  } else if (a.mode == 4) {
    // split-K of a dense product with both operands stored K-inner (activations [M,K], weights [N,K]): slice g
    // reduces over K range seg_offsets[g] .. seg_offsets[g+1] and writes its partial to rows g*Mpad.. of C, where
    // Mpad = M rounded up to 128.  Runs the grouped-K tile loop; used for skinny M (decode), where the N tiles alone
    // would occupy a fraction of the SMs.
    if (a.a_mn || a.b_mn || a.seg_offsets == nullptr || a.accumulate) return -60;
    const int m_pad = ((a.M + kBM - 1) / kBM) * kBM;
    p.mode = kGroupedK;
    a_inner = a.K;  a_outer = a.M;
    b_inner = a.K;  b_outer = a.N;
    p.c_group_stride = m_pad;
    c_outer = groups * static_cast<uint64_t>(m_pad);
  } else if (a.mode == kBatched) {
    // every operand stacks `num_groups` equal problems along its outer dimension
    if (a.M % kBM != 0) return -18;                       // C / A row tiles must not cross batch entries
    if ((a.a_mn || a.b_mn) && (a.K % kBK) != 0) return -19;
    p.a_group_stride = a.a_mn ? a.K : a.M;
    p.b_group_stride = a.b_mn ? a.K : a.N;
    p.c_group_stride = a.M;
    a_inner = a.a_mn ? a.M : a.K;  a_outer = groups * static_cast<uint64_t>(p.a_group_stride);
    b_inner = a.b_mn ? a.N : a.K;  b_outer = groups * static_cast<uint64_t>(p.b_group_stride);
    c_outer = groups * static_cast<uint64_t>(a.M);
  } else {
    return -17;
  }
  const uint64_t lda = a.lda ? a.lda : a_inner;
  const uint64_t ldb = a.ldb ? a.ldb : b_inner;
  const uint64_t ldc = a.ldc ? a.ldc : static_cast<uint64_t>(a.N);

  int r;
  p.out_scale = a.out_scale;
  p.epi_cin = reinterpret_cast<const __nv_bfloat16*>(a.epi_cin);
  p.epi_a = a.epi_a; p.epi_b = a.epi_b; p.epi_c = a.epi_c;
  if (a.epi_cin != nullptr) {
    if (a.out_fp32 || a.accumulate || a.comm != 0 || a.fp8 || (a.N % 64) != 0 || (a.ldc != 0 && a.ldc != a.N) ||
        (reinterpret_cast<uintptr_t>(a.epi_cin) & 15u) != 0)
      return -80;
  }
  const bool mx = a.sfa != nullptr || a.sfb != nullptr;
  p.sfa = static_cast<const uint8_t*>(a.sfa); p.sfb = static_cast<const uint8_t*>(a.sfb);
  p.sf_kchunks = a.K / 128; p.sf_b_tiles = static_cast<int>(b_outer / kBM);
  if (mx) {
    if (a.sfa == nullptr || a.sfb == nullptr || (a.K % 128) != 0 || (b_outer % kBM) != 0) return -71;
    if (a.mode != kDense && a.mode != kGroupedM) return -72;
    if (a.mode == kGroupedM && (a.tile_rows != nullptr || (a.N % kBM) != 0)) return -73;
    if ((reinterpret_cast<uintptr_t>(a.sfa) & 15u) != 0 || (reinterpret_cast<uintptr_t>(a.sfb) & 15u) != 0) return -74;
  }
  if (a.fp8 || mx) {
    // e4m3 operands: one byte per element, 128 elements per 128-byte row of a stage
    if ((a.mode != kDense && !mx) || a.a_mn || a.b_mn || a.out_fp32 || a.accumulate || a.comm != 0) return -70;
    r = make_tmap_2d(&p.tma_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a.a, a_inner, a_outer, lda, 128, kBM);
    if (r != 0) return -20 + r;
    r = make_tmap_2d(&p.tma_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a.b, b_inner, b_outer, ldb, 128,
                     static_cast<uint32_t>(bn));
    if (r != 0) return -30 + r;
  } else {
    r = make_tmap_2d(&p.tma_a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.a, a_inner, a_outer, lda, 64,
                     a.a_mn ? kBK : kBM);
    if (r != 0) return -20 + r;
    r = make_tmap_2d(&p.tma_b, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.b, b_inner, b_outer, ldb, 64,
                     a.b_mn ? kBK : static_cast<uint32_t>(bn));
    if (r != 0) return -30 + r;
  }
  r = make_tmap_2d(&p.tma_c, a.out_fp32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16,
                   out_bytes, a.c, static_cast<uint64_t>(a.N), c_outer, ldc, 128 / out_bytes, kBM);
  if (r != 0) return -40 + r;

  p.symmetric = 0; p.sym_tiles = 0; p.sym_c = nullptr;
  if (a.symmetric) {
    if (a.mode != kBatched || a.M != a.N || a.out_fp32 || a.accumulate || a.comm != 0 || a.fp8 ||
        (a.ldc != 0 && a.ldc != a.N))
      return -81;
    p.symmetric = 1;
    p.sym_c = reinterpret_cast<__nv_bfloat16*>(a.c);
    const int tm = (a.M + kBM - 1) / kBM, tn = (a.N + bn - 1) / bn;
    for (int j = 0; j < tn; ++j) p.sym_tiles += (tm < (j + 1) * (bn / kBM)) ? tm : (j + 1) * (bn / kBM);
  }
  p.comm_world = 1; p.comm_rank = 0; p.comm_blocks_per_rank = 0;
  p.comm_local = nullptr; p.comm_flags = nullptr; p.comm_flag_target = 0; p.comm_row_bytes = 0;
  for (int i = 0; i < 8; ++i) p.comm_peer[i] = nullptr;
  if (a.comm != 0) {
    if (a.comm != 1 && a.comm != 2) return -50;
    if (a.mode != kDense || a.a_mn || a.out_fp32 || a.accumulate) return -51;
    if (a.comm_world < 2 || a.comm_world > 8 || a.comm_rank < 0 || a.comm_rank >= a.comm_world) return -52;
    if (a.comm_rows_per_rank <= 0 || a.comm_rows_per_rank % kBM != 0 ||
        a.comm_rows_per_rank * a.comm_world != a.M) return -53;
    if (a.comm == 1 && (a.comm_flags == nullptr || (a.lda != 0 && a.lda != a.K))) return -54;
    if (a.comm == 2 && (a.N % 64) != 0) return -55;
    for (int r = 0; r < a.comm_world; ++r)
      if (r != a.comm_rank && a.comm_peer[r] == nullptr) return -56;
    p.comm_world = a.comm_world; p.comm_rank = a.comm_rank;
    p.comm_blocks_per_rank = static_cast<int>(a.comm_rows_per_rank / kBM);
    for (int r = 0; r < a.comm_world; ++r) p.comm_peer[r] = a.comm_peer[r];
    p.comm_local = static_cast<uint8_t*>(const_cast<void*>(a.a));
    p.comm_flags = a.comm_flags;
    p.comm_row_bytes = a.comm == 1 ? static_cast<long long>(a.K) * 2 : static_cast<long long>(a.N) * 2;
  }

  const int64_t tiles_m = (p.M + kBM - 1) / kBM;
  const int64_t tiles_n = (a.N + bn - 1) / bn;
  int64_t tiles = tiles_m * tiles_n * ((p.mode == kGroupedK || p.mode == kBatched) ? a.num_groups : 1);
  if (p.symmetric) tiles = static_cast<int64_t>(p.sym_tiles) * a.num_groups;
  const int cap = a.max_ctas > 0 ? a.max_ctas : sm_count();
  const int grid = static_cast<int>(tiles < cap ? tiles : cap);

  if (mx) {
    return bn == 256 ? launch_instance<256, false, false, __nv_bfloat16, 0, 2>(p, grid, stream)
                     : launch_instance<128, false, false, __nv_bfloat16, 0, 2>(p, grid, stream);
  }
  if (a.fp8) {
    return bn == 256 ? launch_instance<256, false, false, __nv_bfloat16, 0, 1>(p, grid, stream)
                     : launch_instance<128, false, false, __nv_bfloat16, 0, 1>(p, grid, stream);
  }
  if (a.comm == 1) {
    cudaError_t e = cudaMemsetAsync(a.comm_flags, 0, sizeof(uint32_t) * static_cast<size_t>(tiles_m), stream);
    if (e != cudaSuccess) return static_cast<int>(e);
    p.comm_flag_target = static_cast<uint32_t>((static_cast<long long>(kBM) * p.comm_row_bytes) >> 4);   // vectors per block
    return bn == 256 ? dispatch_comm<256, 1>(a, p, grid, stream) : dispatch_comm<128, 1>(a, p, grid, stream);
  }
  if (a.comm == 2) {
    return bn == 256 ? dispatch_comm<256, 2>(a, p, grid, stream) : dispatch_comm<128, 2>(a, p, grid, stream);
  }
  if (bn == 256) {
    return a.out_fp32 ? dispatch_layout<256, float>(a, p, grid, stream)
                      : dispatch_layout<256, __nv_bfloat16>(a, p, grid, stream);
  }
  return a.out_fp32 ? dispatch_layout<128, float>(a, p, grid, stream)
                    : dispatch_layout<128, __nv_bfloat16>(a, p, grid, stream);
}

}  // namespace yv
