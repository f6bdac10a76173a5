// Launchers of the peer-memory communication kernels (comm.cu) and the symmetric-memory runtime.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace yv {

constexpr int kCommMaxRanks = 8;

// ---- symmetric memory (CUDA IPC) ------------------------------------------------------------------
// A symmetric buffer is a cudaMalloc allocation of the same size on every rank whose IPC handle is
// exchanged through the process group; every rank maps all peers' buffers.
int symm_alloc(size_t bytes, void** ptr, unsigned char handle_out[64]);
int symm_open(const unsigned char handle[64], void** ptr);
int symm_close(void* ptr);
int symm_free(void* ptr);

// ---- kernels -----------------------------------------------------------------------------------------
int launch_peer_barrier(void* const* flag_ptrs, int my_rank, int world, uint32_t epoch, uint32_t* status,
                        cudaStream_t stream);
int launch_ep_put_counts(const int* seg_offsets, void* const* table_ptrs, void* const* flag_ptrs, int my_rank,
                         int world, int e_local, uint32_t epoch, uint32_t* status, cudaStream_t stream);
int launch_ep_recv_plan(const int* counts_all, int world, int e_local, int cap_rows, int* tile_rows, int* tile_expert,
                        int* num_tiles, int* seg_src, int max_tiles, int expert_major, cudaStream_t stream);
int launch_ep_dispatch(const void* x, const int* idx, int* cursor, const int* seg_offsets, int64_t* row_map,
                       void* const* recv_ptrs, int my_rank, int e_local, int cap_rows, int world, int64_t tokens, int k,
                       int cols, uint32_t* status, cudaStream_t stream);
int launch_ep_zero_pad(const int* seg_offsets, const int* counts, void* const* recv_ptrs, int my_rank, int e_local,
                       int cap_rows, int world, int cols, cudaStream_t stream);
int launch_ep_combine(void* const* y_ptrs, const int64_t* row_map, const float* weights, void* out, int64_t tokens,
                      int k, int cols, int64_t region_rows, int world, cudaStream_t stream);
int launch_ep_combine_bwd(const void* dout, void* const* y_ptrs, void* const* dy_ptrs, const int64_t* row_map,
                          const float* weights, float* dweights, int64_t tokens, int k, int cols, int64_t region_rows,
                          int world, cudaStream_t stream);
int launch_ep_unpermute_sum(void* const* dx_ptrs, const int64_t* row_map, void* dx, int64_t tokens, int k, int cols,
                            int64_t region_rows, int world, cudaStream_t stream);
// ZeRO: for elements [off, off+n) of the flat gradient buffers: g = scale * sum_r grad_r[i]; then
//   mode 0: write g back into my gradient buffer (plain reduce-scatter)
//   mode 1: momentum fold  m = mu * m + g          (Muon; the reduced gradient is not materialised)
//   mode 2: AdamW update of p, m, v                 (bias corrections bc1, bc2 precomputed on the host)
struct ZeroFoldArgs {
  void* const* grad_ptrs;       // [world] base of every rank's flat gradient buffer (bf16)
  int world, my_rank;
  int64_t off, n;
  float scale;
  int mode;
  void* p; void* m; void* v;    // tensors of the owned parameter (bf16 or fp32 per *_fp32 flags)
  int p_fp32, s_fp32;
  float mu, lr, beta1, beta2, eps, wd, bc1, bc2;
  float* sumsq = nullptr;       // optional: += squared norm of the reduced, scaled gradient (fp32 scalar)
};
int launch_zero_reduce_fold(const ZeroFoldArgs& a, cudaStream_t stream);
// dst tile j (rows 128 j ..) = src tile tile_rows[j]; tiles whose index is outside [0, src_tiles) are zero-filled and
// reported through the status word
int launch_tile_gather(const void* src, const int* tile_rows, int n_tiles, void* dst, int cols, int src_tiles,
                       uint32_t* status, cudaStream_t stream);
int launch_peer_copy(void* dst, const void* src, int64_t bytes, cudaStream_t stream);
// table shards: rank r owns rows [r*rows_per_rank, (r+1)*rows_per_rank) of every codebook: layout [C, rows_per_rank, D]
int launch_pq_gather_sum_peer(void* const* table_ptrs, const int* idx, void* out, int64_t tokens, int C,
                              int64_t rows_per_rank, int D, int world, uint32_t* status, cudaStream_t stream);

}  // namespace yv
