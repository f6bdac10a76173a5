// Launcher declarations for the sm_100a kernels of this directory.  The launchers take raw device
// pointers and a stream and include no framework header, so the kernels build in seconds; the
// PyTorch binding (binding.cpp) is the only translation unit that sees torch.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace yv {

// ------------------------------------------------------------------------------------------------
// GEMM (gemm.cu)
// ------------------------------------------------------------------------------------------------
struct GemmArgs {
  const void* a = nullptr;     // bf16
  const void* b = nullptr;     // bf16
  void* c = nullptr;           // bf16 or fp32
  int M = 0, N = 0, K = 0;     // logical problem: C[M,N] = A[M,K] * B[K,N]
  bool a_mn = false;           // false: A stored [M,K] row-major; true: stored [K,M] row-major
  bool b_mn = false;           // false: B stored [N,K] row-major (weight layout); true: stored [K,N] row-major
  int64_t lda = 0, ldb = 0, ldc = 0;   // row pitches in elements (0 = contiguous)
  int out_fp32 = 0;
  int accumulate = 0;
  int mode = 0;                // 0 dense, 1 grouped along M, 2 grouped along K
  int num_groups = 1;
  int64_t rows_total = 0;      // grouped modes: rows of the expert-sorted, padded row dimension
  const int* tile_expert = nullptr;
  const int* tile_rows = nullptr;   // grouped-M only: explicit row-tile index per listed tile (optional)
  bool tile_rows_c_only = false;    // the list addresses C only; A is compact (tile j = rows 128 j ..)
  int64_t c_rows_total = 0;         // rows of C when they differ from A's (0 = rows_total)
  const int* num_m_tiles = nullptr;
  const int* seg_offsets = nullptr;
  uint32_t* status = nullptr;
  int bn = 0;                  // 0 = choose
  int max_ctas = 0;            // 0 = number of SMs
  // Fused tensor-parallel collective (dense mode, A stored [M,K], bf16 C, M = comm_world * comm_rows_per_rank,
  // comm_rows_per_rank a multiple of 128):
  //   1  all-gather -> GEMM: `a` is the local gathered buffer; comm_peer[r] = rank r's published shard
  //      [rows_per_rank, K]; comm_flags = one uint32 per 128-row block (zeroed here before the launch)
  //   2  GEMM -> reduce-scatter push: rows owned by rank r are stored into comm_peer[r] (= r's inbox,
  //      [world][rows_per_rank, N]) at source slot comm_rank; own rows go to `c` (N a multiple of 64)
  int comm = 0;
  int comm_world = 1, comm_rank = 0;
  int64_t comm_rows_per_rank = 0;
  void* comm_peer[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  uint32_t* comm_flags = nullptr;
  // fp8 (e4m3) operands, both stored K-inner, bf16 output scaled by *out_scale in the epilogue (dense mode only)
  bool fp8 = false;
  const float* out_scale = nullptr;
  // block-scaled fp8 ("MX": e4m3 elements, one e8m0 scale per 32 elements of K): scale chunks of A and of B in the
  // 512-byte-per-(128 rows, 128 K) layout written by launch_mx_quantize; dense and grouped-M modes, K % 128 == 0,
  // rows of B (per expert) a multiple of 128.  Implies fp8.
  const void* sfa = nullptr;
  const void* sfb = nullptr;
  // affine epilogue: C = epi_c * (A B) + epi_b * epi_cin + epi_a * I (epi_cin bf16, laid out like C; N % 64 == 0)
  const void* epi_cin = nullptr;
  float epi_a = 0.f, epi_b = 0.f, epi_c = 1.f;
  // Symmetric result (batched mode, M == N, bf16 C, the caller guarantees C = C^T, e.g. X X^T or a polynomial of a
  // symmetric matrix): only the tiles that touch the diagonal or lie above it are computed; their epilogue also writes
  // the mirrored elements of the tiles that were skipped.
  bool symmetric = false;
};
// Returns 0 on success, a negative code when an argument is rejected, a positive cudaError_t otherwise.
int launch_gemm(const GemmArgs& args, cudaStream_t stream);

// ------------------------------------------------------------------------------------------------
// Elementwise / normalisation kernels (elementwise.cu)
// ------------------------------------------------------------------------------------------------
// y = rmsnorm(x (+ residual)) * w, optionally followed by FiLM y*(1+scale)+shift (scale/shift rows are
// selected by  row / film_rows_per_group).  res_out (optional) receives x + residual.  rstd receives 1/rms.
int launch_rmsnorm_fwd(const void* x, const void* residual, const void* w, const void* film_scale,
                       const void* film_shift, int64_t film_rows_per_group, void* y, void* res_out, float* rstd,
                       int64_t rows, int cols, float eps, cudaStream_t stream);
// dx (+= dres_in), dw_partial[blocks, cols] fp32 (reduced by launch_colsum)
int launch_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const void* dres_in,
                       void* dx, float* dw_partial, int dw_blocks, int64_t rows, int cols, cudaStream_t stream);
int launch_colsum(const float* partial, int blocks, int cols, void* out, int out_fp32, int accumulate,
                  cudaStream_t stream);
// Rotary embedding applied in place to q [T, hq, d] and k [T, hk, d] (rotate-half layout, first rot_dim dims).
// cos/sin: fp32 [max_pos, rot_dim/2] tables; positions: int32 [T].  inverse=1 applies the transposed
// rotation (backward).  Row strides are in elements, so q and k may live inside a fused QKV buffer.
int launch_rope_tables(void* q, void* k, const float* cos_t, const float* sin_t, const int* positions,
                       int64_t tokens, int hq, int hk, int head_dim, int rot_dim, int inverse, int64_t q_stride,
                       int64_t k_stride, cudaStream_t stream);
// 3-D (t, h, w) rotary embedding for video tokens: head_dim split in three sections.
int launch_rope3d(void* q, void* k, const int* pos_thw, int64_t tokens, int hq, int hk, int head_dim, int d_t,
                  int d_h, int d_w, float theta, int inverse, cudaStream_t stream);
// SwiGLU: out[r, j] = silu(in[r, j]) * in[r, F + j]   (in is [rows, 2F])
int launch_swiglu_fwd(const void* in, void* out, int64_t rows, int F, cudaStream_t stream);
int launch_swiglu_bwd(const void* in, const void* dout, void* din, int64_t rows, int F, cudaStream_t stream);
// expert rows: din = row_w * dSwiGLU(in, dact), actw = row_w * SwiGLU(in), rowdot = <SwiGLU(in), dact> per row
int launch_swiglu_bwd_rows(const void* in, const void* dact, const float* row_w, void* din, void* actw, float* rowdot,
                           int64_t rows, int F, cudaStream_t stream);
// FiLM: y = x * (1 + scale[g]) + shift[g], g = row / rows_per_group
int launch_film(const void* x, const void* scale, const void* shift, void* y, int64_t rows, int cols,
                int64_t rows_per_group, cudaStream_t stream);
int launch_add(const void* a, const void* b, void* out, int64_t n, cudaStream_t stream);
int launch_l2_flush(void* buf, int64_t bytes, cudaStream_t stream);
// Per-tensor fp8 (e4m3) quantisation for delayed scaling: q = saturate(x * *scale), and the tensor's own absolute
// maximum is folded into *amax (atomic max; the caller turns it into the scale of a later step).
// Knowledge-field FiLM in one kernel: out[t] = h[t] * (1 + s) + b with (s | b) = (sum_c table[c][idx[t][c]]) @ w^T.
// table_ptrs: per rank of the group the base of its shard [C, rows_per_rank, 128] bf16 (peer pointers for the other
// ranks); w [2H, 128] bf16 (scale rows, then shift rows); h, out [tokens, H] bf16 (may alias); e_out [tokens, 128]
// bf16 or null.  D must be 128, H a multiple of 64, C <= 16.
int launch_pq_film(void* const* table_ptrs, int world, const int* idx, const void* w, const void* h, void* out,
                   void* e_out, int64_t tokens, int C, int64_t rows_per_rank, int D, int H, uint32_t* status,
                   cudaStream_t stream);

// In-place merge of two attention partials over disjoint key sets: o_acc / o_b [rows, d] fp32, lse [rows] fp32.
int launch_attn_merge(float* o_acc, float* lse_acc, const float* o_b, const float* lse_b, int64_t rows, int d,
                      cudaStream_t stream);

// Block-scaled quantisation of x [rows, K] (bf16, K % 128 == 0): q [rows, K] e4m3 and the scale chunks
// [ceil(rows / 128)][K / 128][512] described at GemmArgs::sfa.  Scale of a 32-element block = the smallest power of two that
// brings the block's largest magnitude to at most 448, stored as a biased exponent byte; rows past `rows` in the last tile get scale 2^0.
int launch_mx_quantize(const void* x_bf16, void* q_e4m3, void* sf, int64_t rows, int K, cudaStream_t stream);

int launch_fp8_quantize(const void* x_bf16, const float* scale, void* q_e4m3, float* amax, int64_t n,
                        cudaStream_t stream);

// ------------------------------------------------------------------------------------------------
// Selective state-space scan (ssm.cu): fp32 u, delta, y [B, L, D]; A [D, 16]; Bm, Cm [B, L, 16]; Dp [D].
// hs (optional) receives every state [B, L, D, 16] for the backward; h_last (optional, [B, D, 16]) is the initial
// state on entry and the final state on exit (decode carries it from step to step).
// ------------------------------------------------------------------------------------------------
int launch_ssm_scan_fwd(const float* u, const float* delta, const float* A, const float* Bm, const float* Cm,
                        const float* Dp, float* y, float* hs, float* h_last, int batch, int L, int D, int N,
                        cudaStream_t stream);
// dA [D,16], dB, dC [B,L,16] and dD [D] are accumulated into (zero them first); du, ddelta are written
int launch_ssm_scan_bwd(const float* u, const float* delta, const float* A, const float* Bm, const float* Cm,
                        const float* Dp, const float* hs, const float* dy, float* du, float* ddelta, float* dA,
                        float* dB, float* dC, float* dD, int batch, int L, int D, int N, cudaStream_t stream);
// out[M,N] (bf16) = sum over slices of ws[slice][m_pad, N] (fp32) (+ bias[N]): second half of a split-K product
int launch_splitk_reduce(const float* ws, const void* bias, void* out, int slices, int M, int m_pad, int N,
                         cudaStream_t stream);

// ------------------------------------------------------------------------------------------------
// MoE routing (moe.cu)
// ------------------------------------------------------------------------------------------------
// logits fp32 [T, E] (+ bias[E]) -> softmax -> top-k -> renormalise.  Outputs weights fp32 [T,k], idx int32 [T,k],
// probs fp32 [T,E] (optional, for backward), counts int32 [E] (must be zero on entry).
int launch_gate_topk(const float* logits, const float* bias, float* weights, int* idx, float* probs, int* counts,
                     int64_t tokens, int E, int k, int bias_in_combine, int renorm_mode, cudaStream_t stream);
int launch_gate_topk_bwd(const float* dweights, const float* probs, const int* idx, const float* weights,
                         float* dlogits, int64_t tokens, int E, int k, int renorm_mode, cudaStream_t stream);
// counts[E] -> seg_offsets[E+1] (each segment padded to 128 rows), tile_expert[], num_m_tiles, cursor[E] = seg start
int launch_moe_plan(const int* counts, int* seg_offsets, int* tile_expert, int* num_m_tiles, int* cursor, int E,
                    int max_tiles, cudaStream_t stream);
// scatter token rows into expert-sorted order; row_map[t*k+j] = destination row; pad rows are zero-filled
// Deterministic rows: row_map[t*k+j] = seg_offsets[e] + rank of the assignment inside expert e in token order.
int launch_moe_rank(const int* idx, const int* seg_offsets, int* row_map, int64_t n, int E, cudaStream_t stream);
// Capacity rule: per expert keep the `capacity` assignments with the highest probability (ties by token order);
// keep [tokens*k] uint8 scratch, out [tokens,k] = renormalised weights (zeros for fully dropped tokens).
int launch_moe_capacity_mask(const float* weights, const int* idx, const float* probs, const int* counts, uint8_t* keep,
                             float* out, int64_t tokens, int k, int E, int capacity, cudaStream_t stream);
int launch_moe_permute(const void* x, const int* idx, int* cursor, int* row_map, void* xp, int64_t tokens, int k,
                       int cols, cudaStream_t stream);
int launch_moe_zero_pad(void* xp, const int* seg_offsets, const int* counts, int E, int cols, cudaStream_t stream);
// out[t] = sum_j w[t,j] * y[row_map[t,j]] (+ add[t])
int launch_moe_combine(const void* y, const int* row_map, const float* weights, const void* add, void* out,
                       int64_t tokens, int k, int cols, cudaStream_t stream);
// backward of combine: dy[row_map[t,j]] = w[t,j] * dout[t];  dweights[t,j] = <dout[t], y[row]>
int launch_moe_combine_bwd(const void* dout, const void* y, const int* row_map, const float* weights, void* dy,
                           float* dweights, int64_t tokens, int k, int cols, cudaStream_t stream);
// backward of permute: dx[t] = sum_j dxp[row_map[t,j]]
int launch_moe_unpermute_sum(const void* dxp, const int* row_map, void* dx, int64_t tokens, int k, int cols,
                             cudaStream_t stream);
// aux-loss-free bias update: bias += rate * (1/E - counts/total), clamped to [-clamp, clamp]
int launch_gate_bias_update(float* bias, const int* counts, int E, float rate, float clamp, cudaStream_t stream);

// ------------------------------------------------------------------------------------------------
// Attention (attention.cu)
// ------------------------------------------------------------------------------------------------
struct AttnArgs {
  const void* q = nullptr;     // bf16 [Tq, hq, d]   (row stride q_stride elements)
  const void* k = nullptr;     // bf16 [Tk, hk, d]
  const void* v = nullptr;     // bf16 [Tk, hk, d]
  void* o = nullptr;           // bf16 [Tq, hq, d]
  float* lse = nullptr;        // fp32 [hq, Tq]  natural-log LSE of the scaled scores
  const int* cu_q = nullptr;   // int32 [B+1] token offsets of the packed query sequences
  const int* cu_k = nullptr;   // int32 [B+1] token offsets of the packed key sequences
  int batch = 0;
  int max_q = 0, max_k = 0;    // longest sequence (sizes the grid)
  int64_t total_q = 0, total_k = 0;
  int hq = 0, hk = 0, d = 0;
  int64_t q_stride = 0, k_stride = 0, v_stride = 0, o_stride = 0;
  int causal = 1;
  float scale = 1.f;
  uint32_t* status = nullptr;
};
int launch_attn_fwd(const AttnArgs& a, cudaStream_t stream);
struct AttnBwdArgs {
  AttnArgs f;                  // forward tensors (o and lse are inputs here)
  const void* dout = nullptr;  // bf16 [Tq, hq, d]
  void* dq = nullptr;          // bf16 [Tq, hq, d]
  void* dk = nullptr;          // bf16 [Tk, hk, d]
  void* dv = nullptr;          // bf16 [Tk, hk, d]
  float* delta = nullptr;      // fp32 [hq, Tq] scratch
  int64_t do_stride = 0, dq_stride = 0, dk_stride = 0, dv_stride = 0;
};
int launch_attn_bwd(const AttnBwdArgs& a, cudaStream_t stream);
// Paged-KV decode: one query token per sequence.
struct PagedDecodeArgs {
  const void* q = nullptr;         // bf16 [B, hq, d]
  const void* k_cache = nullptr;   // bf16 [num_blocks, block, hk, d]
  const void* v_cache = nullptr;
  const int* block_table = nullptr;  // int32 [B, max_blocks_per_seq]
  const int* seq_lens = nullptr;     // int32 [B]
  void* o = nullptr;               // bf16 [B, hq, d]
  float* partial_o = nullptr;      // fp32 [B, hq, splits, d]   scratch
  float* partial_ml = nullptr;     // fp32 [B, hq, splits, 2]   scratch
  int batch = 0, hq = 0, hk = 0, d = 0, block = 64, max_blocks_per_seq = 0, splits = 1, num_blocks = 0;
  float scale = 1.f;
  uint32_t* status = nullptr;
  bool force_direct = false;       // true: the direct-load kernel (no TMA ring), whatever the block size
};
int launch_paged_decode(const PagedDecodeArgs& a, cudaStream_t stream);
// k, v: [T, hk*d] rows with the given strides; caches: [num_slots, hk*d]; slot_map int32 [T] (-1 = skip)
int launch_kv_cache_write(const void* k, const void* v, void* k_cache, void* v_cache, const int* slot_map,
                          int64_t tokens, int row_elems, int64_t k_stride, int64_t v_stride, int64_t num_slots,
                          uint32_t* status, cudaStream_t stream);

// ------------------------------------------------------------------------------------------------
// Loss / optimizers / misc (loss_optim.cu)
// ------------------------------------------------------------------------------------------------
// Row-wise softmax cross-entropy on fp32 logits [rows, V]: loss[row], lse[row]; in place logits -> dlogits * gscale
// written as bf16 into dlogits (same rows, V) when dlogits != nullptr.
int launch_ce_fwd_bwd(const float* logits, const int64_t* labels, float* loss, void* dlogits_bf16, int64_t rows,
                      int V, int64_t ld, int ignore_index, float grad_scale, cudaStream_t stream);
struct AdamWArgs {
  void* p; const void* g; void* m; void* v; int64_t n;
  int p_dtype, g_dtype, s_dtype;      // 0 = bf16, 1 = fp32
  float lr, beta1, beta2, eps, wd, bc1, bc2, grad_scale;
};
int launch_adamw(const AdamWArgs& a, cudaStream_t stream);
// m = mu * m + g  (fold a gradient into a momentum buffer);  optionally out = g + mu * m (Nesterov)
int launch_momentum(void* m, const void* g, void* out, int64_t n, float mu, float gscale, int nesterov,
                    int first_fold, cudaStream_t stream);
// The same fold on a block-quantised momentum: q int8 [n], scale fp32 [n / 128] (one per 128 consecutive elements),
// re-quantised with stochastic rounding keyed by (seed, element index).  n must be a multiple of 128.
int launch_momentum_q8(void* q, float* scale, const void* g, int64_t n, float mu, float gscale, int first_fold,
                       uint32_t seed, cudaStream_t stream);
// out (bf16) = q * scale
int launch_dequant_q8(const void* q, const float* scale, void* out, int64_t n, cudaStream_t stream);
// p = p * (1 - lr*wd) - lr*scale * u
int launch_muon_apply(void* p, const void* u, int64_t n, float lr, float wd, float scale, cudaStream_t stream);
// x *= 1 / max(||x||_F, eps) per matrix of a batch;  norms scratch fp32 [batch]
int launch_frob_normalize(void* x, float* norms, int batch, int64_t per_matrix, float eps, cudaStream_t stream);
// out = a*x + b*y (bf16 in/out)
int launch_axpby(const void* x, const void* y, void* out, int64_t n, float a, float b, cudaStream_t stream);
// out = a * I + b * A + c * A2 for a batch of n x n bf16 matrices
int launch_ns_poly(const void* A, const void* A2, void* out, int64_t batch, int n, float a, float b, float c,
                   cudaStream_t stream);
int launch_sumsq(const void* x, int dtype, int64_t n, float* out_accum, cudaStream_t stream);
int launch_scale(void* x, int dtype, int64_t n, const float* scale_dev, float scale_host, cudaStream_t stream);
// im2col for non-overlapping patches: img [B,C,H,W] fp32/bf16 -> patches bf16 [B*gh*gw, Kpad] (normalised by mean/std)
int launch_patchify(const void* img, int img_fp32, void* out, int B, int C, int H, int W, int P, int Kpad,
                    const float* mean, const float* stdv, cudaStream_t stream);
// PQ field: out[t] = sum_c table[c][idx[t,c]] (bf16 [C, N, D] table) -> bf16 [T, D]
int launch_pq_gather_sum(const void* table, const int* idx, void* out, int64_t tokens, int C, int64_t N, int D,
                         uint32_t* status, cudaStream_t stream);
int launch_pq_scatter_grad(const void* dout, const int* idx, float* dtable, int64_t tokens, int C, int64_t N, int D,
                           cudaStream_t stream);
int launch_argmax_rows(const void* logits, int dtype, int* out, int64_t rows, int groups, int per_group,
                       cudaStream_t stream);

}  // namespace yv
