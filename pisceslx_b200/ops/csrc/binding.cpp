// PyTorch bindings (torch.ops.yv.*) for the sm_100a kernels.  Every op checks device, dtype, layout
// and alignment on the host, passes raw pointers plus the current stream to a launcher, and raises on
// a non-zero launcher code.  No op allocates: outputs and scratch are passed in by the Python layer.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>
#include <torch/torch.h>

#include "yv_ops.h"

namespace {

using torch::Tensor;

inline cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

inline void check_cuda(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
}
inline void check_bf16(const Tensor& t, const char* name) {
  check_cuda(t, name);
  TORCH_CHECK(t.scalar_type() == at::kBFloat16, name, " must be bfloat16");
}
inline void check_f32(const Tensor& t, const char* name) {
  check_cuda(t, name);
  TORCH_CHECK(t.scalar_type() == at::kFloat, name, " must be float32");
}
inline void check_i32(const Tensor& t, const char* name) {
  check_cuda(t, name);
  TORCH_CHECK(t.scalar_type() == at::kInt, name, " must be int32");
}
inline void check_rc(int rc, const char* what) {
  TORCH_CHECK(rc == 0, "pisceslx_b200 kernel launch failed: ", what, " rc=", rc,
              rc > 0 ? std::string(" (") + cudaGetErrorString(static_cast<cudaError_t>(rc)) + ")" : std::string());
}
inline const void* optp(const c10::optional<Tensor>& t) { return t.has_value() ? t->data_ptr() : nullptr; }
inline uint32_t* statusp(const c10::optional<Tensor>& t) {
  return t.has_value() ? reinterpret_cast<uint32_t*>(t->data_ptr()) : nullptr;
}
inline int dt_code(const Tensor& t) {
  if (t.scalar_type() == at::kFloat) return 1;
  TORCH_CHECK(t.scalar_type() == at::kBFloat16, "expected bf16 or fp32 tensor");
  return 0;
}

// ------------------------------------------------------------------------------------------------
// GEMM.  a: [M,K] (a_mn=false) or [K,M] (a_mn=true); b: [N,K] (b_mn=false) or [K,N] (b_mn=true); 2-D, inner
// stride 1.  c: [M,N] bf16 or fp32.
// ------------------------------------------------------------------------------------------------
void gemm(const Tensor& a, const Tensor& b, Tensor c, bool a_mn, bool b_mn, bool accumulate, int64_t bn,
          const c10::optional<Tensor>& status) {
  check_bf16(a, "a"); check_bf16(b, "b"); check_cuda(c, "c");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && c.dim() == 2, "gemm operands must be 2-D");
  TORCH_CHECK(a.stride(1) == 1 && b.stride(1) == 1 && c.stride(1) == 1, "gemm operands need unit inner stride");
  const c10::cuda::CUDAGuard guard(a.device());
  yv::GemmArgs g;
  g.a = a.data_ptr(); g.b = b.data_ptr(); g.c = c.data_ptr();
  g.a_mn = a_mn; g.b_mn = b_mn;
  g.M = static_cast<int>(a_mn ? a.size(1) : a.size(0));
  g.K = static_cast<int>(a_mn ? a.size(0) : a.size(1));
  g.N = static_cast<int>(b_mn ? b.size(1) : b.size(0));
  const int64_t kb = b_mn ? b.size(0) : b.size(1);
  TORCH_CHECK(kb == g.K, "gemm: inner dimensions differ: ", g.K, " vs ", kb);
  TORCH_CHECK(c.size(0) == g.M && c.size(1) == g.N, "gemm: output shape mismatch");
  g.lda = a.stride(0); g.ldb = b.stride(0); g.ldc = c.stride(0);
  g.out_fp32 = dt_code(c);
  g.accumulate = accumulate ? 1 : 0;
  g.bn = static_cast<int>(bn);
  g.status = statusp(status);
  check_rc(yv::launch_gemm(g, cur_stream()), "gemm");
}

// Grouped along M: a [rows_total, K] expert-sorted/padded; b [E, N, K] (b_mn=false) or [E, K, N] (b_mn=true);
// c [rows_total, N].
void gemm_grouped_m(const Tensor& a, const Tensor& b, Tensor c, const Tensor& tile_expert, const Tensor& num_m_tiles,
                    bool b_mn, int64_t bn, const c10::optional<Tensor>& status) {
  check_bf16(a, "a"); check_bf16(b, "b"); check_cuda(c, "c");
  check_i32(tile_expert, "tile_expert"); check_i32(num_m_tiles, "num_m_tiles");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 3 && c.dim() == 2 && a.is_contiguous() && b.is_contiguous() &&
              c.is_contiguous(), "gemm_grouped_m: contiguous a[rows,K], b[E,*,*], c[rows,N] expected");
  const c10::cuda::CUDAGuard guard(a.device());
  yv::GemmArgs g;
  g.a = a.data_ptr(); g.b = b.data_ptr(); g.c = c.data_ptr();
  g.b_mn = b_mn;
  g.mode = 1;
  g.num_groups = static_cast<int>(b.size(0));
  g.rows_total = a.size(0);
  g.M = static_cast<int>(a.size(0));
  g.K = static_cast<int>(a.size(1));
  g.N = static_cast<int>(b_mn ? b.size(2) : b.size(1));
  TORCH_CHECK((b_mn ? b.size(1) : b.size(2)) == g.K, "gemm_grouped_m: K mismatch");
  TORCH_CHECK(c.size(0) == a.size(0) && c.size(1) == g.N, "gemm_grouped_m: output shape mismatch");
  TORCH_CHECK(tile_expert.numel() * 128 >= a.size(0), "tile_expert too short");
  g.out_fp32 = dt_code(c);
  g.tile_expert = tile_expert.data_ptr<int>();
  g.num_m_tiles = num_m_tiles.data_ptr<int>();
  g.bn = static_cast<int>(bn);
  g.status = statusp(status);
  check_rc(yv::launch_gemm(g, cur_stream()), "gemm_grouped_m");
}

// Grouped along K (weight gradients): a [rows_total, M], b [rows_total, N] (both "MN-major"), c [E, M, N];
// seg_offsets int32 [E+1].
void gemm_grouped_k(const Tensor& a, const Tensor& b, Tensor c, const Tensor& seg_offsets, bool accumulate,
                    int64_t bn, const c10::optional<Tensor>& status) {
  check_bf16(a, "a"); check_bf16(b, "b"); check_cuda(c, "c"); check_i32(seg_offsets, "seg_offsets");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && c.dim() == 3 && a.is_contiguous() && b.is_contiguous() &&
              c.is_contiguous(), "gemm_grouped_k: contiguous a[rows,M], b[rows,N], c[E,M,N] expected");
  TORCH_CHECK(a.size(0) == b.size(0), "gemm_grouped_k: row counts differ");
  const c10::cuda::CUDAGuard guard(a.device());
  yv::GemmArgs g;
  g.a = a.data_ptr(); g.b = b.data_ptr(); g.c = c.data_ptr();
  g.a_mn = true; g.b_mn = true;
  g.mode = 2;
  g.num_groups = static_cast<int>(c.size(0));
  g.rows_total = a.size(0);
  g.M = static_cast<int>(a.size(1));
  g.N = static_cast<int>(b.size(1));
  g.K = 0;
  TORCH_CHECK(c.size(1) == g.M && c.size(2) == g.N, "gemm_grouped_k: output shape mismatch");
  TORCH_CHECK(seg_offsets.numel() == c.size(0) + 1, "seg_offsets must have E+1 entries");
  g.out_fp32 = dt_code(c);
  g.accumulate = accumulate ? 1 : 0;
  g.seg_offsets = seg_offsets.data_ptr<int>();
  g.bn = static_cast<int>(bn);
  g.status = statusp(status);
  check_rc(yv::launch_gemm(g, cur_stream()), "gemm_grouped_k");
}

// Batched: a [G, M, K] (or [G, K, M] when a_mn), b [G, N, K] (or [G, K, N] when b_mn), c [G, M, N]; contiguous.
void gemm_batched(const Tensor& a, const Tensor& b, Tensor c, bool a_mn, bool b_mn, bool accumulate, int64_t bn,
                  const c10::optional<Tensor>& status, bool symmetric) {
  check_bf16(a, "a"); check_bf16(b, "b"); check_cuda(c, "c");
  TORCH_CHECK(a.dim() == 3 && b.dim() == 3 && c.dim() == 3 && a.is_contiguous() && b.is_contiguous() &&
              c.is_contiguous(), "gemm_batched: contiguous 3-D operands expected");
  TORCH_CHECK(a.size(0) == b.size(0) && a.size(0) == c.size(0), "gemm_batched: batch sizes differ");
  const c10::cuda::CUDAGuard guard(a.device());
  yv::GemmArgs g;
  g.a = a.data_ptr(); g.b = b.data_ptr(); g.c = c.data_ptr();
  g.a_mn = a_mn; g.b_mn = b_mn;
  g.mode = 3;
  g.num_groups = static_cast<int>(a.size(0));
  g.M = static_cast<int>(a_mn ? a.size(2) : a.size(1));
  g.K = static_cast<int>(a_mn ? a.size(1) : a.size(2));
  g.N = static_cast<int>(b_mn ? b.size(2) : b.size(1));
  TORCH_CHECK((b_mn ? b.size(1) : b.size(2)) == g.K, "gemm_batched: K mismatch");
  TORCH_CHECK(c.size(1) == g.M && c.size(2) == g.N, "gemm_batched: output shape mismatch");
  g.out_fp32 = dt_code(c);
  g.accumulate = accumulate ? 1 : 0;
  g.bn = static_cast<int>(bn);
  g.status = statusp(status);
  g.symmetric = symmetric;
  check_rc(yv::launch_gemm(g, cur_stream()), "gemm_batched");
}

// c[g] = ec * (a[g] @ b[g]^T) + eb * cin[g] + ea * I   (square [n, n] outputs, n a multiple of 128): the
// Newton-Schulz polynomial b A + c A^2 + a I formed in the epilogue of the A A product
void gemm_batched_affine(const Tensor& a, const Tensor& b, const Tensor& cin, Tensor c, double ea, double eb, double ec,
                         const c10::optional<Tensor>& status, bool symmetric) {
  check_bf16(a, "a"); check_bf16(b, "b"); check_bf16(cin, "cin"); check_bf16(c, "c");
  TORCH_CHECK(a.dim() == 3 && b.dim() == 3 && c.dim() == 3 && a.is_contiguous() && b.is_contiguous() &&
              c.is_contiguous() && cin.is_contiguous(), "gemm_batched_affine: contiguous 3-D operands expected");
  TORCH_CHECK(cin.sizes() == c.sizes() && c.size(1) == c.size(2) && a.size(0) == c.size(0) && b.size(0) == c.size(0),
              "gemm_batched_affine: square outputs with cin of the same shape expected");
  TORCH_CHECK(c.data_ptr() != a.data_ptr() && c.data_ptr() != b.data_ptr() && c.data_ptr() != cin.data_ptr(),
              "gemm_batched_affine: the output must not alias an input");
  const c10::cuda::CUDAGuard guard(a.device());
  yv::GemmArgs g;
  g.a = a.data_ptr(); g.b = b.data_ptr(); g.c = c.data_ptr();
  g.mode = 3;
  g.num_groups = static_cast<int>(a.size(0));
  g.M = static_cast<int>(a.size(1)); g.K = static_cast<int>(a.size(2)); g.N = static_cast<int>(b.size(1));
  TORCH_CHECK(b.size(2) == g.K && c.size(1) == g.M && c.size(2) == g.N, "gemm_batched_affine: shape mismatch");
  g.epi_cin = cin.data_ptr();
  g.epi_a = static_cast<float>(ea); g.epi_b = static_cast<float>(eb); g.epi_c = static_cast<float>(ec);
  g.status = statusp(status);
  g.symmetric = symmetric;
  check_rc(yv::launch_gemm(g, cur_stream()), "gemm_batched_affine");
}

// ------------------------------------------------------------------------------------------------
// elementwise
// ------------------------------------------------------------------------------------------------
void rmsnorm_fwd(const Tensor& x, const c10::optional<Tensor>& residual, const Tensor& w,
                 const c10::optional<Tensor>& film_scale, const c10::optional<Tensor>& film_shift,
                 int64_t film_rows_per_group, Tensor y, const c10::optional<Tensor>& res_out, Tensor rstd, double eps) {
  check_bf16(x, "x"); check_bf16(w, "w"); check_bf16(y, "y"); check_f32(rstd, "rstd");
  TORCH_CHECK(x.is_contiguous() && y.is_contiguous() && w.is_contiguous(), "rmsnorm: contiguous tensors expected");
  const int cols = static_cast<int>(x.size(-1));
  const int64_t rows = x.numel() / cols;
  TORCH_CHECK(w.numel() == cols && rstd.numel() >= rows, "rmsnorm: shape mismatch");
  const c10::cuda::CUDAGuard guard(x.device());
  check_rc(yv::launch_rmsnorm_fwd(x.data_ptr(), optp(residual), w.data_ptr(), optp(film_scale), optp(film_shift),
                                  film_rows_per_group, y.data_ptr(),
                                  res_out.has_value() ? res_out->data_ptr() : nullptr, rstd.data_ptr<float>(), rows,
                                  cols, static_cast<float>(eps), cur_stream()),
           "rmsnorm_fwd");
}

void rmsnorm_bwd(const Tensor& dy, const Tensor& x, const Tensor& w, const Tensor& rstd,
                 const c10::optional<Tensor>& dres_in, Tensor dx, Tensor dw_partial, Tensor dw, bool accumulate_dw) {
  check_bf16(dy, "dy"); check_bf16(x, "x"); check_bf16(w, "w"); check_f32(rstd, "rstd"); check_bf16(dx, "dx");
  check_f32(dw_partial, "dw_partial");
  const int cols = static_cast<int>(x.size(-1));
  const int64_t rows = x.numel() / cols;
  const int blocks = static_cast<int>(dw_partial.size(0));
  TORCH_CHECK(dw_partial.size(1) == cols, "dw_partial must be [blocks, cols]");
  const c10::cuda::CUDAGuard guard(x.device());
  check_rc(yv::launch_rmsnorm_bwd(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr<float>(), optp(dres_in),
                                  dx.data_ptr(), dw_partial.data_ptr<float>(), blocks, rows, cols, cur_stream()),
           "rmsnorm_bwd");
  const int used = static_cast<int>(rows < blocks ? rows : blocks);
  check_rc(yv::launch_colsum(dw_partial.data_ptr<float>(), used, cols, dw.data_ptr(), dt_code(dw),
                             accumulate_dw ? 1 : 0, cur_stream()),
           "colsum");
}

void rope(Tensor q, Tensor k, const Tensor& cos_t, const Tensor& sin_t, const Tensor& positions, int64_t hq,
          int64_t hk, int64_t head_dim, int64_t rot_dim, bool inverse) {
  check_bf16(q, "q"); check_bf16(k, "k"); check_f32(cos_t, "cos"); check_f32(sin_t, "sin");
  check_i32(positions, "positions");
  TORCH_CHECK(q.dim() == 2 && k.dim() == 2 && q.stride(1) == 1 && k.stride(1) == 1, "rope: q,k must be [T, h*d] views");
  const int64_t tokens = q.size(0);
  TORCH_CHECK(positions.numel() == tokens && k.size(0) == tokens, "rope: token count mismatch");
  TORCH_CHECK(cos_t.size(-1) * 2 == rot_dim, "rope: table width must be rot_dim/2");
  const c10::cuda::CUDAGuard guard(q.device());
  check_rc(yv::launch_rope_tables(q.data_ptr(), k.data_ptr(), cos_t.data_ptr<float>(), sin_t.data_ptr<float>(),
                                  positions.data_ptr<int>(), tokens, static_cast<int>(hq), static_cast<int>(hk),
                                  static_cast<int>(head_dim), static_cast<int>(rot_dim), inverse ? 1 : 0, q.stride(0),
                                  k.stride(0), cur_stream()),
           "rope");
}

void rope3d(Tensor q, Tensor k, const Tensor& pos_thw, int64_t hq, int64_t hk, int64_t head_dim, int64_t d_t,
            int64_t d_h, int64_t d_w, double theta, bool inverse) {
  check_bf16(q, "q"); check_bf16(k, "k"); check_i32(pos_thw, "pos_thw");
  TORCH_CHECK(q.is_contiguous() && k.is_contiguous(), "rope3d: contiguous q,k expected");
  const int64_t tokens = pos_thw.size(0);
  const c10::cuda::CUDAGuard guard(q.device());
  check_rc(yv::launch_rope3d(q.data_ptr(), k.data_ptr(), pos_thw.data_ptr<int>(), tokens, static_cast<int>(hq),
                             static_cast<int>(hk), static_cast<int>(head_dim), static_cast<int>(d_t),
                             static_cast<int>(d_h), static_cast<int>(d_w), static_cast<float>(theta), inverse ? 1 : 0,
                             cur_stream()),
           "rope3d");
}

void swiglu_fwd(const Tensor& in, Tensor out) {
  check_bf16(in, "in"); check_bf16(out, "out");
  TORCH_CHECK(in.is_contiguous() && out.is_contiguous(), "swiglu: contiguous expected");
  const int F = static_cast<int>(out.size(-1));
  TORCH_CHECK(in.size(-1) == 2 * F, "swiglu: input must be [rows, 2F]");
  const c10::cuda::CUDAGuard guard(in.device());
  check_rc(yv::launch_swiglu_fwd(in.data_ptr(), out.data_ptr(), out.numel() / F, F, cur_stream()), "swiglu_fwd");
}

void swiglu_bwd_rows(const Tensor& in, const Tensor& dact, const Tensor& row_w, Tensor din, Tensor actw, Tensor rowdot) {
  check_bf16(in, "in"); check_bf16(dact, "dact"); check_bf16(din, "din"); check_bf16(actw, "actw");
  TORCH_CHECK(in.is_contiguous() && dact.is_contiguous() && din.is_contiguous() && actw.is_contiguous() &&
              row_w.is_contiguous() && rowdot.is_contiguous(), "swiglu_bwd_rows: contiguous expected");
  TORCH_CHECK(row_w.scalar_type() == at::kFloat && rowdot.scalar_type() == at::kFloat, "swiglu_bwd_rows: fp32 row vectors");
  const int F = static_cast<int>(dact.size(-1));
  const int64_t rows = dact.numel() / F;
  TORCH_CHECK(in.size(-1) == 2 * F && in.numel() == rows * 2 * F && din.numel() == in.numel() && actw.numel() == dact.numel() &&
              row_w.numel() == rows && rowdot.numel() == rows, "swiglu_bwd_rows: shape mismatch");
  const c10::cuda::CUDAGuard guard(in.device());
  check_rc(yv::launch_swiglu_bwd_rows(in.data_ptr(), dact.data_ptr(), row_w.data_ptr<float>(), din.data_ptr(), actw.data_ptr(),
                                      rowdot.data_ptr<float>(), rows, F, cur_stream()), "swiglu_bwd_rows");
}

void swiglu_bwd(const Tensor& in, const Tensor& dout, Tensor din) {
  check_bf16(in, "in"); check_bf16(dout, "dout"); check_bf16(din, "din");
  TORCH_CHECK(in.is_contiguous() && dout.is_contiguous() && din.is_contiguous(), "swiglu: contiguous expected");
  const int F = static_cast<int>(dout.size(-1));
  const c10::cuda::CUDAGuard guard(in.device());
  check_rc(yv::launch_swiglu_bwd(in.data_ptr(), dout.data_ptr(), din.data_ptr(), dout.numel() / F, F, cur_stream()),
           "swiglu_bwd");
}

void film(const Tensor& x, const Tensor& scale, const Tensor& shift, Tensor y, int64_t rows_per_group) {
  check_bf16(x, "x"); check_bf16(scale, "scale"); check_bf16(shift, "shift"); check_bf16(y, "y");
  const int cols = static_cast<int>(x.size(-1));
  const c10::cuda::CUDAGuard guard(x.device());
  check_rc(yv::launch_film(x.data_ptr(), scale.data_ptr(), shift.data_ptr(), y.data_ptr(), x.numel() / cols, cols,
                           rows_per_group, cur_stream()),
           "film");
}

void add(const Tensor& a, const Tensor& b, Tensor out) {
  check_bf16(a, "a"); check_bf16(b, "b"); check_bf16(out, "out");
  const c10::cuda::CUDAGuard guard(a.device());
  check_rc(yv::launch_add(a.data_ptr(), b.data_ptr(), out.data_ptr(), a.numel(), cur_stream()), "add");
}

// Split-K product for skinny activations: y[M,N] = a[M,K] @ b[N,K]^T (+ bias) with the K range cut into
// seg_offsets.numel()-1 slices (offsets are multiples of 64), each reduced by its own CTAs into the fp32 workspace
// ws [slices, ceil128(M), N]; a second kernel sums the slices in a fixed order (bit-reproducible).
void gemm_splitk(const Tensor& a, const Tensor& b, Tensor ws, const Tensor& seg_offsets,
                 const c10::optional<Tensor>& bias, Tensor out, const c10::optional<Tensor>& status) {
  check_bf16(a, "a"); check_bf16(b, "b"); check_f32(ws, "ws"); check_i32(seg_offsets, "seg_offsets"); check_bf16(out, "out");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && a.stride(1) == 1 && b.stride(1) == 1 && out.is_contiguous() &&
              ws.is_contiguous(), "gemm_splitk: a [M,K], b [N,K] with unit inner stride, contiguous ws and out");
  const int slices = static_cast<int>(seg_offsets.numel()) - 1;
  const int M = static_cast<int>(a.size(0)), K = static_cast<int>(a.size(1)), N = static_cast<int>(b.size(0));
  const int m_pad = (M + 127) / 128 * 128;
  TORCH_CHECK(slices >= 1 && b.size(1) == K && out.size(0) == M && out.size(1) == N, "gemm_splitk: shape mismatch");
  TORCH_CHECK(ws.numel() >= static_cast<int64_t>(slices) * m_pad * N, "gemm_splitk: workspace too small");
  const c10::cuda::CUDAGuard guard(a.device());
  yv::GemmArgs g;
  g.a = a.data_ptr(); g.b = b.data_ptr(); g.c = ws.data_ptr();
  g.M = M; g.N = N; g.K = K;
  g.lda = a.stride(0); g.ldb = b.stride(0); g.ldc = N;
  g.out_fp32 = 1;
  g.mode = 4;
  g.num_groups = slices;
  g.seg_offsets = seg_offsets.data_ptr<int>();
  g.status = statusp(status);
  check_rc(yv::launch_gemm(g, cur_stream()), "gemm_splitk");
  check_rc(yv::launch_splitk_reduce(ws.data_ptr<float>(), bias.has_value() ? bias->data_ptr() : nullptr,
                                    out.data_ptr(), slices, M, m_pad, N, cur_stream()), "splitk_reduce");
}

inline void check_fp8(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && (t.scalar_type() == at::kFloat8_e4m3fn || t.scalar_type() == at::kByte), name,
              " must be a CUDA float8_e4m3fn (or uint8) tensor");
}

// q = saturate_e4m3(x * scale[0]); amax[0] = max(amax[0], max|x|)
void fp8_quantize(const Tensor& x, const Tensor& scale, Tensor q, const c10::optional<Tensor>& amax) {
  check_bf16(x, "x"); check_f32(scale, "scale"); check_fp8(q, "q");
  TORCH_CHECK(x.is_contiguous() && q.is_contiguous() && q.numel() == x.numel(), "fp8_quantize: contiguous, same size");
  const c10::cuda::CUDAGuard guard(x.device());
  check_rc(yv::launch_fp8_quantize(x.data_ptr(), scale.data_ptr<float>(), q.data_ptr(),
                                   amax.has_value() ? amax->data_ptr<float>() : nullptr, x.numel(), cur_stream()),
           "fp8_quantize");
}

// c[M,N] (bf16) = (a_q[M,K] @ b_q[N,K]^T) * out_scale[0], e4m3 operands, fp32 accumulation in TMEM
void gemm_fp8(const Tensor& a, const Tensor& b, Tensor c, const Tensor& out_scale, int64_t bn,
              const c10::optional<Tensor>& status) {
  check_fp8(a, "a"); check_fp8(b, "b"); check_bf16(c, "c"); check_f32(out_scale, "out_scale");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && a.is_contiguous() && b.is_contiguous() && c.is_contiguous() &&
              a.size(1) == b.size(1) && c.size(0) == a.size(0) && c.size(1) == b.size(0),
              "gemm_fp8: a [M,K], b [N,K], c [M,N] contiguous");
  TORCH_CHECK(a.size(1) % 16 == 0, "gemm_fp8: K must be a multiple of 16");
  const c10::cuda::CUDAGuard guard(a.device());
  yv::GemmArgs g;
  g.a = a.data_ptr(); g.b = b.data_ptr(); g.c = c.data_ptr();
  g.M = static_cast<int>(a.size(0)); g.K = static_cast<int>(a.size(1)); g.N = static_cast<int>(b.size(0));
  g.fp8 = true;
  g.out_scale = out_scale.data_ptr<float>();
  g.bn = static_cast<int>(bn);
  g.status = statusp(status);
  check_rc(yv::launch_gemm(g, cur_stream()), "gemm_fp8");
}

void attn_merge(Tensor o_acc, Tensor lse_acc, const Tensor& o_b, const Tensor& lse_b) {
  check_f32(o_acc, "o_acc"); check_f32(lse_acc, "lse_acc"); check_f32(o_b, "o_b"); check_f32(lse_b, "lse_b");
  TORCH_CHECK(o_acc.is_contiguous() && lse_acc.is_contiguous() && o_b.is_contiguous() && lse_b.is_contiguous() &&
              o_acc.sizes() == o_b.sizes() && lse_acc.sizes() == lse_b.sizes() &&
              o_acc.numel() == lse_acc.numel() * o_acc.size(-1), "attn_merge: o [..., d] and lse [...] of both partials");
  const c10::cuda::CUDAGuard guard(o_acc.device());
  check_rc(yv::launch_attn_merge(o_acc.data_ptr<float>(), lse_acc.data_ptr<float>(), o_b.data_ptr<float>(),
                                 lse_b.data_ptr<float>(), lse_acc.numel(), static_cast<int>(o_acc.size(-1)), cur_stream()),
           "attn_merge");
}

// x [rows, K] bf16 -> q [rows, K] e4m3 + sf uint8 [ceil(rows/128), K/128, 512] (one e8m0 scale per 32 elements)
void mx_quantize(const Tensor& x, Tensor q, Tensor sf) {
  check_bf16(x, "x"); check_fp8(q, "q");
  TORCH_CHECK(sf.is_cuda() && sf.scalar_type() == at::kByte && sf.is_contiguous(), "mx_quantize: sf must be CUDA uint8");
  TORCH_CHECK(x.dim() == 2 && x.is_contiguous() && q.is_contiguous() && q.numel() == x.numel(), "mx_quantize: x [rows,K]");
  const int64_t rows = x.size(0), K = x.size(1);
  TORCH_CHECK(K % 128 == 0, "mx_quantize: K must be a multiple of 128");
  TORCH_CHECK(sf.numel() == (rows + 127) / 128 * (K / 128) * 512, "mx_quantize: sf has the wrong size");
  const c10::cuda::CUDAGuard guard(x.device());
  check_rc(yv::launch_mx_quantize(x.data_ptr(), q.data_ptr(), sf.data_ptr(), rows, static_cast<int>(K), cur_stream()),
           "mx_quantize");
}

// c (bf16) = A B^T with block-scaled e4m3 operands (scales sfa / sfb in the chunk layout of mx_quantize).
//   dense:   a [M,K], b [N,K], c [M,N]
//   grouped: a [rows,K] (128-row tiles, tile i multiplies expert tile_expert[i]), b [E,N,K], c [rows,N]
void gemm_mxfp8(const Tensor& a, const Tensor& sfa, const Tensor& b, const Tensor& sfb, Tensor c,
                const c10::optional<Tensor>& tile_expert, const c10::optional<Tensor>& num_m_tiles, int64_t bn,
                const c10::optional<Tensor>& status) {
  check_fp8(a, "a"); check_fp8(b, "b"); check_bf16(c, "c");
  TORCH_CHECK(sfa.is_cuda() && sfa.scalar_type() == at::kByte && sfb.is_cuda() && sfb.scalar_type() == at::kByte &&
              sfa.is_contiguous() && sfb.is_contiguous(), "gemm_mxfp8: scale tensors must be CUDA uint8");
  TORCH_CHECK(a.dim() == 2 && a.is_contiguous() && b.is_contiguous() && c.is_contiguous() && c.dim() == 2,
              "gemm_mxfp8: contiguous operands expected");
  const bool grouped = tile_expert.has_value();
  TORCH_CHECK(b.dim() == (grouped ? 3 : 2), "gemm_mxfp8: b is [N,K], or [E,N,K] with tile_expert");
  const int64_t K = a.size(1), N = grouped ? b.size(1) : b.size(0), brows = grouped ? b.size(0) * b.size(1) : b.size(0);
  TORCH_CHECK(b.size(-1) == K && K % 128 == 0, "gemm_mxfp8: K mismatch or not a multiple of 128");
  TORCH_CHECK(c.size(0) == a.size(0) && c.size(1) == N, "gemm_mxfp8: output shape mismatch");
  TORCH_CHECK(sfa.numel() == (a.size(0) + 127) / 128 * (K / 128) * 512 && sfb.numel() == (brows + 127) / 128 * (K / 128) * 512,
              "gemm_mxfp8: scale tensor size mismatch");
  TORCH_CHECK(brows % 128 == 0 && (!grouped || N % 128 == 0), "gemm_mxfp8: rows of b must come in multiples of 128");
  const c10::cuda::CUDAGuard guard(a.device());
  yv::GemmArgs g;
  g.a = a.data_ptr(); g.b = b.data_ptr(); g.c = c.data_ptr();
  g.sfa = sfa.data_ptr(); g.sfb = sfb.data_ptr();
  g.M = static_cast<int>(a.size(0)); g.K = static_cast<int>(K); g.N = static_cast<int>(N);
  g.fp8 = true;
  if (grouped) {
    TORCH_CHECK(num_m_tiles.has_value(), "gemm_mxfp8: grouped mode needs num_m_tiles");
    check_i32(*tile_expert, "tile_expert"); check_i32(*num_m_tiles, "num_m_tiles");
    TORCH_CHECK(a.size(0) % 128 == 0 && tile_expert->numel() * 128 >= a.size(0), "gemm_mxfp8: grouped rows / tile list");
    g.mode = 1;
    g.num_groups = static_cast<int>(b.size(0));
    g.rows_total = a.size(0);
    g.tile_expert = tile_expert->data_ptr<int>();
    g.num_m_tiles = num_m_tiles->data_ptr<int>();
  }
  g.bn = static_cast<int>(bn);
  g.status = statusp(status);
  check_rc(yv::launch_gemm(g, cur_stream()), "gemm_mxfp8");
}

void ssm_scan_fwd(const Tensor& u, const Tensor& delta, const Tensor& A, const Tensor& Bm, const Tensor& Cm,
                  const Tensor& Dp, Tensor y, const c10::optional<Tensor>& hs, const c10::optional<Tensor>& h_last) {
  check_f32(u, "u"); check_f32(delta, "delta"); check_f32(A, "A"); check_f32(Bm, "B"); check_f32(Cm, "C");
  check_f32(Dp, "D"); check_f32(y, "y");
  TORCH_CHECK(u.dim() == 3 && u.is_contiguous() && delta.is_contiguous() && Bm.is_contiguous() && Cm.is_contiguous() &&
              A.is_contiguous() && y.is_contiguous(), "ssm_scan_fwd: contiguous [B,L,D] / [B,L,N] / [D,N] tensors");
  const c10::cuda::CUDAGuard guard(u.device());
  check_rc(yv::launch_ssm_scan_fwd(u.data_ptr<float>(), delta.data_ptr<float>(), A.data_ptr<float>(),
                                   Bm.data_ptr<float>(), Cm.data_ptr<float>(), Dp.data_ptr<float>(), y.data_ptr<float>(),
                                   hs.has_value() ? hs->data_ptr<float>() : nullptr,
                                   h_last.has_value() ? h_last->data_ptr<float>() : nullptr,
                                   static_cast<int>(u.size(0)), static_cast<int>(u.size(1)), static_cast<int>(u.size(2)),
                                   static_cast<int>(A.size(1)), cur_stream()), "ssm_scan_fwd");
}

void ssm_scan_bwd(const Tensor& u, const Tensor& delta, const Tensor& A, const Tensor& Bm, const Tensor& Cm,
                  const Tensor& Dp, const Tensor& hs, const Tensor& dy, Tensor du, Tensor ddelta, Tensor dA, Tensor dB,
                  Tensor dC, Tensor dD) {
  check_f32(u, "u"); check_f32(hs, "hs"); check_f32(dy, "dy"); check_f32(du, "du"); check_f32(ddelta, "ddelta");
  check_f32(dA, "dA"); check_f32(dB, "dB"); check_f32(dC, "dC"); check_f32(dD, "dD");
  TORCH_CHECK(u.is_contiguous() && delta.is_contiguous() && hs.is_contiguous() && dy.is_contiguous() &&
              du.is_contiguous() && ddelta.is_contiguous(), "ssm_scan_bwd: contiguous tensors expected");
  const c10::cuda::CUDAGuard guard(u.device());
  check_rc(yv::launch_ssm_scan_bwd(u.data_ptr<float>(), delta.data_ptr<float>(), A.data_ptr<float>(),
                                   Bm.data_ptr<float>(), Cm.data_ptr<float>(), Dp.data_ptr<float>(), hs.data_ptr<float>(),
                                   dy.data_ptr<float>(), du.data_ptr<float>(), ddelta.data_ptr<float>(),
                                   dA.data_ptr<float>(), dB.data_ptr<float>(), dC.data_ptr<float>(), dD.data_ptr<float>(),
                                   static_cast<int>(u.size(0)), static_cast<int>(u.size(1)), static_cast<int>(u.size(2)),
                                   static_cast<int>(A.size(1)), cur_stream()), "ssm_scan_bwd");
}

void l2_flush(Tensor buf) {
  check_cuda(buf, "buf");
  const c10::cuda::CUDAGuard guard(buf.device());
  check_rc(yv::launch_l2_flush(buf.data_ptr(), buf.numel() * buf.element_size(), cur_stream()), "l2_flush");
}

// ------------------------------------------------------------------------------------------------
// MoE
// ------------------------------------------------------------------------------------------------
void gate_topk(const Tensor& logits, const c10::optional<Tensor>& bias, Tensor weights, Tensor idx,
               const c10::optional<Tensor>& probs, Tensor counts, bool bias_in_combine, int64_t renorm_mode) {
  check_f32(logits, "logits"); check_f32(weights, "weights"); check_i32(idx, "idx"); check_i32(counts, "counts");
  TORCH_CHECK(logits.is_contiguous(), "gate: contiguous logits expected");
  const int E = static_cast<int>(logits.size(-1));
  const int k = static_cast<int>(weights.size(-1));
  const c10::cuda::CUDAGuard guard(logits.device());
  check_rc(yv::launch_gate_topk(logits.data_ptr<float>(), reinterpret_cast<const float*>(optp(bias)),
                                weights.data_ptr<float>(), idx.data_ptr<int>(),
                                probs.has_value() ? probs->data_ptr<float>() : nullptr, counts.data_ptr<int>(),
                                logits.numel() / E, E, k, bias_in_combine ? 1 : 0, static_cast<int>(renorm_mode),
                                cur_stream()),
           "gate_topk");
}

void gate_topk_bwd(const Tensor& dweights, const Tensor& probs, const Tensor& idx, const Tensor& weights,
                   Tensor dlogits, int64_t renorm_mode) {
  check_f32(dweights, "dweights"); check_f32(probs, "probs"); check_i32(idx, "idx"); check_f32(weights, "weights");
  check_f32(dlogits, "dlogits");
  const int E = static_cast<int>(probs.size(-1));
  const int k = static_cast<int>(weights.size(-1));
  const c10::cuda::CUDAGuard guard(probs.device());
  check_rc(yv::launch_gate_topk_bwd(dweights.data_ptr<float>(), probs.data_ptr<float>(), idx.data_ptr<int>(),
                                    weights.data_ptr<float>(), dlogits.data_ptr<float>(), probs.numel() / E, E, k,
                                    static_cast<int>(renorm_mode), cur_stream()),
           "gate_topk_bwd");
}

void moe_plan(const Tensor& counts, Tensor seg_offsets, Tensor tile_expert, Tensor num_m_tiles, Tensor cursor) {
  check_i32(counts, "counts"); check_i32(seg_offsets, "seg_offsets"); check_i32(tile_expert, "tile_expert");
  check_i32(num_m_tiles, "num_m_tiles"); check_i32(cursor, "cursor");
  const c10::cuda::CUDAGuard guard(counts.device());
  check_rc(yv::launch_moe_plan(counts.data_ptr<int>(), seg_offsets.data_ptr<int>(), tile_expert.data_ptr<int>(),
                               num_m_tiles.data_ptr<int>(), cursor.data_ptr<int>(), static_cast<int>(counts.numel()),
                               static_cast<int>(tile_expert.numel()), cur_stream()),
           "moe_plan");
}

void moe_rank(const Tensor& idx, const Tensor& seg_offsets, Tensor row_map) {
  check_i32(idx, "idx"); check_i32(seg_offsets, "seg_offsets"); check_i32(row_map, "row_map");
  TORCH_CHECK(idx.is_contiguous() && row_map.is_contiguous() && row_map.numel() == idx.numel(), "moe_rank: idx / row_map [T,k]");
  const c10::cuda::CUDAGuard guard(idx.device());
  check_rc(yv::launch_moe_rank(idx.data_ptr<int>(), seg_offsets.data_ptr<int>(), row_map.data_ptr<int>(), idx.numel(),
                               static_cast<int>(seg_offsets.numel() - 1), cur_stream()), "moe_rank");
}

void moe_capacity_mask(const Tensor& weights, const Tensor& idx, const Tensor& probs, const Tensor& counts, Tensor keep,
                       Tensor out, int64_t capacity) {
  check_f32(weights, "weights"); check_i32(idx, "idx"); check_f32(probs, "probs"); check_i32(counts, "counts");
  check_f32(out, "out");
  TORCH_CHECK(keep.is_cuda() && keep.scalar_type() == at::kByte && keep.numel() == idx.numel(), "moe_capacity_mask: keep uint8 [T,k]");
  TORCH_CHECK(weights.is_contiguous() && idx.is_contiguous() && probs.is_contiguous() && out.is_contiguous() &&
              weights.sizes() == idx.sizes() && out.sizes() == idx.sizes() && probs.size(0) == idx.size(0) &&
              probs.size(1) == counts.numel(), "moe_capacity_mask: weights/idx/out [T,k], probs [T,E], counts [E]");
  const c10::cuda::CUDAGuard guard(idx.device());
  check_rc(yv::launch_moe_capacity_mask(weights.data_ptr<float>(), idx.data_ptr<int>(), probs.data_ptr<float>(),
                                        counts.data_ptr<int>(), keep.data_ptr<uint8_t>(), out.data_ptr<float>(), idx.size(0),
                                        static_cast<int>(idx.size(1)), static_cast<int>(counts.numel()),
                                        static_cast<int>(capacity), cur_stream()), "moe_capacity_mask");
}

void moe_permute(const Tensor& x, const Tensor& idx, const c10::optional<Tensor>& cursor, Tensor row_map, Tensor xp) {
  check_bf16(x, "x"); check_i32(idx, "idx"); check_i32(row_map, "row_map"); check_bf16(xp, "xp");
  TORCH_CHECK(x.is_contiguous() && xp.is_contiguous(), "moe_permute: contiguous expected");
  const int cols = static_cast<int>(x.size(-1));
  const int k = static_cast<int>(idx.size(-1));
  const c10::cuda::CUDAGuard guard(x.device());
  check_rc(yv::launch_moe_permute(x.data_ptr(), idx.data_ptr<int>(),
                                  cursor.has_value() ? cursor->data_ptr<int>() : nullptr, row_map.data_ptr<int>(),
                                  xp.data_ptr(), x.numel() / cols, k, cols, cur_stream()),
           "moe_permute");
}

void moe_zero_pad(Tensor xp, const Tensor& seg_offsets, const Tensor& counts) {
  check_bf16(xp, "xp"); check_i32(seg_offsets, "seg_offsets"); check_i32(counts, "counts");
  const c10::cuda::CUDAGuard guard(xp.device());
  check_rc(yv::launch_moe_zero_pad(xp.data_ptr(), seg_offsets.data_ptr<int>(), counts.data_ptr<int>(),
                                   static_cast<int>(counts.numel()), static_cast<int>(xp.size(-1)), cur_stream()),
           "moe_zero_pad");
}

void moe_combine(const Tensor& y, const Tensor& row_map, const Tensor& weights, const c10::optional<Tensor>& addt,
                 Tensor out) {
  check_bf16(y, "y"); check_i32(row_map, "row_map"); check_f32(weights, "weights"); check_bf16(out, "out");
  const int cols = static_cast<int>(out.size(-1));
  const int k = static_cast<int>(weights.size(-1));
  const c10::cuda::CUDAGuard guard(y.device());
  check_rc(yv::launch_moe_combine(y.data_ptr(), row_map.data_ptr<int>(), weights.data_ptr<float>(), optp(addt),
                                  out.data_ptr(), out.numel() / cols, k, cols, cur_stream()),
           "moe_combine");
}

void moe_combine_bwd(const Tensor& dout, const Tensor& y, const Tensor& row_map, const Tensor& weights, Tensor dy,
                     Tensor dweights) {
  check_bf16(dout, "dout"); check_bf16(y, "y"); check_bf16(dy, "dy"); check_f32(dweights, "dweights");
  const int cols = static_cast<int>(dout.size(-1));
  const int k = static_cast<int>(weights.size(-1));
  const c10::cuda::CUDAGuard guard(y.device());
  check_rc(yv::launch_moe_combine_bwd(dout.data_ptr(), y.data_ptr(), row_map.data_ptr<int>(),
                                      weights.data_ptr<float>(), dy.data_ptr(), dweights.data_ptr<float>(),
                                      dout.numel() / cols, k, cols, cur_stream()),
           "moe_combine_bwd");
}

void moe_unpermute_sum(const Tensor& dxp, const Tensor& row_map, Tensor dx, int64_t k) {
  check_bf16(dxp, "dxp"); check_i32(row_map, "row_map"); check_bf16(dx, "dx");
  const int cols = static_cast<int>(dx.size(-1));
  const c10::cuda::CUDAGuard guard(dx.device());
  check_rc(yv::launch_moe_unpermute_sum(dxp.data_ptr(), row_map.data_ptr<int>(), dx.data_ptr(), dx.numel() / cols,
                                        static_cast<int>(k), cols, cur_stream()),
           "moe_unpermute_sum");
}

void gate_bias_update(Tensor bias, const Tensor& counts, double rate, double clampv) {
  check_f32(bias, "bias"); check_i32(counts, "counts");
  const c10::cuda::CUDAGuard guard(bias.device());
  check_rc(yv::launch_gate_bias_update(bias.data_ptr<float>(), counts.data_ptr<int>(), static_cast<int>(bias.numel()),
                                       static_cast<float>(rate), static_cast<float>(clampv), cur_stream()),
           "gate_bias_update");
}

}  // namespace

#include "binding_part2.inc"
