// Allocation-free paged-KV decode: the split-KV scratch of the decode kernels lives in a file-scope device
// array instead of caller-provided tensors.  See noalloc.h for the contract.
#include <cuda_runtime.h>
#include <mutex>
#include <stdio.h>

#include "noalloc.h"
#include "yv_ops.h"

namespace {

// Scratch for the per-split partial results: first the partial outputs [batch, hq, splits, d], then the
// partial (max, sum) pairs [batch, hq, splits, 2].  In host code this name is only a handle for
// cudaGetSymbolAddress; the device address is looked up once per device below.
static __device__ __align__(256) float g_decode_scratch[YV_NOALLOC_SCRATCH_FLOATS];

// Status word of this entry point (bit mask, see yv_noalloc_status); the kernels set bits with atomicOr.
static __device__ uint32_t g_decode_status;

constexpr int kMaxDevices = 64;
float* g_scratch_ptr[kMaxDevices] = {nullptr};
uint32_t* g_status_ptr[kMaxDevices] = {nullptr};
std::mutex g_setup_mutex;

// Device address of the scratch array on the current device (resolved on first use per device).
int scratch_for_current_device(float** out, uint32_t** status_out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) return YV_NOALLOC_SETUP_FAILED;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_scratch_ptr[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_decode_scratch);
    if (e != cudaSuccess || p == nullptr) {
      fprintf(stderr, "pisceslx_b200: cudaGetSymbolAddress(decode scratch) failed on device %d: %s\n", dev,
              cudaGetErrorString(e));
      return YV_NOALLOC_SETUP_FAILED;
    }
    uint32_t* st = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&st), g_decode_status);
    if (e != cudaSuccess || st == nullptr) {
      fprintf(stderr, "pisceslx_b200: cudaGetSymbolAddress(decode status) failed on device %d: %s\n", dev,
              cudaGetErrorString(e));
      return YV_NOALLOC_SETUP_FAILED;
    }
    g_status_ptr[dev] = st;
    g_scratch_ptr[dev] = p;
  }
  *out = g_scratch_ptr[dev];
  *status_out = g_status_ptr[dev];
  return YV_NOALLOC_OK;
}

}  // namespace

extern "C" int yv_paged_decode_noalloc(const void* q, const void* k_cache, const void* v_cache,
                                       const int32_t* block_table, const int32_t* seq_lens, void* o, int batch,
                                       int hq, int hk, int d, int block, int max_blocks_per_seq, int num_blocks,
                                       int splits, float scale, void* stream) {
  if (q == nullptr || k_cache == nullptr || v_cache == nullptr || block_table == nullptr || seq_lens == nullptr ||
      o == nullptr)
    return YV_NOALLOC_BAD_ARGUMENT;
  if (batch <= 0 || hq <= 0 || hk <= 0 || splits < 1 || (d != 64 && d != 128) || hq % hk != 0 || block <= 0 ||
      max_blocks_per_seq <= 0 || num_blocks <= 0)
    return YV_NOALLOC_BAD_ARGUMENT;
  const int g = hq / hk;
  if (g != 1 && g != 2 && g != 4 && g != 8) return YV_NOALLOC_BAD_ARGUMENT;
  const long long need_o = static_cast<long long>(batch) * hq * splits * d;
  const long long need_ml = static_cast<long long>(batch) * hq * splits * 2;
  if (need_o + need_ml > static_cast<long long>(YV_NOALLOC_SCRATCH_FLOATS)) {
    fprintf(stderr,
            "pisceslx_b200: yv_paged_decode_noalloc needs %lld scratch floats (batch %d x heads %d x splits %d x "
            "(d %d + 2)) but the built-in scratch holds %d; lower splits or batch, or use the regular entry point\n",
            need_o + need_ml, batch, hq, splits, d, YV_NOALLOC_SCRATCH_FLOATS);
    return YV_NOALLOC_TOO_LARGE;
  }
  float* scratch = nullptr;
  uint32_t* status = nullptr;
  const int rc = scratch_for_current_device(&scratch, &status);
  if (rc != YV_NOALLOC_OK) return rc;

  yv::PagedDecodeArgs a;
  a.q = q; a.k_cache = k_cache; a.v_cache = v_cache;
  a.block_table = block_table; a.seq_lens = seq_lens;
  a.o = o;
  a.partial_o = scratch;
  a.partial_ml = scratch + need_o;
  a.batch = batch; a.hq = hq; a.hk = hk; a.d = d; a.block = block;
  a.max_blocks_per_seq = max_blocks_per_seq; a.splits = splits; a.num_blocks = num_blocks;
  a.scale = scale;
  a.status = status;
  const int lrc = yv::launch_paged_decode(a, reinterpret_cast<cudaStream_t>(stream));
  return lrc < 0 ? YV_NOALLOC_LAUNCHER_BASE + lrc : lrc;
}

extern "C" int yv_noalloc_status(int reset, void* stream) {
  float* scratch = nullptr;
  uint32_t* status = nullptr;
  if (scratch_for_current_device(&scratch, &status) != YV_NOALLOC_OK) return YV_NOALLOC_SETUP_FAILED;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  uint32_t bits = 0;
  if (cudaMemcpyAsync(&bits, status, sizeof(bits), cudaMemcpyDeviceToHost, s) != cudaSuccess) return YV_NOALLOC_SETUP_FAILED;
  if (cudaStreamSynchronize(s) != cudaSuccess) return YV_NOALLOC_SETUP_FAILED;
  if (reset && bits != 0 && cudaMemsetAsync(status, 0, sizeof(bits), s) != cudaSuccess) return YV_NOALLOC_SETUP_FAILED;
  return static_cast<int>(bits);
}

extern "C" const char* yv_noalloc_strerror(int code) {
  switch (code) {
    case YV_NOALLOC_OK: return "ok";
    case YV_NOALLOC_TOO_LARGE: return "problem exceeds the built-in scratch capacity";
    case YV_NOALLOC_BAD_ARGUMENT: return "unsupported shape or null pointer";
    case YV_NOALLOC_SETUP_FAILED: return "could not resolve the scratch array on this device";
    default:
      if (code > 0) return cudaGetErrorString(static_cast<cudaError_t>(code));
      if (code <= YV_NOALLOC_LAUNCHER_BASE + (-1) && code > 2 * YV_NOALLOC_LAUNCHER_BASE)
        return "the kernel launcher rejected the problem (code - YV_NOALLOC_LAUNCHER_BASE is its own code)";
      return "unknown";
  }
}
