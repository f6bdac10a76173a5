// Allocation-free entry point for paged-KV decode attention.
//
// This entry point has no counterpart in the reference project: it exists for callers of this library that
// are not allowed to allocate device memory at the moment they need a decode step - a serving loop whose
// memory pool was sized up front and handed out completely, a step recorded after the process has frozen
// its allocator, or a host that drives the library from a language runtime without access to the PyTorch
// caching allocator.  The regular path (torch.ops.yv.paged_decode) asks its caller for two fp32 scratch
// tensors for the split-KV partial results; here that scratch lives in a fixed array inside the library.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// Capacity of the built-in scratch: batch * hq * splits * (d + 2) floats must not exceed this number.
// The array is part of the library image: every GPU that loads the library holds these 8.25 MiB until the
// process exits.
#define YV_NOALLOC_SCRATCH_FLOATS 2162688

// Error codes (0 = launched).
#define YV_NOALLOC_OK 0
#define YV_NOALLOC_TOO_LARGE -1      // the problem needs more scratch than YV_NOALLOC_SCRATCH_FLOATS
#define YV_NOALLOC_BAD_ARGUMENT -2   // unsupported head size / group size, null pointer, splits < 1
#define YV_NOALLOC_SETUP_FAILED -3   // the address of the scratch array could not be resolved on this device
// The kernel launcher rejected the problem after the checks above passed (for instance a tensor map that could not
// be encoded).  Its own negative code c is returned as YV_NOALLOC_LAUNCHER_BASE + c, so it cannot be mistaken for
// one of the three codes above.
#define YV_NOALLOC_LAUNCHER_BASE -1000
// positive values are cudaError_t codes from the launch

// One decode step over a paged KV cache, exactly the computation of the regular paged decode:
//   q [batch, hq, d] bf16, caches [num_blocks, block, hk, d] bf16, block_table [batch, max_blocks_per_seq] int32,
//   seq_lens [batch] int32, o [batch, hq, d] bf16 (written).  `stream` is a cudaStream_t (0 = default stream).
//
// Properties a caller can rely on:
//   * allocates and frees no device memory and calls no allocating library routine; inputs and outputs are the
//     caller's.  (The first call of a host thread binds the device's primary context with a null cudaFree, which
//     releases nothing; tensor maps are encoded on the host into kernel parameters.);
//   * the first call on each device resolves the device addresses of the scratch array and of the status word
//     (cudaGetSymbolAddress with that device current) and opts the kernels into their shared-memory size.  Make
//     that first call outside of any stream capture;
//   * every call uses the same scratch array.  Nothing in it has to start at zero: every slot that the merge
//     step reads is written earlier in the same call - also when a device-side wait runs out, in which case the
//     split is written as empty and the status word records the timeout.  The array keeps the last call's
//     partial results afterwards.  Two calls that overlap on the GPU (different streams, or different threads on
//     one device) race on it: serialise calls per device;
//   * sizes beyond the capacity are rejected with YV_NOALLOC_TOO_LARGE and nothing is launched;
//   * a sequence length beyond max_blocks_per_seq * block is cut to that capacity and reported in the status word,
//     as is a block-table entry outside [0, num_blocks).
int yv_paged_decode_noalloc(const void* q, const void* k_cache, const void* v_cache, const int32_t* block_table,
                            const int32_t* seq_lens, void* o, int batch, int hq, int hk, int d, int block,
                            int max_blocks_per_seq, int num_blocks, int splits, float scale, void* stream);

// Device-side conditions of the calls made so far on the current device, as a bit mask: 1 = a bounded wait ran out
// (the output of that call is incomplete), 8 = a sequence length or block-table entry was out of range (cut / skipped).
// 0 = none.  The kernels only ever set bits.  This call copies one word from the device and therefore waits for the
// work queued on `stream`; `reset` != 0 clears the word afterwards.  Returns a negative value (YV_NOALLOC_SETUP_FAILED)
// if the word could not be read.  Allocates nothing.
int yv_noalloc_status(int reset, void* stream);

// Human-readable text for the codes above (static storage).
const char* yv_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
