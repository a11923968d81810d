// Allocation-free C entry point for paged-KV decode attention.
//
// This entry point has no counterpart in the reference; it exists for callers of this library
// that are not allowed to allocate device memory at the moment they need attention: code that
// runs inside a fixed memory budget handed out at start-up (serving engines that pre-plan
// every byte of HBM, real-time control loops of a robot policy), code that runs on a thread
// which must never take the allocator's lock or trigger the implicit device synchronisation
// of cudaMalloc/cudaFree, and plain-C hosts that link this shared object without PyTorch and
// its caching allocator. They pass raw device pointers for inputs and outputs and get the same
// result as `torch.ops.cosmos_b200.paged_decode`.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

// Largest problem the built-in scratch area can hold: B * Hq * n_splits <= this many rows
// (each row is 130 floats: a 128-wide partial output plus its running max and sum), i.e. the
// library keeps 8192 * 130 * 4 B = 4.06 MiB of device memory per GPU for this purpose.
#define COSMOS_PAGED_DECODE_NOALLOC_MAX_ROWS 8192

// Error codes returned by cosmos_paged_decode_noalloc (0 = success).
#define COSMOS_NOALLOC_OK 0
#define COSMOS_NOALLOC_TOO_LARGE 1   // B * Hq * n_splits exceeds COSMOS_PAGED_DECODE_NOALLOC_MAX_ROWS
#define COSMOS_NOALLOC_BAD_ARGUMENT 2
#define COSMOS_NOALLOC_CUDA_ERROR 3

// Decode attention for one new token per sequence over a paged KV cache.
//   q [B, Hq, 128] bf16, k_cache / v_cache [pages, Hkv, page_size, 128] bf16 (contiguous),
//   block_table [B, max_pages] int32, seq_lens [B] int32, out [B, Hq, 128] bf16; all device
//   pointers on the current device. `stream` is a cudaStream_t (NULL = default stream).
//   `n_splits` in [1, 64] splits every sequence along kv across CTAs.
// The split partials live in a fixed device array inside the library, so the call performs no
// cudaMalloc/cudaFree and calls no allocating library routine.
//   * The first call on a device looks up that array's device address (cudaGetSymbolAddress)
//     and loads every kernel variant this entry point can launch (one per GQA group size 1, 2,
//     4, 8, plus the kernel that merges the splits), so that no later call has to load code
//     (with lazy module loading the first launch of a kernel may allocate). Make that first
//     call during start-up: outside of any stream capture and before the real-time phase.
//   * All calls on a device share the one array. Each call overwrites every slot it reads, so
//     nothing has to be cleared in between, but two calls that overlap on the GPU (different
//     streams) race on it: order them on one stream or with events.
//   * Problems with B * Hq * n_splits > COSMOS_PAGED_DECODE_NOALLOC_MAX_ROWS are rejected with
//     COSMOS_NOALLOC_TOO_LARGE; lower n_splits or use the allocating entry point.
//   * COSMOS_NOALLOC_CUDA_ERROR reports an error raised by this call's own launches. An error
//     that an earlier, unrelated call left pending on the thread is reported as such ("pending
//     CUDA error from an earlier call") before anything is launched, and is left for its owner
//     to clear.
// When `errbuf` is not NULL a human-readable message is written there on failure.
int cosmos_paged_decode_noalloc(const void* q, const void* k_cache, const void* v_cache,
                                const int* block_table, const int* seq_lens, void* out, int B, int Hq,
                                int Hkv, int page_size, int max_pages, float scale, int n_splits,
                                void* stream, char* errbuf, int errbuf_len);

#ifdef __cplusplus
}
#endif
