// Allocation-free entry point.  This has no counterpart in the reference implementation (which is pure
// Python and lets PyTorch allocate everything); it exists for hosts that embed these kernels but must not
// allocate device memory themselves at call time: a serving loop whose memory pool is sized and frozen at
// start-up, or a plugin that is only handed pre-allocated tensors by its host application and has no allocator
// of its own.
//
//   int bf_edge_attn_fwd_noalloc(const bf_attn_params* p, cudaStream_t stream);
//
// Same computation as bf_edge_attn_fwd (edge attention forward, including queries with more than
// BF_HUB_DEGREE in-edges), with one difference: the fp32 scratch that the long-row ("hub") kernels accumulate
// into is not supplied by the caller (`p->hub_scratch` is ignored) but lives in a fixed `static __device__` array
// inside the library.  The caller still passes every input and output, including `hub_rows` / `n_hub` /
// `max_hub_degree`.
//
// Limits (rejected with BF_NOALLOC_ERR_TOO_LARGE, nothing is launched):
//   p->n_hub            <= BF_NOALLOC_MAX_HUBS
//   p->hl * p->hn       <= BF_NOALLOC_MAX_WIDTH   (and p->hl <= BF_NOALLOC_MAX_HEADS)
// Arguments the kernels cannot take (an unsupported dtype or head size, n_hub > 0 without hub_rows or without
// max_hub_degree) return cudaErrorInvalidValue, also before anything is queued on the stream.
// The array occupies BF_NOALLOC_SCRATCH_BYTES (about 272 KiB) on every GPU that loads the library, until the
// process exits.
//
// Behaviour to know about:
//   * The first call on a device looks up the array's device address (cudaGetSymbolAddress) and caches it;
//     make that first call outside any stream capture.  Later calls only enqueue work.
//   * No cudaMalloc / cudaFree / allocating library routine is called, on any path.
//   * All calls share the one array, and it still holds the previous call's partial sums: every call clears the
//     part it will use (an asynchronous memset on `stream`) before launching.  Two calls that can overlap on the
//     GPU (different streams without an ordering between them) race on the array; serialise them.
#pragma once
#include "bf_kernels.h"

#ifdef __cplusplus
extern "C" {
#endif

#define BF_NOALLOC_MAX_HUBS 64
#define BF_NOALLOC_MAX_WIDTH 1024
#define BF_NOALLOC_MAX_HEADS 64
#define BF_NOALLOC_SCRATCH_FLOATS (BF_NOALLOC_MAX_HUBS * (BF_NOALLOC_MAX_WIDTH + BF_NOALLOC_MAX_HEADS))
#define BF_NOALLOC_SCRATCH_BYTES (BF_NOALLOC_SCRATCH_FLOATS * 4)

#define BF_NOALLOC_ERR_TOO_LARGE (-101)   // n_hub or row width beyond the fixed scratch
#define BF_NOALLOC_ERR_SETUP (-102)       // the array's device address could not be obtained

// Returns 0 on success, one of the codes above, or a cudaError_t value (> 0) from the launch.
int bf_edge_attn_fwd_noalloc(const bf_attn_params* p, cudaStream_t stream);

// Human-readable text for a return value of bf_edge_attn_fwd_noalloc.
const char* bf_noalloc_strerror(int code);

// sizeof(bf_attn_params) as this library was compiled: a caller that mirrors the struct by hand (ctypes, another
// language's FFI) can check its own layout against it before the first call.
size_t bf_attn_params_size(void);

#ifdef __cplusplus
}
#endif
