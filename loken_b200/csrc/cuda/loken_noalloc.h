// Split-KV decode attention for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference project; it exists for hosts that embed
// the library where every allocation is forbidden at call time: a real-time control loop whose
// memory budget is fixed at start-up, a plug-in running inside another program's CUDA context
// that owns the allocator, or a process whose device heap is locked down after initialisation.
// Such a caller cannot hand `lk_attn_decode` the partial-result workspace it needs when a long
// context is split over several blocks, and cannot let the library allocate one either.
//
// `lk_attn_decode_static` does the same computation as `lk_attn_decode` with the workspace taken
// from a fixed array that is part of the library's own device image.  It never calls
// cudaMalloc / cudaFree or any routine that allocates (no torch, no pools); the `ws`,
// `ws_floats`, `counters` and `n_counters` fields of the argument struct are ignored.
//
// Limits and rules
//   * The array holds LK_DECODE_STATIC_WS_FLOATS floats of partial results and
//     LK_DECODE_STATIC_COUNTERS arrival counters.  A call needs
//     lk_attn_decode_ws_floats(rows, n_q, n_kv, hd, nsplit) floats and rows * n_kv counters;
//     a call that needs more returns LKH_TOO_LARGE (-4) and launches nothing.  A call with
//     nsplit <= 1 uses neither and is never refused for its size.
//     lk_attn_decode_static_limits() reports both limits.
//   * The first call in each CUDA context looks up the array's address (cudaGetSymbolAddress, with
//     that context's device current) and remembers it for that context: the address is a
//     property of the context, so a plug-in called from several contexts on one device, or after
//     the host program reset the device, gets the array of the context it is called in.  Make
//     that first call during start-up, outside any stream capture; later calls in that context
//     only enqueue work on the given stream.  At most 64 contexts are remembered; beyond that
//     (or when the driver's context query is unavailable) the address is looked up on every call.
//   * Every call clears the counters it is about to use on the caller's stream before the
//     kernel runs, so a call that was abandoned half-way cannot poison the next one.
//   * All calls on a device share the one array.  Calls ordered on one stream are safe.  Two
//     calls that may overlap in time (different streams, no dependency between them) race on
//     the partial results and give wrong output; serialise them.
#pragma once
#include "loken_cuda.h"

#ifdef __cplusplus
extern "C" {
#endif

#define LK_DECODE_STATIC_WS_FLOATS (1 << 20)   /* 4 MiB of partial results */
#define LK_DECODE_STATIC_COUNTERS 4096

// Same contract as lk_attn_decode, except for the workspace fields (see above).
int lk_attn_decode_static(const LkDecodeArgs* args, void* stream);
// Writes the two limits; either pointer may be null.
void lk_attn_decode_static_limits(long long* ws_floats, int* counters);

#ifdef __cplusplus
}
#endif
