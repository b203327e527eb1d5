// Allocation-free entry point for the planner's table stage.
//
// This entry point has no counterpart in the reference library: it exists for callers that
// must not allocate device memory at the moment they need a routing plan's tables.  Typical
// cases are a serving thread that may not trigger the implicit device synchronisation of
// cudaMalloc/cudaFree, a process whose device memory is entirely owned by another allocator
// or pool, and code that runs between other people's kernels and must leave the allocator
// state untouched.  The normal path (Buffer.dispatch -> moonep_plan_compute) keeps its work
// area in buffers the Buffer allocated at construction; this variant keeps the work area in a
// fixed array inside the library image instead, so the caller only passes inputs and outputs.
//
// Limits: R <= MOONEP_NOALLOC_MAX_RANKS, E <= MOONEP_NOALLOC_MAX_EXPERTS (larger problems are
// rejected with an error, nothing is launched).  The work area is MOONEP_NOALLOC_SCRATCH_WORDS
// 32-bit words (208 KB) and is held by every GPU that loads the library until the
// process exits.
//
// The first call on a device looks up the device address of the work area
// (cudaGetSymbolAddress, no allocation) with that device current; make that first call
// before any stream capture.  All calls on one device share the single work area, which keeps
// whatever the previous call left in it: the kernel re-initialises every word it reads, but
// two calls that overlap on the GPU (different streams, or concurrent host threads) race
// on it.  Issue them on one stream, or order them with events.
//
// Neither this function nor anything it calls uses cudaMalloc, cudaFree, or an allocating
// library routine.
#pragma once

#define MOONEP_NOALLOC_MAX_RANKS 16
#define MOONEP_NOALLOC_MAX_EXPERTS 1024
#define MOONEP_NOALLOC_SCRATCH_WORDS 53248

#ifdef __cplusplus
extern "C" {
#endif

// tpe:              [R, E] int32 on the device: tokens of expert e that source rank r routes.
// cu_seqlens:       [E+B]   out, inclusive padded end of every group on `rank`.
// experts_to_copy:  [R, B]  out, global table of prefetched remote experts (-1 = empty slot).
// zero_fill:        [E+B,2] out, (first pad row, pad rows) per group on `rank`.
// remote_stats:     [2]     out, (#remote experts received by `rank`, #ranks copying its experts).
// S, K, token_padding, NvS as in the Buffer that will use the tables (capacity per rank = S*K).
// NvS is the number of rows the rank's shard can hold: when the padded groups of `rank` need more than that,
// the kernel stores -1 in remote_stats[0] and the other outputs must not be used (the Buffer's own planner
// records an index error in that case).
// Returns 0 on success; on failure moonep_last_error() explains.
int moonep_plan_tables_noalloc(const int* tpe, int R, int E, int B, int S, int K, int token_padding, int rank, int NvS,
                               int* cu_seqlens, int* experts_to_copy, int* zero_fill, int* remote_stats, void* stream);

#ifdef __cplusplus
}
#endif
