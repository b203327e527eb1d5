// moonep_b200 native library: C API and the device-side context.
//
// One shared object (libmoonep_b200.so) built for sm_100a holds every kernel of the
// library plus the CUDA-VMM symmetric allocator.  Python talks to it through ctypes:
// plain C functions, raw device pointers, a cudaStream_t.  No function here allocates
// device memory except moonep_ctx_create / the VMM calls; operations only launch
// kernels on the stream they are given and never synchronise with the host.
//
// Parity: the kernels replace the reference's Triton kernels K1-K17
// (moonep_td/_common.py, _planning_gpu.py, _dedup_builder.py, dispatch.py,
// dispatch_epilogue.py, combine_prologue.py, combine.py, prefetch.py, grad_reduce.py);
// the allocator replaces its NVSHMEM heap (moonep_td/buffer.py:86-109).
#pragma once

#include <cstdint>

#define MOONEP_VERSION 1

// Packed encodings (must match moonep_b200/constants.py).
#define MOONEP_KIDX_BITS 7
#define MOONEP_NVS_BITS 24
#define MOONEP_NVS_MASK ((1 << MOONEP_NVS_BITS) - 1)
#define MOONEP_MAX_TOPK 32
#define MOONEP_MAX_RANKS 128

// Flag families (one int32 per source rank and family in every meta chunk).
#define MOONEP_FLAG_READY 0
#define MOONEP_FLAG_TPE 1
#define MOONEP_FLAG_PLAN 2
#define MOONEP_FLAG_SENT 3
#define MOONEP_FLAG_COMB 4
#define MOONEP_FLAG_GRAD_READY 5
#define MOONEP_FLAG_GRAD_DONE 6
#define MOONEP_NUM_FLAG_FAMILIES 8

// Status block (int32 words, device memory, zero = healthy).
#define MOONEP_ST_CODE 0      // 0 ok, 1 wait timed out, 2 index out of range
#define MOONEP_ST_KERNEL 1    // id of the kernel that recorded it
#define MOONEP_ST_FAMILY 2    // flag family waited on / kind of index
#define MOONEP_ST_PEER 3      // rank waited on / offending value
#define MOONEP_ST_EXPECT 4    // epoch expected
#define MOONEP_ST_SEEN 5      // value seen
#define MOONEP_ST_WORDS 8

#define MOONEP_STATUS_OK 0
#define MOONEP_STATUS_TIMEOUT 1
#define MOONEP_STATUS_BAD_INDEX 2

// Kernel ids for the status block.
#define MOONEP_K_SIGNAL 1
#define MOONEP_K_PLAN_PUBLISH 2
#define MOONEP_K_PLAN_TABLES 3
#define MOONEP_K_PLAN_TOKENS 4
#define MOONEP_K_DISPATCH_SEND 5
#define MOONEP_K_DISPATCH_EXPAND 6
#define MOONEP_K_COMBINE_PROLOGUE 7
#define MOONEP_K_COMBINE_PULL 8
#define MOONEP_K_PREFETCH 9
#define MOONEP_K_GRAD_ACCUM 10
#define MOONEP_K_GRAD_CLEAR 11
#define MOONEP_K_WAIT 12
#define MOONEP_NUM_KERNEL_IDS 16
// stats[MOONEP_STAT_WAIT_MAX_NS + family]: longest time CTA 0 of any kernel spun on a flag of that family (ns);
// stats[MOONEP_STAT_WAIT_COUNT + family]: number of such waits that did not find the flag already set.
#define MOONEP_STAT_WAIT_MAX_NS 0
#define MOONEP_STAT_WAIT_COUNT 8
// counters[MOONEP_BIAS_OFF + family]: epoch bias added to every epoch argument of that family.
#define MOONEP_BIAS_OFF 32

// link word of a landed row (pushed by the source rank during planning).
#define MOONEP_LINK_PRIMARY (1 << 30)
#define MOONEP_LINK_HAS_NEXT (1 << 29)

// Routing entries per planner block (whole tokens, at most this many entries).
#define MOONEP_PLAN_BLOCK 512

// Copy paths of dispatch/combine/prefetch.
#define MOONEP_PATH_LDST 0  // 16-byte loads/stores from registers
#define MOONEP_PATH_BULK 1  // cp.async.bulk through shared memory (mbarrier pipeline)

// Everything a kernel needs to know about one Buffer; passed by value.
struct MoonepDevCtx {
  int rank, R, E, S, K, H, B, N;
  int NvS, epn, token_padding, num_sms;
  long long nvs_padded;   // rows per hidden chunk
  long long meta_stride;  // int32 words per meta chunk
  int weights_off, tpe_off, plan_off, src_info_off, sync_off, r32;
  int link_off;   // [NvS] per landed row: LINK_PRIMARY | LINK_HAS_NEXT | next row of the same (source, token)
  int local_sms;  // CTAs used by kernels that only touch local memory
  int debug;
  int pad0;
  unsigned long long timeout_ns;
  // Peer tables: base address of every rank's chunk as seen from this GPU.
  uint16_t* const* hidden_peer;  // [R] -> bf16 [nvs_padded, H]
  int* const* meta_peer;         // [R] -> int32 [meta_stride]
  // Local scratch.
  int* status;        // [MOONEP_ST_WORDS]
  int* counters;      // [64] arrival counters of kernel tails, work counters, epoch biases
  int* alloc_cum;     // [E, R]   inclusive cumsum of alloc over destination ranks
  int* expert_off;    // [R, E]   first row of expert e on destination d
  int* tpe_prev;      // [E]      tokens of expert e on source ranks < rank
  int* tables;        // planner work area, see planner.cu
  int* block_hist;    // [planner blocks, E] per-block expert histograms of the local routing
  int* primary_packed;  // [R*S]
  int* kmask;           // [R*S]
  int* kidx_to_loff;    // [R*S*K]
  long long* stats;     // [16] flag-wait statistics, see MOONEP_STAT_*
};

#ifdef __cplusplus
extern "C" {
#endif

int moonep_version(void);
const char* moonep_last_error(void);
int moonep_sizeof_devctx(void);
// Number of kernels this library has launched in the calling process.
long long moonep_launch_count(void);
// Number of int32 words of planner work area needed for (R, E, B).
long long moonep_planner_table_words(int R, int E, int B);

// ctx: params is an int64 array in the order of MoonepDevCtx's integer fields (see runtime.cu),
// followed by the scratch pointers.  Returns an opaque handle or null.
void* moonep_ctx_create(const long long* params, int nparams, const unsigned long long* hidden_peers,
                        const unsigned long long* meta_peers);
void moonep_ctx_destroy(void* ctx);
int moonep_ctx_set_timeout_ms(void* ctx, long long ms);

// Cross-rank flags.  signal: store `epoch` into flag[family][rank] of every peer.
// wait: spin (bounded) until every peer's flag[wait_family] >= wait_epoch.  Either part
// may be skipped by passing family < 0.
int moonep_signal_wait(void* ctx, int signal_family, int signal_epoch, int wait_family, int wait_epoch,
                       void* stream);

// Epoch bias (graph replay support).  Kernels add bias[family] to their epoch arguments.
// mode 0: bias[f] = values[f]; mode 1: bias[f] += values[f], for f < MOONEP_NUM_FLAG_FAMILIES.
// values is a host array read at call time.  Captured as the last node of a CUDA graph with
// mode 1 and the epochs one replay consumes, it makes that graph replayable.
int moonep_epoch_bias(void* ctx, const int* values, int mode, void* stream);

// Planner.  tpe is [E] (pushed to all peers) or [R, E] (tpe_is_2d, used as is).
int moonep_plan_publish(void* ctx, const int* topk, const int* tpe, int tpe_is_2d, int epoch_tpe, void* stream);
int moonep_plan_compute(void* ctx, const int* topk, const int* tpe2d, int* dst, int* cu_seqlens,
                        int* experts_to_copy, int* zero_fill, int* remote_stats, int wait_epoch_tpe,
                        int signal_epoch_plan, void* stream);

// Dispatch.
int moonep_dispatch_send(void* ctx, const void* hidden, const float* weights, const int* dst,
                         const int* zero_fill, int* dup_groups, int* dup_loffs, int* dup_counts,
                         int build_dedup, int wait_family, int wait_epoch, int signal_epoch_sent, int path,
                         void* stream);
int moonep_dispatch_expand(void* ctx, const int* zero_fill, int with_weights, const int* dup_groups,
                           const int* dup_loffs, const int* dup_counts, int wait_epoch_sent, void* stream);

// Combine.
int moonep_combine_prologue(void* ctx, const int* dup_groups, const int* dup_loffs, const int* dup_counts,
                            const void* in_hidden, const float* in_weights, int wait_family, int wait_epoch,
                            int signal_epoch_comb, void* stream);
int moonep_combine_pull(void* ctx, const int* dst, void* out_hidden, float* out_weights, int wait_epoch_comb,
                        int path, void* stream);

// Expert weights: src[i] is [nexperts, H, Hp] bf16 (peer mapped), dst[i] is [nslots, H, Hp] bf16 (local).
int moonep_prefetch(void* ctx, void* const* src3, void* const* dst3, int n_tensors, const int* experts_to_copy_row,
                    long long elems, int nslots, int nexperts, int path, void* stream);
// grads[i]: [E, H, Hp] fp32 (local), reduce[i]: [R, B, H, Hp] fp32 (slot (src, b) lives on rank src).
int moonep_grad_reduce(void* ctx, float* const* grads, float* const* reduce, int n_tensors,
                       const int* experts_to_copy, int Bcols, long long elems, int epoch_ready, int epoch_done,
                       int phase, int path, void* stream);

// Expert computation (tcgen05 tensor cores).  None of these has a counterpart in the reference, which has no GEMM.
// y[rows of g] = x[rows of g] @ w[g]^T for the padded row groups of a dispatched shard; mode 0 plain, 1 SwiGLU
// (w0 = gate, w1 = up; pre_gate / pre_up optionally receive the two pre-activations), 2 scaled by row_scale.
// See grouped_gemm.cu.
int moonep_grouped_gemm(const void* x, const void* w0, const void* w1, void* out, const float* row_scale,
                        const int* cu_seqlens, int G, int rows_cap, int K, int n_per_group, int mode, int* status,
                        long long timeout_ms, int num_sms, const int* group_map, int w_slots, void* pre_gate,
                        void* pre_up, void* stream);
// The same operation on CTA pairs (tcgen05 cta_group::2, 256 x 256 tiles per cluster of two CTAs), see
// grouped_gemm_pair.cu.  Same arguments.
int moonep_grouped_gemm_pair(const void* x, const void* w0, const void* w1, void* out, const float* row_scale,
                             const int* cu_seqlens, int G, int rows_cap, int K, int n_per_group, int mode, int* status,
                             long long timeout_ms, int num_sms, const int* group_map, int w_slots, void* pre_gate,
                             void* pre_up, void* stream);
// y[rows of g] = x[rows of g] @ W[g] with W as [slots, K, N] (N contiguous) on CTA pairs; w1 (optional) continues
// the contraction: x = [a | b], W = [w0; w1].  This is the layout in which activation gradients need the forward
// weights, so no transposed copies are made.  K0, K1 multiples of 64, N a multiple of 256.
int moonep_grouped_gemm_pair_kn(const void* x, const void* w0, int K0, const void* w1, int K1, void* out,
                                const int* cu_seqlens, int G, int rows_cap, int N, int w_slots, int* status,
                                long long timeout_ms, int num_sms, void* stream);
// Host-side walk of the CTA-pair kernel's tile schedule, for tests (grouped_gemm_pair.cu).
int moonep_pair_schedule(const int* cu_seqlens, int G, int rows_cap, int n_tiles, int pair, int npairs, int* out,
                         int max_tiles);
// Weight gradients of all groups: out_ptrs[g][P, Q] fp32 (=, +=) L_g^T R_g with the contraction over the rows of
// group g.  lt = L^T [P, ld], rt = R^T [Q, ld] bf16 (ld a multiple of 8, >= rows_cap).  flags[g]: 0 store (zeros for
// an empty group), 1 accumulate, 2 store and leave empty groups alone.  out_ptrs, flags: device arrays [G].
int moonep_grouped_wgrad(const void* lt, const void* rt, long long ld, int P, int Q, const int* cu_seqlens, int G,
                         void* const* out_ptrs, const int* flags, int rows_cap, int* status, long long timeout_ms,
                         int num_sms, void* stream);
// The same from the operands as they are, l = L [rows, P], r = R [rows, Q] (rows ldl / ldr elements apart): no
// transposed copies, the tiles are staged MN-major.
int moonep_grouped_wgrad_rows(const void* l, long long ldl, const void* r, long long ldr, int rows, int P, int Q,
                              const int* cu_seqlens, int G, void* const* out_ptrs, const int* flags, int* status,
                              long long timeout_ms, int num_sms, void* stream);
// Helpers of the MoE layer's backward pass and optimiser step, see moe_kernels.cu.
int moonep_transpose_experts(const void* src, void* dst, int n, int d0, int d1, long long dst_ld,
                             long long dst_expert_stride, int col0, const int* active, void* stream);
int moonep_swiglu_bwd(const void* a, const void* u, const void* g, const float* w, const int* total_rows, int rows_cap,
                      int I, void* dadu, void* hsw, float* dgate, void* stream);
int moonep_sgd_update(void* w, const float* g, long long n, float lr, void* stream);

// CUDA VMM symmetric allocator (driver API through cudaGetDriverEntryPoint).
int moonep_vmm_granularity(int device, unsigned long long* gran);
int moonep_vmm_create(int device, unsigned long long bytes, unsigned long long* handle, int* fd);
int moonep_vmm_import(int fd, unsigned long long* handle);
int moonep_vmm_reserve(unsigned long long bytes, unsigned long long align, unsigned long long* va);
int moonep_vmm_map(unsigned long long va, unsigned long long bytes, unsigned long long handle, int device);
int moonep_vmm_unmap(unsigned long long va, unsigned long long bytes);
int moonep_vmm_release(unsigned long long handle);
int moonep_vmm_free_va(unsigned long long va, unsigned long long bytes);

#ifdef __cplusplus
}
#endif
