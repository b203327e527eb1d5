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
#define MOONEP_FLAG_PREFETCH 7  // no cross-rank flag: the epoch of prefetch_weight calls (per-slot flags are local)
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
// ids 13-15 are the GEMM kernels' (grouped_gemm, grouped_wgrad, grouped_gemm_pair); the ones below exceed
// MOONEP_NUM_KERNEL_IDS because they own no arrival counter named after them
#define MOONEP_K_COMBINE_PUSH 16
#define MOONEP_K_COMBINE_SUM 17
// counters[]: words 0..15 are arrival counters of kernel tails (indexed by kernel id), then:
#define MOONEP_CTR_SEND_WORK 16      // token hand-out of the send role
#define MOONEP_CTR_PULL_WORK 17      // token hand-out of combine_pull
#define MOONEP_CTR_TABLES_READY 18   // PLAN epoch of the last finished table stage (local release/acquire)
#define MOONEP_CTR_PLAN_DONE 19      // PLAN epoch of the last finished token stage
#define MOONEP_CTR_PLAN_ARRIVE 20    // CTAs that finished the token stage
#define MOONEP_CTR_SEND_ARRIVE 21    // CTAs that finished the send role
#define MOONEP_CTR_DISPATCH_ARRIVE 22  // CTAs of the dispatch kernel that reached its end
#define MOONEP_CTR_PUSH_WORK 23      // row hand-out of the combine push role
#define MOONEP_CTR_SUM_WORK 24       // token hand-out of the combine sum role
#define MOONEP_CTR_COMBINE_ARRIVE 25 // CTAs of the push-combine kernel that reached its end
#define MOONEP_CTR_PREFETCH_ARRIVE 26  // CTAs of the prefetch kernel that reached its end
#define MOONEP_CTR_FOLD_WORK 27      // group hand-out of the combine fold role
#define MOONEP_CTR_PUBLISH_ARRIVE 28 // CTAs of the dispatch kernel that finished the publish role
// stats[MOONEP_STAT_WAIT_MAX_NS + family]: longest time CTA 0 of any kernel spun on a flag of that family (ns);
// stats[MOONEP_STAT_WAIT_COUNT + family]: number of such waits that did not find the flag already set.
#define MOONEP_STAT_WAIT_MAX_NS 0
#define MOONEP_STAT_WAIT_COUNT 8
// stats[MOONEP_STAT_PHASE_NS + p]: longest time (ns, over the CTAs of a role, since the statistics were last reset) of
// phase p of the dispatch and combine kernels, stamped with %globaltimer:
#define MOONEP_STAT_PHASE_NS 16
#define MOONEP_PH_TABLES 0        // TABLES role: wait for the tokens-per-expert rows + table stage
#define MOONEP_PH_TOKENS 1        // TOKENS stage of one CTA (all its blocks)
#define MOONEP_PH_SEND 2          // SEND role: first token grabbed .. all copies of the CTA complete
#define MOONEP_PH_ZERO 3          // EXPAND role: zero fill
#define MOONEP_PH_WAIT_PLAN 4     // EXPAND role: wait for every peer's FLAG_PLAN
#define MOONEP_PH_BUILD_EXPAND 5  // EXPAND role: duplicate map + expansion (includes waiting for rows to land)
#define MOONEP_PH_WAIT_SENT 6     // EXPAND role: final wait for every peer's FLAG_SENT
#define MOONEP_PH_FOLD 7          // combine FOLD role
#define MOONEP_PH_PUSH 8          // combine PUSH role (a copy warp)
#define MOONEP_PH_SUM 9           // combine SUM role
#define MOONEP_STAT_WORDS 32
// counters[MOONEP_BIAS_OFF + family]: epoch bias added to every epoch argument of that family.
#define MOONEP_BIAS_OFF 32

// link word of a landed row (pushed by the source rank during planning).
#define MOONEP_LINK_PRIMARY (1 << 30)
#define MOONEP_LINK_HAS_NEXT (1 << 29)
// bits 24..28 of a primary row's link word: its position among the primaries of its token (ascending k)
#define MOONEP_LINK_ORD_SHIFT 24
#define MOONEP_LINK_ORD_MASK 31

// Roles of the dispatch kernel (bit mask); all of them in one launch is the fused dispatch.
#define MOONEP_ROLE_TABLES 1   // table stage of the planner (one CTA)
#define MOONEP_ROLE_TOKENS 2   // token stage of the planner
#define MOONEP_ROLE_SEND 4     // push rows, gate weights and row flags
#define MOONEP_ROLE_EXPAND 8   // zero fill, duplicate map, duplicate expansion as rows arrive
// Modifier, given to the SEND and the EXPAND launch alike (or to the one launch that has both roles): the rows whose
// token lives on this rank are written by EXPAND straight from the input (primary row and duplicates from one read),
// SEND leaves them out.  Needs src_info of the landed rows: a fresh plan, or a replayed plan that carries src_info.
#define MOONEP_ROLE_LOCAL_ROWS 16
// The launch begins with what plan_publish does as a kernel of its own (push of the tokens-per-expert row, reset of
// src_info, per-block expert counts, FLAG_TPE to every peer), spread over all CTAs of the launch.
#define MOONEP_ROLE_PUBLISH 32
// Roles of the push-combine kernel.
#define MOONEP_ROLE_PUSH 1     // expert side: copy primary rows (folded where they have duplicates) to the tokens' home ranks
#define MOONEP_ROLE_SUM 2      // home side: sum the rows of a token as they arrive
#define MOONEP_ROLE_FOLD 4     // expert side: fold the duplicate groups into a local buffer
// Modifier, given to every launch of one combine alike: rows whose token lives on this rank do not go through the
// PUSH role; the FOLD role writes them (folded, or as they are) straight into this rank's own staging chunk.
#define MOONEP_ROLE_LOCAL_HOME 8

// Routing entries per planner block (whole tokens, at most this many entries).
#define MOONEP_PLAN_BLOCK 512

// Copy paths of dispatch/combine/prefetch.
#define MOONEP_PATH_LDST 0  // 16-byte loads/stores from registers
#define MOONEP_PATH_BULK 1  // cp.async.bulk through shared memory (mbarrier pipeline)
#define MOONEP_PATH_ASYNC 2  // 16-byte cp.async into per-warp shared-memory rings (prefetch only)

// Everything a kernel needs to know about one Buffer; passed by value.
struct MoonepDevCtx {
  int rank, R, E, S, K, H, B, N;
  int NvS, epn, token_padding, num_sms;
  long long nvs_padded;   // rows per hidden chunk
  long long meta_stride;  // int32 words per meta chunk
  int weights_off, tpe_off, plan_off, src_info_off, sync_off, r32;
  int link_off;   // [NvS] per landed row: LINK_PRIMARY | LINK_HAS_NEXT | next row of the same (source, token)
  int local_sms;  // CTAs used by kernels that only touch local memory
  int rowflag_off;  // [NvS] per row: SENT epoch of the dispatch that last put data into it
  int kp;           // staging rows per token in the combine staging chunk: min(K, R)
  unsigned long long timeout_ns;
  // Combine staging (push path): chunk of rank r holds [S*kp, H] bf16 rows, then arrival flags, then gate weights.
  unsigned char* const* stage_peer;  // [R] or null when the Buffer has no staging memory
  long long stage_flag_off;          // byte offset of the [S*kp] int32 COMB epochs of the staged rows
  long long stage_w_off;             // byte offset of the [S*K] fp32 gate weights on their way home
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
  long long* stats;     // [MOONEP_STAT_WORDS] flag-wait and phase statistics, see MOONEP_STAT_*
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
                        const unsigned long long* meta_peers, const unsigned long long* stage_peers);
void moonep_ctx_destroy(void* ctx);
int moonep_ctx_set_timeout_ms(void* ctx, long long ms);
// Programmatic dependent launch for the dispatch and combine kernels of this context (off by default).
int moonep_ctx_set_pdl(void* ctx, int on);

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
                        int* experts_to_copy, int* zero_fill, int* remote_stats, int* dup_counts, int wait_epoch_tpe,
                        int signal_epoch_plan, void* stream);

// Dispatch: one launch of the dispatch kernel with the roles in `roles` (MOONEP_ROLE_*; see dispatch.cu).  With all four
// roles it is the fused fresh dispatch, with SEND | EXPAND the replay of a plan; single roles give the stages of the
// launch-level API.  fresh != 0: the planner arguments (topk .. remote_stats) are used and the duplicate map is built;
// plan_src_info / plan_link ([NvS] each, optional) receive the plan's copy of src_info and the link words.
// build_only: the EXPAND role only rebuilds the duplicate map.
int moonep_dispatch(void* ctx, int roles, int fresh, const int* topk, const int* tpe2d, int* dst, int* cu_seqlens,
                    int* experts_to_copy, int* zero_fill, int* remote_stats, const void* hidden, const float* weights,
                    int with_weights, int* dup_groups, int* dup_loffs, int* dup_counts, int* plan_src_info,
                    int* plan_link, int wait_family, int wait_epoch, int epoch_tpe, int epoch_plan, int epoch_sent,
                    int path, int n_send, int n_expand, int build_only, const int* tpe_row, void* stream);

// Combine.
int moonep_combine_prologue(void* ctx, const int* dup_groups, const int* dup_loffs, const int* dup_counts,
                            const void* in_hidden, const float* in_weights, int wait_family, int wait_epoch,
                            int signal_epoch_comb, void* stream);
int moonep_combine_pull(void* ctx, const int* dst, void* out_hidden, float* out_weights, int wait_epoch_comb,
                        int path, void* stream);
// Push combine (combine_push.cu): roles MOONEP_ROLE_FOLD | MOONEP_ROLE_PUSH | MOONEP_ROLE_SUM.  Needs the Buffer's staging
// memory (stage_peers of moonep_ctx_create, laid out by moonep_stage_layout), the plan's copies of src_info and link
// words, and local scratch for the folded rows.
long long moonep_stage_layout(int S, int K, int H, int kp, long long* flag_off, long long* w_off);
int moonep_combine_push(void* ctx, int roles, const int* src_info, const int* link, const int* dst, const void* in_rows,
                        const float* in_w, void* out_hidden, float* out_weights, int wait_family, int wait_epoch,
                        int epoch_comb, const int* ready, int ready_expect, const int* dup_groups, const int* dup_loffs,
                        const int* dup_counts, void* fold_buf, int* fold_flag, int fold_rows, int n_push, int n_local,
                        void* stream);

// Expert weights: src[i] is [nexperts, H, Hp] bf16 (peer mapped), dst[i] is [nslots, H, Hp] bf16 (local).
// slot_flags / slot_done ([nslots] int32 each, zero-initialised once, optional): slot b's flag receives the prefetch
// epoch when all tensors of the slot have been copied (or at once when the slot stays empty).
int moonep_prefetch(void* ctx, void* const* src3, void* const* dst3, int n_tensors, const int* experts_to_copy_row,
                    long long elems, int nslots, int nexperts, int path, int* slot_flags, int* slot_done, int epoch,
                    void* stream);
// grads[i]: [E, H, Hp] fp32 (local), reduce[i]: [R, B, H, Hp] fp32 (slot (src, b) lives on rank src).
int moonep_grad_reduce(void* ctx, float* const* grads, float* const* reduce, int n_tensors,
                       const int* experts_to_copy, int Bcols, long long elems, int epoch_ready, int epoch_done,
                       int phase, int path, void* stream);

// Hand-off between the communication kernels and the grouped GEMM on CTA pairs, tile by tile.  Every pointer may be
// null.  Epochs are compared as (value + *bias) when bias is given (graph replay, see moonep_epoch_bias).
//   row_flags    [rows] the dispatch kernel's per-row arrival flags: the TMA producer waits (bounded) until all 128
//                rows of a block carry row_epoch before it loads the block, so the GEMM can run beside the dispatch.
//   tables_ready one word the dispatch kernel's table stage publishes: cu_seqlens is read only after it reached
//                tables_epoch.
//   slot_flags   [G - slot_first_group] the prefetch kernel's per-slot flags: the weights of a group
//                g >= slot_first_group are loaded only after slot_flags[g - slot_first_group] reached slot_epoch.
//   done_counter [rows / 128] bumped by every epilogue warp after it stored its part of a tile of the block
//                (4 * column tiles per call and block), for a consumer that starts on finished row blocks
//                (moonep_combine_push: ready / ready_expect).
typedef struct MoonepGemmHooks {
  const int* row_flags;
  const int* row_bias;
  int row_epoch;
  int tables_epoch;
  const int* tables_ready;
  const int* tables_bias;
  const int* slot_flags;
  const int* slot_bias;
  int slot_epoch;
  int slot_first_group;
  int* done_counter;
} MoonepGemmHooks;

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
// moonep_grouped_gemm_pair with the hand-off hooks above (hooks may be null).
int moonep_grouped_gemm_pair_hooked(const void* x, const void* w0, const void* w1, void* out, const float* row_scale,
                                    const int* cu_seqlens, int G, int rows_cap, int K, int n_per_group, int mode,
                                    int* status, long long timeout_ms, int num_sms, const int* group_map, int w_slots,
                                    void* pre_gate, void* pre_up, const MoonepGemmHooks* hooks, void* stream);
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
