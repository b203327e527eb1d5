// Routing planner for sm_100a, host entry points.  No host synchronisation anywhere.
//
//   plan_publish   every rank pushes its tokens-per-expert row into all peers' meta chunks,
//                  resets its own src_info region, counts the experts of every block of its routing and
//                  signals FLAG_TPE (this signal also tells the peers that the rank is done with every
//                  earlier use of the buffers).
//   plan_compute   the table stage (one CTA) and the token stage (planner.cuh) as two roles of the dispatch
//                  kernel in one launch; signals FLAG_PLAN.  A fused dispatch runs the same two roles inside
//                  its own launch instead (dispatch.cu).
//
// Parity: replaces the reference's host-driven planner (moonep_td/_planning_gpu.py:86-592:
// 5 small kernels, dozens of torch ops, ~6+7R host synchronisations per plan).
#include <climits>

#include "common.cuh"
#include "host.h"
#include "planner.cuh"

namespace moonep {

namespace {

constexpr int kTokensThreads = 512;

// One CTA per planner block of whole tokens.  Besides the exchange, each CTA counts the experts
// of its block (block_hist[block][e]); plan_tokens turns these into in-order indices.
__global__ void __launch_bounds__(kTokensThreads)
    plan_publish_kernel(const MoonepDevCtx c, const int* __restrict__ topk, const int* __restrict__ tpe, int tpe_is_2d,
                        int tokens_per_block, int epoch_tpe) {
  extern __shared__ int s_hist[];  // [E]
  griddep_launch();  // the dispatch kernel behind this one may set itself up meanwhile
  const bool live = !poisoned(c);
  if (live) {
    const int tid = blockIdx.x * blockDim.x + threadIdx.x;
    const int nth = gridDim.x * blockDim.x;
    int* src_info = c.meta_peer[c.rank] + c.src_info_off;
    for (int i = tid; i < c.NvS; i += nth) src_info[i] = -1;
    if (!tpe_is_2d) {
      const int total = c.R * c.E;
      for (int i = tid; i < total; i += nth) {
        const int d = i / c.E;
        const int e = i - d * c.E;
        c.meta_peer[d][c.tpe_off + c.rank * c.E + e] = tpe[e];
      }
    }
    const int E = c.E;
    for (int e = threadIdx.x; e < E; e += blockDim.x) s_hist[e] = 0;
    __syncthreads();
    const int start = blockIdx.x * tokens_per_block * c.K;
    const int end = min(c.N, start + tokens_per_block * c.K);
    for (int i = start + threadIdx.x; i < end; i += blockDim.x) {
      const int e = topk[i];
      if (e >= 0 && e < E) atomicAdd(s_hist + e, 1);
    }
    __syncthreads();
    int* out = c.block_hist + (long long)blockIdx.x * E;
    for (int e = threadIdx.x; e < E; e += blockDim.x) out[e] = s_hist[e];
  }
  grid_tail_signal(c, MOONEP_K_PLAN_PUBLISH, live ? MOONEP_FLAG_TPE : -1, epoch_tpe);
}

}  // namespace

}  // namespace moonep

using namespace moonep;

extern "C" long long moonep_planner_table_words(int R, int E, int B) {
  (void)B;
  return table_words(R, E);
}

static int hist_smem_ok(HostCtx* h, const void* kernel, size_t smem, const char* what) {
  if (smem <= 48 * 1024) return 0;
  if ((int)smem + 8192 > h->max_smem_optin) {
    set_error(std::string(what) + ": E too large for the shared-memory histogram");
    return 1;
  }
  return check_cuda(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), what);
}

extern "C" int moonep_plan_publish(void* ctx, const int* topk, const int* tpe, int tpe_is_2d, int epoch_tpe,
                                   void* stream) {
  auto* h = (HostCtx*)ctx;
  const MoonepDevCtx& c = h->dev;
  const int tpb = imax(1, MOONEP_PLAN_BLOCK / c.K);
  const int grid = (c.S + tpb - 1) / tpb;
  const size_t smem = (size_t)c.E * sizeof(int);
  if (int rc = hist_smem_ok(h, (const void*)plan_publish_kernel, smem, "plan_publish_kernel")) return rc;
  plan_publish_kernel<<<grid, kTokensThreads, smem, (cudaStream_t)stream>>>(c, topk, tpe, tpe_is_2d, tpb, epoch_tpe);
  return check_launch("plan_publish_kernel");
}

extern "C" int moonep_plan_compute(void* ctx, const int* topk, const int* tpe2d, int* dst, int* cu_seqlens,
                                   int* experts_to_copy, int* zero_fill, int* remote_stats, int* dup_counts,
                                   int wait_epoch_tpe, int signal_epoch_plan, void* stream) {
  auto* h = (HostCtx*)ctx;
  return moonep_dispatch(ctx, MOONEP_ROLE_TABLES | MOONEP_ROLE_TOKENS, 1, topk, tpe2d, dst, cu_seqlens, experts_to_copy,
                         zero_fill, remote_stats, nullptr, nullptr, 0, nullptr, nullptr, dup_counts, nullptr, nullptr, -1,
                         0, wait_epoch_tpe, signal_epoch_plan, 0, MOONEP_PATH_LDST, imin(h->dev.local_sms, h->sm_count), 0,
                         0, nullptr, stream);
}
