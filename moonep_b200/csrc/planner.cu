// Routing planner for sm_100a: three short kernels, no host synchronisation.
//
//   plan_publish   every rank pushes its tokens-per-expert row into all peers' meta chunks,
//                  resets its own src_info region and signals FLAG_TPE (this signal also
//                  tells the peers that the rank is done with every earlier use of the buffers).
//   plan_tables    one CTA: waits for all FLAG_TPE, then derives the tables that are identical
//                  on every rank (balance quotas, alloc[d][e], per-destination group layout,
//                  experts_to_copy, remote_stats, cu_seqlens, zero_fill, expert offsets).
//   plan_tokens    one CTA per block of whole tokens: in-order index of every routing entry
//                  among the entries of its expert, destination row, duplicate marking, and the
//                  push of src_info into the destination ranks' meta chunks; signals FLAG_PLAN.
//
// Results are exactly those of the host planner (moonep_b200/cpu/planner.py): first-index
// tie-breaking of argmax/argmin, quotas assigned (not accumulated), remote experts sorted by
// (count, expert) descending, remote_stats[0] uncapped.
//
// Parity: replaces the reference's host-driven planner (moonep_td/_planning_gpu.py:86-592:
// 5 small kernels, dozens of torch ops, ~6+7R host synchronisations per plan).
#include <climits>

#include "common.cuh"
#include "host.h"

namespace moonep {

namespace {

constexpr int kTablesThreads = 1024;
constexpr int kTokensThreads = 512;

struct Tables {
  int* expert_count;  // [E]
  int* remaining;     // [E]
  int* alloc;         // [R][E]
  int* z;             // [R][R]
  int* prank;         // [R][E]
  int* cand;          // [R][E]
  int* rs1;           // [R]
};

__host__ __device__ inline long long table_words(int R, int E) {
  return 2ll * E + 3ll * R * E + 1ll * R * R + 2ll * R;
}

__device__ inline Tables carve(int* base, int R, int E) {
  Tables t;
  t.expert_count = base;
  t.remaining = t.expert_count + E;
  t.alloc = t.remaining + E;
  t.z = t.alloc + (long long)R * E;
  t.prank = t.z + R * R;
  t.cand = t.prank + (long long)R * E;
  t.rs1 = t.cand + (long long)R * E;
  return t;
}

// Warp-wide argmax with first-index tie-breaking over v[0..n).
__device__ inline void warp_argmax_first(const int* v, int n, int lane, int& best, int& best_i) {
  best = INT_MIN;
  best_i = INT_MAX;
  for (int i = lane; i < n; i += 32) {
    const int x = v[i];
    if (x > best) {
      best = x;
      best_i = i;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const int ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (ov > best || (ov == best && oi < best_i)) {
      best = ov;
      best_i = oi;
    }
  }
}

__device__ inline void warp_argmin_first(const int* v, int n, int lane, int& best, int& best_i) {
  best = INT_MAX;
  best_i = INT_MAX;
  for (int i = lane; i < n; i += 32) {
    const int x = v[i];
    if (x < best) {
      best = x;
      best_i = i;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const int ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (ov < best || (ov == best && oi < best_i)) {
      best = ov;
      best_i = oi;
    }
  }
}

// One CTA per planner block of whole tokens.  Besides the exchange, each CTA counts the experts
// of its block (block_hist[block][e]); plan_tokens turns these into in-order indices.
__global__ void __launch_bounds__(kTokensThreads)
    plan_publish_kernel(const MoonepDevCtx c, const int* __restrict__ topk, const int* __restrict__ tpe, int tpe_is_2d,
                        int tokens_per_block, int epoch_tpe) {
  extern __shared__ int s_hist[];  // [E]
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

__global__ void __launch_bounds__(kTablesThreads)
    plan_tables_kernel(const MoonepDevCtx c, const int* __restrict__ tpe2d, int* __restrict__ cu_out,
                       int* __restrict__ etc_out, int* __restrict__ zf_out, int* __restrict__ rs_out, int wait_epoch,
                       int work_in_smem) {
  extern __shared__ int s_work[];  // the work tables, when they fit (the serial phases then run at shared-memory latency)
  if (!block_wait_flags(c, MOONEP_FLAG_TPE, wait_epoch, MOONEP_K_PLAN_TABLES)) return;
  const int R = c.R, E = c.E, B = c.B, epn = c.epn, P = c.token_padding;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
  const int* tpe = tpe2d ? tpe2d : (c.meta_peer[c.rank] + c.tpe_off);
  Tables t = carve(work_in_smem ? s_work : c.tables, R, E);
  __shared__ int s_balance[MOONEP_MAX_RANKS];
  __shared__ int s_bad;
  if (tid == 0) s_bad = 0;

  // 1. per-expert totals, prefix of the source ranks before this one, home allocation
  for (int e = tid; e < E; e += blockDim.x) {
    int cum = 0;
    for (int s = 0; s < R; ++s) {
      if (s == c.rank) c.tpe_prev[e] = cum;
      cum += tpe[s * E + e];
    }
    t.expert_count[e] = cum;
    t.remaining[e] = cum;
    const int home = e / epn;
    for (int d = 0; d < R; ++d) t.alloc[(long long)d * E + e] = (d == home) ? cum : 0;
  }
  for (int i = tid; i < R * R; i += blockDim.x) t.z[i] = 0;
  for (int i = tid; i < R; i += blockDim.x) t.rs1[i] = 0;
  __syncthreads();

  // 2. balance of every home group
  for (int h = warp; h < R; h += nwarps) {
    int sum = 0;
    for (int i = lane; i < epn; i += 32) sum += t.expert_count[h * epn + i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (lane == 0) s_balance[h] = sum - c.N;
  }
  __syncthreads();

  // 3. quotas z[h][u]: the most overloaded home fills the emptiest rank completely
  if (warp == 0) {
    for (int it = 0; it < 4 * R + 8; ++it) {
      int bh, h, bu, u;
      warp_argmax_first(s_balance, R, lane, bh, h);
      warp_argmin_first(s_balance, R, lane, bu, u);
      if (bh <= 0) break;
      const int move = -bu;
      if (lane == 0) {
        t.z[h * R + u] = move;
        s_balance[h] = bh - move;
        s_balance[u] = 0;
      }
      __syncwarp();
    }
  }
  __syncthreads();

  // 4. distribution: largest quota takes from the local expert with most tokens left
  for (int h = warp; h < R; h += nwarps) {
    int* q = t.z + h * R;
    int* rem = t.remaining + h * epn;
    for (int it = 0; it < epn + R + 8; ++it) {
      int quota, d, r, le;
      warp_argmax_first(q, R, lane, quota, d);
      if (quota <= 0) break;
      warp_argmax_first(rem, epn, lane, r, le);
      const int take = r < quota ? r : quota;
      if (take <= 0) break;
      if (lane == 0) {
        const int e = h * epn + le;
        t.alloc[(long long)d * E + e] += take;
        t.alloc[(long long)h * E + e] -= take;
        rem[le] = r - take;
        q[d] = quota - take;
      }
      __syncwarp();
    }
  }
  __syncthreads();

  // 5. per-expert inclusive cumsum over destinations (token phase searches it)
  for (int e = tid; e < E; e += blockDim.x) {
    int cum = 0;
    for (int d = 0; d < R; ++d) {
      cum += t.alloc[(long long)d * E + e];
      c.alloc_cum[(long long)e * R + d] = cum;
    }
  }

  // 6. group layout of every destination rank
  for (int d = warp; d < R; d += nwarps) {
    const int* al = t.alloc + (long long)d * E;
    int* prank = t.prank + (long long)d * E;
    int* cand = t.cand + (long long)d * E;
    int n = 0;
    for (int base = 0; base < E; base += 32) {
      const int e = base + lane;
      const int a = e < E ? al[e] : 0;
      const bool is_remote = e < E && a > 0 && (e / epn) != d;
      if (e < E) prank[e] = INT_MAX;
      const unsigned m = __ballot_sync(0xffffffffu, is_remote);
      if (is_remote) cand[n + __popc(m & ((1u << lane) - 1u))] = e;
      n += __popc(m);
    }
    __syncwarp();
    // order among the remote experts: (count, e) descending
    for (int i = lane; i < n; i += 32) {
      const int ei = cand[i], ci = al[ei];
      int pos = 0;
      for (int j = 0; j < n; ++j) {
        const int ej = cand[j], cj = al[ej];
        pos += (cj > ci || (cj == ci && ej > ei)) ? 1 : 0;
      }
      prank[ei] = pos;
      if (pos < B) {
        etc_out[d * B + pos] = ei;
        atomicAdd(t.rs1 + ei / epn, 1);
      }
    }
    for (int b = lane; b < B; b += 32)
      if (b >= n) etc_out[d * B + b] = -1;
    if (d == c.rank && lane == 0) rs_out[0] = n;
    __syncwarp();
    const int npick = n < B ? n : B;
    int carry = 0;
    for (int base = 0; base < E + B; base += 32) {
      const int g = base + lane;
      int cnt = 0, eid = -1;
      if (g < E) {
        if (prank[g] >= B) {
          eid = g;
          cnt = al[g];
        }
      } else if (g < E + B && g - E < npick) {
        eid = etc_out[d * B + (g - E)];
        cnt = al[eid];
      }
      const int padded = cnt > 0 ? ((cnt + P - 1) / P) * P : 0;
      int incl = padded;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
      }
      const int end_aligned = carry + incl;
      const int start = end_aligned - padded;
      if (g < E + B) {
        if (cnt > 0) c.expert_off[(long long)d * E + eid] = start;
        if (d == c.rank) {
          cu_out[g] = end_aligned;
          const bool pad = cnt > 0 && padded > cnt;
          zf_out[2 * g] = pad ? start + cnt : 0;
          zf_out[2 * g + 1] = pad ? padded - cnt : 0;
        }
      }
      carry += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0 && carry > c.NvS) s_bad = carry;
  }
  __syncthreads();
  if (tid == 0) {
    rs_out[1] = t.rs1[c.rank];
    if (s_bad) record_status(c, MOONEP_STATUS_BAD_INDEX, MOONEP_K_PLAN_TABLES, 1, s_bad, c.NvS, 0);
  }
}

__global__ void __launch_bounds__(kTokensThreads)
    plan_tokens_kernel(const MoonepDevCtx c, const int* __restrict__ topk, int* __restrict__ dst_out,
                       int tokens_per_block, int epoch_plan) {
  extern __shared__ int s_hist[];  // [E]
  __shared__ int s_e[MOONEP_PLAN_BLOCK];
  __shared__ int s_lc[MOONEP_PLAN_BLOCK];
  __shared__ int s_dst[MOONEP_PLAN_BLOCK];
  __shared__ short s_dest[MOONEP_PLAN_BLOCK];
  const bool live = !poisoned(c);
  const int R = c.R, E = c.E, K = c.K, NvS = c.NvS;
  const int tid = threadIdx.x;
  const int t0 = blockIdx.x * tokens_per_block;
  const int t1 = min(c.S, t0 + tokens_per_block);
  const int start = t0 * K;
  const int nent = live ? (t1 - t0) * K : 0;

  if (live) {
    // entries of earlier blocks: sum of their per-block histograms
    for (int e = tid; e < E; e += blockDim.x) s_hist[e] = 0;
    __syncthreads();
    {
      const long long total = (long long)blockIdx.x * E;  // rows of the blocks before this one
      for (long long idx = tid; idx < total; idx += blockDim.x) {
        const int v = c.block_hist[idx];
        if (v) atomicAdd(s_hist + (int)(idx % E), v);
      }
    }
    for (int i = tid; i < nent; i += blockDim.x) {
      const int e = topk[start + i];
      const bool valid = e >= 0 && e < E;
      if (!valid) record_status(c, MOONEP_STATUS_BAD_INDEX, MOONEP_K_PLAN_TOKENS, 2, e, E, start + i);
      s_e[i] = valid ? e : -1;
    }
    __syncthreads();
    // in-order index inside this block: entries before i with the same expert
    for (int i = tid; i < nent; i += blockDim.x) {
      const int e = s_e[i];
      int cnt = 0;
      for (int j = 0; j < i; ++j) cnt += (s_e[j] == e) ? 1 : 0;
      s_lc[i] = (e >= 0 ? s_hist[e] : 0) + cnt;
    }
    __syncthreads();
    for (int i = tid; i < nent; i += blockDim.x) {
      const int e = s_e[i];
      int dstv = -1, dest = -1;
      if (e >= 0) {
        const int g = c.tpe_prev[e] + s_lc[i];
        const int* ac = c.alloc_cum + (long long)e * R;
        int prev = 0;
        for (int d = 0; d < R; ++d) {
          const int cum = ac[d];
          if (g < cum) {
            dest = d;
            break;
          }
          prev = cum;
        }
        if (dest >= 0) {
          const int loff = c.expert_off[(long long)dest * E + e] + (g - prev);
          if (loff >= 0 && loff < NvS) {
            dstv = dest * NvS + loff;
          } else {
            record_status(c, MOONEP_STATUS_BAD_INDEX, MOONEP_K_PLAN_TOKENS, 3, loff, NvS, start + i);
            dest = -1;
          }
        } else {
          record_status(c, MOONEP_STATUS_BAD_INDEX, MOONEP_K_PLAN_TOKENS, 4, g, e, start + i);
        }
      }
      s_dst[i] = dstv;
      s_dest[i] = (short)dest;
    }
    __syncthreads();
    for (int i = tid; i < nent; i += blockDim.x) {
      const int dstv = s_dst[i];
      const int dest = s_dest[i];
      if (dest < 0) {
        dst_out[start + i] = 0;
        continue;
      }
      const int k = i % K;
      bool dup = false;
      for (int kk = 0; kk < k; ++kk) dup |= (s_dest[i - k + kk] == dest);
      int next = -1;
      for (int kk = K - 1; kk > k; --kk)
        if (s_dest[i - k + kk] == dest) next = s_dst[i - k + kk] - dest * NvS;
      dst_out[start + i] = dup ? -dstv - 1 : dstv;
      const int loff = dstv - dest * NvS;
      int* meta = c.meta_peer[dest];
      meta[c.src_info_off + loff] = c.rank * NvS + start + i;
      meta[c.link_off + loff] = (dup ? 0 : MOONEP_LINK_PRIMARY) | (next >= 0 ? (MOONEP_LINK_HAS_NEXT | next) : 0);
    }
  }
  grid_tail_signal(c, MOONEP_K_PLAN_TOKENS, live ? MOONEP_FLAG_PLAN : -1, epoch_plan);
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
                                   int* experts_to_copy, int* zero_fill, int* remote_stats, int wait_epoch_tpe,
                                   int signal_epoch_plan, void* stream) {
  auto* h = (HostCtx*)ctx;
  const MoonepDevCtx& c = h->dev;
  cudaStream_t st = (cudaStream_t)stream;
  size_t work_bytes = (size_t)table_words(c.R, c.E) * sizeof(int);
  int work_in_smem = 0;
  if ((int)work_bytes + 8192 <= h->max_smem_optin) {
    work_in_smem = 1;
    if (work_bytes > 48 * 1024) {
      if (int rc = check_cuda(cudaFuncSetAttribute(plan_tables_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                   (int)work_bytes),
                              "cudaFuncSetAttribute(plan_tables_kernel)"))
        return rc;
    }
  } else {
    work_bytes = 0;
  }
  plan_tables_kernel<<<1, kTablesThreads, work_bytes, st>>>(c, tpe2d, cu_seqlens, experts_to_copy, zero_fill, remote_stats,
                                                           wait_epoch_tpe, work_in_smem);
  if (int rc = check_launch("plan_tables_kernel")) return rc;
  const int tpb = imax(1, MOONEP_PLAN_BLOCK / c.K);
  const int grid = (c.S + tpb - 1) / tpb;
  const size_t smem = (size_t)c.E * sizeof(int);
  if (int rc = hist_smem_ok(h, (const void*)plan_tokens_kernel, smem, "plan_tokens_kernel")) return rc;
  plan_tokens_kernel<<<grid, kTokensThreads, smem, st>>>(c, topk, dst, tpb, signal_epoch_plan);
  return check_launch("plan_tokens_kernel");
}
