// Device-side bodies of the routing planner, shared by the stand-alone planner kernels (planner.cu),
// the fused dispatch kernel (dispatch_fused.cu) and the allocation-free table entry point
// (plan_noalloc.cu).
//
//   plan_tables_body   one CTA: from the tokens-per-expert rows of all ranks derive the tables that are
//                      identical on every rank (balance quotas, alloc[d][e], the group layout of every
//                      destination rank, experts_to_copy, remote_stats, cu_seqlens, zero_fill, expert offsets).
//   plan_tokens_block  one CTA per block of whole tokens: in-order index of every routing entry among the
//                      entries of its expert, destination row, duplicate marking, and the push of src_info
//                      and link words into the destination ranks' meta chunks.
//
// Results are exactly those of the host planner (moonep_b200/cpu/planner.py): first-index tie-breaking of
// argmax/argmin, quotas assigned (not accumulated), remote experts sorted by (count, expert) descending,
// remote_stats[0] uncapped.
//
// Parity: the algorithm of the reference's tests/planning_reference.py:33-329, which its package runs as
// moonep_td/_planning_gpu.py:86-592 (5 small kernels, dozens of torch ops, ~6+7R host synchronisations per plan).
#pragma once

#include <climits>

#include "common.cuh"

namespace moonep {

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

// Inputs and outputs of the table stage.  Optional outputs may be null.
struct TablesIO {
  const int* tpe;  // [R, E] tokens of expert e routed by source rank s
  int R, E, B, epn, cap, P, rank, NvS;
  int* cu_out;      // [E+B]    inclusive padded end of every group on `rank`
  int* etc_out;     // [R, B]   experts_to_copy
  int* zf_out;      // [E+B, 2] (first pad row, pad rows) per group on `rank`
  int* rs_out;      // [2]      remote_stats of `rank`
  int* tpe_prev;    // [E]      optional: tokens of expert e on source ranks < rank
  int* alloc_cum;   // [E, R]   optional: inclusive cumsum of alloc over destination ranks
  int* expert_off;  // [R, E]   optional: first row of expert e on destination d (needs the layout of every d)
};

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

// The table stage.  Must be called by all threads of one CTA (any multiple of 32 threads); `t` is carved from
// table_words(R, E) words of shared or global memory, every word of which is written before it is read.
// Returns (to every thread) 0, or the padded row total of a destination rank whose layout does not fit NvS.
__device__ inline int plan_tables_body(const TablesIO& io, const Tables& t) {
  const int R = io.R, E = io.E, B = io.B, epn = io.epn, P = io.P;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
  const int* tpe = io.tpe;
  __shared__ int s_balance[MOONEP_MAX_RANKS];
  __shared__ int s_bad;
  if (tid == 0) s_bad = 0;

  // 1. per-expert totals, prefix of the source ranks before this one, home allocation
  for (int e = tid; e < E; e += blockDim.x) {
    int cum = 0;
    for (int s = 0; s < R; ++s) {
      if (s == io.rank && io.tpe_prev != nullptr) io.tpe_prev[e] = cum;
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
    if (lane == 0) s_balance[h] = sum - io.cap;
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

  // 5. per-expert inclusive cumsum over destinations (the token phase searches it)
  if (io.alloc_cum != nullptr) {
    for (int e = tid; e < E; e += blockDim.x) {
      int cum = 0;
      for (int d = 0; d < R; ++d) {
        cum += t.alloc[(long long)d * E + e];
        io.alloc_cum[(long long)e * R + d] = cum;
      }
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
        io.etc_out[d * B + pos] = ei;
        atomicAdd(t.rs1 + ei / epn, 1);
      }
    }
    for (int b = lane; b < B; b += 32)
      if (b >= n) io.etc_out[d * B + b] = -1;
    if (d == io.rank && lane == 0) io.rs_out[0] = n;
    __syncwarp();
    if (d != io.rank && io.expert_off == nullptr) continue;  // only this rank's layout is an output
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
        eid = io.etc_out[d * B + (g - E)];
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
        if (cnt > 0 && io.expert_off != nullptr) io.expert_off[(long long)d * E + eid] = start;
        if (d == io.rank) {
          io.cu_out[g] = end_aligned;
          const bool pad = cnt > 0 && padded > cnt;
          io.zf_out[2 * g] = pad ? start + cnt : 0;
          io.zf_out[2 * g + 1] = pad ? padded - cnt : 0;
        }
      }
      carry += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0 && carry > io.NvS) s_bad = carry;
  }
  __syncthreads();
  if (tid == 0) io.rs_out[1] = t.rs1[io.rank];
  const int bad = s_bad;
  __syncthreads();
  return bad;
}

// Shared-memory arrays of the token stage (about 7 KB).
struct TokenScratch {
  int e[MOONEP_PLAN_BLOCK];
  int lc[MOONEP_PLAN_BLOCK];
  int dst[MOONEP_PLAN_BLOCK];
  short dest[MOONEP_PLAN_BLOCK];
};

// The token stage for planner block `block` (whole tokens, at most MOONEP_PLAN_BLOCK routing entries).  Must be
// called by all threads of the CTA; s_hist is [E] words of shared memory.  Needs block_hist of all blocks
// (plan_publish), alloc_cum, expert_off and tpe_prev (plan_tables_body).
__device__ inline void plan_tokens_block(const MoonepDevCtx& c, const int* __restrict__ topk, int* __restrict__ dst_out,
                                         int tokens_per_block, int block, int* s_hist, TokenScratch& s) {
  const int R = c.R, E = c.E, K = c.K, NvS = c.NvS;
  const int tid = threadIdx.x;
  const int t0 = block * tokens_per_block;
  const int t1 = min(c.S, t0 + tokens_per_block);
  const int start = t0 * K;
  const int nent = (t1 - t0) * K;

  // entries of earlier blocks: sum of their per-block histograms
  for (int e = tid; e < E; e += blockDim.x) s_hist[e] = 0;
  __syncthreads();
  {
    // column sums over the rows of the blocks before this one: a thread walks one expert's column (coalesced across
    // the threads of a row), `parts` threads share a column and meet in one shared-memory add each
    const int cols = min(E, (int)blockDim.x);
    const int parts = (int)blockDim.x / cols;
    const int part = tid / cols, col0 = tid - part * cols;
    if (part < parts) {
      for (int e = col0; e < E; e += cols) {
        int sum = 0;
        for (int r = part; r < block; r += parts) sum += c.block_hist[(long long)r * E + e];
        if (sum) atomicAdd(s_hist + e, sum);
      }
    }
  }
  for (int i = tid; i < nent; i += blockDim.x) {
    const int e = topk[start + i];
    const bool valid = e >= 0 && e < E;
    if (!valid) record_status(c, MOONEP_STATUS_BAD_INDEX, MOONEP_K_PLAN_TOKENS, 2, e, E, start + i);
    s.e[i] = valid ? e : -1;
  }
  __syncthreads();
  // in-order index inside this block: entries before i with the same expert
  for (int i = tid; i < nent; i += blockDim.x) {
    const int e = s.e[i];
    int cnt = 0;
    for (int j = 0; j < i; ++j) cnt += (s.e[j] == e) ? 1 : 0;
    s.lc[i] = (e >= 0 ? s_hist[e] : 0) + cnt;
  }
  __syncthreads();
  for (int i = tid; i < nent; i += blockDim.x) {
    const int e = s.e[i];
    int dstv = -1, dest = -1;
    if (e >= 0) {
      const int g = c.tpe_prev[e] + s.lc[i];
      // first destination whose running allocation exceeds g; no early exit, so that the loads are independent
      const int* ac = c.alloc_cum + (long long)e * R;
      int prev = 0, last = 0;
      for (int d = 0; d < R; ++d) {
        const int cum = ac[d];
        if (dest < 0 && g < cum) {
          dest = d;
          prev = last;
        }
        last = cum;
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
    s.dst[i] = dstv;
    s.dest[i] = (short)dest;
  }
  __syncthreads();
  for (int i = tid; i < nent; i += blockDim.x) {
    const int dstv = s.dst[i];
    const int dest = s.dest[i];
    if (dest < 0) {
      dst_out[start + i] = 0;
      continue;
    }
    const int k = i % K;
    bool dup = false;
    int ord = 0;  // position of a primary among the primaries of its token (ascending k)
    for (int kk = 0; kk < k; ++kk) {
      const int dk = s.dest[i - k + kk];
      dup |= (dk == dest);
      bool first = dk >= 0;
      for (int q = 0; q < kk; ++q) first &= (s.dest[i - k + q] != dk);
      ord += first ? 1 : 0;
    }
    int next = -1;
    for (int kk = K - 1; kk > k; --kk)
      if (s.dest[i - k + kk] == dest) next = s.dst[i - k + kk] - dest * NvS;
    dst_out[start + i] = dup ? -dstv - 1 : dstv;
    const int loff = dstv - dest * NvS;
    int* meta = c.meta_peer[dest];
    meta[c.src_info_off + loff] = c.rank * NvS + start + i;
    meta[c.link_off + loff] = (dup ? 0 : (MOONEP_LINK_PRIMARY | (ord << MOONEP_LINK_ORD_SHIFT))) |
                              (next >= 0 ? (MOONEP_LINK_HAS_NEXT | next) : 0);
  }
  __syncthreads();
}

}  // namespace moonep
