// Dispatch for sm_100a: push token rows and gate weights into the destination ranks'
// shards over NVLink peer memory, build the duplicate map on the destination, and expand
// duplicates locally.
//
//   dispatch_send    persistent, num_sms CTAs.  Waits (bounded) until every peer is ready
//                    (FLAG_PLAN after a fresh plan, FLAG_READY for a replayed plan).  Tokens are
//                    handed out in small batches from an atomic counter.  Each token row is
//                    read from HBM once and written to every destination rank that owns one of
//                    its experts (only the first entry per rank: per-rank dedup); the K gate
//                    weights go to the rows' weight slots.  Two copy paths:
//                      bulk: one lane per warp drives a 3-stage shared-memory ring with
//                            cp.async.bulk (global->shared on an mbarrier, shared->peer global in
//                            bulk groups); no register traffic, one instruction per 14 KB row.
//                      ldst: 16-byte loads into registers, 16-byte stores to every destination.
//                    Meanwhile, for a fresh
//                    plan, dup_groups/dup_loffs/dup_counts are built from the link words the
//                    peers pushed during planning (all CTAs share the rows).  The last CTA to finish signals FLAG_SENT.
//   dispatch_expand  all SMs: zero-fills the pad rows of the local shard, waits for every peer's
//                    FLAG_SENT, then copies each primary row to its duplicate rows inside the shard.
//
// Parity: reference moonep_td/dispatch.py:42-117 (dispatch_kernel, zero_fill_kernel),
// moonep_td/_dedup_builder.py:23-108 (three dedup kernels), moonep_td/dispatch_epilogue.py:21-40.
// The reference moves 2 bytes per thread per iteration, launches one CTA per (token, k) entry
// and re-reads the source row for every destination.
#include <climits>

#include "common.cuh"
#include "host.h"

namespace moonep {

namespace {

constexpr int kSendThreadsLdst = 512;
constexpr int kSendThreadsBulk = 256;
constexpr int kBulkWarps = 4;    // warps of a CTA that drive bulk copies
constexpr int kBulkStages = 3;   // ring depth per warp
constexpr int kTokenBatch = 4;   // tokens handed out per grab
constexpr int kVecPerLane = 8;   // int4 per lane per register chunk (4 KB per warp)
constexpr int kMaxChunkBytes = 16 * 1024;

struct SendArgs {
  const uint16_t* hidden;  // [S, H] bf16
  const float* weights;    // [S, K] or null
  const int* dst;          // [N]
  const int* zero_fill;    // [E+B, 2]
  int* dup_groups;         // [NvS, 3]
  int* dup_loffs;          // [NvS]
  int* dup_counts;         // [2]
  int build_dedup;
  int wait_family, wait_epoch, signal_epoch;
  int vec_ok;              // rows are 16-byte aligned and a multiple of 16 bytes
  int chunk_bytes, nchunks;  // bulk path: a row is sent in nchunks pieces
};

__device__ __forceinline__ void decode_dst(int d, int NvS, int& dest, int& loff) {
  const int raw = d < 0 ? -d - 1 : d;
  dest = raw / NvS;
  loff = raw - dest * NvS;
}

// ---- destination-side dedup builder (all CTAs share the rows) ----------------------------------
//
// During planning every source pushed, next to src_info, a link word per landed row: whether the
// row is the first of its (source, token) on this rank and which row holds the next entry of the
// same token.  A primary row that has a successor opens a group; walking the chain lists its
// duplicates in ascending k.  Rows are independent, so any number of threads can share them; groups
// and duplicate rows are numbered with one pair of atomics per warp.  dup_counts is zeroed by the
// host wrapper before the launch.
__device__ void build_dedup_rows(const MoonepDevCtx& c, const SendArgs& a, int gthread, int gthreads) {
  const int lane = threadIdx.x & 31;
  const int NvS = c.NvS;
  const int* src_info = c.meta_peer[c.rank] + c.src_info_off;
  const int* link = c.meta_peer[c.rank] + c.link_off;
  const int rounds = (NvS + gthreads - 1) / gthreads;
  for (int it = 0; it < rounds; ++it) {
    const int loff = it * gthreads + gthread;
    int dup_n = 0, first = -1;
    if (loff < NvS && src_info[loff] >= 0) {
      const int l = link[loff];
      if ((l & MOONEP_LINK_PRIMARY) && (l & MOONEP_LINK_HAS_NEXT)) {
        first = l & MOONEP_NVS_MASK;
        int cur = first;
        while (dup_n < MOONEP_MAX_TOPK) {
          if (cur < 0 || cur >= NvS) {
            record_status(c, MOONEP_STATUS_BAD_INDEX, MOONEP_K_DISPATCH_SEND, 5, cur, loff, 0);
            dup_n = 0;
            break;
          }
          ++dup_n;
          const int l2 = link[cur];
          if (!(l2 & MOONEP_LINK_HAS_NEXT)) break;
          cur = l2 & MOONEP_NVS_MASK;
        }
      }
    }
    const unsigned has = __ballot_sync(0xffffffffu, dup_n > 0);
    if (has == 0) continue;
    int incl = dup_n;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    const int total = __shfl_sync(0xffffffffu, incl, 31);
    int gbase = 0, dbase = 0;
    if (lane == 0) {
      gbase = atomicAdd(a.dup_counts, __popc(has));
      dbase = atomicAdd(a.dup_counts + 1, total);
    }
    gbase = __shfl_sync(0xffffffffu, gbase, 0);
    dbase = __shfl_sync(0xffffffffu, dbase, 0);
    if (dup_n > 0) {
      const int g = gbase + __popc(has & ((1u << lane) - 1u));
      int ds = dbase + incl - dup_n;
      if (g < NvS && ds + dup_n <= NvS) {
        a.dup_groups[3 * g] = loff;
        a.dup_groups[3 * g + 1] = ds;
        a.dup_groups[3 * g + 2] = dup_n;
        int cur = first;
        for (int q = 0; q < dup_n; ++q) {
          a.dup_loffs[ds + q] = cur;
          cur = link[cur] & MOONEP_NVS_MASK;
        }
      }
    }
  }
}

// ---- zero fill of pad rows ---------------------------------------------------------------------

// Reads the (start, count) pairs of 32 groups at a time, then spreads the pad rows of every
// non-empty range over all participating warps.
__device__ void zero_fill_rows(const MoonepDevCtx& c, const SendArgs& a, int warp_global, int warps_total, int lane) {
  uint16_t* shard = c.hidden_peer[c.rank];
  float* wbuf = reinterpret_cast<float*>(c.meta_peer[c.rank] + c.weights_off);
  const int ngroups = c.E + c.B;
  const int H = c.H;
  int seen = 0;  // pad rows of the ranges before this one: rows are dealt round-robin across ranges
  for (int base = 0; base < ngroups; base += 32) {
    const int g = base + lane;
    int n_pad = 0, start = 0;
    if (g < ngroups) {
      n_pad = a.zero_fill[2 * g + 1];
      start = a.zero_fill[2 * g];
    }
    unsigned m = __ballot_sync(0xffffffffu, n_pad > 0);
    while (m) {
      const int src = __ffs(m) - 1;
      m &= m - 1;
      const int s0 = __shfl_sync(0xffffffffu, start, src);
      const int np = __shfl_sync(0xffffffffu, n_pad, src);
      const int first = ((warp_global - seen) % warps_total + warps_total) % warps_total;
      seen = (seen + np) % warps_total;
      for (int r = first; r < np; r += warps_total) {
        const int row = s0 + r;
        if (row < 0 || row >= c.NvS) continue;
        uint16_t* p = shard + (long long)row * H;
        if (a.vec_ok) {
          const int nvec = H / 8;
          const int4 z = make_int4(0, 0, 0, 0);
          for (int i = lane; i < nvec; i += 32) st16(reinterpret_cast<int4*>(p) + i, z);
        } else {
          for (int i = lane; i < H; i += 32) p[i] = 0;
        }
        if (a.weights != nullptr && lane == 0) wbuf[row] = 0.f;
      }
    }
  }
}

// Grab the next batch of tokens; lane-uniform result.
__device__ __forceinline__ int grab_tokens(int* counter, int lane) {
  int b = 0;
  if (lane == 0) b = atomicAdd(counter, kTokenBatch);
  return __shfl_sync(0xffffffffu, b, 0);
}

// Store the K gate weights of a token next to the rows they belong to.
__device__ __forceinline__ void push_weights(const MoonepDevCtx& c, const SendArgs& a, int token, int lane, int dest,
                                             int loff) {
  if (a.weights != nullptr && lane < c.K) {
    float* w = reinterpret_cast<float*>(c.meta_peer[dest] + c.weights_off);
    w[loff] = a.weights[token * c.K + lane];
  }
}

__device__ __forceinline__ bool dst_in_range(const MoonepDevCtx& c, int dest, int loff) {
  return dest >= 0 && dest < c.R && loff >= 0 && loff < c.NvS;
}

// ---- send kernel, register path ------------------------------------------------------------------

__global__ void __launch_bounds__(kSendThreadsLdst) dispatch_send_ldst_kernel(const MoonepDevCtx c, const SendArgs a) {
  const bool ok = block_wait_flags(c, a.wait_family, a.wait_epoch, MOONEP_K_DISPATCH_SEND);
  const int lane = threadIdx.x & 31;
  int* work = c.counters + MOONEP_NUM_KERNEL_IDS;  // token counter of this kernel
  if (ok) {
    if (a.build_dedup) build_dedup_rows(c, a, blockIdx.x * blockDim.x + threadIdx.x, gridDim.x * blockDim.x);
    const int H = c.H, K = c.K, S = c.S;
    for (;;) {
      const int b0 = grab_tokens(work, lane);
      if (b0 >= S) break;
      const int b1 = min(S, b0 + kTokenBatch);
      for (int token = b0; token < b1; ++token) {
        int d = 0, dest = 0, loff = 0;
        bool valid = false;
        if (lane < K) {
          d = a.dst[token * K + lane];
          decode_dst(d, c.NvS, dest, loff);
          valid = dst_in_range(c, dest, loff);
          if (!valid) record_status(c, MOONEP_STATUS_BAD_INDEX, MOONEP_K_DISPATCH_SEND, 6, d, token, lane);
        }
        if (valid) push_weights(c, a, token, lane, dest, loff);
        const unsigned prim = __ballot_sync(0xffffffffu, valid && d >= 0);
        const uint16_t* src = a.hidden + (long long)token * H;
        if (a.vec_ok) {
          const int nvec = H / 8;
          const int4* s4 = reinterpret_cast<const int4*>(src);
          for (int c0 = 0; c0 < nvec; c0 += 32 * kVecPerLane) {
            int4 v[kVecPerLane];
#pragma unroll
            for (int j = 0; j < kVecPerLane; ++j) {
              const int i = c0 + j * 32 + lane;
              if (i < nvec) v[j] = ld16(s4 + i);
            }
            unsigned m = prim;
            while (m) {
              const int kk = __ffs(m) - 1;
              m &= m - 1;
              const int dd = __shfl_sync(0xffffffffu, dest, kk);
              const int ll = __shfl_sync(0xffffffffu, loff, kk);
              int4* o4 = reinterpret_cast<int4*>(c.hidden_peer[dd] + (long long)ll * H);
#pragma unroll
              for (int j = 0; j < kVecPerLane; ++j) {
                const int i = c0 + j * 32 + lane;
                if (i < nvec) st16(o4 + i, v[j]);
              }
            }
          }
        } else {
          unsigned m = prim;
          while (m) {
            const int kk = __ffs(m) - 1;
            m &= m - 1;
            const int dd = __shfl_sync(0xffffffffu, dest, kk);
            const int ll = __shfl_sync(0xffffffffu, loff, kk);
            uint16_t* o = c.hidden_peer[dd] + (long long)ll * H;
            for (int i = lane; i < H; i += 32) o[i] = src[i];
          }
        }
      }
    }
  }
  // tail: last CTA resets the token counter and signals
  __shared__ int s_last;
  __syncthreads();
  if (threadIdx.x == 0) {
    fence_sys();
    const int arrived = atomicAdd(c.counters + MOONEP_K_DISPATCH_SEND, 1);
    s_last = arrived == (int)gridDim.x - 1;
    if (s_last) {
      c.counters[MOONEP_K_DISPATCH_SEND] = 0;
      *work = 0;
      fence_sys();
    }
  }
  __syncthreads();
  if (s_last && ok) {
    for (int r = threadIdx.x; r < c.R; r += blockDim.x)
      st_release_sys(flag_ptr(c, r, MOONEP_FLAG_SENT, c.rank), abs_epoch(c, MOONEP_FLAG_SENT, a.signal_epoch));
  }
}

// ---- send kernel, bulk-copy path -----------------------------------------------------------------

__global__ void __launch_bounds__(kSendThreadsBulk) dispatch_send_bulk_kernel(const MoonepDevCtx c, const SendArgs a) {
  extern __shared__ __align__(128) unsigned char s_ring[];  // [kBulkWarps][kBulkStages][chunk_bytes]
  __shared__ __align__(8) unsigned long long s_bar[kBulkWarps][kBulkStages];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  if (threadIdx.x < kBulkWarps * kBulkStages) mbar_init(&s_bar[0][0] + threadIdx.x, 1);
  fence_barrier_init();
  const bool ok = block_wait_flags(c, a.wait_family, a.wait_epoch, MOONEP_K_DISPATCH_SEND);
  int* work = c.counters + MOONEP_NUM_KERNEL_IDS;
  if (ok) {
    if (warp >= kBulkWarps) {
      // helper warps: duplicate map
      const int hw = nwarps - kBulkWarps;
      const int hthreads = hw * 32;
      if (a.build_dedup)
        build_dedup_rows(c, a, blockIdx.x * hthreads + (threadIdx.x - kBulkWarps * 32), gridDim.x * hthreads);
    } else {
      const int H = c.H, K = c.K, S = c.S;
      const long long row_bytes = (long long)H * 2;
      unsigned char* ring = s_ring + (size_t)warp * kBulkStages * a.chunk_bytes;
      unsigned long long* bar = s_bar[warp];
      int ring_tok[kBulkStages], ring_chunk[kBulkStages];
      int batch_next = 0, batch_end = 0, cur_chunk = 0;
      bool more = true;
      int loaded = 0, done = 0;
      bool failed = false;

      auto next_item = [&](int& tok, int& ch) -> bool {
        if (batch_next == batch_end) {
          const int b = grab_tokens(work, lane);
          if (b >= S) return false;
          batch_next = b;
          batch_end = min(S, b + kTokenBatch);
          cur_chunk = 0;
        }
        tok = batch_next;
        ch = cur_chunk;
        if (++cur_chunk == a.nchunks) {
          cur_chunk = 0;
          ++batch_next;
        }
        return true;
      };
      auto chunk_len = [&](int ch) -> unsigned {
        const long long off = (long long)ch * a.chunk_bytes;
        const long long rest = row_bytes - off;
        return (unsigned)(rest < a.chunk_bytes ? rest : a.chunk_bytes);
      };
      auto issue_load = [&](int tok, int ch) {
        const int s = loaded % kBulkStages;
#pragma unroll
        for (int q = 0; q < kBulkStages; ++q)
          if (q == s) {
            ring_tok[q] = tok;
            ring_chunk[q] = ch;
          }
        if (lane == 0) {
          const unsigned len = chunk_len(ch);
          mbar_expect_tx(bar + s, len);
          bulk_g2s(ring + (size_t)s * a.chunk_bytes,
                   reinterpret_cast<const unsigned char*>(a.hidden) + tok * row_bytes + (long long)ch * a.chunk_bytes, len,
                   bar + s);
        }
        ++loaded;
      };

      int tok, ch;
      more = next_item(tok, ch);
      if (more) issue_load(tok, ch);
      while (done < loaded && !failed) {
        if (more) {
          more = next_item(tok, ch);
          if (more) {
            // the stage about to be refilled was read by the bulk group committed two items ago
            if (lane == 0) bulk_wait_read<1>();
            issue_load(tok, ch);
          }
        }
        const int s = done % kBulkStages;
        int ctok = 0, cch = 0;
#pragma unroll
        for (int q = 0; q < kBulkStages; ++q)
          if (q == s) {
            ctok = ring_tok[q];
            cch = ring_chunk[q];
          }
        int d = 0, dest = 0, loff = 0;
        bool valid = false;
        if (lane < K) {
          d = a.dst[ctok * K + lane];
          decode_dst(d, c.NvS, dest, loff);
          valid = dst_in_range(c, dest, loff);
          if (!valid) record_status(c, MOONEP_STATUS_BAD_INDEX, MOONEP_K_DISPATCH_SEND, 6, d, ctok, lane);
        }
        if (valid && cch == 0) push_weights(c, a, ctok, lane, dest, loff);
        unsigned m = __ballot_sync(0xffffffffu, valid && d >= 0);
        int got = 1;
        if (lane == 0) got = mbar_wait(bar + s, (unsigned)((done / kBulkStages) & 1), c.timeout_ns) ? 1 : 0;
        got = __shfl_sync(0xffffffffu, got, 0);
        if (!got) {
          if (lane == 0) record_status(c, MOONEP_STATUS_TIMEOUT, MOONEP_K_DISPATCH_SEND, 100, s, done, ctok);
          failed = true;
          break;
        }
        const unsigned len = chunk_len(cch);
        while (m) {
          const int kk = __ffs(m) - 1;
          m &= m - 1;
          const int dd = __shfl_sync(0xffffffffu, dest, kk);
          const int ll = __shfl_sync(0xffffffffu, loff, kk);
          if (lane == 0) {
            unsigned char* o = reinterpret_cast<unsigned char*>(c.hidden_peer[dd]) + (long long)ll * row_bytes +
                               (long long)cch * a.chunk_bytes;
            bulk_s2g(o, ring + (size_t)s * a.chunk_bytes, len);
          }
        }
        if (lane == 0) bulk_commit();
        ++done;
      }
      if (lane == 0) bulk_wait<0>();
      __syncwarp();
    }
  }
  __shared__ int s_last;
  __syncthreads();
  if (threadIdx.x == 0) {
    fence_sys();
    const int arrived = atomicAdd(c.counters + MOONEP_K_DISPATCH_SEND, 1);
    s_last = arrived == (int)gridDim.x - 1;
    if (s_last) {
      c.counters[MOONEP_K_DISPATCH_SEND] = 0;
      *work = 0;
      fence_sys();
    }
  }
  __syncthreads();
  if (s_last && ok) {
    for (int r = threadIdx.x; r < c.R; r += blockDim.x)
      st_release_sys(flag_ptr(c, r, MOONEP_FLAG_SENT, c.rank), abs_epoch(c, MOONEP_FLAG_SENT, a.signal_epoch));
  }
}

// ---- duplicate expansion --------------------------------------------------------------------------

__global__ void __launch_bounds__(512)
    dispatch_expand_kernel(const MoonepDevCtx c, const int* __restrict__ zero_fill, int with_weights,
                           const int* __restrict__ dup_groups, const int* __restrict__ dup_loffs,
                           const int* __restrict__ dup_counts, int wait_epoch, int vec_ok) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  if (!poisoned(c) && zero_fill != nullptr) {
    // pad rows belong to this rank alone, so they are cleared while the peers' rows are still arriving
    SendArgs z;
    z.zero_fill = zero_fill;
    z.vec_ok = vec_ok;
    z.weights = with_weights ? reinterpret_cast<const float*>(zero_fill) : nullptr;  // only tested for null
    zero_fill_rows(c, z, blockIdx.x * nwarps + warp, gridDim.x * nwarps, lane);
  }
  if (!block_wait_flags(c, MOONEP_FLAG_SENT, wait_epoch, MOONEP_K_DISPATCH_EXPAND)) return;
  const int H = c.H;
  int ngroups = dup_counts[0];
  if (ngroups < 0 || ngroups > c.NvS) ngroups = 0;
  uint16_t* shard = c.hidden_peer[c.rank];
  for (int g = blockIdx.x * nwarps + warp; g < ngroups; g += gridDim.x * nwarps) {
    const int primary = dup_groups[3 * g];
    const int ds = dup_groups[3 * g + 1];
    const int dn = dup_groups[3 * g + 2];
    if (primary < 0 || primary >= c.NvS || ds < 0 || dn < 0 || ds + dn > c.NvS) continue;
    const uint16_t* src = shard + (long long)primary * H;
    // lane q holds the q-th duplicate row (a group has fewer than 32 duplicates)
    const int my_dup = (lane < dn && lane < 32) ? dup_loffs[ds + lane] : -1;
    if (vec_ok) {
      const int nvec = H / 8;
      const int4* s4 = reinterpret_cast<const int4*>(src);
      for (int c0 = 0; c0 < nvec; c0 += 32 * kVecPerLane) {
        int4 v[kVecPerLane];
#pragma unroll
        for (int j = 0; j < kVecPerLane; ++j) {
          const int i = c0 + j * 32 + lane;
          if (i < nvec) v[j] = ld16(s4 + i);
        }
        for (int q = 0; q < dn && q < 32; ++q) {
          const int row = __shfl_sync(0xffffffffu, my_dup, q);
          if (row < 0 || row >= c.NvS) continue;
          int4* o4 = reinterpret_cast<int4*>(shard + (long long)row * H);
#pragma unroll
          for (int j = 0; j < kVecPerLane; ++j) {
            const int i = c0 + j * 32 + lane;
            if (i < nvec) st16(o4 + i, v[j]);
          }
        }
      }
    } else {
      for (int q = 0; q < dn; ++q) {
        const int row = dup_loffs[ds + q];
        if (row < 0 || row >= c.NvS) continue;
        uint16_t* o = shard + (long long)row * H;
        for (int i = lane; i < H; i += 32) o[i] = src[i];
      }
    }
  }
}

}  // namespace

}  // namespace moonep

using namespace moonep;

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

extern "C" int moonep_dispatch_send(void* ctx, const void* hidden, const float* weights, const int* dst,
                                    const int* zero_fill, int* dup_groups, int* dup_loffs, int* dup_counts,
                                    int build_dedup, int wait_family, int wait_epoch, int signal_epoch_sent, int path,
                                    void* stream) {
  auto* h = (HostCtx*)ctx;
  const MoonepDevCtx& c = h->dev;
  SendArgs a;
  a.hidden = (const uint16_t*)hidden;
  a.weights = weights;
  a.dst = dst;
  a.zero_fill = zero_fill;
  a.dup_groups = dup_groups;
  a.dup_loffs = dup_loffs;
  a.dup_counts = dup_counts;
  a.build_dedup = build_dedup;
  a.wait_family = wait_family;
  a.wait_epoch = wait_epoch;
  a.signal_epoch = signal_epoch_sent;
  a.vec_ok = (c.H % 8 == 0) && aligned16(hidden);
  const long long row_bytes = (long long)c.H * 2;
  a.nchunks = (int)((row_bytes + kMaxChunkBytes - 1) / kMaxChunkBytes);
  long long cb = (row_bytes + a.nchunks - 1) / a.nchunks;
  a.chunk_bytes = (int)((cb + 15) / 16 * 16);
  const int grid = imax(1, imin(c.num_sms, h->sm_count));
  cudaStream_t st = (cudaStream_t)stream;
  if (build_dedup) {
    if (int rc = check_cuda(cudaMemsetAsync(dup_counts, 0, 2 * sizeof(int), st), "cudaMemsetAsync(dup_counts)"))
      return rc;
  }
  if (path == MOONEP_PATH_BULK && a.vec_ok) {
    const size_t smem = (size_t)kBulkWarps * kBulkStages * a.chunk_bytes;
    if ((int)smem + 4096 <= h->max_smem_optin) {
      if (int rc = check_cuda(cudaFuncSetAttribute(dispatch_send_bulk_kernel,
                                                   cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem),
                              "cudaFuncSetAttribute(dispatch_send_bulk_kernel)"))
        return rc;
      dispatch_send_bulk_kernel<<<grid, kSendThreadsBulk, smem, st>>>(c, a);
      return check_launch("dispatch_send_bulk_kernel");
    }
  }
  dispatch_send_ldst_kernel<<<grid, kSendThreadsLdst, 0, st>>>(c, a);
  return check_launch("dispatch_send_ldst_kernel");
}

extern "C" int moonep_dispatch_expand(void* ctx, const int* zero_fill, int with_weights, const int* dup_groups,
                                      const int* dup_loffs, const int* dup_counts, int wait_epoch_sent, void* stream) {
  auto* h = (HostCtx*)ctx;
  const MoonepDevCtx& c = h->dev;
  const int grid = imax(1, imin(c.local_sms, h->sm_count));
  dispatch_expand_kernel<<<grid, 512, 0, (cudaStream_t)stream>>>(c, zero_fill, with_weights, dup_groups, dup_loffs,
                                                                dup_counts, wait_epoch_sent, (c.H % 8 == 0) ? 1 : 0);
  return check_launch("dispatch_expand_kernel");
}
