// Dispatch for sm_100a: one kernel whose CTAs take roles; launched with all roles it is the fused
// dispatch (planner tables -> token planning -> row push over NVLink, overlapped with zero fill,
// duplicate-map construction and duplicate expansion on the destination), launched role by role it
// gives the stand-alone stages of the launch-level API and of emulated ranks that share one GPU.
//
//   TABLES   (CTA 0) waits for every peer's tokens-per-expert row (FLAG_TPE), derives the global tables
//            (planner.cuh) and publishes "tables ready" to the other CTAs of this GPU.
//   TOKENS   sender CTAs plan their blocks of tokens (destination rows, duplicate marking, src_info and
//            link words pushed to the destinations); the last one signals FLAG_PLAN to every peer.
//   SEND     persistent sender CTAs; tokens are handed out in small batches from an atomic counter.  Each
//            row is read from HBM once and written to every destination rank that owns one of its experts
//            (only the first entry per rank crosses NVLink: per-rank dedup).  Two copy paths:
//              bulk: one lane per warp drives a 3-stage shared-memory ring with cp.async.bulk
//                    (global->shared on an mbarrier, shared->peer global in bulk groups);
//              ldst: 16-byte loads into registers, 16-byte stores to every destination.
//            When the copies of a row are complete (bulk group retired, or stores issued) the row's
//            flag in the destination's meta chunk is released with the dispatch's SENT epoch, so a
//            consumer there (the EXPAND role, a grouped GEMM's producer warp) can start on that row
//            without waiting for the whole all-to-all.  The last sender CTA signals FLAG_SENT.
//   EXPAND   every other CTA: zero-fills the pad rows of the local shard (flagging them as well), waits for
//            every peer's FLAG_PLAN, builds dup_groups/dup_loffs/dup_counts from the link words (and keeps
//            a copy of src_info and link words in the plan), then copies each primary row to its
//            duplicate rows as soon as the primary's row flag shows it has landed.  Ends with a wait for
//            every peer's FLAG_SENT, so all rows of the shard are present when the kernel is.
//
// CTA order: TABLES is CTA 0, senders follow, expanders come last, so a CTA only ever waits for CTAs with a
// lower index (which the hardware dispatches first) or for other GPUs.  Every wait is bounded.
//
// Parity: reference moonep_td/dispatch.py:42-117 (dispatch_kernel, zero_fill_kernel),
// moonep_td/_dedup_builder.py:23-108 (three dedup kernels), moonep_td/dispatch_epilogue.py:21-40, driven
// by moonep_td/api.py:275-305 with six cross-rank barriers and a host read of dup_counts.  The reference
// moves 2 bytes per thread per iteration, launches one CTA per (token, k) entry and re-reads the source
// row for every destination.
#include <climits>
#include <cstdlib>
#include <cstring>

#include "common.cuh"
#include "host.h"
#include "planner.cuh"

namespace moonep {

namespace {

constexpr int kDispatchThreads = 512;
constexpr int kBulkWarps = 4;    // warps of a sender CTA that drive bulk copies
constexpr int kBulkStages = 3;   // ring depth per warp
constexpr int kTokenBatch = 4;   // tokens handed out per grab
constexpr int kVecPerLane = 8;   // int4 per lane per register chunk (4 KB per warp)
constexpr int kMaxChunkBytes = 16 * 1024;
constexpr int kExpandVec = 14;   // int4 per lane in flight while a row is expanded (a 14 KB row in two steps)
constexpr int kExpandCopyWarps = 12;  // warps of an expander CTA that own a shared-memory piece for bulk copies
constexpr int kExpandSlice = 2048;  // rows whose duplicate groups an expander CTA lists in shared memory at a time

// Base addresses of every rank's shard and meta chunk, copied into shared memory at kernel start: the copy loops
// look them up per destination, and a lookup in global memory is a dependent load of several hundred nanoseconds.
struct PeerTables {
  uint16_t* hidden[MOONEP_MAX_RANKS];
  int* meta[MOONEP_MAX_RANKS];
};

struct DispatchArgs {
  // planner (fresh plans)
  const int* topk;   // [N]
  const int* tpe2d;  // [R, E] or null (rows pushed by plan_publish are used)
  int* dst;          // [N] written by TOKENS, read by SEND
  int* cu_seqlens;
  int* experts_to_copy;
  int* zero_fill;    // [E+B, 2] written by TABLES, read by EXPAND
  int* remote_stats;
  int tokens_per_block, n_blocks, tables_in_smem;
  // send
  const uint16_t* hidden;  // [S, H] bf16
  const float* weights;    // [S, K] or null
  // destination side
  int* dup_groups;     // [NvS, 3]
  int* dup_loffs;      // [NvS]
  int* dup_counts;     // [2]
  int* plan_src_info;  // [NvS] or null: the plan's copy of src_info
  int* plan_link;      // [NvS] or null: the plan's copy of the link words
  int fresh;           // planning and the duplicate map belong to this dispatch
  int roles, n_send;
  int with_weights;    // the zero fill also clears the pad rows' weight slots
  int wait_family, wait_epoch;  // replayed plans: what SEND waits for (FLAG_READY or nothing)
  int epoch_tpe, epoch_plan, epoch_sent;
  int vec_ok;                // rows are 16-byte aligned and a multiple of 16 bytes
  int chunk_bytes, nchunks;  // bulk path: a row is sent in nchunks pieces
  int bulk;
  int expand_bulk;  // EXPAND copies through shared memory with bulk copies (needs (kExpandCopyWarps + 1) pieces of smem)
  int build_only;  // EXPAND: only build the duplicate map (no zero fill, no copies)
  int local_rows;  // rows whose source is this rank are written by EXPAND from the input; SEND skips them
  int publish;     // the launch starts with the exchange plan_publish does as a kernel of its own
  const int* tpe_row;  // [E] this rank's tokens per expert, pushed to every peer by the publish step (null: a [R, E]
                       // table was given and nothing is pushed)
};

__device__ __forceinline__ void decode_dst(int d, int NvS, int& dest, int& loff) {
  const int raw = d < 0 ? -d - 1 : d;
  dest = raw / NvS;
  loff = raw - dest * NvS;
}

__device__ __forceinline__ bool dst_in_range(const MoonepDevCtx& c, int dest, int loff) {
  return dest >= 0 && dest < c.R && loff >= 0 && loff < c.NvS;
}

__device__ __forceinline__ int* rowflag_ptr(const MoonepDevCtx& c, int on_rank, int loff) {
  return c.meta_peer[on_rank] + c.rowflag_off + loff;
}

// CTAs of one role finish: true (to every thread) in the last of `count` CTAs, after a system-scope fence
// that orders every CTA's earlier writes before whatever the last CTA publishes next.
__device__ __forceinline__ bool role_tail(const MoonepDevCtx& c, int counter, int count) {
  __shared__ int s_last;
  __syncthreads();
  if (threadIdx.x == 0) {
    fence_sys();
    const int arrived = atomicAdd(c.counters + counter, 1);
    s_last = (arrived == count - 1);
    if (s_last) {
      c.counters[counter] = 0;
      fence_sys();
    }
  }
  __syncthreads();
  const bool last = s_last != 0;
  __syncthreads();
  return last;
}

// ---- zero fill of pad rows ---------------------------------------------------------------------

// Block-wide.  The (first pad row, pad rows) pairs of up to kZfChunk groups at a time go to shared memory together
// with the running total of pad rows, so that pad row j of the rank is found by a binary search; the pad rows are
// dealt round-robin to all participating warps (warp_global of warps_total).  A warp first clears its rows, then
// (after one completion wait and one fence for all of them) releases their row flags.  With `zeros` (a shared-memory
// piece of chunk_bytes zeros, visible to the async proxy) the rows are cleared by bulk stores from it, one
// instruction per piece of a row, instead of by register stores.  s_start / s_cum: kZfChunk words of shared memory each.
constexpr int kZfChunk = 1024;

__device__ void zero_fill_rows(const MoonepDevCtx& c, const int* __restrict__ zero_fill, int with_weights, int vec_ok,
                               int epoch, int warp_global, int warps_total, int* s_start, int* s_cum,
                               const unsigned char* zeros = nullptr, int chunk_bytes = 0) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint16_t* shard = c.hidden_peer[c.rank];
  float* wbuf = reinterpret_cast<float*>(c.meta_peer[c.rank] + c.weights_off);
  int* rowflag = c.meta_peer[c.rank] + c.rowflag_off;
  const int ngroups = c.E + c.B;
  const int H = c.H;
  for (int gbase = 0; gbase < ngroups; gbase += kZfChunk) {
    const int n = min(kZfChunk, ngroups - gbase);
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      const int np = zero_fill[2 * (gbase + i) + 1];
      s_start[i] = zero_fill[2 * (gbase + i)];
      s_cum[i] = np > 0 ? np : 0;
    }
    __syncthreads();
    if (warp == 0) {  // inclusive running total, 32 groups per step
      int carry = 0;
      for (int i0 = 0; i0 < n; i0 += 32) {
        const int i = i0 + lane;
        int v = i < n ? s_cum[i] : 0;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const int u = __shfl_up_sync(0xffffffffu, v, o);
          if (lane >= o) v += u;
        }
        if (i < n) s_cum[i] = carry + v;
        carry += __shfl_sync(0xffffffffu, v, 31);
      }
    }
    __syncthreads();
    const int total = s_cum[n - 1];
    for (int pass = 0; pass < 2; ++pass) {
      for (int j = warp_global; j < total; j += warps_total) {
        int lo = 0, hi = n - 1;  // first group whose running total exceeds j
        while (lo < hi) {
          const int mid = (lo + hi) >> 1;
          if (s_cum[mid] > j) hi = mid; else lo = mid + 1;
        }
        const int row = s_start[lo] + (j - (lo > 0 ? s_cum[lo - 1] : 0));
        if (row < 0 || row >= c.NvS) continue;
        if (pass == 1) {
          if (lane == 0) st_relaxed_gpu(rowflag + row, epoch);
          continue;
        }
        uint16_t* p = shard + (long long)row * H;
        if (zeros != nullptr) {
          if (lane == 0) {
            const long long row_bytes = (long long)H * 2;
            for (long long off = 0; off < row_bytes; off += chunk_bytes)
              bulk_s2g(reinterpret_cast<unsigned char*>(p) + off, zeros,
                       (unsigned)(row_bytes - off < chunk_bytes ? row_bytes - off : chunk_bytes));
          }
        } else if (vec_ok) {
          const int nvec = H / 8;
          const int4 z = make_int4(0, 0, 0, 0);
          for (int i = lane; i < nvec; i += 32) st16(reinterpret_cast<int4*>(p) + i, z);
        } else {
          for (int i = lane; i < H; i += 32) p[i] = 0;
        }
        if (with_weights && lane == 0) wbuf[row] = 0.f;
      }
      if (pass == 0) {
        // everything this warp cleared must be in memory before the first flag goes out
        __syncwarp();
        if (lane == 0) {
          if (zeros != nullptr) {
            bulk_commit();
            bulk_wait<0>();
          }
          fence_gpu();
        }
        __syncwarp();
      }
    }
    __syncthreads();  // the shared-memory tables are rewritten by the next chunk of groups
  }
}

// Grab the next batch of tokens; lane-uniform result.
__device__ __forceinline__ int grab_tokens(int* counter, int lane) {
  int b = 0;
  if (lane == 0) b = atomicAdd(counter, kTokenBatch);
  return __shfl_sync(0xffffffffu, b, 0);
}

// Store the K gate weights of a token next to the rows they belong to.
__device__ __forceinline__ void push_weights(const MoonepDevCtx& c, const DispatchArgs& a, int token, int lane, int dest,
                                             int loff) {
  if (a.weights != nullptr && lane < c.K) {
    float* w = reinterpret_cast<float*>(c.meta_peer[dest] + c.weights_off);
    w[loff] = a.weights[token * c.K + lane];
  }
}

// Lane `lane` < K holds routing entry d of a token whose copies are complete: release the flags of the rows
// this rank wrote (the token's primary row on every destination rank).
__device__ __forceinline__ void release_row_flags(const MoonepDevCtx& c, int d, int lane, int epoch) {
  __syncwarp();
  if (lane < c.K && d >= 0) {
    int dest, loff;
    decode_dst(d, c.NvS, dest, loff);
    if (dst_in_range(c, dest, loff)) {
      if (dest == c.rank)
        st_release_gpu(rowflag_ptr(c, dest, loff), epoch);  // only kernels of this GPU read it
      else
        st_release_sys(rowflag_ptr(c, dest, loff), epoch);
    }
  }
}

// ---- row flags off the copy path ----------------------------------------------------------------
//
// Releasing a row flag costs a system-scope fence, which would stall the lane that drives the bulk copies.
// Each bulk warp therefore hands the tokens whose copies have completed to a helper warp through a small
// queue in shared memory; the helper re-reads the token's routing entries and releases the flags.

constexpr int kFlagQ = 32;  // tokens a bulk warp may be ahead of its helper
// A row is flagged once its bulk group has completed at the destination, which takes several microseconds over
// NVLink; the copy loop therefore looks kFlagLag items back, so that the completion wait never stalls the issue of
// new copies (the shared-memory stages are recycled as soon as they have been read, as before).
constexpr int kFlagLag = 12;

struct FlagQueue {
  int lagged[kBulkWarps][kFlagLag + 4];  // token of every item in flight whose last piece it is, else -1
  int tok[kBulkWarps][kFlagQ];
  int head[kBulkWarps];  // tokens pushed so far (written by the bulk warp)
  int tail[kBulkWarps];  // tokens consumed so far (written by the helper)
  int done[kBulkWarps];  // 1 once the bulk warp has pushed its last token
};

__device__ __forceinline__ int lds_acquire(const int* p) {
  int v;
  asm volatile("ld.acquire.cta.shared::cta.s32 %0, [%1];" : "=r"(v) : "r"(smem_u32(p)) : "memory");
  return v;
}
__device__ __forceinline__ void sts_release(int* p, int v) {
  asm volatile("st.release.cta.shared::cta.s32 [%0], %1;" ::"r"(smem_u32(p)), "r"(v) : "memory");
}

// Bulk warp w, lane 0 only: the copies of `tok` are complete.
__device__ __forceinline__ bool flagq_push(const MoonepDevCtx& c, FlagQueue& q, int w, int& pushed, int tok) {
  if (pushed - lds_acquire(&q.tail[w]) >= kFlagQ) {
    const unsigned long long t0 = globaltimer_ns();
    unsigned spins = 0;
    while (pushed - lds_acquire(&q.tail[w]) >= kFlagQ) {
      if ((++spins & 255u) == 0 && (globaltimer_ns() - t0 > c.timeout_ns || poisoned(c))) return false;
    }
  }
  q.tok[w][pushed % kFlagQ] = tok;
  ++pushed;
  sts_release(&q.head[w], pushed);
  return true;
}

// Helper warp of bulk warp w: release the row flags of every token the bulk warp hands over.
__device__ void flag_helper(const MoonepDevCtx& c, const DispatchArgs& a, int epoch, FlagQueue& q, int w) {
  const int lane = threadIdx.x & 31;
  int consumed = 0;
  for (;;) {
    int avail = 0;
    if (lane == 0) {
      const unsigned long long t0 = globaltimer_ns();
      unsigned spins = 0;
      for (;;) {
        const int fin = lds_acquire(&q.done[w]);  // read before head: a token pushed before `done` is never missed
        avail = lds_acquire(&q.head[w]) - consumed;
        if (avail > 0) break;
        if (fin) {
          avail = -1;
          break;
        }
        if ((++spins & 255u) == 0 && (globaltimer_ns() - t0 > c.timeout_ns || poisoned(c))) {
          avail = -1;
          break;
        }
        __nanosleep(64);
      }
    }
    avail = __shfl_sync(0xffffffffu, avail, 0);
    if (avail <= 0) break;
    // A system-scope fence waits for everything this SM has in flight, so it is paid once per batch: lane 0
    // fences, then stores the flags of all tokens that have queued up meanwhile.
    if (lane == 0) fence_sys();
    for (int i = 0; i < avail; ++i, ++consumed) {
      const int tok = q.tok[w][consumed % kFlagQ];
      int* f = nullptr;
      if (lane < c.K) {
        const int d = a.dst[tok * c.K + lane];
        int dest, loff;
        decode_dst(d, c.NvS, dest, loff);
        if (d >= 0 && dst_in_range(c, dest, loff) && !(a.local_rows && dest == c.rank)) f = rowflag_ptr(c, dest, loff);
      }
      unsigned m = __ballot_sync(0xffffffffu, f != nullptr);
      while (m) {
        const int kk = __ffs(m) - 1;
        m &= m - 1;
        int* fk = reinterpret_cast<int*>(__shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(f), kk));
        if (lane == 0) st_relaxed_sys(fk, epoch);
      }
    }
    __syncwarp();
    if (lane == 0) sts_release(&q.tail[w], consumed);
  }
}

// ---- send role, register path ------------------------------------------------------------------

__device__ void send_ldst(const MoonepDevCtx& c, const DispatchArgs& a, int epoch) {
  const int lane = threadIdx.x & 31;
  int* work = c.counters + MOONEP_CTR_SEND_WORK;
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
      const bool mine = valid && d >= 0 && !(a.local_rows && dest == c.rank);  // a row this role writes
      const unsigned prim = __ballot_sync(0xffffffffu, mine);
      if (prim == 0) continue;
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
      release_row_flags(c, mine ? d : -1, lane, epoch);
    }
  }
}

// ---- send role, bulk-copy path -----------------------------------------------------------------

// Runs in warps 0..kBulkWarps-1 of a sender CTA.  s_ring: [kBulkWarps][kBulkStages][chunk_bytes],
// s_bar: [kBulkWarps][kBulkStages] initialised mbarriers (count 1).  Returns false after a timeout.
__device__ bool send_bulk(const MoonepDevCtx& c, const DispatchArgs& a, int epoch, unsigned char* s_ring,
                          unsigned long long* s_bar, FlagQueue& fq) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int* work = c.counters + MOONEP_CTR_SEND_WORK;
  const int H = c.H, K = c.K, S = c.S;
  const long long row_bytes = (long long)H * 2;
  unsigned char* ring = s_ring + (size_t)warp * kBulkStages * a.chunk_bytes;
  unsigned long long* bar = s_bar + warp * kBulkStages;
  int ring_tok[kBulkStages], ring_chunk[kBulkStages], ring_d[kBulkStages];
  int pushed = 0;  // lane 0: tokens handed to the helper warp
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
    if (a.local_rows && cur_chunk == 0) {
      // a token whose rows all stay on this rank is the EXPAND role's: only its gate weights are stored here
      for (;;) {
        int d = 0, dest = 0, loff = 0;
        bool valid = false;
        if (lane < K) {
          d = a.dst[batch_next * K + lane];
          decode_dst(d, c.NvS, dest, loff);
          valid = dst_in_range(c, dest, loff);
        }
        if (__ballot_sync(0xffffffffu, valid && d >= 0 && dest != c.rank) != 0) break;
        if (lane < K && !valid) record_status(c, MOONEP_STATUS_BAD_INDEX, MOONEP_K_DISPATCH_SEND, 6, d, batch_next, lane);
        if (valid) push_weights(c, a, batch_next, lane, dest, loff);
        if (++batch_next == batch_end) {
          const int b = grab_tokens(work, lane);
          if (b >= S) return false;
          batch_next = b;
          batch_end = min(S, b + kTokenBatch);
        }
      }
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
    const int d = lane < K ? a.dst[tok * K + lane] : 0;
#pragma unroll
    for (int q = 0; q < kBulkStages; ++q)
      if (q == s) {
        ring_tok[q] = tok;
        ring_chunk[q] = ch;
        ring_d[q] = d;
      }
    if (lane == 0) {
      fq.lagged[warp][loaded % (kFlagLag + 4)] = (ch == a.nchunks - 1) ? tok : -1;
      const unsigned len = chunk_len(ch);
      mbar_expect_tx(bar + s, len);
      bulk_g2s(ring + (size_t)s * a.chunk_bytes,
               reinterpret_cast<const unsigned char*>(a.hidden) + tok * row_bytes + (long long)ch * a.chunk_bytes, len,
               bar + s);
    }
    ++loaded;
  };
  // the stores of item j are complete: if it was the last piece of its token, the helper warp flags the token's rows
  auto flag_item = [&](int j) {
    if (lane == 0) {
      const int ftok = fq.lagged[warp][j % (kFlagLag + 4)];
      if (ftok >= 0 && !flagq_push(c, fq, warp, pushed, ftok)) {
        record_status(c, MOONEP_STATUS_TIMEOUT, MOONEP_K_DISPATCH_SEND, 101, warp, pushed, ftok);
        failed = true;  // lane 0 only; the loop condition below is evaluated after a warp-wide exchange
      }
    }
  };

  // Loads run two items ahead of the stores: while the stores of item n drain, the loads of n+1 and n+2 are in
  // flight, so an iteration does not wait a whole HBM latency for the row it is about to send.
  int tok, ch;
  for (int q = 0; q < kBulkStages - 1 && more; ++q) {
    more = next_item(tok, ch);
    if (more) issue_load(tok, ch);
  }
  while (done < loaded && !failed) {
    const int s = done % kBulkStages;
    int ctok = 0, cch = 0, d = 0;
#pragma unroll
    for (int q = 0; q < kBulkStages; ++q)
      if (q == s) {
        ctok = ring_tok[q];
        cch = ring_chunk[q];
        d = ring_d[q];
      }
    int dest = 0, loff = 0;
    bool valid = false;
    if (lane < K) {
      decode_dst(d, c.NvS, dest, loff);
      valid = dst_in_range(c, dest, loff);
      if (!valid) record_status(c, MOONEP_STATUS_BAD_INDEX, MOONEP_K_DISPATCH_SEND, 6, d, ctok, lane);
    }
    if (valid && cch == 0) push_weights(c, a, ctok, lane, dest, loff);
    unsigned m = __ballot_sync(0xffffffffu, valid && d >= 0 && !(a.local_rows && dest == c.rank));
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
    if (done > kFlagLag) {
      // all but the kFlagLag most recent groups have completed: item done-1-kFlagLag is in its destinations' memory
      if (lane == 0) bulk_wait<kFlagLag>();
      flag_item(done - 1 - kFlagLag);
      failed = __shfl_sync(0xffffffffu, failed ? 1 : 0, 0) != 0;
    }
    if (more && !failed) {
      more = next_item(tok, ch);
      if (more) {
        // the stage to refill held item done-2: every group but the one just committed has read its stage
        if (lane == 0) bulk_wait_read<1>();
        __syncwarp();
        issue_load(tok, ch);  // overwrites the `lagged` entry of item loaded-(kFlagLag+4), flagged long ago
      }
    }
  }
  if (lane == 0) bulk_wait<0>();
  __syncwarp();
  if (!failed)
    for (int j = done > kFlagLag ? done - kFlagLag : 0; j < done; ++j) flag_item(j);
  if (lane == 0) sts_release(&fq.done[warp], 1);
  __syncwarp();
  return !failed;
}

// ---- expand role ---------------------------------------------------------------------------------

// Copy the row at `src` (a row of the local shard, or of the dispatch's input) to the rows of the local shard that
// lane q holds in my_dup (q < dn), then flag them.
__device__ void expand_group(const MoonepDevCtx& c, const uint16_t* src, int my_dup, int dn, int vec_ok, int epoch,
                             int lane) {
  const int H = c.H;
  uint16_t* shard = c.hidden_peer[c.rank];
  if (vec_ok) {
    const int nvec = H / 8;
    const int4* s4 = reinterpret_cast<const int4*>(src);
    for (int c0 = 0; c0 < nvec; c0 += 32 * kExpandVec) {
      int4 v[kExpandVec];
#pragma unroll
      for (int j = 0; j < kExpandVec; ++j) {
        const int i = c0 + j * 32 + lane;
        if (i < nvec) v[j] = ld16(s4 + i);
      }
      for (int q = 0; q < dn && q < 32; ++q) {
        const int row = __shfl_sync(0xffffffffu, my_dup, q);
        if (row < 0 || row >= c.NvS) continue;
        int4* o4 = reinterpret_cast<int4*>(shard + (long long)row * H);
#pragma unroll
        for (int j = 0; j < kExpandVec; ++j) {
          const int i = c0 + j * 32 + lane;
          if (i < nvec) st16(o4 + i, v[j]);
        }
      }
    }
  } else {
    for (int q = 0; q < dn && q < 32; ++q) {
      const int row = __shfl_sync(0xffffffffu, my_dup, q);
      if (row < 0 || row >= c.NvS) continue;
      uint16_t* o = shard + (long long)row * H;
      for (int i = lane; i < H; i += 32) o[i] = src[i];
    }
  }
  // one fence for the group (a fence waits for everything the warp has in flight), then its rows' flags
  __syncwarp();
  if (lane == 0) fence_gpu();
  for (int q = 0; q < dn && q < 32; ++q) {
    const int row = __shfl_sync(0xffffffffu, my_dup, q);
    if (lane == 0 && row >= 0 && row < c.NvS) st_relaxed_gpu(c.meta_peer[c.rank] + c.rowflag_off + row, epoch);
  }
}

// Rows whose copies have been issued but not yet flagged (lane q holds the q-th row).
struct PendingRows {
  int dup, dn;
};

// Lane 0 has waited for the copies of `p` to complete: fence once, then release the rows' flags.
__device__ __forceinline__ void flag_pending(const MoonepDevCtx& c, const PendingRows& p, int epoch, int lane) {
  if (lane == 0) fence_gpu();
  for (int q = 0; q < p.dn && q < 32; ++q) {
    const int row = __shfl_sync(0xffffffffu, p.dup, q);
    if (lane == 0 && row >= 0 && row < c.NvS) st_relaxed_gpu(c.meta_peer[c.rank] + c.rowflag_off + row, epoch);
  }
}

// The same through shared memory with bulk copies: the row piece is loaded once into this warp's stage and stored to
// every duplicate row, no register traffic.  stage: chunk_bytes of shared memory of this warp; bar: its mbarrier
// (count 1), phase: its parity, flipped per use.  The rows of this group are flagged one group late (`pend`: the
// previous group's rows), so that waiting for the completion of a group's stores overlaps the next group's load;
// the caller flushes the last group with expand_flush().  Returns false after a timeout.
__device__ bool expand_group_bulk(const MoonepDevCtx& c, const unsigned char* src_row, int my_dup, int dn, int epoch,
                                  int lane, unsigned char* stage, int chunk_bytes, unsigned long long* bar,
                                  unsigned& phase, PendingRows& pend) {
  const long long row_bytes = (long long)c.H * 2;
  unsigned char* shard = reinterpret_cast<unsigned char*>(c.hidden_peer[c.rank]);
  bool ok = true;
  for (long long off = 0; off < row_bytes && ok; off += chunk_bytes) {
    const unsigned len = (unsigned)(row_bytes - off < chunk_bytes ? row_bytes - off : chunk_bytes);
    int got = 1;
    if (lane == 0) {
      bulk_wait_read<0>();  // the stage is free once the previous stores have read it
      mbar_expect_tx(bar, len);
      bulk_g2s(stage, src_row + off, len, bar);
      got = mbar_wait(bar, phase, c.timeout_ns) ? 1 : 0;
      if (!got) record_status(c, MOONEP_STATUS_TIMEOUT, MOONEP_K_DISPATCH_EXPAND, 100, dn, (int)off, 0);
    }
    phase ^= 1u;
    ok = __shfl_sync(0xffffffffu, got, 0) != 0;
    if (!ok) break;
    for (int q = 0; q < dn && q < 32; ++q) {
      const int row = __shfl_sync(0xffffffffu, my_dup, q);
      if (lane == 0 && row >= 0 && row < c.NvS) bulk_s2g(shard + (long long)row * row_bytes + off, stage, len);
    }
    if (lane == 0) bulk_commit();  // one bulk group per piece: the next piece waits for this one to have read the stage
  }
  if (row_bytes > chunk_bytes) {
    // rows of several pieces (several bulk groups): no lag, everything completes here
    if (lane == 0) bulk_wait<0>();
    if (pend.dn > 0) flag_pending(c, pend, epoch, lane);
    pend.dup = ok ? my_dup : -1;
    pend.dn = ok ? dn : 0;
    if (pend.dn > 0) flag_pending(c, pend, epoch, lane);
    pend.dn = 0;
    return ok;
  }
  if (pend.dn > 0) {
    if (lane == 0) bulk_wait<1>();  // everything but the group just committed has completed
    flag_pending(c, pend, epoch, lane);
  }
  pend.dup = ok ? my_dup : -1;
  pend.dn = ok ? dn : 0;
  return ok;
}

__device__ __forceinline__ void expand_flush(const MoonepDevCtx& c, PendingRows& pend, int epoch, int lane) {
  if (lane == 0) bulk_wait<0>();
  if (pend.dn > 0) flag_pending(c, pend, epoch, lane);
  pend.dn = 0;
}

// Work of this warp in the expansion: `count` entries, entry_of(k) >= 0 a duplicate group (its number), <= -2 a
// primary row without duplicates whose token lives on this rank (row -entry-2), -1 nothing.  With a.local_rows the
// rows whose source is this rank are written here, straight from the dispatch's input (the SEND role skips them): a
// group of such a token gets its primary row and its duplicates from one read of the input row, and nothing is
// waited for.  The other groups are expanded from their primary row in the order in which those rows arrive, not in
// list order: rows land in the senders' token order, which has nothing to do with the order of the rows in the
// shard, and a warp that sat on its first missing row would push all its copies to the end of the kernel.  Lanes poll
// the row flags of up to 32 pending entries per round; a round without progress sleeps, and the usual time limit
// applies to the whole wait.  info: src_info of the rows of this rank (entry src * NvS + token * K + k).
template <class EntryOf>
__device__ bool expand_as_rows_arrive(const MoonepDevCtx& c, const DispatchArgs& a, int count, EntryOf entry_of,
                                      const int* __restrict__ info, int epoch, int lane, bool bulk,
                                      unsigned char* my_stage, unsigned long long* my_bar, unsigned& xphase,
                                      PendingRows& pend) {
  const int* rowflag = c.meta_peer[c.rank] + c.rowflag_off;
  const int NvS = c.NvS;
  const long long row_bytes = (long long)c.H * 2;
  const unsigned char* shard = reinterpret_cast<const unsigned char*>(c.hidden_peer[c.rank]);
  const unsigned char* input = reinterpret_cast<const unsigned char*>(a.hidden);
  for (int k0 = 0; k0 < count; k0 += 32) {
    const int nk = min(32, count - k0);
    unsigned pending = nk == 32 ? 0xffffffffu : ((1u << nk) - 1u);
    unsigned long long t0 = 0;
    unsigned idle = 0;
    while (pending != 0) {
      // lane k looks at entry k0 + k: is it ready (its source row present)?
      int g = -1, primary = -1, token = -1;  // token >= 0: the source is row `token` of the input
      bool ready = false;
      if (lane < nk && ((pending >> lane) & 1u)) {
        const int e = entry_of(k0 + lane);
        if (e >= 0) {
          g = e;
          primary = a.dup_groups[3 * g];
        } else if (e <= -2) {
          primary = -e - 2;
        }
        if (primary < 0 || primary >= NvS) {
          g = primary = -1;
        } else if (a.local_rows && info != nullptr) {
          const int si = info[primary];
          if (si >= 0 && si / NvS == c.rank) token = (si % NvS) / c.K;
          if (token >= c.S) token = -1;
        }
        if (e <= -2 && token < 0) primary = -1;  // a lone row of another rank's token: nothing to do here
        ready = primary < 0 || token >= 0 || ld_acquire_sys(rowflag + primary) - epoch >= 0;
      }
      unsigned now = __ballot_sync(0xffffffffu, ready);
      if (now == 0) {
        if (idle++ == 0) {
          t0 = globaltimer_ns();
          if (bulk) expand_flush(c, pend, epoch, lane);  // nothing to copy: release the flags still held back
        }
        int give_up = 0;
        if (lane == 0 && (idle & 15u) == 0 && (globaltimer_ns() - t0 > c.timeout_ns || poisoned(c))) {
          const int k = __ffs(pending) - 1;
          record_status(c, MOONEP_STATUS_TIMEOUT, MOONEP_K_DISPATCH_EXPAND, 200, entry_of(k0 + k), epoch, (int)pending);
          give_up = 1;
        }
        if (__shfl_sync(0xffffffffu, give_up, 0)) return false;
        __nanosleep(256);
        continue;
      }
      idle = 0;
      pending &= ~now;
      while (now != 0) {
        const int k = __ffs(now) - 1;
        now &= now - 1;
        const int gk = __shfl_sync(0xffffffffu, g, k);
        const int pk = __shfl_sync(0xffffffffu, primary, k);
        const int tk = __shfl_sync(0xffffffffu, token, k);
        if (pk < 0) continue;
        int dn = 0, my_row = -1;
        if (gk >= 0) {
          const int ds = a.dup_groups[3 * gk + 1];
          dn = a.dup_groups[3 * gk + 2];
          if (ds < 0 || dn < 0 || dn >= 32 || ds + dn > NvS) continue;
          if (lane < dn) my_row = a.dup_loffs[ds + lane];
        }
        if (tk >= 0) {  // the primary row itself is written here as well
          if (lane == dn) my_row = pk;
          ++dn;
        }
        if (dn == 0) continue;
        const unsigned char* src = tk >= 0 ? input + (long long)tk * row_bytes : shard + (long long)pk * row_bytes;
        if (bulk) {
          if (!expand_group_bulk(c, src, my_row, dn, epoch, lane, my_stage, a.chunk_bytes, my_bar, xphase, pend)) return false;
        } else {
          expand_group(c, reinterpret_cast<const uint16_t*>(src), my_row, dn, a.vec_ok, epoch, lane);
        }
      }
    }
  }
  return true;
}

// xidx of xcnt expander CTAs.  Returns false after a failed wait.
//
// With a.expand_bulk the copies go through shared memory with bulk copies: warps 0..kExpandCopyWarps-1 own one piece
// of chunk_bytes each in s_dyn, followed by one piece of zeros that the zero fill stores from.
__device__ bool expand_role(const MoonepDevCtx& c, const DispatchArgs& a, int xidx, int xcnt, bool ok, unsigned char* s_dyn,
                            unsigned long long* s_xbar, int* s_scratch) {
  __shared__ int s_groups[kExpandSlice];  // group numbers found by this CTA in the current slice
  __shared__ int s_ngroups;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const bool bulk = a.expand_bulk != 0;
  const int copy_warps = bulk ? kExpandCopyWarps : nwarps;  // warps that expand groups
  unsigned char* my_stage = s_dyn + (size_t)warp * a.chunk_bytes;
  unsigned char* zeros = bulk ? s_dyn + (size_t)kExpandCopyWarps * a.chunk_bytes : nullptr;
  unsigned xphase = 0;
  PendingRows pend = {-1, 0};
  if (bulk) {
    for (int i = threadIdx.x; i < a.chunk_bytes / 16; i += blockDim.x)
      reinterpret_cast<int4*>(zeros)[i] = make_int4(0, 0, 0, 0);
    fence_proxy_async();
    __syncthreads();
  }
  const int NvS = c.NvS;
  const int epoch = abs_epoch(c, MOONEP_FLAG_SENT, a.epoch_sent);
  // zero_fill comes from the table stage of this dispatch when the planner ran on the device
  if (a.fresh && a.wait_family < 0)
    ok = wait_local_epoch(c, MOONEP_CTR_TABLES_READY, abs_epoch(c, MOONEP_FLAG_PLAN, a.epoch_plan),
                          MOONEP_K_DISPATCH_EXPAND) && ok;
  unsigned long long t0 = globaltimer_ns();
  if (ok && a.zero_fill != nullptr && !a.build_only)
    zero_fill_rows(c, a.zero_fill, a.with_weights, a.vec_ok, epoch, xidx * nwarps + warp, xcnt * nwarps, s_groups,
                   s_scratch, zeros, a.chunk_bytes);
  __syncthreads();
  if (threadIdx.x == 0) stat_phase(c, MOONEP_PH_ZERO, t0);
  t0 = globaltimer_ns();
  if (a.fresh) ok = block_wait_flags(c, MOONEP_FLAG_PLAN, a.epoch_plan, MOONEP_K_DISPATCH_EXPAND) && ok;
  if (threadIdx.x == 0) stat_phase(c, MOONEP_PH_WAIT_PLAN, t0);
  t0 = globaltimer_ns();
  if (ok && a.fresh) {
    // Every source pushed, next to src_info, a link word per landed row: whether the row is the first of its
    // (source, token) on this rank and which row holds the next entry of the same token.  A primary row that
    // has a successor opens a group; walking the chain lists its duplicates in ascending k.
    const int* src_info = c.meta_peer[c.rank] + c.src_info_off;
    const int* link = c.meta_peer[c.rank] + c.link_off;
    // rows past the last group are unused: the CTAs share the used part of the shard (and mark the rest as empty
    // in the plan's copies)
    int used = a.cu_seqlens != nullptr ? a.cu_seqlens[c.E + c.B - 1] : NvS;
    if (used < 0 || used > NvS) used = NvS;
    for (int loff = used + xidx * blockDim.x + threadIdx.x; loff < NvS; loff += xcnt * blockDim.x) {
      if (a.plan_src_info != nullptr) a.plan_src_info[loff] = -1;
      if (a.plan_link != nullptr) a.plan_link[loff] = 0;
    }
    const int per_cta = (used + xcnt - 1) / xcnt;
    const int lo = xidx * per_cta, hi = min(used, lo + per_cta);
    for (int s0 = lo; s0 < hi && ok; s0 += kExpandSlice) {
      const int s1 = min(hi, s0 + kExpandSlice);
      if (threadIdx.x == 0) s_ngroups = 0;
      __syncthreads();
      for (int base = s0; base < s1; base += blockDim.x) {  // uniform trip count: the ballots need whole warps
        const int loff = base + threadIdx.x;
        int dup_n = 0, first = -1;
        bool single = false;  // a primary row without duplicates whose token lives on this rank
        if (loff < s1) {
          const int si = src_info[loff];
          const int l = si >= 0 ? link[loff] : 0;
          if (a.plan_src_info != nullptr) a.plan_src_info[loff] = si;
          if (a.plan_link != nullptr) a.plan_link[loff] = l;
          single = a.local_rows && si >= 0 && (l & MOONEP_LINK_PRIMARY) && !(l & MOONEP_LINK_HAS_NEXT) &&
                   si / NvS == c.rank;
          if (si >= 0 && (l & MOONEP_LINK_PRIMARY) && (l & MOONEP_LINK_HAS_NEXT)) {
            first = l & MOONEP_NVS_MASK;
            int cur = first;
            while (dup_n < MOONEP_MAX_TOPK) {
              if (cur < 0 || cur >= NvS) {
                record_status(c, MOONEP_STATUS_BAD_INDEX, MOONEP_K_DISPATCH_EXPAND, 5, cur, loff, 0);
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
        const unsigned lone = __ballot_sync(0xffffffffu, single);
        if (lone != 0) {
          int sbase = 0;
          if (lane == 0) sbase = atomicAdd(&s_ngroups, __popc(lone));
          sbase = __shfl_sync(0xffffffffu, sbase, 0);
          if (single) s_groups[sbase + __popc(lone & ((1u << lane) - 1u))] = -loff - 2;
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
        int gbase = 0, dbase = 0, lbase = 0;
        if (lane == 0) {
          gbase = atomicAdd(a.dup_counts, __popc(has));
          dbase = atomicAdd(a.dup_counts + 1, total);
          lbase = atomicAdd(&s_ngroups, __popc(has));
        }
        gbase = __shfl_sync(0xffffffffu, gbase, 0);
        dbase = __shfl_sync(0xffffffffu, dbase, 0);
        lbase = __shfl_sync(0xffffffffu, lbase, 0);
        if (dup_n > 0) {
          const int before = __popc(has & ((1u << lane) - 1u));
          const int g = gbase + before;
          const int ds = dbase + incl - dup_n;
          if (g < NvS && ds + dup_n <= NvS) {
            a.dup_groups[3 * g] = loff;
            a.dup_groups[3 * g + 1] = ds;
            a.dup_groups[3 * g + 2] = dup_n;
            int cur = first;
            for (int q = 0; q < dup_n; ++q) {
              a.dup_loffs[ds + q] = cur;
              cur = link[cur] & MOONEP_NVS_MASK;
            }
            s_groups[lbase + before] = g;
          } else {
            s_groups[lbase + before] = -1;
          }
        }
      }
      __syncthreads();
      const int ng = a.build_only ? 0 : s_ngroups;
      if (ok && warp < copy_warps && warp < ng)
        ok = expand_as_rows_arrive(
            c, a, (ng - warp + copy_warps - 1) / copy_warps, [&](int k) { return s_groups[warp + k * copy_warps]; },
            src_info, epoch, lane, bulk, my_stage, s_xbar + warp, xphase, pend);
      if (bulk && warp < copy_warps) expand_flush(c, pend, epoch, lane);
      ok = __syncthreads_and(ok ? 1 : 0) != 0;
    }
  } else if (ok) {
    // replayed plan: the groups are in the plan
    int ngroups = a.dup_counts[0];
    if (ngroups < 0 || ngroups > NvS) ngroups = 0;
    const int g0 = xidx * copy_warps + warp, gstride = xcnt * copy_warps;
    if (warp < copy_warps && g0 < ngroups)
      ok = expand_as_rows_arrive(
          c, a, (ngroups - g0 + gstride - 1) / gstride, [&](int k) { return g0 + k * gstride; }, a.plan_src_info, epoch,
          lane, bulk, my_stage, s_xbar + warp, xphase, pend);
    if (a.local_rows && a.plan_src_info != nullptr && a.plan_link != nullptr) {
      // the lone primary rows of this rank's own tokens: found in the plan's copy of the link words, a slice of rows
      // per CTA and round
      const int per_cta = (NvS + xcnt - 1) / xcnt;
      const int lo = xidx * per_cta, hi = min(NvS, lo + per_cta);
      for (int s0 = lo; s0 < hi && ok; s0 += kExpandSlice) {
        const int s1 = min(hi, s0 + kExpandSlice);
        __syncthreads();
        if (threadIdx.x == 0) s_ngroups = 0;
        __syncthreads();
        for (int loff = s0 + threadIdx.x; loff < s1; loff += blockDim.x) {
          const int si = a.plan_src_info[loff];
          const int l = si >= 0 ? a.plan_link[loff] : 0;
          if (si >= 0 && (l & MOONEP_LINK_PRIMARY) && !(l & MOONEP_LINK_HAS_NEXT) && si / NvS == c.rank)
            s_groups[atomicAdd(&s_ngroups, 1)] = -loff - 2;
        }
        __syncthreads();
        const int ng = s_ngroups;
        if (ok && warp < copy_warps && warp < ng)
          ok = expand_as_rows_arrive(
              c, a, (ng - warp + copy_warps - 1) / copy_warps, [&](int k) { return s_groups[warp + k * copy_warps]; },
              a.plan_src_info, epoch, lane, bulk, my_stage, s_xbar + warp, xphase, pend);
        ok = __syncthreads_and(ok ? 1 : 0) != 0;
      }
    }
    if (bulk && warp < copy_warps) expand_flush(c, pend, epoch, lane);
    ok = __syncthreads_and(ok ? 1 : 0) != 0;
  }
  __syncthreads();
  if (threadIdx.x == 0) stat_phase(c, MOONEP_PH_BUILD_EXPAND, t0);
  t0 = globaltimer_ns();
  // the kernel ends when every row of the shard is present
  ok = block_wait_flags(c, MOONEP_FLAG_SENT, a.epoch_sent, MOONEP_K_DISPATCH_EXPAND) && ok;
  if (threadIdx.x == 0) stat_phase(c, MOONEP_PH_WAIT_SENT, t0);
  return ok;
}

// ---- the kernel ------------------------------------------------------------------------------------

__global__ void __launch_bounds__(kDispatchThreads, 1) dispatch_kernel(const MoonepDevCtx c_in, const DispatchArgs a) {
  extern __shared__ __align__(128) unsigned char s_dyn[];  // sender ring / planner tables / expert histogram
  __shared__ PeerTables s_peer;
  for (int r = threadIdx.x; r < c_in.R; r += blockDim.x) {
    s_peer.hidden[r] = c_in.hidden_peer[r];
    s_peer.meta[r] = c_in.meta_peer[r];
  }
  MoonepDevCtx c = c_in;  // same context, peer tables read from shared memory
  c.hidden_peer = s_peer.hidden;
  c.meta_peer = s_peer.meta;
  __shared__ __align__(8) unsigned long long s_bar[kBulkWarps * kBulkStages];
  __shared__ TokenScratch s_tok;
  __shared__ FlagQueue s_fq;
  __shared__ __align__(8) unsigned long long s_xbar[kExpandCopyWarps];
  const int roles = a.roles;
  const int warp = threadIdx.x >> 5;
  if (threadIdx.x < kBulkWarps * kBulkStages) mbar_init(s_bar + threadIdx.x, 1);
  if (threadIdx.x < kExpandCopyWarps) mbar_init(s_xbar + threadIdx.x, 1);
  if (threadIdx.x < kBulkWarps) {
    s_fq.head[threadIdx.x] = 0;
    s_fq.tail[threadIdx.x] = 0;
    s_fq.done[threadIdx.x] = 0;
  }
  fence_barrier_init();
  griddep_wait();  // the set-up above may overlap the previous kernel's tail; its results are needed from here on
  griddep_launch();  // the next kernel of the stream may set itself up on SMs as the CTAs of this one leave them
  __syncthreads();
  bool ok = !poisoned(c);

  if (a.publish) {
    // What plan_publish does as a kernel of its own, on all CTAs of this launch: reset this rank's src_info, push
    // the tokens-per-expert row into every peer's meta chunk, count the experts of every planner block; the last
    // CTA to finish signals FLAG_TPE to every peer (which also tells them that this rank is done with every
    // earlier use of the buffers).
    ok = __syncthreads_and(ok ? 1 : 0) != 0;  // one answer per CTA: the loops below contain barriers
    if (ok) {
      const int tid = blockIdx.x * blockDim.x + threadIdx.x;
      const int nth = gridDim.x * blockDim.x;
      int* src_info = c.meta_peer[c.rank] + c.src_info_off;
      for (int i = tid; i < c.NvS; i += nth) src_info[i] = -1;
      if (a.tpe_row != nullptr) {
        const int total = c.R * c.E;
        for (int i = tid; i < total; i += nth) {
          const int d = i / c.E;
          const int e = i - d * c.E;
          c.meta_peer[d][c.tpe_off + c.rank * c.E + e] = a.tpe_row[e];
        }
      }
      int* s_hist = reinterpret_cast<int*>(s_dyn);
      const int E = c.E;
      for (int b = blockIdx.x; b < a.n_blocks; b += gridDim.x) {
        for (int e = threadIdx.x; e < E; e += blockDim.x) s_hist[e] = 0;
        __syncthreads();
        const int start = b * a.tokens_per_block * c.K;
        const int end = min(c.N, start + a.tokens_per_block * c.K);
        for (int i = start + threadIdx.x; i < end; i += blockDim.x) {
          const int e = a.topk[i];
          if (e >= 0 && e < E) atomicAdd(s_hist + e, 1);
        }
        __syncthreads();
        int* out = c.block_hist + (long long)b * E;
        for (int e = threadIdx.x; e < E; e += blockDim.x) out[e] = s_hist[e];
        __syncthreads();
      }
    }
    if (role_tail(c, MOONEP_CTR_PUBLISH_ARRIVE, gridDim.x) && ok && !poisoned(c)) {
      const int tpe_epoch = abs_epoch(c, MOONEP_FLAG_TPE, a.epoch_tpe);
      for (int r = threadIdx.x; r < c.R; r += blockDim.x) st_release_sys(flag_ptr(c, r, MOONEP_FLAG_TPE, c.rank), tpe_epoch);
    }
    __syncthreads();
  }

  // which roles this CTA plays
  const bool mixed = (roles & MOONEP_ROLE_EXPAND) && (roles & (MOONEP_ROLE_TOKENS | MOONEP_ROLE_SEND));
  const int s0 = (mixed && (roles & MOONEP_ROLE_TABLES)) ? 1 : 0;
  bool is_sender = (roles & (MOONEP_ROLE_TOKENS | MOONEP_ROLE_SEND)) != 0;
  bool is_expander = (roles & MOONEP_ROLE_EXPAND) != 0;
  int scnt = gridDim.x, xidx = blockIdx.x, xcnt = gridDim.x;
  if (mixed) {
    is_sender = (int)blockIdx.x >= s0 && (int)blockIdx.x < s0 + a.n_send;
    is_expander = !is_sender;
    scnt = a.n_send;
    xidx = (int)blockIdx.x < s0 ? blockIdx.x : blockIdx.x - a.n_send;
    xcnt = gridDim.x - a.n_send;
  }
  const int plan_epoch = abs_epoch(c, MOONEP_FLAG_PLAN, a.epoch_plan);

  if ((roles & MOONEP_ROLE_TABLES) && blockIdx.x == 0) {
    const unsigned long long t0 = globaltimer_ns();
    ok = block_wait_flags(c, MOONEP_FLAG_TPE, a.epoch_tpe, MOONEP_K_PLAN_TABLES) && ok;
    if (ok) {
      TablesIO io;
      io.tpe = a.tpe2d != nullptr ? a.tpe2d : (c.meta_peer[c.rank] + c.tpe_off);
      io.R = c.R, io.E = c.E, io.B = c.B, io.epn = c.epn, io.cap = c.N, io.P = c.token_padding, io.rank = c.rank;
      io.NvS = c.NvS;
      io.cu_out = a.cu_seqlens, io.etc_out = a.experts_to_copy, io.zf_out = a.zero_fill, io.rs_out = a.remote_stats;
      io.tpe_prev = c.tpe_prev, io.alloc_cum = c.alloc_cum, io.expert_off = c.expert_off;
      const int bad = plan_tables_body(io, carve(a.tables_in_smem ? reinterpret_cast<int*>(s_dyn) : c.tables, c.R, c.E));
      if (threadIdx.x == 0) {
        if (a.dup_counts != nullptr) {
          a.dup_counts[0] = 0;
          a.dup_counts[1] = 0;
        }
        if (bad) record_status(c, MOONEP_STATUS_BAD_INDEX, MOONEP_K_PLAN_TABLES, 1, bad, c.NvS, 0);
      }
      __syncthreads();
      if (threadIdx.x == 0) {
        __threadfence();
        st_release_gpu(c.counters + MOONEP_CTR_TABLES_READY, plan_epoch);
        stat_phase(c, MOONEP_PH_TABLES, t0);
      }
    }
  }

  if (roles & MOONEP_ROLE_TOKENS) {
    // every CTA of the launch plans blocks of tokens (the expanders have nothing else to do yet)
    ok = wait_local_epoch(c, MOONEP_CTR_TABLES_READY, plan_epoch, MOONEP_K_PLAN_TOKENS) && ok;
    const unsigned long long t0 = globaltimer_ns();
    if (ok)
      for (int b = blockIdx.x; b < a.n_blocks; b += gridDim.x)
        plan_tokens_block(c, a.topk, a.dst, a.tokens_per_block, b, reinterpret_cast<int*>(s_dyn), s_tok);
    if (threadIdx.x == 0 && (int)blockIdx.x < a.n_blocks) stat_phase(c, MOONEP_PH_TOKENS, t0);
    if (role_tail(c, MOONEP_CTR_PLAN_ARRIVE, gridDim.x) && !poisoned(c)) {
      if (threadIdx.x == 0) st_release_gpu(c.counters + MOONEP_CTR_PLAN_DONE, plan_epoch);
      for (int r = threadIdx.x; r < c.R; r += blockDim.x) st_release_sys(flag_ptr(c, r, MOONEP_FLAG_PLAN, c.rank), plan_epoch);
    }
  }

  if (is_sender && (roles & MOONEP_ROLE_SEND)) {
    // a plan made on the device by this dispatch: every sender CTA must have planned its tokens; otherwise
    // (replayed plan, plan made on the host) whatever cross-rank flag the caller named
    if (a.fresh && a.wait_family < 0)
      ok = wait_local_epoch(c, MOONEP_CTR_PLAN_DONE, plan_epoch, MOONEP_K_DISPATCH_SEND) && ok;
    else
      ok = block_wait_flags(c, a.wait_family, a.wait_epoch, MOONEP_K_DISPATCH_SEND) && ok;
    const int epoch = abs_epoch(c, MOONEP_FLAG_SENT, a.epoch_sent);
    const unsigned long long t_send = globaltimer_ns();
    if (ok) {
      if (a.bulk) {
        if (warp < kBulkWarps)
          send_bulk(c, a, epoch, s_dyn, s_bar, s_fq);
        else if (warp < 2 * kBulkWarps)
          flag_helper(c, a, epoch, s_fq, warp - kBulkWarps);
      } else {
        send_ldst(c, a, epoch);
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) stat_phase(c, MOONEP_PH_SEND, t_send);
    if (role_tail(c, MOONEP_CTR_SEND_ARRIVE, scnt)) {
      if (threadIdx.x == 0) c.counters[MOONEP_CTR_SEND_WORK] = 0;
      if (ok && !poisoned(c))
        for (int r = threadIdx.x; r < c.R; r += blockDim.x) st_release_sys(flag_ptr(c, r, MOONEP_FLAG_SENT, c.rank), epoch);
    }
  }

  // the token stage's scratch (>= kZfChunk words) is free by now: the zero fill keeps its tables there
  static_assert(sizeof(TokenScratch) >= kZfChunk * sizeof(int) && kExpandSlice >= kZfChunk, "scratch too small");
  if (is_expander) expand_role(c, a, xidx, xcnt, ok, s_dyn, s_xbar, reinterpret_cast<int*>(&s_tok));
}

}  // namespace

}  // namespace moonep

using namespace moonep;

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// One launch of the dispatch kernel with the given roles (see the head of this file).
//   fresh != 0: topk/tpe2d/dst/cu_seqlens/experts_to_copy/zero_fill/remote_stats are the planner's inputs and
//   outputs and the duplicate map is (re)built; fresh == 0: dst, zero_fill and the duplicate map come from a plan.
//   n_send: sender CTAs (num_sms of the Buffer when <= 0); n_expand: expander CTAs (as many as fit when <= 0).
extern "C" int moonep_dispatch(void* ctx, int roles, int fresh, const int* topk, const int* tpe2d, int* dst,
                               int* cu_seqlens, int* experts_to_copy, int* zero_fill, int* remote_stats,
                               const void* hidden, const float* weights, int with_weights, int* dup_groups,
                               int* dup_loffs, int* dup_counts, int* plan_src_info, int* plan_link, int wait_family,
                               int wait_epoch, int epoch_tpe, int epoch_plan, int epoch_sent, int path, int n_send,
                               int n_expand, int build_only, const int* tpe_row, void* stream) {
  auto* h = (HostCtx*)ctx;
  const MoonepDevCtx& c = h->dev;
  DispatchArgs a;
  a.topk = topk;
  a.tpe2d = tpe2d;
  a.dst = dst;
  a.cu_seqlens = cu_seqlens;
  a.experts_to_copy = experts_to_copy;
  a.zero_fill = zero_fill;
  a.remote_stats = remote_stats;
  a.tokens_per_block = imax(1, MOONEP_PLAN_BLOCK / c.K);
  a.n_blocks = (c.S + a.tokens_per_block - 1) / a.tokens_per_block;
  a.hidden = (const uint16_t*)hidden;
  a.weights = weights;
  a.dup_groups = dup_groups;
  a.dup_loffs = dup_loffs;
  a.dup_counts = dup_counts;
  a.plan_src_info = plan_src_info;
  a.plan_link = plan_link;
  a.fresh = fresh;
  // the modifier needs the input rows in the EXPAND launch and src_info of the landed rows
  a.local_rows = ((roles & MOONEP_ROLE_LOCAL_ROWS) && hidden != nullptr && !build_only &&
                  (fresh || (plan_src_info != nullptr && plan_link != nullptr))) ? 1 : 0;
  roles &= ~MOONEP_ROLE_LOCAL_ROWS;
  a.publish = ((roles & MOONEP_ROLE_PUBLISH) && (roles & MOONEP_ROLE_TOKENS) && topk != nullptr) ? 1 : 0;
  roles &= ~MOONEP_ROLE_PUBLISH;
  a.tpe_row = tpe_row;
  a.roles = roles;
  a.build_only = build_only;
  a.with_weights = with_weights;
  a.wait_family = wait_family;
  a.wait_epoch = wait_epoch;
  a.epoch_tpe = epoch_tpe;
  a.epoch_plan = epoch_plan;
  a.epoch_sent = epoch_sent;
  a.vec_ok = (c.H % 8 == 0) && (hidden == nullptr || aligned16(hidden));
  const long long row_bytes = (long long)c.H * 2;
  a.nchunks = (int)((row_bytes + kMaxChunkBytes - 1) / kMaxChunkBytes);
  const long long cb = (row_bytes + a.nchunks - 1) / a.nchunks;
  a.chunk_bytes = (int)((cb + 15) / 16 * 16);

  // dynamic shared memory: the senders' ring, the table stage's work area, the token stage's histogram
  size_t smem = 0;
  const size_t ring_bytes = (size_t)kBulkWarps * kBulkStages * a.chunk_bytes;
  const size_t limit = (size_t)imax(0, h->max_smem_optin - 20 * 1024);  // static arrays take about 17 KB
  a.bulk = (path == MOONEP_PATH_BULK && a.vec_ok && ring_bytes <= limit) ? 1 : 0;
  if ((roles & MOONEP_ROLE_SEND) && a.bulk) smem = ring_bytes;
  const size_t expand_bytes = (size_t)(kExpandCopyWarps + 1) * a.chunk_bytes;
  // duplicate expansion and zero fill go through shared memory with bulk copies; MOONEP_EXPAND_PATH=ldst selects the
  // register copies (measured on one B200, S=4096: 0.343 vs 0.359 ms per round trip; both are bound by HBM writes)
  const char* xp = getenv("MOONEP_EXPAND_PATH");
  const bool want_bulk = !(xp != nullptr && strcmp(xp, "ldst") == 0);
  a.expand_bulk = (want_bulk && (roles & MOONEP_ROLE_EXPAND) && a.vec_ok && a.chunk_bytes % 16 == 0 && expand_bytes <= limit) ? 1 : 0;
  if (a.expand_bulk && expand_bytes > smem) smem = expand_bytes;
  a.tables_in_smem = 0;
  if (roles & MOONEP_ROLE_TABLES) {
    const size_t tb = (size_t)table_words(c.R, c.E) * sizeof(int);
    if (tb <= limit) {
      a.tables_in_smem = 1;
      if (tb > smem) smem = tb;
    }
  }
  if (roles & MOONEP_ROLE_TOKENS) {
    const size_t hb = (size_t)c.E * sizeof(int);
    if (hb > limit) {
      set_error("moonep_dispatch: E too large for the shared-memory histogram of the token stage");
      return 1;
    }
    if (hb > smem) smem = hb;
  }
  // The attribute belongs to the kernel, not to the launch, and emulated ranks launch from several threads with
  // different sizes: always allow the same maximum, so that no thread lowers it under another one's launch.
  if (int rc = check_cuda(cudaFuncSetAttribute(dispatch_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)limit),
                          "cudaFuncSetAttribute(dispatch_kernel)"))
    return rc;

  const bool senders = (roles & (MOONEP_ROLE_TOKENS | MOONEP_ROLE_SEND)) != 0;
  const bool expanders = (roles & MOONEP_ROLE_EXPAND) != 0;
  int grid = 1;
  a.n_send = 0;
  if (senders) {
    a.n_send = imax(1, imin(n_send > 0 ? n_send : c.num_sms, h->sm_count - (expanders ? 2 : 0)));
    // a single rank whose rows are all written by the EXPAND role: the senders only store gate weights
    if (c.R == 1 && a.local_rows && expanders) a.n_send = imin(a.n_send, 4);
    grid = a.n_send;
  }
  if (expanders) {
    const int room = imax(1, imin(c.local_sms, h->sm_count) - a.n_send);
    const int nx = n_expand > 0 ? imin(n_expand, room) : room;
    grid = a.n_send + imax(1, nx);
  }
  if (int rc = check_cuda(launch_maybe_pdl(dispatch_kernel, grid, kDispatchThreads, smem, (cudaStream_t)stream,
                                           h->enable_pdl != 0, c, a),
                          "launch dispatch_kernel"))
    return rc;
  return check_launch("dispatch_kernel");
}
