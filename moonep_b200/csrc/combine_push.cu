// Push combine for sm_100a: the rank that ran the experts folds each token's duplicate rows and
// pushes the result to the token's home rank over NVLink; the home rank sums the rows of a token as
// they arrive.  One kernel, three roles:
//
//   FOLD  (expert side, the CTAs that do not drive NVLink) duplicate groups of the plan are handed out from an
//         atomic counter; a warp adds the rows of a group (primary, then duplicates in ascending k) in fp32,
//         rounds to bf16 into a local buffer and releases the group's flag.  These CTAs then take the SUM role.
//   PUSH  (expert side, num_sms CTAs, pure copy engines) every primary row of the local expert output - as it
//         is when it has no duplicates, from the FOLD role's buffer otherwise - goes through a shared-memory
//         ring (cp.async.bulk global -> shared -> the home rank's staging chunk, slot (token, position of this
//         rank among the token's destinations)).  The gate weights of all of the token's entries on this rank
//         go to the home rank's weight staging.  Helper warps release the slot's flag with the combine's COMB
//         epoch once the row's bulk group has completed.
//   SUM   (home side) tokens are handed out from an atomic counter; a warp waits (bounded) for the flags of the
//         token's primaries, adds the staged rows in fp32 in ascending k, stores the bf16 result and copies the
//         K gate weights into the [S, K] output.
//
// Compared with pulling (combine.cu) the fold overlaps the transfers instead of preceding them, every NVLink
// transfer is a bulk store (which measured faster than loads from peer memory), and the home-side sum overlaps
// the transfers too.  Numerics are those of the pull path and of the reference: duplicates are added in fp32 and
// rounded to bf16, the per-token sum is fp32 rounded to bf16.  The expert output rows are not modified.
//
// CTA order in a launch with all roles: FOLD/SUM CTAs first, PUSH CTAs last, so that the PUSH role only waits
// for lower-numbered CTAs (which the hardware dispatches first) and the SUM role only for PUSH CTAs of this or
// other GPUs; the grid never exceeds the number of SMs.  Emulated ranks that share one GPU launch the roles one
// after the other.  With a single rank the FOLD role alone writes the results.
//
// Parity: reference moonep_td/combine_prologue.py:19-40 and moonep_td/combine.py:22-68.
#include <cstdlib>

#include "common.cuh"
#include "host.h"

namespace moonep {

namespace {

constexpr int kPushThreads = 512;
constexpr int kPushMaxChunk = 8192;     // bytes of a row piece (one ring stage): 8 warps x 3 stages x 7 KB for H=7168
constexpr int kPushRowBatch = 32;       // rows handed out per grab (the primaries without duplicates among them are sent)
constexpr int kPushGroupBatch = 8;      // duplicate groups handed out per grab
constexpr int kFoldRowBatch = 4;        // rows per work item when the FOLD role copies rows without duplicates: rows of one
                                        // source rank are neighbours in the shard, so a large batch would hand one warp
                                        // dozens of copies in a row
constexpr int kFoldVec = 4;             // int4 per lane per inner step (2 KB per warp)
constexpr int kFoldRows = 4;            // rows of a duplicate group whose loads are in flight together
constexpr int kSumVec = 4;
constexpr int kSumRows = 4;

struct PushArgs {
  const int* src_info;      // [NvS] plan copy: src_rank*NvS + slot, or -1
  const int* link;          // [NvS] plan copy of the link words
  const int* dst;           // [N]
  const uint16_t* in_rows;  // [NvS, H] expert output rows (local)
  const float* in_w;        // [NvS] or null
  uint16_t* out;            // [S, H]
  float* out_w;             // [S, K] or null
  int roles, n_push;
  int wait_family, wait_epoch;  // PUSH: peers are done with their previous use of the staging chunks
  int epoch_comb;
  int vec_ok, chunk_bytes, nchunks;
  const int* ready;         // optional: per 128-row block of in_rows, a counter the producer of the rows bumps
  int ready_expect;         // value a block's counter reaches when all of its rows are final
  const int* dup_groups;    // [NvS, 3] the plan's duplicate groups
  const int* dup_loffs;     // [NvS]
  const int* dup_counts;    // [2]
  uint16_t* fold_buf;       // [fold_rows, H] local: folded row of every duplicate group
  int* fold_flag;           // [fold_rows] local: COMB epoch of the combine that last folded the group
  int fold_rows;
  int direct;               // single rank: FOLD writes the results straight into out / out_w
  int local_home;           // rows of this rank's own tokens go from FOLD straight into the local staging chunk
  int sum_two;              // SUM: a warp holds two tokens and sums the one that completes first
};

__device__ __forceinline__ void acc_add(float* acc, const int4& v) {
  acc[0] += bf16lo((unsigned)v.x);
  acc[1] += bf16hi((unsigned)v.x);
  acc[2] += bf16lo((unsigned)v.y);
  acc[3] += bf16hi((unsigned)v.y);
  acc[4] += bf16lo((unsigned)v.z);
  acc[5] += bf16hi((unsigned)v.z);
  acc[6] += bf16lo((unsigned)v.w);
  acc[7] += bf16hi((unsigned)v.w);
}

__device__ __forceinline__ int4 acc_pack(const float* acc) {
  int4 o;
  o.x = (int)pack_bf16(acc[0], acc[1]);
  o.y = (int)pack_bf16(acc[2], acc[3]);
  o.z = (int)pack_bf16(acc[4], acc[5]);
  o.w = (int)pack_bf16(acc[6], acc[7]);
  return o;
}

__device__ __forceinline__ float bf16_to_f32(uint16_t u) { return __uint_as_float(((unsigned)u) << 16); }
__device__ __forceinline__ uint16_t f32_to_bf16(float f) {
  __nv_bfloat16 b = __float2bfloat16_rn(f);
  return *reinterpret_cast<uint16_t*>(&b);
}

// Warp-wide bounded wait until the producer of in_rows has finished the 128-row block of `row`.
__device__ bool wait_block_ready(const MoonepDevCtx& c, const PushArgs& a, int row, int lane) {
  if (a.ready == nullptr) return true;
  int ok = 1;
  if (lane == 0) {
    const int* f = a.ready + (row >> 7);
    if (ld_acquire_gpu(f) - a.ready_expect < 0) {
      const unsigned long long t0 = globaltimer_ns();
      unsigned spins = 0;
      int v;
      while ((v = ld_acquire_gpu(f)) - a.ready_expect < 0) {
        if ((++spins & 63u) == 0 && (globaltimer_ns() - t0 > c.timeout_ns || poisoned(c))) {
          record_status(c, MOONEP_STATUS_TIMEOUT, MOONEP_K_COMBINE_PUSH, 201, row >> 7, a.ready_expect, v);
          ok = 0;
          break;
        }
        __nanosleep(256);
      }
    }
  }
  return __shfl_sync(0xffffffffu, ok, 0) != 0;
}

// ---- PUSH role -------------------------------------------------------------------------------------

// Rows of one duplicate group, one per lane: lane 0 the primary, lanes 1..dn the duplicates in ascending k.
// Returns -1 in every lane (after recording a status) when the plan's lists are inconsistent.
__device__ __forceinline__ int group_rows(const MoonepDevCtx& c, const PushArgs& a, int g, int lane, int& prow, int& dn,
                                          int kernel_id) {
  prow = a.dup_groups[3 * g];
  const int ds = a.dup_groups[3 * g + 1];
  dn = a.dup_groups[3 * g + 2];
  bool bad = prow < 0 || prow >= c.NvS || ds < 0 || dn < 1 || dn >= MOONEP_MAX_TOPK || ds + dn > c.NvS;
  int my_row = -1;
  if (!bad) {
    if (lane == 0) my_row = prow;
    else if (lane <= dn) my_row = a.dup_loffs[ds + lane - 1];
    bad = __any_sync(0xffffffffu, lane <= dn && (my_row < 0 || my_row >= c.NvS)) != 0;
  }
  if (bad) {
    record_status(c, MOONEP_STATUS_BAD_INDEX, kernel_id, 9, prow, ds, dn);
    return -1;
  }
  return my_row;
}

// ---- FOLD role ---------------------------------------------------------------------------------------

// Duplicate groups are handed out from an atomic counter; a warp adds the rows of a group in fp32 (primary first,
// then the duplicates in ascending k), rounds to bf16 and stores the row into fold_buf[g] (or, with a single rank,
// straight into the token's output row), then releases fold_flag[g] for the PUSH role.
__device__ void fold_role(const MoonepDevCtx& c, const PushArgs& a) {
  const int lane = threadIdx.x & 31;
  const int NvS = c.NvS, K = c.K, H = c.H, S = c.S;
  const long long row_bytes = (long long)H * 2;
  const int epoch = abs_epoch(c, MOONEP_FLAG_COMB, a.epoch_comb);
  int* work = c.counters + MOONEP_CTR_FOLD_WORK;
  int ngroups = a.dup_counts[0];
  if (ngroups < 0 || ngroups > a.fold_rows) {
    if (ngroups > a.fold_rows) record_status(c, MOONEP_STATUS_BAD_INDEX, MOONEP_K_COMBINE_PUSH, 10, ngroups, a.fold_rows, 0);
    ngroups = 0;
  }
  // with a single rank this role also copies the rows that have no duplicates to the output; with local_home it
  // copies those of this rank's own tokens into the local staging chunk (the PUSH role leaves them out)
  const int nbatches = (a.direct || a.local_home) ? (NvS + kFoldRowBatch - 1) / kFoldRowBatch : 0;
  unsigned char* stage_local = a.local_home ? c.stage_peer[c.rank] : nullptr;
  for (;;) {
    int item = 0;
    if (lane == 0) item = atomicAdd(work, 1);
    item = __shfl_sync(0xffffffffu, item, 0);
    if (item >= ngroups + nbatches) break;
    if (item >= ngroups) {
      // single rank: rows without duplicates go to the output as they are
      const int base = (item - ngroups) * kFoldRowBatch;
      int si = -1, l = 0;
      if (lane < kFoldRowBatch && base + lane < NvS) {
        si = a.src_info[base + lane];
        l = si >= 0 ? a.link[base + lane] : 0;
      }
      unsigned prim = __ballot_sync(0xffffffffu, si >= 0 && (l & MOONEP_LINK_PRIMARY) && !(l & MOONEP_LINK_HAS_NEXT));
      while (prim) {
        const int j = __ffs(prim) - 1;
        prim &= prim - 1;
        const int p_si = __shfl_sync(0xffffffffu, si, j);
        const int p_l = __shfl_sync(0xffffffffu, l, j);
        const int slot = p_si % NvS;
        if (slot >= S * K) continue;
        const int prow = base + j;
        uint16_t* o = nullptr;
        int* sflag = nullptr;
        if (a.direct) {
          o = a.out + (long long)(slot / K) * H;
        } else {
          // local_home: only the rows of this rank's own tokens; slot (token, position among the token's primaries)
          const int ord = (p_l >> MOONEP_LINK_ORD_SHIFT) & MOONEP_LINK_ORD_MASK;
          if (p_si / NvS != c.rank || ord >= c.kp) continue;
          const long long stage_row = (long long)(slot / K) * c.kp + ord;
          o = reinterpret_cast<uint16_t*>(stage_local + stage_row * row_bytes);
          sflag = reinterpret_cast<int*>(stage_local + c.stage_flag_off) + stage_row;
        }
        if (!wait_block_ready(c, a, prow, lane)) return;
        if (a.in_w != nullptr && lane == 0) {
          if (a.direct) {
            if (a.out_w != nullptr) a.out_w[slot] = a.in_w[prow];
          } else {
            reinterpret_cast<float*>(stage_local + c.stage_w_off)[slot] = a.in_w[prow];
          }
        }
        const uint16_t* src = a.in_rows + (long long)prow * H;
        if (a.vec_ok) {
          // kFoldVec loads in flight per lane: a plain load-store loop would run one 16-byte round trip at a time
          const int nvec = H / 8;
          const int4* s4 = reinterpret_cast<const int4*>(src);
          int4* o4 = reinterpret_cast<int4*>(o);
          for (int i0 = 0; i0 < nvec; i0 += 32 * kFoldVec) {
            int4 v[kFoldVec];
#pragma unroll
            for (int jv = 0; jv < kFoldVec; ++jv) {
              const int i = i0 + jv * 32 + lane;
              if (i < nvec) v[jv] = ld16(s4 + i);
            }
#pragma unroll
            for (int jv = 0; jv < kFoldVec; ++jv) {
              const int i = i0 + jv * 32 + lane;
              if (i < nvec) st16(o4 + i, v[jv]);
            }
          }
        } else {
          for (int i = lane; i < H; i += 32) o[i] = src[i];
        }
        if (sflag != nullptr) {
          __syncwarp();
          if (lane == 0) {
            fence_gpu();
            st_relaxed_gpu(sflag, epoch);
          }
        }
      }
      continue;
    }
    int prow, dn;
    const int my_row = group_rows(c, a, item, lane, prow, dn, MOONEP_K_COMBINE_PUSH);
    if (__shfl_sync(0xffffffffu, my_row, 0) < 0) continue;
    const int n_rows = 1 + dn;
    // the producer of the rows (a grouped GEMM running beside this kernel) must be done with every block involved
    if (a.ready != nullptr) {
      bool ok = true;
      for (int q = 0; q < n_rows && ok; ++q) ok = wait_block_ready(c, a, __shfl_sync(0xffffffffu, my_row, q), lane);
      if (!ok) return;
    }
    uint16_t* o = a.fold_buf + (long long)item * H;
    int* sflag = nullptr;  // local_home and a token of this rank: the folded row goes straight into the local staging
    if (a.local_home) {
      const int p_si = a.src_info[prow];
      if (p_si >= 0 && p_si / NvS == c.rank) {
        const int slot = p_si - c.rank * NvS;
        const int ord = (a.link[prow] >> MOONEP_LINK_ORD_SHIFT) & MOONEP_LINK_ORD_MASK;
        if (slot >= S * K || ord >= c.kp) {
          record_status(c, MOONEP_STATUS_BAD_INDEX, MOONEP_K_COMBINE_PUSH, 8, p_si, prow, ord);
          continue;
        }
        const long long stage_row = (long long)(slot / K) * c.kp + ord;
        o = reinterpret_cast<uint16_t*>(stage_local + stage_row * row_bytes);
        sflag = reinterpret_cast<int*>(stage_local + c.stage_flag_off) + stage_row;
      }
    }
    if (!a.direct && a.in_w != nullptr && lane < n_rows) {
      // gate weights of all entries of this group travel to the home rank's weight staging
      const int s_q = a.src_info[my_row];
      const int home = a.src_info[prow] / NvS;
      const int slot_q = s_q - home * NvS;
      if (s_q >= 0 && home >= 0 && home < c.R && slot_q >= 0 && slot_q < S * K)
        reinterpret_cast<float*>(c.stage_peer[home] + c.stage_w_off)[slot_q] = a.in_w[my_row];
    }
    if (a.direct) {
      const int p_si = a.src_info[prow];
      const int slot = p_si % NvS;
      if (p_si < 0 || slot >= S * K) {
        record_status(c, MOONEP_STATUS_BAD_INDEX, MOONEP_K_COMBINE_PUSH, 8, p_si, prow, 0);
        continue;
      }
      o = a.out + (long long)(slot / K) * H;
      if (a.in_w != nullptr && a.out_w != nullptr && lane < n_rows) {
        const int s_q = a.src_info[my_row];
        if (s_q >= 0 && s_q % NvS < S * K) a.out_w[s_q % NvS] = a.in_w[my_row];
      }
    }
    if (a.vec_ok) {
      const int nvec = H / 8;
      for (int v0 = 0; v0 < nvec; v0 += 32 * kFoldVec) {
        float acc[kFoldVec][8];
#pragma unroll
        for (int jv = 0; jv < kFoldVec; ++jv)
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[jv][e] = 0.f;
        // loads of up to kFoldRows rows are issued before the first add
        for (int q0 = 0; q0 < n_rows; q0 += kFoldRows) {
          int4 dv[kFoldRows][kFoldVec];
#pragma unroll
          for (int r = 0; r < kFoldRows; ++r) {
            const int row = __shfl_sync(0xffffffffu, my_row, (q0 + r) & 31);
            if (q0 + r < n_rows) {
              const int4* r4 = reinterpret_cast<const int4*>(reinterpret_cast<const unsigned char*>(a.in_rows) +
                                                              (long long)row * row_bytes);
#pragma unroll
              for (int jv = 0; jv < kFoldVec; ++jv) {
                const int i = v0 + jv * 32 + lane;
                if (i < nvec) dv[r][jv] = ld16(r4 + i);
              }
            }
          }
#pragma unroll
          for (int r = 0; r < kFoldRows; ++r) {
            if (q0 + r < n_rows) {
#pragma unroll
              for (int jv = 0; jv < kFoldVec; ++jv)
                if (v0 + jv * 32 + lane < nvec) acc_add(acc[jv], dv[r][jv]);
            }
          }
        }
#pragma unroll
        for (int jv = 0; jv < kFoldVec; ++jv) {
          const int i = v0 + jv * 32 + lane;
          if (i < nvec) st16(reinterpret_cast<int4*>(o) + i, acc_pack(acc[jv]));
        }
      }
    } else {
      // every lane runs the same number of iterations: the shuffles need the whole warp
      for (int i0 = 0; i0 < H; i0 += 32) {
        const int i = i0 + lane;
        float acc = 0.f;
        for (int q = 0; q < n_rows; ++q) {
          const int row = __shfl_sync(0xffffffffu, my_row, q);
          if (i < H) acc += bf16_to_f32(a.in_rows[(long long)row * H + i]);
        }
        if (i < H) o[i] = f32_to_bf16(acc);
      }
    }
    __syncwarp();
    if (lane == 0 && !a.direct) {
      if (sflag != nullptr) {
        fence_gpu();  // row and weights are in this GPU's memory
        st_relaxed_gpu(sflag, epoch);
      } else {
        // the weights went to another GPU: they must have arrived before the PUSH role's flag for this row can
        if (a.in_w != nullptr) fence_sys(); else fence_gpu();
        st_relaxed_gpu(a.fold_flag + item, epoch);
      }
    }
  }
}

// ---- PUSH role ---------------------------------------------------------------------------------------
//
// Pure copy engines: warps 0..kMoveWarps-1 each drive a three-stage shared-memory ring with cp.async.bulk (local
// global -> shared on an mbarrier, shared -> the home rank's staging chunk in bulk groups); warps
// kMoveWarps..2*kMoveWarps-1 release the staging flags of rows whose copies have completed, so that the
// system-scope fence of a release never stalls a lane that issues copies.  Work items, handed out from an atomic
// counter: first batches of rows, of which the primaries without duplicates are sent as they are (they depend on
// nothing), then the duplicate groups in the order the FOLD role finishes them.

constexpr int kMoveWarps = 8;
constexpr int kMoveStages = 3;
constexpr int kMoveQ = 32;
// A row is flagged once its bulk group has completed on the home rank, which takes several microseconds over NVLink;
// the copy loop looks kMoveLag items back so that the completion wait never stalls the issue of new copies.
constexpr int kMoveLag = 12;

struct MoveQueue {
  int* lagged[kMoveWarps][kMoveLag + 4];  // flag of every item in flight that is the last piece of its row, else null
  int* flag[kMoveWarps][kMoveQ];
  int head[kMoveWarps], tail[kMoveWarps], done[kMoveWarps];
};

__device__ __forceinline__ int lds_acquire(const int* p) {
  int v;
  asm volatile("ld.acquire.cta.shared::cta.s32 %0, [%1];" : "=r"(v) : "r"(smem_u32(p)) : "memory");
  return v;
}
__device__ __forceinline__ void sts_release(int* p, int v) {
  asm volatile("st.release.cta.shared::cta.s32 [%0], %1;" ::"r"(smem_u32(p)), "r"(v) : "memory");
}

__device__ void move_helper(const MoonepDevCtx& c, int epoch, MoveQueue& q, int w) {
  const int lane = threadIdx.x & 31;
  int consumed = 0;
  for (;;) {
    int avail = 0;
    if (lane == 0) {
      const unsigned long long t0 = globaltimer_ns();
      unsigned spins = 0;
      for (;;) {
        const int fin = lds_acquire(&q.done[w]);  // read before head: a row pushed before `done` is never missed
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
    // a system-scope fence waits for everything this SM has in flight, so it is paid once per batch
    if (lane == 0) {
      fence_sys();
      for (int i = 0; i < avail; ++i) st_relaxed_sys(q.flag[w][(consumed + i) % kMoveQ], epoch);
    }
    consumed += avail;
    __syncwarp();
    if (lane == 0) sts_release(&q.tail[w], consumed);
  }
}

// Job generator of the PUSH role: one job = one row to stage on its home rank.  Work is handed out in batches of
// kPushRowBatch rows (or groups): the lanes of the warp read the metadata of a whole batch in parallel (row ->
// src_info / link -> home rank, staging slot; the row's gate weight goes to the home rank on the way), then the
// jobs of the batch are taken one by one without further memory traffic.  All lanes call next() together; its
// results are warp-uniform.
struct PushJobs {
  const MoonepDevCtx& c;
  const PushArgs& a;
  int lane, epoch, ngroups, nbatches, ngbatches;
  unsigned pend;  // jobs of the current batch still to hand out
  // this lane's job of the current batch
  const unsigned char* j_src;
  unsigned char* j_dst;
  int* j_flag;
  int j_g, j_row;
  bool failed, drained;

  __device__ PushJobs(const MoonepDevCtx& c_, const PushArgs& a_, int epoch_)
      : c(c_), a(a_), lane(threadIdx.x & 31), epoch(epoch_), pend(0), j_src(nullptr), j_dst(nullptr), j_flag(nullptr),
        j_g(-1), j_row(-1), failed(false), drained(false) {
    ngroups = a.dup_counts[0];
    if (ngroups < 0 || ngroups > a.fold_rows) ngroups = 0;
    nbatches = (c.NvS + kPushRowBatch - 1) / kPushRowBatch;
    ngbatches = (ngroups + kPushGroupBatch - 1) / kPushGroupBatch;
  }

  // Bounded wait of this lane until *f >= want; false on timeout (status recorded).
  __device__ bool lane_wait(const int* f, int want, int what, int id) {
    int v;
    if ((v = ld_acquire_gpu(f)) - want >= 0) return true;
    const unsigned long long t0 = globaltimer_ns();
    unsigned spins = 0;
    while ((v = ld_acquire_gpu(f)) - want < 0) {
      if ((++spins & 63u) == 0 && (globaltimer_ns() - t0 > c.timeout_ns || poisoned(c))) {
        record_status(c, MOONEP_STATUS_TIMEOUT, MOONEP_K_COMBINE_PUSH, what, id, want, v);
        return false;
      }
      __nanosleep(128);
    }
    return true;
  }

  // this lane's primary row `prow` (p_si, p_l its src_info and link word): where it goes; false if the words are bad
  __device__ bool describe(int prow, int p_si, int p_l) {
    const int NvS = c.NvS, K = c.K, S = c.S;
    const int home = p_si / NvS;
    const int slot = p_si - home * NvS;
    const int token = slot / K;
    const int ord = (p_l >> MOONEP_LINK_ORD_SHIFT) & MOONEP_LINK_ORD_MASK;
    if (p_si < 0 || home >= c.R || token >= S || ord >= c.kp || !(p_l & MOONEP_LINK_PRIMARY)) {
      record_status(c, MOONEP_STATUS_BAD_INDEX, MOONEP_K_COMBINE_PUSH, 8, p_si, prow, ord);
      return false;
    }
    if (a.local_home && home == c.rank) return false;  // the FOLD role puts this row into the local staging chunk
    unsigned char* stage_home = c.stage_peer[home];
    const long long stage_row = (long long)token * c.kp + ord;
    j_dst = stage_home + stage_row * ((long long)c.H * 2);
    j_flag = reinterpret_cast<int*>(stage_home + c.stage_flag_off) + stage_row;
    j_row = prow;
    return true;
  }

  __device__ bool next(const unsigned char*& src, unsigned char*& dst, int*& flag) {
    const long long row_bytes = (long long)c.H * 2;
    for (;;) {
      if (failed || drained) return false;
      if (pend) {
        const int j = __ffs(pend) - 1;
        pend &= pend - 1;
        src = reinterpret_cast<const unsigned char*>(__shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(j_src), j));
        dst = reinterpret_cast<unsigned char*>(__shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(j_dst), j));
        flag = reinterpret_cast<int*>(__shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(j_flag), j));
        return true;
      }
      int item = 0;
      if (lane == 0) item = atomicAdd(c.counters + MOONEP_CTR_PUSH_WORK, 1);
      item = __shfl_sync(0xffffffffu, item, 0);
      if (item >= nbatches + ngbatches) {
        drained = true;
        return false;
      }
      bool mine = false;
      j_g = -1;
      if (item < nbatches) {
        // rows without duplicates are sent as they are; their gate weight goes along
        const int row = item * kPushRowBatch + lane;
        if (lane < kPushRowBatch && row < c.NvS) {
          const int si = a.src_info[row];
          const int l = si >= 0 ? a.link[row] : 0;
          if (si >= 0 && (l & MOONEP_LINK_PRIMARY) && !(l & MOONEP_LINK_HAS_NEXT) && describe(row, si, l)) {
            mine = true;
            j_src = reinterpret_cast<const unsigned char*>(a.in_rows) + (long long)row * row_bytes;
            if (a.in_w != nullptr) {
              const int home = si / c.NvS;
              reinterpret_cast<float*>(c.stage_peer[home] + c.stage_w_off)[si - home * c.NvS] = a.in_w[row];
            }
          }
        }
      } else {
        // duplicate groups: the folded row comes from the FOLD role's buffer (which also sent the weights)
        const int g = (item - nbatches) * kPushGroupBatch + lane;
        if (lane < kPushGroupBatch && g < ngroups) {
          const int prow = a.dup_groups[3 * g];
          if (prow >= 0 && prow < c.NvS) {
            if (describe(prow, a.src_info[prow], a.link[prow])) {
              mine = true;
              j_g = g;
              j_src = reinterpret_cast<const unsigned char*>(a.fold_buf) + (long long)g * row_bytes;
            }
          } else {
            record_status(c, MOONEP_STATUS_BAD_INDEX, MOONEP_K_COMBINE_PUSH, 9, prow, g, 0);
          }
        }
      }
      // The rows of the batch must be final before bulk copies read them: groups wait for the FOLD role, rows of a
      // producer that runs beside this kernel for its block counters.  One proxy fence per batch, not per row.
      bool ok = true;
      if (mine && j_g >= 0) ok = lane_wait(a.fold_flag + j_g, epoch, 203, j_g);
      if (mine && j_g < 0 && a.ready != nullptr) ok = lane_wait(a.ready + (j_row >> 7), a.ready_expect, 201, j_row >> 7);
      if (!__all_sync(0xffffffffu, ok)) {
        failed = true;
        return false;
      }
      pend = __ballot_sync(0xffffffffu, mine);
      if (pend && (item >= nbatches || a.ready != nullptr)) fence_proxy_async_all();
    }
  }
};

// Rows that are not multiples of 16 bytes cannot use bulk copies: every warp copies rows element by element.
__device__ void push_role_plain(const MoonepDevCtx& c, const PushArgs& a) {
  const int lane = threadIdx.x & 31;
  const int epoch = abs_epoch(c, MOONEP_FLAG_COMB, a.epoch_comb);
  PushJobs jobs(c, a, epoch);
  const unsigned char* src;
  unsigned char* dst;
  int* flag;
  while (jobs.next(src, dst, flag)) {
    const uint16_t* s16 = reinterpret_cast<const uint16_t*>(src);
    uint16_t* d16 = reinterpret_cast<uint16_t*>(dst);
    for (int i = lane; i < c.H; i += 32) d16[i] = s16[i];
    __syncwarp();
    if (lane == 0) st_release_sys(flag, epoch);
  }
}

// s_ring: this warp's kMoveStages pieces of chunk_bytes; s_bar: its kMoveStages mbarriers (count 1).
__device__ void push_role(const MoonepDevCtx& c, const PushArgs& a, unsigned char* s_ring, unsigned long long* s_bar,
                          MoveQueue& mq, int w) {
  const int lane = threadIdx.x & 31;
  const long long row_bytes = (long long)c.H * 2;
  const int epoch = abs_epoch(c, MOONEP_FLAG_COMB, a.epoch_comb);
  PushJobs jobs(c, a, epoch);
  const unsigned char* j_src = nullptr;
  unsigned char* j_dst = nullptr;
  int* j_flag = nullptr;
  int j_chunk = a.nchunks;  // next piece of the current job; == nchunks: no current job
  bool failed = false;

  // Advance to the next piece to copy: (src, dst, len, flag or null when more pieces of the row follow).
  auto next_item = [&](const unsigned char*& src, unsigned char*& dst, unsigned& len, int*& flag) -> bool {
    if (j_chunk >= a.nchunks) {
      if (!jobs.next(j_src, j_dst, j_flag)) return false;
      j_chunk = 0;
    }
    const long long off = (long long)j_chunk * a.chunk_bytes;
    const long long rest = row_bytes - off;
    len = (unsigned)(rest < a.chunk_bytes ? rest : a.chunk_bytes);
    src = j_src + off;
    dst = j_dst + off;
    ++j_chunk;
    flag = j_chunk >= a.nchunks ? j_flag : nullptr;
    return true;
  };

  // three-stage ring, as in the dispatch send role: the loads of items i+1 and i+2 are in flight while item i is stored
  unsigned char* r_dst[kMoveStages];
  unsigned r_len[kMoveStages];
  int loaded = 0, done = 0, pushed = 0;
  auto issue_load = [&](const unsigned char* src, unsigned char* dst, unsigned len, int* flag) {
    const int s = loaded % kMoveStages;
#pragma unroll
    for (int q = 0; q < kMoveStages; ++q)
      if (q == s) {
        r_dst[q] = dst;
        r_len[q] = len;
      }
    if (lane == 0) {
      mq.lagged[w][loaded % (kMoveLag + 4)] = flag;
      mbar_expect_tx(s_bar + s, len);
      bulk_g2s(s_ring + (size_t)s * a.chunk_bytes, src, len, s_bar + s);
    }
    ++loaded;
  };
  auto flag_item = [&](int j) {
    int* flag = lane == 0 ? mq.lagged[w][j % (kMoveLag + 4)] : nullptr;
    if (flag != nullptr && lane == 0) {
      if (pushed - lds_acquire(&mq.tail[w]) >= kMoveQ) {
        const unsigned long long t0 = globaltimer_ns();
        unsigned spins = 0;
        while (pushed - lds_acquire(&mq.tail[w]) >= kMoveQ) {
          if ((++spins & 255u) == 0 && (globaltimer_ns() - t0 > c.timeout_ns || poisoned(c))) {
            record_status(c, MOONEP_STATUS_TIMEOUT, MOONEP_K_COMBINE_PUSH, 101, w, pushed, 0);
            failed = true;
            return;
          }
        }
      }
      mq.flag[w][pushed % kMoveQ] = flag;
      ++pushed;
      sts_release(&mq.head[w], pushed);
    }
  };

  const unsigned char* src;
  unsigned char* dst;
  unsigned len;
  int* flag;
  // loads run two items ahead of the stores (see the dispatch send role)
  bool more = true;
  for (int q = 0; q < kMoveStages - 1 && more; ++q) {
    more = next_item(src, dst, len, flag);
    if (more) issue_load(src, dst, len, flag);
  }
  while (done < loaded && !failed) {
    const int s = done % kMoveStages;
    unsigned char* o = nullptr;
    unsigned olen = 0;
#pragma unroll
    for (int q = 0; q < kMoveStages; ++q)
      if (q == s) {
        o = r_dst[q];
        olen = r_len[q];
      }
    int got = 1;
    if (lane == 0) got = mbar_wait(s_bar + s, (unsigned)((done / kMoveStages) & 1), c.timeout_ns) ? 1 : 0;
    got = __shfl_sync(0xffffffffu, got, 0);
    if (!got) {
      if (lane == 0) record_status(c, MOONEP_STATUS_TIMEOUT, MOONEP_K_COMBINE_PUSH, 100, s, done, 0);
      failed = true;
      break;
    }
    if (lane == 0) {
      bulk_s2g(o, s_ring + (size_t)s * a.chunk_bytes, olen);
      bulk_commit();
    }
    ++done;
    if (done > kMoveLag) {
      if (lane == 0) bulk_wait<kMoveLag>();  // item done-1-kMoveLag has reached its home rank
      flag_item(done - 1 - kMoveLag);
      failed = __shfl_sync(0xffffffffu, failed ? 1 : 0, 0) != 0;
    }
    if (more && !failed) {
      more = next_item(src, dst, len, flag);
      if (more) {
        if (lane == 0) bulk_wait_read<1>();  // every group but the one just committed has read its stage
        __syncwarp();
        issue_load(src, dst, len, flag);
      }
    }
  }
  if (lane == 0) bulk_wait<0>();
  __syncwarp();
  if (!failed)
    for (int j = done > kMoveLag ? done - kMoveLag : 0; j < done; ++j) flag_item(j);
  if (lane == 0) sts_release(&mq.done[w], 1);
  __syncwarp();
}

// ---- SUM role ----------------------------------------------------------------------------------------

// Sums the staged rows of `token` (all present) in fp32 in ascending k, stores the bf16 result and copies the gate
// weights.  valid: this lane's routing entry is in range; nprim: primaries of the token (rows in its staging slots).
__device__ void sum_token(const MoonepDevCtx& c, const PushArgs& a, int token, bool valid, int nprim, int lane) {
  const int K = c.K, H = c.H, kp = c.kp;
  const long long row_bytes = (long long)H * 2;
  const unsigned char* stage = c.stage_peer[c.rank];
  const float* wst = reinterpret_cast<const float*>(stage + c.stage_w_off);
  if (a.out_w != nullptr && lane < K) a.out_w[token * K + lane] = valid ? wst[token * K + lane] : 0.f;
  const unsigned char* rows = stage + (long long)token * kp * row_bytes;
  uint16_t* orow = a.out + (long long)token * H;
  if (a.vec_ok) {
    const int nvec = H / 8;
    for (int c0 = 0; c0 < nvec; c0 += 32 * kSumVec) {
      float acc[kSumVec][8];
#pragma unroll
      for (int j = 0; j < kSumVec; ++j)
#pragma unroll
        for (int q = 0; q < 8; ++q) acc[j][q] = 0.f;
      for (int p0 = 0; p0 < nprim; p0 += kSumRows) {
        int4 v[kSumRows][kSumVec];
#pragma unroll
        for (int r = 0; r < kSumRows; ++r) {
          if (p0 + r < nprim) {
            const int4* r4 = reinterpret_cast<const int4*>(rows + (long long)(p0 + r) * row_bytes);
#pragma unroll
            for (int j = 0; j < kSumVec; ++j) {
              const int i = c0 + j * 32 + lane;
              if (i < nvec) v[r][j] = ld16(r4 + i);
            }
          }
        }
#pragma unroll
        for (int r = 0; r < kSumRows; ++r) {
          if (p0 + r < nprim) {
#pragma unroll
            for (int j = 0; j < kSumVec; ++j) {
              const int i = c0 + j * 32 + lane;
              if (i < nvec) acc_add(acc[j], v[r][j]);
            }
          }
        }
      }
      int4* o4 = reinterpret_cast<int4*>(orow);
#pragma unroll
      for (int j = 0; j < kSumVec; ++j) {
        const int i = c0 + j * 32 + lane;
        if (i < nvec) st16(o4 + i, acc_pack(acc[j]));
      }
    }
  } else {
    for (int i = lane; i < H; i += 32) {
      float acc = 0.f;
      for (int p = 0; p < nprim; ++p)
        acc += bf16_to_f32(reinterpret_cast<const uint16_t*>(rows + (long long)p * row_bytes)[i]);
      orow[i] = f32_to_bf16(acc);
    }
  }
}

// This lane's routing entry of `token` (lanes >= K: none); false when out of range (status recorded).
__device__ __forceinline__ bool sum_entry(const MoonepDevCtx& c, const PushArgs& a, int token, int lane, int& d) {
  d = 0;
  if (lane >= c.K) return false;
  d = a.dst[token * c.K + lane];
  const int raw = d < 0 ? -d - 1 : d;
  const int dest = raw / c.NvS;
  const int loff = raw - dest * c.NvS;
  const bool valid = dest >= 0 && dest < c.R && loff >= 0 && loff < c.NvS;
  if (!valid) record_status(c, MOONEP_STATUS_BAD_INDEX, MOONEP_K_COMBINE_SUM, 6, d, token, lane);
  return valid;
}

// A warp holds two tokens at a time and sums whichever is complete first.  Rows of a token come from up to min(K, R)
// ranks in no particular order, so most tokens complete late in the transfer; with one token per warp the tokens
// beyond the first wave would only get a warp once an earlier token has completed, and pile up at the end.
__device__ void sum_role_two(const MoonepDevCtx& c, const PushArgs& a) {
  const int lane = threadIdx.x & 31;
  const int S = c.S, kp = c.kp;
  const int epoch = abs_epoch(c, MOONEP_FLAG_COMB, a.epoch_comb);
  int* work = c.counters + MOONEP_CTR_SUM_WORK;
  const int* flags = reinterpret_cast<const int*>(c.stage_peer[c.rank] + c.stage_flag_off);
  int tok[2] = {-1, -1}, dd[2] = {0, 0};
  bool vv[2] = {false, false};
  bool more = true;
  unsigned long long t0 = 0;
  unsigned idle = 0;
  for (;;) {
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      if (tok[q] < 0 && more) {
        int t = 0;
        if (lane == 0) t = atomicAdd(work, 1);
        t = __shfl_sync(0xffffffffu, t, 0);
        if (t >= S) {
          more = false;
        } else {
          tok[q] = t;
          vv[q] = sum_entry(c, a, t, lane, dd[q]);
        }
      }
    }
    if (tok[0] < 0 && tok[1] < 0) break;
    bool progressed = false;
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      if (tok[q] < 0) continue;
      const unsigned prim = __ballot_sync(0xffffffffu, vv[q] && dd[q] >= 0);
      int nprim = __popc(prim);
      if (nprim > kp) nprim = kp;
      const int ord = __popc(prim & ((1u << lane) - 1u));
      bool here = true;
      if (vv[q] && dd[q] >= 0 && ord < kp) here = ld_acquire_sys(flags + (long long)tok[q] * kp + ord) - epoch >= 0;
      if (!__all_sync(0xffffffffu, here)) continue;
      sum_token(c, a, tok[q], vv[q], nprim, lane);
      tok[q] = -1;
      progressed = true;
    }
    if (progressed) {
      idle = 0;
      continue;
    }
    if (idle++ == 0) t0 = globaltimer_ns();
    int give_up = 0;
    if (lane == 0 && (idle & 15u) == 0 && (globaltimer_ns() - t0 > c.timeout_ns || poisoned(c))) {
      record_status(c, MOONEP_STATUS_TIMEOUT, MOONEP_K_COMBINE_SUM, 202, tok[0] >= 0 ? tok[0] : tok[1], epoch, 0);
      give_up = 1;
    }
    if (__shfl_sync(0xffffffffu, give_up, 0)) break;
    __nanosleep(128);
  }
}

__device__ void sum_role(const MoonepDevCtx& c, const PushArgs& a) {
  const int lane = threadIdx.x & 31;
  const int NvS = c.NvS, K = c.K, S = c.S, kp = c.kp;
  const int epoch = abs_epoch(c, MOONEP_FLAG_COMB, a.epoch_comb);
  int* work = c.counters + MOONEP_CTR_SUM_WORK;
  const unsigned char* stage = c.stage_peer[c.rank];
  const int* flags = reinterpret_cast<const int*>(stage + c.stage_flag_off);
  for (;;) {
    int token = 0;
    if (lane == 0) token = atomicAdd(work, 1);
    token = __shfl_sync(0xffffffffu, token, 0);
    if (token >= S) break;
    int d = 0;
    bool valid = false;
    if (lane < K) {
      d = a.dst[token * K + lane];
      const int raw = d < 0 ? -d - 1 : d;
      const int dest = raw / NvS;
      const int loff = raw - dest * NvS;
      valid = dest >= 0 && dest < c.R && loff >= 0 && loff < NvS;
      if (!valid) record_status(c, MOONEP_STATUS_BAD_INDEX, MOONEP_K_COMBINE_SUM, 6, d, token, lane);
    }
    const unsigned prim = __ballot_sync(0xffffffffu, valid && d >= 0);
    int nprim = __popc(prim);
    if (nprim > kp) nprim = kp;
    const int ord = __popc(prim & ((1u << lane) - 1u));
    // wait for the rows of this token
    int ok = 1;
    if (valid && d >= 0 && ord < kp) {
      const int* f = flags + (long long)token * kp + ord;
      if (ld_acquire_sys(f) - epoch < 0) {
        const unsigned long long t0 = globaltimer_ns();
        unsigned spins = 0;
        int v;
        while ((v = ld_acquire_sys(f)) - epoch < 0) {
          if ((++spins & 63u) == 0 && (globaltimer_ns() - t0 > c.timeout_ns || poisoned(c))) {
            record_status(c, MOONEP_STATUS_TIMEOUT, MOONEP_K_COMBINE_SUM, 202, token, epoch, v);
            ok = 0;
            break;
          }
          __nanosleep(128);
        }
      }
    }
    if (!__all_sync(0xffffffffu, ok)) break;
    sum_token(c, a, token, valid, nprim, lane);
  }
}

__global__ void __launch_bounds__(kPushThreads, 1) combine_push_kernel(const MoonepDevCtx c_in, const PushArgs a) {
  extern __shared__ __align__(128) unsigned char s_dyn[];  // PUSH: [kMoveWarps][kMoveStages][chunk_bytes]
  // base addresses of every rank's staging chunk in shared memory: looked up per row, and a lookup in global memory
  // is a dependent load of several hundred nanoseconds
  __shared__ unsigned char* s_stage_peer[MOONEP_MAX_RANKS];
  if (c_in.stage_peer != nullptr)
    for (int r = threadIdx.x; r < c_in.R; r += blockDim.x) s_stage_peer[r] = c_in.stage_peer[r];
  MoonepDevCtx c = c_in;
  if (c_in.stage_peer != nullptr) c.stage_peer = s_stage_peer;
  __shared__ __align__(8) unsigned long long s_bar[kMoveWarps * kMoveStages];
  __shared__ MoveQueue s_mq;
  const int warp = threadIdx.x >> 5;
  if (threadIdx.x < kMoveWarps * kMoveStages) mbar_init(s_bar + threadIdx.x, 1);
  if (threadIdx.x < kMoveWarps) {
    s_mq.head[threadIdx.x] = 0;
    s_mq.tail[threadIdx.x] = 0;
    s_mq.done[threadIdx.x] = 0;
  }
  fence_barrier_init();
  griddep_wait();  // the set-up above may overlap the previous kernel's tail; its results are needed from here on
  griddep_launch();  // the next kernel of the stream may set itself up on SMs as the CTAs of this one leave them
  __syncthreads();
  const bool has_push = (a.roles & MOONEP_ROLE_PUSH) != 0;
  const bool has_local = (a.roles & (MOONEP_ROLE_FOLD | MOONEP_ROLE_SUM)) != 0;
  // PUSH CTAs are the last n_push of the grid
  const bool pusher = has_push && (!has_local || (int)blockIdx.x >= (int)gridDim.x - a.n_push);
  if (pusher) {
    if (block_wait_flags(c, a.wait_family, a.wait_epoch, MOONEP_K_COMBINE_PUSH)) {
      const unsigned long long t0 = globaltimer_ns();
      if (!a.vec_ok) {
        push_role_plain(c, a);
      } else if (warp < kMoveWarps) {
        const size_t stage = (size_t)(a.chunk_bytes + 127) / 128 * 128;
        push_role(c, a, s_dyn + (size_t)warp * kMoveStages * stage, s_bar + warp * kMoveStages, s_mq, warp);
      } else if (warp < 2 * kMoveWarps) {
        move_helper(c, abs_epoch(c, MOONEP_FLAG_COMB, a.epoch_comb), s_mq, warp - kMoveWarps);
      }
      if ((threadIdx.x & 31) == 0 && warp < kMoveWarps) stat_phase(c, MOONEP_PH_PUSH, t0);
    }
  } else if (has_local && !poisoned(c)) {
    unsigned long long t0 = globaltimer_ns();
    if (a.roles & MOONEP_ROLE_FOLD) {
      fold_role(c, a);
      __syncthreads();
      if (threadIdx.x == 0) stat_phase(c, MOONEP_PH_FOLD, t0);
      t0 = globaltimer_ns();
    }
    if (a.roles & MOONEP_ROLE_SUM) {
      if (a.sum_two) sum_role_two(c, a); else sum_role(c, a);
      __syncthreads();
      if (threadIdx.x == 0) stat_phase(c, MOONEP_PH_SUM, t0);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const int arrived = atomicAdd(c.counters + MOONEP_CTR_COMBINE_ARRIVE, 1);
    if (arrived == (int)gridDim.x - 1) {
      c.counters[MOONEP_CTR_COMBINE_ARRIVE] = 0;
      if (a.roles & MOONEP_ROLE_PUSH) c.counters[MOONEP_CTR_PUSH_WORK] = 0;
      if (a.roles & MOONEP_ROLE_SUM) c.counters[MOONEP_CTR_SUM_WORK] = 0;
      if (a.roles & MOONEP_ROLE_FOLD) c.counters[MOONEP_CTR_FOLD_WORK] = 0;
      __threadfence();
    }
  }
}

}  // namespace

}  // namespace moonep

using namespace moonep;

// Bytes of one rank's combine staging chunk for (S, K, H, kp): rows, then flags, then gate weights.
extern "C" long long moonep_stage_layout(int S, int K, int H, int kp, long long* flag_off, long long* w_off) {
  const long long rows = ((long long)S * kp * H * 2 + 127) / 128 * 128;
  const long long flags = ((long long)S * kp * 4 + 127) / 128 * 128;
  const long long w = ((long long)S * K * 4 + 127) / 128 * 128;
  if (flag_off) *flag_off = rows;
  if (w_off) *w_off = rows + flags;
  return rows + flags + w;
}

// roles: MOONEP_ROLE_FOLD | MOONEP_ROLE_PUSH | MOONEP_ROLE_SUM (a single rank launches FOLD alone, which then writes the
// results itself).  src_info / link: the plan's copies ([NvS] each); dup_groups / dup_loffs / dup_counts: the plan's
// duplicate map.  in_rows: the local expert output rows [NvS, H] (the shard or any other local tensor), in_w: their gate
// weights [NvS] or null.  fold_buf [fold_rows, H] bf16 and fold_flag [fold_rows] int32 (zero-initialised once) are
// local scratch of the Buffer; fold_rows bounds the number of duplicate groups.  ready / ready_expect: optional
// per-128-row-block counters bumped by the producer of in_rows (see moonep_grouped_gemm_pair).
extern "C" int moonep_combine_push(void* ctx, int roles, const int* src_info, const int* link, const int* dst,
                                   const void* in_rows, const float* in_w, void* out_hidden, float* out_weights,
                                   int wait_family, int wait_epoch, int epoch_comb, const int* ready, int ready_expect,
                                   const int* dup_groups, const int* dup_loffs, const int* dup_counts, void* fold_buf,
                                   int* fold_flag, int fold_rows, int n_push, int n_local, void* stream) {
  auto* h = (HostCtx*)ctx;
  const MoonepDevCtx& c = h->dev;
  const int local_home = ((roles & MOONEP_ROLE_LOCAL_HOME) && c.R > 1 && c.stage_peer != nullptr) ? 1 : 0;
  roles &= ~MOONEP_ROLE_LOCAL_HOME;
  const int direct = (c.R == 1 && roles == MOONEP_ROLE_FOLD) ? 1 : 0;
  if (c.stage_peer == nullptr && !direct) {
    set_error("moonep_combine_push: this Buffer has no combine staging memory");
    return 1;
  }
  PushArgs a;
  a.src_info = src_info;
  a.link = link;
  a.dst = dst;
  a.in_rows = (const uint16_t*)in_rows;
  a.in_w = in_w;
  a.out = (uint16_t*)out_hidden;
  a.out_w = out_weights;
  a.roles = roles;
  a.wait_family = wait_family;
  a.wait_epoch = wait_epoch;
  a.epoch_comb = epoch_comb;
  a.ready = ready;
  a.ready_expect = ready_expect;
  a.dup_groups = dup_groups;
  a.dup_loffs = dup_loffs;
  a.dup_counts = dup_counts;
  a.fold_buf = (uint16_t*)fold_buf;
  a.fold_flag = fold_flag;
  a.fold_rows = fold_rows;
  a.direct = direct;
  a.local_home = local_home;
  {
    const char* st = getenv("MOONEP_SUM_SLOTS");  // 2: a SUM warp holds two tokens (default 1)
    a.sum_two = (st != nullptr && atoi(st) == 2) ? 1 : 0;
  }
  const bool al = ((reinterpret_cast<uintptr_t>(in_rows) | reinterpret_cast<uintptr_t>(out_hidden) |
                    reinterpret_cast<uintptr_t>(fold_buf)) & 15u) == 0;
  a.vec_ok = (c.H % 8 == 0) && al;
  const long long row_bytes = (long long)c.H * 2;
  a.nchunks = (int)((row_bytes + kPushMaxChunk - 1) / kPushMaxChunk);
  const long long cb = (row_bytes + a.nchunks - 1) / a.nchunks;
  a.chunk_bytes = (int)((cb + 15) / 16 * 16);
  size_t smem = 0;
  if ((roles & MOONEP_ROLE_PUSH) && a.vec_ok)
    smem = (size_t)kMoveWarps * kMoveStages * ((size_t)(a.chunk_bytes + 127) / 128 * 128);
  if ((int)smem + 8192 > h->max_smem_optin) {
    set_error("moonep_combine_push: staging ring does not fit shared memory");
    return 1;
  }
  // The attribute belongs to the kernel, not to the launch, and emulated ranks launch from several threads with
  // different sizes: always allow the same maximum, so that no thread lowers it under another one's launch.
  if (int rc = check_cuda(cudaFuncSetAttribute(combine_push_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               h->max_smem_optin - 8192),
                          "cudaFuncSetAttribute(combine_push_kernel)"))
    return rc;
  const bool local = (roles & (MOONEP_ROLE_FOLD | MOONEP_ROLE_SUM)) != 0;
  int grid = 0;
  a.n_push = 0;
  if (roles & MOONEP_ROLE_PUSH) {
    // num_sms bounds the CTAs that move data between ranks
    a.n_push = imax(1, imin(n_push > 0 ? n_push : c.num_sms, h->sm_count - (local ? 1 : 0)));
    grid = a.n_push;
  }
  if (local) {
    const int room = imax(1, imin(c.local_sms, h->sm_count) - a.n_push);
    grid += n_local > 0 ? imin(n_local, room) : room;
  }
  if (int rc = check_cuda(launch_maybe_pdl(combine_push_kernel, grid, kPushThreads, smem, (cudaStream_t)stream,
                                           h->enable_pdl != 0, c, a),
                          "launch combine_push_kernel"))
    return rc;
  return check_launch("combine_push_kernel");
}
