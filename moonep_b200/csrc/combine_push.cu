// Push combine for sm_100a: the rank that ran the experts folds each token's duplicate rows and
// pushes the result to the token's home rank over NVLink; the home rank sums the rows of a token as
// they arrive.  One kernel, two roles:
//
//   PUSH  (expert side, num_sms CTAs) rows of the local expert output are handed out in small batches.
//         For every primary row (first row of its (source, token) on this rank, known from the plan's
//         copy of src_info and link words) a warp reads the row and its duplicates from local HBM, adds
//         them in fp32 in ascending k, rounds to bf16 into shared memory and sends the row with one
//         cp.async.bulk store into the staging chunk of the home rank, slot (token, position of this
//         rank among the token's destinations).  Gate weights of all of the token's entries on this rank
//         go to the home rank's weight staging.  When the bulk group has completed, the slot's flag is
//         released with the combine's COMB epoch.
//   SUM   (home side, the remaining CTAs) tokens are handed out from an atomic counter; a warp waits
//         (bounded) for the flags of the token's primaries, adds the staged rows in fp32 in ascending k,
//         stores the bf16 result and copies the K gate weights into the [S, K] output.
//
// Compared with pulling (combine.cu) the expert side needs no separate fold pass over its shard, every
// NVLink transfer is a bulk store (which measured faster than loads from peer memory), and the
// home-side sum overlaps the transfers.  Numerics are those of the pull path and of the reference: duplicates
// are added in fp32 and rounded to bf16, the per-token sum is fp32 rounded to bf16.  The expert output rows are
// not modified.
//
// Launched with both roles it is one fused kernel (CTAs 0..n_push-1 push, the rest sum; a SUM CTA only
// waits for other GPUs' PUSH CTAs or for lower-numbered CTAs of its own GPU); emulated ranks that share one GPU
// launch the roles one after the other.
//
// Parity: reference moonep_td/combine_prologue.py:19-40 and moonep_td/combine.py:22-68.
#include "common.cuh"
#include "host.h"

namespace moonep {

namespace {

constexpr int kPushThreads = 384;       // 12 warps, each with one staged row piece in shared memory
constexpr int kPushWarps = kPushThreads / 32;
constexpr int kPushMaxChunk = 14336;    // bytes of a row piece (one stage per warp)
constexpr int kPushRowBatch = 8;        // rows handed out per grab
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
  int direct;               // single rank: PUSH writes the folded rows and the weights straight into out / out_w
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

__device__ __forceinline__ void sts16(void* p, const int4& v) {
  asm volatile("st.shared.v4.s32 [%0], {%1,%2,%3,%4};" ::"r"(smem_u32(p)), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
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

// One group: the row `prow` (primary of its (source, token) on this rank) and its duplicates.  Lane q holds the q-th
// row of the group in my_row (q = 0 the primary, then the duplicates in ascending k), n_rows of them.
struct PushState {
  int* pending_flag;  // lane 0: flag of the row whose last bulk group may still be in flight
  unsigned bar_phase;
  bool failed;
};

__device__ void push_group(const MoonepDevCtx& c, const PushArgs& a, unsigned char* s_stage, unsigned long long* s_bar,
                           PushState& st, int epoch, int prow, int p_si, int p_l, int my_row, int n_rows) {
  const int lane = threadIdx.x & 31;
  const int NvS = c.NvS, K = c.K, H = c.H, S = c.S, kp = c.kp;
  const long long row_bytes = (long long)H * 2;
  const int home = p_si / NvS;
  const int slot = p_si - home * NvS;
  const int token = slot / K;
  const int ord = (p_l >> MOONEP_LINK_ORD_SHIFT) & MOONEP_LINK_ORD_MASK;
  if (p_si < 0 || home >= c.R || token >= S || ord >= kp || !(p_l & MOONEP_LINK_PRIMARY)) {
    record_status(c, MOONEP_STATUS_BAD_INDEX, MOONEP_K_COMBINE_PUSH, 8, p_si, prow, ord);
    return;
  }
  // the producer of the rows (a grouped GEMM running beside this kernel) must be done with every block involved
  if (a.ready != nullptr) {
    for (int q = 0; q < n_rows; ++q) {
      const int row = __shfl_sync(0xffffffffu, my_row, q);
      if (row >= 0 && row < NvS && !wait_block_ready(c, a, row, lane)) {
        st.failed = true;
        return;
      }
    }
  }
  // a single rank needs no staging: the folded row is the token's result
  unsigned char* stage_home = a.direct ? nullptr : c.stage_peer[home];
  // gate weights of all entries of this group travel to the home rank's weight staging
  if (a.in_w != nullptr && lane < n_rows && my_row >= 0 && my_row < NvS) {
    const int s_q = a.src_info[my_row];
    const int slot_q = s_q - home * NvS;
    if (s_q >= 0 && slot_q >= 0 && slot_q < S * K) {
      float* wdst = a.direct ? a.out_w : reinterpret_cast<float*>(stage_home + c.stage_w_off);
      if (wdst != nullptr) wdst[slot_q] = a.in_w[my_row];
    }
  }
  const long long stage_row = (long long)token * kp + ord;
  unsigned char* o_row = a.direct ? reinterpret_cast<unsigned char*>(a.out) + (long long)token * row_bytes
                                  : stage_home + stage_row * row_bytes;
  int* flag = a.direct ? nullptr : reinterpret_cast<int*>(stage_home + c.stage_flag_off) + stage_row;
  if (a.vec_ok) {
    for (int ch = 0; ch < a.nchunks; ++ch) {
      const long long off = (long long)ch * a.chunk_bytes;
      const int len = (int)((row_bytes - off) < a.chunk_bytes ? (row_bytes - off) : a.chunk_bytes);
      const int nvec = len / 16;
      // the stage is free once the previous bulk store has read it
      if (lane == 0) bulk_wait_read<0>();
      __syncwarp();
      const unsigned char* src0 = reinterpret_cast<const unsigned char*>(a.in_rows) + (long long)prow * row_bytes + off;
      if (n_rows == 1) {
        // nothing to fold: the piece goes global -> shared -> home rank without touching registers
        int got = 1;
        if (lane == 0) {
          mbar_expect_tx(s_bar, (unsigned)len);
          bulk_g2s(s_stage, src0, (unsigned)len, s_bar);
          got = mbar_wait(s_bar, st.bar_phase, c.timeout_ns) ? 1 : 0;
          if (!got) record_status(c, MOONEP_STATUS_TIMEOUT, MOONEP_K_COMBINE_PUSH, 100, prow, ch, 0);
        }
        st.bar_phase ^= 1u;
        if (!__shfl_sync(0xffffffffu, got, 0)) {
          st.failed = true;
          return;
        }
      } else {
        for (int v0 = 0; v0 < nvec; v0 += 32 * kFoldVec) {
          float acc[kFoldVec][8];
#pragma unroll
          for (int jv = 0; jv < kFoldVec; ++jv)
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[jv][e] = 0.f;
          // loads of up to kFoldRows rows are issued before the first add; adds keep the order primary, duplicates by k
          for (int q0 = 0; q0 < n_rows; q0 += kFoldRows) {
            int4 dv[kFoldRows][kFoldVec];
#pragma unroll
            for (int r = 0; r < kFoldRows; ++r) {
              int row = __shfl_sync(0xffffffffu, my_row, (q0 + r) & 31);
              if (row < 0 || row >= NvS) row = prow;  // never dereference a bad index (status recorded by the caller)
              if (q0 + r < n_rows) {
                const int4* r4 = reinterpret_cast<const int4*>(reinterpret_cast<const unsigned char*>(a.in_rows) +
                                                                (long long)row * row_bytes + off);
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
            if (i < nvec) sts16(s_stage + (size_t)i * 16, acc_pack(acc[jv]));
          }
        }
      }
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) {
        bulk_s2g(o_row + off, s_stage, (unsigned)len);
        bulk_commit();
        if (st.pending_flag != nullptr) {
          // every group but the one just committed has completed: the previous row is in its home's memory
          bulk_wait<1>();
          st_release_sys(st.pending_flag, epoch);
          st.pending_flag = nullptr;
        }
      }
    }
    if (lane == 0) st.pending_flag = flag;
  } else {
    // rows that are not multiples of 16 bytes: element-wise, straight into the home rank's staging chunk
    uint16_t* o = reinterpret_cast<uint16_t*>(o_row);
    // every lane runs the same number of iterations: the shuffles need the whole warp
    for (int i0 = 0; i0 < H; i0 += 32) {
      const int i = i0 + lane;
      uint16_t v = i < H ? a.in_rows[(long long)prow * H + i] : (uint16_t)0;
      if (n_rows > 1) {
        float acc = bf16_to_f32(v);
        for (int q = 1; q < n_rows; ++q) {
          int row = __shfl_sync(0xffffffffu, my_row, q);
          if (row < 0 || row >= NvS) row = prow;
          if (i < H) acc += bf16_to_f32(a.in_rows[(long long)row * H + i]);
        }
        v = f32_to_bf16(acc);
      }
      if (i < H) o[i] = v;
    }
    __syncwarp();
    if (lane == 0 && flag != nullptr) st_release_sys(flag, epoch);
  }
}

// s_stage: this warp's row piece in shared memory (chunk_bytes, 128-byte aligned).  Work items, handed out from an
// atomic counter: first the duplicate groups of the plan (primary row plus duplicates, folded), then batches of rows
// of which the primaries without duplicates are sent as they are.
__device__ void push_role(const MoonepDevCtx& c, const PushArgs& a, unsigned char* s_stage, unsigned long long* s_bar) {
  const int lane = threadIdx.x & 31;
  const int NvS = c.NvS;
  const int epoch = abs_epoch(c, MOONEP_FLAG_COMB, a.epoch_comb);
  int* work = c.counters + MOONEP_CTR_PUSH_WORK;
  PushState st;
  st.pending_flag = nullptr;
  st.bar_phase = 0;
  st.failed = false;
  int ngroups = a.dup_counts[0];
  if (ngroups < 0 || ngroups > NvS) ngroups = 0;
  const int nbatches = (NvS + kPushRowBatch - 1) / kPushRowBatch;
  for (;;) {
    int item = 0;
    if (lane == 0) item = atomicAdd(work, 1);
    item = __shfl_sync(0xffffffffu, item, 0);
    if (item >= ngroups + nbatches || st.failed) break;
    if (item < ngroups) {
      const int prow = a.dup_groups[3 * item], ds = a.dup_groups[3 * item + 1], dn = a.dup_groups[3 * item + 2];
      if (prow < 0 || prow >= NvS || ds < 0 || dn < 1 || dn >= MOONEP_MAX_TOPK || ds + dn > NvS) {
        record_status(c, MOONEP_STATUS_BAD_INDEX, MOONEP_K_COMBINE_PUSH, 9, prow, ds, dn);
        continue;
      }
      int my_row = -1;
      if (lane == 0) my_row = prow;
      else if (lane <= dn) my_row = a.dup_loffs[ds + lane - 1];
      if (__any_sync(0xffffffffu, lane <= dn && (my_row < 0 || my_row >= NvS))) {
        record_status(c, MOONEP_STATUS_BAD_INDEX, MOONEP_K_COMBINE_PUSH, 5, my_row, prow, 0);
        continue;
      }
      push_group(c, a, s_stage, s_bar, st, epoch, prow, a.src_info[prow], a.link[prow], my_row, 1 + dn);
    } else {
      const int base = (item - ngroups) * kPushRowBatch;
      int si = -1, l = 0;
      if (lane < kPushRowBatch && base + lane < NvS) {
        si = a.src_info[base + lane];
        l = si >= 0 ? a.link[base + lane] : 0;
      }
      unsigned prim = __ballot_sync(0xffffffffu, si >= 0 && (l & MOONEP_LINK_PRIMARY) && !(l & MOONEP_LINK_HAS_NEXT));
      while (prim && !st.failed) {
        const int j = __ffs(prim) - 1;
        prim &= prim - 1;
        const int p_si = __shfl_sync(0xffffffffu, si, j);
        const int p_l = __shfl_sync(0xffffffffu, l, j);
        push_group(c, a, s_stage, s_bar, st, epoch, base + j, p_si, p_l, lane == 0 ? base + j : -1, 1);
      }
    }
  }
  if (lane == 0) {
    bulk_wait<0>();
    if (st.pending_flag != nullptr && !st.failed) st_release_sys(st.pending_flag, epoch);
  }
  __syncwarp();
}

// ---- SUM role ----------------------------------------------------------------------------------------

__device__ void sum_role(const MoonepDevCtx& c, const PushArgs& a) {
  const int lane = threadIdx.x & 31;
  const int NvS = c.NvS, K = c.K, H = c.H, S = c.S, kp = c.kp;
  const long long row_bytes = (long long)H * 2;
  const int epoch = abs_epoch(c, MOONEP_FLAG_COMB, a.epoch_comb);
  int* work = c.counters + MOONEP_CTR_SUM_WORK;
  const unsigned char* stage = c.stage_peer[c.rank];
  const int* flags = reinterpret_cast<const int*>(stage + c.stage_flag_off);
  const float* wst = reinterpret_cast<const float*>(stage + c.stage_w_off);
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
}

__global__ void __launch_bounds__(kPushThreads, 1) combine_push_kernel(const MoonepDevCtx c, const PushArgs a) {
  extern __shared__ __align__(128) unsigned char s_dyn[];  // [kPushWarps][chunk_bytes rounded up to 128]
  __shared__ __align__(8) unsigned long long s_bar[kPushWarps];
  const int warp = threadIdx.x >> 5;
  if (threadIdx.x < kPushWarps) mbar_init(s_bar + threadIdx.x, 1);
  fence_barrier_init();
  __syncthreads();
  const bool mixed = (a.roles & MOONEP_ROLE_PUSH) && (a.roles & MOONEP_ROLE_SUM);
  const bool pusher = (a.roles & MOONEP_ROLE_PUSH) && (!mixed || (int)blockIdx.x < a.n_push);
  if (pusher) {
    if (block_wait_flags(c, a.wait_family, a.wait_epoch, MOONEP_K_COMBINE_PUSH))
      push_role(c, a, s_dyn + (size_t)warp * ((a.chunk_bytes + 127) / 128 * 128), s_bar + warp);
  } else if (a.roles & MOONEP_ROLE_SUM) {
    if (!poisoned(c)) sum_role(c, a);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const int arrived = atomicAdd(c.counters + MOONEP_CTR_COMBINE_ARRIVE, 1);
    if (arrived == (int)gridDim.x - 1) {
      c.counters[MOONEP_CTR_COMBINE_ARRIVE] = 0;
      if (a.roles & MOONEP_ROLE_PUSH) c.counters[MOONEP_CTR_PUSH_WORK] = 0;
      if (a.roles & MOONEP_ROLE_SUM) c.counters[MOONEP_CTR_SUM_WORK] = 0;
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

// roles: MOONEP_ROLE_PUSH | MOONEP_ROLE_SUM (a single rank launches PUSH alone, which then writes the results itself).
// src_info / link: the plan's copies ([NvS] each); dup_groups / dup_loffs / dup_counts: the plan's duplicate map.  in_rows: the local expert
// output rows [NvS, H] (the shard or any other local tensor), in_w: their gate weights [NvS] or null.  ready /
// ready_expect: optional per-128-row-block counters bumped by the producer of in_rows (see moonep_grouped_gemm_pair).
extern "C" int moonep_combine_push(void* ctx, int roles, const int* src_info, const int* link, const int* dst,
                                   const void* in_rows, const float* in_w, void* out_hidden, float* out_weights,
                                   int wait_family, int wait_epoch, int epoch_comb, const int* ready, int ready_expect,
                                   const int* dup_groups, const int* dup_loffs, const int* dup_counts, int n_push,
                                   int n_sum, void* stream) {
  auto* h = (HostCtx*)ctx;
  const MoonepDevCtx& c = h->dev;
  const int direct = (c.R == 1 && roles == MOONEP_ROLE_PUSH) ? 1 : 0;
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
  a.direct = direct;
  const bool al = ((reinterpret_cast<uintptr_t>(in_rows) | reinterpret_cast<uintptr_t>(out_hidden)) & 15u) == 0;
  a.vec_ok = (c.H % 8 == 0) && al;
  const long long row_bytes = (long long)c.H * 2;
  a.nchunks = (int)((row_bytes + kPushMaxChunk - 1) / kPushMaxChunk);
  const long long cb = (row_bytes + a.nchunks - 1) / a.nchunks;
  a.chunk_bytes = (int)((cb + 15) / 16 * 16);
  size_t smem = 0;
  if (roles & MOONEP_ROLE_PUSH) smem = (size_t)kPushWarps * ((a.chunk_bytes + 127) / 128 * 128);
  if ((int)smem + 4096 > h->max_smem_optin) {
    set_error("moonep_combine_push: staging ring does not fit shared memory");
    return 1;
  }
  if (int rc = check_cuda(cudaFuncSetAttribute(combine_push_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               (int)imax((int)smem, 1024)),
                          "cudaFuncSetAttribute(combine_push_kernel)"))
    return rc;
  int grid = 0;
  a.n_push = 0;
  if (roles & MOONEP_ROLE_PUSH) {
    // num_sms bounds the CTAs that move data between ranks; with a single rank nothing leaves the GPU
    const int want = n_push > 0 ? n_push : (direct ? imin(c.local_sms, h->sm_count) : c.num_sms);
    a.n_push = imax(1, imin(want, h->sm_count - ((roles & MOONEP_ROLE_SUM) ? 1 : 0)));
    grid = a.n_push;
  }
  if (roles & MOONEP_ROLE_SUM) {
    const int room = imax(1, imin(c.local_sms, h->sm_count) - a.n_push);
    grid += n_sum > 0 ? imin(n_sum, room) : room;
  }
  combine_push_kernel<<<grid, kPushThreads, smem, (cudaStream_t)stream>>>(c, a);
  return check_launch("combine_push_kernel");
}
