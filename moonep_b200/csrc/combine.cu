// Combine for sm_100a: fold duplicate rows on the expert side, then pull every token's
// primary rows home over NVLink peer memory and sum them.
//
//   combine_prologue  (optionally waits for FLAG_READY) for every duplicate group of the
//                     local shard: primary = bf16(f32(primary) + sum f32(duplicates)), in the
//                     stored order; the last CTA signals FLAG_COMB.
//   combine_pull      waits for every peer's FLAG_COMB; tokens are handed out in batches from an
//                     atomic counter; per token the primary rows (one per destination rank) are
//                     read from the peers with 16-byte loads, several rows in flight per lane,
//                     accumulated in fp32 in ascending k and stored as bf16; all K gate weights
//                     are read back from the rows' weight slots.
//
// Parity: reference moonep_td/combine_prologue.py:19-40 and moonep_td/combine.py:22-68 (which
// re-reads and re-decodes dst for each of the H/128 column chunks of a token).
#include "common.cuh"
#include "host.h"

namespace moonep {

namespace {

constexpr int kTokenBatch = 2;
constexpr int kPullVec = 4;     // int4 per lane per row chunk (2 KB per warp and row)
constexpr int kPullRows = 4;    // rows whose loads are issued before the first add
constexpr int kGroupVec = 8;

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

__global__ void __launch_bounds__(512)
    combine_prologue_kernel(const MoonepDevCtx c, const int* __restrict__ dup_groups, const int* __restrict__ dup_loffs,
                            const int* __restrict__ dup_counts, int wait_family, int wait_epoch, int signal_epoch,
                            int vec_ok) {
  const bool ok = block_wait_flags(c, wait_family, wait_epoch, MOONEP_K_COMBINE_PROLOGUE);
  if (ok) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int H = c.H;
    int ngroups = dup_counts[0];
    if (ngroups < 0 || ngroups > c.NvS) ngroups = 0;
    uint16_t* shard = c.hidden_peer[c.rank];
    for (int g = blockIdx.x * nwarps + warp; g < ngroups; g += gridDim.x * nwarps) {
      const int primary = dup_groups[3 * g];
      const int ds = dup_groups[3 * g + 1];
      const int dn = dup_groups[3 * g + 2];
      if (primary < 0 || primary >= c.NvS || ds < 0 || dn < 0 || ds + dn > c.NvS) continue;
      uint16_t* prow = shard + (long long)primary * H;
      const int my_dup = (lane < dn && lane < 32) ? dup_loffs[ds + lane] : -1;  // lane q: q-th duplicate row
      if (vec_ok) {
        const int nvec = H / 8;
        int4* p4 = reinterpret_cast<int4*>(prow);
        for (int c0 = 0; c0 < nvec; c0 += 32 * kGroupVec) {
          float acc[kGroupVec][8];
#pragma unroll
          for (int j = 0; j < kGroupVec; ++j) {
            const int i = c0 + j * 32 + lane;
#pragma unroll
            for (int q = 0; q < 8; ++q) acc[j][q] = 0.f;
            if (i < nvec) acc_add(acc[j], ld16(p4 + i));
          }
          for (int q = 0; q < dn && q < 32; ++q) {
            const int row = __shfl_sync(0xffffffffu, my_dup, q);
            if (row < 0 || row >= c.NvS) continue;
            const int4* r4 = reinterpret_cast<const int4*>(shard + (long long)row * H);
            int4 v[kGroupVec];
#pragma unroll
            for (int j = 0; j < kGroupVec; ++j) {
              const int i = c0 + j * 32 + lane;
              if (i < nvec) v[j] = ld16(r4 + i);
            }
#pragma unroll
            for (int j = 0; j < kGroupVec; ++j) {
              const int i = c0 + j * 32 + lane;
              if (i < nvec) acc_add(acc[j], v[j]);
            }
          }
#pragma unroll
          for (int j = 0; j < kGroupVec; ++j) {
            const int i = c0 + j * 32 + lane;
            if (i < nvec) st16(p4 + i, acc_pack(acc[j]));
          }
        }
      } else {
        for (int i = lane; i < H; i += 32) {
          float acc = bf16_to_f32(prow[i]);
          for (int q = 0; q < dn; ++q) {
            const int row = dup_loffs[ds + q];
            if (row < 0 || row >= c.NvS) continue;
            acc += bf16_to_f32(shard[(long long)row * H + i]);
          }
          prow[i] = f32_to_bf16(acc);
        }
      }
    }
  }
  grid_tail_signal(c, MOONEP_K_COMBINE_PROLOGUE, ok ? MOONEP_FLAG_COMB : -1, signal_epoch);
}

__global__ void __launch_bounds__(512)
    combine_pull_kernel(const MoonepDevCtx c, const int* __restrict__ dst, uint16_t* __restrict__ out,
                        float* __restrict__ out_w, int wait_epoch, int vec_ok) {
  const bool ok = block_wait_flags(c, MOONEP_FLAG_COMB, wait_epoch, MOONEP_K_COMBINE_PULL);
  const int lane = threadIdx.x & 31;
  int* work = c.counters + MOONEP_NUM_KERNEL_IDS + 1;
  if (ok) {
    const int H = c.H, K = c.K, S = c.S, NvS = c.NvS;
    for (;;) {
      int b0 = 0;
      if (lane == 0) b0 = atomicAdd(work, kTokenBatch);
      b0 = __shfl_sync(0xffffffffu, b0, 0);
      if (b0 >= S) break;
      const int b1 = min(S, b0 + kTokenBatch);
      for (int token = b0; token < b1; ++token) {
        int d = 0, dest = 0, loff = 0;
        bool valid = false;
        if (lane < K) {
          d = dst[token * K + lane];
          const int raw = d < 0 ? -d - 1 : d;
          dest = raw / NvS;
          loff = raw - dest * NvS;
          valid = dest >= 0 && dest < c.R && loff >= 0 && loff < NvS;
          if (!valid) record_status(c, MOONEP_STATUS_BAD_INDEX, MOONEP_K_COMBINE_PULL, 6, d, token, lane);
          if (out_w != nullptr) {
            const float* w = reinterpret_cast<const float*>(c.meta_peer[valid ? dest : c.rank] + c.weights_off);
            out_w[token * K + lane] = valid ? w[loff] : 0.f;
          }
        }
        const unsigned prim = __ballot_sync(0xffffffffu, valid && d >= 0);
        // row pointers of the primaries, compacted into the low lanes
        const int my_pos = __popc(prim & ((1u << lane) - 1u));
        const int nprim = __popc(prim);
        const uint16_t* my_row = (valid && d >= 0) ? c.hidden_peer[dest] + (long long)loff * H : nullptr;
        unsigned long long rows_compact = 0;
        {
          // lane p receives the pointer of the p-th primary (ascending k)
          unsigned m = prim;
          int p = 0;
          while (m) {
            const int kk = __ffs(m) - 1;
            m &= m - 1;
            const unsigned long long ptr = __shfl_sync(0xffffffffu, (unsigned long long)my_row, kk);
            if (lane == p) rows_compact = ptr;
            ++p;
          }
        }
        (void)my_pos;
        uint16_t* orow = out + (long long)token * H;
        if (vec_ok) {
          const int nvec = H / 8;
          for (int c0 = 0; c0 < nvec; c0 += 32 * kPullVec) {
            float acc[kPullVec][8];
#pragma unroll
            for (int j = 0; j < kPullVec; ++j)
#pragma unroll
              for (int q = 0; q < 8; ++q) acc[j][q] = 0.f;
            for (int p0 = 0; p0 < nprim; p0 += kPullRows) {
              int4 v[kPullRows][kPullVec];
#pragma unroll
              for (int r = 0; r < kPullRows; ++r) {
                const unsigned long long ptr = __shfl_sync(0xffffffffu, rows_compact, (p0 + r) & 31);
                if (p0 + r < nprim) {
                  const int4* r4 = reinterpret_cast<const int4*>(ptr);
#pragma unroll
                  for (int j = 0; j < kPullVec; ++j) {
                    const int i = c0 + j * 32 + lane;
                    if (i < nvec) v[r][j] = ld16(r4 + i);
                  }
                }
              }
#pragma unroll
              for (int r = 0; r < kPullRows; ++r) {
                if (p0 + r < nprim) {
#pragma unroll
                  for (int j = 0; j < kPullVec; ++j) {
                    const int i = c0 + j * 32 + lane;
                    if (i < nvec) acc_add(acc[j], v[r][j]);
                  }
                }
              }
            }
            int4* o4 = reinterpret_cast<int4*>(orow);
#pragma unroll
            for (int j = 0; j < kPullVec; ++j) {
              const int i = c0 + j * 32 + lane;
              if (i < nvec) st16(o4 + i, acc_pack(acc[j]));
            }
          }
        } else {
          // every lane runs the same number of iterations: the shuffles need the whole warp
          for (int i0 = 0; i0 < H; i0 += 32) {
            const int i = i0 + lane;
            float acc = 0.f;
            for (int p = 0; p < nprim; ++p) {
              const unsigned long long ptr = __shfl_sync(0xffffffffu, rows_compact, p);
              if (i < H) acc += bf16_to_f32(reinterpret_cast<const uint16_t*>(ptr)[i]);
            }
            if (i < H) orow[i] = f32_to_bf16(acc);
          }
        }
      }
    }
  }
  __shared__ int s_last;
  __syncthreads();
  if (threadIdx.x == 0) {
    const int arrived = atomicAdd(c.counters + MOONEP_K_COMBINE_PULL, 1);
    s_last = arrived == (int)gridDim.x - 1;
    if (s_last) {
      c.counters[MOONEP_K_COMBINE_PULL] = 0;
      *work = 0;
      __threadfence();
    }
  }
}

// ---- pull kernel, bulk-copy path ---------------------------------------------------------------------
//
// Warp 0 is the producer: per (token, row piece) it takes a free slot of a shared-memory ring and
// lets one lane issue one cp.async.bulk per primary row (peer global -> shared, completion counted
// in bytes on the slot's "full" mbarrier).  Warps 1..nslots are consumers, warp w owning slot w-1:
// it waits for the slot, adds the rows in fp32 in ascending k, stores the bf16 result with 16-byte
// stores and releases the slot through its "empty" mbarrier.  Remote reads are therefore issued back to back without waiting for data,
// which keeps the NVLink request queue full with few SMs.

constexpr int kPullConsumerWarps = 8;
constexpr int kPullBulkThreads = 32 * (1 + kPullConsumerWarps);
constexpr int kPullMaxSlots = 8;

struct PullBulkArgs {
  const int* dst;
  uint16_t* out;
  float* out_w;
  int wait_epoch;
  int chunk_bytes;  // bytes of one row piece (multiple of 16)
  int nsplit;       // pieces per row
  int kp;           // rows a slot can hold: min(K, R)
  int nslots;
};

__device__ __forceinline__ int4 lds16(const void* p) {
  int4 v;
  asm volatile("ld.shared.v4.s32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(smem_u32(p)));
  return v;
}

__global__ void __launch_bounds__(kPullBulkThreads) combine_pull_bulk_kernel(const MoonepDevCtx c, const PullBulkArgs a) {
  extern __shared__ __align__(128) unsigned char s_slots[];  // [nslots][kp][chunk_bytes]
  __shared__ __align__(8) unsigned long long s_full[kPullMaxSlots];
  __shared__ __align__(8) unsigned long long s_empty[kPullMaxSlots];
  __shared__ int s_tok[kPullMaxSlots], s_split[kPullMaxSlots], s_np[kPullMaxSlots];
  __shared__ int s_fail;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x < a.nslots) {
    mbar_init(s_full + threadIdx.x, 1);
    mbar_init(s_empty + threadIdx.x, 1);
  }
  if (threadIdx.x == 0) s_fail = 0;
  fence_barrier_init();
  const bool ok = block_wait_flags(c, MOONEP_FLAG_COMB, a.wait_epoch, MOONEP_K_COMBINE_PULL);
  int* work = c.counters + MOONEP_NUM_KERNEL_IDS + 1;
  const long long row_bytes = (long long)c.H * 2;
  const size_t slot_bytes = (size_t)a.kp * a.chunk_bytes;
  if (ok) {
    if (warp == 0) {
      // ---------------- producer ----------------
      const int K = c.K, S = c.S, NvS = c.NvS;
      int item = 0;
      bool failed = false;
      auto acquire_slot = [&](int slot, int use) -> bool {
        int got = 1;
        if (use > 0 && lane == 0) got = mbar_wait(s_empty + slot, (unsigned)((use - 1) & 1), c.timeout_ns) ? 1 : 0;
        got = __shfl_sync(0xffffffffu, got, 0);
        if (!got && lane == 0) {
          record_status(c, MOONEP_STATUS_TIMEOUT, MOONEP_K_COMBINE_PULL, 101, slot, use, 0);
          s_fail = 1;
        }
        return got != 0;
      };
      // A batch is as many tokens as fit their K routing entries into the 32 lanes: one coalesced
      // load of dst and one round of weight gathers serve the whole batch.
      const int TB = K <= 32 ? 32 / K : 1;
      const int tl = lane / K, kl = lane - tl * K;
      // Three batches are in flight so that no load is used in the iteration that issued it:
      // N has its dst load outstanding, Q its weight gather, P is complete and gets its rows fetched.
      struct Batch {
        int b0, d, dest, loff;
        bool valid;
        float w;
      };
      auto stage1 = [&](Batch& n) {
        int b = 0;
        if (lane == 0) b = atomicAdd(work, TB);
        n.b0 = __shfl_sync(0xffffffffu, b, 0);
        n.d = 0;
        const int tok = n.b0 + tl;
        if (tl < TB && tok < S) n.d = a.dst[tok * K + kl];
      };
      auto stage2 = [&](Batch& q) {
        q.valid = false;
        q.dest = 0;
        q.loff = 0;
        q.w = 0.f;
        const int tok = q.b0 + tl;
        if (q.b0 < S && tl < TB && tok < S) {
          const int raw = q.d < 0 ? -q.d - 1 : q.d;
          q.dest = raw / NvS;
          q.loff = raw - q.dest * NvS;
          q.valid = q.dest >= 0 && q.dest < c.R && q.loff >= 0 && q.loff < NvS;
          if (!q.valid) record_status(c, MOONEP_STATUS_BAD_INDEX, MOONEP_K_COMBINE_PULL, 6, q.d, tok, kl);
          if (a.out_w != nullptr && q.valid)
            q.w = reinterpret_cast<const float*>(c.meta_peer[q.dest] + c.weights_off)[q.loff];
        }
      };
      Batch P, Q, N;
      stage1(Q);
      stage2(Q);
      stage1(N);
      for (;;) {
        P = Q;
        Q = N;
        if (P.b0 >= S || failed) break;
        stage2(Q);
        stage1(N);
        const int b0 = P.b0;
        const int my_token = b0 + tl;
        const bool have = tl < TB && my_token < S;
        const int d = P.d, dest = P.dest, loff = P.loff;
        const bool valid = P.valid;
        if (have && a.out_w != nullptr) a.out_w[my_token * K + kl] = valid ? P.w : 0.f;
        const unsigned prim_all = __ballot_sync(0xffffffffu, have && valid && d >= 0);
        const unsigned long long my_row =
            (have && valid && d >= 0)
                ? (unsigned long long)(reinterpret_cast<const unsigned char*>(c.hidden_peer[dest]) + (long long)loff * row_bytes)
                : 0ull;
        const int ntok = min(TB, S - b0);
        for (int tt = 0; tt < ntok && !failed; ++tt) {
          const int token = b0 + tt;
          const unsigned prim = (K >= 32) ? prim_all : ((prim_all >> (tt * K)) & ((1u << K) - 1u));
          int nprim = __popc(prim);
          if (nprim > a.kp) nprim = a.kp;
          unsigned long long rows_compact = 0;
          {
            unsigned m = prim;
            int p = 0;
            while (m) {
              const int kk = __ffs(m) - 1;
              m &= m - 1;
              const unsigned long long ptr = __shfl_sync(0xffffffffu, my_row, tt * K + kk);
              if (lane == p) rows_compact = ptr;
              ++p;
            }
          }
          for (int split = 0; split < a.nsplit; ++split) {
            const int slot = item % a.nslots, use = item / a.nslots;
            if (!acquire_slot(slot, use)) {
              failed = true;
              break;
            }
            const long long off = (long long)split * a.chunk_bytes;
            const unsigned len = (unsigned)((row_bytes - off) < a.chunk_bytes ? (row_bytes - off) : a.chunk_bytes);
            if (lane == 0) {
              s_tok[slot] = token;
              s_split[slot] = split;
              s_np[slot] = nprim;
              if (nprim > 0)
                mbar_expect_tx(s_full + slot, (unsigned)nprim * len);
              else
                mbar_arrive(s_full + slot);
            }
            for (int p = 0; p < nprim; ++p) {
              const unsigned long long ptr = __shfl_sync(0xffffffffu, rows_compact, p);
              if (lane == 0)
                bulk_g2s(s_slots + slot * slot_bytes + (size_t)p * a.chunk_bytes,
                         reinterpret_cast<const unsigned char*>(ptr) + off, len, s_full + slot);
            }
            ++item;
          }
        }
      }
      // end markers: one for each consumer warp (one per slot)
      for (int q = 0; q < a.nslots && !failed; ++q, ++item) {
        const int slot = item % a.nslots, use = item / a.nslots;
        if (!acquire_slot(slot, use)) break;
        if (lane == 0) {
          s_tok[slot] = -1;
          mbar_arrive(s_full + slot);
        }
      }
    } else {
      // ---------------- consumers ----------------
      // Consumer warp w owns slot w-1 and therefore the items w-1, w-1+nslots, ...: it has always
      // finished use u-1 of its slot before it waits for use u, which the parity wait relies on
      // (a warp that could run a whole phase ahead would take the previous fill for its own).
      for (int item = warp - 1; warp <= a.nslots; item += a.nslots) {
        const int slot = item % a.nslots, use = item / a.nslots;
        bool got = mbar_try_wait(s_full + slot, (unsigned)(use & 1));
        if (!got) {
          const unsigned long long t0 = globaltimer_ns();
          unsigned spins = 0;
          while (!(got = mbar_try_wait(s_full + slot, (unsigned)(use & 1)))) {
            if ((++spins & 255u) == 0 && (*(volatile int*)&s_fail || globaltimer_ns() - t0 > c.timeout_ns)) break;
          }
        }
        if (!got) {
          if (!*(volatile int*)&s_fail) record_status(c, MOONEP_STATUS_TIMEOUT, MOONEP_K_COMBINE_PULL, 102, slot, use, 0);
          break;
        }
        const int token = s_tok[slot];
        if (token < 0) break;
        const int split = s_split[slot], np = s_np[slot];
        const long long off = (long long)split * a.chunk_bytes;
        const int len = (int)((row_bytes - off) < a.chunk_bytes ? (row_bytes - off) : a.chunk_bytes);
        const unsigned char* base = s_slots + slot * slot_bytes;
        unsigned char* orow = reinterpret_cast<unsigned char*>(a.out) + (long long)token * row_bytes + off;
        for (int v = lane; v < len / 16; v += 32) {
          float acc[8];
#pragma unroll
          for (int q = 0; q < 8; ++q) acc[q] = 0.f;
          for (int p = 0; p < np; ++p) acc_add(acc, lds16(base + (size_t)p * a.chunk_bytes + (size_t)v * 16));
          st16(orow + (size_t)v * 16, acc_pack(acc));
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(s_empty + slot);
      }
    }
  }
  __shared__ int s_last;
  __syncthreads();
  if (threadIdx.x == 0) {
    const int arrived = atomicAdd(c.counters + MOONEP_K_COMBINE_PULL, 1);
    s_last = arrived == (int)gridDim.x - 1;
    if (s_last) {
      c.counters[MOONEP_K_COMBINE_PULL] = 0;
      *work = 0;
      __threadfence();
    }
  }
}

}  // namespace

}  // namespace moonep

using namespace moonep;

extern "C" int moonep_combine_prologue(void* ctx, const int* dup_groups, const int* dup_loffs, const int* dup_counts,
                                       const void* in_hidden, const float* in_weights, int wait_family, int wait_epoch,
                                       int signal_epoch_comb, void* stream) {
  (void)in_hidden;
  (void)in_weights;
  auto* h = (HostCtx*)ctx;
  const MoonepDevCtx& c = h->dev;
  const int grid = imax(1, imin(c.local_sms, h->sm_count));
  combine_prologue_kernel<<<grid, 512, 0, (cudaStream_t)stream>>>(c, dup_groups, dup_loffs, dup_counts, wait_family,
                                                                 wait_epoch, signal_epoch_comb, (c.H % 8 == 0) ? 1 : 0);
  return check_launch("combine_prologue_kernel");
}

extern "C" int moonep_combine_pull(void* ctx, const int* dst, void* out_hidden, float* out_weights, int wait_epoch_comb,
                                   int path, void* stream) {
  auto* h = (HostCtx*)ctx;
  const MoonepDevCtx& c = h->dev;
  const int grid = imax(1, imin(c.num_sms, h->sm_count));
  const int vec_ok = (c.H % 8 == 0) && ((reinterpret_cast<uintptr_t>(out_hidden) & 15u) == 0);
  if (path == MOONEP_PATH_BULK && vec_ok) {
    PullBulkArgs a;
    a.dst = dst;
    a.out = (uint16_t*)out_hidden;
    a.out_w = out_weights;
    a.wait_epoch = wait_epoch_comb;
    a.kp = imin(c.K, c.R);
    const long long row_bytes = (long long)c.H * 2;
    const long long slot_budget = 28 * 1024;
    a.nsplit = 1;
    for (;;) {
      long long cb = (row_bytes + a.nsplit - 1) / a.nsplit;
      cb = (cb + 15) / 16 * 16;
      a.chunk_bytes = (int)cb;
      if (cb * a.kp <= slot_budget || cb <= 512) break;
      ++a.nsplit;
    }
    const long long slot_bytes = (long long)a.kp * a.chunk_bytes;
    a.nslots = (int)((h->max_smem_optin - 8192) / slot_bytes);
    if (a.nslots > kPullConsumerWarps) a.nslots = kPullConsumerWarps;  // one consumer warp per slot
    if (a.nslots >= 2) {
      const size_t smem = (size_t)a.nslots * slot_bytes;
      if (int rc = check_cuda(cudaFuncSetAttribute(combine_pull_bulk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                   (int)smem),
                              "cudaFuncSetAttribute(combine_pull_bulk_kernel)"))
        return rc;
      combine_pull_bulk_kernel<<<grid, kPullBulkThreads, smem, (cudaStream_t)stream>>>(c, a);
      return check_launch("combine_pull_bulk_kernel");
    }
  }
  combine_pull_kernel<<<grid, 512, 0, (cudaStream_t)stream>>>(c, dst, (uint16_t*)out_hidden, out_weights,
                                                             wait_epoch_comb, vec_ok);
  return check_launch("combine_pull_kernel");
}
