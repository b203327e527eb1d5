// Expert-weight traffic for sm_100a: prefetch of remote experts and reduction of their
// gradients back to the owners, plus the stand-alone signal/wait kernel.
//
//   prefetch     for every slot b of this rank with experts_to_copy[rank][b] = e >= 0, copy expert e
//                (physically on its owner, reached through the peer-mapped part of the weight
//                tensor) into local slot b of the prefetch buffers (slot E+b of the full weight).  Gate, up and down go in one launch; persistent CTAs
//                stride over 16 KB pieces with eight 16-byte loads in flight per lane.
//   grad_accum   the owner of expert e adds every slot (src, b) with experts_to_copy[src][b] == e
//                to its local gradient, in ascending src*B+b order starting from the local value,
//                so results are bitwise reproducible.  Waits for FLAG_GRAD_READY, signals
//                FLAG_GRAD_DONE.
//   grad_clear   after every peer's FLAG_GRAD_DONE each rank zeroes the slots it produced.
//
// Parity: reference moonep_td/prefetch.py:22-64, moonep_td/grad_reduce.py:14-178 (host prescan with
// argsort/bincount and a host sync per tensor, two barriers and two kernels per tensor).
#include <cstdlib>

#include "common.cuh"
#include "host.h"

namespace moonep {

namespace {

constexpr int kMaxTensors = 3;
constexpr int kMaxSlots = 4096;     // R*B entries owned by one rank that grad_accum can list
constexpr int kMaxLocalExperts = 2048;
constexpr int kPieceVec = 4096;     // 16-byte vectors per work item (64 KB)

struct TensorSet {
  void* p[kMaxTensors];
  void* q[kMaxTensors];
  int n;
};

__global__ void __launch_bounds__(256)
    signal_wait_kernel(const MoonepDevCtx c, int signal_family, int signal_epoch, int wait_family, int wait_epoch) {
  if (signal_family >= 0 && !poisoned(c)) {
    if (threadIdx.x == 0) fence_sys();
    __syncthreads();
    for (int r = threadIdx.x; r < c.R; r += blockDim.x)
      st_release_sys(flag_ptr(c, r, signal_family, c.rank), abs_epoch(c, signal_family, signal_epoch));
  }
  if (wait_family >= 0) block_wait_flags(c, wait_family, wait_epoch, MOONEP_K_WAIT);
}

struct BiasValues {
  int v[MOONEP_NUM_FLAG_FAMILIES];
};

__global__ void epoch_bias_kernel(const MoonepDevCtx c, const BiasValues b, int mode) {
  const int f = threadIdx.x;
  if (f < MOONEP_NUM_FLAG_FAMILIES) c.counters[MOONEP_BIAS_OFF + f] = (mode ? c.counters[MOONEP_BIAS_OFF + f] : 0) + b.v[f];
}

// Work items are ordered slot-major, so that the slots fill one after the other; when the last piece of a slot
// (over all tensors) has been copied, the slot's flag is released with the prefetch epoch and a grouped GEMM that
// runs beside this kernel may load that slot's weights (moonep_grouped_gemm_pair_hooked: slot_flags).
__global__ void __launch_bounds__(512)
    prefetch_kernel(const MoonepDevCtx c, const TensorSet w, const int* __restrict__ experts, long long elems,
                    int nslots, int nexperts, int* slot_flags, int* slot_done, int epoch) {
  if (poisoned(c)) return;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const long long nvec = elems / 8;  // bf16: 8 elements per 16 bytes
  const long long pieces = (nvec + kPieceVec - 1) / kPieceVec;
  const long long per_slot = (long long)w.n * pieces;
  const long long total = (long long)nslots * per_slot;
  if (slot_flags != nullptr) {
    epoch = abs_epoch(c, MOONEP_FLAG_PREFETCH, epoch);
    // slots that receive nothing are ready at once
    if (blockIdx.x == 0)
      for (int b = threadIdx.x; b < nslots; b += blockDim.x)
        if (experts[b] < 0 || experts[b] >= nexperts) st_release_gpu(slot_flags + b, epoch);
  }
  for (long long item = (long long)blockIdx.x * nwarps + warp; item < total; item += (long long)gridDim.x * nwarps) {
    const int b = (int)(item / per_slot);
    const long long rest = item - (long long)b * per_slot;
    const int t = (int)(rest / pieces);
    const long long piece = rest - (long long)t * pieces;
    const int e = experts[b];
    if (e < 0) continue;
    if (e >= nexperts) {
      record_status(c, MOONEP_STATUS_BAD_INDEX, MOONEP_K_PREFETCH, 7, e, b, t);
      continue;
    }
    const int4* src = reinterpret_cast<const int4*>(w.p[t]) + (long long)e * nvec;
    int4* dstp = reinterpret_cast<int4*>(w.q[t]) + (long long)b * nvec;
    const long long v0 = piece * kPieceVec;
    const long long v1 = v0 + kPieceVec < nvec ? v0 + kPieceVec : nvec;
    for (long long i0 = v0; i0 < v1; i0 += 32 * 8) {
      int4 v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const long long i = i0 + j * 32 + lane;
        if (i < v1) v[j] = ld16(src + i);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const long long i = i0 + j * 32 + lane;
        if (i < v1) st16(dstp + i, v[j]);
      }
    }
    if (slot_flags != nullptr) {
      __syncwarp();
      if (lane == 0) {
        fence_gpu();
        if (atomicAdd(slot_done + b, 1) == (int)per_slot - 1) {
          slot_done[b] = 0;
          fence_gpu();
          st_relaxed_gpu(slot_flags + b, epoch);
        }
      }
    }
  }
}

__device__ __forceinline__ float4 ld16f(const float4* p) {
  int4 v = ld16(p);
  return make_float4(__int_as_float(v.x), __int_as_float(v.y), __int_as_float(v.z), __int_as_float(v.w));
}

__device__ __forceinline__ void st16f(float4* p, const float4& f) {
  st16(p, make_int4(__float_as_int(f.x), __float_as_int(f.y), __float_as_int(f.z), __float_as_int(f.w)));
}

constexpr int kAccLd = 6;  // 16-byte loads per lane and slot in flight (3 KB per warp; 8 would spill at 24 warps per SM)

// One CTA of 24 warps per SM, num_sms CTAs: remote reads are latency bound, so every resident warp counts, and the
// grid stays within the SMs the Buffer was told to use for traffic between ranks.
constexpr int kAccumThreads = 768;

__global__ void __launch_bounds__(kAccumThreads, 1)
    grad_accum_kernel(const MoonepDevCtx c, const TensorSet ts, const int* __restrict__ etc, int Bcols, long long elems,
                      int wait_epoch, int signal_epoch) {
  __shared__ int s_rb[kMaxSlots];
  __shared__ short s_le[kMaxSlots];
  __shared__ short s_active[kMaxLocalExperts];
  __shared__ unsigned char s_has[kMaxLocalExperts];
  __shared__ int s_n, s_nactive;
  const bool ok = block_wait_flags(c, MOONEP_FLAG_GRAD_READY, wait_epoch, MOONEP_K_GRAD_ACCUM);
  if (ok) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int epn = c.epn, owner0 = c.rank * epn, nslots = c.R * Bcols;
    for (int i = threadIdx.x; i < epn; i += blockDim.x) s_has[i] = 0;
    __syncthreads();
    if (warp == 0) {
      int n = 0;
      for (int base = 0; base < nslots; base += 32) {
        const int rb = base + lane;
        const int e = rb < nslots ? etc[rb] : -1;
        const bool mine = e >= owner0 && e < owner0 + epn;
        const unsigned m = __ballot_sync(0xffffffffu, mine);
        if (mine) {
          const int pos = n + __popc(m & ((1u << lane) - 1u));
          if (pos < kMaxSlots) {
            s_rb[pos] = rb;
            s_le[pos] = (short)(e - owner0);
          }
          s_has[e - owner0] = 1;
        }
        n += __popc(m);
      }
      __syncwarp();
      int na = 0;
      for (int base = 0; base < epn; base += 32) {
        const int le = base + lane;
        const bool has = le < epn && s_has[le];
        const unsigned m = __ballot_sync(0xffffffffu, has);
        if (has) s_active[na + __popc(m & ((1u << lane) - 1u))] = (short)le;
        na += __popc(m);
      }
      if (lane == 0) {
        s_n = n < kMaxSlots ? n : kMaxSlots;
        s_nactive = na;
        if (n > kMaxSlots) record_status(c, MOONEP_STATUS_BAD_INDEX, MOONEP_K_GRAD_ACCUM, 8, n, kMaxSlots, 0);
      }
    }
    __syncthreads();
    const int n = s_n, na = s_nactive;
    const long long nvec = elems / 4;  // fp32: 4 elements per 16 bytes
    const long long pieces = (nvec + kPieceVec - 1) / kPieceVec;
    const long long total = (long long)ts.n * na * pieces;
    for (long long item = (long long)blockIdx.x * nwarps + warp; item < total; item += (long long)gridDim.x * nwarps) {
      const long long piece = item % pieces;
      const int ai = (int)((item / pieces) % na);
      const int t = (int)(item / (pieces * na));
      const int le = s_active[ai];
      float4* g = reinterpret_cast<float4*>(ts.p[t]) + (long long)(owner0 + le) * nvec;
      const float4* red = reinterpret_cast<const float4*>(ts.q[t]);
      const long long v0 = piece * kPieceVec;
      const long long v1 = v0 + kPieceVec < nvec ? v0 + kPieceVec : nvec;
      for (long long i0 = v0; i0 < v1; i0 += 32 * kAccLd) {
        float4 acc[kAccLd];
#pragma unroll
        for (int j = 0; j < kAccLd; ++j) {
          const long long i = i0 + j * 32 + lane;
          if (i < v1) acc[j] = ld16f(g + i);
        }
        for (int s = 0; s < n; ++s) {
          if (s_le[s] != le) continue;
          const float4* src = red + (long long)s_rb[s] * nvec;
          float4 v[kAccLd];
#pragma unroll
          for (int j = 0; j < kAccLd; ++j) {
            const long long i = i0 + j * 32 + lane;
            if (i < v1) v[j] = ld16f(src + i);
          }
#pragma unroll
          for (int j = 0; j < kAccLd; ++j) {
            const long long i = i0 + j * 32 + lane;
            if (i < v1) {
              acc[j].x += v[j].x;
              acc[j].y += v[j].y;
              acc[j].z += v[j].z;
              acc[j].w += v[j].w;
            }
          }
        }
#pragma unroll
        for (int j = 0; j < kAccLd; ++j) {
          const long long i = i0 + j * 32 + lane;
          if (i < v1) st16f(g + i, acc[j]);
        }
      }
    }
  }
  grid_tail_signal(c, MOONEP_K_GRAD_ACCUM, ok ? MOONEP_FLAG_GRAD_DONE : -1, signal_epoch);
}

// prefetch_weight through per-warp cp.async rings (MOONEP_PREFETCH_PATH=async, the default).  Register loads keep at
// most a few KB per warp in flight, which over NVLink (several microseconds per round trip) bounds a pull below the
// link rate.  Here every warp owns a ring of 2 KB shared-memory stages and fills them with 16-byte cp.async copies
// (the same load path as register loads, but the data waits in shared memory, not in registers); every lane stores
// what it copied itself, so the warps need no barrier.  Work items are 256 KB pieces in slot-major order, so the
// first slots complete (and are flagged) first.  Measured on 2 B200 (2.8 GB per rank): 668 GB/s against 629 GB/s of
// the register kernel, the same with 3, 4, 5 or 6 stages.  The same ring under grad_accum measured half the rate of
// its register kernel (244 against 489 GB/s), whatever the ring depth, the piece size, the completion mechanism
// (cp.async groups or an mbarrier per stage) and whether the data was consumed at all; that variant was dropped.
constexpr int kCaThreads = 512;
constexpr int kCaWarps = kCaThreads / 32;
constexpr int kCaStages = 4;
constexpr int kCaMaxStages = 6;
constexpr int kCaLaneVec = 4;                  // 16-byte vectors per lane and stage
constexpr int kCaChunkVec = 32 * kCaLaneVec;   // a stage: 128 vectors = 2 KB
constexpr int kCaPieceVec = 16384;             // work item: 256 KB of one expert

template <int kStages>
__global__ void __launch_bounds__(kCaThreads, 1)
    prefetch_async_kernel(const MoonepDevCtx c, const TensorSet w, const int* __restrict__ experts, long long elems,
                          int nslots, int nexperts, int* slot_flags, int* slot_done, int epoch) {
  extern __shared__ __align__(16) unsigned char s_ca_ring[];
  if (poisoned(c)) return;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long nvec = elems / 8;  // bf16: 8 elements per 16 bytes
  const long long pieces = (nvec + kCaPieceVec - 1) / kCaPieceVec;
  const long long per_slot = (long long)w.n * pieces;
  const long long total = (long long)nslots * per_slot;
  if (slot_flags != nullptr) {
    epoch = abs_epoch(c, MOONEP_FLAG_PREFETCH, epoch);
    if (blockIdx.x == 0)
      for (int b = threadIdx.x; b < nslots; b += blockDim.x)
        if (experts[b] < 0 || experts[b] >= nexperts) st_release_gpu(slot_flags + b, epoch);
  }
  int4* ring = reinterpret_cast<int4*>(s_ca_ring) + (size_t)warp * kStages * kCaChunkVec;
  for (long long item = (long long)blockIdx.x * kCaWarps + warp; item < total; item += (long long)gridDim.x * kCaWarps) {
    const int b = (int)(item / per_slot);
    const long long rest = item - (long long)b * per_slot;
    const int t = (int)(rest / pieces);
    const long long piece = rest - (long long)t * pieces;
    const int e = experts[b];
    if (e < 0) continue;
    if (e >= nexperts) {
      record_status(c, MOONEP_STATUS_BAD_INDEX, MOONEP_K_PREFETCH, 7, e, b, t);
      continue;
    }
    const int4* src = reinterpret_cast<const int4*>(w.p[t]) + (long long)e * nvec;
    int4* dstp = reinterpret_cast<int4*>(w.q[t]) + (long long)b * nvec;
    const long long v0 = piece * kCaPieceVec;
    const long long v1 = v0 + kCaPieceVec < nvec ? v0 + kCaPieceVec : nvec;
    const int steps = (int)((v1 - v0 + kCaChunkVec - 1) / kCaChunkVec);
    auto issue = [&](int q) {
      int4* dst = ring + (size_t)(q % kStages) * kCaChunkVec;
      const long long base = v0 + (long long)q * kCaChunkVec;
#pragma unroll
      for (int k = 0; k < kCaLaneVec; ++k) {
        const long long i = base + k * 32 + lane;
        if (i < v1) cp_async16(dst + k * 32 + lane, src + i);
      }
    };
    for (int q = 0; q < kStages; ++q) {
      if (q < steps) issue(q);
      cp_async_commit();
    }
    for (int q = 0; q < steps; ++q) {
      cp_async_wait<kStages - 1>();
      const int4* st = ring + (size_t)(q % kStages) * kCaChunkVec;
      const long long base = v0 + (long long)q * kCaChunkVec;
#pragma unroll
      for (int k = 0; k < kCaLaneVec; ++k) {
        const long long i = base + k * 32 + lane;
        if (i < v1) st16(dstp + i, st[k * 32 + lane]);
      }
      if (q + kStages < steps) issue(q + kStages);
      cp_async_commit();
    }
    cp_async_wait<0>();
    if (slot_flags != nullptr) {
      __syncwarp();
      if (lane == 0) {
        fence_gpu();
        if (atomicAdd(slot_done + b, 1) == (int)per_slot - 1) {
          slot_done[b] = 0;
          fence_gpu();
          st_relaxed_gpu(slot_flags + b, epoch);
        }
      }
    }
  }
}

// Bulk-copy variant of grad_accum (selected with MOONEP_GRAD_PATH=bulk; measured slower than the register
// path on B200 NVLink, where bulk loads from peer memory run below LSU loads): warp 0 streams the remote slots into a shared-memory ring with
// cp.async.bulk (one 32 KB piece per stage, completion counted on the stage's "full" mbarrier) while
// warps 1..8 hold the local gradient piece in registers, add the staged slots in ascending slot order
// and write the piece back.  All consumer warps work on the same stage, so they advance in lockstep
// and the parity waits stay unambiguous.  The deep ring keeps several hundred KB per SM in flight on
// NVLink, which register loads cannot.
constexpr int kAccConsumerWarps = 8;
constexpr int kAccThreads = 32 * (1 + kAccConsumerWarps);
constexpr int kAccPieceVec = 2048;  // 16-byte vectors per stage (32 KB)
constexpr int kAccMaxStages = 8;

__global__ void __launch_bounds__(kAccThreads)
    grad_accum_bulk_kernel(const MoonepDevCtx c, const TensorSet ts, const int* __restrict__ etc, int Bcols,
                           long long elems, int wait_epoch, int signal_epoch, int nstages) {
  extern __shared__ __align__(128) unsigned char s_ring[];  // [nstages][kAccPieceVec * 16]
  __shared__ __align__(8) unsigned long long s_full[kAccMaxStages], s_empty[kAccMaxStages];
  __shared__ int s_rb[kMaxSlots];
  __shared__ short s_le[kMaxSlots];
  __shared__ short s_active[kMaxLocalExperts];
  __shared__ unsigned char s_has[kMaxLocalExperts];
  __shared__ int s_n, s_nactive, s_fail;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x < nstages) {
    mbar_init(s_full + threadIdx.x, 1);
    mbar_init(s_empty + threadIdx.x, kAccConsumerWarps);
  }
  if (threadIdx.x == 0) s_fail = 0;
  fence_barrier_init();
  const bool ok = block_wait_flags(c, MOONEP_FLAG_GRAD_READY, wait_epoch, MOONEP_K_GRAD_ACCUM);
  if (ok) {
    const int epn = c.epn, owner0 = c.rank * epn, nslots = c.R * Bcols;
    for (int i = threadIdx.x; i < epn; i += blockDim.x) s_has[i] = 0;
    __syncthreads();
    if (warp == 0) {
      int n = 0;
      for (int base = 0; base < nslots; base += 32) {
        const int rb = base + lane;
        const int e = rb < nslots ? etc[rb] : -1;
        const bool mine = e >= owner0 && e < owner0 + epn;
        const unsigned m = __ballot_sync(0xffffffffu, mine);
        if (mine) {
          const int pos = n + __popc(m & ((1u << lane) - 1u));
          if (pos < kMaxSlots) {
            s_rb[pos] = rb;
            s_le[pos] = (short)(e - owner0);
          }
          s_has[e - owner0] = 1;
        }
        n += __popc(m);
      }
      __syncwarp();
      int na = 0;
      for (int base = 0; base < epn; base += 32) {
        const int le = base + lane;
        const bool has = le < epn && s_has[le];
        const unsigned m = __ballot_sync(0xffffffffu, has);
        if (has) s_active[na + __popc(m & ((1u << lane) - 1u))] = (short)le;
        na += __popc(m);
      }
      if (lane == 0) {
        s_n = n < kMaxSlots ? n : kMaxSlots;
        s_nactive = na;
        if (n > kMaxSlots) record_status(c, MOONEP_STATUS_BAD_INDEX, MOONEP_K_GRAD_ACCUM, 8, n, kMaxSlots, 0);
      }
    }
    __syncthreads();
    const int n = s_n, na = s_nactive;
    const long long nvec = elems / 4;
    const long long pieces = (nvec + kAccPieceVec - 1) / kAccPieceVec;
    const long long total = (long long)ts.n * na * pieces;
    if (warp == 0) {
      // ---------------- producer ----------------
      if (lane == 0) {
        long long k = 0;
        bool failed = false;
        for (long long item = blockIdx.x; item < total && !failed; item += gridDim.x) {
          const long long piece = item % pieces;
          const int ai = (int)((item / pieces) % na);
          const int t = (int)(item / (pieces * na));
          const int le = s_active[ai];
          const long long v0 = piece * kAccPieceVec;
          const unsigned bytes = (unsigned)((nvec - v0 < kAccPieceVec ? nvec - v0 : kAccPieceVec) * 16);
          const unsigned char* red = reinterpret_cast<const unsigned char*>(ts.q[t]);
          for (int s = 0; s < n && !failed; ++s) {
            if (s_le[s] != le) continue;
            const int stage = (int)(k % nstages);
            const long long use = k / nstages;
            if (use > 0 && !mbar_wait(s_empty + stage, (unsigned)((use - 1) & 1), c.timeout_ns)) {
              record_status(c, MOONEP_STATUS_TIMEOUT, MOONEP_K_GRAD_ACCUM, 101, stage, (int)use, 0);
              s_fail = 1;
              failed = true;
              break;
            }
            mbar_expect_tx(s_full + stage, bytes);
            bulk_g2s(s_ring + (size_t)stage * kAccPieceVec * 16, red + ((long long)s_rb[s] * nvec + v0) * 16, bytes,
                     s_full + stage);
            ++k;
          }
        }
      }
      __syncwarp();
    } else {
      // ---------------- consumers ----------------
      const int ctid = threadIdx.x - 32, cthreads = kAccConsumerWarps * 32;
      constexpr int kPer = kAccPieceVec / (kAccConsumerWarps * 32);  // vectors per thread and piece
      long long k = 0;
      bool failed = false;
      // the local gradient piece of the next item is loaded while the current one is being reduced
      auto coords = [&](long long item, int& le, long long& v0, long long& v1, float4*& g) {
        const long long piece = item % pieces;
        const int ai = (int)((item / pieces) % na);
        const int t = (int)(item / (pieces * na));
        le = s_active[ai];
        v0 = piece * kAccPieceVec;
        v1 = v0 + kAccPieceVec < nvec ? v0 + kAccPieceVec : nvec;
        g = reinterpret_cast<float4*>(ts.p[t]) + (long long)(owner0 + le) * nvec;
      };
      float4 nxt[kPer];
      if ((long long)blockIdx.x < total) {
        int le0;
        long long a0, a1;
        float4* g0;
        coords(blockIdx.x, le0, a0, a1, g0);
#pragma unroll
        for (int j = 0; j < kPer; ++j) {
          const long long i = a0 + j * cthreads + ctid;
          if (i < a1) nxt[j] = ld16f(g0 + i);
        }
      }
      for (long long item = blockIdx.x; item < total && !failed; item += gridDim.x) {
        int le;
        long long v0, v1;
        float4* g;
        coords(item, le, v0, v1, g);
        float4 acc[kPer];
#pragma unroll
        for (int j = 0; j < kPer; ++j) acc[j] = nxt[j];
        if (item + gridDim.x < total) {
          int le2;
          long long b0, b1;
          float4* g2;
          coords(item + gridDim.x, le2, b0, b1, g2);
#pragma unroll
          for (int j = 0; j < kPer; ++j) {
            const long long i = b0 + j * cthreads + ctid;
            if (i < b1) nxt[j] = ld16f(g2 + i);
          }
        }
        for (int s = 0; s < n && !failed; ++s) {
          if (s_le[s] != le) continue;
          const int stage = (int)(k % nstages);
          const unsigned par = (unsigned)((k / nstages) & 1);
          bool got = mbar_try_wait(s_full + stage, par);
          if (!got) {
            const unsigned long long t0 = globaltimer_ns();
            unsigned spins = 0;
            while (!(got = mbar_try_wait(s_full + stage, par))) {
              if ((++spins & 255u) == 0 && (*(volatile int*)&s_fail || globaltimer_ns() - t0 > c.timeout_ns)) break;
            }
          }
          if (!got) {
            if (!*(volatile int*)&s_fail) record_status(c, MOONEP_STATUS_TIMEOUT, MOONEP_K_GRAD_ACCUM, 102, stage, 0, 0);
            failed = true;
            break;
          }
          const float4* st = reinterpret_cast<const float4*>(s_ring + (size_t)stage * kAccPieceVec * 16);
#pragma unroll
          for (int j = 0; j < kPer; ++j) {
            const long long i = v0 + j * cthreads + ctid;
            if (i < v1) {
              const float4 v = st[j * cthreads + ctid];
              acc[j].x += v.x;
              acc[j].y += v.y;
              acc[j].z += v.z;
              acc[j].w += v.w;
            }
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(s_empty + stage);
          ++k;
        }
        if (failed) break;
#pragma unroll
        for (int j = 0; j < kPer; ++j) {
          const long long i = v0 + j * cthreads + ctid;
          if (i < v1) st16f(g + i, acc[j]);
        }
      }
    }
  }
  grid_tail_signal(c, MOONEP_K_GRAD_ACCUM, ok ? MOONEP_FLAG_GRAD_DONE : -1, signal_epoch);
}

__global__ void __launch_bounds__(512)
    grad_clear_kernel(const MoonepDevCtx c, const TensorSet ts, const int* __restrict__ etc, int Bcols, long long elems,
                      int wait_epoch) {
  if (!block_wait_flags(c, MOONEP_FLAG_GRAD_DONE, wait_epoch, MOONEP_K_GRAD_CLEAR)) return;
  // one (tensor, slot) pair at a time; inside a slot the CTAs stride over 16-byte vectors, so there is no
  // 64-bit division per element and every CTA streams contiguous memory
  const long long nvec = elems / 4;
  const int4 z = make_int4(0, 0, 0, 0);
  for (int t = 0; t < ts.n; ++t) {
    for (int b = 0; b < Bcols; ++b) {
      if (etc[c.rank * Bcols + b] < 0) continue;
      int4* base = reinterpret_cast<int4*>(ts.q[t]) + ((long long)c.rank * Bcols + b) * nvec;
      for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < nvec; v += (long long)gridDim.x * blockDim.x)
        st16(base + v, z);
    }
  }
}

}  // namespace

}  // namespace moonep

using namespace moonep;

extern "C" int moonep_signal_wait(void* ctx, int signal_family, int signal_epoch, int wait_family, int wait_epoch,
                                  void* stream) {
  auto* h = (HostCtx*)ctx;
  signal_wait_kernel<<<1, 128, 0, (cudaStream_t)stream>>>(h->dev, signal_family, signal_epoch, wait_family, wait_epoch);
  return check_launch("signal_wait_kernel");
}

extern "C" int moonep_epoch_bias(void* ctx, const int* values, int mode, void* stream) {
  auto* h = (HostCtx*)ctx;
  BiasValues b;
  for (int f = 0; f < MOONEP_NUM_FLAG_FAMILIES; ++f) b.v[f] = values[f];
  epoch_bias_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(h->dev, b, mode);
  return check_launch("epoch_bias_kernel");
}

// Ring depth of the cp.async kernels: MOONEP_RING_STAGES (2..6), default kCaStages.
static int ring_stages() {
  const char* v = getenv("MOONEP_RING_STAGES");
  const int n = v != nullptr ? atoi(v) : kCaStages;
  return n >= 2 && n <= kCaMaxStages ? n : kCaStages;
}

extern "C" int moonep_prefetch(void* ctx, void* const* src3, void* const* dst3, int n_tensors,
                               const int* experts_to_copy_row, long long elems, int nslots, int nexperts, int path,
                               int* slot_flags, int* slot_done, int epoch, void* stream) {
  auto* h = (HostCtx*)ctx;
  const MoonepDevCtx& c = h->dev;
  if (n_tensors < 1 || n_tensors > kMaxTensors || elems % 8 != 0) {
    set_error("moonep_prefetch: 1..3 tensors with H*Hp a multiple of 8 expected");
    return 1;
  }
  if (nslots <= 0) return 0;
  TensorSet w;
  w.n = n_tensors;
  for (int i = 0; i < kMaxTensors; ++i) {
    w.p[i] = i < n_tensors ? src3[i] : nullptr;
    w.q[i] = i < n_tensors ? dst3[i] : nullptr;
  }
  const int grid = imax(1, imin(c.num_sms, h->sm_count));
  if (path == MOONEP_PATH_ASYNC) {
    const int stages = ring_stages();
    const size_t smem = (size_t)kCaWarps * stages * kCaChunkVec * 16;
    auto launch = [&](auto kernel) -> int {
      if (int rc = check_cuda(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem),
                              "cudaFuncSetAttribute(prefetch_async_kernel)"))
        return rc;
      kernel<<<grid, kCaThreads, smem, (cudaStream_t)stream>>>(c, w, experts_to_copy_row, elems, nslots, nexperts,
                                                               slot_flags, slot_done, epoch);
      return check_launch("prefetch_async_kernel");
    };
    switch (stages) {
      case 2: return launch(prefetch_async_kernel<2>);
      case 4: return launch(prefetch_async_kernel<4>);
      case 5: return launch(prefetch_async_kernel<5>);
      case 6: return launch(prefetch_async_kernel<6>);
      default: return launch(prefetch_async_kernel<3>);
    }
  }
  prefetch_kernel<<<grid, 512, 0, (cudaStream_t)stream>>>(c, w, experts_to_copy_row, elems, nslots, nexperts, slot_flags,
                                                         slot_done, epoch);
  return check_launch("prefetch_kernel");
}

extern "C" int moonep_grad_reduce(void* ctx, float* const* grads, float* const* reduce, int n_tensors,
                                  const int* experts_to_copy, int Bcols, long long elems, int epoch_ready,
                                  int epoch_done, int phase, int path, void* stream) {
  auto* h = (HostCtx*)ctx;
  const MoonepDevCtx& c = h->dev;
  if (n_tensors < 1 || n_tensors > kMaxTensors || elems % 4 != 0) {
    set_error("moonep_grad_reduce: 1..3 tensors with H*Hp a multiple of 4 expected");
    return 1;
  }
  if (c.epn > kMaxLocalExperts) {
    set_error("moonep_grad_reduce: more than 2048 experts per rank");
    return 1;
  }
  TensorSet ts;
  ts.n = n_tensors;
  for (int i = 0; i < kMaxTensors; ++i) {
    ts.p[i] = i < n_tensors ? (void*)grads[i] : nullptr;
    ts.q[i] = i < n_tensors ? (void*)reduce[i] : nullptr;
  }
  const int grid = imax(1, imin(c.num_sms, h->sm_count));
  cudaStream_t st = (cudaStream_t)stream;
  if (phase == 1) {
    const size_t stage_bytes = (size_t)kAccPieceVec * 16;
    int nstages = (int)((h->max_smem_optin - 40 * 1024) / (long long)stage_bytes);  // static tables take ~30 KB
    if (nstages > kAccMaxStages) nstages = kAccMaxStages;
    if (path == MOONEP_PATH_BULK && nstages >= 2) {
      const size_t smem = (size_t)nstages * stage_bytes;
      if (int rc = check_cuda(cudaFuncSetAttribute(grad_accum_bulk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                   (int)smem),
                              "cudaFuncSetAttribute(grad_accum_bulk_kernel)"))
        return rc;
      grad_accum_bulk_kernel<<<grid, kAccThreads, smem, st>>>(c, ts, experts_to_copy, Bcols, elems, epoch_ready,
                                                             epoch_done, nstages);
      return check_launch("grad_accum_bulk_kernel");
    }
    grad_accum_kernel<<<grid, kAccumThreads, 0, st>>>(c, ts, experts_to_copy, Bcols, elems, epoch_ready, epoch_done);
    return check_launch("grad_accum_kernel");
  }
  if (phase == 2) {
    if (Bcols == 0) return 0;
    // the slots are this rank's own memory: all SMs may help
    grad_clear_kernel<<<imax(1, imin(c.local_sms, h->sm_count)), 512, 0, st>>>(c, ts, experts_to_copy, Bcols, elems,
                                                                            epoch_done);
    return check_launch("grad_clear_kernel");
  }
  set_error("moonep_grad_reduce: phase must be 1 (accumulate) or 2 (clear)");
  return 1;
}
