// Device helpers shared by all kernels: epoch flags with bounded waits, the status
// block, vector copies, mbarrier / bulk-copy PTX wrappers.
//
// Cross-rank ordering protocol
// ----------------------------
// Every meta chunk ends with flags[family][src] (int32).  A producer kernel on rank s
// finishes its writes into peer memory, then its last CTA stores the family's epoch into
// flags[family][s] on every peer (st.release.sys after a system fence).  A consumer kernel
// spins at its head on its own flags with ld.acquire.sys until all R flags reached the
// epoch.  Epochs only grow, so a flag never needs to be reset and a late reader cannot
// miss a signal.  This replaces the reference's grid barrier + nvshmem_barrier_all pair
// (moonep_td/_common.py:49-82), whose reset races with late spinners.
//
// Epoch arguments are relative: a kernel adds the per-family bias kept in device memory
// (counters[MOONEP_BIAS_OFF + family]) to the epoch it was launched with.  The bias is zero
// for ordinary launches; a captured CUDA graph carries small epochs relative to its capture
// point and ends with a kernel that advances the bias by the epochs one replay consumes, so
// the same graph can be replayed any number of times (moonep_epoch_bias in moonep.h).
//
// Every wait is bounded by ctx.timeout_ns of %globaltimer.  When it runs out the kernel
// records {code, kernel, family, peer, expected, seen} in the status block and returns;
// later kernels of the same Buffer see the non-zero status and return at once, so a
// lost peer turns into an error the host can read instead of a hang.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "moonep.h"

namespace moonep {

__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ void st_release_gpu(int* p, int v) {
  asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Plain strong stores; with a fence of the matching scope earlier in the same thread they form a release.
__device__ __forceinline__ void st_relaxed_sys(int* p, int v) {
  asm volatile("st.relaxed.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_relaxed_gpu(int* p, int v) {
  asm volatile("st.relaxed.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void fence_gpu() { asm volatile("fence.acq_rel.gpu;" ::: "memory"); }

__device__ __forceinline__ int ld_volatile(const int* p) {
  int v;
  asm volatile("ld.volatile.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ void fence_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }

__device__ __forceinline__ int* flag_ptr(const MoonepDevCtx& c, int on_rank, int family, int src) {
  return c.meta_peer[on_rank] + c.sync_off + family * c.r32 + src;
}

__device__ __forceinline__ void record_status(const MoonepDevCtx& c, int code, int kernel, int family, int peer,
                                              int expect, int seen) {
  if (atomicCAS(c.status + MOONEP_ST_CODE, 0, code) == 0) {
    c.status[MOONEP_ST_KERNEL] = kernel;
    c.status[MOONEP_ST_FAMILY] = family;
    c.status[MOONEP_ST_PEER] = peer;
    c.status[MOONEP_ST_EXPECT] = expect;
    c.status[MOONEP_ST_SEEN] = seen;
    __threadfence();
  }
}

// Phase statistics: one thread of a CTA reports how long a phase took; the longest one over the CTAs is kept.
__device__ __forceinline__ void stat_phase(const MoonepDevCtx& c, int phase, unsigned long long t0) {
  atomicMax(reinterpret_cast<unsigned long long*>(c.stats) + MOONEP_STAT_PHASE_NS + phase, globaltimer_ns() - t0);
}

// Programmatic dependent launch: everything before this call may run while the previous kernel of the stream is
// still finishing; after it, that kernel has completed and its writes are visible.  A no-op for ordinary launches.
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// Lets a kernel launched with programmatic stream serialisation behind this one start its CTAs as soon as SMs have room
// (it still waits in griddepcontrol.wait until this grid has completed and its writes are visible).
__device__ __forceinline__ void griddep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Absolute epoch of a launch argument: argument + this family's bias (see the header comment).
__device__ __forceinline__ int abs_epoch(const MoonepDevCtx& c, int family, int epoch) {
  return epoch + ld_volatile(c.counters + MOONEP_BIAS_OFF + family);
}

// True if an earlier kernel of this Buffer failed; the caller returns immediately.
__device__ __forceinline__ bool poisoned(const MoonepDevCtx& c) { return ld_volatile(c.status + MOONEP_ST_CODE) != 0; }

// Block-wide: wait until flags[family][r] >= epoch for all r.  Returns false (to every
// thread) on timeout or if the context is already poisoned.  Must be called by all threads.
__device__ __forceinline__ bool block_wait_flags(const MoonepDevCtx& c, int family, int epoch, int kernel_id) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = poisoned(c) ? 0 : 1;
  __syncthreads();
  if (family >= 0 && s_ok) {
    epoch = abs_epoch(c, family, epoch);
    for (int r = threadIdx.x; r < c.R; r += blockDim.x) {
      const int* f = flag_ptr(c, c.rank, family, r);
      int v = ld_acquire_sys(f);
      if (v - epoch < 0) {
        const unsigned long long t0 = globaltimer_ns();
        unsigned spins = 0;
        while ((v = ld_acquire_sys(f)) - epoch < 0) {
          if ((++spins & 63u) == 0) {
            if (globaltimer_ns() - t0 > c.timeout_ns || poisoned(c)) {
              record_status(c, MOONEP_STATUS_TIMEOUT, kernel_id, family, r, epoch, v);
              s_ok = 0;
              break;
            }
          }
          __nanosleep(64);
        }
        // wait statistics: longest wait on this family and number of waits that had to spin
        if (blockIdx.x == 0) {
          atomicMax(reinterpret_cast<unsigned long long*>(c.stats) + MOONEP_STAT_WAIT_MAX_NS + family,
                    globaltimer_ns() - t0);
          atomicAdd(reinterpret_cast<unsigned long long*>(c.stats) + MOONEP_STAT_WAIT_COUNT + family, 1ull);
        }
      }
    }
  }
  __syncthreads();
  const bool ok = s_ok != 0;
  __syncthreads();
  return ok;
}

// Block-wide: wait until counters[word] >= epoch, a value another CTA of this GPU publishes with
// st_release_gpu (e.g. "the planner tables of this dispatch are ready").  Returns false (to every thread) on
// timeout or if the context is poisoned.  Must be called by all threads.
__device__ __forceinline__ bool wait_local_epoch(const MoonepDevCtx& c, int word, int epoch, int kernel_id) {
  __shared__ int s_ok;
  __syncthreads();
  if (threadIdx.x == 0) {
    int ok = poisoned(c) ? 0 : 1;
    const int* p = c.counters + word;
    int v;
    if (ok && (v = ld_acquire_gpu(p)) - epoch < 0) {
      const unsigned long long t0 = globaltimer_ns();
      unsigned spins = 0;
      while ((v = ld_acquire_gpu(p)) - epoch < 0) {
        if ((++spins & 63u) == 0 && (globaltimer_ns() - t0 > c.timeout_ns || poisoned(c))) {
          record_status(c, MOONEP_STATUS_TIMEOUT, kernel_id, 64 + word, c.rank, epoch, v);
          ok = 0;
          break;
        }
        __nanosleep(64);
      }
    }
    s_ok = ok;
  }
  __syncthreads();
  const bool ok = s_ok != 0;
  __syncthreads();
  return ok;
}

// Kernel tail: after all of this CTA's writes, the last CTA to arrive stores `epoch` into
// flags[family][rank] on every peer.  Must be called by all threads of every CTA.
__device__ __forceinline__ void grid_tail_signal(const MoonepDevCtx& c, int counter_id, int family, int epoch) {
  __shared__ int s_last;
  __syncthreads();
  if (threadIdx.x == 0) {
    fence_sys();
    const int arrived = atomicAdd(c.counters + counter_id, 1);
    s_last = (arrived == (int)gridDim.x - 1);
    if (s_last) {
      c.counters[counter_id] = 0;
      fence_sys();
    }
  }
  __syncthreads();
  if (s_last && family >= 0) {
    epoch = abs_epoch(c, family, epoch);
    for (int r = threadIdx.x; r < c.R; r += blockDim.x) st_release_sys(flag_ptr(c, r, family, c.rank), epoch);
  }
}

// ---- 16-byte accesses --------------------------------------------------------------------

__device__ __forceinline__ int4 ld16(const void* p) {
  int4 v;
  asm volatile("ld.global.L1::no_allocate.v4.s32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ void st16(void* p, const int4& v) {
  asm volatile("st.global.L1::no_allocate.v4.s32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
}

__device__ __forceinline__ float bf16lo(unsigned u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf16hi(unsigned u) { return __uint_as_float(u & 0xffff0000u); }

__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}

// ---- shared-memory barriers and bulk copies (sm_90+; used here on sm_100a) ---------------

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(unsigned long long* bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}

__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(unsigned long long* bar, unsigned parity) {
  unsigned ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait on an mbarrier phase; false if the budget ran out.
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, unsigned parity, unsigned long long timeout_ns) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = globaltimer_ns();
  unsigned spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 255u) == 0 && globaltimer_ns() - t0 > timeout_ns) return false;
  }
  return true;
}

__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
// All state spaces: orders this thread's view of global memory written with ordinary stores before bulk copies it issues next.
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

// global -> shared of this CTA, completion on an mbarrier.
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gsrc, unsigned bytes, unsigned long long* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

// shared -> global (bulk async group).
__device__ __forceinline__ void bulk_s2g(void* gdst, const void* smem_src, unsigned bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_u32(smem_src)),
               "r"(bytes)
               : "memory");
}

// 16-byte asynchronous copy global -> shared through the load/store path (L2 only), grouped per thread.
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned)__cvta_generic_to_shared(smem)), "l"(gmem)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }

template <int N>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}

template <int N>
__device__ __forceinline__ void bulk_wait() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

}  // namespace moonep
