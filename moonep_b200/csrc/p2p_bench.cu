// Measurement kernel: how fast can SMs push memory to a peer with bulk copies?  `grid` CTAs stream a local buffer into
// a peer's buffer through the same kind of shared-memory ring the dispatch send role uses (cp.async.bulk global ->
// shared on an mbarrier, shared -> peer global in bulk groups, loads two pieces ahead of the stores), without any
// routing, flags or gate weights.  The rate it reaches is the ceiling of the send and push roles; the copy engines'
// rate (a plain device-to-device copy) is measured beside it by bench.py --config p2p_peak.
#include "common.cuh"
#include "host.h"

namespace moonep {

namespace {

constexpr int kPbCopyWarps = 4;  // one lane of each drives a ring
constexpr int kPbThreads = 32 * kPbCopyWarps;
constexpr int kPbStages = 3;

// Warps beyond the first kPbCopyWarps (if the launch has any) do what the flag helpers of the send and push roles do
// all the time, a system-scope fence and one 4-byte store to the peer, until the copy warps are done: the difference
// to a launch without them is what that costs the transfers of the same SM.
__global__ void __launch_bounds__(kPbThreads + 128, 1)
    peer_store_kernel(unsigned char* __restrict__ dst, const unsigned char* __restrict__ src, long long bytes, int chunk,
                      unsigned long long timeout_ns, int* error, int* peer_word) {
  extern __shared__ __align__(128) unsigned char s_ring[];  // [warps][kPbStages][chunk]
  __shared__ __align__(8) unsigned long long s_bar[kPbCopyWarps * kPbStages];
  __shared__ int s_finished;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = kPbCopyWarps;
  if (threadIdx.x < nwarps * kPbStages) mbar_init(s_bar + threadIdx.x, 1);
  if (threadIdx.x == 0) s_finished = 0;
  fence_barrier_init();
  __syncthreads();
  if (lane != 0) return;
  if (warp >= kPbCopyWarps) {
    const unsigned long long t0 = globaltimer_ns();
    int v = 0;
    while (*(volatile int*)&s_finished < kPbCopyWarps && globaltimer_ns() - t0 < timeout_ns) {
      fence_sys();
      if (peer_word != nullptr) st_relaxed_sys(peer_word + (blockIdx.x * 4 + (warp - kPbCopyWarps)) * 32, ++v);
    }
    return;
  }
  unsigned char* ring = s_ring + (size_t)warp * kPbStages * chunk;
  unsigned long long* bar = s_bar + warp * kPbStages;
  const long long pieces = (bytes + chunk - 1) / chunk;
  const long long first = (long long)blockIdx.x * nwarps + warp, stride = (long long)gridDim.x * nwarps;
  long long next = first;
  int loaded = 0, done = 0;
  auto issue = [&]() {
    const int s = loaded % kPbStages;
    const long long off = next * chunk;
    const unsigned len = (unsigned)(bytes - off < chunk ? bytes - off : chunk);
    mbar_expect_tx(bar + s, len);
    bulk_g2s(ring + (size_t)s * chunk, src + off, len, bar + s);
    ++loaded;
    next += stride;
  };
  for (int q = 0; q < kPbStages - 1 && next < pieces; ++q) issue();
  long long item = first;
  while (done < loaded) {
    const int s = done % kPbStages;
    if (!mbar_wait(bar + s, (unsigned)((done / kPbStages) & 1), timeout_ns)) {
      *error = 1;  // a load that never completed: give up, report, leave
      break;
    }
    const long long off = item * chunk;
    const unsigned len = (unsigned)(bytes - off < chunk ? bytes - off : chunk);
    bulk_s2g(dst + off, ring + (size_t)s * chunk, len);
    bulk_commit();
    ++done;
    item += stride;
    if (next < pieces) {
      bulk_wait_read<1>();  // every group but the one just committed has read its stage
      issue();
    }
  }
  bulk_wait<0>();
  atomicAdd(&s_finished, 1);
}

}  // namespace

}  // namespace moonep

using namespace moonep;

// Streams `bytes` (a multiple of 16) from local `src` to `dst` (local or peer memory) with `grid` CTAs and pieces of
// `chunk` bytes (a multiple of 16, at most 16 KB).  `error` is one device word the kernel sets when a wait ran out.
// fence_warps (0..4) extra warps per CTA fence and store a word into peer_word[(cta * 4 + warp) * 32] (peer memory of at
// least grid * 4 * 32 words, or null for fences only) for as long as the copies run.
extern "C" int moonep_peer_store_bench(void* dst, const void* src, long long bytes, int chunk, int grid, int* error,
                                       long long timeout_ms, int fence_warps, int* peer_word, void* stream) {
  if (fence_warps < 0 || fence_warps > 4) {
    set_error("moonep_peer_store_bench: 0..4 fence warps");
    return 1;
  }
  if (bytes <= 0 || bytes % 16 != 0 || chunk <= 0 || chunk % 16 != 0 || chunk > 16 * 1024 || grid <= 0) {
    set_error("moonep_peer_store_bench: bytes and chunk must be multiples of 16, chunk <= 16 KB, grid > 0");
    return 1;
  }
  if (((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) & 15u) != 0) {
    set_error("moonep_peer_store_bench: buffers must be 16-byte aligned");
    return 1;
  }
  const size_t smem = (size_t)kPbCopyWarps * kPbStages * chunk;
  if (int rc = check_cuda(cudaFuncSetAttribute(peer_store_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem),
                          "cudaFuncSetAttribute(peer_store_kernel)"))
    return rc;
  peer_store_kernel<<<grid, kPbThreads + 32 * fence_warps, smem, (cudaStream_t)stream>>>(
      (unsigned char*)dst, (const unsigned char*)src, bytes, chunk, (unsigned long long)timeout_ms * 1000000ull, error,
      peer_word);
  return check_launch("peer_store_kernel");
}
