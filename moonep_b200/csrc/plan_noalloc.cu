// Planner table stage with a built-in work area (see plan_noalloc.h for who needs it and why).
//
// Same arithmetic as plan_tables in planner.cu (balance quotas, per-expert allocation, group layout
// of every destination rank), but the tables it works in live in a file-scope device array instead
// of buffers allocated by the Buffer, the input counts are passed in directly, and nothing waits
// for peers.  The host side resolves the array's device address once per device with
// cudaGetSymbolAddress and hands that pointer to the kernel.
#include <cuda_runtime.h>

#include <climits>
#include <mutex>
#include <string>

#include "host.h"
#include "plan_noalloc.h"
#include "planner.cuh"

namespace moonep {

namespace {

// The work area.  In host code this name is only a handle for cudaGetSymbolAddress, never an address.
static __device__ __align__(256) int g_plan_scratch[MOONEP_NOALLOC_SCRATCH_WORDS];

constexpr int kMaxDevices = 64;
static int* g_scratch_ptr[kMaxDevices] = {nullptr};
static std::mutex g_setup_mutex;

struct NoAllocArgs {
  const int* tpe;  // [R, E]
  int* work;       // device address of g_plan_scratch
  int* cu_out;
  int* etc_out;
  int* zf_out;
  int* rs_out;
  int R, E, B, epn, cap, P, rank, NvS;
};

// One CTA.  The table stage itself is the device function the Buffer's own planner runs (planner.cuh); here its
// work tables are carved from the file-scope array, and only this rank's layout is produced.  A layout whose padded
// rows exceed NvS is reported by remote_stats[0] = -1 (the other outputs are then not to be used).
__global__ void __launch_bounds__(1024) plan_tables_noalloc_kernel(const NoAllocArgs a) {
  TablesIO io;
  io.tpe = a.tpe;
  io.R = a.R, io.E = a.E, io.B = a.B, io.epn = a.epn, io.cap = a.cap, io.P = a.P, io.rank = a.rank, io.NvS = a.NvS;
  io.cu_out = a.cu_out, io.etc_out = a.etc_out, io.zf_out = a.zf_out, io.rs_out = a.rs_out;
  io.tpe_prev = nullptr, io.alloc_cum = nullptr, io.expert_off = nullptr;
  // every word of the work area that is read below is written first in this launch
  const int bad = plan_tables_body(io, carve(a.work, a.R, a.E));
  if (bad && threadIdx.x == 0) a.rs_out[0] = -1;
}

// Device address of the work area on the current device; resolved once per device.
int scratch_for_current_device(int** out) {
  int dev = 0;
  if (int rc = check_cuda(cudaGetDevice(&dev), "cudaGetDevice")) return rc;
  if (dev < 0 || dev >= kMaxDevices) {
    set_error("moonep_plan_tables_noalloc: device index out of range");
    return 1;
  }
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    if (int rc = check_cuda(cudaGetSymbolAddress(&p, g_plan_scratch), "cudaGetSymbolAddress(plan work area)")) return rc;
    g_scratch_ptr[dev] = static_cast<int*>(p);
  }
  *out = g_scratch_ptr[dev];
  return 0;
}

}  // namespace

}  // namespace moonep

using namespace moonep;

extern "C" int moonep_plan_tables_noalloc(const int* tpe, int R, int E, int B, int S, int K, int token_padding, int rank,
                                          int NvS, int* cu_seqlens, int* experts_to_copy, int* zero_fill,
                                          int* remote_stats, void* stream) {
  if (R < 1 || R > MOONEP_NOALLOC_MAX_RANKS || E < R || E > MOONEP_NOALLOC_MAX_EXPERTS || E % R != 0) {
    set_error("moonep_plan_tables_noalloc: supports 1 <= R <= " + std::to_string(MOONEP_NOALLOC_MAX_RANKS) +
              " and E <= " + std::to_string(MOONEP_NOALLOC_MAX_EXPERTS) + " with E a multiple of R; got R=" +
              std::to_string(R) + ", E=" + std::to_string(E));
    return 1;
  }
  if (B < 0 || B > E || rank < 0 || rank >= R || S < 1 || K < 1 || token_padding < 1 || NvS < 1) {
    set_error("moonep_plan_tables_noalloc: B, rank, S, K, token_padding or NvS out of range");
    return 1;
  }
  const long long words = table_words(R, E);
  if (words > MOONEP_NOALLOC_SCRATCH_WORDS) {
    set_error("moonep_plan_tables_noalloc: work area too small for this R and E");
    return 1;
  }
  NoAllocArgs a;
  if (int rc = scratch_for_current_device(&a.work)) return rc;
  a.tpe = tpe;
  a.cu_out = cu_seqlens;
  a.etc_out = experts_to_copy;
  a.zf_out = zero_fill;
  a.rs_out = remote_stats;
  a.R = R;
  a.E = E;
  a.B = B;
  a.epn = E / R;
  a.cap = S * K;
  a.P = token_padding;
  a.rank = rank;
  a.NvS = NvS;
  plan_tables_noalloc_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>(a);
  return check_launch("plan_tables_noalloc_kernel");
}
