// Host-side declarations shared by the .cu files of the library.
#pragma once

#include <cuda_runtime.h>

#include <atomic>
#include <string>
#include <utility>

#include "moonep.h"

namespace moonep {

struct HostCtx {
  MoonepDevCtx dev;
  void* peer_tables = nullptr;
  int sm_count = 0;
  int max_smem_optin = 0;
  int enable_pdl = 0;  // launch the dispatch/combine kernels with programmatic dependent launch
};

void set_error(const std::string& s);
int check_cuda(cudaError_t e, const char* what);

// Every kernel launch of the library goes through check_launch, which also counts it.
extern std::atomic<long long> g_launch_count;
inline int check_launch(const char* what) {
  ++g_launch_count;
  return check_cuda(cudaGetLastError(), what);
}

// Launch with or without programmatic dependent launch.  With it, the kernel's CTAs may be scheduled while the
// previous kernel of the stream drains; the kernel calls griddep_wait() (common.cuh) before it touches anything the
// previous kernel wrote, so only its prologue (shared-memory set-up, barrier initialisation) overlaps.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_maybe_pdl(void (*kernel)(KArgs...), int grid, int block, size_t smem, cudaStream_t stream,
                                    bool pdl, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3((unsigned)block);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

inline int imin(int a, int b) { return a < b ? a : b; }
inline int imax(int a, int b) { return a > b ? a : b; }

}  // namespace moonep
