// Host-side declarations shared by the .cu files of the library.
#pragma once

#include <cuda_runtime.h>

#include <atomic>
#include <string>

#include "moonep.h"

namespace moonep {

struct HostCtx {
  MoonepDevCtx dev;
  void* peer_tables = nullptr;
  int sm_count = 0;
  int max_smem_optin = 0;
};

void set_error(const std::string& s);
int check_cuda(cudaError_t e, const char* what);

// Every kernel launch of the library goes through check_launch, which also counts it.
extern std::atomic<long long> g_launch_count;
inline int check_launch(const char* what) {
  ++g_launch_count;
  return check_cuda(cudaGetLastError(), what);
}

inline int imin(int a, int b) { return a < b ? a : b; }
inline int imax(int a, int b) { return a > b ? a : b; }

}  // namespace moonep
