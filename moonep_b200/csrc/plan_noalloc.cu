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

__device__ inline void argmax_first(const int* v, int n, int lane, int& best, int& best_i) {
  best = INT_MIN;
  best_i = INT_MAX;
  for (int i = lane; i < n; i += 32) {
    const int x = v[i];
    if (x > best) {
      best = x;
      best_i = i;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const int ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (ov > best || (ov == best && oi < best_i)) {
      best = ov;
      best_i = oi;
    }
  }
}

__device__ inline void argmin_first(const int* v, int n, int lane, int& best, int& best_i) {
  best = INT_MAX;
  best_i = INT_MAX;
  for (int i = lane; i < n; i += 32) {
    const int x = v[i];
    if (x < best) {
      best = x;
      best_i = i;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const int ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (ov < best || (ov == best && oi < best_i)) {
      best = ov;
      best_i = oi;
    }
  }
}

__global__ void __launch_bounds__(1024) plan_tables_noalloc_kernel(const NoAllocArgs a) {
  const int R = a.R, E = a.E, B = a.B, epn = a.epn, P = a.P;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
  // carve the work area; every word read below is written first in this launch
  int* expert_count = a.work;
  int* remaining = expert_count + E;
  int* alloc = remaining + E;        // [R][E]
  int* z = alloc + R * E;            // [R][R]
  int* prank = z + R * R;            // [R][E]
  int* cand = prank + R * E;         // [R][E]
  int* rs1 = cand + R * E;           // [R]
  __shared__ int s_balance[MOONEP_NOALLOC_MAX_RANKS];

  for (int e = tid; e < E; e += blockDim.x) {
    int cum = 0;
    for (int s = 0; s < R; ++s) cum += a.tpe[s * E + e];
    expert_count[e] = cum;
    remaining[e] = cum;
    const int home = e / epn;
    for (int d = 0; d < R; ++d) alloc[d * E + e] = (d == home) ? cum : 0;
  }
  for (int i = tid; i < R * R; i += blockDim.x) z[i] = 0;
  for (int i = tid; i < R; i += blockDim.x) rs1[i] = 0;
  __syncthreads();

  for (int h = warp; h < R; h += nwarps) {
    int sum = 0;
    for (int i = lane; i < epn; i += 32) sum += expert_count[h * epn + i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (lane == 0) s_balance[h] = sum - a.cap;
  }
  __syncthreads();

  if (warp == 0) {
    for (int it = 0; it < 4 * R + 8; ++it) {
      int bh, h, bu, u;
      argmax_first(s_balance, R, lane, bh, h);
      argmin_first(s_balance, R, lane, bu, u);
      if (bh <= 0) break;
      const int move = -bu;
      if (lane == 0) {
        z[h * R + u] = move;
        s_balance[h] = bh - move;
        s_balance[u] = 0;
      }
      __syncwarp();
    }
  }
  __syncthreads();

  for (int h = warp; h < R; h += nwarps) {
    int* q = z + h * R;
    int* rem = remaining + h * epn;
    for (int it = 0; it < epn + R + 8; ++it) {
      int quota, d, r, le;
      argmax_first(q, R, lane, quota, d);
      if (quota <= 0) break;
      argmax_first(rem, epn, lane, r, le);
      const int take = r < quota ? r : quota;
      if (take <= 0) break;
      if (lane == 0) {
        const int e = h * epn + le;
        alloc[d * E + e] += take;
        alloc[h * E + e] -= take;
        rem[le] = r - take;
        q[d] = quota - take;
      }
      __syncwarp();
    }
  }
  __syncthreads();

  for (int d = warp; d < R; d += nwarps) {
    const int* al = alloc + d * E;
    int* pr = prank + d * E;
    int* cd = cand + d * E;
    int n = 0;
    for (int base = 0; base < E; base += 32) {
      const int e = base + lane;
      const int cnt = e < E ? al[e] : 0;
      const bool is_remote = e < E && cnt > 0 && (e / epn) != d;
      if (e < E) pr[e] = INT_MAX;
      const unsigned m = __ballot_sync(0xffffffffu, is_remote);
      if (is_remote) cd[n + __popc(m & ((1u << lane) - 1u))] = e;
      n += __popc(m);
    }
    __syncwarp();
    for (int i = lane; i < n; i += 32) {
      const int ei = cd[i], ci = al[ei];
      int pos = 0;
      for (int j = 0; j < n; ++j) {
        const int ej = cd[j], cj = al[ej];
        pos += (cj > ci || (cj == ci && ej > ei)) ? 1 : 0;
      }
      pr[ei] = pos;
      if (pos < B) {
        a.etc_out[d * B + pos] = ei;
        atomicAdd(rs1 + ei / epn, 1);
      }
    }
    for (int b = lane; b < B; b += 32)
      if (b >= n) a.etc_out[d * B + b] = -1;
    if (d == a.rank && lane == 0) a.rs_out[0] = n;
    __syncwarp();
    if (d != a.rank) continue;  // only this rank's layout is an output
    const int npick = n < B ? n : B;
    int carry = 0;
    for (int base = 0; base < E + B; base += 32) {
      const int g = base + lane;
      int cnt = 0;
      if (g < E) {
        if (pr[g] >= B) cnt = al[g];
      } else if (g < E + B && g - E < npick) {
        cnt = al[a.etc_out[d * B + (g - E)]];
      }
      const int padded = cnt > 0 ? ((cnt + P - 1) / P) * P : 0;
      int incl = padded;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
      }
      const int end_aligned = carry + incl;
      const int start = end_aligned - padded;
      if (g < E + B) {
        a.cu_out[g] = end_aligned;
        const bool pad = cnt > 0 && padded > cnt;
        a.zf_out[2 * g] = pad ? start + cnt : 0;
        a.zf_out[2 * g + 1] = pad ? padded - cnt : 0;
      }
      carry += __shfl_sync(0xffffffffu, incl, 31);
    }
  }
  __syncthreads();
  if (tid == 0) a.rs_out[1] = rs1[a.rank];
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
  if (B < 0 || B > E || rank < 0 || rank >= R || S < 1 || K < 1 || token_padding < 1) {
    set_error("moonep_plan_tables_noalloc: B, rank, S, K or token_padding out of range");
    return 1;
  }
  const long long words = 2ll * E + 3ll * R * E + 1ll * R * R + 1ll * R;
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
