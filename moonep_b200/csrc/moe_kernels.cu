// Small dense helpers of the MoE layer's backward pass (sm_100a, plain CUDA cores):
//
//   transpose_experts   dst[n][j][col0 + i] = src[n][i][j] for a stack of bf16 matrices, through a
//                       64x64 shared-memory tile with 16-byte global accesses on both sides.  Builds the
//                       K-major copies of the local experts that the activation-gradient GEMMs read.
//   swiglu_bwd          per row r and column i, from a = x Wg^T, u = x Wu^T and g = dy Wd (unscaled):
//                         h = silu(a) u;  dgate[r] = sum_i g h;  dh = g w[r]
//                         da = dh u s (1 + a (1 - s)),  du = dh a s   (s = sigmoid(a))
//                       writes [da | du] side by side (one GEMM then yields dx), h*w (for the down
//                       projection's weight gradient) and dgate.
//
//   sgd_update          w (bf16) -= lr * g (fp32), vectorised.
//
// The reference has no expert computation; these serve the MoE training-step configuration.
#include <cuda_bf16.h>

#include "common.cuh"
#include "host.h"

namespace moonep {

namespace {

constexpr int kTile = 64;

__global__ void __launch_bounds__(256)
    transpose_experts_kernel(const uint16_t* __restrict__ src, uint16_t* __restrict__ dst, int d0, int d1,
                             long long dst_ld, long long dst_expert_stride, int col0, const int* __restrict__ active) {
  __shared__ uint16_t tile[kTile][kTile + 8];
  const int n = blockIdx.z;
  if (active != nullptr && active[n] < 0) return;  // e.g. a prefetch slot that holds no expert in this step
  const int i0 = blockIdx.y * kTile, j0 = blockIdx.x * kTile;
  const uint16_t* s = src + (long long)n * d0 * d1;
  uint16_t* d = dst + (long long)n * dst_expert_stride;
  // load 64 rows x 64 columns, 8 columns (16 bytes) per thread and step
  for (int v = threadIdx.x; v < kTile * (kTile / 8); v += blockDim.x) {
    const int r = v / (kTile / 8), cv = v % (kTile / 8);
    const int4 x = ld16(s + (long long)(i0 + r) * d1 + j0 + cv * 8);
    const uint16_t* e = reinterpret_cast<const uint16_t*>(&x);
#pragma unroll
    for (int q = 0; q < 8; ++q) tile[r][cv * 8 + q] = e[q];
  }
  __syncthreads();
  // store: output row j (a source column), 8 consecutive i per thread
  for (int v = threadIdx.x; v < kTile * (kTile / 8); v += blockDim.x) {
    const int j = v / (kTile / 8), iv = v % (kTile / 8);
    int4 x;
    uint16_t* e = reinterpret_cast<uint16_t*>(&x);
#pragma unroll
    for (int q = 0; q < 8; ++q) e[q] = tile[iv * 8 + q][j];
    st16(d + (long long)(j0 + j) * dst_ld + col0 + i0 + iv * 8, x);
  }
}

__device__ __forceinline__ float bf(uint16_t u) { return __uint_as_float(((unsigned)u) << 16); }
__device__ __forceinline__ uint16_t tobf(float f) {
  __nv_bfloat16 b = __float2bfloat16_rn(f);
  return *reinterpret_cast<uint16_t*>(&b);
}

// one warp per row; I must be a multiple of 8
__global__ void __launch_bounds__(256)
    swiglu_bwd_kernel(const uint16_t* __restrict__ a, const uint16_t* __restrict__ u, const uint16_t* __restrict__ g,
                      const float* __restrict__ w, const int* __restrict__ total_rows_ptr, int rows_cap, int I,
                      uint16_t* __restrict__ dadu, uint16_t* __restrict__ hsw, float* __restrict__ dgate) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  int rows = total_rows_ptr != nullptr ? *total_rows_ptr : rows_cap;
  if (rows > rows_cap) rows = rows_cap;
  for (int r = blockIdx.x * nwarps + warp; r < rows; r += gridDim.x * nwarps) {
    const float wr = w[r];
    float acc = 0.f;
    const long long base = (long long)r * I;
    for (int c0 = lane * 8; c0 < I; c0 += 32 * 8) {
      const int4 av = ld16(a + base + c0), uv = ld16(u + base + c0), gv = ld16(g + base + c0);
      const uint16_t* ae = reinterpret_cast<const uint16_t*>(&av);
      const uint16_t* ue = reinterpret_cast<const uint16_t*>(&uv);
      const uint16_t* ge = reinterpret_cast<const uint16_t*>(&gv);
      int4 dav, duv, hv;
      uint16_t* dae = reinterpret_cast<uint16_t*>(&dav);
      uint16_t* due = reinterpret_cast<uint16_t*>(&duv);
      uint16_t* he = reinterpret_cast<uint16_t*>(&hv);
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        const float x = bf(ae[q]), y = bf(ue[q]), gg = bf(ge[q]);
        const float s = 1.f / (1.f + __expf(-x));
        const float h = x * s * y;
        acc += gg * h;
        const float dh = gg * wr;
        dae[q] = tobf(dh * y * s * (1.f + x * (1.f - s)));
        due[q] = tobf(dh * x * s);
        he[q] = tobf(h * wr);
      }
      st16(dadu + (long long)r * 2 * I + c0, dav);
      st16(dadu + (long long)r * 2 * I + I + c0, duv);
      st16(hsw + base + c0, hv);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) dgate[r] = acc;
  }
}

// w (bf16) -= lr * g (fp32), 8 elements per thread and step
__global__ void __launch_bounds__(256)
    sgd_update_kernel(uint16_t* __restrict__ w, const float* __restrict__ g, long long n8, float lr) {
  for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < n8; v += (long long)gridDim.x * blockDim.x) {
    int4 wv = ld16(w + v * 8);
    const int4 g0 = ld16(g + v * 8), g1 = ld16(g + v * 8 + 4);
    uint16_t* we = reinterpret_cast<uint16_t*>(&wv);
    const float gf[8] = {__int_as_float(g0.x), __int_as_float(g0.y), __int_as_float(g0.z), __int_as_float(g0.w),
                         __int_as_float(g1.x), __int_as_float(g1.y), __int_as_float(g1.z), __int_as_float(g1.w)};
#pragma unroll
    for (int q = 0; q < 8; ++q) we[q] = tobf(bf(we[q]) - lr * gf[q]);
    st16(w + v * 8, wv);
  }
}

}  // namespace

}  // namespace moonep

using namespace moonep;

// w: [n] bf16, g: [n] fp32, n a multiple of 8: w -= lr * g.
extern "C" int moonep_sgd_update(void* w, const float* g, long long n, float lr, void* stream) {
  if (n % 8 != 0) {
    set_error("moonep_sgd_update: element count must be a multiple of 8");
    return 1;
  }
  if (n == 0) return 0;
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  sgd_update_kernel<<<imax(1, sms * 8), 256, 0, (cudaStream_t)stream>>>((uint16_t*)w, g, n / 8, lr);
  return check_launch("sgd_update_kernel");
}

// src: [n, d0, d1] bf16 -> dst[n][j][col0 + i] with row stride dst_ld and expert stride dst_expert_stride (elements).
// active (optional, device, [n]): matrices with a negative entry are skipped.
extern "C" int moonep_transpose_experts(const void* src, void* dst, int n, int d0, int d1, long long dst_ld,
                                        long long dst_expert_stride, int col0, const int* active, void* stream) {
  if (n <= 0) return 0;
  if (d0 % kTile != 0 || d1 % kTile != 0 || dst_ld % 8 != 0 || col0 % 8 != 0) {
    set_error("moonep_transpose_experts: dimensions must be multiples of 64 and the destination 16-byte aligned");
    return 1;
  }
  dim3 grid(d1 / kTile, d0 / kTile, n);
  transpose_experts_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const uint16_t*)src, (uint16_t*)dst, d0, d1, dst_ld,
                                                                   dst_expert_stride, col0, active);
  return check_launch("transpose_experts_kernel");
}

// a, u, g: [rows_cap, I] bf16; w: [rows_cap] fp32; total_rows: device int (rows in use) or null.
extern "C" int moonep_swiglu_bwd(const void* a, const void* u, const void* g, const float* w, const int* total_rows,
                                 int rows_cap, int I, void* dadu, void* hsw, float* dgate, void* stream) {
  if (I % 8 != 0 || rows_cap <= 0) {
    set_error("moonep_swiglu_bwd: I must be a multiple of 8");
    return 1;
  }
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  swiglu_bwd_kernel<<<imax(1, sms * 4), 256, 0, (cudaStream_t)stream>>>((const uint16_t*)a, (const uint16_t*)u,
                                                                        (const uint16_t*)g, w, total_rows, rows_cap, I,
                                                                        (uint16_t*)dadu, (uint16_t*)hsw, dgate);
  return check_launch("swiglu_bwd_kernel");
}
