// tcgen05 / TMEM / TMA building blocks shared by the GEMM kernels (sm_100a): PTX wrappers for tensor-map
// loads, TMEM allocation, MMA issue and commit, accumulator loads, the shared-memory and instruction
// descriptors of K-major bf16 tiles with the 128-byte swizzle, and the host-side tensor-map encoder.
#pragma once

#include <cuda.h>

#include <string>

#include "common.cuh"
#include "host.h"

namespace moonep {

constexpr int BM = 128;   // rows of an accumulator tile per CTA (TMEM lanes)
constexpr int BN = 256;   // accumulator columns of a tile
constexpr int BK = 64;    // K elements per pipeline stage: one 128-byte swizzle row of bf16
constexpr int UMMA_K = 16;

__device__ __forceinline__ void gemm_fail(int* status, int kernel, int where, int x, int y) {
  if (status != nullptr && atomicCAS(status + MOONEP_ST_CODE, 0, MOONEP_STATUS_TIMEOUT) == 0) {
    status[MOONEP_ST_KERNEL] = kernel;
    status[MOONEP_ST_FAMILY] = where;
    status[MOONEP_ST_PEER] = x;
    status[MOONEP_ST_EXPECT] = y;
    __threadfence();
  }
}

// A group's weights are not on this rank (group_map says -1): an index error, recorded once.
__device__ __forceinline__ void gemm_bad_index(int* status, int kernel, int kind, int x, int y) {
  if (status != nullptr && atomicCAS(status + MOONEP_ST_CODE, 0, MOONEP_STATUS_BAD_INDEX) == 0) {
    status[MOONEP_ST_KERNEL] = kernel;
    status[MOONEP_ST_FAMILY] = kind;
    status[MOONEP_ST_PEER] = x;
    status[MOONEP_ST_EXPECT] = y;
    __threadfence();
  }
}

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* tmap, int c0, int c1,
                                            unsigned long long* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
          smem_u32(smem_dst)),
      "l"(reinterpret_cast<unsigned long long>(tmap)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}

__device__ __forceinline__ void tmem_alloc(unsigned* smem_dst, unsigned ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(unsigned taddr, unsigned ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void umma_bf16(unsigned d_tmem, unsigned long long adesc, unsigned long long bdesc,
                                          unsigned idesc, unsigned accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void umma_commit(unsigned long long* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

__device__ __forceinline__ void tmem_ld32(unsigned taddr, unsigned (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,"
      "%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major tile stored with the 128-byte swizzle: rows are
// 128 bytes apart, groups of eight rows 1024 bytes apart.
__device__ __forceinline__ unsigned long long make_smem_desc(const void* tile) {
  const unsigned addr = smem_u32(tile);
  unsigned long long d = 0;
  d |= (unsigned long long)((addr & 0x3FFFFu) >> 4);  // start address, 16-byte units
  d |= (unsigned long long)1 << 16;                   // leading byte offset (unused for this layout)
  d |= (unsigned long long)(1024 >> 4) << 32;         // stride byte offset: 8 rows * 128 bytes
  d |= (unsigned long long)1 << 46;                   // descriptor version of sm_100
  d |= (unsigned long long)2 << 61;                   // 128-byte swizzle
  return d;
}

// Descriptor of an MN-major tile (the M or N index is contiguous in memory, e.g. a [k, n] row-major slice)
// stored with the 128-byte swizzle as TMA writes it from boxes of 64 columns x 64 rows: a 128-byte line holds
// 64 consecutive M/N elements of one k, eight consecutive k form a 1024-byte swizzle atom, the next eight k
// follow 1024 bytes later (stride byte offset) and the next 64 M/N elements start one box (8192 bytes) later
// (leading byte offset).  One MMA (K = 16) consumes two atoms, so its successor starts 2048 bytes further.
__device__ __forceinline__ unsigned long long make_smem_desc_mn(const void* tile) {
  const unsigned addr = smem_u32(tile);
  unsigned long long d = 0;
  d |= (unsigned long long)((addr & 0x3FFFFu) >> 4);
  d |= (unsigned long long)(8192 >> 4) << 16;  // leading byte offset: next 64 elements along M/N
  d |= (unsigned long long)(1024 >> 4) << 32;  // stride byte offset: next 8 elements along K
  d |= (unsigned long long)1 << 46;
  d |= (unsigned long long)2 << 61;
  return d;
}
constexpr unsigned kDescStepK = 2;       // K-major: 16 elements = 32 bytes along the swizzled row, in 16-byte units
constexpr unsigned kDescStepMn = 128;    // MN-major: 16 k = two 1024-byte atoms, in 16-byte units
constexpr unsigned kMnBoxBytes = 64 * 64 * 2;  // one 64 x 64 bf16 box

// kind::f16 instruction descriptor: bf16 x bf16 -> fp32, M x N; a_mn / b_mn: that operand is MN-major.
__host__ __device__ constexpr unsigned make_idesc(int m, int n, bool a_mn = false, bool b_mn = false) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16) |
         ((unsigned)(n >> 3) << 17) | ((unsigned)(m >> 4) << 24);
}

__device__ __forceinline__ float silu(float x) { return x / (1.f + __expf(-x)); }


enum GemmMode { kPlain = 0, kSwiglu = 1, kScale = 2 };

struct GemmArgs {
  uint16_t* out;           // [rows, ldo] bf16
  const float* row_scale;  // [rows] or null
  const int* cu_seqlens;   // [G] inclusive padded ends
  int* status;             // [MOONEP_ST_WORDS] or null
  unsigned long long timeout_ns;
  int G;
  int n_per_group;   // rows of W per group (N)
  int n_tiles;       // output column tiles per row block
  int k_blocks;      // K / 64
  int ldo;           // row stride of out in elements
  int mode;
  int rows_cap;      // rows of X
  const int* group_map;  // [G] weight slot of every group, or null for the identity
  int w_slots;           // number of weight slots (rows of W = w_slots * n_per_group)
  int b_kn;              // CTA-pair kernel only: W is [slots, K, N] (N contiguous), staged as MN-major tiles
  int k_split;           // with b_kn: K blocks served by the first W tensor, the rest come from the second
  uint16_t* pre_gate;    // SwiGLU only, optional: the pre-activations x Wg^T and x Wu^T, [rows, ldo] bf16 each,
  uint16_t* pre_up;      // kept for the backward pass so that it need not recompute them
  MoonepGemmHooks hooks; // CTA-pair kernel only: hand-off with the communication kernels (all null = none)
};

// ---- CTA pairs (cta_group::2): the two CTAs of a cluster share one MMA --------------------------------

__device__ __forceinline__ unsigned cluster_ctarank() {
  unsigned r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

// shared::cluster address of `p` (a shared-memory object of this CTA) in the CTA `rank` of the cluster
__device__ __forceinline__ unsigned mapa_u32(const void* p, unsigned rank) {
  unsigned r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_u32(p)), "r"(rank));
  return r;
}

__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// arrive on an mbarrier of another CTA of the cluster (address from mapa_u32)
__device__ __forceinline__ void mbar_arrive_cluster(unsigned cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait_cluster(unsigned long long* bar, unsigned parity) {
  unsigned ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait on a barrier that CTAs of the cluster arrive on; false if the budget ran out.
__device__ __forceinline__ bool mbar_wait_cluster(unsigned long long* bar, unsigned parity, unsigned long long timeout_ns) {
  if (mbar_try_wait_cluster(bar, parity)) return true;
  const unsigned long long t0 = globaltimer_ns();
  unsigned spins = 0;
  while (!mbar_try_wait_cluster(bar, parity)) {
    if ((++spins & 255u) == 0 && globaltimer_ns() - t0 > timeout_ns) return false;
  }
  return true;
}

// Tensor-map load of a CTA pair: the data lands in this CTA's shared memory, the bytes complete the
// transaction of `bar_cluster_addr`, which may be a barrier of the other CTA of the pair.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* tmap, int c0, int c1,
                                                 unsigned bar_cluster_addr) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
          smem_u32(smem_dst)),
      "l"(reinterpret_cast<unsigned long long>(tmap)), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
      : "memory");
}

// One MMA over both CTAs of the pair (M = 256: 128 rows per CTA; each CTA holds half of the B tile).
__device__ __forceinline__ void umma_bf16_pair(unsigned d_tmem, unsigned long long adesc, unsigned long long bdesc,
                                               unsigned idesc, unsigned accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Arrive on the barrier at this shared-memory offset in every CTA of `cta_mask` once the pair's earlier MMAs are done.
__device__ __forceinline__ void umma_commit_pair(unsigned long long* bar, unsigned short cta_mask) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
                   smem_u32(bar)),
               "h"(cta_mask)
               : "memory");
}

// ---- host side ----------------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
    else
      cudaGetLastError();
  }
  return fn;
}

// 2-D bf16 row-major [rows, cols] tensor (rows ld elements apart; 0 = cols), box = 64 columns x box_rows rows,
// 128-byte swizzle.
inline int make_tmap(CUtensorMap* m, const void* base, unsigned long long rows, unsigned long long cols,
                     unsigned box_rows, unsigned long long ld = 0) {
  EncodeTiledFn fn = encode_tiled();
  if (fn == nullptr) {
    set_error("cuTensorMapEncodeTiled is not available (no CUDA driver?)");
    return 1;
  }
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {(ld ? ld : cols) * 2};
  cuuint32_t box[2] = {(cuuint32_t)BK, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with CUresult " + std::to_string((int)r));
    return (int)r;
  }
  return 0;
}

}  // namespace moonep
