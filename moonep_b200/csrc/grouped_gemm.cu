// Grouped expert GEMM for sm_100a: tcgen05 tensor cores, TMEM accumulators, TMA-fed shared memory.
//
//   Y[rows of group g, :] = X[rows of group g, :] @ W[g]^T        X: [rows, K] bf16, W: [G, N, K] bf16
//
// Groups are the padded row segments of a dispatched shard: cu_seqlens[g] is the inclusive end of
// group g and every non-empty segment is a multiple of 128 rows, so each 128-row block belongs to
// exactly one group.  The number of row blocks is read from cu_seqlens on the device; the host never
// synchronises.
//
// Persistent kernel, one CTA per SM, 192 threads:
//   warp 0      TMA producer: per 64-wide K block one 128x64 tile of X and two 128x64 tiles of W
//               (cp.async.bulk.tensor.2d, 128-byte swizzle, every CTA loads its own tiles) into a 4-stage ring; the
//               transaction bytes complete the stage's "full" mbarrier.
//   warp 1      allocates 512 TMEM columns (two 128x256 fp32 accumulators) and issues the MMAs from
//               one lane: four tcgen05.mma (M=128, N=256, K=16, bf16 -> fp32) per stage;
//               tcgen05.commit releases the stage and, after the last K block, publishes the
//               accumulator to the epilogue.
//   warps 2..5  epilogue: tcgen05.ld 32 columns at a time from their 32 TMEM lanes, apply the
//               epilogue, convert to bf16, store.  While they drain one accumulator the MMA warp
//               fills the other.
// Epilogues: PLAIN  y = acc                                   (256 output columns per tile)
//            SWIGLU y = silu(acc[:, :128]) * acc[:, 128:]      (W tiles come from W_gate and W_up;
//                                                              128 output columns per tile)
//            SCALE  y = acc * row_scale[row]                   (down projection times the gate
//                                                              weight carried with the row)
// Every mbarrier wait is bounded; on expiry the role records a status word and leaves its loop, the
// CTA still frees its TMEM before it returns.
//
// The reference has no GEMM; this kernel serves the MoE-layer benchmark configuration (dispatch ->
// prefetch_weight -> grouped GEMM -> combine) named beside the reference's Buffer API
// (reference README.md:46-48).
#include <cstring>

#include "umma.cuh"

namespace moonep {

namespace {

constexpr int kStages = 4;
constexpr int kGemmThreads = 192;
constexpr int kTmemCols = 512;
constexpr unsigned kATileBytes = BM * BK * 2;        // 16 KB
constexpr unsigned kBHalfBytes = 128 * BK * 2;       // 16 KB
constexpr unsigned kStageBytes = kATileBytes + 2 * kBHalfBytes;  // 48 KB

__global__ void __launch_bounds__(kGemmThreads, 1)
    grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b0,
                        const __grid_constant__ CUtensorMap tmap_b1, const GemmArgs a) {
  extern __shared__ unsigned char s_raw[];
  __shared__ __align__(8) unsigned long long s_full[kStages], s_empty[kStages], s_tfull[2], s_tempty[2];
  __shared__ unsigned s_tmem_base;
  unsigned char* s_tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(s_raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(s_full + s, 1);
      mbar_init(s_empty + s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(s_tfull + b, 1);
      mbar_init(s_tempty + b, 4);
    }
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(&s_tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const unsigned tmem_base = s_tmem_base;

  const int total_rows = min(a.cu_seqlens[a.G - 1], a.rows_cap);
  const int row_blocks = total_rows / BM;
  const long long num_tiles = (long long)row_blocks * a.n_tiles;
  const int b_rows_per_tile = (a.mode == kSwiglu) ? 128 : 256;  // W rows consumed per output tile and tensor map

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int stage = 0;
      unsigned phase = 0;
      bool failed = false;
      for (long long t = blockIdx.x; t < num_tiles && !failed; t += gridDim.x) {
        const int mb = (int)(t / a.n_tiles), nb = (int)(t % a.n_tiles);
        const int row0 = mb * BM;
        int lo = 0, hi = a.G - 1;  // first group whose end is beyond row0
        while (lo < hi) {
          const int mid = (lo + hi) >> 1;
          if (a.cu_seqlens[mid] > row0) hi = mid; else lo = mid + 1;
        }
        int wslot = a.group_map != nullptr ? a.group_map[lo] : lo;
        if (wslot < 0 || wslot >= a.w_slots) {
          // a group whose weights this rank does not hold: reported, computed with slot 0 (in bounds), never trusted
          gemm_bad_index(a.status, 13, 13, lo, wslot);
          wslot = 0;
        }
        const int wrow0 = wslot * a.n_per_group + nb * b_rows_per_tile;
        for (int kb = 0; kb < a.k_blocks; ++kb) {
          if (!mbar_wait(s_empty + stage, phase ^ 1u, a.timeout_ns)) {
            gemm_fail(a.status, 13, 1, stage, kb);
            failed = true;
            break;
          }
          unsigned char* st = s_tiles + (size_t)stage * kStageBytes;
          mbar_expect_tx(s_full + stage, kStageBytes);
          tma_load_2d(st, &tmap_a, kb * BK, row0, s_full + stage);
          tma_load_2d(st + kATileBytes, &tmap_b0, kb * BK, wrow0, s_full + stage);
          if (a.mode == kSwiglu)
            tma_load_2d(st + kATileBytes + kBHalfBytes, &tmap_b1, kb * BK, wrow0, s_full + stage);
          else
            tma_load_2d(st + kATileBytes + kBHalfBytes, &tmap_b0, kb * BK, wrow0 + 128, s_full + stage);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr unsigned idesc = make_idesc(BM, BN);
      int stage = 0;
      unsigned phase = 0;
      unsigned tphase[2] = {0, 0};
      int it = 0;
      bool failed = false;
      for (long long t = blockIdx.x; t < num_tiles && !failed; t += gridDim.x, ++it) {
        const int buf = it & 1;
        if (!mbar_wait(s_tempty + buf, tphase[buf] ^ 1u, a.timeout_ns)) {
          gemm_fail(a.status, 13, 2, buf, it);
          break;
        }
        tphase[buf] ^= 1u;
        tc_fence_after();
        const unsigned d_tmem = tmem_base + (unsigned)(buf * BN);
        for (int kb = 0; kb < a.k_blocks; ++kb) {
          if (!mbar_wait(s_full + stage, phase, a.timeout_ns)) {
            gemm_fail(a.status, 13, 3, stage, kb);
            failed = true;
            break;
          }
          tc_fence_after();
          const unsigned char* st = s_tiles + (size_t)stage * kStageBytes;
          const unsigned long long adesc = make_smem_desc(st);
          const unsigned long long bdesc = make_smem_desc(st + kATileBytes);
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            // 16 bf16 = 32 bytes further along K inside the swizzled 128-byte rows
            umma_bf16(d_tmem, adesc + (unsigned long long)(kk * 2), bdesc + (unsigned long long)(kk * 2), idesc,
                      (kb | kk) != 0 ? 1u : 0u);
          }
          umma_commit(s_empty + stage);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!failed) umma_commit(s_tfull + buf);
      }
    }
    __syncwarp();
  } else {
    // ---------------- epilogue (warps 2..5) ----------------
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    unsigned tphase[2] = {0, 0};
    int it = 0;
    for (long long t = blockIdx.x; t < num_tiles; t += gridDim.x, ++it) {
      const int buf = it & 1;
      const int mb = (int)(t / a.n_tiles), nb = (int)(t % a.n_tiles);
      int got = 1;
      if (lane == 0) got = mbar_wait(s_tfull + buf, tphase[buf], a.timeout_ns) ? 1 : 0;
      got = __shfl_sync(0xffffffffu, got, 0);
      if (!got) {
        if (lane == 0) gemm_fail(a.status, 13, 4, buf, it);
        break;
      }
      tphase[buf] ^= 1u;
      tc_fence_after();
      const int row = mb * BM + q * 32 + lane;
      const unsigned taddr = tmem_base + ((unsigned)(q * 32) << 16) + (unsigned)(buf * BN);
      if (a.mode == kSwiglu) {
        uint16_t* orow = a.out + (long long)row * a.ldo + (long long)nb * 128;
#pragma unroll 1
        for (int c0 = 0; c0 < 128; c0 += 32) {
          unsigned g[32], u[32];
          tmem_ld32(taddr + (unsigned)c0, g);
          tmem_ld32(taddr + (unsigned)(128 + c0), u);
          tmem_ld_wait();
          unsigned o[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float y0 = silu(__uint_as_float(g[2 * j])) * __uint_as_float(u[2 * j]);
            const float y1 = silu(__uint_as_float(g[2 * j + 1])) * __uint_as_float(u[2 * j + 1]);
            o[j] = pack_bf16(y0, y1);
          }
#pragma unroll
          for (int j = 0; j < 4; ++j)
            st16(orow + c0 + j * 8, make_int4((int)o[4 * j], (int)o[4 * j + 1], (int)o[4 * j + 2], (int)o[4 * j + 3]));
          if (a.pre_gate != nullptr) {
            const long long off = (long long)row * a.ldo + (long long)nb * 128 + c0;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              g[j] = pack_bf16(__uint_as_float(g[2 * j]), __uint_as_float(g[2 * j + 1]));
              u[j] = pack_bf16(__uint_as_float(u[2 * j]), __uint_as_float(u[2 * j + 1]));
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              st16(a.pre_gate + off + j * 8, make_int4((int)g[4 * j], (int)g[4 * j + 1], (int)g[4 * j + 2], (int)g[4 * j + 3]));
              st16(a.pre_up + off + j * 8, make_int4((int)u[4 * j], (int)u[4 * j + 1], (int)u[4 * j + 2], (int)u[4 * j + 3]));
            }
          }
        }
      } else {
        const float scale = (a.mode == kScale && a.row_scale != nullptr) ? a.row_scale[row] : 1.f;
        uint16_t* orow = a.out + (long long)row * a.ldo + (long long)nb * BN;
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
          unsigned v[32];
          tmem_ld32(taddr + (unsigned)c0, v);
          tmem_ld_wait();
          unsigned o[16];
#pragma unroll
          for (int j = 0; j < 16; ++j)
            o[j] = pack_bf16(__uint_as_float(v[2 * j]) * scale, __uint_as_float(v[2 * j + 1]) * scale);
#pragma unroll
          for (int j = 0; j < 4; ++j)
            st16(orow + c0 + j * 8, make_int4((int)o[4 * j], (int)o[4 * j + 1], (int)o[4 * j + 2], (int)o[4 * j + 3]));
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(s_tempty + buf);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ---- weight gradients: contraction over the rows of a group ----------------------------------------
//
//   dW[g] (P x Q, fp32) = L[rows of g, :P]^T  @  R[rows of g, :Q]
//
// The operands are taken as stored (L: [rows, P], R: [rows, Q]; tiles are staged MN-major, see
// make_smem_desc_mn) or transposed (Lt: [P, ld], Rt: [Q, ld], the row index contiguous, K-major tiles as
// in the forward kernel).  The K loop of a tile runs over the group's rows (k0 = first row of the group,
// any multiple of 16 rows long; the last 64-row block issues only the MMAs that lie inside the group).
// One tile is 128 x 256 of one group's dW.  The groups that have anything to do are listed once per CTA
// in shared memory (in group order, the same list in every CTA), so empty groups cost nothing.  Per group, flags[g] selects: 0 store (and store zeros if the group has no rows),
// 1 add to what is there, 2 store, leave the target alone if the group has no rows.  A null
// out_ptrs[g] skips the group; rows without a target are reported through the status block.
constexpr int kWgradStageLd = 36;  // floats per row of an epilogue warp's 32 x 32 staging block (16-byte aligned, conflict free)
constexpr size_t kWgradStageBytes = 4 * 32 * kWgradStageLd * sizeof(float);

struct WgradArgs {
  float* const* out_ptrs;  // [G] device array
  const int* flags;        // [G]
  const int* cu_seqlens;   // [G] inclusive padded ends
  int* status;
  unsigned long long timeout_ns;
  int G, P, Q, p_tiles, q_tiles, rows_cap;
  int row_major;  // operands are L [rows, P] and R [rows, Q] as they are (MN-major tiles) instead of their transposes
};

constexpr int kWgradMaxGroups = 512;  // groups per launch (their work list lives in shared memory)

struct WgradGroups {  // per listed group: which group, its first row, its rows, target and mode
  int n;
  short g[kWgradMaxGroups];
  int start[kWgradMaxGroups];
  int krows[kWgradMaxGroups];
  int flag[kWgradMaxGroups];
  float* out[kWgradMaxGroups];
};

// Warp-collective: list the groups with rows, and the empty ones whose target must be zeroed, in group order.
__device__ __forceinline__ void wgrad_list_groups(const WgradArgs& a, WgradGroups& sg, int lane) {
  int n = 0;
  for (int base = 0; base < a.G; base += 32) {
    const int g = base + lane;
    bool listed = false;
    int start = 0, krows = 0, flag = 0;
    float* out = nullptr;
    if (g < a.G) {
      start = g > 0 ? min(a.cu_seqlens[g - 1], a.rows_cap) : 0;
      const int end = min(a.cu_seqlens[g], a.rows_cap);
      krows = end > start ? end - start : 0;
      out = a.out_ptrs[g];
      flag = a.flags[g];
      // the K coordinate of a TMA copy must be a multiple of 8 elements and the MMAs take 16 rows at a time:
      // a group that does not start and end on a multiple of 16 is refused (reported as rows without a target)
      if (((start | end) & 15) != 0) out = nullptr;
      listed = krows > 0 || (out != nullptr && flag == 0);
    }
    const unsigned mask = __ballot_sync(0xffffffffu, listed);
    const int pos = n + __popc(mask & ((1u << lane) - 1u));
    if (listed && pos < kWgradMaxGroups) {
      sg.g[pos] = (short)g;
      sg.start[pos] = start;
      sg.krows[pos] = krows;
      sg.flag[pos] = flag;
      sg.out[pos] = out;
    }
    n += __popc(mask);
  }
  if (lane == 0) sg.n = min(n, kWgradMaxGroups);
}

struct WgradTile {
  int g, pb, qb, k0, krows, flag;
  float* out;
};

__device__ __forceinline__ WgradTile wgrad_tile(const WgradArgs& a, const WgradGroups& sg, long long t) {
  WgradTile w;
  const int per_group = a.p_tiles * a.q_tiles;
  const int idx = (int)(t / per_group);
  const int rem = (int)(t % per_group);
  w.pb = rem / a.q_tiles;
  w.qb = rem % a.q_tiles;
  w.g = sg.g[idx];
  w.k0 = sg.start[idx];
  w.krows = sg.krows[idx];
  w.flag = sg.flag[idx];
  w.out = sg.out[idx];
  return w;
}

__global__ void __launch_bounds__(kGemmThreads, 1)
    grouped_wgrad_kernel(const __grid_constant__ CUtensorMap tmap_l, const __grid_constant__ CUtensorMap tmap_r,
                         const WgradArgs a) {
  extern __shared__ unsigned char s_raw[];
  __shared__ __align__(8) unsigned long long s_full[kStages], s_empty[kStages], s_tfull[2], s_tempty[2];
  __shared__ unsigned s_tmem_base;
  __shared__ WgradGroups s_groups;
  unsigned char* s_tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(s_raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp == 0) wgrad_list_groups(a, s_groups, lane);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(s_full + s, 1);
      mbar_init(s_empty + s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(s_tfull + b, 1);
      mbar_init(s_tempty + b, 4);
    }
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(&s_tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const unsigned tmem_base = s_tmem_base;
  const long long num_tiles = (long long)s_groups.n * a.p_tiles * a.q_tiles;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int stage = 0;
      unsigned phase = 0;
      bool failed = false;
      for (long long t = blockIdx.x; t < num_tiles && !failed; t += gridDim.x) {
        const WgradTile w = wgrad_tile(a, s_groups, t);
        if (w.krows == 0 || w.out == nullptr) continue;
        const int kbs = (w.krows + BK - 1) / BK;
        for (int kb = 0; kb < kbs; ++kb) {
          if (!mbar_wait(s_empty + stage, phase ^ 1u, a.timeout_ns)) {
            gemm_fail(a.status, 14, 1, stage, kb);
            failed = true;
            break;
          }
          unsigned char* st = s_tiles + (size_t)stage * kStageBytes;
          mbar_expect_tx(s_full + stage, kStageBytes);
          if (a.row_major) {
            // boxes of 64 columns (P or Q) x 64 rows (K): two for the L tile, four for the R tile
            const int k = w.k0 + kb * BK;
#pragma unroll
            for (int c = 0; c < 2; ++c) tma_load_2d(st + c * kMnBoxBytes, &tmap_l, w.pb * BM + 64 * c, k, s_full + stage);
#pragma unroll
            for (int c = 0; c < 4; ++c)
              tma_load_2d(st + kATileBytes + c * kMnBoxBytes, &tmap_r, w.qb * BN + 64 * c, k, s_full + stage);
          } else {
            tma_load_2d(st, &tmap_l, w.k0 + kb * BK, w.pb * BM, s_full + stage);
            tma_load_2d(st + kATileBytes, &tmap_r, w.k0 + kb * BK, w.qb * BN, s_full + stage);
            tma_load_2d(st + kATileBytes + kBHalfBytes, &tmap_r, w.k0 + kb * BK, w.qb * BN + 128, s_full + stage);
          }
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr unsigned idesc = make_idesc(BM, BN);
      constexpr unsigned idesc_mn = make_idesc(BM, BN, true, true);
      const unsigned kstep = a.row_major ? kDescStepMn : kDescStepK;
      int stage = 0;
      unsigned phase = 0;
      unsigned tphase[2] = {0, 0};
      int it = 0;
      bool failed = false;
      for (long long t = blockIdx.x; t < num_tiles && !failed; t += gridDim.x) {
        const WgradTile w = wgrad_tile(a, s_groups, t);
        if (w.krows == 0 || w.out == nullptr) continue;
        const int buf = it & 1;
        ++it;
        if (!mbar_wait(s_tempty + buf, tphase[buf] ^ 1u, a.timeout_ns)) {
          gemm_fail(a.status, 14, 2, buf, it);
          break;
        }
        tphase[buf] ^= 1u;
        tc_fence_after();
        const unsigned d_tmem = tmem_base + (unsigned)(buf * BN);
        const int kbs = (w.krows + BK - 1) / BK;
        for (int kb = 0; kb < kbs; ++kb) {
          if (!mbar_wait(s_full + stage, phase, a.timeout_ns)) {
            gemm_fail(a.status, 14, 3, stage, kb);
            failed = true;
            break;
          }
          tc_fence_after();
          const unsigned char* st = s_tiles + (size_t)stage * kStageBytes;
          const unsigned long long adesc = a.row_major ? make_smem_desc_mn(st) : make_smem_desc(st);
          const unsigned long long bdesc = a.row_major ? make_smem_desc_mn(st + kATileBytes) : make_smem_desc(st + kATileBytes);
          const int nkk = min(BK / UMMA_K, (w.krows - kb * BK) / UMMA_K);  // MMAs inside the group
          for (int kk = 0; kk < nkk; ++kk)
            umma_bf16(d_tmem, adesc + (unsigned long long)(kk * kstep), bdesc + (unsigned long long)(kk * kstep),
                      a.row_major ? idesc_mn : idesc, (kb | kk) != 0 ? 1u : 0u);
          umma_commit(s_empty + stage);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!failed) umma_commit(s_tfull + buf);
      }
    }
    __syncwarp();
  } else {
    // ---------------- epilogue (warps 2..5): one output row per thread ----------------
    const int q = warp & 3;
    float* stage_w = reinterpret_cast<float*>(s_tiles + (size_t)kStages * kStageBytes) + (warp - 2) * 32 * kWgradStageLd;
    unsigned tphase[2] = {0, 0};
    int it = 0;
    for (long long t = blockIdx.x; t < num_tiles; t += gridDim.x) {
      const WgradTile w = wgrad_tile(a, s_groups, t);
      const int flag = w.flag;
      if (w.out == nullptr) {
        if (w.krows != 0 && q == 0 && lane == 0 && w.pb == 0 && w.qb == 0 && a.status != nullptr &&
            atomicCAS(a.status + MOONEP_ST_CODE, 0, MOONEP_STATUS_BAD_INDEX) == 0) {
          a.status[MOONEP_ST_KERNEL] = 14;
          a.status[MOONEP_ST_FAMILY] = 100;  // kind: rows of a group whose gradient has no target
          a.status[MOONEP_ST_PEER] = w.g;
          a.status[MOONEP_ST_EXPECT] = 0;
          a.status[MOONEP_ST_SEEN] = w.krows;
          __threadfence();
        }
        continue;
      }
      float* orow = w.out + (long long)(w.pb * BM + q * 32 + lane) * a.Q + (long long)w.qb * BN;
      if (w.krows == 0) {
        if (flag == 0) {
          const int4 z = make_int4(0, 0, 0, 0);
#pragma unroll 4
          for (int c = 0; c < BN; c += 4) st16(orow + c, z);
        }
        continue;
      }
      const int buf = it & 1;
      ++it;
      int got = 1;
      if (lane == 0) got = mbar_wait(s_tfull + buf, tphase[buf], a.timeout_ns) ? 1 : 0;
      got = __shfl_sync(0xffffffffu, got, 0);
      if (!got) {
        if (lane == 0) gemm_fail(a.status, 14, 4, buf, it);
        break;
      }
      tphase[buf] ^= 1u;
      tc_fence_after();
      const unsigned taddr = tmem_base + ((unsigned)(q * 32) << 16) + (unsigned)(buf * BN);
      // A thread reads one accumulator row (32 columns) from TMEM; the chunk is turned through shared memory
      // so that eight lanes write one full 128-byte line and a warp instruction covers four rows.
      float* tile_out = w.out + (long long)(w.pb * BM + q * 32) * a.Q + (long long)w.qb * BN;
      const int sub_row = lane >> 3, col4 = (lane & 7) * 4;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        unsigned v[32];
        tmem_ld32(taddr + (unsigned)c0, v);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 8; ++j)
          *reinterpret_cast<uint4*>(stage_w + lane * kWgradStageLd + 4 * j) =
              make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int r = 4 * i + sub_row;
          const float4 x = *reinterpret_cast<const float4*>(stage_w + r * kWgradStageLd + col4);
          float* dst = tile_out + (long long)r * a.Q + c0 + col4;
          if (flag == 1)
            asm volatile("red.global.add.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(dst), "f"(x.x), "f"(x.y), "f"(x.z), "f"(x.w)
                         : "memory");
          else
            st16(dst, make_int4(__float_as_int(x.x), __float_as_int(x.y), __float_as_int(x.z), __float_as_int(x.w)));
        }
        __syncwarp();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(s_tempty + buf);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace

// ---- host side --------------------------------------------------------------------------------------

}  // namespace moonep

using namespace moonep;

// x: [rows_cap, K] bf16.  w0 (and w1 for SwiGLU): [G, n_per_group, K] bf16.  out: [rows_cap, n_out] bf16 with
// n_out = n_per_group (plain, scale) or n_per_group (swiglu: gate and up each have n_per_group rows).
// cu_seqlens: [G] int32 inclusive padded ends (multiples of 128).  mode: 0 plain, 1 swiglu, 2 scale by row_scale.
// group_map (optional): [G] int32, weight slot of every group when w holds only w_slots < G experts.
// pre_gate, pre_up (optional, SwiGLU): [rows_cap, n_per_group] bf16, receive x Wg^T and x Wu^T.
extern "C" int moonep_grouped_gemm(const void* x, const void* w0, const void* w1, void* out, const float* row_scale,
                                   const int* cu_seqlens, int G, int rows_cap, int K, int n_per_group, int mode,
                                   int* status, long long timeout_ms, int num_sms, const int* group_map, int w_slots,
                                   void* pre_gate, void* pre_up, void* stream) {
  if (group_map == nullptr || w_slots <= 0) w_slots = G;
  if ((pre_gate != nullptr) != (pre_up != nullptr) || (pre_gate != nullptr && mode != kSwiglu)) {
    set_error("moonep_grouped_gemm: pre_gate and pre_up go together and only with SwiGLU");
    return 1;
  }
  if (K % BK != 0 || K <= 0) {
    set_error("moonep_grouped_gemm: K must be a positive multiple of 64");
    return 1;
  }
  const int tile_n = (mode == kSwiglu) ? 128 : BN;
  if (n_per_group % tile_n != 0 || n_per_group <= 0) {
    set_error("moonep_grouped_gemm: N per group must be a multiple of " + std::to_string(tile_n));
    return 1;
  }
  if (mode == kSwiglu && w1 == nullptr) {
    set_error("moonep_grouped_gemm: SwiGLU needs the up-projection weights");
    return 1;
  }
  CUtensorMap ta, tb0, tb1;
  if (int rc = make_tmap(&ta, x, (unsigned long long)rows_cap, (unsigned long long)K, BM)) return rc;
  if (int rc = make_tmap(&tb0, w0, (unsigned long long)w_slots * n_per_group, (unsigned long long)K, 128)) return rc;
  if (int rc = make_tmap(&tb1, mode == kSwiglu ? w1 : w0, (unsigned long long)w_slots * n_per_group,
                         (unsigned long long)K, 128))
    return rc;
  GemmArgs a;
  a.out = (uint16_t*)out;
  a.row_scale = row_scale;
  a.cu_seqlens = cu_seqlens;
  a.status = status;
  a.timeout_ns = (unsigned long long)(timeout_ms > 0 ? timeout_ms : 10000) * 1000000ull;
  a.G = G;
  a.n_per_group = n_per_group;
  a.n_tiles = n_per_group / tile_n;
  a.k_blocks = K / BK;
  a.ldo = n_per_group;
  a.mode = mode;
  a.rows_cap = rows_cap;
  a.group_map = group_map;
  a.w_slots = w_slots;
  a.pre_gate = (uint16_t*)pre_gate;
  a.pre_up = (uint16_t*)pre_up;
  a.b_kn = 0;
  a.k_split = a.k_blocks;
  memset(&a.hooks, 0, sizeof(a.hooks));
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int grid = imax(1, num_sms > 0 ? imin(num_sms, sms) : sms);
  const size_t smem = (size_t)kStages * kStageBytes + 1024;
  static bool attr_set = false;
  if (!attr_set) {
    if (int rc = check_cuda(cudaFuncSetAttribute(grouped_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 (int)smem),
                            "cudaFuncSetAttribute(grouped_gemm_kernel)"))
      return rc;
    attr_set = true;
  }
  grouped_gemm_kernel<<<grid, kGemmThreads, smem, (cudaStream_t)stream>>>(ta, tb0, tb1, a);
  return check_launch("grouped_gemm_kernel");
}

static int launch_wgrad(const CUtensorMap& tl, const CUtensorMap& tr, const WgradArgs& a, int num_sms, void* stream);

// lt: [P, ld] bf16 = L^T, rt: [Q, ld] bf16 = R^T (ld elements per row, a multiple of 8; the column index is the
// row of the dispatched shard).  For every group g with rows [cu[g-1], cu[g]) (a multiple of 16 long):
// out_ptrs[g][P, Q] fp32 = or += L_g^T R_g according to flags[g] (see the kernel).  out_ptrs and flags are
// device arrays of G entries.  P % 128 == 0, Q % 256 == 0.
extern "C" int moonep_grouped_wgrad(const void* lt, const void* rt, long long ld, int P, int Q, const int* cu_seqlens,
                                    int G, void* const* out_ptrs, const int* flags, int rows_cap, int* status,
                                    long long timeout_ms, int num_sms, void* stream) {
  if (P <= 0 || Q <= 0 || P % BM != 0 || Q % BN != 0) {
    set_error("moonep_grouped_wgrad: P must be a multiple of 128 and Q a multiple of 256");
    return 1;
  }
  if (G < 1 || G > kWgradMaxGroups) {
    set_error("moonep_grouped_wgrad: at most " + std::to_string(kWgradMaxGroups) + " groups per launch");
    return 1;
  }
  if (ld <= 0 || ld % 8 != 0 || rows_cap > ld) {
    set_error("moonep_grouped_wgrad: ld must be a multiple of 8 and at least rows_cap");
    return 1;
  }
  CUtensorMap tl, tr;
  if (int rc = make_tmap(&tl, lt, (unsigned long long)P, (unsigned long long)ld, 128)) return rc;
  if (int rc = make_tmap(&tr, rt, (unsigned long long)Q, (unsigned long long)ld, 128)) return rc;
  WgradArgs a;
  a.out_ptrs = (float* const*)out_ptrs;
  a.flags = flags;
  a.cu_seqlens = cu_seqlens;
  a.status = status;
  a.timeout_ns = (unsigned long long)(timeout_ms > 0 ? timeout_ms : 10000) * 1000000ull;
  a.G = G;
  a.P = P;
  a.Q = Q;
  a.p_tiles = P / BM;
  a.q_tiles = Q / BN;
  a.rows_cap = rows_cap;
  a.row_major = 0;
  return launch_wgrad(tl, tr, a, num_sms, stream);
}

// The same with the operands as they are: l = L [rows, P] and r = R [rows, Q] bf16, rows ldl / ldr elements apart
// (multiples of 8), so that column slices of wider tensors can be passed.  No transposed copies are needed: the
// tiles are staged MN-major (see make_smem_desc_mn).
extern "C" int moonep_grouped_wgrad_rows(const void* l, long long ldl, const void* r, long long ldr, int rows, int P,
                                         int Q, const int* cu_seqlens, int G, void* const* out_ptrs, const int* flags,
                                         int* status, long long timeout_ms, int num_sms, void* stream) {
  if (P <= 0 || Q <= 0 || P % BM != 0 || Q % BN != 0) {
    set_error("moonep_grouped_wgrad_rows: P must be a multiple of 128 and Q a multiple of 256");
    return 1;
  }
  if (G < 1 || G > kWgradMaxGroups) {
    set_error("moonep_grouped_wgrad_rows: at most " + std::to_string(kWgradMaxGroups) + " groups per launch");
    return 1;
  }
  if (ldl < P || ldr < Q || ldl % 8 != 0 || ldr % 8 != 0 || rows <= 0) {
    set_error("moonep_grouped_wgrad_rows: row strides must be multiples of 8 and at least the matrix width");
    return 1;
  }
  CUtensorMap tl, tr;
  if (int rc = make_tmap(&tl, l, (unsigned long long)rows, (unsigned long long)P, 64, (unsigned long long)ldl)) return rc;
  if (int rc = make_tmap(&tr, r, (unsigned long long)rows, (unsigned long long)Q, 64, (unsigned long long)ldr)) return rc;
  WgradArgs a;
  a.out_ptrs = (float* const*)out_ptrs;
  a.flags = flags;
  a.cu_seqlens = cu_seqlens;
  a.status = status;
  a.timeout_ns = (unsigned long long)(timeout_ms > 0 ? timeout_ms : 10000) * 1000000ull;
  a.G = G;
  a.P = P;
  a.Q = Q;
  a.p_tiles = P / BM;
  a.q_tiles = Q / BN;
  a.rows_cap = rows;
  a.row_major = 1;
  return launch_wgrad(tl, tr, a, num_sms, stream);
}

static int launch_wgrad(const CUtensorMap& tl, const CUtensorMap& tr, const WgradArgs& a, int num_sms, void* stream) {
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int grid = imax(1, num_sms > 0 ? imin(num_sms, sms) : sms);
  const size_t smem = (size_t)kStages * kStageBytes + 1024 + kWgradStageBytes;
  static bool attr_set = false;
  if (!attr_set) {
    if (int rc = check_cuda(cudaFuncSetAttribute(grouped_wgrad_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 (int)smem),
                            "cudaFuncSetAttribute(grouped_wgrad_kernel)"))
      return rc;
    attr_set = true;
  }
  grouped_wgrad_kernel<<<grid, kGemmThreads, smem, (cudaStream_t)stream>>>(tl, tr, a);
  return check_launch("grouped_wgrad_kernel");
}
