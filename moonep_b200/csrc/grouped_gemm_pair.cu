// Grouped expert GEMM on CTA pairs (tcgen05 cta_group::2): the same operation as grouped_gemm.cu,
//
//   Y[rows of group g, :] = X[rows of group g, :] @ W[g]^T,
//
// with two CTAs of a cluster computing one 256 x 256 tile.  Each CTA stages its own 128 rows of X and
// HALF of the 256 x 64 W tile per K block, one lane of the leader CTA (cluster rank 0) issues MMAs that
// read both CTAs' shared memory and write 128 x 256 fp32 accumulators into both CTAs' TMEM.  Compared
// with one CTA per 128 x 256 tile this halves the W bytes every SM moves through shared memory (32 KB
// instead of 48 KB per K block for the same MMA work), which is what bounds the single-CTA kernel, and
// leaves room for a 6-stage ring.
//
// Per CTA, 192 threads:
//   warp 0      TMA producer (both CTAs): X tile and W half tile of this CTA per K block; the bytes of
//               both CTAs complete the transaction of the LEADER's "full" barrier of the stage.
//   warp 1      allocates this CTA's 512 TMEM columns; in the leader one lane issues four
//               tcgen05.mma.cta_group::2 (M=256, N=256, K=16) per stage and commits to the stage's
//               "empty" barrier in both CTAs, and after the last K block to both "accumulator full" barriers.
//   warps 2..5  epilogue of this CTA's 128 rows (same epilogues as the single-CTA kernel); one arrival
//               per warp on the leader's "accumulator empty" barrier, which counts both CTAs' warps.
//
// Tiles: the 128-row blocks of a group are taken two at a time.  When a group has an odd number of
// blocks the second CTA of its last pair has no rows of that group: it still feeds the MMA (with rows
// that are simply not stored) and skips its stores.  SwiGLU: the leader's W half is the gate tile, the
// other CTA's the up tile, so accumulator columns 0-127 / 128-255 are gate / up as in the single-CTA kernel.
//
// Every mbarrier wait is bounded; on expiry the role records a status word and leaves its loop.  Both
// CTAs always reach the cluster barrier at the end before they free their TMEM and exit, and the leader's
// MMA lane first waits (bounded) for its own last MMA, so no CTA leaves while the pair still works on it.
//
// No counterpart in the reference, which has no GEMM.
#include <cstring>

#include "umma.cuh"

namespace moonep {

namespace {

constexpr int kPairStages = 6;
constexpr int kPairThreads = 192;
constexpr int kPairTmemCols = 512;
constexpr unsigned kPairATileBytes = BM * BK * 2;                         // 16 KB: this CTA's rows of X
constexpr unsigned kPairBHalfBytes = 128 * BK * 2;                        // 16 KB: this CTA's half of the W tile
constexpr unsigned kPairStageBytes = kPairATileBytes + kPairBHalfBytes;   // 32 KB per CTA and stage
constexpr int kPairKernelId = 15;
constexpr int kPairGroupsInSmem = 2048;  // group ends are walked from shared memory up to this many groups

// Walks the pair tiles in order: group-major, then pairs of row blocks, then column tiles (fastest).
struct PairSched {
  const GemmArgs& a;
  const int* cu;     // group ends: the shared-memory copy when it fits, else global memory
  int g;             // current group
  long long t_base;  // index of its first tile
  int blk0;          // its first 128-row block
  int nblk;          // its number of 128-row blocks
  long long tiles;   // its number of pair tiles

  __host__ __device__ PairSched(const GemmArgs& args, const int* ends)
      : a(args), cu(ends), g(-1), t_base(0), blk0(0), nblk(0), tiles(0) {}

  __host__ __device__ void load_group() {
    const int start = g > 0 ? (cu[g - 1] < a.rows_cap ? cu[g - 1] : a.rows_cap) : 0;
    const int end = cu[g] < a.rows_cap ? cu[g] : a.rows_cap;
    blk0 = start / BM;
    nblk = end > start ? (end - start) / BM : 0;
    tiles = (long long)((nblk + 1) / 2) * a.n_tiles;
  }

  // tile t (t never decreases between calls) -> pair index inside the group and column tile; false past the end
  __host__ __device__ bool locate(long long t, int& pair_in_group, int& nb) {
    if (g < 0) {
      g = 0;
      load_group();
    }
    while (t >= t_base + tiles) {
      t_base += tiles;
      if (++g >= a.G) return false;
      load_group();
    }
    const long long r = t - t_base;
    pair_in_group = (int)(r / a.n_tiles);
    nb = (int)(r % a.n_tiles);
    return true;
  }
};

// Bounded wait until *p (+ *bias) reaches `want`; false when the budget ran out.
__device__ __forceinline__ bool hook_wait(const int* p, const int* bias, int want, unsigned long long timeout_ns) {
  if (bias != nullptr) want += ld_volatile(bias);
  if (ld_acquire_sys(p) - want >= 0) return true;
  const unsigned long long t0 = globaltimer_ns();
  unsigned spins = 0;
  while (ld_acquire_sys(p) - want < 0) {
    if ((++spins & 63u) == 0 && globaltimer_ns() - t0 > timeout_ns) return false;
    __nanosleep(200);
  }
  return true;
}

// Warp-wide: all 128 row flags of the block that starts at row0 have reached the epoch.
__device__ __forceinline__ bool rows_arrived(const MoonepGemmHooks& h, int row0, int lane, unsigned long long timeout_ns) {
  const int want = h.row_epoch + (h.row_bias != nullptr ? ld_volatile(h.row_bias) : 0);
  const int4* f4 = reinterpret_cast<const int4*>(h.row_flags + row0) + lane;  // 4 flags per lane; row0 is a multiple of 128
  const unsigned long long t0 = globaltimer_ns();
  unsigned spins = 0;
  for (;;) {
    int4 v;
    asm volatile("ld.acquire.sys.global.v4.s32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(f4) : "memory");
    const bool ok = v.x - want >= 0 && v.y - want >= 0 && v.z - want >= 0 && v.w - want >= 0;
    if (__all_sync(0xffffffffu, ok)) return true;
    const bool late = (++spins & 63u) == 0 && globaltimer_ns() - t0 > timeout_ns;
    if (__any_sync(0xffffffffu, late)) return false;
    __nanosleep(500);
  }
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPairThreads, 1)
    grouped_gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b0,
                             const __grid_constant__ CUtensorMap tmap_b1, const GemmArgs a) {
  extern __shared__ unsigned char s_raw[];
  __shared__ __align__(8) unsigned long long s_full[kPairStages], s_empty[kPairStages], s_tfull[2], s_tempty[2], s_done;
  __shared__ unsigned s_tmem_base;
  __shared__ int s_cu[kPairGroupsInSmem];
  unsigned char* s_tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(s_raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const unsigned rank = cluster_ctarank();  // 0: leader (issues the MMAs), 1: its peer
  // every role walks the groups once; from shared memory a group costs a few cycles instead of an L2 round trip
  const int* cu = a.G <= kPairGroupsInSmem ? s_cu : a.cu_seqlens;
  __shared__ int s_hook_ok;
  if (threadIdx.x == 0) {
    s_hook_ok = 1;
    // the group ends may still be on their way out of the dispatch kernel's table stage
    if (a.hooks.tables_ready != nullptr &&
        !hook_wait(a.hooks.tables_ready, a.hooks.tables_bias, a.hooks.tables_epoch, a.timeout_ns)) {
      gemm_fail(a.status, kPairKernelId, 10, 0, 0);
      s_hook_ok = 0;
    }
  }
  __syncthreads();
  if (a.G <= kPairGroupsInSmem)
    for (int g = threadIdx.x; g < a.G; g += blockDim.x) s_cu[g] = a.cu_seqlens[g];
  const long long pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPairStages; ++s) {
      mbar_init(s_full + s, 1);   // used in the leader: its own arrive.expect_tx; both CTAs' copies complete the bytes
      mbar_init(s_empty + s, 1);  // one commit of the leader's MMA lane, delivered to both CTAs
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(s_tfull + b, 1);   // one commit, delivered to both CTAs
      mbar_init(s_tempty + b, 8);  // used in the leader: four epilogue warps of each CTA
    }
    mbar_init(&s_done, 1);
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(&s_tmem_base, kPairTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers exist before anything is delivered to them
  tc_fence_after();
  const unsigned tmem_base = s_tmem_base;
  // Both CTAs own their whole TMEM, so both accumulators start at column 0; the MMA addresses the peer's
  // TMEM with the leader's address.  Anything else means the SM is shared with another TMEM user: give up.
  const bool tmem_ok = (tmem_base & 0xFFFFu) == 0 && s_hook_ok != 0;
  if ((tmem_base & 0xFFFFu) != 0 && threadIdx.x == 0) gemm_fail(a.status, kPairKernelId, 9, (int)tmem_base, 0);
  const int b_rows_per_tile = (a.mode == kSwiglu) ? 128 : 256;
  // The producer may legitimately spend a whole budget waiting for another kernel's flag; the roles behind it wait
  // longer, so that the status block names the wait that actually ran out.
  const bool hooked = a.hooks.row_flags != nullptr || a.hooks.slot_flags != nullptr;
  const unsigned long long pipe_timeout_ns = hooked ? 3 * a.timeout_ns : a.timeout_ns;

  if (warp == 0) {
    // ---------------- TMA producer (both CTAs) ----------------
    // Lane 0 issues the copies; the whole warp takes part in the (bounded) waits for rows that the dispatch kernel is
    // still delivering and for weight slots the prefetch kernel is still filling.
    if (tmem_ok) {
      PairSched sched(a, cu);
      int stage = 0;
      unsigned phase = 0;
      bool failed = false;
      int pig, nb;
      int checked_blk = -1, checked_slot = -1;
      for (long long t = pair; !failed && sched.locate(t, pig, nb); t += npairs) {
        const int blk = sched.blk0 + 2 * pig + (int)rank;
        const int row0 = blk * BM;  // beyond the group for the odd last block: loaded, never stored
        if (a.hooks.row_flags != nullptr && 2 * pig + (int)rank < sched.nblk && blk != checked_blk) {
          if (!rows_arrived(a.hooks, row0, lane, a.timeout_ns)) {
            if (lane == 0) gemm_fail(a.status, kPairKernelId, 11, blk, sched.g);
            failed = true;
            break;
          }
          checked_blk = blk;
        }
        if (a.hooks.slot_flags != nullptr && sched.g >= a.hooks.slot_first_group && sched.g != checked_slot) {
          int ok = 1;
          if (lane == 0)
            ok = hook_wait(a.hooks.slot_flags + (sched.g - a.hooks.slot_first_group), a.hooks.slot_bias, a.hooks.slot_epoch,
                           a.timeout_ns) ? 1 : 0;
          if (!__shfl_sync(0xffffffffu, ok, 0)) {
            if (lane == 0) gemm_fail(a.status, kPairKernelId, 12, sched.g, 0);
            failed = true;
            break;
          }
          checked_slot = sched.g;
        }
        int wslot = a.group_map != nullptr ? a.group_map[sched.g] : sched.g;
        if (wslot < 0 || wslot >= a.w_slots) {
          // a group whose weights this rank does not hold: reported once, computed with slot 0 (in bounds), never trusted
          if (lane == 0 && sched.nblk > 0) gemm_bad_index(a.status, kPairKernelId, 13, sched.g, wslot);
          wslot = 0;
        }
        const int wrow0 = wslot * a.n_per_group + nb * b_rows_per_tile;
        const CUtensorMap* tb = (a.mode == kSwiglu && rank == 1) ? &tmap_b1 : &tmap_b0;
        const int brow = (a.mode == kSwiglu) ? wrow0 : wrow0 + (int)rank * 128;
        for (int kb = 0; kb < a.k_blocks; ++kb) {
          int got = 1;
          if (lane == 0) got = mbar_wait_cluster(s_empty + stage, phase ^ 1u, pipe_timeout_ns) ? 1 : 0;
          if (!__shfl_sync(0xffffffffu, got, 0)) {
            if (lane == 0) gemm_fail(a.status, kPairKernelId, 1, stage, kb);
            failed = true;
            break;
          }
          if (lane == 0) {
            unsigned char* st = s_tiles + (size_t)stage * kPairStageBytes;
            if (rank == 0) mbar_expect_tx(s_full + stage, 2 * kPairStageBytes);
            const unsigned full_of_leader = mapa_u32(s_full + stage, 0);
            tma_load_2d_pair(st, &tmap_a, kb * BK, row0, full_of_leader);
            if (a.b_kn) {
              // W is [slots, K, N]: this CTA's 128 columns of the tile as two boxes of 64 columns x 64 k
              const bool second = kb >= a.k_split;
              const int kdim = (second ? a.k_blocks - a.k_split : a.k_split) * BK;  // K rows per expert in that tensor
              const int y = wslot * kdim + (second ? kb - a.k_split : kb) * BK;
              const int x0 = nb * BN + (int)rank * 128;
              const CUtensorMap* tw = second ? &tmap_b1 : &tmap_b0;
              tma_load_2d_pair(st + kPairATileBytes, tw, x0, y, full_of_leader);
              tma_load_2d_pair(st + kPairATileBytes + kMnBoxBytes, tw, x0 + 64, y, full_of_leader);
            } else {
              tma_load_2d_pair(st + kPairATileBytes, tb, kb * BK, brow, full_of_leader);
            }
          }
          if (++stage == kPairStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader only) ----------------
    if (lane == 0 && rank == 0 && tmem_ok) {
      constexpr unsigned idesc = make_idesc(2 * BM, BN);
      constexpr unsigned idesc_kn = make_idesc(2 * BM, BN, false, true);
      const unsigned bstep = a.b_kn ? kDescStepMn : kDescStepK;
      PairSched sched(a, cu);
      int stage = 0;
      unsigned phase = 0;
      unsigned tphase[2] = {0, 0};
      int it = 0;
      bool failed = false;
      int pig, nb;
      for (long long t = pair; !failed && sched.locate(t, pig, nb); t += npairs, ++it) {
        const int buf = it & 1;
        if (!mbar_wait_cluster(s_tempty + buf, tphase[buf] ^ 1u, pipe_timeout_ns)) {
          gemm_fail(a.status, kPairKernelId, 2, buf, it);
          failed = true;
          break;
        }
        tphase[buf] ^= 1u;
        tc_fence_after();
        const unsigned d_tmem = tmem_base + (unsigned)(buf * BN);
        for (int kb = 0; kb < a.k_blocks; ++kb) {
          if (!mbar_wait_cluster(s_full + stage, phase, pipe_timeout_ns)) {
            gemm_fail(a.status, kPairKernelId, 3, stage, kb);
            failed = true;
            break;
          }
          tc_fence_after();
          const unsigned char* st = s_tiles + (size_t)stage * kPairStageBytes;
          const unsigned long long adesc = make_smem_desc(st);
          const unsigned long long bdesc = a.b_kn ? make_smem_desc_mn(st + kPairATileBytes) : make_smem_desc(st + kPairATileBytes);
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk)
            umma_bf16_pair(d_tmem, adesc + (unsigned long long)(kk * kDescStepK), bdesc + (unsigned long long)(kk * bstep),
                           a.b_kn ? idesc_kn : idesc, (kb | kk) != 0 ? 1u : 0u);
          umma_commit_pair(s_empty + stage, 3);
          if (++stage == kPairStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!failed) umma_commit_pair(s_tfull + buf, 3);
      }
      // the pair must not be torn down under a running MMA: wait for everything issued so far
      umma_commit_pair(&s_done, 1);
      if (!mbar_wait_cluster(&s_done, 0, pipe_timeout_ns)) gemm_fail(a.status, kPairKernelId, 5, 0, 0);
    }
    __syncwarp();
  } else {
    // ---------------- epilogue (warps 2..5, both CTAs) ----------------
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    const unsigned tempty_of_leader[2] = {mapa_u32(s_tempty + 0, 0), mapa_u32(s_tempty + 1, 0)};
    PairSched sched(a, cu);
    unsigned tphase[2] = {0, 0};
    int it = 0;
    int pig, nb;
    for (long long t = pair; tmem_ok && sched.locate(t, pig, nb); t += npairs, ++it) {
      const int buf = it & 1;
      const int blk_in_group = 2 * pig + (int)rank;
      const bool valid = blk_in_group < sched.nblk;
      int got = 1;
      if (lane == 0) got = mbar_wait_cluster(s_tfull + buf, tphase[buf], pipe_timeout_ns) ? 1 : 0;
      got = __shfl_sync(0xffffffffu, got, 0);
      if (!got) {
        if (lane == 0) gemm_fail(a.status, kPairKernelId, 4, buf, it);
        break;
      }
      tphase[buf] ^= 1u;
      tc_fence_after();
      if (valid) {
        const int row = (sched.blk0 + blk_in_group) * BM + q * 32 + lane;
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
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive_cluster(tempty_of_leader[buf]);
        if (valid && a.hooks.done_counter != nullptr) {
          // this warp's 32 rows x 256 columns of the block are in memory: a consumer counts 4 * column tiles per block
          __threadfence();
          atomicAdd(a.hooks.done_counter + (sched.blk0 + blk_in_group), 1);
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // nobody delivers to, or computes on, a CTA that has left
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kPairTmemCols);
  }
}

}  // namespace

}  // namespace moonep

using namespace moonep;

static int launch_pair(const CUtensorMap& ta, const CUtensorMap& tb0, const CUtensorMap& tb1, const GemmArgs& a,
                       int num_sms, void* stream);

// Same contract as moonep_grouped_gemm (moonep.h).  Returns an error (and launches nothing) when the device
// cannot co-schedule a pair of these CTAs.
extern "C" int moonep_grouped_gemm_pair(const void* x, const void* w0, const void* w1, void* out, const float* row_scale,
                                        const int* cu_seqlens, int G, int rows_cap, int K, int n_per_group, int mode,
                                        int* status, long long timeout_ms, int num_sms, const int* group_map,
                                        int w_slots, void* pre_gate, void* pre_up, void* stream) {
  return moonep_grouped_gemm_pair_hooked(x, w0, w1, out, row_scale, cu_seqlens, G, rows_cap, K, n_per_group, mode, status,
                                         timeout_ms, num_sms, group_map, w_slots, pre_gate, pre_up, nullptr, stream);
}

extern "C" int moonep_grouped_gemm_pair_hooked(const void* x, const void* w0, const void* w1, void* out,
                                               const float* row_scale, const int* cu_seqlens, int G, int rows_cap, int K,
                                               int n_per_group, int mode, int* status, long long timeout_ms, int num_sms,
                                               const int* group_map, int w_slots, void* pre_gate, void* pre_up,
                                               const MoonepGemmHooks* hooks, void* stream) {
  if (group_map == nullptr || w_slots <= 0) w_slots = G;
  if ((pre_gate != nullptr) != (pre_up != nullptr) || (pre_gate != nullptr && mode != kSwiglu)) {
    set_error("moonep_grouped_gemm_pair: pre_gate and pre_up go together and only with SwiGLU");
    return 1;
  }
  if (K % BK != 0 || K <= 0) {
    set_error("moonep_grouped_gemm_pair: K must be a positive multiple of 64");
    return 1;
  }
  const int tile_n = (mode == kSwiglu) ? 128 : BN;
  if (n_per_group % tile_n != 0 || n_per_group <= 0) {
    set_error("moonep_grouped_gemm_pair: N per group must be a multiple of " + std::to_string(tile_n));
    return 1;
  }
  if (mode == kSwiglu && w1 == nullptr) {
    set_error("moonep_grouped_gemm_pair: SwiGLU needs the up-projection weights");
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
  if (hooks != nullptr) a.hooks = *hooks; else memset(&a.hooks, 0, sizeof(a.hooks));
  if (a.hooks.row_flags != nullptr && (reinterpret_cast<uintptr_t>(a.hooks.row_flags) & 15u) != 0) {
    set_error("moonep_grouped_gemm_pair_hooked: row_flags must be 16-byte aligned");
    return 1;
  }
  return launch_pair(ta, tb0, tb1, a, num_sms, stream);
}

// y[rows of g] = x[rows of g] @ W[g] with W given as [slots, K, N] (N contiguous): the layout in which the
// activation gradients need the forward weights, so no transposed copies are made.  x: [rows_cap, K0 + K1];
// w0: [w_slots, K0, N]; w1 (optional): [w_slots, K1, N], continuing the contraction (x = [a | b], W = [w0; w1]).
// out: [rows_cap, N] bf16.  K0, K1 multiples of 64, N a multiple of 256.
extern "C" int moonep_grouped_gemm_pair_kn(const void* x, const void* w0, int K0, const void* w1, int K1, void* out,
                                           const int* cu_seqlens, int G, int rows_cap, int N, int w_slots, int* status,
                                           long long timeout_ms, int num_sms, void* stream) {
  if (w1 == nullptr) K1 = 0;
  if (K0 <= 0 || K0 % BK != 0 || K1 < 0 || K1 % BK != 0 || N <= 0 || N % BN != 0 || w_slots <= 0) {
    set_error("moonep_grouped_gemm_pair_kn: K0, K1 must be multiples of 64 and N a multiple of 256");
    return 1;
  }
  CUtensorMap ta, tb0, tb1;
  if (int rc = make_tmap(&ta, x, (unsigned long long)rows_cap, (unsigned long long)(K0 + K1), BM)) return rc;
  if (int rc = make_tmap(&tb0, w0, (unsigned long long)w_slots * K0, (unsigned long long)N, 64)) return rc;
  if (int rc = make_tmap(&tb1, K1 ? w1 : w0, (unsigned long long)w_slots * (K1 ? K1 : K0), (unsigned long long)N, 64))
    return rc;
  GemmArgs a;
  a.out = (uint16_t*)out;
  a.row_scale = nullptr;
  a.cu_seqlens = cu_seqlens;
  a.status = status;
  a.timeout_ns = (unsigned long long)(timeout_ms > 0 ? timeout_ms : 10000) * 1000000ull;
  a.G = G;
  a.n_per_group = N;
  a.n_tiles = N / BN;
  a.k_blocks = (K0 + K1) / BK;
  a.ldo = N;
  a.mode = kPlain;
  a.rows_cap = rows_cap;
  a.group_map = nullptr;
  a.w_slots = w_slots;
  a.pre_gate = nullptr;
  a.pre_up = nullptr;
  a.b_kn = 1;
  a.k_split = K0 / BK;
  memset(&a.hooks, 0, sizeof(a.hooks));
  return launch_pair(ta, tb0, tb1, a, num_sms, stream);
}

static int launch_pair(const CUtensorMap& ta, const CUtensorMap& tb0, const CUtensorMap& tb1, const GemmArgs& a,
                       int num_sms, void* stream) {
  const size_t smem = (size_t)kPairStages * kPairStageBytes + 1024;
  static int max_pairs = -1;  // pairs of these CTAs the device runs at once
  if (max_pairs < 0) {
    if (int rc = check_cuda(cudaFuncSetAttribute(grouped_gemm_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 (int)smem),
                            "cudaFuncSetAttribute(grouped_gemm_pair_kernel)"))
      return rc;
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(sms / 2 * 2));
    cfg.blockDim = dim3(kPairThreads);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (int rc = check_cuda(cudaOccupancyMaxActiveClusters(&n, grouped_gemm_pair_kernel, &cfg),
                            "cudaOccupancyMaxActiveClusters(grouped_gemm_pair_kernel)"))
      return rc;
    max_pairs = n;
  }
  if (max_pairs < 1) {
    set_error("moonep_grouped_gemm_pair: the device cannot run a pair of these CTAs");
    return 1;
  }
  int pairs = max_pairs;
  if (num_sms > 0) pairs = imax(1, imin(pairs, num_sms / 2));
  grouped_gemm_pair_kernel<<<2 * pairs, kPairThreads, smem, (cudaStream_t)stream>>>(ta, tb0, tb1, a);
  return check_launch("grouped_gemm_pair_kernel");
}

// Host-side walk of the tile schedule of one CTA pair (for tests): writes, for every tile that pair `pair` of
// `npairs` visits, {group, first row of the leader's block, first row of the peer's block or -1 when the group has no
// such block, column tile} into out[4 * i]; returns the number of tiles (at most max_tiles are written).
extern "C" int moonep_pair_schedule(const int* cu_seqlens, int G, int rows_cap, int n_tiles, int pair, int npairs,
                                    int* out, int max_tiles) {
  GemmArgs a = {};
  a.G = G;
  a.rows_cap = rows_cap;
  a.n_tiles = n_tiles;
  PairSched sched(a, cu_seqlens);
  int n = 0, pig = 0, nb = 0;
  for (long long t = pair; sched.locate(t, pig, nb); t += npairs) {
    if (n < max_tiles) {
      out[4 * n + 0] = sched.g;
      out[4 * n + 1] = (sched.blk0 + 2 * pig) * BM;
      out[4 * n + 2] = 2 * pig + 1 < sched.nblk ? (sched.blk0 + 2 * pig + 1) * BM : -1;
      out[4 * n + 3] = nb;
    }
    ++n;
  }
  return n;
}
