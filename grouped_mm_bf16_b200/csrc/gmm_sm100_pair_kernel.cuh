// CTA-pair variant of the persistent grouped GEMM for sm_100a (all three modes).
//
// Two CTAs on the two SMs of one TPC (a cluster of 2) share every 256 x 256 output tile:
// CTA r loads rows [128 r, 128 r + 128) of the A tile and columns [128 r, 128 r + 128) of the B
// tile into its own shared memory, the leader (r = 0) issues tcgen05.mma.cta_group::2
// (256 x 256 x 16), which reads both CTAs' shared memory and accumulates rows 128 r.. into CTA r's
// tensor memory, and each CTA's epilogue warps store their own 128 rows. Per SM this moves 32 KiB
// per 64-deep k-block from L2 instead of the 48 KiB of the single-CTA kernel, and leaves room for a
// 6-stage ring; both are what the single-CTA kernel is short of on large problems.
//
// Every TMA load has exactly one destination CTA. Cross-CTA signalling uses mbarriers only:
//   full[s]      lives in the leader; both CTAs' loads credit their bytes to it
//   empty[s]     one per CTA; the leader's tcgen05.commit arrives on both
//   acc_full[b]  one per CTA; same
//   acc_empty[b] lives in the leader; the 2 x 128 epilogue threads arrive on it
//
// K-ragged mode (KRAGGED = true) loads through per-group tensor maps whose K extent ends at the
// group's end (FastParams::maps_a / maps_b), so the k-rows a group's last k-block reads past its
// end arrive as zeros in both CTAs and the main loop is the same as in the other modes; tiles are
// dealt in cost order (gmm_common.cuh) and an empty group's tiles are stored as zeros.
#pragma once

#include "gmm_sm100_kernel.cuh"

namespace gmm {

constexpr int kPairBM = 256;       // rows of a pair tile (128 per CTA)
constexpr int kPairBNHalf = 128;   // B columns held by one CTA
constexpr int kPairStages = 6;
constexpr int kPairAStageBytes = 128 * kBK * 2;            // 16 KiB
constexpr int kPairBStageBytes = kPairBNHalf * kBK * 2;    // 16 KiB
constexpr int kPairStageBytes = kPairAStageBytes + kPairBStageBytes;

struct PairSmemTail {
  uint64_t full[kPairStages];
  uint64_t empty[kPairStages];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
  SchedSmem sched;
};

constexpr size_t kPairSmemBytes =
    1024 + size_t(kPairStages) * kPairStageBytes + kEpilogueStageBytes + sizeof(PairSmemTail);

enum PairStatus : int {
  ST_PAIR_PRODUCER_TIMEOUT = 0x201,
  ST_PAIR_MMA_TIMEOUT = 0x202,
  ST_PAIR_EPILOGUE_TIMEOUT = 0x203,
};

// SWIGLU (row-ragged mode): B holds [gate | up], 2 N columns per group; the leader CTA loads the
// tile's 128 gate columns, its peer the matching 128 up columns, so that every accumulator row holds
// gate in columns 0..127 and up in 128..255, and the stored tile is 256 x 128.
// ES: operand element size, 2 (bf16/fp16) or 4 (fp32 read as TF32), as in the single-CTA kernel.
template <bool KRAGGED, typename TOut, bool SWIGLU = false, int ES = 2>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kFastThreads, 1)
gmm_sm100_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                      const __grid_constant__ CUtensorMap tmap_c, const __grid_constant__ FastParams fp) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + kPairStages * kPairAStageBytes;
  uint8_t* epi_stage = smem + kPairStages * kPairStageBytes;  // 1024-byte aligned
  PairSmemTail& tail = *reinterpret_cast<PairSmemTail*>(epi_stage + kEpilogueStageBytes);
  volatile int* abort_flag = &tail.abort_flag;

  using EG = ElemGeom<ES>;
  constexpr int BK = EG::BK;
  constexpr int kChunks = 128 / EG::CHUNK_W;   // MN-major chunks per 128-wide operand half
  constexpr int BNT = SWIGLU ? kBN / 2 : kBN;  // output columns per tile
  static_assert(!SWIGLU || (!KRAGGED && ES == 2), "the fused activation exists for 16-bit row-ragged problems");
  const CanonProblem& p = fp.p;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = leader
  const int pair = blockIdx.x >> 1;
  const int n_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPairStages; ++s) {
      mbar_init(&tail.full[s], 1);
      mbar_init(&tail.empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tail.acc_full[b], 1);
      mbar_init(&tail.acc_empty[b], 2 * kEpilogueThreads);
    }
    tail.abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc_pair(&tail.tmem_base, kTmemCols);
    tmem_relinquish_pair();
  }
  sched_init<kPairBM, BNT>(p, tail.sched);
  tcgen05_fence_before_sync();
  cluster_sync_all();  // barriers of both CTAs are initialised before anyone signals across
  tcgen05_fence_after_sync();

  const uint32_t tmem_base = tail.tmem_base;
  const int total = tail.sched.total;
  const int a_batched = (p.mode == MODE_UNIFORM);

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (one thread per CTA)
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      const CUtensorMap* ta = &tmap_a;
      const CUtensorMap* tb = &tmap_b;
      int map_g = -1;
      const uint32_t full0_leader = map_to_cta(smem_u32(&tail.full[0]), 0);
      for (int round = 0; ok; ++round) {
        const int t = tile_of_round<KRAGGED>(round, pair, n_pairs);
        if (t >= total) break;
        const TileInfo ti = decode_tile<kPairBM, BNT>(p, tail.sched, t);
        const int nkb = (ti.klen + BK - 1) / BK;
        const int az = a_batched ? ti.g : 0;
        const int bz = KRAGGED ? 0 : ti.g;
        const int row0 = ti.m0 + int(rank) * 128;
        const int col0 = SWIGLU ? (rank ? p.N + ti.n0 : ti.n0) : ti.n0 + int(rank) * kPairBNHalf;
        if constexpr (KRAGGED) {
          if (nkb > 0 && ti.g != map_g) {
            map_g = ti.g;
            ta = fp.maps_a + map_g;
            tb = fp.maps_b + map_g;
            tensormap_fence_acquire(ta);
            tensormap_fence_acquire(tb);
          }
        }
        for (int kb = 0; kb < nkb; ++kb) {
          if (!mbar_wait(&tail.empty[s], ph ^ 1, abort_flag)) {
            atomicCAS(p.status, 0, ST_PAIR_PRODUCER_TIMEOUT);
            ok = false;
            break;
          }
          // Both CTAs' loads are credited to the leader's full[s].
          if (rank == 0) mbar_arrive_expect_tx(&tail.full[s], 2 * kPairStageBytes);
          const uint32_t bar = full0_leader + s * (uint32_t)sizeof(uint64_t);
          const int k = ti.k0 + kb * BK;
          uint8_t* sa = smem_a + s * kPairAStageBytes;
          uint8_t* sb = smem_b + s * kPairBStageBytes;
          auto load_a = [&](void* dst, int x, int y) { tma_load_3d_pair(dst, ta, bar, x, y, az); };
          auto load_b = [&](void* dst, int x, int y) { tma_load_3d_pair(dst, tb, bar, x, y, bz); };
          if (!fp.a_mn) {
            load_a(sa, k, row0);
          } else {
#pragma unroll
            for (int c = 0; c < kChunks; ++c) load_a(sa + c * EG::CHUNK_BYTES, row0 + c * EG::CHUNK_W, k);
          }
          if (!fp.b_mn) {
            load_b(sb, k, col0);
          } else {
#pragma unroll
            for (int c = 0; c < kChunks; ++c) load_b(sb + c * EG::CHUNK_BYTES, col0 + c * EG::CHUNK_W, k);
          }
          if (++s == kPairStages) { s = 0; ph ^= 1; }
        }
      }
      // After a give-up: a bounded time for the copies already requested (by either CTA: all are
      // credited to the leader's barriers) to land before the pair leaves.
      if (!ok && rank == 0) drain_ring<kPairStages>(tail.full, s, ph);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA, one thread)
    if (rank == 0 && lane == 0) {
      // descriptor geometry: see the single-CTA kernel
      const uint32_t a_lbo = fp.a_mn ? EG::CHUNK_BYTES : 16;
      const uint32_t b_lbo = fp.b_mn ? EG::CHUNK_BYTES : 16;
      const uint32_t a_kstep = fp.a_mn ? (EG::UMMA_K * 128) : 32;
      const uint32_t b_kstep = fp.b_mn ? (EG::UMMA_K * 128) : 32;
      const uint32_t a_sbo = (ES == 4 && fp.a_mn) ? 512 : 1024;
      const uint32_t b_sbo = (ES == 4 && fp.b_mn) ? 512 : 1024;
      const uint32_t a_swz = (ES == 4 && fp.a_mn) ? kSwizzle128BBase32B : kSwizzle128B;
      const uint32_t b_swz = (ES == 4 && fp.b_mn) ? kSwizzle128BBase32B : kSwizzle128B;
      int s = 0;
      uint32_t ph = 0;
      int it = 0;
      bool ok = true;
      for (; ok; ++it) {
        const int t = tile_of_round<KRAGGED>(it, pair, n_pairs);
        if (t >= total) break;
        const int klen = tile_klen(p, tail.sched, t);  // the issuer needs no tile coordinates
        const int nkb = (klen + BK - 1) / BK;
        const int buf = it & 1;
        const uint32_t aph = (it >> 1) & 1;
        if (!mbar_wait_cluster(&tail.acc_empty[buf], aph ^ 1, abort_flag)) {
          atomicCAS(p.status, 0, ST_PAIR_MMA_TIMEOUT);
          break;
        }
        tcgen05_fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * kBN;
        for (int kb = 0; kb < nkb; ++kb) {
          if (!mbar_wait(&tail.full[s], ph, abort_flag)) {
            atomicCAS(p.status, 0, ST_PAIR_MMA_TIMEOUT + 0x10);
            ok = false;
            break;
          }
          tcgen05_fence_after_sync();
          const uint64_t a_desc = make_smem_desc_sw128(smem_u32(smem_a + s * kPairAStageBytes), a_lbo, a_sbo, a_swz);
          const uint64_t b_desc = make_smem_desc_sw128(smem_u32(smem_b + s * kPairBStageBytes), b_lbo, b_sbo, b_swz);
#pragma unroll
          for (int k = 0; k < BK / EG::UMMA_K; ++k) {
            if constexpr (ES == 4)
              umma_tf32_ss_pair(d_tmem, a_desc + ((k * a_kstep) >> 4), b_desc + ((k * b_kstep) >> 4), fp.idesc,
                                (kb | k) != 0 ? 1u : 0u);
            else
              umma_f16_ss_pair(d_tmem, a_desc + ((k * a_kstep) >> 4), b_desc + ((k * b_kstep) >> 4), fp.idesc,
                               (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit_pair(&tail.empty[s], 0x3);  // frees the stage in both CTAs
          if (++s == kPairStages) { s = 0; ph ^= 1; }
        }
        if (ok) umma_commit_pair(&tail.acc_full[buf], 0x3);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5 of both CTAs)
    const int q = warp & 3;
    TOut* c_base = reinterpret_cast<TOut*>(p.c);
    int it = 0;
    bool ok = true;
    for (; ok; ++it) {
      const int t = tile_of_round<KRAGGED>(it, pair, n_pairs);
      if (t >= total) break;
      const TileInfo ti = decode_tile<kPairBM, BNT>(p, tail.sched, t);
      const int buf = it & 1;
      const uint32_t aph = (it >> 1) & 1;
      // warp-uniform outcome, as in the single-CTA kernel
      if (!__all_sync(0xffffffffu, mbar_wait(&tail.acc_full[buf], aph, abort_flag, kEpilogueBackoffNs))) {
        if (lane == 0) atomicCAS(p.status, 0, ST_PAIR_EPILOGUE_TIMEOUT);
        ok = false;
        break;
      }
      tcgen05_fence_after_sync();
      const int row0 = int(rank) * 128 + q * 32;  // first row of this warp inside the pair tile
      TOut* c_warp = c_base + (long long)ti.g * p.c_sg + (long long)(ti.m0 + row0) * p.c_sm +
                     (long long)ti.n0 * p.c_sn;
      const uint32_t t_row = tmem_base + (uint32_t(q * 32) << 16) + buf * kBN;
      const int ncols_tile = min(BNT, p.N - ti.n0);
      // A warp whose rows lie wholly past the group's end has nothing to read or store.
      if (row0 < ti.rows) {
        if constexpr (SWIGLU)
          epilogue_store_warp_swiglu<TOut>(t_row, c_warp, p.c_sm, p.c_sn, ti.rows - row0, ncols_tile,
                                           epi_stage + (warp - 2) * kWarpStageBytes, lane);
        else
          epilogue_store_warp<TOut>(t_row, c_warp, p.c_sm, p.c_sn, ti.rows - row0, ncols_tile,
                                    epi_stage + (warp - 2) * kWarpStageBytes, KRAGGED && ti.klen == 0, lane,
                                    fp.c_tma ? &tmap_c : nullptr, ti.n0, ti.m0 + row0,
                                    p.mode == MODE_MRAGGED ? 0 : ti.g);
      }
      tcgen05_fence_before_sync();
      mbar_arrive_cluster(map_to_cta(smem_u32(&tail.acc_empty[buf]), 0));
    }
    if (fp.c_tma && lane == 0) tma_store_wait_all();  // the staging area outlives its last store
  }

  // ------------------------------------------------------------ teardown
  __syncwarp();
  tcgen05_fence_before_sync();
  cluster_sync_all();  // neither CTA leaves while its peer may still read its shared memory or signal it
  if (warp == 1) {
    tcgen05_fence_after_sync();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

}  // namespace gmm
