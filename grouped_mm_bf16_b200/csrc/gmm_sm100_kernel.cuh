// Persistent, warp-specialised grouped GEMM for sm_100a.
//
//   warp 0      TMA producer   : cp.async.bulk.tensor loads of A/B k-blocks into a 4-stage ring
//   warp 1      MMA issuer     : tcgen05.mma (128 x 256 x 16, bf16/fp16 in, fp32 accumulate in TMEM;
//                                or 128 x 256 x 8 with fp32 operands read as TF32)
//   warps 2..5  epilogue       : tcgen05.ld -> one rounding to the output type -> masked global stores
//
// Each CTA owns 512 TMEM columns = two 128 x 256 fp32 accumulators, so the epilogue of tile i
// overlaps the main loop of tile i+1. Tiles are (group, m-tile, n-tile) items decoded on the
// device from `offs` (gmm_common.cuh); every role walks the same sequence of tiles, one per
// round (tile_of_round): blockIdx.x, blockIdx.x + gridDim.x, ... and, in K-ragged mode where
// tiles are sorted by cost, every other round backwards.
//
// Replaces the reference's Triton kernels for the same math: kernels.py:197-245 (3D x 3D),
// kernels.py:304-419 (2D x 3D main + prologue pair) and kernels.py:248-301 (2D x 2D), all of
// which accumulate in fp32 and round once at the store, as this kernel does.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "gmm_common.cuh"
#include "sm100_ptx.cuh"

namespace gmm {

constexpr int kBM = 128;
constexpr int kBN = 256;
constexpr int kBK = 64;   // 64 16-bit elements = one 128-byte swizzle row
constexpr int kUmmaK = 16;
constexpr int kStages = 4;
constexpr int kAStageBytes = kBM * kBK * 2;          // 16 KiB
constexpr int kBStageBytes = kBN * kBK * 2;          // 32 KiB
constexpr int kStageBytes = kAStageBytes + kBStageBytes;
constexpr int kChunkBytes = 64 * kBK * 2;            // one 64-wide MN chunk of an MN-major operand: 8 KiB
constexpr int kTmemCols = 512;

// Tile geometry by operand element size ES (2: bf16/fp16, 4: fp32 read as TF32). A stage always
// holds 128-byte swizzle rows, so its size in bytes does not depend on ES; its extent along K does.
template <int ES>
struct ElemGeom {
  static constexpr int BK = 128 / ES;           // elements of K per stage: 64 or 32
  static constexpr int UMMA_K = 32 / ES;        // K per tcgen05.mma: 16 or 8
  static constexpr int CHUNK_W = 128 / ES;      // MN elements per 128-byte row of an MN-major chunk
  static constexpr int CHUNK_BYTES = BK * 128;  // one MN chunk: BK k-rows of 128 bytes (8 KiB or 4 KiB)
};
constexpr int kFastThreads = 192;
constexpr int kEpilogueThreads = 128;
constexpr unsigned kEpilogueBackoffNs = 128;  // sleep between polls while an epilogue warp waits for a tile

struct FastSmemTail {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
  SchedSmem sched;
};

// Per-warp staging area used to turn "one thread = one output row" (the TMEM read layout) into
// row-contiguous global stores: 32 rows of 128 bytes, the 16-byte segments of row r stored at
// position (segment ^ (r & 7)). That is the 128-byte swizzle of the tensor maps, so a TMA store can
// read the area as a 32-row box, and it keeps both the row-wise writes and the transposed reads
// free of bank conflicts. Each warp's area starts on a 1024-byte boundary.
constexpr int kStageRowBytes = 128;
constexpr int kWarpStageBytes = 32 * kStageRowBytes;
constexpr int kEpilogueStageBytes = 4 * kWarpStageBytes;

__device__ __forceinline__ uint4* stage_seg(uint8_t* stage, int row, int seg) {
  return reinterpret_cast<uint4*>(stage + row * kStageRowBytes + ((seg ^ (row & 7)) << 4));
}

constexpr size_t kFastSmemBytes =
    1024 /*alignment slack*/ + size_t(kStages) * kStageBytes + kEpilogueStageBytes + sizeof(FastSmemTail);

struct FastParams {
  CanonProblem p;
  uint32_t idesc;  // tcgen05 instruction descriptor (formats, majors, M=128, N=256)
  int a_mn;        // 1: A is MN-major in memory (column-major [M,K]); 0: K-major
  int b_mn;        // 1: B is MN-major in memory (row-major [K,N]);    0: K-major
  int c_tma;       // 1: the output has a tensor map (unit column stride, 16-byte aligned rows): whole
                   //    32-row x 128-byte pieces of a tile are written with TMA stores
  // K-ragged mode only: one tensor map per group and operand, in global memory, written by
  // build_group_maps_kernel just before this launch. Map g equals the operand's map except that
  // its K extent ends at the group's end, so a k-block that reaches past the group arrives with
  // zeros in the rows that belong to the next group and contributes exactly nothing.
  const CUtensorMap* maps_a;
  const CUtensorMap* maps_b;
  // Single-CTA kernel, row-ragged and uniform modes: a tile with at most 64 valid rows (the tail of a
  // group) is multiplied with M = 64 instructions, which read rows 0..63 of the A stage and leave
  // rows 16 w .. 16 w + 15 in lanes 0..15 of TMEM lane quarter w. 0 = off (every tile M = 128).
  uint32_t idesc_half;
  CUtensorMap tmap_a_half;  // K-major A with a 64-row box, for those tiles (unused when A is MN-major)
};

// Writes the per-group tensor maps of the K-ragged mode: thread g copies both operands' maps and
// sets their K extent (dimension 1: both operands are MN-major there) to the clamped end of group g.
// An empty group gets extent 1; no copy is ever issued with its maps.
__global__ void build_group_maps_kernel(const __grid_constant__ CUtensorMap tmap_a,
                                        const __grid_constant__ CUtensorMap tmap_b, const int* __restrict__ offs,
                                        int n_groups, int k_total, CUtensorMap* maps_a, CUtensorMap* maps_b) {
  const int g = blockIdx.x * blockDim.x + threadIdx.x;
  if (g >= n_groups) return;
  int e = offs[g];
  e = e < 0 ? 0 : (e > k_total ? k_total : e);
  const uint32_t extent = e > 0 ? (uint32_t)e : 1u;
  const uint4* src_a = reinterpret_cast<const uint4*>(&tmap_a);
  const uint4* src_b = reinterpret_cast<const uint4*>(&tmap_b);
  uint4* dst_a = reinterpret_cast<uint4*>(maps_a + g);
  uint4* dst_b = reinterpret_cast<uint4*>(maps_b + g);
#pragma unroll
  for (int i = 0; i < (int)(sizeof(CUtensorMap) / sizeof(uint4)); ++i) {
    dst_a[i] = src_a[i];
    dst_b[i] = src_b[i];
  }
  tensormap_set_dim1(maps_a + g, extent);
  tensormap_set_dim1(maps_b + g, extent);
  tensormap_fence_release();
}

// Producer give-up path: waits, for a bounded time per stage, until the copies requested so far
// have landed. `s` and `ph` are the producer's ring position: stages before `s` were last requested
// in the phase of parity `ph`, the others in the phase before (never, on the first trip round the
// ring: waiting for the phase before a barrier's first returns at once).
template <int STAGES>
__device__ __forceinline__ void drain_ring(uint64_t* full, int s, uint32_t ph) {
  for (int i = 0; i < STAGES; ++i) {
    const uint32_t parity = (i < s) ? ph : (ph ^ 1u);
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000LL) {
      if (mbar_try_wait(&full[i], parity)) break;
    }
  }
}

// Status codes written to CanonProblem::status when a bounded wait gives up.
enum FastStatus : int {
  ST_OK = 0,
  ST_PRODUCER_TIMEOUT = 0x101,
  ST_MMA_TIMEOUT = 0x102,
  ST_EPILOGUE_TIMEOUT = 0x103,
};

template <typename TOut>
struct OutCvt;
template <>
struct OutCvt<__nv_bfloat16> {
  static __device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  static __device__ __forceinline__ __nv_bfloat16 one(float x) { return __float2bfloat16_rn(x); }
};
template <>
struct OutCvt<__half> {
  static __device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  static __device__ __forceinline__ __half one(float x) { return __float2half_rn(x); }
};
template <>
struct OutCvt<float> {
  static __device__ __forceinline__ float one(float x) { return x; }
};

// Stores up to 32 consecutive columns of one output row. `r` holds fp32 bit patterns.
template <typename TOut>
__device__ __forceinline__ void store_row_chunk(TOut* dst, long long col_stride, const uint32_t (&r)[32],
                                                int ncols) {
  const bool vec = (col_stride == 1) && (ncols == 32) && ((reinterpret_cast<uintptr_t>(dst) & 15u) == 0);
  if (vec) {
    if constexpr (sizeof(TOut) == 4) {
      uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
      for (int i = 0; i < 8; ++i) d4[i] = make_uint4(r[4 * i], r[4 * i + 1], r[4 * i + 2], r[4 * i + 3]);
    } else {
      uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        uint4 v;
        v.x = OutCvt<TOut>::pack2(__uint_as_float(r[8 * i + 0]), __uint_as_float(r[8 * i + 1]));
        v.y = OutCvt<TOut>::pack2(__uint_as_float(r[8 * i + 2]), __uint_as_float(r[8 * i + 3]));
        v.z = OutCvt<TOut>::pack2(__uint_as_float(r[8 * i + 4]), __uint_as_float(r[8 * i + 5]));
        v.w = OutCvt<TOut>::pack2(__uint_as_float(r[8 * i + 6]), __uint_as_float(r[8 * i + 7]));
        d4[i] = v;
      }
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      if (i < ncols) dst[i * col_stride] = OutCvt<TOut>::one(__uint_as_float(r[i]));
    }
  }
}

// Stores this warp's 32 rows of one accumulator tile. `t_row` is the TMEM address of the warp's
// lane quarter at column 0 of the tile, `c_warp` points at (first row of the warp, first column of
// the tile), `rows` is how many of the warp's 32 rows are valid (<= 0: none), `ncols` how many of
// the tile's columns are. Whole-warp call: tcgen05.ld is warp-collective.
//
// Fast path (unit column stride, 16-byte aligned rows, full 128-byte chunk): each thread converts
// 128 bytes of its row and parks them in shared memory; the warp then writes 4 rows x 128 bytes per
// instruction, i.e. whole cache lines, instead of 32 scattered 16-byte pieces. When the output has a
// tensor map (`tmap_c`, else null) and all 32 rows are valid, one TMA store of the 32 x 128-byte
// box replaces those loads and stores; (cx, cy, cz) are the box coordinates of the warp's first
// row at column 0 of the tile.
template <typename TOut>
__device__ __forceinline__ void epilogue_store_warp(uint32_t t_row, TOut* c_warp, long long c_sm, long long c_sn,
                                                    int rows, int ncols, uint8_t* stage, bool zero_tile, int lane,
                                                    const CUtensorMap* tmap_c = nullptr, int cx = 0, int cy = 0,
                                                    int cz = 0) {
  constexpr int CW = 128 / (int)sizeof(TOut);  // columns per 128-byte chunk: 32 (fp32) or 64 (16-bit)
  const bool by_tma = tmap_c != nullptr && rows >= 32;
  const bool rows_aligned = (c_sn == 1) && ((reinterpret_cast<uintptr_t>(c_warp) & 15u) == 0) &&
                            (((c_sm * (long long)sizeof(TOut)) & 15) == 0);
  const bool row_ok = lane < rows;
  TOut* c_row = c_warp + (long long)lane * c_sm;
#pragma unroll 1
  for (int c0 = 0; c0 < ncols; c0 += CW) {
    uint32_t r[CW];
    {
      uint32_t (&lo)[32] = *reinterpret_cast<uint32_t (*)[32]>(&r[0]);
      tmem_ld_32x32b_x32(t_row + c0, lo);
      if constexpr (CW == 64) {
        uint32_t (&hi)[32] = *reinterpret_cast<uint32_t (*)[32]>(&r[32]);
        tmem_ld_32x32b_x32(t_row + c0 + 32, hi);
      }
      tmem_ld_wait();
    }
    if (zero_tile) {
#pragma unroll
      for (int i = 0; i < CW; ++i) r[i] = 0;
    }
    if (rows_aligned && c0 + CW <= ncols) {
      if (tmap_c != nullptr) {
        // A TMA store issued for the previous chunk, or for the previous tile, may still be reading
        // the staging area (lane 0 issues them all, so its wait covers them all).
        if (lane == 0) tma_store_wait_read();
        __syncwarp();
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        uint4 v;
        if constexpr (sizeof(TOut) == 4) {
          v = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
        } else {
          v.x = OutCvt<TOut>::pack2(__uint_as_float(r[8 * j + 0]), __uint_as_float(r[8 * j + 1]));
          v.y = OutCvt<TOut>::pack2(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]));
          v.z = OutCvt<TOut>::pack2(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]));
          v.w = OutCvt<TOut>::pack2(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]));
        }
        *stage_seg(stage, lane, j) = v;
      }
      if (by_tma) {
        fence_proxy_async_smem();  // this thread's row is visible to the TMA engine
        __syncwarp();
        if (lane == 0) {
          tma_store_3d(tmap_c, stage, cx + c0, cy, cz);
          tma_store_commit();
        }
        continue;
      }
      __syncwarp();
      const int seg = lane & 7;   // 16-byte segment of the 128-byte row chunk
      const int sub = lane >> 3;  // which of the 4 rows of this instruction
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int row = i * 4 + sub;
        const uint4 v = *stage_seg(stage, row, seg);
        if (row < rows) {
          uint8_t* dst = reinterpret_cast<uint8_t*>(c_warp + (long long)row * c_sm + c0) + seg * 16;
          *reinterpret_cast<uint4*>(dst) = v;
        }
      }
      __syncwarp();
    } else if (row_ok) {
      // Edge chunk, strided or unaligned output: every thread stores its own row.
      uint32_t (&lo)[32] = *reinterpret_cast<uint32_t (*)[32]>(&r[0]);
      store_row_chunk<TOut>(c_row + (long long)c0 * c_sn, c_sn, lo, min(32, ncols - c0));
      if constexpr (CW == 64) {
        if (c0 + 32 < ncols) {
          uint32_t (&hi)[32] = *reinterpret_cast<uint32_t (*)[32]>(&r[32]);
          store_row_chunk<TOut>(c_row + (long long)(c0 + 32) * c_sn, c_sn, hi, min(32, ncols - c0 - 32));
        }
      }
    }
  }
}

// The same for a tile whose accumulator holds two 128-column halves, G (columns 0..127) and U
// (128..255): the stored tile has 128 columns, silu(G) * U evaluated on the fp32 accumulators.
// Works through 32 columns at a time (one tcgen05.ld of each half) to keep the register count down.
__device__ __forceinline__ float silu_mul(float g, float u) { return __fdividef(g, 1.0f + __expf(-g)) * u; }

template <typename TOut>
__device__ __forceinline__ void epilogue_store_warp_swiglu(uint32_t t_row, TOut* c_warp, long long c_sm,
                                                           long long c_sn, int rows, int ncols, uint8_t* stage,
                                                           int lane) {
  constexpr int CW = 128 / (int)sizeof(TOut);
  const bool rows_aligned = (c_sn == 1) && ((reinterpret_cast<uintptr_t>(c_warp) & 15u) == 0) &&
                            (((c_sm * (long long)sizeof(TOut)) & 15) == 0);
  const bool row_ok = lane < rows;
  TOut* c_row = c_warp + (long long)lane * c_sm;
#pragma unroll 1
  for (int c0 = 0; c0 < ncols; c0 += CW) {
    const bool whole = rows_aligned && c0 + CW <= ncols;
#pragma unroll 1
    for (int h = 0; h < CW / 32; ++h) {
      const int c = c0 + 32 * h;
      if (c >= ncols) break;
      uint32_t v[32], up[32];
      tmem_ld_32x32b_x32(t_row + c, v);
      tmem_ld_32x32b_x32(t_row + 128 + c, up);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(silu_mul(__uint_as_float(v[i]), __uint_as_float(up[i])));
      if (whole) {
        if constexpr (sizeof(TOut) == 4) {
#pragma unroll
          for (int j = 0; j < 8; ++j)
            *stage_seg(stage, lane, j) = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 w;
            w.x = OutCvt<TOut>::pack2(__uint_as_float(v[8 * j + 0]), __uint_as_float(v[8 * j + 1]));
            w.y = OutCvt<TOut>::pack2(__uint_as_float(v[8 * j + 2]), __uint_as_float(v[8 * j + 3]));
            w.z = OutCvt<TOut>::pack2(__uint_as_float(v[8 * j + 4]), __uint_as_float(v[8 * j + 5]));
            w.w = OutCvt<TOut>::pack2(__uint_as_float(v[8 * j + 6]), __uint_as_float(v[8 * j + 7]));
            *stage_seg(stage, lane, h * 4 + j) = w;
          }
        }
      } else if (row_ok) {
        store_row_chunk<TOut>(c_row + (long long)c * c_sn, c_sn, v, min(32, ncols - c));
      }
    }
    if (whole) {
      __syncwarp();
      const int seg = lane & 7;
      const int sub = lane >> 3;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int row = i * 4 + sub;
        const uint4 w = *stage_seg(stage, row, seg);
        if (row < rows) {
          uint8_t* dst = reinterpret_cast<uint8_t*>(c_warp + (long long)row * c_sm + c0) + seg * 16;
          *reinterpret_cast<uint4*>(dst) = w;
        }
      }
      __syncwarp();
    }
  }
}

// SWIGLU (row-ragged mode, 16-bit operands): B holds 2 N columns per group, [gate | up]; an output
// tile has 128 columns, its accumulator the matching 128 gate and 128 up columns side by side.
template <bool KRAGGED, typename TOut, int ES = 2, bool SWIGLU = false>
__global__ void __launch_bounds__(kFastThreads, 1)
gmm_sm100_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ CUtensorMap tmap_c, const __grid_constant__ FastParams fp) {
  extern __shared__ uint8_t smem_raw[];
  // 128-byte swizzled tiles must start on 1024-byte boundaries.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + kStages * kAStageBytes;
  uint8_t* epi_stage = smem + kStages * kStageBytes;  // 1024-byte aligned, like the stages before it
  FastSmemTail& tail = *reinterpret_cast<FastSmemTail*>(epi_stage + kEpilogueStageBytes);
  volatile int* abort_flag = &tail.abort_flag;

  using EG = ElemGeom<ES>;
  constexpr int BK = EG::BK;
  constexpr int BNT = SWIGLU ? kBN / 2 : kBN;  // output columns per tile
  static_assert(!SWIGLU || (!KRAGGED && ES == 2), "the fused activation exists for 16-bit row-ragged problems");
  const CanonProblem& p = fp.p;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&tail.full[s], 1);
      mbar_init(&tail.empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tail.acc_full[b], 1);
      mbar_init(&tail.acc_empty[b], kEpilogueThreads);
    }
    tail.abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(&tail.tmem_base, kTmemCols);
    tmem_relinquish();
  }
  sched_init<kBM, BNT>(p, tail.sched);  // ends with __syncthreads()
  tcgen05_fence_before_sync();
  __syncthreads();
  tcgen05_fence_after_sync();

  const uint32_t tmem_base = tail.tmem_base;
  const int total = tail.sched.total;
  const int a_batched = (p.mode == MODE_UNIFORM);
  const int b_batched = (p.mode != MODE_KRAGGED);

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (one thread)
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      const CUtensorMap* ta = &tmap_a;
      const CUtensorMap* tb = &tmap_b;
      int map_g = -1;
      for (int round = 0; ok; ++round) {
        const int t = tile_of_round<KRAGGED>(round, blockIdx.x, gridDim.x);
        if (t >= total) break;
        const TileInfo ti = decode_tile<kBM, BNT>(p, tail.sched, t);
        const int nkb = (ti.klen + BK - 1) / BK;
        const int az = a_batched ? ti.g : 0;
        const int bz = b_batched ? ti.g : 0;
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
            atomicCAS(p.status, 0, ST_PRODUCER_TIMEOUT);
            ok = false;
            break;
          }
          // A tile of at most 64 valid rows is multiplied with M = 64: only those rows are fetched.
          const bool half = !KRAGGED && !SWIGLU && fp.idesc_half != 0 && ti.rows <= 64;
          mbar_arrive_expect_tx(&tail.full[s], half ? kStageBytes - kAStageBytes / 2 : kStageBytes);
          const int k = ti.k0 + kb * BK;
          uint8_t* sa = smem_a + s * kAStageBytes;
          uint8_t* sb = smem_b + s * kBStageBytes;
          auto load_a = [&](void* dst, int x, int y) { tma_load_3d(dst, ta, &tail.full[s], x, y, az); };
          auto load_b = [&](void* dst, int x, int y) { tma_load_3d(dst, tb, &tail.full[s], x, y, bz); };
          if (!fp.a_mn) {
            if (half) tma_load_3d(sa, &fp.tmap_a_half, &tail.full[s], k, ti.m0, az);
            else load_a(sa, k, ti.m0);
          } else {
            const int chunks = (half ? 64 : kBM) / EG::CHUNK_W;
            for (int c = 0; c < chunks; ++c)
              load_a(sa + c * EG::CHUNK_BYTES, ti.m0 + c * EG::CHUNK_W, k);
          }
          if constexpr (SWIGLU) {
            // gate columns [n0, n0 + 128) and up columns [N + n0, N + n0 + 128) of B
            if (!fp.b_mn) {
              load_b(sb, k, ti.n0);  // boxes of 128 rows here
              load_b(sb + kBStageBytes / 2, k, p.N + ti.n0);
            } else {
#pragma unroll
              for (int c = 0; c < 4; ++c)
                load_b(sb + c * EG::CHUNK_BYTES, (c < 2 ? 0 : p.N - 128) + ti.n0 + c * 64, k);
            }
          } else if (!fp.b_mn) {
            load_b(sb, k, ti.n0);
          } else {
#pragma unroll
            for (int c = 0; c < kBN / EG::CHUNK_W; ++c)
              load_b(sb + c * EG::CHUNK_BYTES, ti.n0 + c * EG::CHUNK_W, k);
          }
          if (++s == kStages) { s = 0; ph ^= 1; }
        }
      }
      // After a give-up: a bounded time for the copies already requested to land before the CTA exits.
      if (!ok) drain_ring<kStages>(tail.full, s, ph);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (one thread)
    // Descriptor geometry. K-major tile: rows of 128 B, 8-row swizzle atoms 1024 B apart; one
    // k-step (16 16-bit or 8 32-bit elements) advances 32 B inside the swizzled row. MN-major
    // tile: chunks of [BK k-rows][128 B] covering 128 B of the MN dimension each; chunks are
    // CHUNK_BYTES apart (leading offset), 8-k-row atoms 1024 B apart (stride offset); a k-step
    // advances UMMA_K rows of 128 B. An MN-major 32-bit operand is swizzled in 32-byte units over
    // 4-row atoms instead (the tensor map loads it that way), so its atoms are 512 B apart.
    // In K-ragged mode the k-rows past a group's end arrive as zeros (per-group tensor maps), so
    // the last k-block of a group needs no special treatment here.
    if (lane == 0) {
      const uint32_t a_lbo = fp.a_mn ? EG::CHUNK_BYTES : 16;
      const uint32_t b_lbo = fp.b_mn ? EG::CHUNK_BYTES : 16;
      const uint32_t a_sbo = (ES == 4 && fp.a_mn) ? 512 : 1024;
      const uint32_t b_sbo = (ES == 4 && fp.b_mn) ? 512 : 1024;
      const uint32_t a_swz = (ES == 4 && fp.a_mn) ? kSwizzle128BBase32B : kSwizzle128B;
      const uint32_t b_swz = (ES == 4 && fp.b_mn) ? kSwizzle128BBase32B : kSwizzle128B;
      const uint32_t a_kstep = fp.a_mn ? (EG::UMMA_K * 128) : 32;
      const uint32_t b_kstep = fp.b_mn ? (EG::UMMA_K * 128) : 32;
      int s = 0;
      uint32_t ph = 0;
      int it = 0;
      bool ok = true;
      for (; ok; ++it) {
        const int t = tile_of_round<KRAGGED>(it, blockIdx.x, gridDim.x);
        if (t >= total) break;
        const int klen = tile_klen(p, tail.sched, t);
        const int nkb = (klen + BK - 1) / BK;
        uint32_t idesc = fp.idesc;
        if constexpr (!KRAGGED && !SWIGLU) {
          if (fp.idesc_half != 0 && decode_tile<kBM, BNT>(p, tail.sched, t).rows <= 64) idesc = fp.idesc_half;
        }
        const int buf = it & 1;
        const uint32_t aph = (it >> 1) & 1;
        if (!mbar_wait(&tail.acc_empty[buf], aph ^ 1, abort_flag)) {
          atomicCAS(p.status, 0, ST_MMA_TIMEOUT);
          break;
        }
        tcgen05_fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * kBN;
        for (int kb = 0; kb < nkb; ++kb) {
          if (!mbar_wait(&tail.full[s], ph, abort_flag)) {
            atomicCAS(p.status, 0, ST_MMA_TIMEOUT + 0x10);
            ok = false;
            break;
          }
          tcgen05_fence_after_sync();
          const uint64_t a_desc = make_smem_desc_sw128(smem_u32(smem_a + s * kAStageBytes), a_lbo, a_sbo, a_swz);
          const uint64_t b_desc = make_smem_desc_sw128(smem_u32(smem_b + s * kBStageBytes), b_lbo, b_sbo, b_swz);
#pragma unroll
          for (int k = 0; k < BK / EG::UMMA_K; ++k) {
            if constexpr (ES == 4)
              umma_tf32_ss(d_tmem, a_desc + ((k * a_kstep) >> 4), b_desc + ((k * b_kstep) >> 4), idesc,
                           (kb | k) != 0 ? 1u : 0u);
            else
              umma_f16_ss(d_tmem, a_desc + ((k * a_kstep) >> 4), b_desc + ((k * b_kstep) >> 4), idesc,
                          (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(&tail.empty[s]);  // frees the stage once these MMAs have read it
          if (++s == kStages) { s = 0; ph ^= 1; }
        }
        if (ok) umma_commit(&tail.acc_full[buf]);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;              // TMEM lane quarter this warp may read
    TOut* c_base = reinterpret_cast<TOut*>(p.c);
    int it = 0;
    bool ok = true;
    for (; ok; ++it) {
      const int t = tile_of_round<KRAGGED>(it, blockIdx.x, gridDim.x);
      if (t >= total) break;
      const TileInfo ti = decode_tile<kBM, BNT>(p, tail.sched, t);
      const int buf = it & 1;
      const uint32_t aph = (it >> 1) & 1;
      // The lanes poll on their own, so one of them may see the barrier complete just as another
      // runs out of budget; the vote makes the whole warp take the same way (tcgen05.ld below is
      // a whole-warp instruction).
      if (!__all_sync(0xffffffffu, mbar_wait(&tail.acc_full[buf], aph, abort_flag, kEpilogueBackoffNs))) {
        if (lane == 0) atomicCAS(p.status, 0, ST_EPILOGUE_TIMEOUT);
        ok = false;
        break;
      }
      tcgen05_fence_after_sync();
      const bool zero_tile = (ti.klen == 0);  // empty KRAGGED group: the block is all zeros
      TOut* c_warp = c_base + (long long)ti.g * p.c_sg + (long long)(ti.m0 + q * 32) * p.c_sm +
                     (long long)ti.n0 * p.c_sn;
      const uint32_t t_row = tmem_base + (uint32_t(q * 32) << 16) + buf * kBN;
      const int ncols_tile = min(BNT, p.N - ti.n0);
      if constexpr (SWIGLU)
        epilogue_store_warp_swiglu<TOut>(t_row, c_warp, p.c_sm, p.c_sn, ti.rows - q * 32, ncols_tile,
                                         epi_stage + (warp - 2) * kWarpStageBytes, lane);
      else if (!KRAGGED && fp.idesc_half != 0 && ti.rows <= 64) {
        // M = 64 tile: this warp's lanes 0..15 hold rows 16 q .. 16 q + 15; stored row by row
        // through the staging area, never by TMA (the other 16 lanes hold nothing).
        if (fp.c_tma) {
          if (lane == 0) tma_store_wait_read();  // an earlier TMA store may still read the staging area
          __syncwarp();
        }
        TOut* c_half = c_base + (long long)ti.g * p.c_sg + (long long)(ti.m0 + q * 16) * p.c_sm +
                       (long long)ti.n0 * p.c_sn;
        epilogue_store_warp<TOut>(t_row, c_half, p.c_sm, p.c_sn, min(16, ti.rows - q * 16), ncols_tile,
                                  epi_stage + (warp - 2) * kWarpStageBytes, false, lane);
      } else
        epilogue_store_warp<TOut>(t_row, c_warp, p.c_sm, p.c_sn, ti.rows - q * 32, ncols_tile,
                                  epi_stage + (warp - 2) * kWarpStageBytes, zero_tile, lane,
                                  fp.c_tma ? &tmap_c : nullptr, ti.n0, ti.m0 + q * 32,
                                  p.mode == MODE_MRAGGED ? 0 : ti.g);
      tcgen05_fence_before_sync();
      mbar_arrive(&tail.acc_empty[buf]);
    }
    if (fp.c_tma && lane == 0) tma_store_wait_all();  // the staging area outlives its last store
  }

  // ------------------------------------------------------------ teardown
  tcgen05_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace gmm
