// Canonical problem description and the on-device tile scheduler shared by the tcgen05 kernel
// and the generic kernel.
//
// The four shape forms of grouped_mm (reference: grouped_mm_bf16/api.py:134-149) reduce to
// three canonical modes once the N-ragged form is transposed on the host:
//   UNIFORM  (3D x 3D)  C[g]        = A[g] * B[g]
//   MRAGGED  (2D x 3D)  C[rows_g,:] = A[rows_g,:] * B[g]        rows_g = [offs[g-1], offs[g])
//   KRAGGED  (2D x 2D)  C[g]        = A[:,ks:ke] * B[ks:ke,:]   [ks,ke) = [offs[g-1], offs[g])
//   (3D x 2D is MRAGGED on C^T = B^T * A^T.)
// `offs` holds int32 END indices (reference: grouped_mm_bf16/kernels.py:162-172); it is read
// on the device only, so no launch ever waits for the host.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace gmm {

enum Mode : int { MODE_UNIFORM = 0, MODE_MRAGGED = 1, MODE_KRAGGED = 2 };
enum DType : int { DT_BF16 = 0, DT_F16 = 1, DT_F32 = 2 };

constexpr int kMaxGroups = 1024;  // the operator rejects offs.numel() >= 1024 (api.py:115-116)

struct CanonProblem {
  int mode;
  int G;
  int M;  // rows of one output block (UNIFORM, KRAGGED) or total rows (MRAGGED)
  int N;
  int K;  // contraction length (UNIFORM, MRAGGED) or total contraction length (KRAGGED)
  const void* a;
  const void* b;
  void* c;
  const int* offs;
  // Element strides. Group strides are 0 where the operand has no group dimension.
  long long a_sg, a_sm, a_sk;
  long long b_sg, b_sk, b_sn;
  long long c_sg, c_sm, c_sn;
  int in_dtype;
  int out_dtype;
  int* status;  // device word; stays 0 unless a bounded wait gave up
};

// One unit of work: an output tile of one group.
struct TileInfo {
  int g;     // group
  int m0;    // first row (global row for MRAGGED, row inside the group otherwise)
  int rows;  // valid rows in the tile
  int n0;    // first column
  int k0;    // first contraction index
  int klen;  // contraction length (0 for an empty KRAGGED group: the tile is stored as zeros)
};

struct SchedSmem {
  int ends[kMaxGroups];        // group end indices, clamped into [0, extent]
  int prefix[kMaxGroups + 1];  // MRAGGED: prefix[g] = number of m-tiles before group g
  int mt_total;                // number of (group, m-tile) pairs
  int m_tiles;                 // m-tiles per group (UNIFORM, KRAGGED)
  int n_tiles;
  int total;                   // total tiles
};

constexpr int kBand = 8;  // m-tiles that share one sweep over the n-tiles (L2 reuse of A and B panels)

// Builds the schedule in shared memory. Called by every thread of the block; ends with a barrier.
template <int BM, int BN>
__device__ __forceinline__ void sched_init(const CanonProblem& p, SchedSmem& s) {
  const int tid = threadIdx.x;
  const int nthr = blockDim.x;
  const int n_tiles = (p.N + BN - 1) / BN;
  if (p.mode == MODE_UNIFORM) {
    if (tid == 0) {
      s.m_tiles = (p.M + BM - 1) / BM;
      s.n_tiles = n_tiles;
      s.mt_total = s.m_tiles * p.G;
      s.total = s.mt_total * n_tiles;
    }
    __syncthreads();
    return;
  }
  const int extent = (p.mode == MODE_MRAGGED) ? p.M : p.K;
  for (int g = tid; g < p.G; g += nthr) {
    int e = p.offs[g];
    e = e < 0 ? 0 : (e > extent ? extent : e);
    s.ends[g] = e;
  }
  __syncthreads();
  if (p.mode == MODE_KRAGGED) {
    if (tid == 0) {
      s.m_tiles = (p.M + BM - 1) / BM;
      s.n_tiles = n_tiles;
      s.mt_total = s.m_tiles * p.G;
      s.total = s.mt_total * n_tiles;
    }
    __syncthreads();
    return;
  }
  // MRAGGED: per-group m-tile counts, then an exclusive prefix sum.
  for (int g = tid; g < p.G; g += nthr) {
    const int start = g ? s.ends[g - 1] : 0;
    const int sz = s.ends[g] - start;
    s.prefix[g + 1] = sz > 0 ? (sz + BM - 1) / BM : 0;
  }
  if (tid == 0) s.prefix[0] = 0;
  __syncthreads();
  if (tid < 32) {
    const int chunk = (p.G + 31) / 32;
    const int lo = tid * chunk;
    const int hi = min(lo + chunk, p.G);
    int sum = 0;
    for (int g = lo; g < hi; ++g) sum += s.prefix[g + 1];
    int incl = sum;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, d);
      if (tid >= d) incl += v;
    }
    int run = incl - sum;
    for (int g = lo; g < hi; ++g) {
      run += s.prefix[g + 1];
      s.prefix[g + 1] = run;
    }
    const int all = __shfl_sync(0xffffffffu, incl, 31);
    if (tid == 0) {
      s.m_tiles = 0;
      s.n_tiles = n_tiles;
      s.mt_total = all;
      s.total = all * n_tiles;
    }
  }
  __syncthreads();
}

// Maps a linear tile index to its work item. Tiles are ordered in bands of kBand m-tiles; inside
// a band the n-tile is the slow index, so the CTAs running at the same time share A and B panels.
template <int BM, int BN>
__device__ __forceinline__ TileInfo decode_tile(const CanonProblem& p, const SchedSmem& s, int t) {
  const int band_tiles = kBand * s.n_tiles;
  const int band = t / band_tiles;
  const int w = t - band * band_tiles;
  const int band_m0 = band * kBand;
  const int bsz = min(kBand, s.mt_total - band_m0);
  const int nt = w / bsz;
  const int mtg = band_m0 + (w - nt * bsz);

  TileInfo ti;
  ti.n0 = nt * BN;
  if (p.mode == MODE_MRAGGED) {
    int lo = 0, hi = p.G - 1;
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (s.prefix[mid] <= mtg) lo = mid; else hi = mid - 1;
    }
    const int start = lo ? s.ends[lo - 1] : 0;
    ti.g = lo;
    ti.m0 = start + (mtg - s.prefix[lo]) * BM;
    ti.rows = min(BM, s.ends[lo] - ti.m0);
    ti.k0 = 0;
    ti.klen = p.K;
  } else {
    const int g = mtg / s.m_tiles;
    const int mt = mtg - g * s.m_tiles;
    ti.g = g;
    ti.m0 = mt * BM;
    ti.rows = min(BM, p.M - ti.m0);
    if (p.mode == MODE_KRAGGED) {
      const int start = g ? s.ends[g - 1] : 0;
      const int len = s.ends[g] - start;
      ti.k0 = start;
      ti.klen = len > 0 ? len : 0;
    } else {
      ti.k0 = 0;
      ti.klen = p.K;
    }
  }
  return ti;
}

}  // namespace gmm
