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
  int panel;    // n-tiles per resident B panel (0 = default); see decode_tile
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
  int panel;                   // n-tiles per B panel
  short order[kMaxGroups];     // KRAGGED: groups by decreasing contraction length (see sched_init)
};

constexpr int kSortGroupsMax = 256;  // above this many groups the K-ragged order is left as given

constexpr int kDefaultPanel = 16;

// Builds the schedule in shared memory. Called by every thread of the block; ends with a barrier.
template <int BM, int BN>
__device__ __forceinline__ void sched_init(const CanonProblem& p, SchedSmem& s) {
  const int tid = threadIdx.x;
  const int nthr = blockDim.x;
  const int n_tiles = (p.N + BN - 1) / BN;
  if (tid == 0) s.panel = p.panel > 0 ? p.panel : kDefaultPanel;
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
    // A tile's cost is its group's contraction length, which varies widely between groups, while
    // tiles are dealt to CTAs round-robin. Dealing them in order of decreasing cost (and reversing
    // every other round, see tile_of_round) keeps the CTAs' totals within a few percent of each
    // other. Rank by counting: O(G^2 / threads), done only for moderate G.
    for (int g = tid; g < p.G; g += nthr) {
      if (p.G > kSortGroupsMax) { s.order[g] = (short)g; continue; }
      const int len = max(0, s.ends[g] - (g ? s.ends[g - 1] : 0));
      int rank = 0;
      for (int j = 0; j < p.G; ++j) {
        const int lj = max(0, s.ends[j] - (j ? s.ends[j - 1] : 0));
        rank += (lj > len) || (lj == len && j < g);
      }
      s.order[rank] = (short)g;
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

// Maps a linear tile index to its work item. Tiles are ordered group by group; inside a group the
// n-tiles are cut into panels of `panel` tiles, and for each panel all m-tiles of the group are
// swept with the n-tile as the fast index. The CTAs running at the same time therefore work on one
// B panel (panel x BN columns, which stays in L2 for the whole sweep) and on a few consecutive
// m-tiles of A, each shared by `panel` CTAs: B is read from HBM once, A once per panel.
template <int BM, int BN>
__device__ __forceinline__ TileInfo decode_tile(const CanonProblem& p, const SchedSmem& s, int t) {
  TileInfo ti;
  int g, idx, mt_g, start = 0;
  if (p.mode == MODE_MRAGGED) {
    const int key = t / s.n_tiles;  // group g holds tiles [prefix[g] * n_tiles, prefix[g+1] * n_tiles)
    int lo = 0, hi = p.G - 1;
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (s.prefix[mid] <= key) lo = mid; else hi = mid - 1;
    }
    g = lo;
    idx = t - s.prefix[g] * s.n_tiles;
    mt_g = s.prefix[g + 1] - s.prefix[g];
    start = g ? s.ends[g - 1] : 0;
  } else {
    const int per_group = s.m_tiles * s.n_tiles;
    const int gpos = t / per_group;
    idx = t - gpos * per_group;
    g = (p.mode == MODE_KRAGGED) ? (int)s.order[gpos] : gpos;
    mt_g = s.m_tiles;
  }
  const int panel_tiles = mt_g * s.panel;
  const int ns = idx / panel_tiles;
  const int rem = idx - ns * panel_tiles;
  const int width = min(s.panel, s.n_tiles - ns * s.panel);
  const int mt = rem / width;
  const int nt = ns * s.panel + (rem - mt * width);

  ti.g = g;
  ti.n0 = nt * BN;
  if (p.mode == MODE_MRAGGED) {
    ti.m0 = start + mt * BM;
    ti.rows = min(BM, s.ends[g] - ti.m0);
    ti.k0 = 0;
    ti.klen = p.K;
  } else {
    ti.m0 = mt * BM;
    ti.rows = min(BM, p.M - ti.m0);
    if (p.mode == MODE_KRAGGED) {
      const int ks = g ? s.ends[g - 1] : 0;
      const int len = s.ends[g] - ks;
      ti.k0 = ks;
      ti.klen = len > 0 ? len : 0;
    } else {
      ti.k0 = 0;
      ti.klen = p.K;
    }
  }
  return ti;
}

// Tile taken by work unit `unit` (a CTA or a CTA pair) of `units` in round `round`. With SNAKE the
// odd rounds run backwards, which evens out a cost-sorted tile sequence (K-ragged mode).
template <bool SNAKE>
__device__ __forceinline__ int tile_of_round(int round, int unit, int units) {
  if (SNAKE && (round & 1)) return round * units + (units - 1 - unit);
  return round * units + unit;
}

// Contraction length of tile `t` without the full decode: all the MMA issuer needs. It is a
// constant except in KRAGGED mode, where it is the length of the tile's group.
__device__ __forceinline__ int tile_klen(const CanonProblem& p, const SchedSmem& s, int t) {
  if (p.mode != MODE_KRAGGED) return p.K;
  const int g = s.order[t / (s.m_tiles * s.n_tiles)];
  const int len = s.ends[g] - (g ? s.ends[g - 1] : 0);
  return len > 0 ? len : 0;
}

}  // namespace gmm
