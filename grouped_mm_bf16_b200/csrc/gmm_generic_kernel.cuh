// Generic grouped GEMM kernel: any element strides, any alignment, bf16 / fp16 / fp32 inputs,
// fp32 FMA accumulation (true fp32 for fp32 inputs, as the reference's fp32 tests assume:
// tests/test_grouped_mm.py:680,711,741 against kernels.py:185-194 with TF32 off).
//
// It serves the shapes the TMA path cannot take: leading strides or base addresses that are not
// 16-byte aligned (odd K or N, which the reference accepts: tests/test_grouped_mm.py:378,421),
// fp32 inputs, and ragged dimensions that are contiguous in memory (where a group boundary can
// fall on any element, so a TMA box cannot start there). Same scheduler, same masking rules and
// the same single rounding at the store as the tcgen05 kernel.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "gmm_common.cuh"

namespace gmm {

constexpr int kGBM = 64;    // small tile: few or short groups
constexpr int kGBN = 64;
constexpr int kGBML = 128;  // large tile: enough tiles of this size to fill the GPU
constexpr int kGBNL = 128;
constexpr int kGBK = 16;
constexpr int kGenericThreads = 256;

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <>
__device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }

template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <>
__device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }

// BM x BN output tile per block, 16 x 16 threads, (BM/16) x (BN/16) outputs per thread held as
// 4 x 4 blocks spaced 64 apart (so that the shared-memory reads of a warp are conflict-free
// float4 loads). The k-slab after the current one is fetched into registers while the current one
// is multiplied, and parked in the second shared-memory buffer: one barrier per slab.
template <typename TIn, typename TOut, int BM, int BN>
__global__ void __launch_bounds__(kGenericThreads) gmm_generic_kernel(const CanonProblem p) {
  static_assert(BM % 64 == 0 && BN % 64 == 0, "tiles are made of 64 x 64 quadrants");
  constexpr int QM = BM / 64, QN = BN / 64;          // quadrants per tile
  constexpr int EA = BM * kGBK / kGenericThreads;    // A elements a thread fetches per slab
  constexpr int EB = BN * kGBK / kGenericThreads;
  __shared__ SchedSmem sched;
  __shared__ __align__(16) float As[2][kGBK][BM + 4];  // two slabs: one multiplied while the next is filled
  __shared__ __align__(16) float Bs[2][kGBK][BN + 4];

  sched_init<BM, BN>(p, sched);
  const int total = sched.total;
  const int tid = threadIdx.x;
  const int tx = tid & 15;  // columns tx*4 .. tx*4+3 of every quadrant
  const int ty = tid >> 4;  // rows    ty*4 .. ty*4+3 of every quadrant

  const TIn* a_all = reinterpret_cast<const TIn*>(p.a);
  const TIn* b_all = reinterpret_cast<const TIn*>(p.b);
  TOut* c_all = reinterpret_cast<TOut*>(p.c);

  // Which element of a slab this thread fetches: walk the unit-stride dimension fastest for
  // whichever layout the operand has.
  int am[EA], ak[EA], bn[EB], bk[EB];
#pragma unroll
  for (int e = 0; e < EA; ++e) {
    const int idx = tid + e * kGenericThreads;
    if (p.a_sk == 1) { ak[e] = idx % kGBK; am[e] = idx / kGBK; } else { am[e] = idx % BM; ak[e] = idx / BM; }
  }
#pragma unroll
  for (int e = 0; e < EB; ++e) {
    const int idx = tid + e * kGenericThreads;
    if (p.b_sn == 1) { bn[e] = idx % BN; bk[e] = idx / BN; } else { bk[e] = idx % kGBK; bn[e] = idx / kGBK; }
  }

  for (int t = blockIdx.x; t < total; t += gridDim.x) {
    const TileInfo ti = decode_tile<BM, BN>(p, sched, t);
    const int ncols = min(BN, p.N - ti.n0);
    // Element (row m, contraction index 0) of A and (0, column n) of B for this thread's fetches.
    const TIn* a_src[EA];
    const TIn* b_src[EB];
#pragma unroll
    for (int e = 0; e < EA; ++e)
      a_src[e] = a_all + (long long)ti.g * p.a_sg + (long long)(ti.m0 + am[e]) * p.a_sm +
                 (long long)(ti.k0 + ak[e]) * p.a_sk;
#pragma unroll
    for (int e = 0; e < EB; ++e)
      b_src[e] = b_all + (long long)ti.g * p.b_sg + (long long)(ti.k0 + bk[e]) * p.b_sk +
                 (long long)(ti.n0 + bn[e]) * p.b_sn;

    float acc[QM][QN][4][4];
#pragma unroll
    for (int qm = 0; qm < QM; ++qm)
#pragma unroll
      for (int qn = 0; qn < QN; ++qn)
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[qm][qn][i][j] = 0.f;

    float a_reg[EA], b_reg[EB];
    auto fetch = [&](int kk) {
#pragma unroll
      for (int e = 0; e < EA; ++e) {
        const bool ok = am[e] < ti.rows && kk + ak[e] < ti.klen;
        a_reg[e] = ok ? to_f32<TIn>(a_src[e][(long long)kk * p.a_sk]) : 0.f;
      }
#pragma unroll
      for (int e = 0; e < EB; ++e) {
        const bool ok = bn[e] < ncols && kk + bk[e] < ti.klen;
        b_reg[e] = ok ? to_f32<TIn>(b_src[e][(long long)kk * p.b_sk]) : 0.f;
      }
    };

    auto stash = [&](int buf) {
#pragma unroll
      for (int e = 0; e < EA; ++e) As[buf][ak[e]][am[e]] = a_reg[e];
#pragma unroll
      for (int e = 0; e < EB; ++e) Bs[buf][bk[e]][bn[e]] = b_reg[e];
    };
    int cur = 0;
    if (ti.klen > 0) {
      fetch(0);
      stash(0);
    }
    __syncthreads();
    for (int kk = 0; kk < ti.klen; kk += kGBK) {
      const bool more = kk + kGBK < ti.klen;
      if (more) fetch(kk + kGBK);  // in flight during the multiply below
#pragma unroll
      for (int k = 0; k < kGBK; ++k) {
        float4 av[QM], bv[QN];
#pragma unroll
        for (int qm = 0; qm < QM; ++qm) av[qm] = *reinterpret_cast<const float4*>(&As[cur][k][qm * 64 + ty * 4]);
#pragma unroll
        for (int qn = 0; qn < QN; ++qn) bv[qn] = *reinterpret_cast<const float4*>(&Bs[cur][k][qn * 64 + tx * 4]);
#pragma unroll
        for (int qm = 0; qm < QM; ++qm) {
          const float a4[4] = {av[qm].x, av[qm].y, av[qm].z, av[qm].w};
#pragma unroll
          for (int qn = 0; qn < QN; ++qn) {
            const float b4[4] = {bv[qn].x, bv[qn].y, bv[qn].z, bv[qn].w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
              for (int j = 0; j < 4; ++j) acc[qm][qn][i][j] = fmaf(a4[i], b4[j], acc[qm][qn][i][j]);
          }
        }
      }
      if (more) stash(cur ^ 1);  // the other slab: nobody reads it during this iteration
      __syncthreads();
      cur ^= 1;
    }

    TOut* c_g = c_all + (long long)ti.g * p.c_sg;
#pragma unroll
    for (int qm = 0; qm < QM; ++qm)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int m = qm * 64 + ty * 4 + i;
        if (m >= ti.rows) continue;
#pragma unroll
        for (int qn = 0; qn < QN; ++qn)
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int n = qn * 64 + tx * 4 + j;
            if (n < ncols)
              c_g[(long long)(ti.m0 + m) * p.c_sm + (long long)(ti.n0 + n) * p.c_sn] =
                  from_f32<TOut>(acc[qm][qn][i][j]);
          }
      }
  }
}

}  // namespace gmm
