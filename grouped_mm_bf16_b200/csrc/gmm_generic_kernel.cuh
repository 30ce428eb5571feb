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

constexpr int kGBM = 64;
constexpr int kGBN = 64;
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

template <typename TIn, typename TOut>
__global__ void __launch_bounds__(kGenericThreads) gmm_generic_kernel(const CanonProblem p) {
  __shared__ SchedSmem sched;
  __shared__ float As[kGBK][kGBM + 4];
  __shared__ float Bs[kGBK][kGBN + 4];

  sched_init<kGBM, kGBN>(p, sched);
  const int total = sched.total;
  const int tid = threadIdx.x;
  const int tx = tid & 15;  // 4 output columns each
  const int ty = tid >> 4;  // 4 output rows each

  const TIn* a_all = reinterpret_cast<const TIn*>(p.a);
  const TIn* b_all = reinterpret_cast<const TIn*>(p.b);
  TOut* c_all = reinterpret_cast<TOut*>(p.c);

  for (int t = blockIdx.x; t < total; t += gridDim.x) {
    const TileInfo ti = decode_tile<kGBM, kGBN>(p, sched, t);
    const TIn* a_g = a_all + (long long)ti.g * p.a_sg;
    const TIn* b_g = b_all + (long long)ti.g * p.b_sg;
    const int ncols = min(kGBN, p.N - ti.n0);

    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int kk = 0; kk < ti.klen; kk += kGBK) {
      // A tile: kGBM x kGBK, B tile: kGBK x kGBN; 1024 elements each, 4 per thread.
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int idx = tid + e * kGenericThreads;
        {
          // Walk the unit-stride dimension fastest for whichever layout A has.
          int m, k;
          if (p.a_sk == 1) { k = idx % kGBK; m = idx / kGBK; } else { m = idx % kGBM; k = idx / kGBM; }
          float v = 0.f;
          if (m < ti.rows && kk + k < ti.klen)
            v = to_f32<TIn>(a_g[(long long)(ti.m0 + m) * p.a_sm + (long long)(ti.k0 + kk + k) * p.a_sk]);
          As[k][m] = v;
        }
        {
          int n, k;
          if (p.b_sn == 1) { n = idx % kGBN; k = idx / kGBN; } else { k = idx % kGBK; n = idx / kGBK; }
          float v = 0.f;
          if (n < ncols && kk + k < ti.klen)
            v = to_f32<TIn>(b_g[(long long)(ti.k0 + kk + k) * p.b_sk + (long long)(ti.n0 + n) * p.b_sn]);
          Bs[k][n] = v;
        }
      }
      __syncthreads();
#pragma unroll
      for (int k = 0; k < kGBK; ++k) {
        float av[4], bv[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) av[i] = As[k][ty * 4 + i];
#pragma unroll
        for (int j = 0; j < 4; ++j) bv[j] = Bs[k][tx * 4 + j];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
      }
      __syncthreads();
    }

    TOut* c_g = c_all + (long long)ti.g * p.c_sg;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int m = ty * 4 + i;
      if (m >= ti.rows) continue;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int n = tx * 4 + j;
        if (n < ncols)
          c_g[(long long)(ti.m0 + m) * p.c_sm + (long long)(ti.n0 + n) * p.c_sn] = from_f32<TOut>(acc[i][j]);
      }
    }
  }
}

}  // namespace gmm
