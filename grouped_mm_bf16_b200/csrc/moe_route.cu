// Caller-side MoE steps next to the grouped GEMM: turning per-token expert choices into the
// group-contiguous row order and the int32 END offsets that grouped_mm's 2D x 3D form consumes,
// gathering token rows into that order, and the weighted scatter back. Declared in
// include/grouped_mm_b200.h.
//
// The reference only shows the first half of this on the host, in its benchmark: expert ids ->
// torch.bincount -> cumsum -> int32 offs (bench/bench_2d3d.py:131-138); the rows it multiplies are
// random, so it never needs the permutation. Here all of it runs on the device, without a host
// sync, as byte/index work bounded by HBM bandwidth:
//
//   route_build   stable counting sort of the assignments by expert, in three launches:
//                 (1) one histogram per 1024-assignment chunk (one warp each),
//                 (2) per-expert prefix over the chunks + cumulative sum over the experts,
//                 (3) each warp replays its chunk in order and hands out positions.
//   permute_rows  dst[r] = src[perm[r] / topk]                      (16-byte vector copies)
//   combine_rows  out[t] = sum_k w[t,k] * y[inv_perm[t*topk + k]]   (fp32 accumulation)
//
// Stable means: inside a group, rows keep the order of their assignment index, so the result is
// the same on every run and equals a stable argsort on the host (the oracle).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "../../include/grouped_mm_b200.h"

namespace {

constexpr int kChunk = 1024;         // assignments per warp
constexpr int kWarpsPerBlock = 4;
constexpr int kMaxExperts = 1023;    // same limit as the operator (offs.numel() < 1024)

__device__ __forceinline__ int load_id(const int32_t* ids, long long i, long long n, int n_experts) {
  if (i >= n) return -1;
  const int e = ids[i];
  return (e >= 0 && e < n_experts) ? e : -1;  // out-of-range ids are not routed anywhere
}

// (1) chunk_hist[chunk][e] = number of assignments of chunk `chunk` that go to expert e.
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
route_count_kernel(const int32_t* ids, long long n, int n_experts, int* chunk_hist, long long n_chunks) {
  extern __shared__ int smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int* hist = smem + warp * n_experts;
  const long long chunk = (long long)blockIdx.x * kWarpsPerBlock + warp;
  if (chunk >= n_chunks) return;
  for (int e = lane; e < n_experts; e += 32) hist[e] = 0;
  __syncwarp();
  const long long base = chunk * kChunk;
  for (int s = 0; s < kChunk; s += 32) {
    const int e = load_id(ids, base + s + lane, n, n_experts);
    if (e >= 0) atomicAdd(&hist[e], 1);
  }
  __syncwarp();
  int* out = chunk_hist + chunk * n_experts;
  for (int e = lane; e < n_experts; e += 32) out[e] = hist[e];
}

// (2) One block. chunk_hist becomes, in place, the first sorted position of (chunk, expert);
//     offs[e] receives the END offset of expert e.
__global__ void __launch_bounds__(1024)
route_scan_kernel(int* chunk_hist, long long n_chunks, int n_experts, int32_t* offs) {
  __shared__ int warp_sums[32];
  const int e = threadIdx.x;
  int total = 0;
  if (e < n_experts) {
    for (long long c = 0; c < n_chunks; ++c) {  // exclusive prefix over the chunks of this expert
      int* cell = chunk_hist + c * n_experts + e;
      const int v = *cell;
      *cell = total;
      total += v;
    }
  }
  // inclusive scan of the per-expert totals over the experts
  int incl = total;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int v = __shfl_up_sync(0xffffffffu, incl, d);
    if (lane >= d) incl += v;
  }
  if (lane == 31) warp_sums[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    int w = warp_sums[lane];
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, w, d);
      if (lane >= d) w += v;
    }
    warp_sums[lane] = w;
  }
  __syncthreads();
  incl += warp ? warp_sums[warp - 1] : 0;
  if (e < n_experts) {
    offs[e] = incl;
    const int start = incl - total;  // first sorted position of expert e
    for (long long c = 0; c < n_chunks; ++c) chunk_hist[c * n_experts + e] += start;
  }
}

// (3) perm[pos] = assignment index, inv_perm[assignment] = pos (or -1 if not routed).
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
route_scatter_kernel(const int32_t* ids, long long n, int n_experts, const int* chunk_base, long long n_chunks,
                     int32_t* perm, int32_t* inv_perm) {
  extern __shared__ int smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int* cursor = smem + warp * n_experts;
  const long long chunk = (long long)blockIdx.x * kWarpsPerBlock + warp;
  if (chunk >= n_chunks) return;
  const int* base_row = chunk_base + chunk * n_experts;
  for (int e = lane; e < n_experts; e += 32) cursor[e] = base_row[e];
  __syncwarp();
  const long long base = chunk * kChunk;
  const unsigned lt = (1u << lane) - 1u;
  for (int s = 0; s < kChunk; s += 32) {
    const long long i = base + s + lane;
    const int e = load_id(ids, i, n, n_experts);
    // lanes with the same expert, in lane (= assignment) order
    const unsigned same = __match_any_sync(0xffffffffu, e);
    int pos = -1;
    if (e >= 0) pos = cursor[e] + __popc(same & lt);
    __syncwarp();
    if (e >= 0 && (same & lt) == 0) cursor[e] += __popc(same);  // first lane of each expert advances it
    __syncwarp();
    if (i < n) {
      if (pos >= 0) perm[pos] = (int32_t)i;
      if (inv_perm) inv_perm[i] = pos;
    }
  }
}

// dst row r = src row perm[r] / topk. One block per output row.
template <typename V>
__global__ void __launch_bounds__(128)
permute_rows_kernel(const unsigned char* src, long long src_stride, const int32_t* perm, int topk,
                    unsigned char* dst, long long dst_stride, long long n_rows, long long src_rows, int n_vec) {
  const long long r = blockIdx.x;
  if (r >= n_rows) return;
  const long long a = perm[r];
  const long long t = a / topk;
  if (a < 0 || t >= src_rows) return;
  const V* s = reinterpret_cast<const V*>(src + t * src_stride);
  V* d = reinterpret_cast<V*>(dst + r * dst_stride);
  // four loads in flight per thread before the first store
  int i = threadIdx.x;
  for (; i + 3 * (int)blockDim.x < n_vec; i += 4 * blockDim.x) {
    const V v0 = s[i], v1 = s[i + blockDim.x], v2 = s[i + 2 * blockDim.x], v3 = s[i + 3 * blockDim.x];
    d[i] = v0;
    d[i + blockDim.x] = v1;
    d[i + 2 * blockDim.x] = v2;
    d[i + 3 * blockDim.x] = v3;
  }
  for (; i < n_vec; i += blockDim.x) d[i] = s[i];
}

template <typename T>
__device__ __forceinline__ float cvt_in(T v);
template <>
__device__ __forceinline__ float cvt_in<float>(float v) { return v; }
template <>
__device__ __forceinline__ float cvt_in<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <>
__device__ __forceinline__ float cvt_in<__half>(__half v) { return __half2float(v); }
template <typename T>
__device__ __forceinline__ T cvt_out(float v);
template <>
__device__ __forceinline__ float cvt_out<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 cvt_out<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <>
__device__ __forceinline__ __half cvt_out<__half>(float v) { return __float2half_rn(v); }

// out[t, c] = sum_k w[t, k] * y[inv_perm[t * topk + k], c]. One block per token.
template <typename TIn, typename TOut>
__global__ void __launch_bounds__(256)
combine_rows_kernel(const TIn* y, long long y_stride, const int32_t* inv_perm, const float* weights, int topk,
                    long long n_tokens, int n_cols, TOut* out, long long out_stride) {
  const long long t = blockIdx.x;
  if (t >= n_tokens) return;
  for (int c = threadIdx.x; c < n_cols; c += blockDim.x) {
    float acc = 0.f;
    for (int k = 0; k < topk; ++k) {
      const int pos = inv_perm[t * topk + k];
      if (pos < 0) continue;
      const float w = weights ? weights[t * topk + k] : 1.f;
      acc = fmaf(w, cvt_in<TIn>(y[(long long)pos * y_stride + c]), acc);
    }
    out[t * out_stride + c] = cvt_out<TOut>(acc);
  }
}

// Same sum for 16-bit inputs whose rows are 16-byte aligned: 8 columns per thread, 16-byte loads.
template <typename TIn, typename TOut>
__global__ void __launch_bounds__(256)
combine_rows_vec8_kernel(const TIn* y, long long y_stride, const int32_t* inv_perm, const float* weights, int topk,
                         long long n_tokens, int n_cols, TOut* out, long long out_stride) {
  const long long t = blockIdx.x;
  if (t >= n_tokens) return;
  for (int c = threadIdx.x * 8; c < n_cols; c += blockDim.x * 8) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int k = 0; k < topk; ++k) {
      const int pos = inv_perm[t * topk + k];
      if (pos < 0) continue;
      const float w = weights ? weights[t * topk + k] : 1.f;
      const uint4 raw = *reinterpret_cast<const uint4*>(y + (long long)pos * y_stride + c);
      const TIn* v = reinterpret_cast<const TIn*>(&raw);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = fmaf(w, cvt_in<TIn>(v[j]), acc[j]);
    }
    TOut* dst = out + t * out_stride + c;
    if constexpr (sizeof(TOut) == 2) {
      uint4 packed;
      TOut* pv = reinterpret_cast<TOut*>(&packed);
#pragma unroll
      for (int j = 0; j < 8; ++j) pv[j] = cvt_out<TOut>(acc[j]);
      *reinterpret_cast<uint4*>(dst) = packed;
    } else {
      *reinterpret_cast<float4*>(dst) = make_float4(acc[0], acc[1], acc[2], acc[3]);
      *reinterpret_cast<float4*>(dst + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
    }
  }
}

size_t route_ws_bytes(long long n_assign, int n_experts) {
  const long long n_chunks = (n_assign + kChunk - 1) / kChunk;
  return (size_t)(n_chunks > 0 ? n_chunks : 1) * (size_t)n_experts * sizeof(int);
}

template <typename TIn>
int launch_combine(const void* y, long long y_stride, const int32_t* inv_perm, const float* weights, int topk,
                   long long n_tokens, int n_cols, void* out, int out_dtype, long long out_stride, cudaStream_t st) {
  const unsigned grid = (unsigned)n_tokens;
  const TIn* yy = reinterpret_cast<const TIn*>(y);
  if constexpr (sizeof(TIn) == 2) {
    const size_t out_es = out_dtype == GMM_F32 ? 4 : 2;
    const bool vec = (n_cols % 8 == 0) && (y_stride % 8 == 0) && ((out_stride * out_es) % 16 == 0) &&
                     ((reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(out)) & 15u) == 0;
    if (vec) {
      switch (out_dtype) {
        case GMM_BF16:
          combine_rows_vec8_kernel<TIn, __nv_bfloat16><<<grid, 256, 0, st>>>(
              yy, y_stride, inv_perm, weights, topk, n_tokens, n_cols, reinterpret_cast<__nv_bfloat16*>(out), out_stride);
          break;
        case GMM_F16:
          combine_rows_vec8_kernel<TIn, __half><<<grid, 256, 0, st>>>(
              yy, y_stride, inv_perm, weights, topk, n_tokens, n_cols, reinterpret_cast<__half*>(out), out_stride);
          break;
        default:
          combine_rows_vec8_kernel<TIn, float><<<grid, 256, 0, st>>>(
              yy, y_stride, inv_perm, weights, topk, n_tokens, n_cols, reinterpret_cast<float*>(out), out_stride);
          break;
      }
      return cudaGetLastError() == cudaSuccess ? GMM_OK : GMM_ERR_CUDA;
    }
  }
  switch (out_dtype) {
    case GMM_BF16:
      combine_rows_kernel<TIn, __nv_bfloat16><<<grid, 256, 0, st>>>(yy, y_stride, inv_perm, weights, topk, n_tokens,
                                                                  n_cols, reinterpret_cast<__nv_bfloat16*>(out), out_stride);
      break;
    case GMM_F16:
      combine_rows_kernel<TIn, __half><<<grid, 256, 0, st>>>(yy, y_stride, inv_perm, weights, topk, n_tokens, n_cols,
                                                           reinterpret_cast<__half*>(out), out_stride);
      break;
    default:
      combine_rows_kernel<TIn, float><<<grid, 256, 0, st>>>(yy, y_stride, inv_perm, weights, topk, n_tokens, n_cols,
                                                          reinterpret_cast<float*>(out), out_stride);
      break;
  }
  return cudaGetLastError() == cudaSuccess ? GMM_OK : GMM_ERR_CUDA;
}

}  // namespace

extern "C" {

size_t gmm_route_workspace_bytes(int64_t n_assignments, int32_t n_experts) {
  if (n_assignments < 0 || n_experts <= 0 || n_experts > kMaxExperts) return 0;
  return route_ws_bytes(n_assignments, n_experts);
}

int gmm_route_build(const int32_t* expert_ids, int64_t n_assignments, int32_t n_experts, int32_t* offs,
                    int32_t* perm, int32_t* inv_perm, void* workspace, size_t workspace_bytes, void* stream) {
  if (n_assignments < 0 || n_assignments > 0x7fffffffLL || !offs) return GMM_ERR_INVALID_ARGUMENT;
  if (n_experts <= 0) return GMM_ERR_INVALID_ARGUMENT;
  if (n_experts > kMaxExperts) return GMM_ERR_TOO_MANY_GROUPS;
  if (n_assignments > 0 && (!expert_ids || !perm)) return GMM_ERR_INVALID_ARGUMENT;
  if (!workspace || workspace_bytes < route_ws_bytes(n_assignments, n_experts)) return GMM_ERR_WORKSPACE;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const long long n_chunks = n_assignments > 0 ? (n_assignments + kChunk - 1) / kChunk : 1;
  int* hist = reinterpret_cast<int*>(workspace);
  const unsigned blocks = (unsigned)((n_chunks + kWarpsPerBlock - 1) / kWarpsPerBlock);
  const size_t smem = (size_t)kWarpsPerBlock * n_experts * sizeof(int);
  route_count_kernel<<<blocks, kWarpsPerBlock * 32, smem, st>>>(expert_ids, n_assignments, n_experts, hist, n_chunks);
  route_scan_kernel<<<1, 1024, 0, st>>>(hist, n_chunks, n_experts, offs);
  if (n_assignments > 0) {
    // Positions past the last routed assignment (ids outside [0, n_experts) are not routed) stay -1.
    if (cudaMemsetAsync(perm, 0xFF, (size_t)n_assignments * sizeof(int32_t), st) != cudaSuccess) return GMM_ERR_CUDA;
    route_scatter_kernel<<<blocks, kWarpsPerBlock * 32, smem, st>>>(expert_ids, n_assignments, n_experts, hist,
                                                                   n_chunks, perm, inv_perm);
  }
  return cudaGetLastError() == cudaSuccess ? GMM_OK : GMM_ERR_CUDA;
}

int gmm_permute_rows(const void* src, int64_t src_rows, int64_t row_bytes, int64_t src_stride_bytes,
                     const int32_t* perm, int32_t topk, void* dst, int64_t dst_stride_bytes, int64_t n_out_rows,
                     void* stream) {
  if (n_out_rows < 0 || row_bytes < 0 || topk <= 0 || src_rows < 0) return GMM_ERR_INVALID_ARGUMENT;
  if (n_out_rows == 0 || row_bytes == 0) return GMM_OK;
  if (!src || !dst || !perm || n_out_rows > 0x7fffffffLL) return GMM_ERR_INVALID_ARGUMENT;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const unsigned char* s = reinterpret_cast<const unsigned char*>(src);
  unsigned char* d = reinterpret_cast<unsigned char*>(dst);
  const bool vec16 = ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst) | (uintptr_t)row_bytes |
                       (uintptr_t)src_stride_bytes | (uintptr_t)dst_stride_bytes) & 15u) == 0;
  if (vec16) {
    permute_rows_kernel<uint4><<<(unsigned)n_out_rows, 128, 0, st>>>(s, src_stride_bytes, perm, topk, d,
                                                                    dst_stride_bytes, n_out_rows, src_rows,
                                                                    (int)(row_bytes / 16));
  } else if (((row_bytes | src_stride_bytes | dst_stride_bytes) & 1) == 0 &&
             ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 1u) == 0) {
    permute_rows_kernel<unsigned short><<<(unsigned)n_out_rows, 128, 0, st>>>(s, src_stride_bytes, perm, topk, d,
                                                                             dst_stride_bytes, n_out_rows, src_rows,
                                                                             (int)(row_bytes / 2));
  } else {
    permute_rows_kernel<unsigned char><<<(unsigned)n_out_rows, 128, 0, st>>>(s, src_stride_bytes, perm, topk, d,
                                                                            dst_stride_bytes, n_out_rows, src_rows,
                                                                            (int)row_bytes);
  }
  return cudaGetLastError() == cudaSuccess ? GMM_OK : GMM_ERR_CUDA;
}

int gmm_combine_rows(const void* y, int32_t y_dtype, int64_t y_stride, const int32_t* inv_perm, const float* weights,
                     int32_t topk, int64_t n_tokens, int32_t n_cols, void* out, int32_t out_dtype, int64_t out_stride,
                     void* stream) {
  if (n_tokens < 0 || n_cols < 0 || topk <= 0 || n_tokens > 0x7fffffffLL) return GMM_ERR_INVALID_ARGUMENT;
  if (y_dtype < GMM_BF16 || y_dtype > GMM_F32 || out_dtype < GMM_BF16 || out_dtype > GMM_F32)
    return GMM_ERR_UNSUPPORTED_DTYPE;
  if (n_tokens == 0 || n_cols == 0) return GMM_OK;
  if (!y || !inv_perm || !out) return GMM_ERR_INVALID_ARGUMENT;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  switch (y_dtype) {
    case GMM_BF16:
      return launch_combine<__nv_bfloat16>(y, y_stride, inv_perm, weights, topk, n_tokens, n_cols, out, out_dtype,
                                           out_stride, st);
    case GMM_F16:
      return launch_combine<__half>(y, y_stride, inv_perm, weights, topk, n_tokens, n_cols, out, out_dtype,
                                    out_stride, st);
    default:
      return launch_combine<float>(y, y_stride, inv_perm, weights, topk, n_tokens, n_cols, out, out_dtype, out_stride,
                                   st);
  }
}

}  // extern "C"
