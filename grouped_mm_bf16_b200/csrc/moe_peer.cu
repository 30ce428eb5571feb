// Expert-parallel dispatch and combine over peer memory (NVLink): the two row movements of a
// routed feed-forward block whose experts live on several GPUs, done with plain stores to and loads
// from the peers' buffers instead of a pack -> all-to-all -> unpack sequence. Declared in
// include/grouped_mm_b200.h. The reference has no multi-GPU code; nothing here has a counterpart.
//
//   scatter_rows_to_peers     dst = peer[dst_rank[r]] + dst_row[r]:  dst[:] = src[perm[r] / topk][:]
//                             every routed row goes straight to its final, expert-grouped position in
//                             the buffer of the GPU that owns its expert (16-byte stores over NVLink)
//   combine_rows_from_peers   out[t] = sum_k w[t,k] * peer[src_rank[a]][src_row[a]],  a = t*topk + k
//                             every token pulls its topk result rows from the GPUs that produced them
//
// `peers` is a device array of base pointers, one per rank, this rank's own buffer included (the
// mapping comes from the caller: CUDA IPC, cuMem fabric handles, torch symmetric memory ...).
// Rank and row come from index tables the caller computes on the device, so neither kernel waits
// for the host. Neither kernel waits for another GPU either: the caller orders "all rows written"
// before "rows read" with a collective on the stream. Every index is checked against the number of
// peers and the buffer's capacity; a row that fails the check is skipped and GMM_STATUS_BAD_PEER_INDEX
// is set in *status, so a wrong table cannot turn into a stray write to another GPU's memory.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "../../include/grouped_mm_b200.h"

namespace {

template <typename V>
__global__ void __launch_bounds__(128)
scatter_rows_to_peers_kernel(const unsigned char* src, long long src_rows, long long src_stride, const int32_t* perm,
                             int topk, const int32_t* dst_rank, const int32_t* dst_row, unsigned char* const* peers,
                             int n_peers, long long dst_stride, long long capacity_rows, long long n_rows, int n_vec,
                             int* status) {
  const long long r = blockIdx.x;
  if (r >= n_rows) return;
  const long long a = perm[r];
  const int rank = dst_rank[r];
  if (a < 0 || rank < 0) return;  // an assignment that is routed nowhere
  const long long t = a / topk;
  const long long row = dst_row[r];
  if (t >= src_rows || rank >= n_peers || row < 0 || row >= capacity_rows) {
    if (threadIdx.x == 0) atomicOr(status, GMM_STATUS_BAD_PEER_INDEX);
    return;
  }
  const V* s = reinterpret_cast<const V*>(src + t * src_stride);
  V* d = reinterpret_cast<V*>(peers[rank] + row * dst_stride);
  int i = threadIdx.x;  // four loads in flight per thread before the first store
  for (; i + 3 * (int)blockDim.x < n_vec; i += 4 * blockDim.x) {
    const V v0 = s[i], v1 = s[i + blockDim.x], v2 = s[i + 2 * blockDim.x], v3 = s[i + 3 * blockDim.x];
    d[i] = v0;
    d[i + blockDim.x] = v1;
    d[i + 2 * blockDim.x] = v2;
    d[i + 3 * blockDim.x] = v3;
  }
  for (; i < n_vec; i += blockDim.x) d[i] = s[i];
  __threadfence_system();  // the stores are on their way to the peer before the block retires
}

template <typename T>
__device__ __forceinline__ float to_float(T v);
template <>
__device__ __forceinline__ float to_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <>
__device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }
template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ float from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <>
__device__ __forceinline__ __half from_float<__half>(float v) { return __float2half_rn(v); }

// One block per token; 16-byte loads when VEC (16-bit rows, everything 16-byte aligned).
template <typename TIn, typename TOut, bool VEC>
__global__ void __launch_bounds__(256)
combine_rows_from_peers_kernel(const unsigned char* const* peers, int n_peers, long long y_stride_bytes,
                               long long capacity_rows, const int32_t* src_rank, const int32_t* src_row,
                               const float* weights, int topk, long long n_tokens, int n_cols, TOut* out,
                               long long out_stride, int* status) {
  constexpr int W = VEC ? 8 : 1;
  const long long t = blockIdx.x;
  if (t >= n_tokens) return;
  for (int c = threadIdx.x * W; c < n_cols; c += blockDim.x * W) {
    float acc[W];
#pragma unroll
    for (int j = 0; j < W; ++j) acc[j] = 0.f;
    for (int k = 0; k < topk; ++k) {
      const int rank = src_rank[t * topk + k];
      if (rank < 0) continue;
      const long long row = src_row[t * topk + k];
      if (rank >= n_peers || row < 0 || row >= capacity_rows) {
        if (c == 0) atomicOr(status, GMM_STATUS_BAD_PEER_INDEX);
        continue;
      }
      const float w = weights ? weights[t * topk + k] : 1.f;
      const TIn* y = reinterpret_cast<const TIn*>(peers[rank] + row * y_stride_bytes) + c;
      if constexpr (VEC) {
        const uint4 raw = *reinterpret_cast<const uint4*>(y);
        const TIn* v = reinterpret_cast<const TIn*>(&raw);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = fmaf(w, to_float<TIn>(v[j]), acc[j]);
      } else {
        acc[0] = fmaf(w, to_float<TIn>(*y), acc[0]);
      }
    }
    TOut* dst = out + t * out_stride + c;
    if constexpr (VEC) {
      if constexpr (sizeof(TOut) == 2) {
        uint4 packed;
        TOut* pv = reinterpret_cast<TOut*>(&packed);
#pragma unroll
        for (int j = 0; j < 8; ++j) pv[j] = from_float<TOut>(acc[j]);
        *reinterpret_cast<uint4*>(dst) = packed;
      } else {
        *reinterpret_cast<float4*>(dst) = make_float4(acc[0], acc[1], acc[2], acc[3]);
        *reinterpret_cast<float4*>(dst + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
      }
    } else {
      *dst = from_float<TOut>(acc[0]);
    }
  }
}

template <typename TIn, typename TOut>
int launch_combine_peers(const void* const* peers, int n_peers, long long y_stride_bytes, long long capacity_rows,
                         const int32_t* src_rank, const int32_t* src_row, const float* weights, int topk,
                         long long n_tokens, int n_cols, void* out, long long out_stride, bool vec, int* status,
                         cudaStream_t st) {
  auto pp = reinterpret_cast<const unsigned char* const*>(peers);
  TOut* o = reinterpret_cast<TOut*>(out);
  if (vec)
    combine_rows_from_peers_kernel<TIn, TOut, true><<<(unsigned)n_tokens, 256, 0, st>>>(
        pp, n_peers, y_stride_bytes, capacity_rows, src_rank, src_row, weights, topk, n_tokens, n_cols, o, out_stride,
        status);
  else
    combine_rows_from_peers_kernel<TIn, TOut, false><<<(unsigned)n_tokens, 256, 0, st>>>(
        pp, n_peers, y_stride_bytes, capacity_rows, src_rank, src_row, weights, topk, n_tokens, n_cols, o, out_stride,
        status);
  return cudaGetLastError() == cudaSuccess ? GMM_OK : GMM_ERR_CUDA;
}

template <typename TIn>
int launch_combine_peers_in(int out_dtype, const void* const* peers, int n_peers, long long y_stride_bytes,
                            long long capacity_rows, const int32_t* src_rank, const int32_t* src_row,
                            const float* weights, int topk, long long n_tokens, int n_cols, void* out,
                            long long out_stride, bool vec, int* status, cudaStream_t st) {
  switch (out_dtype) {
    case GMM_BF16:
      return launch_combine_peers<TIn, __nv_bfloat16>(peers, n_peers, y_stride_bytes, capacity_rows, src_rank, src_row,
                                                      weights, topk, n_tokens, n_cols, out, out_stride, vec, status, st);
    case GMM_F16:
      return launch_combine_peers<TIn, __half>(peers, n_peers, y_stride_bytes, capacity_rows, src_rank, src_row,
                                               weights, topk, n_tokens, n_cols, out, out_stride, vec, status, st);
    default:
      return launch_combine_peers<TIn, float>(peers, n_peers, y_stride_bytes, capacity_rows, src_rank, src_row,
                                              weights, topk, n_tokens, n_cols, out, out_stride, vec, status, st);
  }
}

}  // namespace

extern "C" {

int gmm_scatter_rows_to_peers(const void* src, int64_t src_rows, int64_t row_bytes, int64_t src_stride_bytes,
                              const int32_t* perm, int32_t topk, const int32_t* dst_rank, const int32_t* dst_row,
                              void* const* peers, int32_t n_peers, int64_t dst_stride_bytes, int64_t capacity_rows,
                              int64_t n_rows, int32_t* status, void* stream) {
  if (n_rows < 0 || row_bytes < 0 || topk <= 0 || src_rows < 0 || n_peers <= 0 || capacity_rows < 0)
    return GMM_ERR_INVALID_ARGUMENT;
  if (n_rows == 0 || row_bytes == 0) return GMM_OK;
  if (!src || !perm || !dst_rank || !dst_row || !peers || !status || n_rows > 0x7fffffffLL)
    return GMM_ERR_INVALID_ARGUMENT;
  if (dst_stride_bytes < row_bytes) return GMM_ERR_INVALID_ARGUMENT;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  auto s = reinterpret_cast<const unsigned char*>(src);
  auto pp = reinterpret_cast<unsigned char* const*>(peers);
  // Peer buffers are assumed 16-byte aligned (any allocation is); strides and row size decide the vector width.
  const bool vec16 = ((reinterpret_cast<uintptr_t>(src) | (uintptr_t)row_bytes | (uintptr_t)src_stride_bytes |
                       (uintptr_t)dst_stride_bytes) & 15u) == 0;
  if (vec16)
    scatter_rows_to_peers_kernel<uint4><<<(unsigned)n_rows, 128, 0, st>>>(
        s, src_rows, src_stride_bytes, perm, topk, dst_rank, dst_row, pp, n_peers, dst_stride_bytes, capacity_rows,
        n_rows, (int)(row_bytes / 16), status);
  else if (((row_bytes | src_stride_bytes | dst_stride_bytes) & 1) == 0 && (reinterpret_cast<uintptr_t>(src) & 1u) == 0)
    scatter_rows_to_peers_kernel<unsigned short><<<(unsigned)n_rows, 128, 0, st>>>(
        s, src_rows, src_stride_bytes, perm, topk, dst_rank, dst_row, pp, n_peers, dst_stride_bytes, capacity_rows,
        n_rows, (int)(row_bytes / 2), status);
  else
    scatter_rows_to_peers_kernel<unsigned char><<<(unsigned)n_rows, 128, 0, st>>>(
        s, src_rows, src_stride_bytes, perm, topk, dst_rank, dst_row, pp, n_peers, dst_stride_bytes, capacity_rows,
        n_rows, (int)row_bytes, status);
  return cudaGetLastError() == cudaSuccess ? GMM_OK : GMM_ERR_CUDA;
}

int gmm_combine_rows_from_peers(const void* const* peers, int32_t n_peers, int32_t y_dtype, int64_t y_stride,
                                int64_t capacity_rows, const int32_t* src_rank, const int32_t* src_row,
                                const float* weights, int32_t topk, int64_t n_tokens, int32_t n_cols, void* out,
                                int32_t out_dtype, int64_t out_stride, int32_t* status, void* stream) {
  if (n_tokens < 0 || n_cols < 0 || topk <= 0 || n_tokens > 0x7fffffffLL || n_peers <= 0 || capacity_rows < 0)
    return GMM_ERR_INVALID_ARGUMENT;
  if (y_dtype < GMM_BF16 || y_dtype > GMM_F32 || out_dtype < GMM_BF16 || out_dtype > GMM_F32)
    return GMM_ERR_UNSUPPORTED_DTYPE;
  if (n_tokens == 0 || n_cols == 0) return GMM_OK;
  if (!peers || !src_rank || !src_row || !out || !status || y_stride < n_cols) return GMM_ERR_INVALID_ARGUMENT;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const long long in_es = y_dtype == GMM_F32 ? 4 : 2;
  const long long out_es = out_dtype == GMM_F32 ? 4 : 2;
  const bool vec = in_es == 2 && (n_cols % 8 == 0) && (y_stride % 8 == 0) && ((out_stride * out_es) % 16 == 0) &&
                   (reinterpret_cast<uintptr_t>(out) & 15u) == 0;
  switch (y_dtype) {
    case GMM_BF16:
      return launch_combine_peers_in<__nv_bfloat16>(out_dtype, peers, n_peers, y_stride * in_es, capacity_rows, src_rank,
                                                    src_row, weights, topk, n_tokens, n_cols, out, out_stride, vec,
                                                    status, st);
    case GMM_F16:
      return launch_combine_peers_in<__half>(out_dtype, peers, n_peers, y_stride * in_es, capacity_rows, src_rank,
                                             src_row, weights, topk, n_tokens, n_cols, out, out_stride, vec, status, st);
    default:
      return launch_combine_peers_in<float>(out_dtype, peers, n_peers, y_stride * in_es, capacity_rows, src_rank,
                                            src_row, weights, topk, n_tokens, n_cols, out, out_stride, false, status,
                                            st);
  }
}

}  // extern "C"
