// gmm_zero_past_offsets: zero-fills the part of a 2-D tensor that lies at or past offs[-1] along its
// ragged dimension. The grouped GEMM leaves that part of its output untouched (it belongs to no
// group); a gradient must hold zeros there. The end offset is read on the device, so the host
// never waits; when offs[-1] equals the extent (the usual case) every thread returns at once, so
// the gradient is not swept a second time just to define a tail that is empty.
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/grouped_mm_b200.h"

namespace {

template <typename T>
__global__ void zero_past_offsets_kernel(T* data, long long extent, long long other, long long stride_ragged,
                                         long long stride_other, const int* __restrict__ offs, int n_groups) {
  long long end = n_groups > 0 ? (long long)offs[n_groups - 1] : 0;
  end = end < 0 ? 0 : (end > extent ? extent : end);
  const long long tail = extent - end;
  const long long total = tail * other;
  const long long step = (long long)gridDim.x * blockDim.x;
  const bool ragged_fast = stride_ragged <= stride_other;  // walk the contiguous dimension fastest
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += step) {
    long long i, j;
    if (ragged_fast) { i = idx % tail; j = idx / tail; }
    else { j = idx % other; i = idx / other; }
    data[(end + i) * stride_ragged + j * stride_other] = T(0);
  }
}

}  // namespace

extern "C" int gmm_zero_past_offsets(void* data, int32_t elem_bytes, int64_t extent, int64_t other,
                                     int64_t stride_ragged, int64_t stride_other, const int32_t* offs,
                                     int32_t n_groups, void* stream) {
  if (extent < 0 || other < 0 || n_groups < 0 || (elem_bytes != 2 && elem_bytes != 4)) return GMM_ERR_INVALID_ARGUMENT;
  if (extent == 0 || other == 0) return GMM_OK;
  if (!data || (n_groups > 0 && !offs)) return GMM_ERR_INVALID_ARGUMENT;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int grid = 592, block = 256;
  if (elem_bytes == 2)
    zero_past_offsets_kernel<uint16_t><<<grid, block, 0, st>>>(reinterpret_cast<uint16_t*>(data), extent, other,
                                                              stride_ragged, stride_other, offs, n_groups);
  else
    zero_past_offsets_kernel<uint32_t><<<grid, block, 0, st>>>(reinterpret_cast<uint32_t*>(data), extent, other,
                                                              stride_ragged, stride_other, offs, n_groups);
  return cudaGetLastError() == cudaSuccess ? GMM_OK : GMM_ERR_CUDA;
}
