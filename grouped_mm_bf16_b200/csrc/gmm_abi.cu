// Host side of libgrouped_mm_b200.so: argument checking, reduction of the four shape forms to
// the three canonical modes, kernel selection, tensor-map encoding and launch. Declared in
// include/grouped_mm_b200.h. Nothing here allocates device memory or waits for the device
// (gmm_check_status excepted, which exists to wait).
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdlib>
#include <mutex>
#include <string>

#include "../../include/grouped_mm_b200.h"
#include "gmm_common.cuh"
#include "gmm_generic_kernel.cuh"
#include "gmm_sm100_kernel.cuh"
#include "gmm_sm100_pair_kernel.cuh"

namespace {

using namespace gmm;

thread_local std::string g_last_cuda_error;

int cuda_fail(cudaError_t e, const char* what) {
  g_last_cuda_error = std::string(what) + ": " + cudaGetErrorString(e);
  return GMM_ERR_CUDA;
}

#define GMM_CUDA_TRY(expr)                               \
  do {                                                   \
    cudaError_t e__ = (expr);                            \
    if (e__ != cudaSuccess) return cuda_fail(e__, #expr); \
  } while (0)

// ------------------------------------------------------------------ per-device facts

constexpr int kMaxDevices = 64;
struct DeviceInfo {
  std::once_flag once;
  int status = GMM_OK;
  int sm_count = 0;
  int cc_major = 0;
};
DeviceInfo g_dev[kMaxDevices];

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
std::once_flag g_encode_once;
EncodeTiledFn g_encode = nullptr;

EncodeTiledFn get_encode() {
  std::call_once(g_encode_once, [] {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  });
  return g_encode;
}

template <typename K>
int set_smem_attr(K kernel, size_t bytes = kFastSmemBytes) {
  GMM_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
  return GMM_OK;
}

int init_device(int dev) {
  DeviceInfo& d = g_dev[dev];
  std::call_once(d.once, [&] {
    cudaError_t e = cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, dev);
    if (e != cudaSuccess) { d.status = cuda_fail(e, "cudaDeviceGetAttribute"); return; }
    if (d.cc_major != 10) { d.status = GMM_ERR_NOT_SM100; return; }
    int rc = GMM_OK;
    if (rc == GMM_OK) rc = set_smem_attr(gmm_sm100_kernel<false, __nv_bfloat16>);
    if (rc == GMM_OK) rc = set_smem_attr(gmm_sm100_kernel<false, __half>);
    if (rc == GMM_OK) rc = set_smem_attr(gmm_sm100_kernel<false, float>);
    if (rc == GMM_OK) rc = set_smem_attr(gmm_sm100_kernel<true, __nv_bfloat16>);
    if (rc == GMM_OK) rc = set_smem_attr(gmm_sm100_kernel<true, __half>);
    if (rc == GMM_OK) rc = set_smem_attr(gmm_sm100_kernel<true, float>);
    if (rc == GMM_OK) rc = set_smem_attr(gmm_sm100_kernel<false, float, 4>);
    if (rc == GMM_OK) rc = set_smem_attr(gmm_sm100_kernel<true, float, 4>);
    if (rc == GMM_OK) rc = set_smem_attr(gmm_sm100_pair_kernel<false, float, false, 4>, kPairSmemBytes);
    if (rc == GMM_OK) rc = set_smem_attr(gmm_sm100_pair_kernel<true, float, false, 4>, kPairSmemBytes);
    if (rc == GMM_OK) rc = set_smem_attr(gmm_sm100_kernel<false, __nv_bfloat16, 2, true>);
    if (rc == GMM_OK) rc = set_smem_attr(gmm_sm100_kernel<false, __half, 2, true>);
    if (rc == GMM_OK) rc = set_smem_attr(gmm_sm100_kernel<false, float, 2, true>);
    if (rc == GMM_OK) rc = set_smem_attr(gmm_sm100_pair_kernel<false, __nv_bfloat16, true>, kPairSmemBytes);
    if (rc == GMM_OK) rc = set_smem_attr(gmm_sm100_pair_kernel<false, __half, true>, kPairSmemBytes);
    if (rc == GMM_OK) rc = set_smem_attr(gmm_sm100_pair_kernel<false, float, true>, kPairSmemBytes);
    if (rc == GMM_OK) rc = set_smem_attr(gmm_sm100_pair_kernel<false, __nv_bfloat16>, kPairSmemBytes);
    if (rc == GMM_OK) rc = set_smem_attr(gmm_sm100_pair_kernel<false, __half>, kPairSmemBytes);
    if (rc == GMM_OK) rc = set_smem_attr(gmm_sm100_pair_kernel<false, float>, kPairSmemBytes);
    if (rc == GMM_OK) rc = set_smem_attr(gmm_sm100_pair_kernel<true, __nv_bfloat16>, kPairSmemBytes);
    if (rc == GMM_OK) rc = set_smem_attr(gmm_sm100_pair_kernel<true, __half>, kPairSmemBytes);
    if (rc == GMM_OK) rc = set_smem_attr(gmm_sm100_pair_kernel<true, float>, kPairSmemBytes);
    d.status = rc;
  });
  return d.status;
}

// ------------------------------------------------------------------ canonicalisation

bool tensor_ok(const gmm_tensor_t* t, int ndim) {
  if (!t || t->ndim != ndim) return false;
  if (t->dtype < GMM_BF16 || t->dtype > GMM_F32) return false;
  for (int i = 0; i < ndim; ++i)
    if (t->size[i] < 0 || t->size[i] > 0x7fffffffLL) return false;
  return true;
}

long long numel(const gmm_tensor_t* t) {
  long long n = 1;
  for (int i = 0; i < t->ndim; ++i) n *= t->size[i];
  return n;
}

// form: 0 = 3d3d, 1 = 2d3d, 2 = 3d2d, 3 = 2d2d. On success *nothing is set when the call has no
// work (empty output or no groups). `swiglu` (form 1 only): b holds [gate | up], twice the output's
// columns; the canonical N is the output's.
int canonicalise(int form, const gmm_tensor_t* a, const gmm_tensor_t* b, const int32_t* offs, int n_groups,
                 const gmm_tensor_t* out, CanonProblem* cp, bool* nothing, bool need_pointers,
                 bool swiglu = false) {
  *nothing = false;
  if (swiglu && form != 1) return GMM_ERR_INVALID_ARGUMENT;
  const int a_nd = (form == 0 || form == 2) ? 3 : 2;
  const int b_nd = (form == 0 || form == 1) ? 3 : 2;
  const int c_nd = (form == 0 || form == 3) ? 3 : 2;
  if (form < 0 || form > 3) return GMM_ERR_INVALID_ARGUMENT;
  if (!tensor_ok(a, a_nd) || !tensor_ok(b, b_nd) || !tensor_ok(out, c_nd)) {
    if (a && b && out && (a->dtype < GMM_BF16 || a->dtype > GMM_F32 || b->dtype < GMM_BF16 ||
                          b->dtype > GMM_F32 || out->dtype < GMM_BF16 || out->dtype > GMM_F32))
      return GMM_ERR_UNSUPPORTED_DTYPE;
    return GMM_ERR_INVALID_ARGUMENT;
  }
  if (a->dtype != b->dtype) return GMM_ERR_INVALID_ARGUMENT;
  if (form != 0) {
    if (n_groups < 0) return GMM_ERR_INVALID_ARGUMENT;
    if (n_groups >= kMaxGroups) return GMM_ERR_TOO_MANY_GROUPS;
    if (need_pointers && n_groups > 0 && !offs) return GMM_ERR_INVALID_ARGUMENT;
  }

  CanonProblem p = {};
  p.a = a->data;
  p.b = b->data;
  p.c = out->data;
  p.offs = offs;
  p.in_dtype = a->dtype;
  p.out_dtype = out->dtype;
  switch (form) {
    case 0: {  // [G,M,K] x [G,K,N] -> [G,M,N]
      if (a->size[0] != b->size[0] || a->size[2] != b->size[1]) return GMM_ERR_INVALID_ARGUMENT;
      if (out->size[0] != a->size[0] || out->size[1] != a->size[1] || out->size[2] != b->size[2])
        return GMM_ERR_INVALID_ARGUMENT;
      p.mode = MODE_UNIFORM;
      p.G = (int)a->size[0]; p.M = (int)a->size[1]; p.K = (int)a->size[2]; p.N = (int)b->size[2];
      p.a_sg = a->stride[0]; p.a_sm = a->stride[1]; p.a_sk = a->stride[2];
      p.b_sg = b->stride[0]; p.b_sk = b->stride[1]; p.b_sn = b->stride[2];
      p.c_sg = out->stride[0]; p.c_sm = out->stride[1]; p.c_sn = out->stride[2];
      p.offs = nullptr;
      break;
    }
    case 1: {  // [Mt,K] x [G,K,N] -> [Mt,N]
      if (a->size[1] != b->size[1] || b->size[0] != n_groups) return GMM_ERR_INVALID_ARGUMENT;
      if (out->size[0] != a->size[0] || out->size[1] * (swiglu ? 2 : 1) != b->size[2])
        return GMM_ERR_INVALID_ARGUMENT;
      p.mode = MODE_MRAGGED;
      p.G = n_groups; p.M = (int)a->size[0]; p.K = (int)a->size[1]; p.N = (int)out->size[1];
      p.a_sg = 0; p.a_sm = a->stride[0]; p.a_sk = a->stride[1];
      p.b_sg = b->stride[0]; p.b_sk = b->stride[1]; p.b_sn = b->stride[2];
      p.c_sg = 0; p.c_sm = out->stride[0]; p.c_sn = out->stride[1];
      break;
    }
    case 2: {  // [G,M,K] x [K,Nt] -> [M,Nt], computed as out^T = b^T * a[g]^T (row-ragged)
      if (a->size[2] != b->size[0] || a->size[0] != n_groups) return GMM_ERR_INVALID_ARGUMENT;
      if (out->size[0] != a->size[1] || out->size[1] != b->size[1]) return GMM_ERR_INVALID_ARGUMENT;
      p.mode = MODE_MRAGGED;
      p.G = n_groups; p.M = (int)b->size[1]; p.K = (int)a->size[2]; p.N = (int)a->size[1];
      p.a = b->data; p.b = a->data;
      p.a_sg = 0; p.a_sm = b->stride[1]; p.a_sk = b->stride[0];
      p.b_sg = a->stride[0]; p.b_sk = a->stride[2]; p.b_sn = a->stride[1];
      p.c_sg = 0; p.c_sm = out->stride[1]; p.c_sn = out->stride[0];
      break;
    }
    default: {  // [M,Kt] x [Kt,N] -> [G,M,N]
      if (a->size[1] != b->size[0]) return GMM_ERR_INVALID_ARGUMENT;
      if (out->size[0] != n_groups || out->size[1] != a->size[0] || out->size[2] != b->size[1])
        return GMM_ERR_INVALID_ARGUMENT;
      p.mode = MODE_KRAGGED;
      p.G = n_groups; p.M = (int)a->size[0]; p.K = (int)a->size[1]; p.N = (int)b->size[1];
      p.a_sg = 0; p.a_sm = a->stride[0]; p.a_sk = a->stride[1];
      p.b_sg = 0; p.b_sk = b->stride[0]; p.b_sn = b->stride[1];
      p.c_sg = out->stride[0]; p.c_sm = out->stride[1]; p.c_sn = out->stride[2];
      break;
    }
  }
  if (numel(out) == 0 || p.G == 0) { *nothing = true; *cp = p; return GMM_OK; }
  if (need_pointers) {
    if (!p.c) return GMM_ERR_INVALID_ARGUMENT;
    if (p.K > 0 && (!p.a || !p.b)) return GMM_ERR_INVALID_ARGUMENT;
  }
  *cp = p;
  return GMM_OK;
}

// ------------------------------------------------------------------ kernel selection

struct FastPlan {
  bool ok = false;
  int a_mn = 0;
  int b_mn = 0;
  bool pair = false;  // CTA-pair kernel (256-row tiles) instead of the single-CTA kernel (128-row tiles)
};

int env_int(const char* name, int fallback) {
  const char* v = std::getenv(name);
  return (v && *v) ? std::atoi(v) : fallback;
}

bool aligned16(const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15u) == 0; }

// The TMA path needs 16-byte aligned bases and leading/group strides, and the ragged dimension
// must not be the contiguous one (a group may start at any index of it, while a TMA box must start
// on a 16-byte boundary of the contiguous dimension). 16-bit inputs always qualify; fp32 inputs
// only when the caller allows TF32 arithmetic (GMM_FLAG_ALLOW_TF32) and the output is fp32 -
// otherwise fp32 stays on the generic kernel, which multiplies in true fp32.
FastPlan plan_fast(const CanonProblem& p, uint32_t flags, bool swiglu = false) {
  FastPlan f;
  if (p.K < 1) return f;
  const bool tf32 = (p.in_dtype == DT_F32);
  if (swiglu && tf32) return f;
  if (tf32 && (!(flags & GMM_FLAG_ALLOW_TF32) || p.out_dtype != DT_F32)) return f;
  const int q = tf32 ? 4 : 8;  // elements per 16 bytes
  if (!aligned16(p.a) || !aligned16(p.b)) return f;
  if (p.a_sk == 1 && p.a_sm % q == 0 && p.a_sm >= p.K) f.a_mn = 0;
  else if (p.a_sm == 1 && p.a_sk % q == 0 && p.a_sk >= p.M) f.a_mn = 1;
  else return f;
  if (p.b_sk == 1 && p.b_sn % q == 0 && p.b_sn >= p.K) f.b_mn = 0;
  else if (p.b_sn == 1 && p.b_sk % q == 0 && p.b_sk >= p.N) f.b_mn = 1;
  else return f;
  if (p.mode == MODE_UNIFORM && p.G > 1 && (p.a_sg <= 0 || p.a_sg % q != 0)) return f;
  if (p.mode != MODE_KRAGGED && p.G > 1 && (p.b_sg <= 0 || p.b_sg % q != 0)) return f;
  if (p.mode == MODE_MRAGGED && f.a_mn) return f;
  if (p.mode == MODE_KRAGGED && !(f.a_mn && f.b_mn)) return f;
  // The up half of a row-major B starts at column N: a TMA box may only start there if N is a multiple of 16 bytes.
  if (swiglu && f.b_mn && (p.N % q != 0 || p.b_sk < 2ll * p.N)) return f;
  f.ok = true;
  // 256-row pair tiles pay off when groups are tall (little tail waste) and N spans both halves.
  // The group sizes live on the device, so the host decides on the mean rows per group.
  if (p.N > kPairBNHalf || swiglu) {
    const long long mean_rows = (p.mode == MODE_MRAGGED) ? (long long)p.M / (p.G > 0 ? p.G : 1) : p.M;
    f.pair = mean_rows >= 512;
    if (flags & GMM_FLAG_FORCE_PAIR) f.pair = true;
    if (flags & GMM_FLAG_NO_PAIR) f.pair = false;
    const int env = env_int("GROUPED_MM_B200_PAIR", -1);  // tuning knob: 0 / 1 overrides the heuristic
    if (env == 0) f.pair = false;
    if (env == 1) f.pair = true;
  }
  return f;
}

// ------------------------------------------------------------------ tensor maps

// 3-D map (inner, outer, batch) over an operand with a 128-byte-swizzled box: 64 16-bit or 32
// 32-bit elements wide. `mn_major`: the inner dimension is M or N rather than K; a 32-bit operand
// is then swizzled in 32-byte units, the layout tcgen05.mma reads such an operand in.
int encode_map(CUtensorMap* map, const void* base, int in_dtype, bool mn_major, long long inner, long long outer,
               long long batch, long long outer_stride_elems, long long batch_stride_elems, int box_outer) {
  EncodeTiledFn enc = get_encode();
  if (!enc) {
    g_last_cuda_error = "cuTensorMapEncodeTiled entry point not found";
    return GMM_ERR_CUDA;
  }
  cuuint64_t dims[3] = {(cuuint64_t)inner, (cuuint64_t)outer, (cuuint64_t)(batch > 0 ? batch : 1)};
  if (batch <= 1) batch_stride_elems = outer_stride_elems * outer;
  const unsigned es = (in_dtype == DT_F32) ? 4 : 2;
  cuuint64_t strides[2] = {(cuuint64_t)outer_stride_elems * es, (cuuint64_t)batch_stride_elems * es};
  cuuint32_t box[3] = {128 / es, (cuuint32_t)box_outer, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  const CUtensorMapDataType dt = in_dtype == DT_BF16  ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                 : in_dtype == DT_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                      : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  const CUtensorMapSwizzle swz =
      (es == 4 && mn_major) ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B;
  CUresult r = enc(map, dt, 3,
                   const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    g_last_cuda_error = "cuTensorMapEncodeTiled failed with CUresult " + std::to_string((int)r);
    return GMM_ERR_CUDA;
  }
  return GMM_OK;
}

uint32_t make_idesc(int in_dtype, int a_mn, int b_mn, int mma_m) {
  // kind::f16: 0 = f16, 1 = bf16; kind::tf32: 2 = tf32
  const uint32_t fmt = (in_dtype == DT_BF16) ? 1u : (in_dtype == DT_F32) ? 2u : 0u;
  uint32_t d = 0;
  d |= 1u << 4;                        // accumulator format: f32
  d |= fmt << 7;                       // A format
  d |= fmt << 10;                      // B format
  d |= (uint32_t)(a_mn ? 1 : 0) << 15; // A major: 0 = K, 1 = MN
  d |= (uint32_t)(b_mn ? 1 : 0) << 16; // B major
  d |= (uint32_t)(kBN >> 3) << 17;     // N / 8
  d |= (uint32_t)(mma_m >> 4) << 24;   // M / 16 (128 for one CTA, 256 for a CTA pair)
  return d;
}

// ------------------------------------------------------------------ launches

template <typename TIn, int BM, int BN>
int launch_generic_in(const CanonProblem& p, int grid, cudaStream_t st) {
  switch (p.out_dtype) {
    case DT_BF16: gmm_generic_kernel<TIn, __nv_bfloat16, BM, BN><<<grid, kGenericThreads, 0, st>>>(p); break;
    case DT_F16: gmm_generic_kernel<TIn, __half, BM, BN><<<grid, kGenericThreads, 0, st>>>(p); break;
    default: gmm_generic_kernel<TIn, float, BM, BN><<<grid, kGenericThreads, 0, st>>>(p); break;
  }
  GMM_CUDA_TRY(cudaGetLastError());
  return GMM_OK;
}

long long tile_upper_bound(const CanonProblem& p, int bm, int bn) {
  const long long nt = (p.N + bn - 1) / bn;
  long long mt;
  if (p.mode == MODE_MRAGGED) mt = (p.M + bm - 1) / bm + p.G;  // at most one partial tile more per group
  else mt = (long long)p.G * ((p.M + bm - 1) / bm);
  return mt * nt;
}

template <int BM, int BN>
int launch_generic_tile(const CanonProblem& p, long long tiles, int blocks_per_sm, const DeviceInfo& d,
                        cudaStream_t st) {
  const long long cap = (long long)d.sm_count * blocks_per_sm;
  const int grid = (int)(tiles < cap ? tiles : cap);
  switch (p.in_dtype) {
    case DT_BF16: return launch_generic_in<__nv_bfloat16, BM, BN>(p, grid, st);
    case DT_F16: return launch_generic_in<__half, BM, BN>(p, grid, st);
    default: return launch_generic_in<float, BM, BN>(p, grid, st);
  }
}

int launch_generic(const CanonProblem& p, const DeviceInfo& d, cudaStream_t st) {
  const long long ub = tile_upper_bound(p, kGBM, kGBN);
  if (ub <= 0) return GMM_OK;
  if (ub > 0x7fffffffLL) return GMM_ERR_INVALID_ARGUMENT;
  // 128 x 128 tiles (64 outputs per thread) once there are enough of them to occupy every SM twice;
  // 64 x 64 tiles otherwise, which waste less on short groups and spread a small problem wider.
  const long long ub_large = tile_upper_bound(p, kGBML, kGBNL);
  const bool tall = (p.mode == MODE_MRAGGED ? (long long)p.M / (p.G > 0 ? p.G : 1) : p.M) >= kGBML;
  if (tall && p.N >= kGBNL && ub_large >= 2ll * d.sm_count)
    return launch_generic_tile<kGBML, kGBNL>(p, ub_large, 1, d, st);  // 244 registers: one block per SM
  return launch_generic_tile<kGBM, kGBN>(p, ub, 8, d, st);
}

template <bool KR>
int launch_fast_kr(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const FastParams& fp, int grid,
                   cudaStream_t st) {
  switch (fp.p.out_dtype) {
    case DT_BF16:
      gmm_sm100_kernel<KR, __nv_bfloat16><<<grid, kFastThreads, kFastSmemBytes, st>>>(ta, tb, tc, fp);
      break;
    case DT_F16:
      gmm_sm100_kernel<KR, __half><<<grid, kFastThreads, kFastSmemBytes, st>>>(ta, tb, tc, fp);
      break;
    default:
      gmm_sm100_kernel<KR, float><<<grid, kFastThreads, kFastSmemBytes, st>>>(ta, tb, tc, fp);
      break;
  }
  GMM_CUDA_TRY(cudaGetLastError());
  return GMM_OK;
}

template <typename TOut>
int launch_pair_t(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const FastParams& fp, int grid,
                  cudaStream_t st) {
  if (fp.p.mode == MODE_KRAGGED)
    gmm_sm100_pair_kernel<true, TOut><<<grid, kFastThreads, kPairSmemBytes, st>>>(ta, tb, tc, fp);
  else
    gmm_sm100_pair_kernel<false, TOut><<<grid, kFastThreads, kPairSmemBytes, st>>>(ta, tb, tc, fp);
  GMM_CUDA_TRY(cudaGetLastError());
  return GMM_OK;
}

// n-tiles per B panel: as many as keep one panel (panel x BN columns x K rows) within a budget
// that stays resident in L2 while every m-tile of the group is swept over it.
int choose_panel(const CanonProblem& p) {
  const int env = env_int("GROUPED_MM_B200_PANEL", 0);  // tuning knob
  if (env > 0) return env;
  const long long tile_bytes = (long long)kBN * p.K * (p.in_dtype == DT_F32 ? 4 : 2);
  long long panel = (32ll << 20) / (tile_bytes > 0 ? tile_bytes : 1);
  if (panel < 2) panel = 2;
  if (panel > 64) panel = 64;
  return (int)panel;
}

template <typename TOut>
int launch_swiglu_t(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const FastParams& fp, bool pair,
                    int grid, cudaStream_t st) {
  if (pair)
    gmm_sm100_pair_kernel<false, TOut, true><<<grid, kFastThreads, kPairSmemBytes, st>>>(ta, tb, tc, fp);
  else
    gmm_sm100_kernel<false, TOut, 2, true><<<grid, kFastThreads, kFastSmemBytes, st>>>(ta, tb, tc, fp);
  GMM_CUDA_TRY(cudaGetLastError());
  return GMM_OK;
}

int launch_fast(const CanonProblem& p_in, const FastPlan& plan, const DeviceInfo& d, cudaStream_t st,
                bool swiglu = false, void* group_maps = nullptr) {
  CanonProblem p = p_in;
  const int bm = plan.pair ? kPairBM : kBM;
  p.panel = choose_panel(p);
  const long long ub = tile_upper_bound(p, bm, swiglu ? kBN / 2 : kBN);
  if (ub <= 0) return GMM_OK;
  if (ub > 0x7fffffffLL) return GMM_ERR_INVALID_ARGUMENT;
  const int units = plan.pair ? d.sm_count / 2 : d.sm_count;
  const int grid = (int)(ub < units ? ub : units) * (plan.pair ? 2 : 1);

  const bool a_batched = (p.mode == MODE_UNIFORM);
  const bool b_batched = (p.mode != MODE_KRAGGED);
  const bool tf32 = (p.in_dtype == DT_F32);
  const int bk = tf32 ? ElemGeom<4>::BK : ElemGeom<2>::BK;  // k-rows per box of an MN-major operand
  CUtensorMap ta, tb;
  int rc;
  if (!plan.a_mn)
    rc = encode_map(&ta, p.a, p.in_dtype, false, p.K, p.M, a_batched ? p.G : 1, p.a_sm, p.a_sg, 128);
  else
    rc = encode_map(&ta, p.a, p.in_dtype, true, p.M, p.K, a_batched ? p.G : 1, p.a_sk, p.a_sg, bk);
  if (rc != GMM_OK) return rc;
  const long long b_cols = swiglu ? 2ll * p.N : p.N;  // [gate | up] when the activation is fused
  if (!plan.b_mn)
    rc = encode_map(&tb, p.b, p.in_dtype, false, p.K, b_cols, b_batched ? p.G : 1, p.b_sn, p.b_sg,
                    (plan.pair || swiglu) ? kPairBNHalf : kBN);
  else
    rc = encode_map(&tb, p.b, p.in_dtype, true, b_cols, p.K, b_batched ? p.G : 1, p.b_sk, p.b_sg, bk);
  if (rc != GMM_OK) return rc;

  // Output map for TMA stores of whole 32-row x 128-byte pieces: needs a unit column stride and
  // 16-byte aligned rows (the operator's own outputs have both; a caller's strided view may not).
  CUtensorMap tc = {};
  const long long c_es = (p.out_dtype == DT_F32) ? 4 : 2;
  const bool c_batched = (p.mode != MODE_MRAGGED);
  bool c_tma = !swiglu && p.c_sn == 1 && aligned16(p.c) && (p.c_sm * c_es) % 16 == 0 && p.c_sm >= p.N &&
               (!c_batched || p.G <= 1 || (p.c_sg > 0 && (p.c_sg * c_es) % 16 == 0)) &&
               env_int("GROUPED_MM_B200_TMA_STORE", 1) != 0;
  if (c_tma) {
    rc = encode_map(&tc, p.c, p.out_dtype, false, p.N, p.M, c_batched ? p.G : 1, p.c_sm, p.c_sg, 32);
    if (rc != GMM_OK) return rc;
  }

  FastParams fp;
  fp.p = p;
  fp.a_mn = plan.a_mn;
  fp.b_mn = plan.b_mn;
  fp.c_tma = c_tma ? 1 : 0;
  fp.idesc = make_idesc(p.in_dtype, plan.a_mn, plan.b_mn, plan.pair ? 256 : 128);
  fp.idesc_half = 0;
  fp.tmap_a_half = ta;
  if (!plan.pair && !swiglu && p.mode != MODE_KRAGGED && env_int("GROUPED_MM_B200_HALF_TILES", 1) != 0) {
    fp.idesc_half = make_idesc(p.in_dtype, plan.a_mn, plan.b_mn, 64);
    if (!plan.a_mn) {
      rc = encode_map(&fp.tmap_a_half, p.a, p.in_dtype, false, p.K, p.M, a_batched ? p.G : 1, p.a_sm, p.a_sg, 64);
      if (rc != GMM_OK) return rc;
    }
  }
  fp.maps_a = fp.maps_b = nullptr;
  if (p.mode == MODE_KRAGGED) {
    // Per-group copies of both maps, each ending at its group's end along K, written on the device
    // from `offs` ahead of the GEMM kernel on the same stream.
    fp.maps_a = reinterpret_cast<const CUtensorMap*>(group_maps);
    fp.maps_b = fp.maps_a + p.G;
    build_group_maps_kernel<<<(p.G + 127) / 128, 128, 0, st>>>(ta, tb, p.offs, p.G, p.K,
                                                              const_cast<CUtensorMap*>(fp.maps_a),
                                                              const_cast<CUtensorMap*>(fp.maps_b));
    GMM_CUDA_TRY(cudaGetLastError());
  }
  if (swiglu) {
    switch (p.out_dtype) {
      case DT_BF16: return launch_swiglu_t<__nv_bfloat16>(ta, tb, tc, fp, plan.pair, grid, st);
      case DT_F16: return launch_swiglu_t<__half>(ta, tb, tc, fp, plan.pair, grid, st);
      default: return launch_swiglu_t<float>(ta, tb, tc, fp, plan.pair, grid, st);
    }
  }
  if (tf32) {
    if (plan.pair) {
      if (p.mode == MODE_KRAGGED)
        gmm_sm100_pair_kernel<true, float, false, 4><<<grid, kFastThreads, kPairSmemBytes, st>>>(ta, tb, tc, fp);
      else
        gmm_sm100_pair_kernel<false, float, false, 4><<<grid, kFastThreads, kPairSmemBytes, st>>>(ta, tb, tc, fp);
    } else if (p.mode == MODE_KRAGGED) {
      gmm_sm100_kernel<true, float, 4><<<grid, kFastThreads, kFastSmemBytes, st>>>(ta, tb, tc, fp);
    } else {
      gmm_sm100_kernel<false, float, 4><<<grid, kFastThreads, kFastSmemBytes, st>>>(ta, tb, tc, fp);
    }
    GMM_CUDA_TRY(cudaGetLastError());
    return GMM_OK;
  }
  if (plan.pair) {
    switch (p.out_dtype) {
      case DT_BF16: return launch_pair_t<__nv_bfloat16>(ta, tb, tc, fp, grid, st);
      case DT_F16: return launch_pair_t<__half>(ta, tb, tc, fp, grid, st);
      default: return launch_pair_t<float>(ta, tb, tc, fp, grid, st);
    }
  }
  return p.mode == MODE_KRAGGED ? launch_fast_kr<true>(ta, tb, tc, fp, grid, st)
                                : launch_fast_kr<false>(ta, tb, tc, fp, grid, st);
}

constexpr size_t kStatusBytes = 256;  // the workspace of every form: the status word and padding

size_t group_maps_bytes(int n_groups) { return n_groups > 0 ? 2 * sizeof(CUtensorMap) * (size_t)n_groups : 0; }

int run(int form, const gmm_tensor_t* a, const gmm_tensor_t* b, const int32_t* offs, int n_groups,
        const gmm_tensor_t* out, const gmm_launch_t* launch, bool swiglu = false) {
  if (!launch) return GMM_ERR_INVALID_ARGUMENT;
  CanonProblem p;
  bool nothing;
  int rc = canonicalise(form, a, b, offs, n_groups, out, &p, &nothing, true, swiglu);
  if (rc != GMM_OK) return rc;
  if (nothing) return GMM_OK;
  if (!launch->workspace || launch->workspace_bytes < kStatusBytes ||
      (reinterpret_cast<uintptr_t>(launch->workspace) & 255u))
    return GMM_ERR_WORKSPACE;
  p.status = reinterpret_cast<int*>(launch->workspace);

  int dev = 0;
  GMM_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return GMM_ERR_INVALID_ARGUMENT;
  rc = init_device(dev);
  if (rc != GMM_OK) return rc;
  const DeviceInfo& d = g_dev[dev];
  cudaStream_t st = reinterpret_cast<cudaStream_t>(launch->stream);

  const FastPlan plan =
      (launch->flags & GMM_FLAG_FORCE_GENERIC) ? FastPlan() : plan_fast(p, launch->flags, swiglu);
  if (swiglu) return plan.ok ? launch_fast(p, plan, d, st, true) : GMM_ERR_NOT_FUSABLE;
  if (!plan.ok) return launch_generic(p, d, st);
  if (p.mode == MODE_KRAGGED &&
      (!launch->group_maps || launch->group_maps_bytes < group_maps_bytes(p.G) ||
       (reinterpret_cast<uintptr_t>(launch->group_maps) & 127u)))
    return GMM_ERR_WORKSPACE;
  return launch_fast(p, plan, d, st, false, launch->group_maps);
}

// ------------------------------------------------------------------ library-owned scratch
//
// Scratch for grouped_mm_2d3d_static_scratch(): the same 256-byte block (status word first) that
// other entry points receive as `workspace`, but owned by the library image itself, so that the
// caller has nothing to allocate. Every GPU that loads the library holds these 256 bytes until the
// process exits. In host code the array's name only stands for the symbol; the device address
// comes from cudaGetSymbolAddress(), once per device, with that device current.
constexpr size_t kStaticScratchBytes = 256;
static_assert(kStatusBytes <= kStaticScratchBytes, "the row-ragged form's scratch need must fit the library-owned array");
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

struct StaticScratch {
  std::once_flag once;
  int status = GMM_OK;
  void* ptr = nullptr;
};
StaticScratch g_static[kMaxDevices];

// Must run with device `dev` current. The first call on a device does the symbol lookup.
int static_scratch(int dev, void** ptr) {
  StaticScratch& ss = g_static[dev];
  std::call_once(ss.once, [&] {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess || p == nullptr) {
      ss.status = cuda_fail(e, "cudaGetSymbolAddress(g_static_scratch)");
      return;
    }
    ss.ptr = p;
  });
  *ptr = ss.ptr;
  return ss.status;
}

// ------------------------------------------------------------------ wait self-test
//
// One CTA waits, with a short budget, on an mbarrier that nothing will ever complete: the wait
// gives up, the status word is set, the kernel returns normally and the context stays usable.
// This is the path every bounded wait of the GEMM kernels takes if a producer or consumer goes
// missing; it is exercised here without any real failure.
__global__ void wait_selftest_kernel(int* status, long long budget_cycles) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    abort_flag = 0;
    fence_barrier_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    if (!mbar_wait(&bar, 0, &abort_flag, 0, budget_cycles)) atomicCAS(status, 0, 0x7E57);
  }
}

}  // namespace

// ====================================================================== C ABI

extern "C" {

int gmm_abi_version(void) { return GMM_ABI_VERSION; }

const char* gmm_error_string(int status) {
  switch (status) {
    case GMM_OK: return "ok";
    case GMM_ERR_INVALID_ARGUMENT: return "invalid argument (null pointer, rank, size or shape mismatch)";
    case GMM_ERR_UNSUPPORTED_DTYPE: return "unsupported dtype (expected bf16, fp16 or fp32)";
    case GMM_ERR_TOO_MANY_GROUPS: return "Can't process more than 1024 groups";
    case GMM_ERR_WORKSPACE: return "workspace (or, for grouped_mm_2d2d, group_maps) missing, misaligned or too small";
    case GMM_ERR_CUDA: return "CUDA call failed";
    case GMM_ERR_NOT_SM100: return "device is not compute capability 10.x (B200)";
    case GMM_ERR_DEVICE_WAIT: return "a bounded wait inside the kernel gave up; outputs are invalid";
    case GMM_ERR_NOT_FUSABLE:
      return "operands not addressable by the tensor-core path; run grouped_mm_2d3d and apply the activation separately";
    default: return "unknown status";
  }
}

const char* gmm_last_cuda_error(void) { return g_last_cuda_error.c_str(); }

size_t gmm_workspace_bytes(void) { return kStatusBytes; }

size_t gmm_group_maps_bytes(int32_t n_groups) { return group_maps_bytes(n_groups); }

int grouped_mm_3d3d(const gmm_tensor_t* a, const gmm_tensor_t* b, const gmm_tensor_t* out,
                    const gmm_launch_t* launch) {
  return run(0, a, b, nullptr, 0, out, launch);
}

int grouped_mm_2d3d(const gmm_tensor_t* a, const gmm_tensor_t* b, const int32_t* offs, int32_t n_groups,
                    const gmm_tensor_t* out, const gmm_launch_t* launch) {
  return run(1, a, b, offs, n_groups, out, launch);
}

int grouped_mm_3d2d(const gmm_tensor_t* a, const gmm_tensor_t* b, const int32_t* offs, int32_t n_groups,
                    const gmm_tensor_t* out, const gmm_launch_t* launch) {
  return run(2, a, b, offs, n_groups, out, launch);
}

int grouped_mm_2d3d_swiglu(const gmm_tensor_t* a, const gmm_tensor_t* b_gate_up, const int32_t* offs,
                           int32_t n_groups, const gmm_tensor_t* out, const gmm_launch_t* launch) {
  return run(1, a, b_gate_up, offs, n_groups, out, launch, true);
}

int grouped_mm_2d2d(const gmm_tensor_t* a, const gmm_tensor_t* b, const int32_t* offs, int32_t n_groups,
                    const gmm_tensor_t* out, const gmm_launch_t* launch) {
  return run(3, a, b, offs, n_groups, out, launch);
}

int grouped_mm_2d3d_static_scratch(const gmm_tensor_t* a, const gmm_tensor_t* b, const int32_t* offs,
                                   int32_t n_groups, const gmm_tensor_t* out, void* stream, uint32_t flags,
                                   void** scratch_address) {
  // Check the arguments before touching the shared block: a rejected call, or one with no work,
  // must leave the status word of an earlier call as it is.
  CanonProblem p;
  bool nothing;
  int rc = canonicalise(1, a, b, offs, n_groups, out, &p, &nothing, true);
  if (rc != GMM_OK) return rc;
  int dev = 0;
  GMM_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return GMM_ERR_INVALID_ARGUMENT;
  void* scratch = nullptr;
  rc = static_scratch(dev, &scratch);
  if (rc != GMM_OK) return rc;
  if (scratch_address) *scratch_address = scratch;
  if (nothing) return GMM_OK;
  // The block keeps whatever the previous call left. Only the status word has to start at zero;
  // a code an earlier call left there unread is lost at this point.
  GMM_CUDA_TRY(cudaMemsetAsync(scratch, 0, sizeof(int), reinterpret_cast<cudaStream_t>(stream)));
  gmm_launch_t launch;
  launch.stream = stream;
  launch.workspace = scratch;
  launch.workspace_bytes = kStaticScratchBytes;
  launch.flags = flags;
  launch.group_maps = nullptr;  // the row-ragged form needs none
  launch.group_maps_bytes = 0;
  return run(1, a, b, offs, n_groups, out, &launch);
}

int gmm_select_kernel(int32_t form, const gmm_tensor_t* a, const gmm_tensor_t* b, const gmm_tensor_t* out,
                      uint32_t flags) {
  CanonProblem p;
  bool nothing;
  int n_groups = 0;
  if (form == 1 && b) n_groups = (int)b->size[0];
  if (form == 2 && a) n_groups = (int)a->size[0];
  if (form == 3 && out) n_groups = (int)out->size[0];
  int rc = canonicalise(form, a, b, nullptr, n_groups, out, &p, &nothing, false);
  if (rc != GMM_OK) return rc;
  if (nothing) return GMM_KERNEL_NONE;
  if (flags & GMM_FLAG_FORCE_GENERIC) return GMM_KERNEL_GENERIC;
  const FastPlan plan = plan_fast(p, flags);
  if (!plan.ok) return GMM_KERNEL_GENERIC;
  return plan.pair ? GMM_KERNEL_TCGEN05_PAIR : GMM_KERNEL_TCGEN05;
}

int gmm_selftest_wait_timeout(void* workspace, void* stream, int64_t budget_cycles) {
  if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 3u)) return GMM_ERR_WORKSPACE;
  if (budget_cycles <= 0 || budget_cycles > kWaitBudgetCycles) return GMM_ERR_INVALID_ARGUMENT;
  wait_selftest_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(reinterpret_cast<int*>(workspace),
                                                                           (long long)budget_cycles);
  GMM_CUDA_TRY(cudaGetLastError());
  return GMM_OK;
}

int gmm_check_status(void* workspace, void* stream, int32_t* raw) {
  if (!workspace) return GMM_ERR_WORKSPACE;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  GMM_CUDA_TRY(cudaStreamSynchronize(st));
  int32_t v = 0;
  GMM_CUDA_TRY(cudaMemcpy(&v, workspace, sizeof(v), cudaMemcpyDeviceToHost));
  if (raw) *raw = v;
  if (v != 0) {
    GMM_CUDA_TRY(cudaMemset(workspace, 0, sizeof(v)));
    return GMM_ERR_DEVICE_WAIT;
  }
  return GMM_OK;
}

}  // extern "C"
