/*
 * grouped_mm_b200 — C ABI of the B200 (sm_100a) grouped GEMM library, libgrouped_mm_b200.so.
 *
 * This is the drop-in boundary for the forward path of lostmsu/grouped_mm_bf16: the four
 * functions that the reference's api.py imports from kernels.py and calls with a pre-allocated
 * output (grouped_mm_bf16/api.py:8-17, call sites api.py:195,201,207,213). Each entry point
 * below names the reference function it replaces. Conventions, identical to the reference's:
 * the caller owns every buffer; `out` is written in place; element strides are honoured as
 * given; the call only enqueues work on the given CUDA stream of the current device and never
 * synchronises with the host, so `offs` is read on the device only.
 *
 * Plain C: pointers and integers only, no C++ or torch types. Every function returns 0 on
 * success or a negative gmm_status code; gmm_error_string() turns a code into text.
 */
#ifndef GROUPED_MM_B200_H_
#define GROUPED_MM_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define GMM_ABI_VERSION 2

/* Element types (reference: _as_tl_dtype, grouped_mm_bf16/kernels.py:175-182). */
enum gmm_dtype { GMM_BF16 = 0, GMM_F16 = 1, GMM_F32 = 2 };

enum gmm_status {
  GMM_OK = 0,
  GMM_ERR_INVALID_ARGUMENT = -1, /* null pointer, bad rank, negative size, mismatched shapes */
  GMM_ERR_UNSUPPORTED_DTYPE = -2,
  GMM_ERR_TOO_MANY_GROUPS = -3,  /* more than 1023 groups (reference: api.py:115-116) */
  GMM_ERR_WORKSPACE = -4,        /* workspace missing, misaligned or smaller than gmm_workspace_bytes() */
  GMM_ERR_CUDA = -5,             /* a CUDA runtime/driver call failed; see gmm_last_cuda_error() */
  GMM_ERR_NOT_SM100 = -6,        /* the current device is not compute capability 10.x */
  GMM_ERR_DEVICE_WAIT = -7,      /* a bounded wait inside a kernel gave up (reported by gmm_check_status) */
  GMM_ERR_NOT_FUSABLE = -8       /* grouped_mm_2d3d_swiglu: operands the tensor-core path cannot address */
};

/* Which kernel a call is routed to. */
enum gmm_kernel_kind {
  GMM_KERNEL_NONE = 0,    /* nothing to launch (empty problem) */
  GMM_KERNEL_TCGEN05 = 1,      /* TMA + tcgen05.mma persistent kernel, one CTA per 128 x 256 tile */
  GMM_KERNEL_GENERIC = 2,      /* any-stride fp32-FMA kernel */
  GMM_KERNEL_TCGEN05_PAIR = 3  /* TMA + tcgen05.mma.cta_group::2 kernel, a CTA pair per 256 x 256 tile */
};

/* Flags for gmm_launch_t.flags. */
#define GMM_FLAG_FORCE_GENERIC 0x1u /* route to the generic kernel even where the TMA path applies */
#define GMM_FLAG_FORCE_PAIR 0x2u    /* tcgen05 path: always use the CTA-pair (cta_group::2) kernel if legal */
#define GMM_FLAG_NO_PAIR 0x4u       /* tcgen05 path: never use the CTA-pair kernel */
/* fp32 operands with an fp32 result may be multiplied as TF32 on the tensor cores (fp32 accumulate).
 * Without it fp32 operands are multiplied in true fp32. Counterpart of the reference's ALLOW_TF32
 * kernel argument, which it takes from torch.backends.cuda.matmul.allow_tf32
 * (grouped_mm_bf16/kernels.py:185-194, 242). */
#define GMM_FLAG_ALLOW_TF32 0x8u

/*
 * A 2-D or 3-D strided tensor in device memory. Sizes and strides are in elements, outermost
 * dimension first, exactly as torch reports them (the reference passes mat.stride(i) straight
 * to its kernels: grouped_mm_bf16/kernels.py:535-543).
 */
typedef struct gmm_tensor {
  void* data;
  int32_t dtype; /* enum gmm_dtype */
  int32_t ndim;  /* 2 or 3 */
  int64_t size[3];
  int64_t stride[3];
} gmm_tensor_t;

/*
 * Launch context. `workspace` is device memory owned by the caller, at least
 * gmm_workspace_bytes() long and 256-byte aligned, zero-filled once when it is allocated; it
 * may be reused by every later call on the same device. Its first 32-bit word is the device
 * status word read by gmm_check_status().
 */
typedef struct gmm_launch {
  void* stream; /* cudaStream_t; NULL = the legacy default stream */
  void* workspace;
  size_t workspace_bytes;
  uint32_t flags;
  /*
   * grouped_mm_2d2d() on the tensor-core path only; NULL / 0 for every other call. Device memory,
   * 128-byte aligned, at least gmm_group_maps_bytes(n_groups) long, contents irrelevant: the call
   * first writes one tensor map per group and operand there (each bounded at that group's end of
   * the ragged K dimension, so that TMA fills what a group's last block reads past its end with
   * zeros) and its GEMM kernel then loads through them. The buffer must stay untouched until the
   * call's work on `stream` has finished, and calls that may be in flight at the same time need
   * separate buffers. Without it such a call returns GMM_ERR_WORKSPACE.
   */
  void* group_maps;
  size_t group_maps_bytes;
} gmm_launch_t;

int gmm_abi_version(void);
const char* gmm_error_string(int status);
/* Text of the last CUDA error seen by the calling thread inside this library ("" if none). */
const char* gmm_last_cuda_error(void);
size_t gmm_workspace_bytes(void);
/* Size of gmm_launch_t.group_maps for a grouped_mm_2d2d() call with n_groups groups (0 if n_groups < 1). */
size_t gmm_group_maps_bytes(int32_t n_groups);

/*
 * out[g] = a[g] @ b[g]; a [G,M,K], b [G,K,N], out [G,M,N].
 * Replaces grouped_mm_3d3d(mat_a, mat_b, out), grouped_mm_bf16/kernels.py:524-550.
 */
int grouped_mm_3d3d(const gmm_tensor_t* a, const gmm_tensor_t* b, const gmm_tensor_t* out,
                    const gmm_launch_t* launch);

/*
 * out[g] = a[:, ks:ke] @ b[ks:ke, :] with [ks,ke) = [offs[g-1], offs[g]); a [M,K_total],
 * b [K_total,N], out [G,M,N]; an empty range stores zeros.
 * Replaces grouped_mm_2d2d(mat_a, mat_b, offs, out), grouped_mm_bf16/kernels.py:553-580.
 */
int grouped_mm_2d2d(const gmm_tensor_t* a, const gmm_tensor_t* b, const int32_t* offs, int32_t n_groups,
                    const gmm_tensor_t* out, const gmm_launch_t* launch);

/*
 * out[r,:] = a[r,:] @ b[g(r)] where group g owns rows [offs[g-1], offs[g]); a [M_total,K],
 * b [G,K,N], out [M_total,N]. Rows at or past offs[G-1] are left untouched.
 * Replaces grouped_mm_2d3d(mat_a, mat_b, offs, out), grouped_mm_bf16/kernels.py:583-686.
 */
int grouped_mm_2d3d(const gmm_tensor_t* a, const gmm_tensor_t* b, const int32_t* offs, int32_t n_groups,
                    const gmm_tensor_t* out, const gmm_launch_t* launch);

/*
 * out[:,c] = a[g(c)] @ b[:,c] where group g owns columns [offs[g-1], offs[g]); a [G,M,K],
 * b [K,N_total], out [M,N_total]. Columns at or past offs[G-1] are left untouched.
 * Replaces grouped_mm_3d2d(mat_a, mat_b, offs, out), grouped_mm_bf16/kernels.py:689-717.
 */
int grouped_mm_3d2d(const gmm_tensor_t* a, const gmm_tensor_t* b, const int32_t* offs, int32_t n_groups,
                    const gmm_tensor_t* out, const gmm_launch_t* launch);

/*
 * The gated up-projection of an MoE feed-forward block in one pass:
 *   out[r,:] = silu(a[r,:] @ gate[g(r)]) * (a[r,:] @ up[g(r)])
 * with b_gate_up [G,K,2N] holding gate in columns [0,N) and up in [N,2N) of every group (the usual
 * fused "gate_up" weight), a [M_total,K], out [M_total,N], offs as for grouped_mm_2d3d. Both
 * products accumulate in fp32 and the activation is evaluated on the fp32 accumulators, so the
 * result is rounded once; the [M_total,2N] intermediate never reaches memory.
 *
 * No counterpart in the reference, whose callers run grouped_mm_2d3d and then an element-wise
 * kernel. Tensor-core path only: 16-bit operands, 16-byte aligned bases and pitches, row-major a,
 * N a multiple of 8 when b is row-major. Anything else returns GMM_ERR_NOT_FUSABLE and launches
 * nothing; the caller then uses grouped_mm_2d3d followed by its own activation.
 */
int grouped_mm_2d3d_swiglu(const gmm_tensor_t* a, const gmm_tensor_t* b_gate_up, const int32_t* offs,
                           int32_t n_groups, const gmm_tensor_t* out, const gmm_launch_t* launch);

/*
 * grouped_mm_2d3d() for callers that cannot provide a workspace because they cannot allocate
 * device memory: code running after an application has handed all device memory to its own
 * arena, plugin hosts that forbid allocations once initialisation is over, and latency-critical
 * loops that must never enter the allocator (cudaMalloc and cudaFree also synchronise the whole
 * device). Same arguments and results as grouped_mm_2d3d(); the 256-byte scratch block (status
 * word first) lives in a fixed array inside the library image instead, held by every GPU that
 * loads the library until the process exits. This call allocates nothing and calls no allocating
 * routine. No counterpart in the reference.
 *
 *  - Limit: the scratch is 256 bytes, which covers every problem grouped_mm_2d3d() accepts (the
 *    scratch need of the row-ragged form does not grow with the problem; the library checks this
 *    at compile time). The group limit (n_groups <= 1023) is unchanged.
 *  - The first call on each device looks up the array's device address (cudaGetSymbolAddress, with
 *    that device current). Make that first call before any stream capture is begun.
 *  - All calls on a device share the one block, which keeps what the last call left in it. The
 *    arguments are checked first; a call that is rejected, or has no work, touches nothing. A call
 *    that launches clears the status word (the only part that must start at zero) on `stream`
 *    just before its kernel, so a status code that an earlier call left there and nobody read with
 *    gmm_check_status() is lost at that point. Calls that overlap on the GPU (different streams)
 *    race on the status word and must be avoided or serialised by the caller.
 *  - *scratch_address, when not NULL, receives the block's device address, usable as the
 *    `workspace` argument of gmm_check_status().
 */
int grouped_mm_2d3d_static_scratch(const gmm_tensor_t* a, const gmm_tensor_t* b, const int32_t* offs,
                                   int32_t n_groups, const gmm_tensor_t* out, void* stream, uint32_t flags,
                                   void** scratch_address);

/*
 * Zero-fills the elements of a 2-D tensor whose index along the ragged dimension is at or past
 * offs[n_groups - 1] (clamped into [0, extent]; everything when n_groups is 0). `extent` and
 * `stride_ragged` describe the ragged dimension, `other` and `stride_other` the remaining one;
 * sizes and strides in elements of `elem_bytes` (2 or 4) bytes. The grouped_mm_* calls leave that
 * part of their output untouched; a gradient needs zeros there. The offset is read on the device
 * and nothing is written when it equals `extent`. The reference's backward kernels zero these
 * elements as part of their own stores (grouped_mm_bf16/kernels.py:1093-1390).
 */
int gmm_zero_past_offsets(void* data, int32_t elem_bytes, int64_t extent, int64_t other, int64_t stride_ragged,
                          int64_t stride_other, const int32_t* offs, int32_t n_groups, void* stream);

/*
 * Which kernel the corresponding grouped_mm_* call would use for these arguments (enum
 * gmm_kernel_kind, or a negative gmm_status). `form`: 0 = 3d3d, 1 = 2d3d, 2 = 3d2d, 3 = 2d2d.
 * Launches nothing. No counterpart in the reference, whose kernels take any strides.
 */
int gmm_select_kernel(int32_t form, const gmm_tensor_t* a, const gmm_tensor_t* b, const gmm_tensor_t* out,
                      uint32_t flags);

/*
 * Waits for `stream`, reads the status word of `workspace` and clears it. Returns GMM_OK, or
 * GMM_ERR_DEVICE_WAIT if a kernel gave up on a bounded wait (its outputs are then invalid);
 * *raw, when not NULL, receives the device code. Diagnostic only: the forward calls never
 * need it. No counterpart in the reference, whose device code reports no errors.
 */
int gmm_check_status(void* workspace, void* stream, int32_t* raw);

/*
 * Launches a one-CTA kernel that waits, for at most `budget_cycles` SM clocks (1 .. 4e9), on a
 * barrier nothing completes. The wait gives up, writes code 0x7E57 to the status word of
 * `workspace` and the kernel returns normally; gmm_check_status() then reports
 * GMM_ERR_DEVICE_WAIT. It exercises, without any real failure, the give-up path that every
 * bounded wait inside the GEMM kernels takes. No counterpart in the reference.
 */
int gmm_selftest_wait_timeout(void* workspace, void* stream, int64_t budget_cycles);

/* ------------------------------------------------------------------------------------------
 * Caller-side MoE steps around the 2D x 3D form: from per-token expert choices to the grouped row
 * order and back. The reference does the first step on the host in its benchmark only
 * (expert ids -> torch.bincount -> cumsum -> int32 offs, bench/bench_2d3d.py:131-138) and has no
 * counterpart for the others. All of it runs on the device here, with no host synchronisation.
 * "Assignment" i = (token i / topk, choice i % topk); ids outside [0, n_experts) are not routed.
 */

/* Bytes of device workspace gmm_route_build() needs (0 for invalid arguments). */
size_t gmm_route_workspace_bytes(int64_t n_assignments, int32_t n_experts);

/*
 * Stable counting sort of the assignments by expert.
 *   offs[e]     END offset of expert e's rows (int32, n_experts entries): grouped_mm's `offs`
 *   perm[p]     assignment placed at sorted position p (-1 past the last routed assignment)
 *   inv_perm[i] sorted position of assignment i, -1 if not routed (may be NULL)
 * Inside an expert, rows keep the order of their assignment index.
 */
int gmm_route_build(const int32_t* expert_ids, int64_t n_assignments, int32_t n_experts, int32_t* offs,
                    int32_t* perm, int32_t* inv_perm, void* workspace, size_t workspace_bytes, void* stream);

/* dst row r = src row perm[r] / topk for r < n_out_rows; rows whose perm entry is -1 are left untouched. */
int gmm_permute_rows(const void* src, int64_t src_rows, int64_t row_bytes, int64_t src_stride_bytes,
                     const int32_t* perm, int32_t topk, void* dst, int64_t dst_stride_bytes, int64_t n_out_rows,
                     void* stream);

/*
 * out[t, :] = sum over k < topk of weights[t * topk + k] * y[inv_perm[t * topk + k], :], accumulated
 * in fp32 (weights NULL = all ones; unrouted choices are skipped). Strides in elements.
 */
int gmm_combine_rows(const void* y, int32_t y_dtype, int64_t y_stride, const int32_t* inv_perm, const float* weights,
                     int32_t topk, int64_t n_tokens, int32_t n_cols, void* out, int32_t out_dtype, int64_t out_stride,
                     void* stream);

/*
 * Expert-parallel dispatch and combine over peer memory (no counterpart in the reference, which is
 * single-GPU). `peers` is a DEVICE array of n_peers base pointers, entry i the buffer of rank i as
 * mapped into this process (the caller sets the mapping up: CUDA IPC, fabric handles, symmetric
 * memory), this rank's own buffer included; every buffer has capacity_rows rows. Rank and row of
 * every transfer come from index tables in device memory; an index outside [0, n_peers) x
 * [0, capacity_rows) is skipped and GMM_STATUS_BAD_PEER_INDEX is or-ed into *status (a device word).
 * Neither call waits for the host or for another GPU: the caller puts a collective on the stream
 * between "all ranks have scattered" and the first read of the received rows, and again between
 * "all ranks have produced their results" and the combine.
 *
 * gmm_scatter_rows_to_peers: for r < n_rows with perm[r] >= 0 and dst_rank[r] >= 0,
 *   row dst_row[r] of peers[dst_rank[r]]  =  src row perm[r] / topk      (strides in bytes)
 * gmm_combine_rows_from_peers: out[t, :] = sum over k < topk of
 *   weights[t*topk + k] * (row src_row[t*topk + k] of peers[src_rank[t*topk + k]]),
 *   entries with src_rank < 0 skipped, fp32 accumulation (y_stride, out_stride in elements).
 */
#define GMM_STATUS_BAD_PEER_INDEX 0x40000000

int gmm_scatter_rows_to_peers(const void* src, int64_t src_rows, int64_t row_bytes, int64_t src_stride_bytes,
                              const int32_t* perm, int32_t topk, const int32_t* dst_rank, const int32_t* dst_row,
                              void* const* peers, int32_t n_peers, int64_t dst_stride_bytes, int64_t capacity_rows,
                              int64_t n_rows, int32_t* status, void* stream);

int gmm_combine_rows_from_peers(const void* const* peers, int32_t n_peers, int32_t y_dtype, int64_t y_stride,
                                int64_t capacity_rows, const int32_t* src_rank, const int32_t* src_row,
                                const float* weights, int32_t topk, int64_t n_tokens, int32_t n_cols, void* out,
                                int32_t out_dtype, int64_t out_stride, int32_t* status, void* stream);

#ifdef __cplusplus
}
#endif

#endif /* GROUPED_MM_B200_H_ */
