/*
 * Plain-C restatement of grouped_mm on dense row-major fp32 arrays — TEST INFRASTRUCTURE.
 *
 * An independent second opinion for oracle/grouped_mm_oracle.py (which leans on torch.matmul):
 * three nested loops, double accumulation, one rounding to float. It follows the reference's
 * group ownership rule (group g owns [offs[g-1], offs[g]) with int32 END offsets, clamped to the
 * extent: grouped_mm_bf16/kernels.py:162-172, 339) and its output shapes
 * (grouped_mm_bf16/api.py:134-149). 16-bit inputs are widened to fp32 by the caller (exact).
 *
 * form: 0 = 3d3d  a[G,M,K] b[G,K,N] -> c[G,M,N]
 *       1 = 2d3d  a[M,K]   b[G,K,N] -> c[M,N]      (M = total rows, ragged by offs)
 *       2 = 3d2d  a[G,M,K] b[K,N]   -> c[M,N]      (N = total columns, ragged by offs)
 *       3 = 2d2d  a[M,K]   b[K,N]   -> c[G,M,N]    (K = total contraction, ragged by offs)
 * Elements owned by no group are left as they are. Returns 0, or -1 for a bad argument.
 */
#include <stddef.h>
#include <stdint.h>

static int clampi(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }

static void mm(const float* a, size_t lda, const float* b, size_t ldb, float* c, size_t ldc, int m, int n, int k) {
  for (int i = 0; i < m; ++i)
    for (int j = 0; j < n; ++j) {
      double acc = 0.0;
      for (int p = 0; p < k; ++p) acc += (double)a[(size_t)i * lda + p] * (double)b[(size_t)p * ldb + j];
      c[(size_t)i * ldc + j] = (float)acc;
    }
}

int gmm_oracle_f32(int form, int G, int M, int N, int K, const float* a, const float* b, const int32_t* offs,
                   float* c) {
  if (G < 0 || M < 0 || N < 0 || K < 0 || !c) return -1;
  if (form != 0 && G > 0 && !offs) return -1;
  if (form == 0) {
    for (int g = 0; g < G; ++g)
      mm(a + (size_t)g * M * K, K, b + (size_t)g * K * N, N, c + (size_t)g * M * N, N, M, N, K);
    return 0;
  }
  int start = 0;
  for (int g = 0; g < G; ++g) {
    const int extent = form == 1 ? M : (form == 2 ? N : K);
    const int end = clampi(offs[g], 0, extent);
    const int len = end > start ? end - start : 0;
    if (form == 1) {
      if (len) mm(a + (size_t)start * K, K, b + (size_t)g * K * N, N, c + (size_t)start * N, N, len, N, K);
    } else if (form == 2) {
      if (len) mm(a + (size_t)g * M * K, K, b + start, N, c + start, N, M, len, K);
    } else if (form == 3) {
      /* an empty range stores zeros: mm with k = 0 does exactly that */
      mm(a + start, K, b + (size_t)start * N, N, c + (size_t)g * M * N, N, M, N, len);
    } else {
      return -1;
    }
    start = end;
  }
  return 0;
}
