// The grouped product of a mixture of experts on CUDA cores, 32-bit accumulation with FFMA, k ascending:
//
//   C[pos, :] = act( A[src(pos), :] * W[expert(pos)]^T )
//
// Rows are in the order that jv_moe_align made: tiles of TILE rows, a tile all of one expert
// (tile_expert[tile], -1: nothing to do).  `gather` (sorted_token) names the row of A for a row of C (-1: padding,
// the row of C is left alone), or is null: row pos of A.  act: none, or the exact gelu 0.5 z (1 + erf(z / sqrt 2)).
// This is the product of the 32-bit path and of sizes that the tensor-core product does not take.
#include "common.cuh"
#include <math.h>

namespace {
constexpr int BM = 32, BN = 64, BK = 16;    // BM is the row tile that jv_moe_align pads to

template <typename TA, typename TW, typename TC>
__global__ void __launch_bounds__(256) moe_gemm_simt_kernel(const TA* __restrict__ A, int lda, const int* __restrict__ gather,
                                                            int a_rows, const TW* __restrict__ W, size_t w_expert_stride,
                                                            int ldw, const int* __restrict__ tile_expert,
                                                            TC* __restrict__ C, int ldc, int N, int K, int act,
                                                            int* __restrict__ status) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  __shared__ int src[BM];
  pdl_trigger();
  pdl_wait();
  const int e = tile_expert[blockIdx.y];
  if (e < 0) return;
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;     // 16 x 16 threads: 2 rows x 4 columns each
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  if (tid < BM) {
    int r = gather ? gather[m0 + tid] : m0 + tid;
    if (r >= a_rows) { atomicOr(status, JV_STATUS_BAD_ROW); r = -1; }
    src[tid] = r;
  }
  __syncthreads();
  const TW* We = W + (size_t)e * w_expert_stride;
  float acc[2][4];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int idx = tid + i * 256;
      const int row = idx >> 4, kk = idx & 15;
      const int k = k0 + kk;
      float a = 0.f;
      if (k < K && src[row] >= 0) a = to_f32(A[(size_t)src[row] * lda + k]);
      As[kk][row] = a;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int idx = tid + i * 256;
      const int row = idx >> 4, kk = idx & 15;
      const int k = k0 + kk;
      float w = 0.f;
      if (k < K && n0 + row < N) w = to_f32(We[(size_t)(n0 + row) * ldw + k]);
      Ws[kk][row] = w;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[2], w[4];
#pragma unroll
      for (int i = 0; i < 2; ++i) a[i] = As[kk][ty * 2 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) w[j] = Ws[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int m = ty * 2 + i;
    if (src[m] < 0) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= N) continue;
      float v = acc[i][j];
      if (act == 1) v = 0.5f * v * (1.f + erff(v * 0.70710678118654752f));
      C[(size_t)(m0 + m) * ldc + n] = from_f32<TC>(v);
    }
  }
}
}  // namespace

JV_EXPORT int jv_moe_gemm_simt_tile() { return BM; }

// A: rows of lda elements (a_rows of them); gather: [max_tiles * BM] or null; W: [experts][N, K] rows of ldw,
// experts w_expert_stride elements apart; C: [max_tiles * BM, N] rows of ldc.
JV_EXPORT int jv_moe_gemm_simt(const void* A, int a_dtype, int lda, const int* gather, int a_rows, const void* W,
                               int w_dtype, long long w_expert_stride, int ldw, const int* tile_expert, int max_tiles,
                               void* C, int c_dtype, int ldc, int N, int K, int act, int* status, cudaStream_t stream) {
  if (max_tiles == 0 || N == 0) return JV_OK;
  dim3 grid((N + BN - 1) / BN, max_tiles);
  if (grid.y > 65535) return JV_ERR_UNSUPPORTED;
  JV_DISPATCH_DTYPE(a_dtype, TA, JV_DISPATCH_DTYPE(w_dtype, TW, JV_DISPATCH_DTYPE(c_dtype, TC,
      return jv_launch(moe_gemm_simt_kernel<TA, TW, TC>, grid, dim3(256), 0, stream, (const TA*)A, lda, gather, a_rows,
                       (const TW*)W, (size_t)w_expert_stride, ldw, tile_expert, (TC*)C, ldc, N, K, act, status))));
  return JV_ERR_UNSUPPORTED;
}
