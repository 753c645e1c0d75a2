// C[M, N] = A[M, K] * W[N, K]^T in true float32 on the CUDA cores (no tensor-core mode of any
// kind): the matrix product of the 32-bit path.  Each output element is one chain of fused
// multiply-adds over k = 0..K-1 in ascending order, whatever M is and wherever the row falls in
// a tile, so a token's result does not depend on what else is in the batch, bit for bit.
//
// It stands where 12vivi/tandem runs torch.nn.functional.linear on float32 tensors
// (python/tandem/layers/linear.py:14; python/tandem/models/llama_family.py:115).
#include "common.cuh"

namespace tb {

constexpr int BM = 64, BN = 64, BK = 16;

// 256 threads; thread (ty, tx) of a 16x16 grid owns rows ty*4..+3 and columns tx*4..+3 of the tile.
__global__ void __launch_bounds__(256) gemm_f32_kernel(const float* __restrict__ A, const float* __restrict__ W,
                                                        float* __restrict__ C, int M, int N, int K, int lda,
                                                        int ldc) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[4][4] = {};
  // loader: thread reads 4 consecutive k of one row: row = tid / 4 (0..63), k = (tid % 4) * 4
  const int lrow = tid >> 2, lk = (tid & 3) * 4;
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int k = k0 + lk + i;
      const int am = m0 + lrow, wn = n0 + lrow;
      As[lk + i][lrow] = (am < M && k < K) ? A[(size_t)am * lda + k] : 0.f;
      Ws[lk + i][lrow] = (wn < N && k < K) ? W[(size_t)wn * K + k] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[4], w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { a[i] = As[k][ty * 4 + i]; w[i] = Ws[k][tx * 4 + i]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < N) C[(size_t)m * ldc + n] = acc[i][j];
    }
  }
}

}  // namespace tb

extern "C" int tb_gemm_f32(void* stream, const float* A, const float* W, float* C, int M, int N, int K, int lda,
                           int ldc) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || lda < K || ldc < N) return TB_ERR_BAD_SIZE;
  dim3 grid((N + tb::BN - 1) / tb::BN, (M + tb::BM - 1) / tb::BM);
  return tb::launch(tb::gemm_f32_kernel, grid, dim3(256), 0, stream, A, W, C, M, N, K, lda, ldc);
}
