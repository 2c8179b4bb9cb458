// C[M,N] = A[M,K] * B[N,K]^T on the CUDA cores, float32 multiply-add, any M, N, K.
//
// Used where a product must be true 32-bit and independent of the batch: the router logits
// (src/quanta/minimax/moe.py:44, "logits = fp32(x) @ fp32(gate).T").  Every output element is one
// sequential sum over k in a fixed order, so a token's logits are bit-identical however the step is
// cut.  64x64 tile per block, 16-deep k slices in shared memory, 4x4 outputs per thread.  With
// k_chunk > 0 the inner dimension is cut at multiples of k_chunk (independent of M): block z writes
// the partial product of its chunk to C + z*M*ldc, and the consumer adds the partials in index order;
// few rows then still fill the machine.
#include "common.cuh"

constexpr int GS_BM = 64, GS_BN = 64, GS_BK = 16;

template <typename TA, typename TB, typename TC>
__global__ void gemm_nt_simt_kernel(const TA* __restrict__ A, const TB* __restrict__ B, TC* __restrict__ C,
                                    int M, int N, int K, int lda, int ldb, int ldc, int k_chunk) {
  __shared__ float As[GS_BK][GS_BM + 4];
  __shared__ float Bs[GS_BK][GS_BN + 4];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * GS_BM, n0 = blockIdx.x * GS_BN;
  const int tx = tid % 16, ty = tid / 16;       // thread owns rows ty*4.., cols tx*4..
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  const int k_begin = k_chunk > 0 ? blockIdx.z * k_chunk : 0;
  const int k_stop = k_chunk > 0 ? min(K, k_begin + k_chunk) : K;
  C += (size_t)blockIdx.z * M * ldc;
  // 64 rows x 16 k = 1024 elements per operand and slice, 4 per thread; the next slice is fetched into
  // registers while the current one is multiplied
  float ra[4], rb[4];
  auto fetch = [&](int k0) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int idx = tid + e * 256;
      const int r = idx / GS_BK, kk = idx % GS_BK;
      const int gm = m0 + r, gn = n0 + r, gk = k0 + kk;
      ra[e] = (gm < M && gk < k_stop) ? qb_to_float<TA>(A[(size_t)gm * lda + gk]) : 0.f;
      rb[e] = (gn < N && gk < k_stop) ? qb_to_float<TB>(B[(size_t)gn * ldb + gk]) : 0.f;
    }
  };
  fetch(k_begin);
  for (int k0 = k_begin; k0 < k_stop; k0 += GS_BK) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int idx = tid + e * 256;
      As[idx % GS_BK][idx / GS_BK] = ra[e];
      Bs[idx % GS_BK][idx / GS_BK] = rb[e];
    }
    __syncthreads();
    if (k0 + GS_BK < k_stop) fetch(k0 + GS_BK);
#pragma unroll
    for (int kk = 0; kk < GS_BK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gm = m0 + ty * 4 + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tx * 4 + j;
      if (gn < N) C[(size_t)gm * ldc + gn] = qb_from_float<TC>(acc[i][j]);
    }
  }
}

extern "C" int qb_gemm_nt_simt(const void* A, int a_dtype, const void* B, int b_dtype, void* C, int c_dtype,
                               int M, int N, int K, int lda, int ldb, int ldc, int k_chunk,
                               cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || k_chunk < 0 || (k_chunk % GS_BK)) return QB_ERR_BAD_ARG;
  const int splits = k_chunk > 0 ? (K + k_chunk - 1) / k_chunk : 1;
  dim3 grid((N + GS_BN - 1) / GS_BN, (M + GS_BM - 1) / GS_BM, splits);
  QB_DISPATCH_DTYPE(a_dtype, TA, QB_DISPATCH_DTYPE(b_dtype, TB, QB_DISPATCH_DTYPE(c_dtype, TC, {
    gemm_nt_simt_kernel<TA, TB, TC><<<grid, 256, 0, stream>>>((const TA*)A, (const TB*)B, (TC*)C, M, N, K,
                                                              lda, ldb, ldc, k_chunk);
  })));
  QB_LAUNCH_CHECK();
  return 0;
}
