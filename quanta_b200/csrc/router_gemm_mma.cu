// Router logits of many tokens on the tensor cores, to float32 accuracy:
//   logits[t, e] = sum_k x[t, k] * gate[e, k],  x bfloat16, gate float32.
//
// The float32 gate is held as THREE bfloat16 matrices hi + mid + lo (each the bfloat16 rounding of what
// the ones before leave over: 3 x 8 mantissa bits carry the 24 of a float32), so every product
// x * piece is exact in float32 and the sum runs in the float32 accumulators of mma.m16n8k16.  The inner
// dimension is taken in chunks of 64: a chunk's sum starts from zero and is then added to the running
// total, in chunk order, whatever the number of tokens, so a token's logits do not depend on the step.
// The inner dimension is also cut into ranges of RG_KSPLIT (a constant), one block a range, whose sums
// come out side by side, [ranges][T][E]; the selection kernel adds them in range order.
// (src/quanta/minimax/moe.py:44, "logits = fp32(x) @ fp32(gate).T".)  Prompt portions use this kernel;
// steps of few tokens keep the SIMT kernel, which reads the float32 gate once.
//
// Block = 128 tokens x 64 experts, eight warps of 32 tokens x 32 experts each (a fragment of the gate serves
// two fragments of tokens); operands come through shared memory in two stages filled by cp.async.  Needs K % 8 == 0 (16-byte rows).
#include "common.cuh"

namespace {

constexpr int RG_BM = 128, RG_BN = 64, RG_BK = 64, RG_PAD = 8, RG_LD = RG_BK + RG_PAD, RG_THREADS = 256;
constexpr int RG_KSPLIT = 768;      // inner-dimension range of one block: a multiple of RG_BK

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;      // 0 source bytes: the 16 destination bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(dst)), "l"(src), "r"(n));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// pieces: [3][E][K] bfloat16
__global__ void __launch_bounds__(RG_THREADS)
router_gemm_mma_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ pieces,
                       float* __restrict__ logits, int T, int E, int K) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(smem_raw);            // [2][RG_BM][RG_LD]
  __nv_bfloat16* ws = xs + 2 * RG_BM * RG_LD;                                // [2][3][RG_BN][RG_LD]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int t0 = blockIdx.y * RG_BM, e0 = blockIdx.x * RG_BN;
  const int k_begin = blockIdx.z * RG_KSPLIT, k_end = min(K, k_begin + RG_KSPLIT);
  const int n_stages = (k_end - k_begin + RG_BK - 1) / RG_BK;
  const int wt = warp & 3, we = warp >> 2;      // this warp's 32 tokens and 32 experts of the block's
  logits += (size_t)blockIdx.z * T * E;

  auto fetch = [&](int stage, int buf) {
    const int k0 = k_begin + stage * RG_BK;
    // 64 rows x 8 chunks of 16 bytes per operand
    for (int c = tid; c < RG_BM * (RG_BK / 8); c += RG_THREADS) {
      const int r = c / (RG_BK / 8), kc = (c % (RG_BK / 8)) * 8;
      const bool ok = t0 + r < T && k0 + kc < K;
      cp_async16(xs + ((size_t)buf * RG_BM + r) * RG_LD + kc, ok ? x + (size_t)(t0 + r) * K + k0 + kc : x, ok);
    }
    for (int c = tid; c < 3 * RG_BN * (RG_BK / 8); c += RG_THREADS) {
      const int p = c / (RG_BN * (RG_BK / 8)), rem = c % (RG_BN * (RG_BK / 8));
      const int r = rem / (RG_BK / 8), kc = (rem % (RG_BK / 8)) * 8;
      const bool ok = e0 + r < E && k0 + kc < K;
      cp_async16(ws + (((size_t)buf * 3 + p) * RG_BN + r) * RG_LD + kc,
                 ok ? pieces + ((size_t)p * E + e0 + r) * K + k0 + kc : pieces, ok);
    }
    asm volatile("cp.async.commit_group;\n" ::);
  };

  constexpr int NT = RG_BN / 2 / 8;             // accumulator tiles of 8 experts a warp
  constexpr int MT = 2;                         // fragments of 16 tokens a warp
  float total[MT][NT][4];
#pragma unroll
  for (int m = 0; m < MT; ++m)
#pragma unroll
    for (int i = 0; i < NT; ++i) total[m][i][0] = total[m][i][1] = total[m][i][2] = total[m][i][3] = 0.f;

  fetch(0, 0);
  for (int s = 0; s < n_stages; ++s) {
    const int buf = s & 1;
    if (s + 1 < n_stages) {
      fetch(s + 1, buf ^ 1);
      asm volatile("cp.async.wait_group 1;\n" ::);
    } else {
      asm volatile("cp.async.wait_group 0;\n" ::);
    }
    __syncthreads();
    float acc[MT][NT][4];
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
      for (int i = 0; i < NT; ++i) acc[m][i][0] = acc[m][i][1] = acc[m][i][2] = acc[m][i][3] = 0.f;
    const __nv_bfloat16* xa = xs + ((size_t)buf * RG_BM + wt * 16 * MT) * RG_LD;
#pragma unroll
    for (int kk = 0; kk < RG_BK / 16; ++kk) {
      uint32_t a[MT][4];
#pragma unroll
      for (int m = 0; m < MT; ++m)
        ldmatrix_x4(a[m], xa + (size_t)(m * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * RG_LD + kk * 16 + 8 * (lane >> 4));
#pragma unroll
      for (int np = 0; np < NT / 2; ++np) {
#pragma unroll
        for (int p = 0; p < 3; ++p) {         // hi, then mid, then lo
          const __nv_bfloat16* wb = ws + (((size_t)buf * 3 + p) * RG_BN + we * (RG_BN / 2) + np * 16) * RG_LD;
          uint32_t b[4];
          ldmatrix_x4(b, wb + (size_t)((lane & 7) + 8 * (lane >> 4)) * RG_LD + kk * 16 + 8 * ((lane >> 3) & 1));
#pragma unroll
          for (int m = 0; m < MT; ++m) {
            mma16816(acc[m][2 * np], a[m], b[0], b[1]);
            mma16816(acc[m][2 * np + 1], a[m], b[2], b[3]);
          }
        }
      }
    }
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
      for (int i = 0; i < NT; ++i) {
        total[m][i][0] += acc[m][i][0]; total[m][i][1] += acc[m][i][1];
        total[m][i][2] += acc[m][i][2]; total[m][i][3] += acc[m][i][3];
      }
    __syncthreads();
  }
  // accumulator element: row (lane >> 2) + 8 * (i >> 1), column nt * 8 + (lane & 3) * 2 + (i & 1)
  const int g = lane >> 2, q = lane & 3;
#pragma unroll
  for (int m = 0; m < MT; ++m)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int t = t0 + wt * 16 * MT + m * 16 + g + 8 * (i >> 1), e = e0 + we * (RG_BN / 2) + nt * 8 + q * 2 + (i & 1);
        if (t < T && e < E) logits[(size_t)t * E + e] = total[m][nt][i];
      }
}

// out[p][i] = the p-th bfloat16 piece of w[i]: hi, mid, lo
__global__ void split3_kernel(const float* __restrict__ w, __nv_bfloat16* __restrict__ out, size_t n) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const float v = w[i];
    const __nv_bfloat16 hi = __float2bfloat16_rn(v);
    const float r1 = v - __bfloat162float(hi);
    const __nv_bfloat16 mid = __float2bfloat16_rn(r1);
    const float r2 = r1 - __bfloat162float(mid);
    out[i] = hi;
    out[n + i] = mid;
    out[2 * n + i] = __float2bfloat16_rn(r2);
  }
}

}  // namespace

// w float32 [n] -> out bfloat16 [3][n]
extern "C" int qb_split3_bf16(const float* w, void* out, long long n, cudaStream_t stream) {
  if (n <= 0) return 0;
  const int blocks = (int)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096);
  split3_kernel<<<blocks, 256, 0, stream>>>(w, (__nv_bfloat16*)out, (size_t)n);
  QB_LAUNCH_CHECK();
  return 0;
}

// how many ranges the inner dimension is cut into: the first size of the logits
extern "C" int qb_router_gemm_mma_parts(int K) { return K <= 0 ? 0 : (K + RG_KSPLIT - 1) / RG_KSPLIT; }

// x bf16 [T, K]; pieces bf16 [3, E, K] (qb_split3_bf16 of the float32 gate); logits float32 [parts, T, E]
extern "C" int qb_router_gemm_mma(const void* x, const void* pieces, float* logits, int T, int E, int K,
                                  cudaStream_t stream) {
  if (T <= 0 || E <= 0) return 0;
  if (K <= 0 || K % 8) return QB_ERR_UNSUPPORTED;
  if ((((uintptr_t)x | (uintptr_t)pieces) & 15) != 0) return QB_ERR_UNSUPPORTED;
  const size_t smem = (size_t)(2 * RG_BM + 2 * 3 * RG_BN) * RG_LD * sizeof(__nv_bfloat16);
  cudaError_t err = cudaFuncSetAttribute(router_gemm_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (err != cudaSuccess) return (int)err;
  dim3 grid((E + RG_BN - 1) / RG_BN, (T + RG_BM - 1) / RG_BM, (K + RG_KSPLIT - 1) / RG_KSPLIT);
  if (grid.y > 65535 || grid.z > 65535) return QB_ERR_UNSUPPORTED;
  router_gemm_mma_kernel<<<grid, RG_THREADS, smem, stream>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)pieces,
                                                            logits, T, E, K);
  QB_LAUNCH_CHECK();
  return 0;
}
