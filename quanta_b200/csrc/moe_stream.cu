// Routed experts for few rows per expert: a weight-streaming product on the tensor cores.
//
// In decoding every expert sees a handful of token rows, so the step is bound by reading each chosen
// expert's weights once.  Here the WEIGHTS are the 16-row operand of mma.m16n8k16 and the token rows
// are the 8-column operand ("swap A/B"): a warp loads weight rows straight from global memory into
// the A fragment with 16-byte loads (no shared-memory staging, each byte read once), the few token
// rows sit in shared memory, and the accumulators hold [16 output features x 8 tokens] in float32.
// A thread's 16-byte load covers 8 consecutive k, which it feeds to two MMAs as k-slots
// {2q,2q+1,2q+8,2q+9}; the token operand is loaded with the same rule, so the permutation of k inside
// a 32-wide block cancels.
//
// Block = 4 warps = one expert x 16 output features; the inner dimension is split over the warps in
// a fixed way and the partial sums are added in warp order, so a row's result does not depend on
// what else the expert received.  Rows beyond 8*NT per expert are handled in further passes.
//
//   MODE 1: act[p, j] = silu(W13_e[j] . x[tok(p)]) * (W13_e[I + j] . x[tok(p)])       (bf16 out)
//   MODE 2: y[pair(p), n] = w[pair(p)] * (W2_e[n] . act[p])                            (float32 out)
// (src/quanta/minimax/moe.py:59-88.)  Needs K % 8 == 0 (16-byte rows); other sizes use the SIMT path.
#include "common.cuh"

constexpr int MS_WARPS = 4;
constexpr int MS_ROWS = 16;     // output features per block

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ld_stream16(const void* p) {
  uint4 v;
  asm("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

template <int MODE, int NT>
__global__ void __launch_bounds__(MS_WARPS * 32)
moe_stream_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ weights,
                  void* __restrict__ out, const int* __restrict__ sorted_pair, const float* __restrict__ pair_w,
                  const int* __restrict__ plan, int E, int top_k, int K, int N, int smem_rows, int x_stride) {
  constexpr int NM = MODE == 1 ? 2 : 1;           // weight matrices per output feature (gate and up)
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(smem_raw);                     // [smem_rows][x_stride]
  float* red = reinterpret_cast<float*>(smem_raw + (size_t)smem_rows * x_stride * 2);  // [MS_WARPS-1][32][NM*NT*4]
  __shared__ int src_row[NT * 8];

  const int num_active = plan[3 * E + 2];
  if ((int)blockIdx.y >= num_active) return;
  const int e = plan[3 * E + 4 + blockIdx.y];
  const int* offsets = plan + 2 * E;
  const int row0 = offsets[e], n_rows = offsets[e + 1] - row0;
  const int j0 = blockIdx.x * MS_ROWS;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, q = lane & 3;

  // the warp's share of the inner dimension, in whole 32-wide blocks
  const int k_blocks = (K + 31) / 32;
  const int per_warp = (k_blocks + MS_WARPS - 1) / MS_WARPS;
  const int kb_begin = warp * per_warp, kb_end = min(k_blocks, kb_begin + per_warp);

  const __nv_bfloat16* wbase = weights + (size_t)e * NM * N * K;
  const int ra = j0 + g, rb = j0 + g + 8;                         // the two feature rows of this thread
  const bool ra_ok = ra < N, rb_ok = rb < N;
  const __nv_bfloat16* wrow[NM][2];
#pragma unroll
  for (int m = 0; m < NM; ++m) {
    wrow[m][0] = wbase + ((size_t)m * N + (ra_ok ? ra : 0)) * K;
    wrow[m][1] = wbase + ((size_t)m * N + (rb_ok ? rb : 0)) * K;
  }

  for (int pass0 = 0; pass0 < n_rows; pass0 += NT * 8) {
    const int rows_here = min(NT * 8, n_rows - pass0);
    if (tid < NT * 8) {
      int r = -1;
      if (tid < rows_here) {
        const int p = row0 + pass0 + tid;
        r = MODE == 1 ? sorted_pair[p] / top_k : p;
      }
      src_row[tid] = r;
    }
    __syncthreads();
    // each warp stages its own k-range of the token rows (zero rows past the end)
    const int k_lo = kb_begin * 32, k_hi = min(K, kb_end * 32);
    for (int r = 0; r < min(smem_rows, NT * 8); ++r) {
      const int sr = src_row[r];
      for (int k = k_lo + lane * 8; k < kb_end * 32; k += 256) {
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (sr >= 0 && k < k_hi) v = *reinterpret_cast<const uint4*>(x + (size_t)sr * K + k);
        *reinterpret_cast<uint4*>(xs + (size_t)r * x_stride + k) = v;
      }
    }
    __syncwarp();

    float acc[NM][NT][4];
#pragma unroll
    for (int m = 0; m < NM; ++m)
#pragma unroll
      for (int t = 0; t < NT; ++t)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[m][t][i] = 0.f;

    // Weights are fetched a group of U k-blocks ahead of the MMAs that use them, in two register
    // buffers, so that a thread always has a group of 16-byte loads in flight.
    constexpr int U = MODE == 1 ? 2 : 4;
    uint4 bufA[U][NM][2], bufB[U][NM][2];
    auto fetch = [&](uint4 (&buf)[U][NM][2], int kb0) {
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int k = (kb0 + u) * 32 + q * 8;
        const bool k_ok = kb0 + u < kb_end && k < K;
#pragma unroll
        for (int m = 0; m < NM; ++m) {
          buf[u][m][0] = (k_ok && ra_ok) ? ld_stream16(wrow[m][0] + k) : make_uint4(0u, 0u, 0u, 0u);
          buf[u][m][1] = (k_ok && rb_ok) ? ld_stream16(wrow[m][1] + k) : make_uint4(0u, 0u, 0u, 0u);
        }
      }
    };
    auto consume = [&](const uint4 (&buf)[U][NM][2], int kb0) {
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (kb0 + u >= kb_end) break;
        const int k = (kb0 + u) * 32 + q * 8;
#pragma unroll
        for (int t = 0; t < NT; ++t) {
          const int xr = t * 8 + g;
          uint4 xb = make_uint4(0u, 0u, 0u, 0u);
          if (xr < smem_rows) xb = *reinterpret_cast<const uint4*>(xs + (size_t)xr * x_stride + k);
#pragma unroll
          for (int m = 0; m < NM; ++m) {
            mma_bf16_16816(acc[m][t], buf[u][m][0].x, buf[u][m][1].x, buf[u][m][0].y, buf[u][m][1].y, xb.x, xb.y);
            mma_bf16_16816(acc[m][t], buf[u][m][0].z, buf[u][m][1].z, buf[u][m][0].w, buf[u][m][1].w, xb.z, xb.w);
          }
        }
      }
    };
    fetch(bufA, kb_begin);
    for (int kb = kb_begin; kb < kb_end; kb += 2 * U) {
      fetch(bufB, kb + U);
      consume(bufA, kb);
      fetch(bufA, kb + 2 * U);
      consume(bufB, kb + U);
    }

    // partial sums of warps 1.. go through shared memory and are added in warp order by warp 0
    constexpr int PER = NM * NT * 4;
    if (warp > 0) {
      float* dst = red + ((size_t)(warp - 1) * 32 + lane) * PER;
#pragma unroll
      for (int m = 0; m < NM; ++m)
#pragma unroll
        for (int t = 0; t < NT; ++t)
#pragma unroll
          for (int i = 0; i < 4; ++i) dst[(m * NT + t) * 4 + i] = acc[m][t][i];
    }
    __syncthreads();
    if (warp == 0) {
      for (int w = 1; w < MS_WARPS; ++w) {
        const float* src = red + ((size_t)(w - 1) * 32 + lane) * PER;
#pragma unroll
        for (int m = 0; m < NM; ++m)
#pragma unroll
          for (int t = 0; t < NT; ++t)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[m][t][i] += src[(m * NT + t) * 4 + i];
      }
      // accumulator element i: feature row (i < 2 ? ra : rb), token column t*8 + q*2 + (i & 1)
#pragma unroll
      for (int t = 0; t < NT; ++t)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int feat = i < 2 ? ra : rb;
          const int col = t * 8 + q * 2 + (i & 1);
          if (feat >= N || col >= rows_here) continue;
          const int p = row0 + pass0 + col;
          if (MODE == 1) {
            const float gv = acc[0][t][i], uv = acc[NM - 1][t][i];
            reinterpret_cast<__nv_bfloat16*>(out)[(size_t)p * N + feat] =
                __float2bfloat16_rn(gv / (1.f + expf(-gv)) * uv);
          } else {
            const int pair = sorted_pair[p];
            reinterpret_cast<float*>(out)[(size_t)pair * N + feat] = pair_w[pair] * acc[0][t][i];
          }
        }
    }
    __syncthreads();
  }
}

// x: bf16 [T, K] (mode 1) or [pairs, K] (mode 2); weights bf16 [E, (mode 1 ? 2 : 1) * N, K].
// max_rows: the most rows one expert can have in this step (the number of tokens).
extern "C" int qb_moe_stream(int mode, const void* x, const void* weights, void* out, const int* sorted_pair,
                             const float* pair_w, const int* plan, int E, int top_k, int K, int N, int max_active,
                             int max_rows, cudaStream_t stream) {
  if (max_active <= 0) return 0;
  if (K % 8 || K <= 0 || N <= 0) return QB_ERR_UNSUPPORTED;
  if (max_active > 65535) return QB_ERR_UNSUPPORTED;
  const int nt = max_rows <= 8 ? 1 : 2;
  const int smem_rows = max_rows < nt * 8 ? max_rows : nt * 8;
  const int k_pad = ((K + 31) / 32 + MS_WARPS - 1) / MS_WARPS * MS_WARPS * 32;   // every warp's range is staged whole
  const int x_stride = k_pad + 32;              // +64 bytes a row: the 8 lanes of a 16-byte load phase hit distinct banks
  const int nm = mode == 1 ? 2 : 1;
  const size_t smem = (size_t)smem_rows * x_stride * 2 + (size_t)(MS_WARPS - 1) * 32 * nm * nt * 4 * sizeof(float);
  if (smem > 200 * 1024) return QB_ERR_UNSUPPORTED;
  dim3 grid((N + MS_ROWS - 1) / MS_ROWS, max_active);
#define QB_STREAM(MODE_, NT_)                                                                               \
  do {                                                                                                      \
    auto kern = moe_stream_kernel<MODE_, NT_>;                                                              \
    if (smem > 48 * 1024) {                                                                                 \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);   \
      if (e != cudaSuccess) return (int)e;                                                                  \
    }                                                                                                       \
    kern<<<grid, MS_WARPS * 32, smem, stream>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)weights, out, \
                                                sorted_pair, pair_w, plan, E, top_k, K, N, smem_rows, x_stride); \
  } while (0)
  if (mode == 1 && nt == 1) QB_STREAM(1, 1);
  else if (mode == 1) QB_STREAM(1, 2);
  else if (mode == 2 && nt == 1) QB_STREAM(2, 1);
  else if (mode == 2) QB_STREAM(2, 2);
  else return QB_ERR_BAD_ARG;
#undef QB_STREAM
  QB_LAUNCH_CHECK();
  return 0;
}
