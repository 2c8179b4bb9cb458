// Embedding gather and RMSNorm fused with the residual sum.
//
// The residual stream h is float32 in both precisions.  A layer's output ("delta") is not added to h
// by the layer itself: the next norm adds it (in float32, slots in index order) while it reads the
// row anyway, writes the new h and the normed row.  One thread block owns one token row, so a row's
// numbers never depend on the rest of the batch.
#include "common.cuh"

// ---------------------------------------------------------------------------------------------
// h[t,:] = float(table[ids[t],:])     (reference: src/quanta/minimax/model.py:91)
// ---------------------------------------------------------------------------------------------
template <typename W>
__global__ void embedding_kernel(float* __restrict__ h, const W* __restrict__ table,
                                 const int* __restrict__ ids, int T, int H, int V, int* status) {
  const int t = blockIdx.x;
  if (t >= T) return;
  const int id = ids[t];
  float* out = h + (size_t)t * H;
  if (id < 0 || id >= V) {
    if (threadIdx.x == 0) qb_set_status(status, QB_STATUS_BAD_TOKEN, id, 1);
    for (int i = threadIdx.x; i < H; i += blockDim.x) out[i] = 0.f;
    return;
  }
  const W* row = table + (size_t)id * H;
  if (H % 8 == 0) {
    for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
      float v[8];
      QbVec8<W>::load(row + i, v);
      QbVec8<float>::store(out + i, v);
    }
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x) out[i] = qb_to_float<W>(row[i]);
  }
}

extern "C" int qb_embedding(float* h, const void* table, int table_dtype, const int* ids, int T, int H,
                            int V, int* status, cudaStream_t stream) {
  if (T <= 0) return 0;
  QB_DISPATCH_DTYPE(table_dtype, W,
                    embedding_kernel<W><<<T, 256, 0, stream>>>(h, (const W*)table, ids, T, H, V, status));
  QB_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------------------------
// row r (token rows[r] if rows != null, else r):
//   x = h[tok,:] + sum_s delta[tok,s,:]          (float32, s ascending)
//   if store_h: h[tok,:] = x
//   out[r,:] = w * (x * rsqrt(mean(x^2) + eps))  (reference: src/quanta/minimax/model_m3.py:60-65)
// out may be null (only fold the delta into h).  The row is held in shared memory between the passes.
// ---------------------------------------------------------------------------------------------
template <typename D, typename O>
__global__ void add_rmsnorm_kernel(float* __restrict__ h, const D* __restrict__ delta, int S,
                                   const float* __restrict__ w, O* __restrict__ out,
                                   const int* __restrict__ rows, int n_rows, int H, float eps,
                                   int store_h) {
  extern __shared__ float row_buf[];      // H floats + 32 scratch
  float* scratch = row_buf + H;
  const int r = blockIdx.x;
  if (r >= n_rows) return;
  const int tok = rows ? rows[r] : r;
  float* hrow = h + (size_t)tok * H;
  const D* drow = delta ? delta + (size_t)tok * S * H : nullptr;
  float ss = 0.f;
  // the gains of this thread's first chunk are asked for now: they come from memory that the layer's weights
  // have pushed out of L2, and would else be waited for after the row's sum
  float w_first[8];
  if (H % 8 == 0 && out != nullptr && (int)threadIdx.x * 8 < H) QbVec8<float>::load(w + threadIdx.x * 8, w_first);
  if (H % 8 == 0) {
    // 8 elements a thread and step, vector loads; the slots of the delta are still added in index order
    for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
      float x[8];
      QbVec8<float>::load(hrow + i, x);
      if (drow) {
#pragma unroll 8
        for (int s = 0; s < S; ++s) {
          float dv[8];
          QbVec8<D>::load(drow + (size_t)s * H + i, dv);
#pragma unroll
          for (int e = 0; e < 8; ++e) x[e] += dv[e];
        }
        if (store_h) QbVec8<float>::store(hrow + i, x);
      }
      QbVec8<float>::store(row_buf + i, x);
#pragma unroll
      for (int e = 0; e < 8; ++e) ss += x[e] * x[e];
    }
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      float x = hrow[i];
      if (drow) {
        for (int s = 0; s < S; ++s) x += qb_to_float<D>(drow[(size_t)s * H + i]);
      }
      row_buf[i] = x;
      if (store_h && drow) hrow[i] = x;
      ss += x * x;
    }
  }
  const float total = qb_block_sum(ss, scratch);
  if (out == nullptr) return;
  const float r_inv = rsqrtf(total / (float)H + eps);
  O* orow = out + (size_t)r * H;
  if (H % 8 == 0) {
    for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
      float x[8], wv[8];
      QbVec8<float>::load(row_buf + i, x);
      if (i == (int)threadIdx.x * 8) {
#pragma unroll
        for (int e = 0; e < 8; ++e) wv[e] = w_first[e];
      } else {
        QbVec8<float>::load(w + i, wv);
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) x[e] = wv[e] * (x[e] * r_inv);
      QbVec8<O>::store(orow + i, x);
    }
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x)
      orow[i] = qb_from_float<O>(w[i] * (row_buf[i] * r_inv));
  }
}

extern "C" int qb_add_rmsnorm(float* h, const void* delta, int delta_dtype, int S, const float* w,
                              void* out, int out_dtype, const int* rows, int n_rows, int H, float eps,
                              int store_h, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  const size_t smem = (size_t)(H + 32) * sizeof(float);
  if (smem > 200 * 1024) return QB_ERR_UNSUPPORTED;
  const int threads = H >= 2048 ? 512 : 256;
  QB_DISPATCH_DTYPE(delta_dtype, D, QB_DISPATCH_DTYPE(out_dtype, O, {
    auto kern = add_rmsnorm_kernel<D, O>;
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return (int)e;
    }
    kern<<<n_rows, threads, smem, stream>>>(h, (const D*)delta, S, w, (O*)out, rows, n_rows, H, eps,
                                            store_h);
  }));
  QB_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------------------------
// out[r,:] = silu(gu[r, 0:I]) * gu[r, I:2I]     (dense SwiGLU feed-forward; float32 inside)
// ---------------------------------------------------------------------------------------------
template <typename A>
__global__ void silu_mul_kernel(const A* __restrict__ gu, A* __restrict__ out, int n_rows, int I) {
  const size_t n = (size_t)n_rows * I;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / I, c = i % I;
    const float g = qb_to_float<A>(gu[r * 2 * I + c]);
    const float u = qb_to_float<A>(gu[r * 2 * I + I + c]);
    out[i] = qb_from_float<A>(g / (1.f + expf(-g)) * u);
  }
}

extern "C" int qb_silu_mul(const void* gu, void* out, int dtype, int n_rows, int I, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  const size_t n = (size_t)n_rows * I;
  const int blocks = (int)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096);
  QB_DISPATCH_DTYPE(dtype, A, silu_mul_kernel<A><<<blocks, 256, 0, stream>>>((const A*)gu, (A*)out, n_rows, I));
  QB_LAUNCH_CHECK();
  return 0;
}
