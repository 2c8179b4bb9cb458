// q/k RMSNorm + partial rotary position encoding + write of K and V into the paged cache, one kernel.
//
// Input is the fused projection row [q | k | v] of every token of the step.  For each token:
//   q, k  <- RMSNorm (none | over all heads of the row | per head), float32
//            (src/quanta/minimax/model_m3.py:15-17 / src/quanta/minimax/attention.py:172-182)
//   q, k  <- rotate-half on the first `rd` dims of each head, pair j using position axis
//            pair_axis[j] and angle float(pos) * inv_freq[j]  (src/quanta/minimax/model_m3.py:83-96)
//   q     -> q_out [T, nq, hd];  k, v -> cache pages [page, kv_head, slot, hd] through the block table
// One rounding to the activation dtype, at the store.  One block per token.
#include "common.cuh"

#define NORM_NONE 0
#define NORM_PER_LAYER 1
#define NORM_PER_HEAD 2

template <typename A>
__global__ void qknorm_rope_write_kernel(
    const A* __restrict__ qkv, A* __restrict__ q_out, A* __restrict__ k_cache, A* __restrict__ v_cache,
    const float* __restrict__ q_norm_w, const float* __restrict__ k_norm_w, int norm_kind, float eps,
    const float* __restrict__ inv_freq, const int* __restrict__ pair_axis,
    const int* __restrict__ positions, int n_axes, const int* __restrict__ tok_pos,
    const int* __restrict__ tok_req, const int* __restrict__ block_table, int bt_stride, int T, int nq,
    int nkv, int hd, int rd, int page_size, int num_pages, int* status) {
  extern __shared__ float smem[];
  const int t = blockIdx.x;
  if (t >= T) return;
  const int qn = nq * hd, kn = nkv * hd;
  float* buf = smem;                 // [qn + kn]  q then k
  float* cs = buf + qn + kn;         // [rd/2] cos, [rd/2] sin
  float* scratch = cs + rd;          // 32 + (nq + nkv) head statistics
  float* head_r = scratch + 32;
  const A* row = qkv + (size_t)t * (qn + 2 * kn);
  const int half = rd / 2;
  // Where this token's K and V go is a chain of three dependent loads (position, request, page id), and the
  // norm gains come from memory that the layer's expert weights have pushed out of L2: both are asked for
  // now, so that their latency passes under the phases below instead of after them.
  int pos = 0, page = -1;
  if (k_cache != nullptr) {
    pos = tok_pos[t];
    page = block_table[(size_t)tok_req[t] * bt_stride + pos / page_size];
  }
  const int n_chunks = (qn + kn) / 8;
  float w_first[8];                  // the gains of this thread's first chunk (NORM_PER_LAYER)
  if (norm_kind == NORM_PER_LAYER && (int)threadIdx.x < n_chunks) {
    const int i = threadIdx.x * 8;
    QbVec8<float>::load(i < qn ? q_norm_w + i : k_norm_w + (i - qn), w_first);
  }

  // 16-byte loads, all of a thread's loads issued before their first use
#pragma unroll 4
  for (int c = threadIdx.x; c < n_chunks; c += blockDim.x) {
    float v[8];
    QbVec8<A>::load(row + c * 8, v);
    QbVec8<float>::store(buf + c * 8, v);
  }
  for (int j = threadIdx.x; j < half; j += blockDim.x) {
    const int ax = pair_axis ? pair_axis[j] : 0;
    const float ang = (float)positions[(size_t)t * n_axes + ax] * inv_freq[j];
    float s, c;
    sincosf(ang, &s, &c);
    cs[j] = c;
    cs[half + j] = s;
  }
  __syncthreads();

  if (norm_kind == NORM_PER_LAYER) {
    // a warp per head, then the heads' sums in head order: the same additions whatever the block size
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    for (int h = warp; h < nq + nkv; h += nwarps) {
      float sh = 0.f;
      for (int d = lane; d < hd; d += 32) sh += buf[h * hd + d] * buf[h * hd + d];
      sh = qb_warp_sum(sh);
      if (lane == 0) head_r[h] = sh;
    }
    __syncthreads();
    float tq = 0.f, tk = 0.f;
    for (int h = 0; h < nq; ++h) tq += head_r[h];
    for (int h = 0; h < nkv; ++h) tk += head_r[nq + h];
    const float rq = rsqrtf(tq / (float)qn + eps), rk = rsqrtf(tk / (float)kn + eps);
#pragma unroll 4
    for (int c = threadIdx.x; c < n_chunks; c += blockDim.x) {
      const int i = c * 8;
      float w[8], v[8];
      if (c == (int)threadIdx.x) {
#pragma unroll
        for (int e = 0; e < 8; ++e) w[e] = w_first[e];
      } else {
        QbVec8<float>::load(i < qn ? q_norm_w + i : k_norm_w + (i - qn), w);
      }
      QbVec8<float>::load(buf + i, v);
      const float r = i < qn ? rq : rk;
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] = w[e] * (v[e] * r);
      QbVec8<float>::store(buf + i, v);
    }
    __syncthreads();
  } else if (norm_kind == NORM_PER_HEAD) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    for (int h = warp; h < nq + nkv; h += nwarps) {
      float s = 0.f;
      for (int d = lane; d < hd; d += 32) s += buf[h * hd + d] * buf[h * hd + d];
      s = qb_warp_sum(s);
      if (lane == 0) head_r[h] = rsqrtf(s / (float)hd + eps);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < qn + kn; i += blockDim.x) {
      const int h = i / hd, d = i % hd;
      const float w = h < nq ? q_norm_w[d] : k_norm_w[d];
      buf[i] = w * (buf[i] * head_r[h]);
    }
    __syncthreads();
  }

  // rotation: each (head, pair) is owned by one thread
  for (int i = threadIdx.x; i < (nq + nkv) * half; i += blockDim.x) {
    const int h = i / half, j = i % half;
    const float a = buf[h * hd + j], b = buf[h * hd + half + j];
    const float c = cs[j], s = cs[half + j];
    buf[h * hd + j] = a * c - b * s;
    buf[h * hd + half + j] = b * c + a * s;
  }
  __syncthreads();

  A* qo = q_out + (size_t)t * qn;
  for (int c = threadIdx.x; c < qn / 8; c += blockDim.x) {
    float v[8];
    QbVec8<float>::load(buf + c * 8, v);
    QbVec8<A>::store(qo + c * 8, v);
  }

  if (k_cache == nullptr) return;
  if (page < 0 || page >= num_pages) {
    if (threadIdx.x == 0) qb_set_status(status, QB_STATUS_BAD_PAGE, page, 2);
    return;
  }
  const int slot = pos % page_size;
  const A* vrow = row + qn + kn;
  for (int c = threadIdx.x; c < kn / 8; c += blockDim.x) {
    const int i = c * 8, h = i / hd, d = i % hd;
    const size_t dst = (((size_t)page * nkv + h) * page_size + slot) * hd + d;
    float kv[8], vv[8];
    QbVec8<float>::load(buf + qn + i, kv);
    QbVec8<A>::load(vrow + i, vv);
    QbVec8<A>::store(k_cache + dst, kv);
    QbVec8<A>::store(v_cache + dst, vv);        // V passes through unchanged (the float round trip is exact)
  }
}

extern "C" int qb_qknorm_rope_write(
    const void* qkv, int dtype, void* q_out, void* k_cache, void* v_cache, const float* q_norm_w,
    const float* k_norm_w, int norm_kind, float eps, const float* inv_freq, const int* pair_axis,
    const int* positions, int n_axes, const int* tok_pos, const int* tok_req, const int* block_table,
    int bt_stride, int T, int nq, int nkv, int hd, int rd, int page_size, int num_pages, int* status,
    cudaStream_t stream) {
  if (T <= 0) return 0;
  if (rd % 2 || rd > hd || rd < 0 || nq <= 0 || nkv <= 0 || page_size <= 0) return QB_ERR_BAD_ARG;
  if (norm_kind != NORM_NONE && (q_norm_w == nullptr || k_norm_w == nullptr)) return QB_ERR_BAD_ARG;
  if (hd % 8) return QB_ERR_UNSUPPORTED;        // rows are moved in 16-byte pieces
  const size_t smem = (size_t)((nq + nkv) * hd + rd + 32 + nq + nkv) * sizeof(float);
  if (smem > 200 * 1024) return QB_ERR_UNSUPPORTED;
  QB_DISPATCH_DTYPE(dtype, A, {
    auto kern = qknorm_rope_write_kernel<A>;
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return (int)e;
    }
    // steps of few tokens: more threads a token, so that each of the kernel's phases is short
    const int threads = T <= 64 ? 1024 : 256;
    kern<<<T, threads, smem, stream>>>((const A*)qkv, (A*)q_out, (A*)k_cache, (A*)v_cache, q_norm_w, k_norm_w,
                                   norm_kind, eps, inv_freq, pair_axis, positions, n_axes, tok_pos, tok_req,
                                   block_table, bt_stride, T, nq, nkv, hd, rd, page_size, num_pages, status);
  });
  QB_LAUNCH_CHECK();
  return 0;
}
