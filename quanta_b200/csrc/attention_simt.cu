// Paged causal attention over the cache, plain SIMT version (float32 arithmetic throughout).
//
// This is the kernel of the true 32-bit path, and the reference the tensor-core kernels are checked
// against.  Every token of the step is its own problem: token t of request r at absolute position p
// attends the keys [lo, p] of r's pages (lo = 0, or p-window+1 for a windowed layer), whatever else is
// in the batch, so prompt portions and single decoded tokens run in one launch.  K and V of the
// step's own tokens have been written to the pages before this kernel runs.
//
//   s = (q . k) * scale;  softmax over keys in float32;  out = P V
//   (src/quanta/minimax/attention.py:194-203; grouped heads: q head h reads kv head h / (nq/nkv))
//
// One warp per (token, q head): lanes own keys for the scores, then own dims for P V.
#include "common.cuh"

template <typename A> struct Vec16;
template <> struct Vec16<float> {
  static constexpr int N = 4;
  __device__ static void load(const float* p, float* o) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
  }
};
template <> struct Vec16<__nv_bfloat16> {
  static constexpr int N = 8;
  __device__ static void load(const __nv_bfloat16* p, float* o) {
    const uint4 v = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      o[2 * i] = __uint_as_float(w[i] << 16);
      o[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
};

constexpr int ATT_WARPS = 4;
constexpr int ATT_MAX_HD = 256;

template <typename A>
__global__ void paged_attention_simt_kernel(
    const A* __restrict__ q, const A* __restrict__ k_cache, const A* __restrict__ v_cache,
    A* __restrict__ out, const int* __restrict__ tok_pos, const int* __restrict__ tok_req,
    const int* __restrict__ block_table, int bt_stride, int T, int nq, int nkv, int hd, int page_size,
    int num_pages, float scale, int window, int* status) {
  extern __shared__ float qs_all[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long wid = (long)blockIdx.x * ATT_WARPS + warp;
  if (wid >= (long)T * nq) return;
  const int t = (int)(wid / nq), h = (int)(wid % nq);
  const int kvh = h / (nq / nkv);
  float* qs = qs_all + warp * hd;
  const A* qrow = q + ((size_t)t * nq + h) * hd;
  for (int d = lane; d < hd; d += 32) qs[d] = qb_to_float<A>(qrow[d]);
  __syncwarp();

  const int pos = tok_pos[t];
  const int* bt = block_table + (size_t)tok_req[t] * bt_stride;
  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;

  float m = -INFINITY, l = 0.f;
  float acc[ATT_MAX_HD / 32];
#pragma unroll
  for (int i = 0; i < ATT_MAX_HD / 32; ++i) acc[i] = 0.f;

  for (int kb = lo - (lo & 31); kb <= pos; kb += 32) {
    const int key = kb + lane;
    const bool valid = key >= lo && key <= pos;
    float s = -INFINITY;
    long base = -1;     // element offset of this lane's key row (K and V share the layout)
    if (valid) {
      const int page = bt[key / page_size];
      if (page < 0 || page >= num_pages) {
        qb_set_status(status, QB_STATUS_BAD_PAGE, page, 3);
      } else {
        base = (((long)page * nkv + kvh) * page_size + key % page_size) * hd;
        const A* kp = k_cache + base;
        float dot = 0.f;
        for (int d = 0; d < hd; d += Vec16<A>::N) {
          float kv[Vec16<A>::N];
          Vec16<A>::load(kp + d, kv);
#pragma unroll
          for (int i = 0; i < Vec16<A>::N; ++i) dot += qs[d + i] * kv[i];
        }
        s = dot * scale;
      }
    }
    const float mb = qb_warp_max(s);
    if (mb == -INFINITY) continue;
    const float m_new = fmaxf(m, mb);
    const float p = (base >= 0) ? expf(s - m_new) : 0.f;
    const float corr = expf(m - m_new);
    l = l * corr + qb_warp_sum(p);
#pragma unroll
    for (int i = 0; i < ATT_MAX_HD / 32; ++i) acc[i] *= corr;
    const int n_here = min(32, pos - kb + 1);
    for (int j = 0; j < n_here; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
      const long bj = __shfl_sync(0xffffffffu, base, j);
      if (bj < 0) continue;
      const A* vp = v_cache + bj;
#pragma unroll
      for (int i = 0; i < ATT_MAX_HD / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < hd) acc[i] += pj * qb_to_float<A>(vp[d]);
      }
    }
    m = m_new;
  }
  A* orow = out + ((size_t)t * nq + h) * hd;
  const float inv_l = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
  for (int i = 0; i < ATT_MAX_HD / 32; ++i) {
    const int d = lane + 32 * i;
    if (d < hd) orow[d] = qb_from_float<A>(acc[i] * inv_l);
  }
}

extern "C" int qb_paged_attention_simt(const void* q, int dtype, const void* k_cache, const void* v_cache,
                                       void* out, const int* tok_pos, const int* tok_req,
                                       const int* block_table, int bt_stride, int T, int nq, int nkv, int hd,
                                       int page_size, int num_pages, float scale, int window, int* status,
                                       cudaStream_t stream) {
  if (T <= 0) return 0;
  if (hd % 16 || hd > ATT_MAX_HD || nq % nkv || page_size <= 0) return QB_ERR_UNSUPPORTED;
  const long warps = (long)T * nq;
  const int blocks = (int)((warps + ATT_WARPS - 1) / ATT_WARPS);
  const size_t smem = (size_t)ATT_WARPS * hd * sizeof(float);
  QB_DISPATCH_DTYPE(dtype, A,
                    paged_attention_simt_kernel<A><<<blocks, ATT_WARPS * 32, smem, stream>>>(
                        (const A*)q, (const A*)k_cache, (const A*)v_cache, (A*)out, tok_pos, tok_req,
                        block_table, bt_stride, T, nq, nkv, hd, page_size, num_pages, scale, window, status));
  QB_LAUNCH_CHECK();
  return 0;
}
