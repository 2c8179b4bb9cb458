// Sampling on the device: one thread block per logits row.
//
//   temperature <= 0: greedy, the first maximum (src/quanta/minimax/generate.py:71-72)
//   else lg = logits / temperature; top-k keeps lg >= k-th largest; top-p keeps a token while the
//   mass strictly before it (descending order) is < p; min-p drops p < min_p * p_max
//   (src/quanta/minimax/generate.py:34-53, 74-79); then a categorical draw.
// The draw is the Gumbel-max rule, argmax(lg + g), with g from a counter-based generator
// (Philox-4x32-10) keyed by the request's seed and indexed by (token, draw number): a request's
// draws depend on nothing else in the batch.  Penalties over earlier generated tokens
// (src/quanta/shim/omlx.py:344-363) are a separate in-place kernel.
#include "common.cuh"

constexpr int SAMP_THREADS = 1024;

__device__ __forceinline__ uint32_t order_key(float x) {
  const uint32_t b = __float_as_uint(x);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ __forceinline__ uint32_t philox_word0(uint32_t c0, uint32_t c1, uint32_t k0, uint32_t k1) {
  uint32_t c2 = 0, c3 = 0;
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
    const uint32_t n0 = hi1 ^ c1 ^ k0, n2 = hi0 ^ c3 ^ k1;
    c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
    k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
  }
  return c0;
}

__device__ __forceinline__ float gumbel(uint32_t token, uint32_t draw, uint32_t k0, uint32_t k1) {
  const uint32_t r = philox_word0(token, draw, k0, k1);
  float u = (float)(((double)r + 0.5) * 2.3283064365386963e-10);
  u = fminf(u, 1.f - 5.9604644775390625e-8f);
  return -logf(-logf(u));
}

struct ArgBest { float v; int i; };

// first maximum over the block; every thread gets the result
__device__ __forceinline__ ArgBest block_argmax(float v, int i, float* sv, int* si) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, i, o);
    if (oi >= 0 && (i < 0 || ov > v || (ov == v && oi < i))) { v = ov; i = oi; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) { sv[warp] = v; si[warp] = i; }
  __syncthreads();
  ArgBest b{sv[0], si[0]};
  for (int w = 1; w < (int)(blockDim.x >> 5); ++w) {
    if (si[w] >= 0 && (b.i < 0 || sv[w] > b.v || (sv[w] == b.v && si[w] < b.i))) { b.v = sv[w]; b.i = si[w]; }
  }
  return b;
}

// Descending radix search over 32-bit keys.  Finds the key at which the running total (count or
// mass, taken from the largest key downwards) first reaches `target`.  `floor_key`: only keys >=
// floor_key take part.  Returns the key on every thread.
template <bool MASS>
__device__ uint32_t radix_threshold(const float* __restrict__ row, int V, float inv_t, float m, float target,
                                    uint32_t floor_key, float* hist, uint32_t* s_prefix, float* s_above) {
  uint32_t prefix = 0;
  float above = 0.f;
  for (int level = 0; level < 4; ++level) {
    const int shift = 24 - 8 * level;
    const uint32_t hi_mask = level == 0 ? 0u : (0xffffffffu << (shift + 8));
    for (int b = threadIdx.x; b < 256; b += blockDim.x) hist[b] = 0.f;
    __syncthreads();
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float lg = row[i] * inv_t;
      const uint32_t key = order_key(lg);
      if (key < floor_key || (key & hi_mask) != prefix) continue;
      atomicAdd(&hist[(key >> shift) & 255u], MASS ? expf(lg - m) : 1.f);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      float run = above;
      int pick = 0;
      for (int b = 255; b >= 0; --b) {
        if (run + hist[b] >= target) { pick = b; break; }
        run += hist[b];
        if (b == 0) { pick = 0; run -= hist[0]; }
      }
      *s_prefix = prefix | ((uint32_t)pick << shift);
      *s_above = run;
    }
    __syncthreads();
    prefix = *s_prefix;
    above = *s_above;
    __syncthreads();
  }
  return prefix;
}

__global__ void sample_rows_kernel(const float* __restrict__ logits, int V, const float* __restrict__ fparams,
                                   const int* __restrict__ iparams, int* __restrict__ out) {
  __shared__ float sv[32];
  __shared__ int si[32];
  __shared__ float hist[256];
  __shared__ uint32_t s_prefix;
  __shared__ float s_above;
  const int r = blockIdx.x;
  const float* row = logits + (size_t)r * V;
  // null parameters: every row is greedy
  const float temperature = fparams ? fparams[r * 4 + 0] : 0.f;
  const float top_p = fparams ? fparams[r * 4 + 1] : 1.f, min_p = fparams ? fparams[r * 4 + 2] : 0.f;
  const int top_k = iparams ? iparams[r * 4 + 0] : 0;
  const uint32_t k0 = iparams ? (uint32_t)iparams[r * 4 + 1] : 0u, k1 = iparams ? (uint32_t)iparams[r * 4 + 2] : 0u;
  const uint32_t draw = iparams ? (uint32_t)iparams[r * 4 + 3] : 0u;

  if (temperature <= 0.f) {
    float bv = -INFINITY; int bi = -1;
    for (int i = threadIdx.x; i < V; i += blockDim.x)
      if (bi < 0 || row[i] > bv) { bv = row[i]; bi = i; }
    const ArgBest b = block_argmax(bv, bi, sv, si);
    if (threadIdx.x == 0) out[r] = b.i;
    return;
  }
  const float inv_t = 1.f / temperature;
  float bv = -INFINITY; int bi = -1;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float lg = row[i] * inv_t;
    if (bi < 0 || lg > bv) { bv = lg; bi = i; }
  }
  const float m = block_argmax(bv, bi, sv, si).v;
  uint32_t floor_key = 0u;
  if (top_k > 0 && top_k < V)
    floor_key = radix_threshold<false>(row, V, inv_t, m, (float)top_k, 0u, hist, &s_prefix, &s_above);
  if (top_p > 0.f && top_p < 1.f) {
    float z = 0.f;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float lg = row[i] * inv_t;
      if (order_key(lg) >= floor_key) z += expf(lg - m);
    }
    const float Z = qb_block_sum(z, sv);
    __syncthreads();
    const uint32_t kp = radix_threshold<true>(row, V, inv_t, m, top_p * Z, floor_key, hist, &s_prefix, &s_above);
    floor_key = max(floor_key, kp);
  }
  const float min_lg = min_p > 0.f ? m + logf(min_p) : -INFINITY;
  bv = -INFINITY; bi = -1;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float lg = row[i] * inv_t;
    if (order_key(lg) < floor_key || lg < min_lg) continue;
    const float v = lg + gumbel((uint32_t)i, draw, k0, k1);
    if (bi < 0 || v > bv) { bv = v; bi = i; }
  }
  const ArgBest b = block_argmax(bv, bi, sv, si);
  if (threadIdx.x == 0) out[r] = b.i;
}

// fparams [n,4]: temperature, top_p, min_p, -.  iparams [n,4]: top_k, seed low word, seed high word, draw.
extern "C" int qb_sample_rows(const float* logits, int n, int V, const float* fparams, const int* iparams,
                              int* out, cudaStream_t stream) {
  if (n <= 0) return 0;
  sample_rows_kernel<<<n, SAMP_THREADS, 0, stream>>>(logits, V, fparams, iparams, out);
  QB_LAUNCH_CHECK();
  return 0;
}

// Greedy over many blocks: a row of a large vocabulary is cut into `parts` chunks, each block leaves the
// first maximum of its chunk, and a second kernel takes the first maximum of those (chunks in index order,
// so the result is the first maximum of the row, whatever `parts`).
__global__ void argmax_partial_kernel(const float* __restrict__ logits, int V, int parts, float* __restrict__ pv,
                                      int* __restrict__ pi) {
  __shared__ float sv[32];
  __shared__ int si[32];
  const int r = blockIdx.y, part = blockIdx.x;
  const int chunk = (V + parts - 1) / parts;
  const int lo = part * chunk, hi = min(V, lo + chunk);
  const float* row = logits + (size_t)r * V;
  float bv = -INFINITY; int bi = -1;
  for (int i = lo + threadIdx.x; i < hi; i += blockDim.x)
    if (bi < 0 || row[i] > bv) { bv = row[i]; bi = i; }
  const ArgBest b = block_argmax(bv, bi, sv, si);
  if (threadIdx.x == 0) { pv[r * parts + part] = b.v; pi[r * parts + part] = b.i; }
}

__global__ void argmax_final_kernel(const float* __restrict__ pv, const int* __restrict__ pi, int parts,
                                    int* __restrict__ out) {
  const int r = blockIdx.x;
  if (threadIdx.x != 0) return;
  float bv = -INFINITY; int bi = -1;
  for (int p = 0; p < parts; ++p) {
    const int i = pi[r * parts + p];
    const float v = pv[r * parts + p];
    if (i >= 0 && (bi < 0 || v > bv)) { bv = v; bi = i; }
  }
  out[r] = bi;
}

// scratch: parts floats and parts ints per row
extern "C" int qb_argmax_rows(const float* logits, int n, int V, int parts, float* scratch_v, int* scratch_i,
                              int* out, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (parts <= 0 || n > 65535) return QB_ERR_BAD_ARG;
  argmax_partial_kernel<<<dim3(parts, n), 256, 0, stream>>>(logits, V, parts, scratch_v, scratch_i);
  argmax_final_kernel<<<n, 32, 0, stream>>>(scratch_v, scratch_i, parts, out);
  QB_LAUNCH_CHECK();
  return 0;
}

// Penalties, in place on a float32 logits row.  prev[prev_off[r] .. prev_off[r+1]) are the tokens the
// request has generated.  The first occurrence of a token applies the penalty with its full count.
// pparams [n,3]: repetition, frequency, presence.
__global__ void penalties_kernel(float* __restrict__ logits, int V, const int* __restrict__ prev,
                                 const int* __restrict__ prev_off, const float* __restrict__ pparams) {
  const int r = blockIdx.x;
  const float rep = pparams[r * 3 + 0], freq = pparams[r * 3 + 1], pres = pparams[r * 3 + 2];
  if (rep == 1.f && freq == 0.f && pres == 0.f) return;
  const int lo = prev_off[r], hi = prev_off[r + 1];
  float* row = logits + (size_t)r * V;
  for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    const int tok = prev[i];
    if (tok < 0 || tok >= V) continue;
    bool first = true;
    for (int j = lo; j < i; ++j)
      if (prev[j] == tok) { first = false; break; }
    if (!first) continue;
    int count = 0;
    for (int j = i; j < hi; ++j) count += prev[j] == tok;
    float x = row[tok];
    if (rep != 1.f) x = x > 0.f ? x / rep : x * rep;
    row[tok] = x - (float)count * freq - pres;
  }
}

extern "C" int qb_apply_penalties(float* logits, int n, int V, const int* prev, const int* prev_off,
                                  const float* pparams, cudaStream_t stream) {
  if (n <= 0) return 0;
  penalties_kernel<<<n, 256, 0, stream>>>(logits, V, prev, prev_off, pparams);
  QB_LAUNCH_CHECK();
  return 0;
}
