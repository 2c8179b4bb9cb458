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
//
// A row's options (temperature, top-k, top-p, min-p, seed) and the number of its draw come from the
// state slot of its request (request_state.h); the kernel counts the draw there and leaves the token.
// The thresholds of top-k and top-p come from histograms of integers (counts; probabilities in fixed
// point, 2^-40 of the largest), so their sums do not depend on the order in which threads add: the
// same row always keeps the same set.
#include "common.cuh"
#include "request_state.h"

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
// floor_key take part.  Totals are integers (MASS: exp(lg - m) * 2^40, at most 2^40 each, so 2^24
// of them fit), added with integer atomics: exact, whatever the order.  target == 0 with MASS asks
// for the total of all keys first (top-p of the mass that top-k left): target = frac * total.
// Returns the key on every thread.
constexpr double SAMP_FIXED_ONE = 1099511627776.0;      // 2^40

template <bool MASS>
__device__ uint32_t radix_threshold(const float* __restrict__ row, int V, float inv_t, float m, double frac_or_count,
                                    uint32_t floor_key, unsigned long long* hist, uint32_t* s_prefix,
                                    unsigned long long* s_above, unsigned long long* s_target) {
  uint32_t prefix = 0;
  unsigned long long above = 0ull;
  for (int level = 0; level < 4; ++level) {
    const int shift = 24 - 8 * level;
    const uint32_t hi_mask = level == 0 ? 0u : (0xffffffffu << (shift + 8));
    for (int b = threadIdx.x; b < 256; b += blockDim.x) hist[b] = 0ull;
    __syncthreads();
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float lg = row[i] * inv_t;
      const uint32_t key = order_key(lg);
      if (key < floor_key || (key & hi_mask) != prefix) continue;
      const unsigned long long add = MASS ? (unsigned long long)((double)expf(lg - m) * SAMP_FIXED_ONE) : 1ull;
      atomicAdd(&hist[(key >> shift) & 255u], add);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      if (level == 0) {
        if (MASS) {
          unsigned long long total = 0ull;
          for (int b = 0; b < 256; ++b) total += hist[b];
          const unsigned long long t = (unsigned long long)(frac_or_count * (double)total);
          *s_target = t > 0ull ? t : 1ull;              // the largest key is always kept
        } else {
          *s_target = (unsigned long long)frac_or_count;
        }
      }
      const unsigned long long target = *s_target;
      unsigned long long run = above;
      int pick = 0;
      for (int b = 255; b >= 0; --b) {
        // a key is kept while the total strictly before it is below the target: the search stops at the
        // first bin whose own total carries the sum to the target or past it
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

// slots: the state records (null: every row greedy, nothing recorded); row_slot[r]: the slot of row r.
__global__ void sample_rows_kernel(const float* __restrict__ logits, int V, int* __restrict__ slots,
                                   const int* __restrict__ row_slot, int n_slots, int* __restrict__ out) {
  __shared__ float sv[32];
  __shared__ int si[32];
  __shared__ unsigned long long hist[256];
  __shared__ uint32_t s_prefix;
  __shared__ unsigned long long s_above, s_target;
  const int r = blockIdx.x;
  const float* row = logits + (size_t)r * V;
  int* rec = nullptr;
  if (slots != nullptr) {
    const int slot = row_slot[r];
    if (slot >= 0 && slot < n_slots) rec = slots + (size_t)slot * QB_SLOT_WORDS;
  }
  const float temperature = rec ? __int_as_float(rec[QB_SLOT_TEMPERATURE]) : 0.f;
  const float top_p = rec ? __int_as_float(rec[QB_SLOT_TOP_P]) : 1.f;
  const float min_p = rec ? __int_as_float(rec[QB_SLOT_MIN_P]) : 0.f;
  const int top_k = rec ? rec[QB_SLOT_TOP_K] : 0;
  const uint32_t k0 = rec ? (uint32_t)rec[QB_SLOT_SEED_LO] : 0u, k1 = rec ? (uint32_t)rec[QB_SLOT_SEED_HI] : 0u;
  const uint32_t draw = rec ? (uint32_t)rec[QB_SLOT_DRAWN] : 0u;
  __syncthreads();                  // every thread has read the record before thread 0 changes it

  int token;
  if (temperature <= 0.f) {
    float bv = -INFINITY; int bi = -1;
    for (int i = threadIdx.x; i < V; i += blockDim.x)
      if (bi < 0 || row[i] > bv) { bv = row[i]; bi = i; }
    token = block_argmax(bv, bi, sv, si).i;
  } else {
    const float inv_t = 1.f / temperature;
    float bv = -INFINITY; int bi = -1;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float lg = row[i] * inv_t;
      if (bi < 0 || lg > bv) { bv = lg; bi = i; }
    }
    const float m = block_argmax(bv, bi, sv, si).v;
    uint32_t floor_key = 0u;
    if (top_k > 0 && top_k < V)
      floor_key = radix_threshold<false>(row, V, inv_t, m, (double)top_k, 0u, hist, &s_prefix, &s_above, &s_target);
    if (top_p > 0.f && top_p < 1.f) {
      const uint32_t kp = radix_threshold<true>(row, V, inv_t, m, (double)top_p, floor_key, hist, &s_prefix, &s_above,
                                                &s_target);
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
    token = block_argmax(bv, bi, sv, si).i;
  }
  if (threadIdx.x == 0) {
    out[r] = token;
    if (rec) {
      rec[QB_SLOT_LAST] = token;
      rec[QB_SLOT_DRAWN] = (int)(draw + 1u);
    }
  }
}

extern "C" int qb_sample_rows(const float* logits, int n, int V, int* slots, const int* row_slot, int n_slots,
                              int* out, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (slots != nullptr && (row_slot == nullptr || n_slots <= 0)) return QB_ERR_BAD_ARG;
  sample_rows_kernel<<<n, SAMP_THREADS, 0, stream>>>(logits, V, slots, row_slot, n_slots, out);
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
  // eight loads in flight a thread (the chunk is a few thousand logits: its time is the loads' latency), taken in
  // index order so that the first maximum wins
  for (int i0 = lo + threadIdx.x; i0 < hi; i0 += 8 * blockDim.x) {
    float v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int i = i0 + u * blockDim.x;
      v[u] = i < hi ? __ldg(row + i) : -INFINITY;
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int i = i0 + u * blockDim.x;
      if (i < hi && (bi < 0 || v[u] > bv)) { bv = v[u]; bi = i; }
    }
  }
  const ArgBest b = block_argmax(bv, bi, sv, si);
  if (threadIdx.x == 0) { pv[r * parts + part] = b.v; pi[r * parts + part] = b.i; }
}

__global__ void argmax_final_kernel(const float* __restrict__ pv, const int* __restrict__ pi, int parts,
                                    int* __restrict__ slots, const int* __restrict__ row_slot, int n_slots,
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
  if (slots != nullptr) {
    const int slot = row_slot[r];
    if (slot >= 0 && slot < n_slots) {
      int* rec = slots + (size_t)slot * QB_SLOT_WORDS;
      rec[QB_SLOT_LAST] = bi;
      rec[QB_SLOT_DRAWN] += 1;
    }
  }
}

// Every row greedy.  scratch: parts floats and parts ints per row.  slots / row_slot as in qb_sample_rows.
extern "C" int qb_argmax_rows(const float* logits, int n, int V, int parts, float* scratch_v, int* scratch_i,
                              int* slots, const int* row_slot, int n_slots, int* out, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (parts <= 0 || n > 65535) return QB_ERR_BAD_ARG;
  if (slots != nullptr && (row_slot == nullptr || n_slots <= 0)) return QB_ERR_BAD_ARG;
  argmax_partial_kernel<<<dim3(parts, n), 256, 0, stream>>>(logits, V, parts, scratch_v, scratch_i);
  argmax_final_kernel<<<n, 32, 0, stream>>>(scratch_v, scratch_i, parts, slots, row_slot, n_slots, out);
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


// The step's part in the state slots: each request's position moves to the tokens it will hold after the
// step.  Before that the record is checked against what the host packed: the slot must be live and its
// position must be where the step's first token of the request goes; a difference means host and device
// disagree about a request, which is recorded in the status words (the step's writes then land where
// the host said; the host raises when it next reads the status).
__global__ void slots_advance_kernel(int* __restrict__ slots, int n_slots, const int* __restrict__ req_slot,
                                     const int* __restrict__ req_start, const int* __restrict__ req_len_after, int R,
                                     int* status) {
  for (int r = blockIdx.x * blockDim.x + threadIdx.x; r < R; r += gridDim.x * blockDim.x) {
    const int slot = req_slot[r];
    if (slot < 0 || slot >= n_slots) { qb_set_status(status, QB_STATUS_SLOT_MISMATCH, slot, 8); continue; }
    int* rec = slots + (size_t)slot * QB_SLOT_WORDS;
    const int before = req_len_after[r] - (req_start[r + 1] - req_start[r]);
    if (rec[QB_SLOT_LIVE] != 1 || rec[QB_SLOT_POSITION] != before) qb_set_status(status, QB_STATUS_SLOT_MISMATCH, slot, 8);
    rec[QB_SLOT_POSITION] = req_len_after[r];
  }
}

extern "C" int qb_slots_advance(int* slots, int n_slots, const int* req_slot, const int* req_start,
                                const int* req_len_after, int R, int* status, cudaStream_t stream) {
  if (R <= 0) return 0;
  if (n_slots <= 0) return QB_ERR_BAD_ARG;
  slots_advance_kernel<<<(R + 127) / 128, 128, 0, stream>>>(slots, n_slots, req_slot, req_start, req_len_after, R, status);
  QB_LAUNCH_CHECK();
  return 0;
}
