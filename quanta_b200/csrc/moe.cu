// Routed experts: top-k routing, the plan that sorts (token, slot) pairs by expert, and the plain
// SIMT grouped products.  Nothing here reads a size back to the host: grids are sized for the worst
// case and blocks past the planned tile count return.
//
//   scores = sigmoid(logits); choice = scores + bias (selection only); top-k by (choice desc, expert
//   asc); w = scores[idx]; w /= sum(w) + 1e-20 if renorm and k > 1; w *= scale
//   (src/quanta/minimax/moe.py:36-56).
//   expert e on row x: down_e( silu(gate_e x) * up_e x ), times w, summed over the k slots in slot
//   order by the next norm kernel (src/quanta/minimax/moe.py:59-88).
#include "common.cuh"

// ---------------------------------------------------------------------------------------------
// routing: one warp per token
// ---------------------------------------------------------------------------------------------
// One warp selects for one token: the k largest of sigmoid(logit) (+ bias), the lower expert index first
// among equals; the weights are the bias-free scores, renormalised and scaled.  Lane l holds experts
// l, l + 32, ...; s_score: k floats of shared memory that belong to this warp.
// bias: the lane's own values, bias[i] for expert lane + 32 i (zeros when the router has none).
template <int NPL>
__device__ __forceinline__ void lane_bias(const float* __restrict__ bias, int E, float (&out)[NPL]) {
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int i = 0; i < NPL; ++i) {
    const int e = lane + 32 * i;
    out[i] = (bias != nullptr && e < E) ? bias[e] : 0.f;
  }
}

// s_idx: if not null, the chosen experts are left there too (shared memory).
template <int NPL>
__device__ __forceinline__ void select_topk(const float (&logit)[NPL], const float (&bias)[NPL],
                                            int* __restrict__ idx_row, float* __restrict__ w_row, float* s_score,
                                            int E, int k, int renorm, float scale, int* s_idx = nullptr) {
  const int lane = threadIdx.x & 31;
  float choice[NPL], score[NPL];
  unsigned taken = 0u;
#pragma unroll
  for (int i = 0; i < NPL; ++i) {
    const int e = lane + 32 * i;
    score[i] = 0.f;
    if (e < E) {
      const float x = logit[i];
      const float s = 1.f / (1.f + expf(-x));
      score[i] = s;
      choice[i] = s + bias[i];
    } else {
      choice[i] = -INFINITY;
      taken |= 1u << i;
    }
  }
  float sum = 0.f;
  for (int r = 0; r < k; ++r) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
      // i ascending is expert index ascending within the lane: the first maximum wins a tie
      if (!((taken >> i) & 1u) && (bi == 0x7fffffff || choice[i] > bv)) {
        bv = choice[i];
        bi = lane + 32 * i;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      const bool take = (oi != 0x7fffffff) && (bi == 0x7fffffff || ov > bv || (ov == bv && oi < bi));
      if (take) { bv = ov; bi = oi; }
    }
    float mine = 0.f;
    if ((bi & 31) == lane) {
      taken |= 1u << (bi >> 5);
#pragma unroll
      for (int i = 0; i < NPL; ++i)
        if (i == (bi >> 5)) mine = score[i];
    }
    const float sc = __shfl_sync(0xffffffffu, mine, bi & 31);     // the bias-free score of the chosen expert
    sum += sc;
    if (lane == 0) {
      idx_row[r] = bi;
      s_score[r] = sc;
      if (s_idx != nullptr) s_idx[r] = bi;
    }
  }
  __syncwarp();
  const float denom = (renorm && k > 1) ? sum + 1e-20f : 1.f;
  for (int r = lane; r < k; r += 32) w_row[r] = s_score[r] / denom * scale;
}

template <int NPL>   // experts per lane, E <= 32*NPL
__device__ __forceinline__ void route_token(const float* __restrict__ logits, int n_partials,
                                            const float* __restrict__ bias, int* __restrict__ idx_out,
                                            float* __restrict__ w_out, int T, int E, int k, int renorm, float scale,
                                            float* s_logit, float* s_part) {
  // logits: [n_partials][T][E], partial products of chunks of the inner dimension.  One block per token.
  // The partials of an expert are added by `groups` threads, each a contiguous range in index order, and
  // the groups' sums are then added in group order: the order depends on E and n_partials only, never on
  // the step, and every thread has only a few independent loads to wait for.  The first warp selects;
  // its lane 0 writes the chosen experts.  s_logit: 1024 floats, s_part: 1056.
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  const float* lg = logits + (size_t)t * E;
  const size_t pstride = (size_t)T * E;
  const int e_round = (E + 31) / 32 * 32;
  const int groups = max(1, min((int)blockDim.x / e_round, n_partials));
  const int per = (n_partials + groups - 1) / groups;
  for (int i = threadIdx.x; i < groups * e_round; i += blockDim.x) {
    const int g = i / e_round, e = i % e_round;
    if (e < E) {
      const int p_end = min(n_partials, (g + 1) * per);
      float x = 0.f;
#pragma unroll 8
      for (int p = g * per; p < p_end; ++p) x += lg[p * pstride + e];
      s_part[i] = x;
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    float x = s_part[e];
    for (int g = 1; g < groups; ++g) x += s_part[g * e_round + e];
    s_logit[e] = x;
  }
  __syncthreads();
  if (threadIdx.x >= 32) return;      // of this function: the caller's other warps go on
  float logit[NPL], b[NPL];
  lane_bias<NPL>(bias, E, b);
#pragma unroll
  for (int i = 0; i < NPL; ++i) {
    const int e = lane + 32 * i;
    logit[i] = e < E ? s_logit[e] : 0.f;
  }
  select_topk<NPL>(logit, b, idx_out + (size_t)t * k, w_out + (size_t)t * k, s_part, E, k, renorm, scale);
}

template <int NPL>
__global__ void router_topk_kernel(const float* __restrict__ logits, int n_partials,
                                   const float* __restrict__ bias, int* __restrict__ idx_out,
                                   float* __restrict__ w_out, int T, int E, int k, int renorm, float scale) {
  __shared__ float s_logit[1024];
  __shared__ float s_part[1056];
  if ((int)blockIdx.x >= T) return;
  route_token<NPL>(logits, n_partials, bias, idx_out, w_out, T, E, k, renorm, scale, s_logit, s_part);
}

// Steps of many tokens: one warp a token, eight tokens a block; the few partial logits of an expert are
// added in index order by the lane that holds the expert (the additions of route_token for as few).
constexpr int TOPK_WARPS = 8, TOPK_WARP_MAX_PARTIALS = 4;

template <int NPL>
__global__ void __launch_bounds__(TOPK_WARPS * 32)
router_topk_warp_kernel(const float* __restrict__ logits, int n_partials, const float* __restrict__ bias,
                        int* __restrict__ idx_out, float* __restrict__ w_out, int T, int E, int k, int renorm,
                        float scale) {
  extern __shared__ float s_scores[];            // [TOPK_WARPS][k]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t = blockIdx.x * TOPK_WARPS + warp;
  if (t >= T) return;
  const float* lg = logits + (size_t)t * E;
  const size_t pstride = (size_t)T * E;
  float logit[NPL], b[NPL];
  lane_bias<NPL>(bias, E, b);
#pragma unroll
  for (int i = 0; i < NPL; ++i) {
    const int e = lane + 32 * i;
    float x = 0.f;
    if (e < E)
      for (int p = 0; p < n_partials; ++p) x += lg[p * pstride + e];
    logit[i] = x;
  }
  select_topk<NPL>(logit, b, idx_out + (size_t)t * k, w_out + (size_t)t * k, s_scores + (size_t)warp * k, E, k,
                   renorm, scale);
}

extern "C" int qb_router_topk(const float* logits, int n_partials, const float* bias, int* idx_out, float* w_out,
                              int T, int E, int k, int renorm, float scale, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (k <= 0 || k > E || n_partials <= 0) return QB_ERR_BAD_ARG;
  if (E > 1024) return QB_ERR_UNSUPPORTED;
  if (T >= 64 && n_partials <= TOPK_WARP_MAX_PARTIALS) {
    const int blocks = (T + TOPK_WARPS - 1) / TOPK_WARPS;
    const size_t smem = (size_t)TOPK_WARPS * k * sizeof(float);       // at most 32 KB
#define QB_ROUTE_W(N) router_topk_warp_kernel<N><<<blocks, TOPK_WARPS * 32, smem, stream>>>(logits, n_partials, bias, idx_out, w_out, T, E, k, renorm, scale)
    if (E <= 32) QB_ROUTE_W(1);
    else if (E <= 64) QB_ROUTE_W(2);
    else if (E <= 128) QB_ROUTE_W(4);
    else if (E <= 256) QB_ROUTE_W(8);
    else if (E <= 512) QB_ROUTE_W(16);
    else QB_ROUTE_W(32);
#undef QB_ROUTE_W
    QB_LAUNCH_CHECK();
    return 0;
  }
  // many threads add the partials side by side; the selecting warp's arrays set the register need for large E
  const int warps = E <= 256 ? 32 : 8, blocks = T;
#define QB_ROUTE(N) router_topk_kernel<N><<<blocks, warps * 32, 0, stream>>>(logits, n_partials, bias, idx_out, w_out, T, E, k, renorm, scale)
  if (E <= 32) QB_ROUTE(1);
  else if (E <= 64) QB_ROUTE(2);
  else if (E <= 128) QB_ROUTE(4);
  else if (E <= 256) QB_ROUTE(8);
  else if (E <= 512) QB_ROUTE(16);
  else QB_ROUTE(32);
#undef QB_ROUTE
  QB_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------------------------
// plan: counts per expert -> offsets, tile list, pairs sorted by expert
//   plan layout (int32): counts[E] | cursor[E] | offsets[E+1] | num_tiles | num_active | pad |
//                        active[E] (experts that have rows, ascending)   -- 4E+4 words
// ---------------------------------------------------------------------------------------------
__global__ void moe_count_kernel(const int* __restrict__ idx, int n_pairs, int E, int* __restrict__ counts,
                                 int* status) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n_pairs; i += gridDim.x * blockDim.x) {
    const int e = idx[i];
    if (e < 0 || e >= E) { qb_set_status(status, QB_STATUS_BAD_EXPERT, e, 4); continue; }
    atomicAdd(&counts[e], 1);
  }
}

// one block of 1024 threads; thread e owns expert e
__global__ void moe_scan_kernel(const int* __restrict__ counts, int* __restrict__ offsets,
                                int* __restrict__ num_tiles, int* __restrict__ active,
                                int* __restrict__ tile_expert, int* __restrict__ tile_row0, int E, int BM,
                                int max_tiles) {
  __shared__ int s_cnt[1024];
  __shared__ int s_til[1024];
  __shared__ int s_act[1024];
  const int e = threadIdx.x;
  const int c = e < E ? counts[e] : 0;
  const int nt = (c + BM - 1) / BM;
  s_cnt[e] = c;
  s_til[e] = nt;
  s_act[e] = c > 0;
  __syncthreads();
  for (int o = 1; o < 1024; o <<= 1) {
    int a = 0, b = 0, d = 0;
    if (e >= o) { a = s_cnt[e - o]; b = s_til[e - o]; d = s_act[e - o]; }
    __syncthreads();
    s_cnt[e] += a;
    s_til[e] += b;
    s_act[e] += d;
    __syncthreads();
  }
  const int off = s_cnt[e] - c, toff = s_til[e] - nt;     // exclusive prefixes
  if (e < E) offsets[e] = off;
  if (c > 0) active[s_act[e] - 1] = e;                    // experts with rows, in index order
  if (e == E - 1) { offsets[E] = s_cnt[e]; num_tiles[0] = min(s_til[e], max_tiles); num_tiles[1] = s_act[e]; }
  for (int i = 0; i < nt; ++i) {
    if (toff + i < max_tiles) {
      tile_expert[toff + i] = e;
      tile_row0[toff + i] = off + i * BM;
    }
  }
}

__global__ void moe_scatter_kernel(const int* __restrict__ idx, int n_pairs, int E,
                                   const int* __restrict__ offsets, int* __restrict__ cursor,
                                   int* __restrict__ sorted_pair) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n_pairs; i += gridDim.x * blockDim.x) {
    const int e = idx[i];
    if (e < 0 || e >= E) continue;
    const int p = offsets[e] + atomicAdd(&cursor[e], 1);
    sorted_pair[p] = i;
  }
}

// The whole plan in one block, for steps with few pairs (decoding): counts in shared memory, the same
// scans as above, then the scatter.  One launch instead of a memset and three kernels.
struct PlanShared {
  int cur[1024];
  int warp_tot[32][3];
};

// The plan of up to 4096 pairs by the first NTH threads of a block (NTH >= E, a multiple of 32), thread e
// for expert e; `sync` is a barrier of exactly these threads.  Counts by shared-memory atomics, the three
// prefix sums (rows, tiles, active experts) by warp shuffles and one pass over the warps' totals.  idx is
// read past L1 (another block of the same launch may have written it), or from shared memory (IDX_SHARED).
template <int NTH, bool IDX_SHARED = false, typename Sync>
__device__ __forceinline__ void plan_small_body(const int* idx, int n_pairs, int E, int BM, int* __restrict__ plan,
                                                int* __restrict__ sorted_pair, int* __restrict__ tile_expert,
                                                int* __restrict__ tile_row0, int max_tiles, int* status,
                                                PlanShared& sh, Sync sync) {
  int* s_cur = sh.cur;
  const int e = threadIdx.x, lane = e & 31, warp = e >> 5;
  s_cur[e] = 0;
  sync();
  for (int i = e; i < n_pairs; i += NTH) {
    const int x = IDX_SHARED ? idx[i] : __ldcg(idx + i);
    if (x < 0 || x >= E) { qb_set_status(status, QB_STATUS_BAD_EXPERT, x, 4); continue; }
    atomicAdd(&s_cur[x], 1);
  }
  sync();
  const int c = e < E ? s_cur[e] : 0;
  const int nt = (c + BM - 1) / BM;
  int sc = c, st = nt, sa = c > 0;             // inclusive sums over the experts up to e
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int a = __shfl_up_sync(0xffffffffu, sc, o), b = __shfl_up_sync(0xffffffffu, st, o),
              d = __shfl_up_sync(0xffffffffu, sa, o);
    if (lane >= o) { sc += a; st += b; sa += d; }
  }
  if (lane == 31) { sh.warp_tot[warp][0] = sc; sh.warp_tot[warp][1] = st; sh.warp_tot[warp][2] = sa; }
  sync();
  for (int w = 0; w < warp; ++w) { sc += sh.warp_tot[w][0]; st += sh.warp_tot[w][1]; sa += sh.warp_tot[w][2]; }
  const int off = sc - c, toff = st - nt;
  int* counts = plan;
  int* offsets = plan + 2 * E;
  int* num_tiles = plan + 3 * E + 1;
  int* active = plan + 3 * E + 4;
  if (e < E) { counts[e] = c; offsets[e] = off; }
  if (c > 0) active[sa - 1] = e;
  if (e == E - 1) { offsets[E] = sc; num_tiles[0] = min(st, max_tiles); num_tiles[1] = sa; }
  for (int i = 0; i < nt; ++i) {
    if (toff + i < max_tiles) {
      tile_expert[toff + i] = e;
      tile_row0[toff + i] = off + i * BM;
    }
  }
  s_cur[e] = off;                     // running write position of each expert
  sync();
  for (int i = e; i < n_pairs; i += NTH) {
    const int x = IDX_SHARED ? idx[i] : __ldcg(idx + i);
    if (x < 0 || x >= E) continue;
    sorted_pair[atomicAdd(&s_cur[x], 1)] = i;
  }
}

__global__ void __launch_bounds__(1024)
moe_plan_small_kernel(const int* __restrict__ idx, int n_pairs, int E, int BM, int* __restrict__ plan,
                      int* __restrict__ sorted_pair, int* __restrict__ tile_expert,
                      int* __restrict__ tile_row0, int max_tiles, int* status) {
  __shared__ PlanShared sh;
  plan_small_body<1024>(idx, n_pairs, E, BM, plan, sorted_pair, tile_expert, tile_row0, max_tiles, status, sh,
                        [] { __syncthreads(); });
}

// ---------------------------------------------------------------------------------------------
// The router of steps of few tokens, whole, in one launch: float32 logits, selection, plan.
//
//   logits[t][e] = sum_k float(x[t][k]) * gate[e][k]        (src/quanta/minimax/moe.py:44)
//
// A block takes RS_TT tokens and RS_EPB experts; RS_KW warps share an expert, each a contiguous quarter of
// the inner dimension.  The tokens' rows are staged in shared memory once; a warp's lanes walk their part of
// the gate row in groups of 4 elements (lane l takes groups l, l + 32, ...), each lane adds its products in
// that order, the lanes' sums are added by a butterfly and the quarters' sums in index order.  The order of
// a logit's additions depends on the inner dimension alone: a token's logits are bit-identical whatever
// else the step holds and however it is cut.  Few experts a block put the gate's rows on many SMs, and every
// lane has all its loads of the row in flight at once.
// With `select`: the block that finishes a token tile last (a counter in global memory) selects for the
// tile's tokens, a warp a token; the block that finishes the last tile lays the expert plan down for the
// whole step.  Every block ends by itself, nothing waits; the counters are zero again afterwards.
// ---------------------------------------------------------------------------------------------
constexpr int RS_TT = 8, RS_WARPS = 8, RS_QUARTERS = 4, RS_BATCH = 8;

__device__ __forceinline__ float4 rs_load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 rs_load4(const __nv_bfloat16* p) {      // a bfloat16 is the upper half of a float32
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  return make_float4(__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xffff0000u), __uint_as_float(raw.y << 16),
                     __uint_as_float(raw.y & 0xffff0000u));
}

// KW: warps that share an expert (4: a quarter each, two experts a block, for steps of few tokens, whose
// gate rows then come from many SMs at once; 1: a warp takes the four quarters in turn, eight experts a
// block, so that a step of many tokens stages its rows in fewer blocks).  The sums are the same in both.
template <typename TX, int NPL, bool VEC, int KW>
__global__ void __launch_bounds__(RS_WARPS * 32)
router_small_kernel(const TX* __restrict__ x, const float* __restrict__ gate, const float* __restrict__ bias,
                    float* logits, int* idx_out, float* __restrict__ w_out, int T, int E, int K, int k, int renorm,
                    float scale, int select, int* counters, int BM, int* __restrict__ plan,
                    int* __restrict__ sorted_pair, int* __restrict__ tile_expert, int* __restrict__ tile_row0,
                    int max_tiles, int* status) {
  constexpr int EPB = RS_WARPS / KW;                            // experts a block
  extern __shared__ __align__(16) unsigned char rs_smem[];      // [RS_TT][K] of TX: the tile's token rows
  __shared__ PlanShared sh;
  __shared__ float s_score[RS_WARPS][256];
  __shared__ float s_quarter[RS_WARPS * RS_QUARTERS / KW][RS_TT];     // [expert of the block][quarter][token]
  __shared__ int s_chosen[RS_TT * 32];                                // a single tile's choices, for its plan (k <= 32)
  __shared__ int s_last;
  TX* xs = reinterpret_cast<TX*>(rs_smem);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int t0 = blockIdx.y * RS_TT, nt = min(RS_TT, T - t0);
  const int le = warp / KW, e = blockIdx.x * EPB + le;

  const int units = VEC ? K / 4 : K;                       // groups of 4 elements (16 bytes), or single elements
  const int per = (units + RS_QUARTERS - 1) / RS_QUARTERS;
  const float* grow = gate + (size_t)(e < E ? e : 0) * K;
  // The warp's work is a list of batches: RS_BATCH groups a lane (f, f + 32, ...) of one quarter; a warp
  // reads 512 contiguous bytes of the gate row and of each token row at a time.  The gate values of the
  // batch after the current one are in flight while the current one is multiplied.
  const int q_first = warp % KW;
  const int batches_per_q = (per + 32 * RS_BATCH - 1) / (32 * RS_BATCH);
  const int n_batches = VEC ? ((RS_QUARTERS - q_first + KW - 1) / KW) * batches_per_q : 0;
  auto fetch = [&](int b, float4 (&g)[RS_BATCH]) {
    const int q = q_first + (b / batches_per_q) * KW;
    const int u0 = q * per, u1 = min(units, u0 + per);
    const int f0 = u0 + (b % batches_per_q) * 32 * RS_BATCH + lane;
#pragma unroll
    for (int u = 0; u < RS_BATCH; ++u) {
      const int f = f0 + 32 * u;
      if (f < u1) g[u] = *reinterpret_cast<const float4*>(grow + (size_t)f * 4);
    }
  };
  float4 g0[RS_BATCH], g1[RS_BATCH], g2[RS_BATCH];
  if (n_batches > 0) fetch(0, g0);                         // into flight before anything else
  if (n_batches > 1) fetch(1, g1);

  if (VEC) {
    // asynchronous copies, all in flight at once (rows of K elements, K a multiple of 4: whole 8-byte words)
    const int n8 = nt * K * (int)sizeof(TX) / 8;
    const unsigned char* src = reinterpret_cast<const unsigned char*>(x + (size_t)t0 * K);
    const uint32_t dst = (uint32_t)__cvta_generic_to_shared(xs);
    for (int i = tid; i < n8; i += RS_WARPS * 32)
      asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst + 8u * (uint32_t)i), "l"(src + 8 * (size_t)i) : "memory");
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 0;" ::: "memory");
  } else {
    for (int i = tid; i < nt * K; i += RS_WARPS * 32) xs[i] = x[(size_t)t0 * K + i];
  }
  __syncthreads();
  float acc[RS_TT];
#pragma unroll
  for (int t = 0; t < RS_TT; ++t) acc[t] = 0.f;
  auto multiply = [&](int b, const float4 (&g)[RS_BATCH]) {
    const int q = q_first + (b / batches_per_q) * KW;
    const int u0 = q * per, u1 = min(units, u0 + per);
    const int f0 = u0 + (b % batches_per_q) * 32 * RS_BATCH + lane;
#pragma unroll
    for (int u = 0; u < RS_BATCH; ++u) {
      const int f = f0 + 32 * u;
      if (f < u1) {
#pragma unroll
        for (int t = 0; t < RS_TT; ++t) {
          if (t < nt) {
            const float4 xv = rs_load4(xs + (size_t)t * K + (size_t)f * 4);
            acc[t] = fmaf(xv.x, g[u].x, acc[t]);
            acc[t] = fmaf(xv.y, g[u].y, acc[t]);
            acc[t] = fmaf(xv.z, g[u].z, acc[t]);
            acc[t] = fmaf(xv.w, g[u].w, acc[t]);
          }
        }
      }
    }
    if ((b + 1) % batches_per_q == 0) {                    // the quarter is done: its sums go to shared memory
#pragma unroll
      for (int t = 0; t < RS_TT; ++t) {
        const float v = qb_warp_sum(acc[t]);
        if (lane == 0) s_quarter[le * RS_QUARTERS + q][t] = v;
        acc[t] = 0.f;
      }
    }
  };
  if (VEC) {
    // three buffers in turn: the gate values of the next two batches are in flight while one is multiplied
    for (int b = 0; b < n_batches; b += 3) {
      if (b + 2 < n_batches) fetch(b + 2, g2);
      multiply(b, g0);
      if (b + 1 < n_batches) {
        if (b + 3 < n_batches) fetch(b + 3, g0);
        multiply(b + 1, g1);
      }
      if (b + 2 < n_batches) {
        if (b + 4 < n_batches) fetch(b + 4, g1);
        multiply(b + 2, g2);
      }
    }
  } else {
    for (int q = q_first; q < RS_QUARTERS; q += KW) {
      const int u0 = q * per, u1 = min(units, u0 + per);
      for (int kk = u0 + lane; kk < u1; kk += 32) {
        const float gv = grow[kk];
#pragma unroll
        for (int t = 0; t < RS_TT; ++t)
          if (t < nt) acc[t] = fmaf(qb_to_float<TX>(xs[(size_t)t * K + kk]), gv, acc[t]);
      }
#pragma unroll
      for (int t = 0; t < RS_TT; ++t) {
        const float v = qb_warp_sum(acc[t]);
        if (lane == 0) s_quarter[le * RS_QUARTERS + q][t] = v;
        acc[t] = 0.f;
      }
    }
  }
  __syncthreads();
  if (tid < EPB * RS_TT) {
    const int l2 = tid / RS_TT, t = tid % RS_TT, ee = blockIdx.x * EPB + l2;
    if (ee < E && t < nt) {
      float v = s_quarter[l2 * RS_QUARTERS][t];
#pragma unroll
      for (int q = 1; q < RS_QUARTERS; ++q) v += s_quarter[l2 * RS_QUARTERS + q][t];
      __stcg(logits + (size_t)(t0 + t) * E + ee, v);
    }
  }
  if (!select) return;
  // the selecting warps will want the bias: fetched now, under the hand-over below
  float my_bias[NPL];
  lane_bias<NPL>(bias, E, my_bias);
  // ---- the last block of this token tile selects ----
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    const int before = atomicAdd(&counters[1 + blockIdx.y], 1);
    s_last = before == (int)gridDim.x - 1;
    if (s_last) counters[1 + blockIdx.y] = 0;      // every other block of the tile has counted already
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  for (int t = warp; t < nt; t += RS_WARPS) {
    float logit[NPL];
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
      const int ee = lane + 32 * i;
      logit[i] = ee < E ? __ldcg(logits + (size_t)(t0 + t) * E + ee) : 0.f;
    }
    select_topk<NPL>(logit, my_bias, idx_out + (size_t)(t0 + t) * k, w_out + (size_t)(t0 + t) * k, s_score[warp], E, k,
                     renorm, scale, (gridDim.y == 1 && k <= 32) ? s_chosen + t * k : nullptr);
  }
  // ---- the block that finishes the last tile lays the plan down ----
  __syncthreads();
  if (gridDim.y > 1) {
    if (tid == 0) {
      __threadfence();
      const int before = atomicAdd(&counters[0], 1);
      s_last = before == (int)gridDim.y - 1;
      if (s_last) counters[0] = 0;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
  }
  if (gridDim.y == 1 && k <= 32)       // the step is this one tile: its choices are still in shared memory
    plan_small_body<RS_WARPS * 32, true>(s_chosen, T * k, E, BM, plan, sorted_pair, tile_expert, tile_row0, max_tiles,
                                         status, sh, [] { __syncthreads(); });
  else
    plan_small_body<RS_WARPS * 32>(idx_out, T * k, E, BM, plan, sorted_pair, tile_expert, tile_row0, max_tiles, status, sh,
                                   [] { __syncthreads(); });
}

// Token rows of at most this many bytes fit the shared-memory tile.
constexpr size_t RS_MAX_TILE_BYTES = 200 * 1024;

// 1 if qb_router_small can also select and plan (select = 1) for these sizes.
extern "C" int qb_router_small_selects(int T, int E, int k) {
  return (E <= RS_WARPS * 32 && k <= 256 && (long long)T * k <= 4096) ? 1 : 0;
}

// x [T, K] float32 or bfloat16, gate [E, K] float32, logits [T, E] float32 (always written).  select = 1 (see
// qb_router_small_selects): idx_out / w_out [T, k] and the expert plan as qb_moe_plan lays it down;
// counters: 1 + ceil(T / 8) int32 that are zero before the call and zero after it.
extern "C" int qb_router_small(const void* x, int x_dtype, const float* gate, const float* bias, float* logits,
                               int* idx_out, float* w_out, int T, int E, int K, int k, int renorm, float scale,
                               int select, int* counters, int BM, int* plan, int* sorted_pair, int* tile_expert,
                               int* tile_row0, int max_tiles, int* status, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (E <= 0 || K <= 0) return QB_ERR_BAD_ARG;
  if (select && (!qb_router_small_selects(T, E, k) || counters == nullptr || k <= 0 || k > E)) return QB_ERR_BAD_ARG;
  const size_t smem = (size_t)RS_TT * K * (x_dtype == QB_F32 ? 4 : 2);
  if (smem > RS_MAX_TILE_BYTES) return QB_ERR_UNSUPPORTED;
  const bool vec = K % 4 == 0 && (((uintptr_t)x | (uintptr_t)gate) & 15) == 0;      // rows start on 8 (x) and 16 (gate) bytes
  // few tokens: two experts a block (more SMs pull the gate at once); many: eight (fewer blocks stage the rows)
  const int kw = T <= 16 ? 4 : 1;
  const int epb = RS_WARPS / kw;
  const dim3 grid((E + epb - 1) / epb, (T + RS_TT - 1) / RS_TT);
  if (grid.y > 65535) return QB_ERR_UNSUPPORTED;
  cudaError_t err = cudaSuccess;
#define QB_RS(TX, N, V, KW_)                                                                                       \
  do {                                                                                                             \
    err = cudaFuncSetAttribute(router_small_kernel<TX, N, V, KW_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    if (err != cudaSuccess) return (int)err;                                                                       \
    router_small_kernel<TX, N, V, KW_><<<grid, RS_WARPS * 32, smem, stream>>>(                                     \
        (const TX*)x, gate, bias, logits, idx_out, w_out, T, E, K, k, renorm, scale, select, counters, BM, plan,  \
        sorted_pair, tile_expert, tile_row0, max_tiles, status);                                                   \
  } while (0)
#define QB_RS_K(TX, N, V)                                \
  do {                                                   \
    if (kw == 4) QB_RS(TX, N, V, 4); else QB_RS(TX, N, V, 1); \
  } while (0)
  // the selecting warp holds eight experts a lane whatever E (at most 256 here): fewer instances to compile
#define QB_RS_E(TX, V) QB_RS_K(TX, 8, V)
  if (x_dtype == QB_F32) { if (vec) QB_RS_E(float, true); else QB_RS_E(float, false); }
  else if (x_dtype == QB_BF16) { if (vec) QB_RS_E(__nv_bfloat16, true); else QB_RS_E(__nv_bfloat16, false); }
  else return QB_ERR_BAD_ARG;
#undef QB_RS_E
#undef QB_RS_K
#undef QB_RS
  QB_LAUNCH_CHECK();
  return 0;
}

extern "C" int qb_moe_plan(const int* idx, int n_pairs, int E, int BM, int* plan, int* sorted_pair,
                           int* tile_expert, int* tile_row0, int max_tiles, int* status,
                           cudaStream_t stream) {
  if (n_pairs <= 0) return 0;
  if (E > 1024) return QB_ERR_UNSUPPORTED;
  if (n_pairs <= 4096) {
    moe_plan_small_kernel<<<1, 1024, 0, stream>>>(idx, n_pairs, E, BM, plan, sorted_pair, tile_expert, tile_row0,
                                                  max_tiles, status);
    QB_LAUNCH_CHECK();
    return 0;
  }
  int* counts = plan;
  int* cursor = plan + E;
  int* offsets = plan + 2 * E;
  int* num_tiles = plan + 3 * E + 1;
  cudaError_t err = cudaMemsetAsync(plan, 0, sizeof(int) * (size_t)(3 * E + 4), stream);
  if (err != cudaSuccess) return (int)err;
  const int blocks = min((n_pairs + 255) / 256, 1024);
  moe_count_kernel<<<blocks, 256, 0, stream>>>(idx, n_pairs, E, counts, status);
  moe_scan_kernel<<<1, 1024, 0, stream>>>(counts, offsets, num_tiles, plan + 3 * E + 4, tile_expert, tile_row0, E,
                                          BM, max_tiles);
  moe_scatter_kernel<<<blocks, 256, 0, stream>>>(idx, n_pairs, E, offsets, cursor, sorted_pair);
  QB_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------------------------
// grouped products, SIMT.  Tile = 32 sorted rows of one expert x 64 output features, k slices of 16.
//   MODE 1: act[p, j]   = silu(x[tok(p)] . W13[e][j]) * (x[tok(p)] . W13[e][I + j]),  j < I
//   MODE 2: y[pair(p), n] = w[pair(p)] * (act[p] . W2[e][n]),  n < H
// Each output is one sequential float32 sum over the inner dimension.
// ---------------------------------------------------------------------------------------------
constexpr int MG_BM = 32, MG_BN = 64, MG_BK = 16;

template <typename X, typename W, typename O, int MODE>
__global__ void moe_grouped_simt_kernel(const X* __restrict__ x, const W* __restrict__ weights,
                                        O* __restrict__ out, const int* __restrict__ sorted_pair,
                                        const float* __restrict__ pair_w, const int* __restrict__ plan,
                                        const int* __restrict__ tile_expert, const int* __restrict__ tile_row0,
                                        int E, int top_k, int K, int N) {
  // MODE 1: K = hidden, N = I (weights [E, 2N, K]); MODE 2: K = I, N = hidden (weights [E, N, K])
  const int* offsets = plan + 2 * E;
  const int num_tiles = plan[3 * E + 1];
  const int tile = blockIdx.y;
  if (tile >= num_tiles) return;
  const int e = tile_expert[tile];
  const int row0 = tile_row0[tile];
  const int row_end = offsets[e + 1];
  const int n0 = blockIdx.x * MG_BN;
  __shared__ float Xs[MG_BK][MG_BM + 1];
  __shared__ float Ws[MODE == 1 ? 2 : 1][MG_BK][MG_BN + 4];
  __shared__ int src_row[MG_BM];
  const int tid = threadIdx.x;
  if (tid < MG_BM) {
    const int p = row0 + tid;
    int r = -1;
    if (p < row_end) r = (MODE == 1) ? sorted_pair[p] / top_k : p;
    src_row[tid] = r;
  }
  __syncthreads();
  const W* wbase = weights + (size_t)e * (MODE == 1 ? 2 : 1) * N * K;
  const int tx = tid % 16, ty = tid / 16;   // rows ty*2.., cols tx*4..
  float acc[MODE == 1 ? 2 : 1][2][4];
#pragma unroll
  for (int a = 0; a < (MODE == 1 ? 2 : 1); ++a)
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[a][i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += MG_BK) {
    // X tile: 32 x 16 = 512 elements, 2 per thread
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      const int id = tid + q * 256;
      const int r = id / MG_BK, kk = id % MG_BK;
      const int sr = src_row[r];
      Xs[kk][r] = (sr >= 0 && k0 + kk < K) ? qb_to_float<X>(x[(size_t)sr * K + k0 + kk]) : 0.f;
    }
    // W tile(s): 64 x 16 = 1024 elements, 4 per thread
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int id = tid + q * 256;
      const int r = id / MG_BK, kk = id % MG_BK;
      const int gn = n0 + r;
      const bool ok = gn < N && k0 + kk < K;
      Ws[0][kk][r] = ok ? qb_to_float<W>(wbase[(size_t)gn * K + k0 + kk]) : 0.f;
      if (MODE == 1) Ws[MODE == 1 ? 1 : 0][kk][r] = ok ? qb_to_float<W>(wbase[(size_t)(N + gn) * K + k0 + kk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < MG_BK; ++kk) {
      float a[2], b[4];
      a[0] = Xs[kk][ty * 2];
      a[1] = Xs[kk][ty * 2 + 1];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Ws[0][kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[0][i][j] = fmaf(a[i], b[j], acc[0][i][j]);
      if (MODE == 1) {
#pragma unroll
        for (int j = 0; j < 4; ++j) b[j] = Ws[MODE == 1 ? 1 : 0][kk][tx * 4 + j];
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[MODE == 1 ? 1 : 0][i][j] = fmaf(a[i], b[j], acc[MODE == 1 ? 1 : 0][i][j]);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int p = row0 + ty * 2 + i;
    if (p >= row_end) continue;
    if (MODE == 1) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int gn = n0 + tx * 4 + j;
        if (gn >= N) continue;
        const float g = acc[0][i][j], u = acc[MODE == 1 ? 1 : 0][i][j];
        out[(size_t)p * N + gn] = qb_from_float<O>(g / (1.f + expf(-g)) * u);
      }
    } else {
      const int pair = sorted_pair[p];
      const float w = pair_w[pair];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int gn = n0 + tx * 4 + j;
        if (gn < N) out[(size_t)pair * N + gn] = qb_from_float<O>(w * acc[0][i][j]);
      }
    }
  }
}

// x: [T, H] activations (MODE 1) or [pairs, I] act rows (MODE 2).
extern "C" int qb_moe_grouped_simt(int mode, const void* x, int x_dtype, const void* weights, int w_dtype,
                                   void* out, int out_dtype, const int* sorted_pair, const float* pair_w,
                                   const int* plan, const int* tile_expert, const int* tile_row0,
                                   int max_tiles, int E, int top_k, int K, int N, cudaStream_t stream) {
  if (max_tiles <= 0) return 0;
  if (max_tiles > 65535) return QB_ERR_UNSUPPORTED;
  dim3 grid((N + MG_BN - 1) / MG_BN, max_tiles);
  QB_DISPATCH_DTYPE(x_dtype, X, QB_DISPATCH_DTYPE(w_dtype, W, QB_DISPATCH_DTYPE(out_dtype, O, {
    if (mode == 1)
      moe_grouped_simt_kernel<X, W, O, 1><<<grid, 256, 0, stream>>>(
          (const X*)x, (const W*)weights, (O*)out, sorted_pair, pair_w, plan, tile_expert, tile_row0, E,
          top_k, K, N);
    else if (mode == 2)
      moe_grouped_simt_kernel<X, W, O, 2><<<grid, 256, 0, stream>>>(
          (const X*)x, (const W*)weights, (O*)out, sorted_pair, pair_w, plan, tile_expert, tile_row0, E,
          top_k, K, N);
    else
      return QB_ERR_BAD_ARG;
  })));
  QB_LAUNCH_CHECK();
  return 0;
}
