// Paged causal attention on the tensor cores (bfloat16 in, float32 softmax and accumulation).
//
// Two kernels share one inner loop (flash style: S = Q K^T by mma.m16n8k16, online softmax in
// float32 with exp2, O += P V with P rounded to bfloat16):
//
//  * span kernel: a tile of 128 (64 for head sizes above 128) query rows of ONE request and ONE kv
//    head, where a row is a (token, q head of the group) pair, so grouped heads fill the 16-row MMA
//    operand.  Each row is masked by its own token's position, so prompt portions of any length run,
//    from the cache that earlier steps and this step's rope kernel wrote.  A producer warp streams
//    K/V blocks of 64 keys through a ring in shared memory (TMA, one box per page); consumer warps
//    own 16 rows each.
//  * decode kernel: persistent blocks, a producer warp that issues bulk asynchronous copies of 64-key
//    tiles into a ring in shared memory and four consumer warps; the partial (max, sum, O) of each
//    tile goes to scratch and a merge kernel adds a token's tiles in index order.  Tile boundaries are
//    multiples of 64 in absolute position, so a token's result does not depend on the batch.
//
// (src/quanta/minimax/attention.py:194-203: scores * head_dim^-0.5, causal mask, softmax in float32,
// probabilities cast to the activation dtype, P V; q head h reads kv head h / (n_q / n_kv).)
// head_dim: any multiple of 16 up to 256 (template padding 64 / 128 / 256, dims past head_dim are zero).
#include <cuda.h>

#include <cstring>
#include <type_traits>

#include "common.cuh"

namespace {

constexpr int AT_BN = 64;           // keys per block (span kernel) and per warp (decode kernel)
constexpr int AT_WARPS = 4;
constexpr int AT_BM = 16 * AT_WARPS; // query rows per span tile
constexpr int AT_PAD = 8;            // +16 bytes a row: ldmatrix rows fall on distinct banks

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;      // 0 source bytes: the 16 destination bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(dst)), "l"(src), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Gather `n_keys` key rows starting at absolute position key0 of one request / kv head from the
// pages into shared memory rows [n_keys][HDP + AT_PAD] (dims >= hd and keys outside [0, key_end] are
// zero).  All threads of the block take part.
template <int HDP>
__device__ __forceinline__ void load_kv_block(__nv_bfloat16* dst, const __nv_bfloat16* __restrict__ cache,
                                              const int* __restrict__ bt, int key0, int n_keys, int key_end,
                                              int kvh, int nkv, int hd, int page_size, int num_pages, int* status,
                                              int pi0 = 0) {
  constexpr int CH = HDP / 8;        // 16-byte chunks per row
  // pages of a power-of-two size (the usual case) are found with a shift instead of a division
  const int shift = (page_size & (page_size - 1)) == 0 ? __ffs(page_size) - 1 : -1;
  for (int c = threadIdx.x; c < n_keys * CH; c += blockDim.x) {
    const int r = c / CH, d = (c % CH) * 8;
    const int key = key0 + r;
    bool ok = key >= 0 && key <= key_end && d < hd;
    const __nv_bfloat16* src = cache;
    if (ok) {
      const int pi = shift >= 0 ? key >> shift : key / page_size;
      const int slot = shift >= 0 ? key & (page_size - 1) : key % page_size;
      const int page = bt[pi - pi0];       // bt may be a copy of the table's entries from pi0 on
      if (page < 0 || page >= num_pages) {
        qb_set_status(status, QB_STATUS_BAD_PAGE, page, 7);
        ok = false;
      } else {
        src = cache + (((size_t)page * nkv + kvh) * page_size + slot) * hd + d;
      }
    }
    cp_async16(dst + (size_t)r * (HDP + AT_PAD) + d, src, ok);
  }
}

// One warp: 16 query rows against AT_BN keys held in shared memory.
//   qs: the warp's 16 rows [16][HDP+PAD]; ks, vs: [AT_BN][HDP+PAD]
//   row_hi[2], row_lo[2]: last / first visible key of the thread's two rows (g and g+8), absolute
//   key0: absolute position of ks row 0.   m, l, o: running max (log2 domain), partial sum, output.
// How a K or V tile of 64 keys lies in shared memory.
//  PaddedKV:   rows of HDP + 8 elements (what cp.async / per-row bulk copies write).
//  SwizzledKV: what TMA tensor loads with the 128-byte swizzle write: head_dim in slabs of 64 dims, each
//              slab [64 keys][64 dims] with rows of 128 bytes whose 16-byte chunks are XORed with (row & 7);
//              the tile is 1024-byte aligned.  Both are free of bank conflicts for ldmatrix.
template <int HDP>
struct PaddedKV {
  static __device__ __forceinline__ const __nv_bfloat16* at(const __nv_bfloat16* base, int row, int dim) {
    return base + (size_t)row * (HDP + AT_PAD) + dim;
  }
};
struct SwizzledKV {
  static __device__ __forceinline__ const __nv_bfloat16* at(const __nv_bfloat16* base, int row, int dim) {
    const int chunk = (dim & 63) >> 3;
    return base + (dim >> 6) * (AT_BN * 64) + row * 64 + ((chunk ^ (row & 7)) << 3) + (dim & 7);
  }
};

template <int HDP, typename KV = PaddedKV<HDP>>
__device__ __forceinline__ void attend_block(const __nv_bfloat16* qs, const __nv_bfloat16* ks, const __nv_bfloat16* vs,
                                             int key0, const int (&row_lo)[2], const int (&row_hi)[2],
                                             float scale_log2, float (&m)[2], float (&l)[2], float (&o)[HDP / 8][4]) {
  constexpr int LD = HDP + AT_PAD;
  const int lane = threadIdx.x & 31, g = lane >> 2, q = lane & 3;
  float s[AT_BN / 8][4];
#pragma unroll
  for (int i = 0; i < AT_BN / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
  for (int kk = 0; kk < HDP / 16; ++kk) {
    uint32_t a[4];
    ldmatrix_x4(a, qs + (size_t)((lane & 7) + 8 * ((lane >> 3) & 1)) * LD + kk * 16 + 8 * (lane >> 4));
#pragma unroll
    for (int nt = 0; nt < AT_BN / 16; ++nt) {
      uint32_t b[4];
      ldmatrix_x4(b, KV::at(ks, nt * 16 + (lane & 7) + 8 * (lane >> 4), kk * 16 + 8 * ((lane >> 3) & 1)));
      mma16816(s[2 * nt], a, b[0], b[1]);
      mma16816(s[2 * nt + 1], a, b[2], b[3]);
    }
  }
  // scale, mask, running max
  float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
  for (int i = 0; i < AT_BN / 8; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int key = key0 + i * 8 + q * 2 + (e & 1), r = e >> 1;
      const float v = (key >= row_lo[r] && key <= row_hi[r]) ? s[i][e] * scale_log2 : -INFINITY;
      s[i][e] = v;
      mx[r] = fmaxf(mx[r], v);
    }
  float corr[2], msafe[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
    const float mn = fmaxf(m[r], mx[r]);
    msafe[r] = mn == -INFINITY ? 0.f : mn;
    corr[r] = exp2f(m[r] - msafe[r]);          // m = -inf: 0
    m[r] = mn;
    l[r] *= corr[r];
  }
#pragma unroll
  for (int i = 0; i < HDP / 8; ++i) {
    o[i][0] *= corr[0]; o[i][1] *= corr[0]; o[i][2] *= corr[1]; o[i][3] *= corr[1];
  }
#pragma unroll
  for (int i = 0; i < AT_BN / 8; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float p = exp2f(s[i][e] - msafe[e >> 1]);
      s[i][e] = p;
      l[e >> 1] += p;
    }
  // O += P V
#pragma unroll
  for (int j = 0; j < AT_BN / 16; ++j) {
    uint32_t a[4];
    a[0] = pack_bf16(s[2 * j][0], s[2 * j][1]);
    a[1] = pack_bf16(s[2 * j][2], s[2 * j][3]);
    a[2] = pack_bf16(s[2 * j + 1][0], s[2 * j + 1][1]);
    a[3] = pack_bf16(s[2 * j + 1][2], s[2 * j + 1][3]);
#pragma unroll
    for (int dt = 0; dt < HDP / 16; ++dt) {
      uint32_t b[4];
      ldmatrix_x4_trans(b, KV::at(vs, j * 16 + (lane & 7) + 8 * ((lane >> 3) & 1), dt * 16 + 8 * (lane >> 4)));
      mma16816(o[2 * dt], a, b[0], b[1]);
      mma16816(o[2 * dt + 1], a, b[2], b[3]);
    }
  }
}

// ------------------------------------------------------------------------------------------------
// decode kernel: single query tokens against the cache, bound by reading K and V once.
//
// Persistent blocks (one per SM) of one PRODUCER warp and four CONSUMER warps around a ring of tiles
// in shared memory.  A tile is 64 keys of one (token, kv head): its K rows, V rows and the group's Q
// rows.  The producer resolves a batch of 32 candidate tiles at a time (token -> position -> page
// ids, all lanes in parallel, so the dependent loads are paid once per batch), then issues one bulk
// asynchronous copy per row (cp.async.bulk, completion counted on the tile's mbarrier).  Each
// consumer warp takes every fourth tile: S = Q K^T, softmax, P V on the tensor cores as in the span
// kernel, and leaves the tile's (max, sum, O) in the scratch; a merge kernel adds a token's tiles in
// index order.  Tile boundaries are multiples of 64 in absolute position, so a token's result does
// not depend on the batch.  The ring keeps several tiles in flight per SM whatever a single warp waits
// for.  Every wait is bounded.
// scratch: part_o float [n_dec][nq][n_splits_max][hd], part_ml float [n_dec][nq][n_splits_max][2]
// ------------------------------------------------------------------------------------------------
constexpr int AD_CONSUMERS = 4;
constexpr int AD_THREADS = (AD_CONSUMERS + 1) * 32;
constexpr int AD_MAX_STAGES = 8;
constexpr uint32_t AD_SPIN_LIMIT = 4u * 1000u * 1000u;
constexpr uint64_t AD_WAIT_NS = 200ull * 1000ull * 1000ull;

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ uint64_t global_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait: false when another warp gave up or the limit (iterations and 0.2 s) is reached.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = global_ns();
  for (uint32_t it = 0; it < AD_SPIN_LIMIT; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if ((it & 63u) == 63u && global_ns() - t0 > AD_WAIT_NS) break;
  }
  *abort_flag = 1;
  return false;
}
// one row, global -> shared, completion counted in bytes on the mbarrier; 16-byte aligned, size % 16 == 0
__device__ __forceinline__ void bulk_copy_row(void* dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

// one [box rows x 64 dims] box of a cache seen as a 2-D tensor [rows, head_dim]; no multicast
__device__ __forceinline__ void tma_load_tile(void* dst, const CUtensorMap* map, int dim0, int row, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(dim0), "r"(row), "r"(bar) : "memory");
}

struct AdDesc { int valid, z, kvh, split, pos, lo; };

// Elements of one ring stage: the Q rows (padded rows), then the K tile and the V tile.  With TMA the
// tiles are swizzled slabs and every part starts on a 1024-byte boundary.
__host__ __device__ constexpr size_t ad_q_elems(int hdp, int q_rows, bool tma) {
  return tma ? ((size_t)q_rows * (hdp + AT_PAD) + 511) / 512 * 512 : (size_t)q_rows * (hdp + AT_PAD);
}
__host__ __device__ constexpr size_t ad_tile_elems(int hdp, bool tma) {
  return tma ? (size_t)(hdp / 64) * AT_BN * 64 : (size_t)AT_BN * (hdp + AT_PAD);
}

// TMA: K and V tiles come as tensor loads of [rows of one page x 64 dims] boxes with the 128-byte swizzle
// (a page's keys of one kv head are contiguous rows of the cache seen as [pages*kv_heads*page_size, hd]):
// 16 requests per tile instead of 128 row copies.  Needs hd % 64 == 0 and a power-of-two page size.
template <int HDP, bool TMA>
__global__ void __launch_bounds__(AD_THREADS, 1)
attn_decode_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                   const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_cache,
                   const __nv_bfloat16* __restrict__ v_cache, float* __restrict__ part_o, float* __restrict__ part_ml,
                   const int* __restrict__ dec_tok, int n_dec, const int* __restrict__ tok_pos,
                   const int* __restrict__ tok_req, const int* __restrict__ block_table, int bt_stride, int nq, int nkv,
                   int hd, int page_size, int num_pages, float scale_log2, int window, int n_splits_max, int stages,
                   int q_rows, int* status) {
  constexpr int LD = HDP + AT_PAD;
  using KV = typename std::conditional<TMA, SwizzledKV, PaddedKV<HDP>>::type;
  extern __shared__ __align__(16) unsigned char smem_dyn[];
  unsigned char* smem_raw = reinterpret_cast<unsigned char*>(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
  __nv_bfloat16* ring = reinterpret_cast<__nv_bfloat16*>(smem_raw);       // [stages][Q | K tile | V tile]
  const size_t q_elems = ad_q_elems(HDP, q_rows, TMA), tile_elems = ad_tile_elems(HDP, TMA);
  const size_t stage_elems = q_elems + 2 * tile_elems;
  __shared__ uint64_t full[AD_MAX_STAGES], empty[AD_MAX_STAGES];
  __shared__ AdDesc desc[AD_MAX_STAGES];
  __shared__ int s_pages[32][AT_BN + 1];        // page ids of the producer's batch, one row per lane
  __shared__ int abort_word;
  volatile int* abort_flag = &abort_word;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int G = nq / nkv;

  // The ring starts as zeros: padding columns and Q rows past the group are never copied into, and a
  // tile's unused key rows only ever hold older (finite) keys.
  for (size_t i = tid; i < stage_elems * stages / 8; i += blockDim.x) reinterpret_cast<uint4*>(ring)[i] = make_uint4(0, 0, 0, 0);
  if (tid == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(smem_u32(&full[s]), 1);
      mbar_init(smem_u32(&empty[s]), 1);
    }
    abort_word = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // the zeros above before any bulk copy lands
  __syncthreads();

  const uint32_t row_bytes = (uint32_t)hd * 2u;
  if (warp == AD_CONSUMERS) {
    // ---------------- producer ----------------
    const long pairs = (long)n_dec * nkv, total = pairs * n_splits_max;
    long seq = 0;
    bool ok = true;
    // Candidate tiles are numbered split-major and dealt to the blocks round robin, so every block gets
    // the same mix of early and late tiles; a lane resolves one candidate, 32 at a time.
    for (long round = 0; blockIdx.x + round * 32 * (long)gridDim.x < total && ok; ++round) {
      const long item = blockIdx.x + (round * 32 + lane) * (long)gridDim.x;
      int valid = item < total, z = 0, kvh = 0, split = 0, pos = 0, lo = 0, t = 0, pi0 = 0;
      if (valid) {
        split = (int)(item / pairs);
        const int rem = (int)(item % pairs);
        z = rem / nkv;
        kvh = rem % nkv;
        t = dec_tok[z];
        pos = tok_pos[t];
        lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
        const int key0 = split * AT_BN;
        valid = key0 <= pos && key0 + AT_BN > lo;
        if (valid) {
          const int* bt = block_table + (size_t)tok_req[t] * bt_stride;
          const int last = min(pos, key0 + AT_BN - 1);
          pi0 = key0 / page_size;
          const int n_pi = last / page_size - pi0 + 1;
          for (int i = 0; i < n_pi; ++i) {
            const int pg = bt[pi0 + i];
            // a page wholly before the window may have been given back already: it is not read
            const bool needed = (pi0 + i + 1) * page_size > lo;
            if (needed && (pg < 0 || pg >= num_pages)) {
              qb_set_status(status, QB_STATUS_BAD_PAGE, pg, 6);
              valid = 0;
            }
            s_pages[lane][i] = pg;
          }
        }
      }
      __syncwarp();
      for (int src = 0; src < 32 && ok; ++src) {
        if (!__shfl_sync(0xffffffffu, valid, src)) continue;
        const int b_z = __shfl_sync(0xffffffffu, z, src), b_kvh = __shfl_sync(0xffffffffu, kvh, src);
        const int b_split = __shfl_sync(0xffffffffu, split, src), b_pos = __shfl_sync(0xffffffffu, pos, src);
        const int b_lo = __shfl_sync(0xffffffffu, lo, src), b_t = __shfl_sync(0xffffffffu, t, src);
        const int b_pi0 = __shfl_sync(0xffffffffu, pi0, src);
        const int slot = (int)(seq % stages);
        const uint32_t ph = (uint32_t)(seq / stages) & 1u;
        ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&empty[slot]), ph ^ 1u, abort_flag) ? 1 : 0);   // one answer per warp
        if (!ok) break;
        const int key0 = b_split * AT_BN;
        const int n_keys = min(AT_BN, b_pos - key0 + 1);
        const uint32_t bar = smem_u32(&full[slot]);
        __nv_bfloat16* qs = ring + (size_t)slot * stage_elems;
        __nv_bfloat16* ks = qs + q_elems;
        __nv_bfloat16* vs = ks + tile_elems;
        // boxes of the TMA path: rows of one page (or 64 rows of a larger page) x 64 dims
        const int box_rows = min(page_size, AT_BN), n_slabs = hd / 64;
        const int n_boxes = (n_keys + box_rows - 1) / box_rows;          // pages of the tile that hold visible keys
        // keys before the window are not fetched (their rows keep older, finite values and are masked)
        const int key_skip = b_lo > key0 ? b_lo - key0 : 0;
        const int box_first = key_skip / box_rows;
        if (lane == 0) {
          desc[slot] = AdDesc{1, b_z, b_kvh, b_split, b_pos, b_lo};
          const uint32_t kv_bytes = TMA ? (uint32_t)(2 * (n_boxes - box_first) * n_slabs * box_rows) * 128u
                                        : (uint32_t)(2 * (n_keys - key_skip)) * row_bytes;
          mbar_expect_tx(bar, (uint32_t)G * row_bytes + kv_bytes);
        }
        __syncwarp();
        for (int r = lane; r < G; r += 32)
          bulk_copy_row(qs + (size_t)r * LD, q + ((size_t)b_t * nq + b_kvh * G + r) * hd, row_bytes, bar);
        if (TMA) {
          for (int i = lane; i < 2 * (n_boxes - box_first) * n_slabs; i += 32) {
            const int which = i & 1, slab = (i >> 1) % n_slabs, box = box_first + (i >> 1) / n_slabs;
            const int key = key0 + box * box_rows;
            const int pg = s_pages[src][key / page_size - b_pi0];
            const int row = (pg * nkv + b_kvh) * page_size + key % page_size;       // row of the cache seen as 2-D
            __nv_bfloat16* dst = (which ? vs : ks) + (size_t)slab * (AT_BN * 64) + (size_t)box * box_rows * 64;
            tma_load_tile(dst, which ? &tm_v : &tm_k, slab * 64, row, bar);
          }
        } else {
          for (int r = key_skip + lane; r < n_keys; r += 32) {
            const int key = key0 + r;
            const int pg = s_pages[src][key / page_size - b_pi0];
            const size_t off = (((size_t)pg * nkv + b_kvh) * page_size + key % page_size) * hd;
            bulk_copy_row(ks + (size_t)r * LD, k_cache + off, row_bytes, bar);
            bulk_copy_row(vs + (size_t)r * LD, v_cache + off, row_bytes, bar);
          }
        }
        ++seq;
      }
      __syncwarp();
    }
    // a terminator in every slot: each consumer meets one on a slot of its own
    for (int c = 0; c < stages && ok; ++c, ++seq) {
      const int slot = (int)(seq % stages);
      const uint32_t ph = (uint32_t)(seq / stages) & 1u;
      ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&empty[slot]), ph ^ 1u, abort_flag) ? 1 : 0);
      if (!ok) break;
      if (lane == 0) {
        desc[slot] = AdDesc{0, 0, 0, 0, 0, 0};
        mbar_arrive(smem_u32(&full[slot]));
      }
      __syncwarp();
    }
    if (!ok) {
      // gave up: let the copies already issued land before the block's shared memory is given away
      const uint64_t t0 = global_ns();
      while (global_ns() - t0 < 2000000ull) __nanosleep(1000);
    }
  } else {
    // ---------------- consumers ----------------
    const int g = lane >> 2, qd = lane & 3;
    // A consumer owns the slots s with s % 4 == warp and sees every phase of them, in order: the
    // parity it waits for is then never more than one phase ahead of the barrier.
    for (long seq = 0; warp < stages; ++seq) {
      const int slot = (int)(seq % stages);
      if (slot % AD_CONSUMERS != warp) continue;
      const uint32_t ph = (uint32_t)(seq / stages) & 1u;
      if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&full[slot]), ph, abort_flag) ? 1 : 0)) break;
      const AdDesc d = desc[slot];
      if (!d.valid) {          // the terminator: give the slot back (the producer may still need it) and stop
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&empty[slot]));
        break;
      }
      const __nv_bfloat16* qs = ring + (size_t)slot * stage_elems;
      const __nv_bfloat16* ks = qs + q_elems;
      const __nv_bfloat16* vs = ks + tile_elems;
      const int key0 = d.split * AT_BN;
      for (int rb = 0; rb < G; rb += 16) {
        float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
        float o[HDP / 8][4];
#pragma unroll
        for (int i = 0; i < HDP / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
        int row_lo[2], row_hi[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          row_hi[r] = (rb + g + 8 * r < G) ? d.pos : -1;
          row_lo[r] = d.lo;
        }
        attend_block<HDP, KV>(qs + (size_t)rb * LD, ks, vs, key0, row_lo, row_hi, scale_log2, m, l, o);
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
          l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
          const int row = rb + g + 8 * r;
          if (row >= G) continue;
          const size_t at = ((size_t)d.z * nq + d.kvh * G + row) * n_splits_max + d.split;
          if (qd == 0) { part_ml[at * 2] = m[r]; part_ml[at * 2 + 1] = l[r]; }
#pragma unroll
          for (int i = 0; i < HDP / 8; ++i) {
            const int dd = i * 8 + qd * 2;
            if (dd < hd) *reinterpret_cast<float2*>(part_o + at * hd + dd) = make_float2(o[i][2 * r], o[i][2 * r + 1]);
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&empty[slot]));      // the tile's rows have been read: the slot is free
    }
  }
  __syncthreads();
  if (tid == 0 && abort_word) qb_set_status(status, QB_STATUS_WAIT_TIMEOUT, blockIdx.x, 6);
}

// ------------------------------------------------------------------------------------------------
// span kernel: prompt portions.  tiles[t] = {request row, first token row of the span, tokens in the
// span, first flattened row (token*G + head) of this tile}; grid (n_tiles, n_kv).
//
// One block = NC*16 query rows (a row is a (token, q head of the group) pair) of ONE request and ONE kv
// head, NC consumer warps of 16 rows each and one producer warp.  The producer streams the request's
// keys in blocks of 64 through a ring of K/V tiles in shared memory (TMA tensor loads, one box per
// page, or per-row bulk copies when the shapes do not allow TMA); consumers wait on a tile's mbarrier,
// run S = Q K^T, the online softmax and P V for their rows, and release the tile.  No block-wide
// barrier in the loop.  Each row is masked by its own token's position.
// ------------------------------------------------------------------------------------------------
constexpr int SP_MAX_PAGES = 2048;

template <int HDP, bool TMA, int NC>
__global__ void __launch_bounds__((NC + 1) * 32, 1)
attn_span_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                 const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_cache,
                 const __nv_bfloat16* __restrict__ v_cache, __nv_bfloat16* __restrict__ out,
                 const int* __restrict__ tok_pos, const int* __restrict__ block_table, int bt_stride,
                 const int* __restrict__ tiles, int nq, int nkv, int hd, int page_size, int num_pages,
                 float scale_log2, int window, int stages, int* status) {
  constexpr int LD = HDP + AT_PAD, BM = NC * 16;
  using KV = typename std::conditional<TMA, SwizzledKV, PaddedKV<HDP>>::type;
  extern __shared__ __align__(16) unsigned char smem_dyn[];
  unsigned char* smem_raw = reinterpret_cast<unsigned char*>(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
  const size_t q_elems = ad_q_elems(HDP, BM, TMA), tile_elems = ad_tile_elems(HDP, TMA);
  __nv_bfloat16* qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);         // [BM][LD]
  __nv_bfloat16* ring = qs + q_elems;                                      // [stages][K tile | V tile]
  __shared__ uint64_t full[AD_MAX_STAGES], empty[AD_MAX_STAGES];
  __shared__ int s_page[SP_MAX_PAGES];
  __shared__ int abort_word;
  volatile int* abort_flag = &abort_word;

  const int* tile = tiles + 4 * blockIdx.x;
  const int req = tile[0], tok0 = tile[1], n_tok = tile[2], row0 = tile[3];
  const int kvh = blockIdx.y, G = nq / nkv;
  const int n_rows = min(BM, n_tok * G - row0);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, qd = lane & 3;
  const int* bt = block_table + (size_t)req * bt_stride;

  const int first_tok = tok0 + row0 / G, last_tok = tok0 + (row0 + n_rows - 1) / G;
  const int key_end = tok_pos[last_tok];
  const int p_first = tok_pos[first_tok];
  const int key_begin = (window > 0 && p_first - window + 1 > 0) ? (p_first - window + 1) / AT_BN * AT_BN : 0;
  const int n_blocks = (key_end - key_begin) / AT_BN + 1;
  const int lo_min = (window > 0 && p_first - window + 1 > 0) ? p_first - window + 1 : 0;   // the lowest key any row reads

  // Q rows (zero past head_dim and past the last row), the ring as zeros, the page ids of the keys read
  for (int c = tid; c < BM * (HDP / 8); c += blockDim.x) {
    const int r = c / (HDP / 8), d = (c % (HDP / 8)) * 8;
    const int R = row0 + r;
    const bool ok = r < n_rows && d < hd;
    const __nv_bfloat16* src = q;
    if (ok) src = q + ((size_t)(tok0 + R / G) * nq + kvh * G + R % G) * hd + d;
    cp_async16(qs + (size_t)r * LD + d, src, ok);
  }
  cp_async_commit();
  for (size_t i = tid; i < 2 * tile_elems * stages / 8; i += blockDim.x) reinterpret_cast<uint4*>(ring)[i] = make_uint4(0, 0, 0, 0);
  int pi0 = key_begin / page_size;
  const int n_pi = key_end / page_size - pi0 + 1;
  const bool pages_in_smem = n_pi <= SP_MAX_PAGES;
  if (pages_in_smem)
    for (int i = tid; i < n_pi; i += blockDim.x) s_page[i] = bt[pi0 + i];
  if (tid == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(smem_u32(&full[s]), 1);
      mbar_init(smem_u32(&empty[s]), NC);
    }
    abort_word = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  cp_async_wait<0>();
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  __syncthreads();

  if (warp == NC) {
    // ---------------- producer ----------------
    const uint32_t row_bytes = (uint32_t)hd * 2u;
    const int box_rows = min(page_size, AT_BN), n_slabs = hd / 64;
    bool ok = true;
    for (int b = 0; b < n_blocks && ok; ++b) {
      const int slot = b % stages;
      const uint32_t ph = (uint32_t)(b / stages) & 1u;
      ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&empty[slot]), ph ^ 1u, abort_flag) ? 1 : 0);
      if (!ok) break;
      const int key0 = key_begin + b * AT_BN;
      const int n_keys = min(AT_BN, key_end - key0 + 1);
      const int n_boxes = (n_keys + box_rows - 1) / box_rows;
      const uint32_t bar = smem_u32(&full[slot]);
      __nv_bfloat16* ks = ring + (size_t)slot * 2 * tile_elems;
      __nv_bfloat16* vs = ks + tile_elems;
      // a page id outside the pool is recorded and its rows are not copied (the byte count must match);
      // keys before every row's window are not fetched: their pages may have been given back already
      int bad = 0;
      const int n_req = TMA ? 2 * n_boxes * n_slabs : n_keys;
      for (int i = lane; i < n_req; i += 32) {
        const int key = TMA ? key0 + ((i >> 1) / n_slabs) * box_rows : key0 + i;
        if ((TMA ? key + box_rows - 1 : key) < lo_min) { ++bad; continue; }
        const int pg = pages_in_smem ? s_page[key / page_size - pi0] : bt[key / page_size];
        if (pg < 0 || pg >= num_pages) { qb_set_status(status, QB_STATUS_BAD_PAGE, pg, 7); ++bad; }
      }
      bad = __reduce_add_sync(0xffffffffu, bad);
      if (lane == 0) {
        const uint32_t per = TMA ? (uint32_t)box_rows * 128u : 2u * row_bytes;
        mbar_expect_tx(bar, (uint32_t)(n_req - bad) * per);
      }
      __syncwarp();
      for (int i = lane; i < n_req; i += 32) {
        if (TMA) {
          const int which = i & 1, slab = (i >> 1) % n_slabs, box = (i >> 1) / n_slabs;
          const int key = key0 + box * box_rows;
          if (key + box_rows - 1 < lo_min) continue;
          const int pg = pages_in_smem ? s_page[key / page_size - pi0] : bt[key / page_size];
          if (pg < 0 || pg >= num_pages) continue;
          const int row = (pg * nkv + kvh) * page_size + key % page_size;
          __nv_bfloat16* dst = (which ? vs : ks) + (size_t)slab * (AT_BN * 64) + (size_t)box * box_rows * 64;
          tma_load_tile(dst, which ? &tm_v : &tm_k, slab * 64, row, bar);
        } else {
          const int key = key0 + i;
          if (key < lo_min) continue;
          const int pg = pages_in_smem ? s_page[key / page_size - pi0] : bt[key / page_size];
          if (pg < 0 || pg >= num_pages) continue;
          const size_t off = (((size_t)pg * nkv + kvh) * page_size + key % page_size) * hd;
          bulk_copy_row(ks + (size_t)i * LD, k_cache + off, row_bytes, bar);
          bulk_copy_row(vs + (size_t)i * LD, v_cache + off, row_bytes, bar);
        }
      }
    }
    if (!ok) {
      const uint64_t t0 = global_ns();
      while (global_ns() - t0 < 2000000ull) __nanosleep(1000);
    }
  } else {
    // ---------------- consumers: 16 rows each ----------------
    int row_lo[2], row_hi[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int lr = warp * 16 + g + 8 * r;
      if (lr < n_rows) {
        const int p = tok_pos[tok0 + (row0 + lr) / G];
        row_hi[r] = p;
        row_lo[r] = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
      } else {
        row_hi[r] = -1;
        row_lo[r] = 0;
      }
    }
    int any_hi = max(row_hi[0], row_hi[1]);
    any_hi = max(any_hi, __shfl_xor_sync(0xffffffffu, any_hi, 4));
    any_hi = max(any_hi, __shfl_xor_sync(0xffffffffu, any_hi, 8));
    any_hi = max(any_hi, __shfl_xor_sync(0xffffffffu, any_hi, 16));
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float o[HDP / 8][4];
#pragma unroll
    for (int i = 0; i < HDP / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    bool ok = true;
    for (int b = 0; b < n_blocks; ++b) {
      const int slot = b % stages;
      const uint32_t ph = (uint32_t)(b / stages) & 1u;
      ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&full[slot]), ph, abort_flag) ? 1 : 0);
      if (!ok) break;
      const int key0 = key_begin + b * AT_BN;
      const __nv_bfloat16* ks = ring + (size_t)slot * 2 * tile_elems;
      // a warp whose rows all end before this block has nothing to add
      if (any_hi >= key0)
        attend_block<HDP, KV>(qs + (size_t)warp * 16 * LD, ks, ks + tile_elems, key0, row_lo, row_hi, scale_log2, m, l, o);
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&empty[slot]));
    }
    if (ok) {
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
      }
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int lr = warp * 16 + g + 8 * r;
        if (lr >= n_rows) continue;
        const int R = row0 + lr;
        __nv_bfloat16* dst = out + ((size_t)(tok0 + R / G) * nq + kvh * G + R % G) * hd;
        const float inv = l[r] > 0.f ? 1.f / l[r] : 0.f;
#pragma unroll
        for (int i = 0; i < HDP / 8; ++i) {
          const int d = i * 8 + qd * 2;
          if (d < hd) *reinterpret_cast<uint32_t*>(dst + d) = pack_bf16(o[i][2 * r] * inv, o[i][2 * r + 1] * inv);
        }
      }
    }
  }
  __syncthreads();
  if (tid == 0 && abort_word) qb_set_status(status, QB_STATUS_WAIT_TIMEOUT, blockIdx.x, 7);
}

// out[t, head, :] = sum_s 2^(m_s - M) O_s / sum_s 2^(m_s - M) l_s over the splits that hold visible keys
__global__ void attn_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                  __nv_bfloat16* __restrict__ out, const int* __restrict__ dec_tok,
                                  const int* __restrict__ tok_pos, int nq, int hd, int window, int n_splits_max,
                                  int split_keys) {
  const int z = blockIdx.y, t = dec_tok[z], head = blockIdx.x;
  const int pos = tok_pos[t];
  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int s_first = lo / split_keys, s_last = min(pos / split_keys, n_splits_max - 1);
  const size_t base = ((size_t)z * nq + head) * n_splits_max;
  float M = -INFINITY;
  for (int s = s_first; s <= s_last; ++s) M = fmaxf(M, part_ml[(base + s) * 2]);
  for (int d = threadIdx.x; d < hd; d += blockDim.x) {
    float acc = 0.f, L = 0.f;
    for (int s = s_first; s <= s_last; ++s) {
      const float ms = part_ml[(base + s) * 2];
      const float f = ms == -INFINITY ? 0.f : exp2f(ms - M);
      acc += f * part_o[(base + s) * hd + d];
      L += f * part_ml[(base + s) * 2 + 1];
    }
    out[((size_t)t * nq + head) * hd + d] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}

// A cache [rows, hd] bfloat16 row-major, boxes of [box_rows, 64 dims], 128-byte swizzle
int make_kv_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t hd, uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return QB_ERR_UNSUPPORTED;
  const cuuint64_t dims[2] = {hd, rows};
  const cuuint64_t strides[1] = {hd * 2};
  const cuuint32_t box[2] = {64, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : QB_ERR_BAD_ARG;
}

template <typename Kern>
int set_smem(Kern kern, size_t smem) {
  if (smem > 32 * 1024) {      // the kernels also have static shared memory; the default limit counts both
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  return 0;
}

}  // namespace

// Query rows (token x head of the group) per tile of the span kernel, for a head size.
extern "C" int qb_attn_span_rows(int hd) { return hd <= 128 ? 128 : 64; }

extern "C" int qb_attn_span(const void* q, const void* k_cache, const void* v_cache, void* out, const int* tok_pos,
                            const int* block_table, int bt_stride, const int* tiles, int n_tiles, int nq, int nkv,
                            int hd, int page_size, int num_pages, float scale, int window, int* status,
                            cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  if (hd % 16 || hd > 256 || hd <= 0 || nq % nkv || nkv > 65535) return QB_ERR_UNSUPPORTED;
  const float scale_log2 = scale * 1.4426950408889634f;
  dim3 grid(n_tiles, nkv);
  const bool pow2 = (page_size & (page_size - 1)) == 0;
  const bool tma = hd % 64 == 0 && pow2 && (page_size <= AT_BN || page_size % AT_BN == 0) && encode_fn() != nullptr &&
                   (((uintptr_t)k_cache | (uintptr_t)v_cache) & 15) == 0;
  CUtensorMap tm_k, tm_v;
  memset(&tm_k, 0, sizeof(tm_k));
  memset(&tm_v, 0, sizeof(tm_v));
  if (tma) {
    const uint64_t rows = (uint64_t)num_pages * nkv * page_size;
    const uint32_t box_rows = (uint32_t)(page_size < AT_BN ? page_size : AT_BN);
    int rc = make_kv_map(&tm_k, k_cache, rows, (uint64_t)hd, box_rows);
    if (rc == 0) rc = make_kv_map(&tm_v, v_cache, rows, (uint64_t)hd, box_rows);
    if (rc) return rc;
  }
#define QB_SPAN(HDP, TMA_, NC_)                                                                            \
  do {                                                                                                     \
    const size_t q_bytes = ad_q_elems(HDP, NC_ * 16, TMA_) * 2, stage_bytes = 2 * ad_tile_elems(HDP, TMA_) * 2; \
    int stages = (int)(((size_t)(192 * 1024) - q_bytes) / stage_bytes);                                    \
    if (stages > AD_MAX_STAGES) stages = AD_MAX_STAGES;                                                    \
    if (stages < 2) return QB_ERR_UNSUPPORTED;                                                             \
    const size_t smem = q_bytes + stage_bytes * stages + 1024;                                             \
    int rc = set_smem(attn_span_kernel<HDP, TMA_, NC_>, smem);                                             \
    if (rc) return rc;                                                                                     \
    attn_span_kernel<HDP, TMA_, NC_><<<grid, (NC_ + 1) * 32, smem, stream>>>(                              \
        tm_k, tm_v, (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache,  \
        (__nv_bfloat16*)out, tok_pos, block_table, bt_stride, tiles, nq, nkv, hd, page_size, num_pages,     \
        scale_log2, window, stages, status);                                                               \
  } while (0)
  if (tma) {
    if (hd <= 64) QB_SPAN(64, true, 8);
    else if (hd <= 128) QB_SPAN(128, true, 8);
    else QB_SPAN(256, true, 4);
  } else {
    if (hd <= 64) QB_SPAN(64, false, 8);
    else if (hd <= 128) QB_SPAN(128, false, 8);
    else QB_SPAN(256, false, 4);
  }
#undef QB_SPAN
  QB_LAUNCH_CHECK();
  return 0;
}

// Keys per decode split for a head size (the Python side sizes the scratch with it).
extern "C" int qb_attn_decode_split_keys(int hd) { (void)hd; return AT_BN; }

// Scratch, in floats: part_o n_dec*nq*n_splits_max*hd, part_ml n_dec*nq*n_splits_max*2, where
// n_splits_max >= ceil(longest context / split keys).
extern "C" int qb_attn_decode(const void* q, const void* k_cache, const void* v_cache, void* out, float* part_o,
                              float* part_ml, const int* dec_tok, int n_dec, const int* tok_pos, const int* tok_req,
                              const int* block_table, int bt_stride, int nq, int nkv, int hd, int page_size,
                              int num_pages, float scale, int window, int n_splits_max, int* status,
                              cudaStream_t stream) {
  if (n_dec <= 0) return 0;
  if (hd % 16 || hd > 256 || hd <= 0 || nq % nkv || nkv > 65535 || n_dec > 65535 || n_splits_max <= 0)
    return QB_ERR_UNSUPPORTED;
  const float scale_log2 = scale * 1.4426950408889634f;
  const int split_keys = AT_BN;
  const int G = nq / nkv, q_rows = (G + 15) / 16 * 16;
  int dev = 0, sms = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err == cudaSuccess) err = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (err != cudaSuccess) return (int)err;
  const long total = (long)n_dec * nkv * n_splits_max;
  const int blocks = (int)(total < sms ? total : sms);
  // TMA tensor loads when the shapes allow (whole 64-dim slabs, pages that tile 64 keys), else row copies
  const bool pow2 = (page_size & (page_size - 1)) == 0;
  const bool tma = hd % 64 == 0 && pow2 && (page_size <= AT_BN || page_size % AT_BN == 0) && encode_fn() != nullptr &&
                   (((uintptr_t)k_cache | (uintptr_t)v_cache) & 15) == 0;
  CUtensorMap tm_k, tm_v;
  memset(&tm_k, 0, sizeof(tm_k));
  memset(&tm_v, 0, sizeof(tm_v));
  if (tma) {
    const uint64_t rows = (uint64_t)num_pages * nkv * page_size;
    const uint32_t box_rows = (uint32_t)(page_size < AT_BN ? page_size : AT_BN);
    int rc = make_kv_map(&tm_k, k_cache, rows, (uint64_t)hd, box_rows);
    if (rc == 0) rc = make_kv_map(&tm_v, v_cache, rows, (uint64_t)hd, box_rows);
    if (rc) return rc;
  }
#define QB_DEC(HDP, TMA_)                                                                                  \
  do {                                                                                                     \
    const size_t stage_bytes = (ad_q_elems(HDP, q_rows, TMA_) + 2 * ad_tile_elems(HDP, TMA_)) * 2;         \
    int stages = (int)((size_t)(194 * 1024) / stage_bytes);                                                \
    stages = stages >= 8 ? 8 : (stages >= 4 ? 4 : stages);   /* a multiple of the consumers: equal shares */ \
    if (stages < 2) return QB_ERR_UNSUPPORTED;                                                             \
    const size_t smem = stage_bytes * stages + 1024;         /* room to align the ring to 1024 bytes */    \
    int rc = set_smem(attn_decode_kernel<HDP, TMA_>, smem);                                                \
    if (rc) return rc;                                                                                     \
    attn_decode_kernel<HDP, TMA_><<<blocks, AD_THREADS, smem, stream>>>(                                   \
        tm_k, tm_v, (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, \
        part_o, part_ml, dec_tok, n_dec, tok_pos, tok_req, block_table, bt_stride, nq, nkv, hd, page_size, \
        num_pages, scale_log2, window, n_splits_max, stages, q_rows, status);                              \
  } while (0)
  if (tma) {
    if (hd <= 64) QB_DEC(64, true);
    else if (hd <= 128) QB_DEC(128, true);
    else QB_DEC(256, true);
  } else {
    if (hd <= 64) QB_DEC(64, false);
    else if (hd <= 128) QB_DEC(128, false);
    else QB_DEC(256, false);
  }
#undef QB_DEC
  attn_merge_kernel<<<dim3(nq, n_dec), 128, 0, stream>>>(part_o, part_ml, (__nv_bfloat16*)out, dec_tok, tok_pos, nq,
                                                         hd, window, n_splits_max, split_keys);
  QB_LAUNCH_CHECK();
  return 0;
}

// ------------------------------------------------------------------------------------------------
// The same decode attention for callers that cannot allocate: the scratch is a static device array.
// (No counterpart in the reference; contract and reasons in no_alloc.h.)
// ------------------------------------------------------------------------------------------------
#include "no_alloc.h"

// Partial results of the split-key kernel for one call at a time.  Host code must not hand this
// name to a kernel: on the host it is only a stand-in for the symbol; the device address is looked
// up once per device below.
static __device__ __align__(256) float qb_noalloc_scratch[QB_NOALLOC_SCRATCH_FLOATS];

namespace {
constexpr int NOALLOC_MAX_DEVICES = 64;
float* g_noalloc_ptr[NOALLOC_MAX_DEVICES] = {};
}  // namespace

extern "C" long long qb_attn_decode_noalloc_floats(int n_dec, int nq, int hd, int n_splits_max) {
  if (n_dec <= 0 || nq <= 0 || hd <= 0 || n_splits_max <= 0) return 0;
  return (long long)n_dec * nq * n_splits_max * (hd + 2);
}

extern "C" long long qb_attn_decode_noalloc_capacity(void) { return (long long)QB_NOALLOC_SCRATCH_FLOATS; }

extern "C" int qb_attn_decode_noalloc(const void* q, const void* k_cache, const void* v_cache, void* out,
                                      const int* dec_tok, int n_dec, const int* tok_pos, const int* tok_req,
                                      const int* block_table, int bt_stride, int nq, int nkv, int hd, int page_size,
                                      int num_pages, float scale, int window, int n_splits_max, int* status,
                                      cudaStream_t stream) {
  if (n_dec <= 0) return 0;
  if (nq <= 0 || hd <= 0 || n_splits_max <= 0) return QB_ERR_BAD_ARG;
  const long long need = qb_attn_decode_noalloc_floats(n_dec, nq, hd, n_splits_max);
  if (need > (long long)QB_NOALLOC_SCRATCH_FLOATS) return QB_NOALLOC_TOO_LARGE;
  int dev = -1;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return (int)err;
  if (dev < 0 || dev >= NOALLOC_MAX_DEVICES) return QB_ERR_UNSUPPORTED;
  if (g_noalloc_ptr[dev] == nullptr) {
    // first call on this device (which is current): the array's address in this device's memory
    float* p = nullptr;
    err = cudaGetSymbolAddress((void**)&p, qb_noalloc_scratch);
    if (err != cudaSuccess) return (int)err;
    if (p == nullptr) return QB_ERR_UNSUPPORTED;
    g_noalloc_ptr[dev] = p;
  }
  float* part_o = g_noalloc_ptr[dev];
  // the (max, sum) pairs follow the partial outputs; the offset keeps them 8-byte aligned
  float* part_ml = part_o + (size_t)n_dec * nq * n_splits_max * hd;
  return qb_attn_decode(q, k_cache, v_cache, out, part_o, part_ml, dec_tok, n_dec, tok_pos, tok_req, block_table,
                        bt_stride, nq, nkv, hd, page_size, num_pages, scale, window, n_splits_max, status, stream);
}
