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
//  * decode kernel: the 64-key tiles of all single tokens form one list that persistent blocks cut
//    into equal ranges; in a block a producer warp streams the tiles through a ring in shared memory
//    (TMA, one box per page) and four consumer warps share each tile, keeping their running softmax
//    state in registers along a (token, kv head) pair; pairs that a range boundary cuts leave partial
//    results that a small merge kernel adds.
//
// (src/quanta/minimax/attention.py:194-203: scores * head_dim^-0.5, causal mask, softmax in float32,
// probabilities cast to the activation dtype, P V; q head h reads kv head h / (n_q / n_kv).)
// head_dim: any multiple of 16 up to 256 (template padding 64 / 128 / 256, dims past head_dim are zero).
#include <cuda.h>

#include <cstdlib>
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

// One warp: 16 query rows against NK keys (rows koff .. koff+NK-1 of a tile) held in shared memory.
//   qs: the warp's 16 rows [16][HDP+PAD]; ks, vs: a tile of AT_BN keys
//   row_hi[2], row_lo[2]: last / first visible key of the thread's two rows (g and g+8), absolute
//   key0: absolute position of tile row koff.   m, l, o: running max (log2 domain), partial sum, output.
// How a K or V tile of 64 keys lies in shared memory.
//  PaddedKV:   rows of HDP + 8 elements (what cp.async / per-row bulk copies write).
//  SwizzledKV: what 2-D TMA tensor loads with the 128-byte swizzle write: head_dim in slabs of 64 dims, each
//              slab [64 keys][64 dims] with rows of 128 bytes whose 16-byte chunks are XORed with (row & 7);
//              the tile is 1024-byte aligned.  Free of bank conflicts for ldmatrix, like PaddedKV.
//  BoxedKV:    what 3-D TMA tensor loads write when ONE box is a whole page of a kv head (all slabs), so that
//              a tile needs few requests.  A tile is its boxes one after the other.  Inside a box either the
//              slabs follow one another, each [box rows][64 dims] (slab-major: conflict-free from 8 rows a
//              box on), or a key's slabs lie side by side (interleaved: two-way conflicts for ldmatrix when
//              the number of slabs is even).  Lines of 128 bytes, chunks XORed with (line & 7).
template <int HDP>
struct PaddedKV {
  __device__ __forceinline__ const __nv_bfloat16* at(const __nv_bfloat16* base, int row, int dim) const {
    return base + (size_t)row * (HDP + AT_PAD) + dim;
  }
};
struct SwizzledKV {
  __device__ __forceinline__ const __nv_bfloat16* at(const __nv_bfloat16* base, int row, int dim) const {
    const int chunk = (dim & 63) >> 3;
    return base + (dim >> 6) * (AT_BN * 64) + row * 64 + ((chunk ^ (row & 7)) << 3) + (dim & 7);
  }
};
template <int NS>
struct BoxedKV {
  int box_shift;       // log2 of the rows of a box
  int slab_major;
  __device__ __forceinline__ const __nv_bfloat16* at(const __nv_bfloat16* base, int row, int dim) const {
    const int slab = dim >> 6;
    const int line = slab_major ? ((((row >> box_shift) * NS + slab) << box_shift) + (row & ((1 << box_shift) - 1)))
                                : row * NS + slab;
    return base + line * 64 + ((((dim & 63) >> 3) ^ (line & 7)) << 3) + (dim & 7);
  }
};

// QREG: the Q rows are already MMA fragments in registers (qf[k step][4]) and qs is not read.
template <int HDP, typename KV = PaddedKV<HDP>, int NK = AT_BN, bool QREG = false>
__device__ __forceinline__ void attend_block(const __nv_bfloat16* qs, const __nv_bfloat16* ks, const __nv_bfloat16* vs,
                                             int key0, const int (&row_lo)[2], const int (&row_hi)[2],
                                             float scale_log2, float (&m)[2], float (&l)[2], float (&o)[HDP / 8][4],
                                             int koff = 0, const uint32_t (*qf)[4] = nullptr, const KV kv = KV()) {
  constexpr int LD = HDP + AT_PAD;
  const int lane = threadIdx.x & 31, g = lane >> 2, q = lane & 3;
  float s[NK / 8][4];
#pragma unroll
  for (int i = 0; i < NK / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
  if (NK == 16) {
    // two keys' worth of accumulators only: sum the even and the odd 16-dim steps apart, so that two
    // chains of dependent MMAs run at a time instead of one
    float s2[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
    for (int kk = 0; kk < HDP / 16; ++kk) {
      uint32_t a[4], b[4];
      if (QREG) { a[0] = qf[kk][0]; a[1] = qf[kk][1]; a[2] = qf[kk][2]; a[3] = qf[kk][3]; }
      else ldmatrix_x4(a, qs + (size_t)((lane & 7) + 8 * ((lane >> 3) & 1)) * LD + kk * 16 + 8 * (lane >> 4));
      ldmatrix_x4(b, kv.at(ks, koff + (lane & 7) + 8 * (lane >> 4), kk * 16 + 8 * ((lane >> 3) & 1)));
      if (kk & 1) {
        mma16816(s2[0], a, b[0], b[1]);
        mma16816(s2[1], a, b[2], b[3]);
      } else {
        mma16816(s[0], a, b[0], b[1]);
        mma16816(s[1], a, b[2], b[3]);
      }
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) { s[0][e] += s2[0][e]; s[1][e] += s2[1][e]; }
  } else {
#pragma unroll
    for (int kk = 0; kk < HDP / 16; ++kk) {
      uint32_t a[4];
      if (QREG) { a[0] = qf[kk][0]; a[1] = qf[kk][1]; a[2] = qf[kk][2]; a[3] = qf[kk][3]; }
      else ldmatrix_x4(a, qs + (size_t)((lane & 7) + 8 * ((lane >> 3) & 1)) * LD + kk * 16 + 8 * (lane >> 4));
#pragma unroll
      for (int nt = 0; nt < NK / 16; ++nt) {
        uint32_t b[4];
        ldmatrix_x4(b, kv.at(ks, koff + nt * 16 + (lane & 7) + 8 * (lane >> 4), kk * 16 + 8 * ((lane >> 3) & 1)));
        mma16816(s[2 * nt], a, b[0], b[1]);
        mma16816(s[2 * nt + 1], a, b[2], b[3]);
      }
    }
  }
  // scale, mask, running max
  float mx[2] = {-INFINITY, -INFINITY};
  // far from the ends of a request every key of the block is visible to every row: no compares then
  const bool all_visible = __all_sync(0xffffffffu, key0 >= max(row_lo[0], row_lo[1]) &&
                                                   key0 + NK - 1 <= min(row_hi[0], row_hi[1]));
  if (all_visible) {
#pragma unroll
    for (int i = 0; i < NK / 8; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        s[i][e] *= scale_log2;
        mx[e >> 1] = fmaxf(mx[e >> 1], s[i][e]);
      }
  } else {
#pragma unroll
    for (int i = 0; i < NK / 8; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = key0 + i * 8 + q * 2 + (e & 1), r = e >> 1;
        const float v = (key >= row_lo[r] && key <= row_hi[r]) ? s[i][e] * scale_log2 : -INFINITY;
        s[i][e] = v;
        mx[r] = fmaxf(mx[r], v);
      }
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
  // most blocks leave the running maximum where it was: nothing to rescale then
  if (__any_sync(0xffffffffu, corr[0] != 1.f || corr[1] != 1.f)) {
#pragma unroll
    for (int i = 0; i < HDP / 8; ++i) {
      o[i][0] *= corr[0]; o[i][1] *= corr[0]; o[i][2] *= corr[1]; o[i][3] *= corr[1];
    }
  }
#pragma unroll
  for (int i = 0; i < NK / 8; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float p = exp2f(s[i][e] - msafe[e >> 1]);
      s[i][e] = p;
      l[e >> 1] += p;
    }
  // O += P V
#pragma unroll
  for (int j = 0; j < NK / 16; ++j) {
    uint32_t a[4];
    a[0] = pack_bf16(s[2 * j][0], s[2 * j][1]);
    a[1] = pack_bf16(s[2 * j][2], s[2 * j][3]);
    a[2] = pack_bf16(s[2 * j + 1][0], s[2 * j + 1][1]);
    a[3] = pack_bf16(s[2 * j + 1][2], s[2 * j + 1][3]);
#pragma unroll
    for (int dt = 0; dt < HDP / 16; ++dt) {
      uint32_t b[4];
      ldmatrix_x4_trans(b, kv.at(vs, koff + j * 16 + (lane & 7) + 8 * ((lane >> 3) & 1), dt * 16 + 8 * (lane >> 4)));
      mma16816(o[2 * dt], a, b[0], b[1]);
      mma16816(o[2 * dt + 1], a, b[2], b[3]);
    }
  }
}

// ------------------------------------------------------------------------------------------------
// decode kernel: single query tokens against the cache, bound by reading K and V once.
//
// The work is the list of all 64-key tiles of all (token, kv head) pairs, token-major.  Persistent
// blocks (one per SM) cut that list into equal contiguous ranges (a block's range may begin and end
// inside a pair), so every SM reads the same number of bytes whatever the mix of context lengths.
// A block is two PRODUCER warps and four CONSUMER warps around a ring of tiles in shared memory.  A tile
// is 64 keys of one pair: its K rows, V rows and the group's Q rows.  Starting a tensor load holds the
// issuing warp for a time that grows with the bytes, and one warp that issues all of a tile's boxes is slower
// than the consumers and than memory; so one producer issues the Q rows and the K boxes and the other the V
// boxes, each counting its own bytes on the tile's barrier.  Each producer resolves 32 tiles at
// a time (pair by binary search in a prefix sum of the tokens' tile counts held in shared memory, then
// the page ids, all lanes in parallel) and issues TMA tensor loads (one box per page) or, where the
// shapes do not allow them, one bulk copy per row; completion is counted on the tile's mbarrier.
// The four consumers work on the SAME tile: with up to 16 q heads per kv head each takes 16 of its 64
// keys (17..32 heads: two row blocks x two key halves; 33..64: a row block each), so a tile is consumed
// in a fraction of the time it takes to arrive, and they keep their running (max, sum, O) in registers
// over the consecutive tiles of a pair.  Where the block's range leaves a pair the consumers merge
// their parts through the tile's shared memory and write ONE partial result for the segment, or the
// final output if the segment is the whole pair; a small merge kernel adds the segments of the pairs that
// were cut.  At most (pairs + blocks) partials are written whatever the context length.  A token's result
// depends on the batch only through the order of these float32 additions.  Every wait is bounded.
//
// scratch: part_o float [n_dec][nq][n_parts][hd], part_ml float [n_dec][nq][n_parts][2]; the last of
// the n_parts entries of a row holds, as an integer, how many segments the merge kernel has to add
// (0: the output is already final).
// ------------------------------------------------------------------------------------------------
constexpr int AD_CONSUMERS = 4;
constexpr int AD_PRODUCERS = 2;      // one issues the Q rows and the K boxes of a tile, the other its V boxes
constexpr int AD_THREADS = (AD_CONSUMERS + AD_PRODUCERS) * 32;
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
// Bounded wait: false when another warp gave up or the limit (iterations and 0.2 s) is reached.  The
// clock and the abort flag are read only now and then: a read of the global timer costs more than
// most waits last.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  uint64_t t0 = 0;
  for (uint32_t it = 0; it < AD_SPIN_LIMIT; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 127u) == 127u) {
      if (*abort_flag) return false;
      const uint64_t now = global_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > AD_WAIT_NS) break;
    }
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
// one box of whole rows (all slabs of 64 dims) of a cache seen as a 3-D tensor whose middle and outer
// dimensions are (rows, slabs) when slab-major, (slabs, rows) when interleaved; no multicast
__device__ __forceinline__ void tma_load_rows(void* dst, const CUtensorMap* map, int row, int slab_major, uint32_t bar) {
  const int c1 = slab_major ? row : 0, c2 = slab_major ? 0 : row;
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(0), "r"(c1), "r"(c2), "r"(bar) : "memory");
}
template <int H> __device__ __forceinline__ PaddedKV<H> make_kv(PaddedKV<H>*, int, int) { return PaddedKV<H>(); }
template <int NS> __device__ __forceinline__ BoxedKV<NS> make_kv(BoxedKV<NS>*, int box_shift, int slab_major) {
  return BoxedKV<NS>{box_shift, slab_major};
}

constexpr int AD_MAX_DEC = 256;      // tokens per launch: their positions and tile counts live in shared memory
constexpr int AD_FIRST = 1, AD_LAST = 2, AD_WHOLE = 4, AD_PAIR_END = 8;

// One tile of the block's range.  valid: 1 a tile, 2 a tile that is passed over (a page id outside the
// pool; the status word says so).  flags: the first / last tile of a segment (the part of a pair inside
// this block's range), whether that segment is the whole pair, whether the tile ends its pair.
// qslot: where in the ring of Q rows the pair's queries lie.  48 bytes, read as three 16-byte words.
struct __align__(16) AdDesc { int valid, z, tok, kvh, key0, pos, lo, flags, seg, pi0, qslot, pad; };

// Elements of the Q rows of one tile (span kernel: of the block), and of a K or V tile.  With TMA the
// tiles are swizzled slabs and start on 1024-byte boundaries.
__host__ __device__ constexpr size_t ad_q_elems(int hdp, int q_rows, bool tma) {
  return tma ? ((size_t)q_rows * (hdp + AT_PAD) + 511) / 512 * 512 : (size_t)q_rows * (hdp + AT_PAD);
}
__host__ __device__ constexpr size_t ad_tile_elems(int hdp, bool tma) {
  return tma ? (size_t)(hdp / 64) * AT_BN * 64 : (size_t)AT_BN * (hdp + AT_PAD);
}
// Q rows kept per pair: a multiple of 8 up to 16 heads (the MMA reads 16 rows; the rows past them
// belong to the next entry of the ring, or to 8 rows of zeros after the last, and are masked), else
// whole row blocks of 16.
__host__ __device__ constexpr int ad_q_rows(int group) { return group <= 16 ? (group + 7) / 8 * 8 : (group + 15) / 16 * 16; }

__device__ __forceinline__ int ad_tiles_of(int pos, int window) {
  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  return pos / AT_BN - lo / AT_BN + 1;
}

// TMA: K and V tiles come as tensor loads of one box per page, [rows of the page][head_dim], with the
// 128-byte swizzle (a page's keys of one kv head are contiguous rows of the cache seen as
// [pages*kv_heads*page_size][hd / 64][64]): 8 requests per tile with pages of 16 keys, 2 with pages of 64,
// instead of 128 row copies.  An instruction that starts a tensor load holds the issuing warp for some
// tens of cycles, so their number per tile decides how fast a producer can go.  Needs a head size of 64,
// 128 or 256 and a power-of-two page size.
template <int HDP, bool TMA>
__global__ void __launch_bounds__(AD_THREADS, 1)
attn_decode_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                   const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_cache,
                   const __nv_bfloat16* __restrict__ v_cache, __nv_bfloat16* __restrict__ out,
                   float* __restrict__ part_o, float* __restrict__ part_ml, const int* __restrict__ dec_tok, int n_dec,
                   const int* __restrict__ tok_pos, const int* __restrict__ tok_req,
                   const int* __restrict__ block_table, int bt_stride, int nq, int nkv, int hd, int page_size,
                   int num_pages, float scale_log2, int window, int n_parts, int stages, int pages_ld,
                   int slab_major, int* status) {
  constexpr int LD = HDP + AT_PAD;
  using KV = typename std::conditional<TMA, BoxedKV<HDP / 64>, PaddedKV<HDP>>::type;
  extern __shared__ __align__(16) unsigned char smem_dyn[];
  unsigned char* smem_raw = reinterpret_cast<unsigned char*>(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
  const int G = nq / nkv, q_rows = ad_q_rows(G), q_slots = stages + 1;
  const size_t tile_elems = ad_tile_elems(HDP, TMA);
  __nv_bfloat16* ring = reinterpret_cast<__nv_bfloat16*>(smem_raw);          // [stages][K tile | V tile]
  __nv_bfloat16* qring = ring + (size_t)stages * 2 * tile_elems;             // [q_slots][q_rows][LD], then 8 zero rows
  int* s_pos = reinterpret_cast<int*>(qring + ((size_t)q_slots * q_rows + 8) * LD);   // [AD_MAX_DEC] position of token z
  int* s_req = s_pos + AD_MAX_DEC;                                           // its block-table row
  int* s_tok = s_req + AD_MAX_DEC;                                           // its row among the step's tokens
  int* s_cum = s_tok + AD_MAX_DEC;                                           // [AD_MAX_DEC + 1] tiles of the tokens before z
  int* s_pages_all = s_cum + AD_MAX_DEC + 1;                                 // [producers][32][pages_ld] page ids of a batch
  __shared__ uint64_t full[AD_MAX_STAGES], empty[AD_MAX_STAGES], cbar;
  __shared__ AdDesc s_desc[2][32];            // the tiles of a batch of 32, double-buffered (the first producer's)
  __shared__ AdDesc s_desc_v[2][32];          // the second producer's own copy
  __shared__ float s_ml[AD_CONSUMERS][16][2];
  __shared__ float s_fw[AD_CONSUMERS][16];    // segment end: the weight of each warp's part of a row
  __shared__ float s_row[16 * AD_CONSUMERS][4];     // and the row's (max, sum, 1 / sum)
  __shared__ int abort_word;
  volatile int* abort_flag = &abort_word;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  for (int z = tid; z < n_dec; z += blockDim.x) {
    const int t = dec_tok[z];
    s_tok[z] = t;
    s_pos[z] = tok_pos[t];
    s_req[z] = tok_req[t];
  }
  // The rings start as zeros: padding columns and Q rows past the group are never copied into, and a
  // tile's unused key rows only ever hold older (finite) keys or zeros.
  {
    const size_t n16 = ((size_t)stages * 2 * tile_elems + ((size_t)q_slots * q_rows + 8) * LD) / 8;
    for (size_t i = tid; i < n16; i += blockDim.x) reinterpret_cast<uint4*>(ring)[i] = make_uint4(0, 0, 0, 0);
  }
  if (tid == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(smem_u32(&full[s]), AD_PRODUCERS);
      mbar_init(smem_u32(&empty[s]), AD_CONSUMERS);
    }
    mbar_init(smem_u32(&cbar), AD_CONSUMERS);
    abort_word = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (warp == 0) {
    // exclusive prefix sum of the tokens' tile counts
    const int per = (n_dec + 31) / 32, z0 = lane * per, z1 = min(n_dec, z0 + per);
    int sum = 0;
    for (int z = z0; z < z1; ++z) sum += ad_tiles_of(s_pos[z], window);
    int incl = sum;
    for (int off = 1; off < 32; off <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, off);
      if (lane >= off) incl += v;
    }
    int run = incl - sum;
    for (int z = z0; z < z1; ++z) {
      s_cum[z] = run;
      run += ad_tiles_of(s_pos[z], window);
    }
    if (lane == 31) s_cum[n_dec] = incl;
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // the zeros above before any bulk copy lands
  __syncthreads();

  // this block's range of the tile list
  const long T = (long)nkv * s_cum[n_dec];
  const long A = T < (long)gridDim.x ? T : (long)gridDim.x;
  const long b = blockIdx.x;
  const long start = b < A ? b * T / A : 0, end = b < A ? (b + 1) * T / A : 0;
  const int n_tiles = (int)(end - start);

  const uint32_t row_bytes = (uint32_t)hd * 2u;
  if (warp >= AD_CONSUMERS) {
    // ---------------- producers: both resolve the same tiles; `which` 0 issues Q and K, 1 issues V ----------------
    const int which = warp - AD_CONSUMERS;
    int* s_pages = s_pages_all + which * 32 * pages_ld;
    AdDesc (*my_desc)[32] = which == 0 ? s_desc : s_desc_v;
    bool ok = true;
    int slot = 0, q_count = 0;
    uint32_t phase = 0;
    const int box_rows = min(page_size, AT_BN);
    const int page_shift = 31 - __clz(page_size), box_shift = 31 - __clz(box_rows);     // TMA path: powers of two
    // page ids of a tile fit four registers when pages are powers of two of at least 16 keys: then the
    // next batch's ids are fetched while this batch is being issued
    const bool few_pages = (page_size & (page_size - 1)) == 0 && page_size >= 16;
    AdDesc nd;                       // this lane's tile of the batch being resolved
    int npg[4] = {0, 0, 0, 0};
    auto resolve = [&](int first_tile) {
      const int n = first_tile + lane;
      nd = AdDesc{0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0};
      if (n < n_tiles) {
        const long gt = start + n;
        int a = 0, c = n_dec;                   // nkv * s_cum[a] <= gt < nkv * s_cum[c]
        while (c - a > 1) {
          const int mid = (a + c) >> 1;
          if ((long)nkv * s_cum[mid] <= gt) a = mid; else c = mid;
        }
        nd.valid = 1;
        nd.z = a;
        nd.tok = s_tok[a];
        nd.pos = s_pos[a];
        nd.lo = (window > 0 && nd.pos - window + 1 > 0) ? nd.pos - window + 1 : 0;
        const int cnt = s_cum[a + 1] - s_cum[a];
        const long base = (long)nkv * s_cum[a];
        const int rem = (int)(gt - base);
        nd.kvh = rem / cnt;
        const int i = rem - nd.kvh * cnt;
        nd.key0 = (nd.lo / AT_BN + i) * AT_BN;
        const long g0 = base + (long)nd.kvh * cnt, g1 = g0 + cnt - 1;      // the pair's first and last tile
        nd.flags = ((n == 0 || i == 0) ? AD_FIRST : 0) | ((n == n_tiles - 1 || i == cnt - 1) ? AD_LAST : 0) |
                   ((g0 >= start && g1 < end) ? AD_WHOLE : 0) | (i == cnt - 1 ? AD_PAIR_END : 0);
        nd.seg = (int)(b - ((g0 + 1) * A - 1) / T);      // blocks since the one that holds the pair's first tile
        nd.pi0 = nd.key0 / page_size;
        if (few_pages) {
          const int* bt = block_table + (size_t)s_req[a] * bt_stride + nd.pi0;
          const int last = min(nd.pos, nd.key0 + AT_BN - 1);
          const int n_pi = last / page_size - nd.pi0 + 1;
#pragma unroll
          for (int j = 0; j < 4; ++j) npg[j] = j < n_pi ? bt[j] : 0;
        }
      }
    };
    resolve(0);
    for (int first_tile = 0; first_tile < n_tiles && ok; first_tile += 32) {
      const int buf = (first_tile >> 5) & 1;
      // ---- finish resolving this batch: page ids checked and laid down, Q slots numbered ----
      if (nd.valid) {
        const int last = min(nd.pos, nd.key0 + AT_BN - 1);
        const int n_pi = last / page_size - nd.pi0 + 1;
        const int* bt = block_table + (size_t)s_req[nd.z] * bt_stride + nd.pi0;
        auto lay_down = [&](int j, int pg) {
          // a page wholly before the window may have been given back already: it is not read
          const bool needed = (nd.pi0 + j + 1) * page_size > nd.lo;
          if (needed && (pg < 0 || pg >= num_pages)) {
            qb_set_status(status, QB_STATUS_BAD_PAGE, pg, 6);
            nd.valid = 2;
          }
          s_pages[lane * pages_ld + j] = pg;
        };
        if (few_pages) {
#pragma unroll
          for (int j = 0; j < 4; ++j)
            if (j < n_pi) lay_down(j, npg[j]);
        } else {
          for (int j = 0; j < n_pi; ++j) lay_down(j, bt[j]);
        }
      }
      const uint32_t firsts = __ballot_sync(0xffffffffu, nd.valid && (nd.flags & AD_FIRST));
      nd.qslot = (q_count + __popc(firsts & (0xffffffffu >> (31 - lane))) + q_slots - 1) % q_slots;
      q_count = (q_count + __popc(firsts)) % q_slots;
      my_desc[buf][lane] = nd;
      __syncwarp();
      const int in_batch = min(32, n_tiles - first_tile);
      if (first_tile + 32 < n_tiles) resolve(first_tile + 32);     // its loads are in flight while this batch is issued
      // ---- issue the batch ----
      for (int src = 0; src < in_batch && ok; ++src) {
        const AdDesc d = my_desc[buf][src];
        ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&empty[slot]), phase ^ 1u, abort_flag) ? 1 : 0);   // one answer per warp
        if (!ok) break;
        const uint32_t bar = smem_u32(&full[slot]);
        if (d.valid != 1) {
          if (lane == 0) mbar_arrive(bar);
        } else {
          const int n_keys = min(AT_BN, d.pos - d.key0 + 1);
          __nv_bfloat16* ks = ring + (size_t)slot * 2 * tile_elems;
          __nv_bfloat16* vs = ks + tile_elems;
          // boxes of the TMA path: rows of one page (or 64 rows of a larger page) x 64 dims
          const int n_boxes = (n_keys + box_rows - 1) >> box_shift;       // pages of the tile that hold visible keys
          // keys before the window are not fetched (their rows keep older, finite values and are masked)
          const int key_skip = d.lo > d.key0 ? d.lo - d.key0 : 0;
          const int box_first = TMA ? key_skip >> box_shift : 0;
          const bool new_q = which == 0 && (d.flags & AD_FIRST) != 0;
          if (lane == 0) {
            const uint32_t my_bytes = TMA ? (uint32_t)((n_boxes - box_first) * box_rows) * row_bytes
                                    : (uint32_t)(n_keys - key_skip) * row_bytes;
            mbar_expect_tx(bar, (new_q ? (uint32_t)G * row_bytes : 0u) + my_bytes);
          }
          __syncwarp();
          if (new_q) {
            __nv_bfloat16* qs = qring + (size_t)d.qslot * q_rows * LD;
            for (int r = lane; r < G; r += 32)
              bulk_copy_row(qs + (size_t)r * LD, q + ((size_t)d.tok * nq + d.kvh * G + r) * hd, row_bytes, bar);
          }
          if (TMA) {
            for (int i = lane; i < n_boxes - box_first; i += 32) {
              const int box = box_first + i;
              const int key = d.key0 + (box << box_shift);
              const int pg = s_pages[src * pages_ld + (key >> page_shift) - d.pi0];
              const int row = ((pg * nkv + d.kvh) << page_shift) + (key & (page_size - 1));   // row of the cache [rows][hd]
              __nv_bfloat16* dst = (which ? vs : ks) + ((size_t)box << box_shift) * HDP;
              tma_load_rows(dst, which ? &tm_v : &tm_k, row, slab_major, bar);
            }
          } else {
            for (int r = key_skip + lane; r < n_keys; r += 32) {
              const int key = d.key0 + r;
              const int pg = s_pages[src * pages_ld + key / page_size - d.pi0];
              const size_t off = (((size_t)pg * nkv + d.kvh) * page_size + key % page_size) * hd;
              if (which == 0) bulk_copy_row(ks + (size_t)r * LD, k_cache + off, row_bytes, bar);
              else bulk_copy_row(vs + (size_t)r * LD, v_cache + off, row_bytes, bar);
            }
          }
        }
        if (++slot == stages) { slot = 0; phase ^= 1u; }
      }
      __syncwarp();
    }
    if (!ok) {
      // gave up: let the copies already issued land before the block's shared memory is given away
      const uint64_t t0 = global_ns();
      while (global_ns() - t0 < 2000000ull) __nanosleep(1000);
    }
  } else {
    // ---------------- consumers: all four on the same tile ----------------
    const int g = lane >> 2, qd = lane & 3;
    const int kv_box_rows = min(page_size, AT_BN);
    const KV kv = make_kv((KV*)nullptr, 31 - __clz(kv_box_rows), slab_major);
    const int RB = (G + 15) / 16;                        // row blocks of 16 q heads (1..4)
    const int KS = RB == 1 ? 4 : (RB == 2 ? 2 : 1);      // key slices of a tile
    const int my_rb = RB == 1 ? 0 : (RB == 2 ? (warp & 1) : warp);
    const int my_ks = RB == 1 ? warp : (RB == 2 ? (warp >> 1) : 0);
    const int NK = AT_BN / KS;
    const bool active = my_rb < RB;
    const int n_seg_max = n_parts - 1;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float o[HDP / 8][4];
    // up to 128 dims the Q rows stay in registers as MMA fragments while a pair's tiles go by
    constexpr bool QR = HDP <= 128;
    constexpr int QF = QR ? HDP / 16 : 1;
    uint32_t qf[QF][4];
#pragma unroll
    for (int i = 0; i < HDP / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
#pragma unroll
    for (int i = 0; i < QF; ++i) qf[i][0] = qf[i][1] = qf[i][2] = qf[i][3] = 0u;
    uint32_t cph = 0, phase = 0;
    int slot = 0;
    // a barrier of the four consumer warps, bounded like every other wait
    auto cons_sync = [&]() -> bool {
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&cbar));
      const bool fine = __all_sync(0xffffffffu, mbar_wait(smem_u32(&cbar), cph, abort_flag) ? 1 : 0);
      cph ^= 1u;
      return fine;
    };
    for (int n = 0; n < n_tiles; ++n) {
      const int my_slot = slot;
      if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&full[my_slot]), phase, abort_flag) ? 1 : 0)) break;
      if (++slot == stages) { slot = 0; phase ^= 1u; }
      const AdDesc d = s_desc[(n >> 5) & 1][n & 31];
      if (d.valid != 1) {          // a tile that was passed over
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&empty[my_slot]));
        continue;
      }
      if (d.flags & AD_FIRST) {
        m[0] = m[1] = -INFINITY;
        l[0] = l[1] = 0.f;
#pragma unroll
        for (int i = 0; i < HDP / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
      }
      const __nv_bfloat16* qs = qring + ((size_t)d.qslot * q_rows + (size_t)my_rb * 16) * LD;
      if (QR && (d.flags & AD_FIRST)) {
        // the pair's Q rows came with this tile: keep them as MMA fragments for all of its tiles
#pragma unroll
        for (int kk = 0; kk < QF; ++kk)
          ldmatrix_x4(qf[kk], qs + (size_t)((lane & 7) + 8 * ((lane >> 3) & 1)) * LD + kk * 16 + 8 * (lane >> 4));
      }
      __nv_bfloat16* ks = ring + (size_t)my_slot * 2 * tile_elems;
      const __nv_bfloat16* vs = ks + tile_elems;
      const int kb = d.key0 + my_ks * NK;                // first key of this warp's slice
      if (active && kb <= d.pos && kb + NK - 1 >= d.lo) {
        int row_lo[2], row_hi[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          row_hi[r] = d.pos;      // rows past the group are computed like the others and never written
          row_lo[r] = d.lo;
        }
        if (KS == 4) attend_block<HDP, KV, 16, QR>(qs, ks, vs, kb, row_lo, row_hi, scale_log2, m, l, o, my_ks * 16, qf, kv);
        else if (KS == 2) attend_block<HDP, KV, 32, QR>(qs, ks, vs, kb, row_lo, row_hi, scale_log2, m, l, o, my_ks * 32, qf, kv);
        else attend_block<HDP, KV, 64, QR>(qs, ks, vs, kb, row_lo, row_hi, scale_log2, m, l, o, 0, qf, kv);
      }
      if (!(d.flags & AD_LAST)) {
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&empty[my_slot]));      // this warp has read the tile
        continue;
      }
      // ---- the segment ends here: one partial result (or the final output) per q head ----
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
      }
      const bool fits = d.seg < n_seg_max;
      if (!fits && tid == 0) qb_set_status(status, QB_STATUS_SCRATCH_SMALL, d.seg, 6);
      const int count = (d.flags & AD_WHOLE) ? 0 : min(d.seg + 1, n_seg_max);
      if (KS == 1) {
        if (active) {
#pragma unroll
          for (int r = 0; r < 2; ++r) {
            const int row = my_rb * 16 + g + 8 * r;
            if (row >= G) continue;
            const int head = d.kvh * G + row;
            const size_t row_at = ((size_t)d.z * nq + head) * n_parts;
            if (d.flags & AD_WHOLE) {
              const float inv = l[r] > 0.f ? 1.f / l[r] : 0.f;
              __nv_bfloat16* dst = out + ((size_t)d.tok * nq + head) * hd;
#pragma unroll
              for (int i = 0; i < HDP / 8; ++i) {
                const int dd = i * 8 + qd * 2;
                if (dd < hd) *reinterpret_cast<uint32_t*>(dst + dd) = pack_bf16(o[i][2 * r] * inv, o[i][2 * r + 1] * inv);
              }
            } else if (fits) {
              const size_t at = row_at + d.seg;
              if (qd == 0) { part_ml[at * 2] = m[r]; part_ml[at * 2 + 1] = l[r]; }
#pragma unroll
              for (int i = 0; i < HDP / 8; ++i) {
                const int dd = i * 8 + qd * 2;
                if (dd < hd) *reinterpret_cast<float2*>(part_o + at * hd + dd) = make_float2(o[i][2 * r], o[i][2 * r + 1]);
              }
            }
            if (qd == 0 && (d.flags & AD_PAIR_END)) part_ml[(row_at + n_parts - 1) * 2] = __int_as_float(count);
          }
        }
      } else {
        // the warps hold key slices of the same rows: merge them through the tile's own shared memory
        // With at most 8 q heads a kv head the four warps' rows fit the K half of the tile ([4][8][HDP] floats):
        // what they leave there can only reach scores that the mask replaces, so the tile need not be wiped,
        // and each warp gives the tile back when it has read what it merges.  With more heads the parts
        // fill K and V ([4][16][HDP]) and the tile goes back as zeros (V rows that a later, shorter copy does
        // not cover must stay finite).
        const bool compact = RB == 1 && G <= 8 && hd == HDP;      // no padded dims: every K element of a row is copied over
        const int sc_rows = compact ? 8 : 16;
        if (!cons_sync()) break;                         // every warp has read the tile
        float* sc = reinterpret_cast<float*>(ks);        // [4 warps][sc_rows][HDP], columns XORed by (row & 3) * 8
        if (active) {
#pragma unroll
          for (int r = 0; r < 2; ++r) {
            const int rr = g + 8 * r;
            if (my_rb * 16 + rr >= G) continue;
            if (qd == 0) { s_ml[warp][rr][0] = m[r]; s_ml[warp][rr][1] = l[r]; }
#pragma unroll
            for (int i = 0; i < HDP / 8; ++i) {
              const int col = (i * 8 + qd * 2) ^ ((rr & 3) * 8);
              *reinterpret_cast<float2*>(sc + (size_t)(warp * sc_rows + rr) * HDP + col) = make_float2(o[i][2 * r], o[i][2 * r + 1]);
            }
          }
        }
        if (!cons_sync()) break;
        const int ctid = warp * 32 + lane;
        // A thread a row first: the weights of the row's parts and its (max, sum); then every thread adds the
        // weighted parts of its columns, row after row, with nothing but independent loads in the loop (one
        // warp a scheduler: a chain of dependent shared-memory reads and exponentials per element was 4 us).
        if (ctid < G) {
          const int R = ctid, rb = R >> 4, rr = R & 15;
          float M = -INFINITY, L = 0.f;
          for (int sl = 0; sl < KS; ++sl) M = fmaxf(M, s_ml[RB == 1 ? sl : (rb | (sl << 1))][rr][0]);
          for (int sl = 0; sl < KS; ++sl) {
            const int w = RB == 1 ? sl : (rb | (sl << 1));
            const float ms = s_ml[w][rr][0];
            const float f = ms == -INFINITY ? 0.f : exp2f(ms - M);
            L += f * s_ml[w][rr][1];
            s_fw[w][rr] = f;
          }
          s_row[R][0] = M;
          s_row[R][1] = L;
          s_row[R][2] = L > 0.f ? 1.f / L : 0.f;
        }
        if (!cons_sync()) break;
#pragma unroll 2
        for (int R = 0; R < G; ++R) {
          const int rb = R >> 4, rr = R & 15, head = d.kvh * G + R;
          const float M = s_row[R][0], L = s_row[R][1], inv_l = s_row[R][2];
          const size_t row_at = ((size_t)d.z * nq + head) * n_parts;
          for (int dd = ctid; dd < hd; dd += AD_CONSUMERS * 32) {
            float acc = 0.f;
#pragma unroll
            for (int sl = 0; sl < 4; ++sl) {
              if (sl < KS) {
                const int w = RB == 1 ? sl : (rb | (sl << 1));
                acc += s_fw[w][rr] * sc[(size_t)(w * sc_rows + rr) * HDP + (dd ^ ((rr & 3) * 8))];
              }
            }
            if (d.flags & AD_WHOLE) {
              out[((size_t)d.tok * nq + head) * hd + dd] = __float2bfloat16_rn(acc * inv_l);
            } else if (fits) {
              part_o[(row_at + d.seg) * hd + dd] = acc;
            }
          }
          if (ctid == 0) {
            if (!(d.flags & AD_WHOLE) && fits) { part_ml[(row_at + d.seg) * 2] = M; part_ml[(row_at + d.seg) * 2 + 1] = L; }
            if (d.flags & AD_PAIR_END) part_ml[(row_at + n_parts - 1) * 2] = __int_as_float(count);
          }
        }
        if (!compact) {
          if (!cons_sync()) break;                       // the merged rows have been read
          for (size_t i = ctid; i < 2 * tile_elems / 8; i += AD_CONSUMERS * 32) reinterpret_cast<uint4*>(ks)[i] = make_uint4(0, 0, 0, 0);
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&empty[my_slot]));
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

  // blocks are handed out in the order of blockIdx.x: all kv heads of the first tile, then of the second, so the
  // order of the tile list (the caller puts the tiles with the most keys first) is the order of the work
  const int* tile = tiles + 4 * (blockIdx.x / nkv);
  const int req = tile[0], tok0 = tile[1], n_tok = tile[2], row0 = tile[3];
  const int kvh = blockIdx.x % nkv, G = nq / nkv;
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
  if (tid == 0 && abort_word) qb_set_status(status, QB_STATUS_WAIT_TIMEOUT, blockIdx.x / nkv, 7);
}

// The pairs that the blocks' ranges cut: out[t, head, :] = sum_s 2^(m_s - M) O_s / sum_s 2^(m_s - M) l_s over
// the pair's segments, in index order.  The last entry of a row of part_ml holds the number of segments
// (0: the decode kernel wrote the final output itself).
// When the status words hold a refusal (a page id outside the pool: that tile was passed over, and if it ended
// its pair the pair's segment count was never written) nothing is merged: the host raises at its next read.
__global__ void attn_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                  __nv_bfloat16* __restrict__ out, const int* __restrict__ dec_tok, int nq, int hd,
                                  int n_parts, const int* __restrict__ status) {
  if (status != nullptr && status[0] != 0) return;
  const int z = blockIdx.y, head = blockIdx.x;
  const size_t base = ((size_t)z * nq + head) * n_parts;
  int n = __float_as_int(part_ml[(base + n_parts - 1) * 2]);
  if (n <= 0) return;
  n = min(n, n_parts - 1);
  const int t = dec_tok[z];
  if (n > 64) {
    // very many segments (few kv heads): one after the other
    float M = -INFINITY;
    for (int s = 0; s < n; ++s) M = fmaxf(M, part_ml[(base + s) * 2]);
    for (int d = threadIdx.x; d < hd; d += blockDim.x) {
      float acc = 0.f, L = 0.f;
      for (int s = 0; s < n; ++s) {
        const float ms = part_ml[(base + s) * 2];
        const float f = ms == -INFINITY ? 0.f : exp2f(ms - M);
        acc += f * part_o[(base + s) * hd + d];
        L += f * part_ml[(base + s) * 2 + 1];
      }
      out[((size_t)t * nq + head) * hd + d] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
    }
    return;
  }
  // the segments' (max, sum) once into shared memory, all loads side by side; then their weights
  __shared__ float s_f[64], s_l[64];
  const int lane = threadIdx.x & 31;
  if (threadIdx.x < 32) {
    float ms[2], ls[2], M = -INFINITY;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int s = lane + 32 * i;
      ms[i] = s < n ? part_ml[(base + s) * 2] : -INFINITY;
      ls[i] = s < n ? part_ml[(base + s) * 2 + 1] : 0.f;
      M = fmaxf(M, ms[i]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      s_f[lane + 32 * i] = ms[i] == -INFINITY ? 0.f : exp2f(ms[i] - M);
      s_l[lane + 32 * i] = ls[i];
    }
  }
  __syncthreads();
  for (int d = threadIdx.x; d < hd; d += blockDim.x) {
    float acc = 0.f, L = 0.f;
#pragma unroll 8
    for (int s = 0; s < n; ++s) {         // in segment order
      acc += s_f[s] * part_o[(base + s) * hd + d];
      L += s_f[s] * s_l[s];
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

// The same cache seen as 3-D so that one box is box_rows whole rows (all slabs of 64 dims): slab-major
// [slabs][rows][64] if the driver takes strides that do not grow, else interleaved [rows][slabs][64].
// QUANTA_B200_KV_BOXES=interleaved asks for the second form (for tests).
int make_kv_map_rows(CUtensorMap* map, const void* base, uint64_t rows, uint64_t hd, uint32_t box_rows, int* slab_major) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return QB_ERR_UNSUPPORTED;
  const cuuint32_t estr[3] = {1, 1, 1};
  const char* want = getenv("QUANTA_B200_KV_BOXES");
  const bool try_slab_major = !(want != nullptr && strcmp(want, "interleaved") == 0) && *slab_major != 0;
  if (try_slab_major) {
    const cuuint64_t dims[3] = {64, rows, hd / 64};
    const cuuint64_t strides[2] = {hd * 2, 128};
    const cuuint32_t box[3] = {64, box_rows, (cuuint32_t)(hd / 64)};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r == CUDA_SUCCESS) { *slab_major = 1; return 0; }
  }
  *slab_major = 0;
  const cuuint64_t dims[3] = {64, hd / 64, rows};
  const cuuint64_t strides[2] = {128, hd * 2};
  const cuuint32_t box[3] = {64, (cuuint32_t)(hd / 64), box_rows};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : QB_ERR_UNSUPPORTED;
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

// Query rows (token x head of the group) per tile of the span kernels, for the shapes of a layer
// (nq <= 0: of the mma.sync kernel alone).
extern "C" int qb_attn_span_tc_supported(int nq, int nkv, int hd, int page_size);
extern "C" int qb_attn_span_tc_rows(void);
static bool span_uses_tc(int nq, int nkv, int hd, int page_size) {
  const char* want = getenv("QUANTA_B200_SPAN_KERNEL");
  const bool force_mma = want != nullptr && strcmp(want, "mma") == 0;
  return !force_mma && nq > 0 && qb_attn_span_tc_supported(nq, nkv, hd, page_size);
}
extern "C" int qb_attn_span_rows(int hd, int nq, int nkv, int page_size) {
  if (span_uses_tc(nq, nkv, hd, page_size)) return qb_attn_span_tc_rows();
  return hd <= 128 ? 128 : 64;
}

// the tcgen05 kernels for the shapes they take (attention_tc.cu)
extern "C" int qb_attn_span_tc(const void* q, const void* k_cache, const void* v_cache, void* out, const int* tok_pos,
                               const int* block_table, int bt_stride, const int* tiles, int n_tiles, int nq, int nkv,
                               int hd, int page_size, int num_pages, float scale, int window, int* status,
                               cudaStream_t stream);

// QUANTA_B200_SPAN_KERNEL=mma keeps the mma.sync kernel for every shape (for tests and measurements).
extern "C" int qb_attn_span(const void* q, const void* k_cache, const void* v_cache, void* out, const int* tok_pos,
                            const int* block_table, int bt_stride, const int* tiles, int n_tiles, int nq, int nkv,
                            int hd, int page_size, int num_pages, float scale, int window, int* status,
                            cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  if (hd % 16 || hd > 256 || hd <= 0 || nq % nkv || nkv > 65535) return QB_ERR_UNSUPPORTED;
  if (span_uses_tc(nq, nkv, hd, page_size))
    return qb_attn_span_tc(q, k_cache, v_cache, out, tok_pos, block_table, bt_stride, tiles, n_tiles, nq, nkv, hd,
                           page_size, num_pages, scale, window, status, stream);
  const float scale_log2 = scale * 1.4426950408889634f;
  dim3 grid((unsigned)n_tiles * (unsigned)nkv);
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

// Entries per (token, q head) row of the decode scratch for contexts of up to max_len keys: the most
// segments a pair can be cut into by the blocks' equal ranges, and one entry for their count.
extern "C" int qb_attn_decode_parts(int nkv, int max_len) {
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
    return QB_ERR_UNSUPPORTED;
  if (nkv <= 0 || max_len <= 0) return QB_ERR_BAD_ARG;
  const int tiles = (max_len + AT_BN - 1) / AT_BN;
  const int cut = 2 * sms / nkv + 2;
  return (tiles < cut ? tiles : cut) + 1;
}

// Scratch, in floats: part_o n_dec*nq*n_parts*hd, part_ml n_dec*nq*n_parts*2, with
// n_parts >= qb_attn_decode_parts(nkv, longest context).  Up to 64 q heads per kv head.
extern "C" int qb_attn_decode(const void* q, const void* k_cache, const void* v_cache, void* out, float* part_o,
                              float* part_ml, const int* dec_tok, int n_dec, const int* tok_pos, const int* tok_req,
                              const int* block_table, int bt_stride, int nq, int nkv, int hd, int page_size,
                              int num_pages, float scale, int window, int n_parts, int* status,
                              cudaStream_t stream) {
  if (n_dec <= 0) return 0;
  if (hd % 16 || hd > 256 || hd <= 0 || nq % nkv || nkv > 65535 || n_dec > 65535 || n_parts < 2 || page_size <= 0)
    return QB_ERR_UNSUPPORTED;
  const float scale_log2 = scale * 1.4426950408889634f;
  const int G = nq / nkv, q_rows = ad_q_rows(G);
  if (G > 16 * AD_CONSUMERS) return QB_ERR_UNSUPPORTED;
  int dev = 0, sms = 0, smem_optin = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err == cudaSuccess) err = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (err == cudaSuccess) err = cudaDeviceGetAttribute(&smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
  if (err != cudaSuccess) return (int)err;
  // TMA tensor loads when the shapes allow (whole 64-dim slabs, pages that tile 64 keys), else row copies
  const bool pow2 = (page_size & (page_size - 1)) == 0;
  const bool tma = (hd == 64 || hd == 128 || hd == 256) && pow2 && (page_size <= AT_BN || page_size % AT_BN == 0) && encode_fn() != nullptr &&
                   (((uintptr_t)k_cache | (uintptr_t)v_cache) & 15) == 0;
  CUtensorMap tm_k, tm_v;
  int slab_major = 1;
  memset(&tm_k, 0, sizeof(tm_k));
  memset(&tm_v, 0, sizeof(tm_v));
  if (tma) {
    const uint64_t rows = (uint64_t)num_pages * nkv * page_size;
    const uint32_t box_rows = (uint32_t)(page_size < AT_BN ? page_size : AT_BN);
    int rc = make_kv_map_rows(&tm_k, k_cache, rows, (uint64_t)hd, box_rows, &slab_major);
    if (rc == 0) rc = make_kv_map_rows(&tm_v, v_cache, rows, (uint64_t)hd, box_rows, &slab_major);
    if (rc) return rc;
  }
  const int pages_ld = AT_BN / (page_size < AT_BN ? page_size : AT_BN) + 2;     // page ids a tile can touch
#define QB_DEC(HDP, TMA_)                                                                                  \
  do {                                                                                                     \
    cudaFuncAttributes fa;                                                                                 \
    err = cudaFuncGetAttributes(&fa, attn_decode_kernel<HDP, TMA_>);                                       \
    if (err != cudaSuccess) return (int)err;                                                               \
    const size_t q_bytes = (size_t)q_rows * (HDP + AT_PAD) * 2;  /* one more Q slot than tiles, 8 zero rows */ \
    const size_t stage_bytes = 2 * ad_tile_elems(HDP, TMA_) * 2 + q_bytes;                                 \
    const size_t fixed = 1024 + q_bytes + 8 * (HDP + AT_PAD) * 2 +                                         \
                         (size_t)(4 * AD_MAX_DEC + 1 + AD_PRODUCERS * 32 * pages_ld) * sizeof(int);        \
    const long room = (long)smem_optin - (long)fa.sharedSizeBytes - (long)fixed;                           \
    int stages = room > 0 ? (int)((size_t)room / stage_bytes) : 0;                                         \
    if (stages > AD_MAX_STAGES) stages = AD_MAX_STAGES;                                                    \
    if (stages < 2) return QB_ERR_UNSUPPORTED;                                                             \
    const size_t smem = stage_bytes * stages + fixed;        /* 1024 of it to align the ring */            \
    int rc = set_smem(attn_decode_kernel<HDP, TMA_>, smem);                                                \
    if (rc) return rc;                                                                                     \
    for (int z0 = 0; z0 < n_dec; z0 += AD_MAX_DEC) {                                                       \
      const int n = n_dec - z0 < AD_MAX_DEC ? n_dec - z0 : AD_MAX_DEC;                                     \
      attn_decode_kernel<HDP, TMA_><<<sms, AD_THREADS, smem, stream>>>(                                    \
          tm_k, tm_v, (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, \
          (__nv_bfloat16*)out, part_o + (size_t)z0 * nq * n_parts * hd, part_ml + (size_t)z0 * nq * n_parts * 2, \
          dec_tok + z0, n, tok_pos, tok_req, block_table, bt_stride, nq, nkv, hd, page_size, num_pages,    \
          scale_log2, window, n_parts, stages, pages_ld, slab_major, status);                              \
    }                                                                                                      \
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
  attn_merge_kernel<<<dim3(nq, n_dec), 128, 0, stream>>>(part_o, part_ml, (__nv_bfloat16*)out, dec_tok, nq, hd, n_parts, status);
  QB_LAUNCH_CHECK();
  return 0;
}

// ------------------------------------------------------------------------------------------------
// The same decode attention for callers that cannot allocate: the scratch is a static device array.
// (No counterpart in the reference; contract and reasons in no_alloc.h.)
// ------------------------------------------------------------------------------------------------
#include "no_alloc.h"

// Partial results of the decode kernel for one call at a time.  Host code must not hand this
// name to a kernel: on the host it is only a stand-in for the symbol; the device address is looked
// up once per device below.
static __device__ __align__(256) float qb_noalloc_scratch[QB_NOALLOC_SCRATCH_FLOATS];

namespace {
constexpr int NOALLOC_MAX_DEVICES = 64;
float* g_noalloc_ptr[NOALLOC_MAX_DEVICES] = {};
}  // namespace

extern "C" long long qb_attn_decode_noalloc_floats(int n_dec, int nq, int hd, int n_parts) {
  if (n_dec <= 0 || nq <= 0 || hd <= 0 || n_parts <= 0) return 0;
  return (long long)n_dec * nq * n_parts * (hd + 2);
}

extern "C" long long qb_attn_decode_noalloc_capacity(void) { return (long long)QB_NOALLOC_SCRATCH_FLOATS; }

extern "C" int qb_attn_decode_noalloc(const void* q, const void* k_cache, const void* v_cache, void* out,
                                      const int* dec_tok, int n_dec, const int* tok_pos, const int* tok_req,
                                      const int* block_table, int bt_stride, int nq, int nkv, int hd, int page_size,
                                      int num_pages, float scale, int window, int n_parts, int* status,
                                      cudaStream_t stream) {
  if (n_dec <= 0) return 0;
  if (nq <= 0 || hd <= 0 || n_parts <= 0) return QB_ERR_BAD_ARG;
  const long long need = qb_attn_decode_noalloc_floats(n_dec, nq, hd, n_parts);
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
  float* part_ml = part_o + (size_t)n_dec * nq * n_parts * hd;
  return qb_attn_decode(q, k_cache, v_cache, out, part_o, part_ml, dec_tok, n_dec, tok_pos, tok_req, block_table,
                        bt_stride, nq, nkv, hd, page_size, num_pages, scale, window, n_parts, status, stream);
}
