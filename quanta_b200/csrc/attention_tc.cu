// Paged causal attention for prompt portions on the 5th-generation tensor cores (head size 128).
//
// A block takes query rows of ONE request and ONE kv head, where a row is a (token, q head of the group)
// pair, against the request's keys in blocks of 128: S = Q K^T and O += P V are tcgen05.mma (M = 128 rows,
// N = 128, eight steps of K = 16 each; Q, K and P are K-major operands in shared memory with the 128-byte
// swizzle, V is the MN-major operand exactly as it lies in the cache), S and O live in TMEM, and softmax
// warps turn S into P between the two products (tcgen05.ld, float32 online softmax in the exp2 domain,
// P as bfloat16 into the swizzled tile).  K and V come by TMA tensor loads, one box per page and 64-dim
// slab.  One query tile a block, O accumulated in TMEM; the kernel is described where it stands.
//
// (src/quanta/minimax/attention.py:194-203: scores * head_dim^-0.5, causal mask, softmax in float32,
// probabilities cast to the activation dtype, P V; q head h reads kv head h / (n_q / n_kv).)
// Each row is masked by its own token's position (and window), so portions of any length run, from the
// cache that earlier steps and this step's rope kernel wrote.  No multicast, no clusters.  Every wait is
// bounded; when one runs out the block records it in the status words, frees its TMEM and returns.
#include <cuda.h>

#include <cstdlib>
#include <cstring>

#include "common.cuh"

namespace {

constexpr int TC_BM = 128;           // query rows per block (UMMA M)
constexpr int TC_BN = 128;           // keys per block
constexpr int TC_HD = 128;           // head size
constexpr int TC_MAX_PAGES = 2048;
constexpr uint32_t TC_TILE_BYTES = TC_BM * TC_HD * 2;       // 32 KB: Q, P, and each K or V stage
constexpr uint32_t TC_SLAB_BYTES = TC_BM * 128;             // one slab: 128 rows x 64 elements
constexpr uint32_t TC_SPIN_LIMIT = 4u * 1000u * 1000u;
constexpr uint64_t TC_WAIT_NS = 200ull * 1000ull * 1000ull;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// The thread sleeps in the instruction until the phase completes or about a microsecond has passed, so
// that a waiting warp leaves the issue slots of its scheduler to the warps that work.
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity), "r"(1000u) : "memory");
  return ok != 0;
}
__device__ __forceinline__ uint64_t global_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait: false when another role gave up or the limit (iterations and 0.2 s) is reached.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  uint64_t t0 = 0;
  for (uint32_t it = 0; it < TC_SPIN_LIMIT; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 127u) == 127u) {
      if (*abort_flag) return false;
      const uint64_t now = global_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > TC_WAIT_NS) break;
    }
  }
  *abort_flag = 1;
  return false;
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;      // 0 source bytes: the 16 destination bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(n));
}
// one [box rows x 64 dims] box of a cache seen as a 2-D tensor [rows, head_dim]; no multicast
__device__ __forceinline__ void tma_load_box(uint32_t dst, const CUtensorMap* map, int dim0, int row, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(dim0), "r"(row), "r"(bar) : "memory");
}

// Operand tile in shared memory in lines of 128 bytes with the 128-byte swizzle, 8-line groups 1024 bytes
// apart.  K-major (Q, K, P: a line is 64 k elements of one row): stride offset 1024, leading offset unused.
// MN-major (V as the N operand: a line is 64 dims of one key): stride offset 1024 between groups of 8
// keys, leading offset one slab between groups of 64 dims.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr, uint32_t leading_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((leading_bytes >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;                                // descriptor version (sm_100)
  d |= (uint64_t)2 << 61;                                // 128-byte swizzle
  return d;
}
// kind::f16, bfloat16 x bfloat16 -> float32; b_mn: the B operand is MN-major
__device__ __forceinline__ uint32_t umma_idesc(int m, int n, bool b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn ? (1u << 16) : 0u) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc) : "memory");
}
// the same with the A operand in TMEM (a row a lane, two bfloat16 a column, K along the columns)
__device__ __forceinline__ void umma_bf16_ta(uint32_t tmem_d, uint32_t tmem_a, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(b_desc), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// 2^x on the special-function unit; x is at most 0 here, tiny results flush to zero
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// ------------------------------------------------------------------------------------------------
// One query tile per block, O accumulated in TMEM, two softmax threads per row.
//
//   warps 0-1: TMA producers of K blocks, warps 2-3: of V blocks (two stages each; a warp takes one 64-dim slab of
//   every page, since an instruction that starts a copy holds its warp for some hundred cycles and a block of
//   128 keys in pages of 16 is sixteen boxes), warp 4: MMA issuer,
//   warps 5-12: softmax; warps 5-8 take keys 0..63 of a block, warps 9-12 keys 64..127, of the row that is
//   their TMEM lane.  TMEM: two S buffers, ONE O of 128 columns that every P V adds to, and two P buffers
//   of 64 columns (bfloat16 pairs): the probabilities never pass through shared memory, P V takes them as
//   its TMEM operand, and the softmax of the next block runs while P V of this one does.
//   The exponentials use a reference maximum that is only raised when the row maximum has grown by more
//   than 2^8 since (then the row's O and sum are rescaled, each thread its 64 columns, after the P V
//   before has finished); otherwise P V (j) needs nothing from the threads but P(j), and the threads
//   never read O until the end.  Both threads of a row take the maximum over all 128 keys (the same
//   decision without talking to each other) and the exponentials of their own 64.
// ------------------------------------------------------------------------------------------------
constexpr int TCS_THREADS = 13 * 32;
constexpr float TCS_TAU = 8.0f;

struct TcsShared {
  uint64_t k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2], o_full, p_full[2], p_empty[2], fin;
  uint64_t mx_full[4];      // the two warps of a lane quadrant have both written their maxima of a block
  uint32_t tmem_base;
  int abort_flag;
};

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}

__global__ void __launch_bounds__(TCS_THREADS, 1)
attn_span_tc_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                     const __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ out,
                     const int* __restrict__ tok_pos, const int* __restrict__ block_table, int bt_stride,
                     const int* __restrict__ tiles, int nq, int nkv, int page_size, int num_pages,
                     float scale_log2, int window, int* status) {
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* base = reinterpret_cast<unsigned char*>(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
  const uint32_t q_s = smem_u32(base), k_s = q_s + TC_TILE_BYTES, v_s = k_s + 2 * TC_TILE_BYTES;
  __shared__ TcsShared sh;
  __shared__ int s_page[TC_MAX_PAGES];
  __shared__ float s_l[2][TC_BM];
  __shared__ float s_mx[2][2][TC_BM];      // [block parity][half][row]
  volatile int* abort_flag = &sh.abort_flag;

  // blocks are handed out in the order of blockIdx.x: all kv heads of the first tile, then of the second, so the
  // order of the tile list (the caller puts the tiles with the most keys first) is the order of the work
  const int* tile = tiles + 4 * (blockIdx.x / nkv);
  const int req = tile[0], tok0 = tile[1], n_tok = tile[2], row0 = tile[3];
  const int kvh = blockIdx.x % nkv, G = nq / nkv;
  const int n_rows = min(TC_BM, n_tok * G - row0);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int* bt = block_table + (size_t)req * bt_stride;

  const int first_tok = tok0 + row0 / G, last_tok = tok0 + (row0 + n_rows - 1) / G;
  const int key_end = tok_pos[last_tok];
  const int p_first = tok_pos[first_tok];
  const int lo_min = (window > 0 && p_first - window + 1 > 0) ? p_first - window + 1 : 0;   // the lowest key any row reads
  const int key_begin = lo_min / TC_BN * TC_BN;
  const int n_blocks = (key_end - key_begin) / TC_BN + 1;

  for (int c = tid; c < TC_BM * (TC_HD / 8); c += TCS_THREADS) {
    const int r = c / (TC_HD / 8), ch = c % (TC_HD / 8);      // 16-byte chunk ch of row r
    const int R = row0 + r;
    const bool ok = r < n_rows;
    const __nv_bfloat16* src = q;
    if (ok) src = q + ((size_t)(tok0 + R / G) * nq + kvh * G + R % G) * TC_HD + ch * 8;
    cp_async16(q_s + (ch >> 3) * TC_SLAB_BYTES + r * 128 + (((ch & 7) ^ (r & 7)) << 4), src, ok);
  }
  asm volatile("cp.async.commit_group;\n" ::);
  for (uint32_t i = tid; i < 4 * TC_TILE_BYTES / 16; i += TCS_THREADS)
    reinterpret_cast<uint4*>(base + TC_TILE_BYTES)[i] = make_uint4(0, 0, 0, 0);
  const int pi0 = key_begin / page_size;
  const int n_pi = key_end / page_size - pi0 + 1;
  const bool pages_in_smem = n_pi <= TC_MAX_PAGES;
  if (pages_in_smem)
    for (int i = tid; i < n_pi; i += TCS_THREADS) s_page[i] = bt[pi0 + i];
  if (tid == 0) {
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&sh.k_full[s]), 2);      // the two producer warps
      mbar_init(smem_u32(&sh.k_empty[s]), 1);
      mbar_init(smem_u32(&sh.v_full[s]), 2);
      mbar_init(smem_u32(&sh.v_empty[s]), 1);
      mbar_init(smem_u32(&sh.s_full[s]), 1);
    }
    mbar_init(smem_u32(&sh.o_full), 1);
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&sh.p_full[b]), 256);
      mbar_init(smem_u32(&sh.p_empty[b]), 1);
    }
    mbar_init(smem_u32(&sh.fin), 256);
    for (int q4 = 0; q4 < 4; ++q4) mbar_init(smem_u32(&sh.mx_full[q4]), 64);
    sh.abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 4) {      // two S buffers and O: 384 columns, allocated as 512
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(&sh.tmem_base)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("cp.async.wait_group 0;\n" ::);
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // Q and the zeros, before TMA and the MMAs
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = sh.tmem_base;
  const uint32_t o_col = 2 * TC_BN;                 // S(0), S(1), O, then
  const uint32_t p_col = 2 * TC_BN + TC_HD;         // P(0), P(1): 64 columns each

  if (warp < 4) {
    // ---------------- TMA producers: warps 0-1 stream K blocks, warps 2-3 V blocks, each one slab ----------------
    const bool is_k = warp < 2;
    const int slab = warp & 1;
    const CUtensorMap* map = is_k ? &tm_k : &tm_v;
    uint64_t* full = is_k ? sh.k_full : sh.v_full;
    uint64_t* empty = is_k ? sh.k_empty : sh.v_empty;
    const uint32_t ring = is_k ? k_s : v_s;
    const int box_rows = min(page_size, TC_BN);
    bool ok = true;
    for (int b = 0; b < n_blocks && ok; ++b) {
      const int slot = b & 1;
      const uint32_t ph = (uint32_t)(b >> 1) & 1u;
      ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&empty[slot]), ph ^ 1u, abort_flag) ? 1 : 0);
      if (!ok) break;
      const int key0 = key_begin + b * TC_BN;
      const int n_keys = min(TC_BN, key_end - key0 + 1);
      const int n_req = (n_keys + box_rows - 1) / box_rows;      // boxes of this warp: the pages with visible keys
      const uint32_t bar = smem_u32(&full[slot]);
      int skipped = 0;
      for (int i = lane; i < n_req; i += 32) {
        const int key = key0 + i * box_rows;
        if (key + box_rows - 1 < lo_min) { ++skipped; continue; }
        const int pg = pages_in_smem ? s_page[key / page_size - pi0] : bt[key / page_size];
        if (pg < 0 || pg >= num_pages) { qb_set_status(status, QB_STATUS_BAD_PAGE, pg, 7); ++skipped; }
      }
      skipped = __reduce_add_sync(0xffffffffu, skipped);
      if (lane == 0) mbar_expect_tx(bar, (uint32_t)(n_req - skipped) * (uint32_t)box_rows * 128u);
      __syncwarp();
      for (int box = lane; box < n_req; box += 32) {
        const int key = key0 + box * box_rows;
        if (key + box_rows - 1 < lo_min) continue;
        const int pg = pages_in_smem ? s_page[key / page_size - pi0] : bt[key / page_size];
        if (pg < 0 || pg >= num_pages) continue;
        const int row = (pg * nkv + kvh) * page_size + key % page_size;
        tma_load_box(ring + slot * TC_TILE_BYTES + slab * TC_SLAB_BYTES + box * box_rows * 128, map, slab * 64, row, bar);
      }
    }
    if (!ok) {
      const uint64_t t0 = global_ns();
      while (global_ns() - t0 < 2000000ull) __nanosleep(1000);
    }
  } else if (warp == 4) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      const uint32_t idesc_qk = umma_idesc(TC_BM, TC_BN, false), idesc_pv = umma_idesc(TC_BM, TC_HD, true);
      bool ok = true;
      auto issue_qk = [&](int i) {
        const int slot = i & 1;
        ok = mbar_wait(smem_u32(&sh.k_full[slot]), (uint32_t)(i >> 1) & 1u, abort_flag);
        if (!ok) return;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t kt = k_s + slot * TC_TILE_BYTES;
#pragma unroll
        for (int k16 = 0; k16 < TC_HD / 16; ++k16) {
          const uint32_t off = (k16 >> 2) * TC_SLAB_BYTES + (k16 & 3) * 32;
          umma_bf16(tmem_base + (uint32_t)(slot * TC_BN), umma_desc(q_s + off, 0), umma_desc(kt + off, 0), idesc_qk,
                    k16 != 0 ? 1u : 0u);
        }
        umma_commit(smem_u32(&sh.k_empty[slot]));
        umma_commit(smem_u32(&sh.s_full[slot]));
      };
      issue_qk(0);
      if (ok && n_blocks > 1) issue_qk(1);
      for (int j = 0; j < n_blocks && ok; ++j) {
        const int slot = j & 1;
        ok = mbar_wait(smem_u32(&sh.p_full[slot]), (uint32_t)(j >> 1) & 1u, abort_flag);      // P(j) written, S(j) read, O rescaled if need be
        if (!ok) break;
        ok = mbar_wait(smem_u32(&sh.v_full[slot]), (uint32_t)(j >> 1) & 1u, abort_flag);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t vt = v_s + slot * TC_TILE_BYTES;
        const uint32_t pt = tmem_base + p_col + (uint32_t)(slot * (TC_BN / 2));
#pragma unroll
        for (int k16 = 0; k16 < TC_BN / 16; ++k16) {
          // 16 keys further: 8 columns of P, 16 rows of V
          umma_bf16_ta(tmem_base + o_col, pt + (uint32_t)(k16 * 8), umma_desc(vt + k16 * 2048, TC_SLAB_BYTES), idesc_pv,
                       (j | k16) != 0 ? 1u : 0u);
        }
        umma_commit(smem_u32(&sh.v_empty[slot]));
        umma_commit(smem_u32(&sh.p_empty[slot]));
        umma_commit(smem_u32(&sh.o_full));
        if (j + 2 < n_blocks) issue_qk(j + 2);
      }
    }
  } else {
    // ---------------- softmax: two threads a row, 64 keys of a block each ----------------
    const int quad = warp & 3, half = (warp - 5) >> 2;
    const int r = quad * 32 + lane;
    const int R = row0 + r;
    const bool valid = r < n_rows;
    const int pos_r = valid ? tok_pos[tok0 + R / G] : -1;
    const int lo_r = (window > 0 && pos_r - window + 1 > 0) ? pos_r - window + 1 : 0;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16);
    const uint32_t o_addr = lane_addr + o_col + (uint32_t)(half * 64);       // this thread's 64 columns of O
    const uint32_t p_addr = lane_addr + p_col + (uint32_t)(half * 32);       // its 64 keys: 32 columns of a P buffer
    float m_true = -INFINITY, m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_blocks; ++j) {
      const int slot = j & 1;
      ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&sh.s_full[slot]), (uint32_t)(j >> 1) & 1u, abort_flag) ? 1 : 0);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int key0 = key_begin + j * TC_BN;
      const bool all_visible = key0 >= lo_r && key0 + TC_BN - 1 <= pos_r;
      const uint32_t s_addr = lane_addr + (uint32_t)(slot * TC_BN);
      // this thread's 64 keys of the block, read once and kept; the row's maximum over all 128 keys is the larger
      // of this thread's and its partner's (the same lane of the warp four further on), handed over through
      // shared memory and a barrier of the two warps
      const int kbase = key0 + half * 64;
      uint32_t va[32], vb[32];
      {
        const uint32_t mine = s_addr + (uint32_t)(half * 64);
        tmem_ld32(mine, va);
        tmem_ld32(mine + 32u, vb);
        tmem_wait_ld();
      }
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      if (all_visible) {
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          mx4[(i >> 1) & 3] = max3(mx4[(i >> 1) & 3], __uint_as_float(va[i]), __uint_as_float(va[i + 1]));
          mx4[(i >> 1) & 3] = max3(mx4[(i >> 1) & 3], __uint_as_float(vb[i]), __uint_as_float(vb[i + 1]));
        }
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int ka = kbase + i, kb = kbase + 32 + i;
          if (ka >= lo_r && ka <= pos_r) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(va[i]));
          if (kb >= lo_r && kb <= pos_r) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(vb[i]));
        }
      }
      const float mx_own = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      s_mx[j & 1][half][r] = mx_own;
      mbar_arrive(smem_u32(&sh.mx_full[quad]));
      ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&sh.mx_full[quad]), (uint32_t)j & 1u, abort_flag) ? 1 : 0);
      if (!ok) break;
      const float mx = fmaxf(mx_own, s_mx[j & 1][half ^ 1][r]) * scale_log2;
      m_true = fmaxf(m_true, mx);
      // raise the reference only when the maximum has grown a lot: O and the sum are rescaled then
      const bool raise = m_true > m_ref + TCS_TAU;          // also true while the reference is -inf and a key is visible
      if (__any_sync(0xffffffffu, raise && j > 0)) {
        ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&sh.o_full), (uint32_t)(j - 1) & 1u, abort_flag) ? 1 : 0);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        // tcgen05.ld / st / wait are .sync.aligned: the WHOLE warp runs them, whichever of its rows raise
        // (a row that does not multiplies by exactly 1); run by some lanes only they can hang the warp
        const float f = raise ? ex2(m_ref - m_true) : 1.f;  // reference -inf: 0
        l *= f;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t v[16];
          tmem_ld16(o_addr + (uint32_t)(c * 16), v);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 16; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * f);
          tmem_st16(o_addr + (uint32_t)(c * 16), v);
        }
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      }
      if (raise) m_ref = m_true;
      const float msafe = m_ref == -INFINITY ? 0.f : m_ref;
      // the P buffer of this block is free once the P V of the block before the last has read it
      if (j > 1) {
        ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&sh.p_empty[slot]), (uint32_t)((j >> 1) - 1) & 1u, abort_flag) ? 1 : 0);
        if (!ok) break;
      }
      // the probabilities of this thread's 64 keys, as bfloat16 pairs into its columns of P
      float sum2[2] = {0.f, 0.f};
      {
        const bool vis = all_visible;
        auto take = [&](const uint32_t (&v)[32], int c) {        // keys kbase + c*32 .. +31
          uint32_t pk[16];
          if (vis) {
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              const float p0 = ex2(__uint_as_float(v[i]) * scale_log2 - msafe);
              const float p1 = ex2(__uint_as_float(v[i + 1]) * scale_log2 - msafe);
              sum2[0] += p0;
              sum2[1] += p1;
              pk[i >> 1] = pack_bf16(p0, p1);
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              const int key = kbase + c * 32 + i;
              float p0 = ex2(__uint_as_float(v[i]) * scale_log2 - msafe);
              float p1 = ex2(__uint_as_float(v[i + 1]) * scale_log2 - msafe);
              if (key < lo_r || key > pos_r) p0 = 0.f;
              if (key + 1 < lo_r || key + 1 > pos_r) p1 = 0.f;
              sum2[0] += p0;
              sum2[1] += p1;
              pk[i >> 1] = pack_bf16(p0, p1);
            }
          }
          tmem_st16(p_addr + (uint32_t)(slot * (TC_BN / 2) + c * 16), pk);
        };
        take(va, 0);
        take(vb, 1);
      }
      l += sum2[0] + sum2[1];
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");      // P, before the MMA reads it
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      mbar_arrive(smem_u32(&sh.p_full[slot]));
    }
    if (ok) {
      // the end: both halves' sums, then each thread its 64 columns of O
      s_l[half][r] = l;
      mbar_arrive(smem_u32(&sh.fin));
      ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&sh.fin), 0u, abort_flag) ? 1 : 0);
      if (ok) ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&sh.o_full), (uint32_t)(n_blocks - 1) & 1u, abort_flag) ? 1 : 0);
      if (ok) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const float lt = s_l[0][r] + s_l[1][r];
        const float inv = lt > 0.f ? 1.f / lt : 0.f;
        __nv_bfloat16* dst = out + ((size_t)(tok0 + R / G) * nq + kvh * G + R % G) * TC_HD + half * 64;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t v[16];
          tmem_ld16(o_addr + (uint32_t)(c * 16), v);
          tmem_wait_ld();
          if (valid) {
#pragma unroll
            for (int i = 0; i < 16; i += 8) {
              uint4 w;
              w.x = pack_bf16(__uint_as_float(v[i]) * inv, __uint_as_float(v[i + 1]) * inv);
              w.y = pack_bf16(__uint_as_float(v[i + 2]) * inv, __uint_as_float(v[i + 3]) * inv);
              w.z = pack_bf16(__uint_as_float(v[i + 4]) * inv, __uint_as_float(v[i + 5]) * inv);
              w.w = pack_bf16(__uint_as_float(v[i + 6]) * inv, __uint_as_float(v[i + 7]) * inv);
              *reinterpret_cast<uint4*>(dst + c * 16 + i) = w;
            }
          }
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 4) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
  if (tid == 0 && sh.abort_flag) qb_set_status(status, QB_STATUS_WAIT_TIMEOUT, blockIdx.x / nkv, 7);
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

// A cache [rows, 128] bfloat16 row-major, boxes of [box_rows, 64 dims], 128-byte swizzle
int make_kv_map(CUtensorMap* map, const void* base, uint64_t rows, uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return QB_ERR_UNSUPPORTED;
  const cuuint64_t dims[2] = {TC_HD, rows};
  const cuuint64_t strides[1] = {TC_HD * 2};
  const cuuint32_t box[2] = {64, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : QB_ERR_UNSUPPORTED;
}

}  // namespace

// 1 if the tcgen05 kernel takes these shapes (head size 128, power-of-two pages that tile 128 keys).
extern "C" int qb_attn_span_tc_supported(int nq, int nkv, int hd, int page_size) {
  if (hd != TC_HD || nkv <= 0 || nq % nkv || nkv > 65535 || page_size <= 0) return 0;
  if ((page_size & (page_size - 1)) != 0) return 0;
  if (!(page_size <= TC_BN || page_size % TC_BN == 0)) return 0;
  return encode_fn() != nullptr ? 1 : 0;
}

// Query rows per tile of the tcgen05 kernel.
extern "C" int qb_attn_span_tc_rows(void) { return TC_BM; }

// Same arguments as qb_attn_span; the tile list has qb_attn_span_tc_rows() rows a tile.
extern "C" int qb_attn_span_tc(const void* q, const void* k_cache, const void* v_cache, void* out, const int* tok_pos,
                               const int* block_table, int bt_stride, const int* tiles, int n_tiles, int nq, int nkv,
                               int hd, int page_size, int num_pages, float scale, int window, int* status,
                               cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  if (!qb_attn_span_tc_supported(nq, nkv, hd, page_size)) return QB_ERR_UNSUPPORTED;
  if ((((uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)q | (uintptr_t)out) & 15) != 0) return QB_ERR_UNSUPPORTED;
  const float scale_log2 = scale * 1.4426950408889634f;
  CUtensorMap tm_k, tm_v;
  memset(&tm_k, 0, sizeof(tm_k));
  memset(&tm_v, 0, sizeof(tm_v));
  const uint64_t rows = (uint64_t)num_pages * nkv * page_size;
  const uint32_t box_rows = (uint32_t)(page_size < TC_BN ? page_size : TC_BN);
  int rc = make_kv_map(&tm_k, k_cache, rows, box_rows);
  if (rc == 0) rc = make_kv_map(&tm_v, v_cache, rows, box_rows);
  if (rc) return rc;
  const size_t smem = 5 * (size_t)TC_TILE_BYTES + 1024;      // Q and two stages each of K and V
  cudaError_t err = cudaFuncSetAttribute(attn_span_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (err != cudaSuccess) return (int)err;
  attn_span_tc_kernel<<<dim3((unsigned)n_tiles * (unsigned)nkv), TCS_THREADS, smem, stream>>>(
      tm_k, tm_v, (const __nv_bfloat16*)q, (__nv_bfloat16*)out, tok_pos, block_table, bt_stride, tiles, nq, nkv,
      page_size, num_pages, scale_log2, window, status);
  QB_LAUNCH_CHECK();
  return 0;
}
