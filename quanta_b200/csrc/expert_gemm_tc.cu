// Routed experts on the 5th-generation tensor cores: TMA-fed tcgen05.mma with accumulators in TMEM.
//
// One block = one tile of up to NT token rows of ONE expert x 128 of its output features.  The
// expert's WEIGHTS are the 128-row operand (M = 128) and the token rows are the N operand ("swap
// A/B"), so an expert with few rows still uses the full height of the MMA and its weights stream
// through shared memory exactly once per token tile:
//
//   warp 0   : TMA producer.  Per 64-wide k block: weight tile(s) [128 x 64] and token tile [NT x 64],
//              bfloat16, 128-byte swizzle, into a ring of shared-memory stages (mbarrier expect_tx); lane 0
//              fetches the boxes, all lanes share the rows where the token rows are fetched one by one.
//   warp 1   : MMA issuer.  4 x tcgen05.mma (K = 16 each) per stage and matrix, D[128 x NT] float32 in
//              TMEM; tcgen05.commit frees the stage and, at the end, signals the epilogue.
//   warps 2-5: epilogue (2-9 in the blocks of a pair).  tcgen05.ld (one TMEM lane = one output feature per thread), then
//              MODE 1: act[p, j] = silu(gate) * up  (bfloat16),  gate/up = two accumulators;
//              MODE 2: y[pair(p), n] = w[pair(p)] * acc  (float32).
//   (src/quanta/minimax/moe.py:59-88; rows p sorted by expert, see the plan kernels.)
//
// The token rows are read in p order: MODE 1 reads a gathered copy of x (gather kernel below) as one box a
// stage, or, for steps of few tokens, the rows of x themselves as one box of one row each (gather_k);
// MODE 2 reads the act rows MODE 1 wrote.  Rows past the expert's last row compute garbage
// that the epilogue drops; TMA zero-fills past the end of a tensor, so K need not be a multiple of 64
// (it must be a multiple of 8: 16-byte rows).  No multicast: every tile comes from this GPU's memory through
// a plain per-block TMA load.  Tiles of 256 token rows are taken by two blocks together (see PAIR below).
//
// Every wait on an mbarrier is bounded; when one runs out the block records it in the status words,
// lets its copies in flight land, frees its TMEM and returns.
#include <cuda.h>

#include "common.cuh"

namespace {

constexpr int EG_M = 128;            // output features per block (UMMA M)
constexpr int EG_BK = 64;            // k elements per stage: 128 bytes, one swizzle row
constexpr int EG_THREADS = 192;        // producer warp, MMA warp, four epilogue warps
constexpr int EG_PAIR_THREADS = 320;   // a pair's blocks: eight epilogue warps
constexpr uint32_t EG_SPIN_LIMIT = 4u * 1000u * 1000u;
constexpr uint64_t EG_WAIT_NS = 200ull * 1000ull * 1000ull;   // no wait is longer than 0.2 s

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
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
// Bounded wait.  Returns false when another role gave up or the limit is reached (and then raises the flag).
__device__ __forceinline__ uint64_t global_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = global_ns();
  for (uint32_t it = 0; it < EG_SPIN_LIMIT; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if ((it & 63u) == 63u && global_ns() - t0 > EG_WAIT_NS) break;      // both an iteration and a time limit
  }
  *abort_flag = 1;
  return false;
}

// L2 policies: weights are read once per step by small tiles (evict first), token tiles by every row block (evict last)
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar,
                                            uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
      " [%0], [%1, {%2, %3}], [%4], %5;"
      ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar), "l"(policy) : "memory");
}

// K-major operand tile in shared memory, rows of 128 bytes, 128-byte swizzle: 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);          // start address
  // leading byte offset (bits 16-29): 0, the tile is one swizzle atom wide along k
  d |= (uint64_t)(1024 >> 4) << 32;                      // stride byte offset: 8 rows x 128 B
  d |= (uint64_t)1 << 46;                                // descriptor version (sm_100)
  d |= (uint64_t)2 << 61;                                // 128-byte swizzle
  return d;
}
// kind::f16, bfloat16 x bfloat16 -> float32, both operands K-major
__device__ __forceinline__ uint32_t umma_idesc(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// ---- a pair of blocks on neighbouring SMs computing one tile (cta_group::2) ----
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// the address, in the cluster's shared window, of the same variable in the block of rank `rank`
__device__ __forceinline__ uint32_t mapa_u32(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
// a block's own box, its bytes counted on a barrier that may be the pair's other block's
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar_cluster,
                                                 uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
      " [%0], [%1, {%2, %3}], [%4], %5;"
      ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar_cluster), "l"(policy) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc) : "memory");
}
// arrives, once the MMAs issued so far are done, on the barrier at this offset in both blocks of the pair
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(bar), "h"((uint16_t)3) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr) : "memory");
}

// silu(g) * u.  The exponential and the quotient are the fast ones (2 ulp); the result is rounded to bfloat16.
__device__ __forceinline__ float silu_mul(float g, float u) { return __fdividef(g, 1.f + __expf(-g)) * u; }

struct EgShared {
  uint64_t full[8];
  uint64_t empty[8];
  uint64_t tmem_full;
  uint32_t tmem_base;
  int abort_flag;
};

// NM: weight tiles of 128 features a block (accumulators side by side in TMEM).  MODE 1 has two by its nature
// (gate and up rows of the same features).  MODE 2 takes two neighbouring blocks of 128 features when the
// token tile is 256 rows (steps bound by the tensor cores): the token tile, half of what a stage holds then,
// is fetched from L2 once for 256 features instead of once for 128.
//
// PAIR: two blocks on neighbouring SMs (a cluster of two) take one tile of 256 token rows together, each
// 128 (MODE 1) or 256 (MODE 2) of its features: tcgen05.mma.cta_group::2 with M = 256.  Each block fetches
// its own weight tiles and HALF of the token tile, and the tensor cores of both read both halves, so a block
// takes three quarters of the bytes from L2, and reads two thirds of the bytes from its shared memory, that
// it would alone.  The first block of the pair issues all MMAs; every copy of either block counts on the
// first block's barrier; a commit frees the stage in both.
template <int MODE, int NM, bool PAIR>
__device__ __forceinline__ void
expert_gemm_tc_body(const CUtensorMap& tm_w, const CUtensorMap& tm_x,
                    void* __restrict__ out, const int* __restrict__ sorted_pair, const float* __restrict__ pair_w,
                    const int* __restrict__ plan, const int* __restrict__ tile_expert,
                    const int* __restrict__ tile_row0, int E, int K, int N_out, int NT, int stages,
                    int tmem_cols, int gather_k, int* status) {
  constexpr int FEATS = MODE == 1 ? EG_M : NM * EG_M;      // output features a block
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;     // 0: the block that issues the MMAs
  extern __shared__ unsigned char smem_dyn[];
  // stage buffers need 1024-byte alignment for the 128-byte swizzle
  unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
  __shared__ EgShared sh;
  __shared__ int s_pair[256];
  __shared__ float s_w[256];

  const int num_tiles = plan[3 * E + 1];
  const int tile = blockIdx.y;
  if (tile >= num_tiles) return;
  const int e = tile_expert[tile], row0 = tile_row0[tile];
  const int rows = min(NT, plan[2 * E + e + 1] - row0);          // valid token rows of this tile
  const int j0 = blockIdx.x * FEATS;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // the MMA's N is what this tile holds, in steps of 16: an expert's last tile of a few rows costs the
  // tensor cores a few columns, not a whole tile (the box that TMA fetches keeps its size)
  const int n_mma = min(NT, (rows + 15) & ~15);
  // a pair's block holds half of the MMA's token rows: rows [rank * n_mma / 2, +n_mma / 2) of the tile, as
  // the first rows of a box of NT / 2
  const uint32_t a_bytes = EG_M * EG_BK * 2, b_bytes = (uint32_t)(PAIR ? NT / 2 : NT) * EG_BK * 2;
  const uint32_t stage_bytes = NM * a_bytes + b_bytes;
  const int k_blocks = (K + EG_BK - 1) / EG_BK;
  volatile int* abort_flag = &sh.abort_flag;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(smem_u32(&sh.full[s]), 1);
      mbar_init(smem_u32(&sh.empty[s]), 1);
    }
    mbar_init(smem_u32(&sh.tmem_full), 1);
    sh.abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {      // one warp allocates the accumulator columns (in a pair: the same warp of both blocks)
    if (PAIR) {
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                   ::"r"(smem_u32(&sh.tmem_base)), "r"((uint32_t)tmem_cols) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                   ::"r"(smem_u32(&sh.tmem_base)), "r"((uint32_t)tmem_cols) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  if (MODE == 1 && gather_k > 0) {
    // the token rows are fetched one by one from the step's activations: row i of the tile is the token
    // of the i-th pair of this expert
    for (int i = threadIdx.x; i < rows; i += blockDim.x) s_pair[i] = sorted_pair[row0 + i] / gather_k;
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (PAIR) cluster_sync_all();      // both blocks' barriers exist before either counts on the other's
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = sh.tmem_base;

  if (warp == 0) {
    // ---------------- TMA producer: lane 0 waits and fetches the boxes; where the token rows are fetched
    // one by one, all lanes take their share of them ----------------
    const int w_row = MODE == 1 ? e * 2 * N_out + j0 : e * N_out + j0;
    // weights are read once per step by tiles of few rows (evict first); the 256-row tiles of one expert run at
    // about the same time and read the same weights, so those stay (measured: 5 % on a 16,384-token step)
    const uint64_t pol_w = PAIR ? l2_policy_evict_last() : l2_policy_evict_first(), pol_x = l2_policy_evict_last();
    const bool by_row = MODE == 1 && gather_k > 0;
    // the tile rows this block fetches: all of them, or a pair's half
    const int r_lo = PAIR ? (int)rank * (n_mma / 2) : 0;
    const int r_hi = PAIR ? min(rows, r_lo + n_mma / 2) : rows;
    int armed = 0;
    for (int kb = 0; kb < k_blocks; ++kb) {
      const int s = kb % stages;
      const uint32_t ph = (uint32_t)(kb / stages) & 1u;
      int ok = 1;
      if (lane == 0) ok = mbar_wait(smem_u32(&sh.empty[s]), ph ^ 1u, abort_flag) ? 1 : 0;
      if (!__shfl_sync(0xffffffffu, ok, 0)) break;
      const uint32_t full = smem_u32(&sh.full[s]);
      // a pair: every copy of either block counts on the first block's barrier, which expects both blocks'
      // bytes (the second block's copies may count before the first has said so)
      const uint32_t bar = PAIR ? mapa_u32(full, 0u) : full;
      unsigned char* st = tiles + (size_t)s * stage_bytes;
      if (lane == 0) {
        const uint32_t x_bytes = by_row ? (uint32_t)rows * EG_BK * 2 : (PAIR ? 2u : 1u) * b_bytes;
        if (rank == 0) mbar_expect_tx(full, (PAIR ? 2u : 1u) * NM * a_bytes + x_bytes);
        // the second weight tile: the up rows of the same features, or the next 128 features (rows past the
        // expert's last are another expert's and give columns that the epilogue drops)
        if (PAIR) {
          tma_load_2d_pair(smem_u32(st), &tm_w, kb * EG_BK, w_row, bar, pol_w);
          if (NM == 2) tma_load_2d_pair(smem_u32(st + a_bytes), &tm_w, kb * EG_BK, w_row + (MODE == 1 ? N_out : EG_M), bar, pol_w);
          if (!by_row) tma_load_2d_pair(smem_u32(st + NM * a_bytes), &tm_x, kb * EG_BK, row0 + r_lo, bar, pol_x);
        } else {
          tma_load_2d(smem_u32(st), &tm_w, kb * EG_BK, w_row, bar, pol_w);
          if (NM == 2) tma_load_2d(smem_u32(st + a_bytes), &tm_w, kb * EG_BK, w_row + (MODE == 1 ? N_out : EG_M), bar, pol_w);
          if (!by_row) tma_load_2d(smem_u32(st + NM * a_bytes), &tm_x, kb * EG_BK, row0, bar, pol_x);
        }
      }
      if (by_row) {
        // boxes of one row: the swizzle follows the shared-memory address, so a row lands where a box of
        // many rows would have put it; the rows past the expert's last keep what the stage held before, and
        // their columns of the product are never read
        for (int i = r_lo + lane; i < r_hi; i += 32) {
          const uint32_t dst = smem_u32(st + NM * a_bytes + (i - r_lo) * (EG_BK * 2));
          if (PAIR) tma_load_2d_pair(dst, &tm_x, kb * EG_BK, s_pair[i], bar, pol_x);
          else tma_load_2d(dst, &tm_x, kb * EG_BK, s_pair[i], bar, pol_x);
        }
      }
      armed = kb + 1;
    }
    if (lane == 0) {
      if (*abort_flag && PAIR && rank != 0) {
        // this block's copies count on the other block's barriers, which it cannot wait on: give them time
        const uint64_t t0 = global_ns();
        for (uint32_t it = 0; it < EG_SPIN_LIMIT && global_ns() - t0 < 100000ull; ++it) __nanosleep(1000);
      } else if (*abort_flag) {
        // let the copies that were issued land before this block's shared memory is given away
        for (int kb = max(0, armed - stages); kb < armed; ++kb) {
          const int s = kb % stages;
          const uint32_t ph = (uint32_t)(kb / stages) & 1u;
          const uint64_t t0 = global_ns();
          for (uint32_t it = 0; it < EG_SPIN_LIMIT && !mbar_try_wait(smem_u32(&sh.full[s]), ph); ++it)
            if ((it & 63u) == 63u && global_ns() - t0 > EG_WAIT_NS) break;
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = umma_idesc(PAIR ? 2 * EG_M : EG_M, n_mma);
      bool ok = true;
      for (int kb = 0; kb < k_blocks && ok; ++kb) {
        const int s = kb % stages;
        const uint32_t ph = (uint32_t)(kb / stages) & 1u;
        ok = mbar_wait(smem_u32(&sh.full[s]), ph, abort_flag);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t st = smem_u32(tiles + (size_t)s * stage_bytes);
        const uint64_t b_desc = umma_desc_sw128(st + NM * a_bytes);
#pragma unroll
        for (int m = 0; m < NM; ++m) {
          const uint64_t a_desc = umma_desc_sw128(st + m * a_bytes);
#pragma unroll
          for (int k16 = 0; k16 < EG_BK / 16; ++k16) {
            // 16 k elements = 32 bytes further along the swizzled row: +2 in the 16-byte address field
            if (PAIR)
              umma_bf16_pair(tmem_base + (uint32_t)(m * NT), a_desc + (uint64_t)(k16 * 2), b_desc + (uint64_t)(k16 * 2),
                             idesc, (kb | k16) != 0 ? 1u : 0u);
            else
              umma_bf16(tmem_base + (uint32_t)(m * NT), a_desc + (uint64_t)(k16 * 2), b_desc + (uint64_t)(k16 * 2), idesc,
                        (kb | k16) != 0 ? 1u : 0u);
          }
        }
        // the stage is free once these MMAs have read it
        if (PAIR) umma_commit_pair(smem_u32(&sh.empty[s])); else umma_commit(smem_u32(&sh.empty[s]));
      }
      if (ok) {
        if (PAIR) umma_commit_pair(smem_u32(&sh.tmem_full)); else umma_commit(smem_u32(&sh.tmem_full));
      }
    }
  } else {
    // ---------------- epilogue: one TMEM lane quadrant a warp (a warp reaches the 32 lanes of its index
    // modulo 4); a pair's blocks have two warps a quadrant that take the column chunks in turn ----------------
    constexpr int SPLIT = PAIR ? 2 : 1;
    constexpr int EPI_THREADS = SPLIT * 128;
    const int quad = warp & 3, sub = (warp - 2) >> 2;
    const int feat = j0 + quad * 32 + lane;
    if (MODE == 2) {
      // where each row goes and its routing weight: fetched here, under the main loop, by the warps that
      // need them at its end (two dependent reads that the producer and the issuer do not wait for)
      for (int i = threadIdx.x - 64; i < NT; i += EPI_THREADS) {
        const int pr = i < rows ? sorted_pair[row0 + i] : 0;
        s_pair[i] = pr;
        s_w[i] = i < rows ? pair_w[pr] : 0.f;
      }
      asm volatile("bar.sync 1, %0;" ::"n"(EPI_THREADS) : "memory");      // the epilogue warps
    }
    // tcgen05.ld / wait::ld are .sync.aligned: the whole warp runs them or none of it does, so the lanes
    // vote on the wait's answer (a lane may see another role's abort flag before its neighbour does)
    const bool acc_ready = __all_sync(0xffffffffu, mbar_wait(smem_u32(&sh.tmem_full), 0u, abort_flag) ? 1 : 0) != 0;
    if (acc_ready) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16);
      for (int c0 = 16 * sub; c0 < rows; c0 += 16 * SPLIT) {
        uint32_t v0[16], v1[16];
        tmem_ld16(lane_addr + (uint32_t)c0, v0);
        if (NM == 2) tmem_ld16(lane_addr + (uint32_t)(NT + c0), v1);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        // all 16 columns are computed (independent chains, one warp a scheduler has nothing else to hide
        // latency with); only the stores look at the row count
        if (MODE == 1) {
          __nv_bfloat16 r[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float g = __uint_as_float(v0[i]), u = __uint_as_float(v1[i]);
            r[i] = __float2bfloat16_rn(silu_mul(g, u));
          }
          if (feat < N_out) {
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(out) + (size_t)(row0 + c0) * N_out + feat;
#pragma unroll
            for (int i = 0; i < 16; ++i)
              if (c0 + i < rows) dst[(size_t)i * N_out] = r[i];
          }
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int col = c0 + i;
            if (col < rows) {
              float* dst = reinterpret_cast<float*>(out) + (size_t)s_pair[col] * N_out;
              const float w = s_w[col];
              if (feat < N_out) dst[feat] = w * __uint_as_float(v0[i]);
              if (NM == 2 && feat + EG_M < N_out) dst[feat + EG_M] = w * __uint_as_float(v1[i]);
            }
          }
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  // neither block of a pair leaves, or gives its accumulators back, while the other's MMAs may read its
  // shared memory or its epilogue its TMEM
  if (PAIR) cluster_sync_all();
  if (warp == 1) {
    if (PAIR)
      asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)tmem_cols) : "memory");
    else
      asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)tmem_cols) : "memory");
  }
  if (threadIdx.x == 0 && sh.abort_flag) qb_set_status(status, QB_STATUS_WAIT_TIMEOUT, tile, 5);
}

#define QB_EG_PARAMS                                                                                              \
  const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x, void* __restrict__ out,     \
      const int* __restrict__ sorted_pair, const float* __restrict__ pair_w, const int* __restrict__ plan,        \
      const int* __restrict__ tile_expert, const int* __restrict__ tile_row0, int E, int K, int N_out, int NT,    \
      int stages, int tmem_cols, int gather_k, int* status
#define QB_EG_ARGS tm_w, tm_x, out, sorted_pair, pair_w, plan, tile_expert, tile_row0, E, K, N_out, NT, stages, tmem_cols, gather_k, status

template <int MODE, int NM>
__global__ void __launch_bounds__(EG_THREADS, 2) expert_gemm_tc_kernel(QB_EG_PARAMS) {
  expert_gemm_tc_body<MODE, NM, false>(QB_EG_ARGS);
}
template <int MODE>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(EG_PAIR_THREADS, 1) expert_gemm_tc_pair_kernel(QB_EG_PARAMS) {
  expert_gemm_tc_body<MODE, 2, true>(QB_EG_ARGS);
}

// out[p, :] = x[sorted_pair[p] / top_k, :]   (rows of 16-byte chunks)
__global__ void gather_rows_kernel(const uint4* __restrict__ x, uint4* __restrict__ out,
                                   const int* __restrict__ sorted_pair, int n_pairs, int top_k, int chunks) {
  const size_t total = (size_t)n_pairs * chunks;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int p = (int)(i / chunks), c = (int)(i % chunks);
    out[i] = x[(size_t)(sorted_pair[p] / top_k) * chunks + c];
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}

// 2-D bfloat16 tensor [rows, K] row-major, boxes of [box_rows, 64] with the 128-byte swizzle
int make_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t K, uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return QB_ERR_UNSUPPORTED;
  const cuuint64_t dims[2] = {K, rows};
  const cuuint64_t strides[1] = {K * 2};
  const cuuint32_t box[2] = {EG_BK, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : QB_ERR_BAD_ARG;
}

}  // namespace

extern "C" int qb_gather_rows(const void* x, void* out, const int* sorted_pair, int n_pairs, int top_k, int K,
                              cudaStream_t stream) {
  if (n_pairs <= 0) return 0;
  if (K % 8) return QB_ERR_UNSUPPORTED;
  const size_t total = (size_t)n_pairs * (K / 8);
  const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  gather_rows_kernel<<<blocks, 256, 0, stream>>>((const uint4*)x, (uint4*)out, sorted_pair, n_pairs, top_k, K / 8);
  QB_LAUNCH_CHECK();
  return 0;
}

// x_rows: bf16 [n_pairs, K] in sorted order (mode 1: the gathered activations; mode 2: the act rows); or,
// mode 1 with gather_k > 0, the step's activations [n_rows, K] themselves: the kernel fetches the row of
// token sorted_pair[p] / gather_k for pair p (one TMA box a row: for steps of few tokens).
// weights: bf16 [E, (mode 1 ? 2 : 1) * N_out, K].  NT: token tile (16..256, a multiple of 16); the plan's
// tile list must have been made with the same NT.
extern "C" int qb_expert_gemm_tc(int mode, const void* x_rows, const void* weights, void* out, const int* sorted_pair,
                                 const float* pair_w, const int* plan, const int* tile_expert, const int* tile_row0,
                                 int max_tiles, int n_pairs, int E, int K, int N_out, int NT, int gather_k, int n_rows,
                                 int* status, cudaStream_t stream) {
  if (max_tiles <= 0 || n_pairs <= 0) return 0;
  if (K % 8 || K <= 0 || N_out <= 0 || NT < 16 || NT > 256 || NT % 16 || max_tiles > 65535) return QB_ERR_UNSUPPORTED;
  if (mode != 1 && mode != 2) return QB_ERR_BAD_ARG;
  // weight tiles a block: gate and up (mode 1); two blocks of 128 features for the down product of 256-row
  // token tiles (see the kernel)
  const int nm = (mode == 1 || NT >= 128) ? 2 : 1;
  const int feats = mode == 1 ? EG_M : nm * EG_M;
  // tiles of 256 token rows (steps bound by the tensor cores) are taken by pairs of blocks, see the kernel
  const bool pair = NT == 256;
  if (((uintptr_t)x_rows | (uintptr_t)weights) & 15) return QB_ERR_BAD_ARG;
  CUtensorMap tm_w, tm_x;
  int rc = make_map(&tm_w, weights, (uint64_t)E * (mode == 1 ? 2 : 1) * N_out, (uint64_t)K, EG_M);
  if (rc) return rc;
  if (gather_k < 0 || (gather_k > 0 && (mode != 1 || n_rows <= 0))) return QB_ERR_BAD_ARG;
  rc = gather_k > 0 ? make_map(&tm_x, x_rows, (uint64_t)n_rows, (uint64_t)K, 1u)
                    : make_map(&tm_x, x_rows, (uint64_t)n_pairs, (uint64_t)K, (uint32_t)(pair ? NT / 2 : NT));
  if (rc) return rc;
  const size_t stage_bytes = (size_t)nm * EG_M * EG_BK * 2 + (size_t)(pair ? NT / 2 : NT) * EG_BK * 2;
  // Two blocks share an SM (shared memory is the limit), so that one block's prologue and epilogue run
  // under the other's main loop; each gets a ring of about 105 KB.
  // a tile of 256 token rows has a block to itself on its SM (its two accumulators fill the TMEM)
  // and so has every block of a launch of no more blocks than there are SMs (a single token's step)
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
      sms = 1;
  }
  int grid_x = (N_out + feats - 1) / feats;
  if (pair) grid_x = (grid_x + 1) & ~1;      // a pair's second block may lie past the last feature: it drops its columns
  const size_t blocks = (size_t)grid_x * (size_t)max_tiles;
  const bool alone = NT > 128 || blocks <= (size_t)sms;
  // Token tiles of at most 32 rows (decode steps of a few tokens: short blocks, one expert's 128 features
  // each): three blocks an SM with rings of about 70 KB hide a block's prologue and epilogue better than
  // two with 105 KB (measured at 8 tokens: 154 + 80 us against 161 + 86 us for the two products of a layer).
  int stages = (int)((size_t)(alone ? 200 * 1024 : 105 * 1024) / stage_bytes);
  if (!alone && NT <= 32 && 72000 / stage_bytes >= 2) stages = (int)(72000 / stage_bytes);    // three blocks an SM
  // the down product of 64-row tiles (steps of 33 to 64 tokens): four blocks an SM with two stages each
  // (measured at 64 tokens: 308 us against 330 us)
  if (!alone && mode == 2 && NT == 64 && 50000 / stage_bytes >= 2) stages = (int)(50000 / stage_bytes);
  if (stages > 8) stages = 8;
  const int k_blocks = (K + EG_BK - 1) / EG_BK;
  if (stages > k_blocks) stages = k_blocks;
  if (stages < 2 && k_blocks >= 2) return QB_ERR_UNSUPPORTED;
  const size_t smem = stage_bytes * stages + 1024;
  int tmem_cols = 32;
  while (tmem_cols < nm * NT) tmem_cols *= 2;
  dim3 grid(grid_x, max_tiles);
  cudaError_t err;
#define QB_EG(KERNEL_, GK, THREADS_)                                                                                       \
  do {                                                                                                             \
    err = cudaFuncSetAttribute(KERNEL_, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                  \
    if (err != cudaSuccess) return (int)err;                                                                       \
    KERNEL_<<<grid, THREADS_, smem, stream>>>(tm_w, tm_x, out, sorted_pair, pair_w, plan, tile_expert, tile_row0, E, K, \
                                               N_out, NT, stages, tmem_cols, GK, status);                          \
  } while (0)
  if (pair && mode == 1) QB_EG(expert_gemm_tc_pair_kernel<1>, gather_k, EG_PAIR_THREADS);
  else if (pair) QB_EG(expert_gemm_tc_pair_kernel<2>, 0, EG_PAIR_THREADS);
  else if (mode == 1) QB_EG((expert_gemm_tc_kernel<1, 2>), gather_k, EG_THREADS);
  else if (nm == 2) QB_EG((expert_gemm_tc_kernel<2, 2>), 0, EG_THREADS);
  else QB_EG((expert_gemm_tc_kernel<2, 1>), 0, EG_THREADS);
#undef QB_EG
  QB_LAUNCH_CHECK();
  return 0;
}
