// Causal attention of a prefill chunk on the sm_100a tensor cores (tcgen05.mma, accumulators in TMEM).
//
// One CTA per (128-query tile, query head); keys and values come from the fp16 cache in tiles of 64 rows through
// four-stage rings fed by 3-D tiled TMA loads (no multicast; rows past the end of the sequence are outside the tensor
// map's extent and arrive as zeros).  Per PAIR of key tiles (2 p, 2 p + 1):
//   S[128 x 128] = Q[128 x 128] . (K_2p ; K_2p+1)^T  tcgen05.mma, A and B K-major (128-byte swizzle), fp32 in TMEM; the
//                                                    two K tiles sit in adjacent ring slots and form one N = 128 operand
// and per key tile j:
//   P            = exp2(S_j - m) with the causal mask four warps, one query row per thread (tcgen05.ld), P rounded to
//                                                    fp16 and stored to shared memory as the next A operand
//   O[128 x 128] += P[128 x 64] . V_j[64 x 128]      tcgen05.mma, B read MN-major straight from the [key][dim] rows
// An MMA of 128 rows occupies the tensor pipe for about 70 cycles whatever its N (measured: eight N = 64 score MMAs
// and four N = 128 P . V MMAs per tile took 1150 cycles of issue time), so the scores are issued 128 keys wide.
// TWO CHAINS per CTA: even key tiles belong to chain 0, odd ones to chain 1, each with its own four softmax warps, P
// tile, running (maximum, sum) and O accumulator; at the end the two partial results are merged per row like two
// splits of the key range.  One tile's chain - scores committed, TMEM read, P stored and fenced, P . V issued and
// committed - is a few thousand cycles of latency that one chain cannot hide.  CTAs are numbered from the heaviest
// query tile down, so the block scheduler's in-order hand-out is longest-job-first over the SMs.
// The running row maximum is only raised when it grew by more than 2^8 (P stays below 256, far inside fp16), so the
// accumulator in TMEM is rescaled a handful of times per row instead of once per tile; the row sums follow the same
// stale maximum and the final division makes the result exact again.  Roles: one thread feeds the K ring and one the
// V ring (a K slot is free again as soon as its S product is done, a V slot after its P . V), one thread issues the
// score MMAs and one the P . V MMAs.  The scores have two buffers of 128 TMEM columns; a buffer is free again as soon
// as both chains have read it into registers, so the scores run a pair ahead and the softmax warps only wait (for
// "O has taken the chain's previous tile", one commit) before they overwrite P or rescale O.  The query tile arrives
// by TMA as fp16 (the kernel before this one stores the rotated queries that way, pre-scaled).  One CTA per SM
// (193 KB of shared memory, all 512 TMEM columns).  Every wait is bounded (status 4).
#ifndef QMK_ATTENTION_TCGEN05_CUH_
#define QMK_ATTENTION_TCGEN05_CUH_

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "gemm_tcgen05.cuh"

namespace qmk_attn {

constexpr int D = 128, NQ = 16;                  // head dimension, query heads (two per kv head)
constexpr int TQ = 128, TK = 64;                 // queries per CTA, keys per tile
constexpr int CHAINS = 2;                        // even / odd key tiles
constexpr int THREADS = 64 + 128 * CHAINS + 64;  // warp 0 loads K, warp 1 issues the score MMAs, warps 2..5 / 6..9 own the 128 query rows of chain 0 / 1, warp 10 issues P . V, warp 11 loads V
constexpr uint32_t Q_BYTES = TQ * D * 2;         // two [128 x 64] swizzled tiles
constexpr uint32_t KV_STAGE_BYTES = 2 * TK * D * 2;   // K tile (two [64 x 64] halves of the head dimension), then the V tile
constexpr uint32_t P_BYTES = TQ * TK * 2;
constexpr int STAGES = 4;
constexpr uint32_t K_HALF_BYTES = TK * 128;      // one [64 keys x 64 dims] swizzled tile
// K: one ring per 64-wide half of the head dimension, slots adjacent (slots 2 q and 2 q + 1 form one 128-key operand);
// V: slots of two [64 keys x 64 dims] tiles
constexpr uint32_t OFF_K = Q_BYTES, OFF_V = OFF_K + 2 * STAGES * K_HALF_BYTES, OFF_P = OFF_V + STAGES * 2 * K_HALF_BYTES,
                   OFF_BARS = OFF_P + CHAINS * P_BYTES;
static_assert(OFF_P == Q_BYTES + STAGES * KV_STAGE_BYTES, "ring sizes");
constexpr size_t SMEM_BYTES = OFF_BARS + 256;
constexpr uint32_t TMEM_COLS = 512;              // scores of pair p in columns [128 (p mod 2), +128) (chain c: +64 c), O of chain c in [256 + 128 c, +128)
constexpr float RESCALE_THRESHOLD = 8.0f;        // log2 units

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, int c0, int c1, int c2, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(bar)
      : "memory");
}
// MN-major operand with the 128-byte swizzle: rows of 64 contiguous MN elements per K index; 8-row K groups 1024 bytes
// apart (stride byte offset), the next 64 MN elements `lbo_bytes` further on (leading byte offset).
__device__ __forceinline__ uint64_t smem_desc_mn_sw128(uint32_t addr, uint32_t lbo_bytes) {
  return static_cast<uint64_t>((addr & 0x3FFFFu) >> 4) | (static_cast<uint64_t>(lbo_bytes >> 4) << 16) | (64ull << 32) |
         (1ull << 46) | (2ull << 61);
}
constexpr uint32_t IDESC_S = (1u << 4) | (static_cast<uint32_t>(TK >> 3) << 17) | (static_cast<uint32_t>(TQ >> 4) << 24);
constexpr uint32_t IDESC_S2 = (1u << 4) | (static_cast<uint32_t>((2 * TK) >> 3) << 17) | (static_cast<uint32_t>(TQ >> 4) << 24);
constexpr uint32_t IDESC_PV = (1u << 4) | (1u << 16) /* B MN-major */ | (static_cast<uint32_t>(D >> 3) << 17) |
                              (static_cast<uint32_t>(TQ >> 4) << 24);

// 2^x for x <= 8 or so (differences to the row maximum in use): the hardware approximation, flushing the far tail to 0
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

#define QMK_TMEM_LD32(r, taddr)                                                                                       \
  asm volatile(                                                                                                       \
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "                                                                       \
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "                                       \
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"                       \
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),   \
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),        \
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),       \
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])                     \
      : "r"(taddr)                                                                                                    \
      : "memory")
#define QMK_TMEM_ST32(taddr, r)                                                                                       \
  asm volatile(                                                                                                       \
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "                                                                 \
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "                                      \
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"                              \
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), \
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),    \
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),   \
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])                                                    \
      : "memory")

// map_q: 2-D map of the fp16 queries [rows][16 heads x 128] (normalised, rotated, times scale * log2 e), boxes of
// {64, 128}, 128-byte swizzle; query t sits at position pos0 + t and sees
// cache rows 0 .. pos0 + t).  map_k / map_v: 3-D maps {128 dims, pos0 + T rows, layers x 8 kv heads} of the fp16
// caches, boxes of {64, 64, 1}, 128-byte swizzle.  out: fp16 [T][2048].  grid = ceil(T / 128) * 16 CTAs in one
// dimension, numbered from the heaviest (last) query tile down: causal tile i sees 2 (i + 1) key tiles of 64.
//
// Packed prompts (items != null): the rows hold several sequences, each padded to whole query tiles.  CTA i takes
// items[i] = {sequence, first row of the query tile, its position within the sequence, head | length << 8} (sorted
// from the heaviest down by the host) and reads that sequence's caches through maps_dev[2 seq], maps_dev[2 seq + 1]
// in device memory; T and pos0 are then not used.
__global__ void __launch_bounds__(THREADS, 1)
causal_attention_tc(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                    int layer_head0, __half *out, int T, int pos0, float scale, unsigned int *status,
                    unsigned long long budget_ns, const int4 *items, const CUtensorMap *maps_dev) {
  using namespace qmk_gemm;
  extern __shared__ __align__(1024) unsigned char attn_smem[];
  const uint32_t base = s32(attn_smem);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int total = static_cast<int>(gridDim.x), id = static_cast<int>(blockIdx.x);
  int head = id % NQ;
  int q0 = (total / NQ - 1 - id / NQ) * TQ;
  int pbase = pos0 + q0;                       // position of the tile's first query in its sequence
  const CUtensorMap *mk = &map_k, *mv = &map_v;
  if (items != nullptr) {
    const int4 it = items[id];
    head = it.w & 0xff;
    q0 = it.y;
    pbase = it.z;
    T = it.y - it.z + (it.w >> 8);             // the sequence's end among the rows
    mk = maps_dev + 2 * it.x;
    mv = mk + 1;
  }
  const int g = head >> 1;
  const int last_q = (q0 + TQ < T ? q0 + TQ : T) - 1;                                        // last live query of the tile
  const int ntiles = (pbase + last_q - q0) / TK + 1;                                        // key tiles it can see
  const uint32_t bars = base + OFF_BARS;
  auto k_full = [&](int s) { return bars + 8u * s; };
  auto k_empty = [&](int s) { return bars + 8u * (4 + s); };
  auto v_full = [&](int s) { return bars + 8u * (8 + s); };
  auto v_empty = [&](int s) { return bars + 8u * (12 + s); };
  auto s_full = [&](int b) { return bars + 8u * (16 + b); };       // two score buffers (pairs of tiles)
  auto s_free = [&](int b) { return bars + 8u * (18 + b); };
  auto p_ready = [&](int c) { return bars + 8u * (20 + c); };      // per chain
  auto pv_done = [&](int c) { return bars + 8u * (22 + c); };
  const uint32_t q_full = bars + 8u * 24;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(attn_smem + OFF_BARS + 8 * 25);
  static_assert(STAGES == 4 && CHAINS == 2, "barrier layout above");
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

  if ((base & 1023u) != 0u) {   // the swizzled tiles need a 1024-byte aligned window: report instead of computing garbage
    if (threadIdx.x == 0) atomicCAS(status, 0u, 5u);
    return;
  }
  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_q)) : "memory");
    if (items == nullptr) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_k)) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_v)) : "memory");
    }
    for (int s = 0; s < STAGES; ++s) {
      bar_init(k_full(s), 1); bar_init(k_empty(s), 1); bar_init(v_full(s), 1); bar_init(v_empty(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      bar_init(s_full(b), 1);
      bar_init(s_free(b), 4 * CHAINS);   // one arrival per softmax warp of either chain
    }
    for (int c = 0; c < CHAINS; ++c) {
      bar_init(p_ready(c), 4);      // one arrival per softmax warp of the chain
      bar_init(pv_done(c), 1);
    }
    bar_init(q_full, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s32(tmem_slot)), "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  pdl_wait();   // queries and this chunk's cache rows come from the kernel launched just before
  pdl_trigger();
  // the query tile and the K ring's first fill go out at once (thread 0 is the K producer and has just initialised
  // the barriers itself); a CTA's fixed costs weigh as much as its first key tiles
  auto load_tile = [&](bool is_v, int j) {
    const int s = j % STAGES;
    const uint32_t full = is_v ? v_full(s) : k_full(s);
    const uint32_t d0 = base + (is_v ? OFF_V + s * 2 * K_HALF_BYTES : OFF_K + s * K_HALF_BYTES);
    const uint32_t d1 = d0 + (is_v ? K_HALF_BYTES : STAGES * K_HALF_BYTES);
    bar_expect_tx(full, 2 * K_HALF_BYTES);
    tma_load_3d(d0, is_v ? mv : mk, 0, j * TK, layer_head0 + g, full);
    tma_load_3d(d1, is_v ? mv : mk, 64, j * TK, layer_head0 + g, full);
  };
  int k_prefilled = 0;
  if (items != nullptr && lane == 0 && (warp == 0 || warp == 3 + 4 * CHAINS)) {
    // descriptors written by a copy before this launch: the loading threads make them visible to their TMA unit
    asm volatile("fence.proxy.tensormap::generic.acquire.sys [%0], 128;" ::"l"(reinterpret_cast<uint64_t>(mk)) : "memory");
    asm volatile("fence.proxy.tensormap::generic.acquire.sys [%0], 128;" ::"l"(reinterpret_cast<uint64_t>(mv)) : "memory");
  }
  if (threadIdx.x == 0) {
    // the query tile: fp16, already times scale * log2 e (the softmax is an exp2), as two [128 x 64] boxes in the
    // K-major 128-byte-swizzled layout the score MMAs read; rows past the live ones hold other tokens' or stale
    // finite values and are never stored
    bar_expect_tx(q_full, Q_BYTES);
    tma_load_2d(base, &map_q, head * D, q0, q_full);
    tma_load_2d(base + TQ * 128, &map_q, head * D + 64, q0, q_full);
    for (; k_prefilled < STAGES && k_prefilled < ntiles; ++k_prefilled) load_tile(false, k_prefilled);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_o0 = tmem_base + 256u;  // S buffer b at tmem_base + 64 b, O of chain c at tmem_o0 + 128 c

  if (warp == 0 || warp == 3 + 4 * CHAINS) {
    if (lane == 0) {                       // ---- producers: the K ring (warp 0) and the V ring, tiles of 64 rows
      const bool is_v = warp != 0;
      int issued = is_v ? 0 : k_prefilled;
      for (int j = issued; j < ntiles; ++j) {
        const int s = j % STAGES;
        if (j >= STAGES && !bar_wait(is_v ? v_empty(s) : k_empty(s), ((j / STAGES) - 1) & 1, abort_flag, status, budget_ns)) break;
        if (*abort_flag) break;
        load_tile(is_v, j);
        issued = j + 1;
      }
      if (*abort_flag) {                   // copies already issued must land before the CTA may exit
        for (int jj = (issued > STAGES ? issued - STAGES : 0); jj < issued; ++jj) {
          const uint32_t bar = is_v ? v_full(jj % STAGES) : k_full(jj % STAGES);
          const unsigned long long t0 = gtime();
          while (!bar_try(bar, (jj / STAGES) & 1)) {
            if (gtime() - t0 > (budget_ns > 2000000ull ? budget_ns : 2000000ull)) break;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {                       // ---- score MMAs: S of tiles 2 p and 2 p + 1 as one N = 128 product
      bool ok = true;
      const int npairs = (ntiles + 1) >> 1;
      for (int p = 0; p < npairs && ok; ++p) {
        const int j0 = 2 * p, s0 = j0 % STAGES;               // s0 is 0 or 2: slots s0 and s0 + 1 are adjacent
        const bool two = j0 + 1 < ntiles;                     // (an odd last tile goes alone, 64 wide)
        ok = (p > 0 || bar_wait(q_full, 0, abort_flag, status, budget_ns)) &&
             bar_wait(k_full(s0), (j0 / STAGES) & 1, abort_flag, status, budget_ns) &&
             (!two || bar_wait(k_full(s0 + 1), (j0 / STAGES) & 1, abort_flag, status, budget_ns)) &&
             (p < 2 || bar_wait(s_free(p & 1), ((p >> 1) - 1) & 1, abort_flag, status, budget_ns));   // both chains have read pair p - 2
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t ts = tmem_base + 128u * static_cast<uint32_t>(p & 1);
#pragma unroll
        for (int kb = 0; kb < 2; ++kb) {                      // 64-wide halves of the head dimension, four K = 16 steps each
          const uint64_t da = smem_desc_sw128(base + kb * (TQ * 128));
          const uint64_t db = smem_desc_sw128(base + OFF_K + kb * (STAGES * K_HALF_BYTES) + s0 * K_HALF_BYTES);
#pragma unroll
          for (int i = 0; i < 4; ++i) mma_f16_ss(ts, da + 2u * i, db + 2u * i, (kb > 0 || i > 0) ? 1u : 0u, two ? IDESC_S2 : IDESC_S);
        }
        mma_commit(s_full(p & 1));
        mma_commit(k_empty(s0));             // the K slots can be refilled as soon as this product is done
        if (two) mma_commit(k_empty(s0 + 1));
      }
    }
  } else if (warp == 2 + 4 * CHAINS) {
    if (lane == 0) {                       // ---- P . V MMAs, tiles in order (chains alternate)
      bool ok = true;
      for (int j = 0; j < ntiles && ok; ++j) {
        const int c = j & 1, n = j >> 1;   // chain, and the tile's index within it
        ok = bar_wait(p_ready(c), n & 1, abort_flag, status, budget_ns) &&
             bar_wait(v_full(j % STAGES), (j / STAGES) & 1, abort_flag, status, budget_ns);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        // O_c += P_c . V_j: four steps of 16 keys; V rows are [key][dim], i.e. MN-major for the B operand
        const uint32_t vt = base + OFF_V + (j % STAGES) * 2 * K_HALF_BYTES;
        const uint64_t dp = smem_desc_sw128(base + OFF_P + static_cast<uint32_t>(c) * P_BYTES);
        const uint32_t to = tmem_o0 + 128u * static_cast<uint32_t>(c);
#pragma unroll
        for (int i = 0; i < 4; ++i)
          mma_f16_ss(to, dp + 2u * i, smem_desc_mn_sw128(vt + i * 16 * 128, K_HALF_BYTES), (n > 0 || i > 0) ? 1u : 0u, IDESC_PV);
        mma_commit(pv_done(c));            // O_c has taken tile j: P_c may be overwritten, O_c rescaled (or, at the end, read)
        mma_commit(v_empty(j % STAGES));
      }
    }
  } else {                                 // ---- softmax: chain = warp group, thread = query row = TMEM lane
    const int chain = (warp - 2) >> 2;
    const int quarter = warp & 3, row = quarter * 32 + lane;
    const int qpos = pbase + row;          // (rows past T compute on zeros and are not stored)
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t tmem_o = tmem_o0 + 128u * static_cast<uint32_t>(chain);
    const uint32_t p_tile = base + OFF_P + static_cast<uint32_t>(chain) * P_BYTES;
    float m_used = -INFINITY, l = 0.f;     // (m_used stays -inf while every key the chain has seen is masked for this row)
    bool ok = true;
    for (int j = chain; j < ntiles && ok; j += CHAINS) {
      const int n = j >> 1;               // the tile's index within the chain = its pair
      ok = __all_sync(0xffffffffu, bar_wait(s_full(n & 1), (n >> 1) & 1, abort_flag, status, budget_ns));
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t tmem_s = tmem_base + 128u * static_cast<uint32_t>(n & 1) + 64u * static_cast<uint32_t>(chain);
      uint32_t s0[32], s1[32];
      QMK_TMEM_LD32(s0, tmem_s + lane_base);
      QMK_TMEM_LD32(s1, tmem_s + lane_base + 32u);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");  // the scores are in registers: the buffer may be overwritten
      __syncwarp();
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(s_free(n & 1)) : "memory");
      const int k0 = j * TK;
      const bool diagonal = k0 + TK - 1 > pbase;            // some key of the tile is ahead of some query of the CTA
      if (diagonal) {
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          if (k0 + c > qpos) s0[c] = __float_as_uint(-INFINITY);
          if (k0 + 32 + c > qpos) s1[c] = __float_as_uint(-INFINITY);
        }
      }
      // (four independent chains: a single running maximum would be 64 dependent instructions)
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int c = 0; c < 32; ++c) mx4[c & 3] = fmaxf(mx4[c & 3], fmaxf(__uint_as_float(s0[c]), __uint_as_float(s1[c])));
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      // raise the maximum in use only when it is far behind (always from -inf)
      const bool raise = mx > m_used + RESCALE_THRESHOLD;
      const float m_new = raise ? mx : m_used;
      const float alpha = raise ? exp2f(m_used - m_new) : 1.0f;     // from -inf: exp2(-inf) = 0, l and O hold zeros at most
      if (n > 0) {   // P of the chain's previous tile must have been consumed, and O must be at rest, before either is touched
        ok = __all_sync(0xffffffffu, bar_wait(pv_done(chain), (n - 1) & 1, abort_flag, status, budget_ns));
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      }
      if (n > 0 && __any_sync(0xffffffffu, raise)) {
#pragma unroll 1
        for (int c = 0; c < D / 32; ++c) {
          uint32_t o[32];
          QMK_TMEM_LD32(o, tmem_o + lane_base + static_cast<uint32_t>(c * 32));
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          QMK_TMEM_ST32(tmem_o + lane_base + static_cast<uint32_t>(c * 32), o);
        }
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      }
      l *= alpha;
      m_used = m_new;
      const float m_sub = m_used == -INFINITY ? 0.f : m_used;   // a fully masked row so far: P = exp2(-inf - 0) = 0, not NaN
      // P = exp2(S - m), fp16, into the swizzled A tile: row `row`, eight 16-byte segments of eight keys
      const uint32_t prow = p_tile + static_cast<uint32_t>(row) * 128u;
      const uint32_t x = static_cast<uint32_t>(row & 7);
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int seg = 0; seg < 8; ++seg) {
        uint32_t packed[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int c = seg * 8 + 2 * i;
          const float a = fast_exp2(__uint_as_float(c < 32 ? s0[c] : s1[c - 32]) - m_sub);
          const float b = fast_exp2(__uint_as_float(c + 1 < 32 ? s0[c + 1] : s1[c + 1 - 32]) - m_sub);
          sum4[i] += a + b;
          const __half2 h = __floats2half2_rn(a, b);
          packed[i] = *reinterpret_cast<const uint32_t *>(&h);
        }
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(prow + ((static_cast<uint32_t>(seg) ^ x) << 4)),
                     "r"(packed[0]), "r"(packed[1]), "r"(packed[2]), "r"(packed[3]) : "memory");
      }
      l += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // P before the MMA's async-proxy reads
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");  // S reads / O writes before the MMAs that follow
      __syncwarp();
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(p_ready(chain)) : "memory");
    }
    const int my_tiles = (ntiles - chain + 1) / CHAINS;
    if (ok && my_tiles > 0) ok = __all_sync(0xffffffffu, bar_wait(pv_done(chain), (my_tiles - 1) & 1, abort_flag, status, budget_ns));
    // ---- merge of the two chains.  (m, l) of this chain's row go through its own P tile, which its last product has
    // finished reading; every softmax warp reaches the barrier whatever its waits returned.
    asm volatile("st.shared.v2.f32 [%0], {%1, %2};" ::"r"(p_tile + static_cast<uint32_t>(row) * 8u), "f"(m_used), "f"(l) : "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    asm volatile("bar.sync 1, %0;" ::"n"(128 * CHAINS) : "memory");
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    float m_other, l_other;
    asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(m_other), "=f"(l_other)
                 : "r"(base + OFF_P + static_cast<uint32_t>(chain ^ 1) * P_BYTES + static_cast<uint32_t>(row) * 8u) : "memory");
    ok = ok && !*abort_flag;
    if (ok) {
      // chain 0 always holds key 0, which every query sees: the common maximum is finite
      const bool two = ntiles > 1;                           // chain 1 has an accumulator at all
      const float m_a = chain == 0 ? m_used : m_other, l_a = chain == 0 ? l : l_other;
      const float m_b = chain == 0 ? m_other : m_used, l_b = chain == 0 ? l_other : l;
      const float m_all = two ? fmaxf(m_a, m_b) : m_a;
      const float f_a = exp2f(m_a - m_all), f_b = two ? exp2f(m_b - m_all) : 0.f;   // (m_b = -inf: every key masked, 0)
      const float inv = 1.0f / (l_a * f_a + (two ? l_b * f_b : 0.f));
      const float fa = f_a * inv, fb = f_b * inv;
      const int t = q0 + row;
      // this warp group writes dims [64 chain, +64) of the row from both accumulators
      __half *orow = out + static_cast<size_t>(t < T ? t : 0) * (NQ * D) + head * D + 64 * chain;
#pragma unroll 1
      for (int c = 0; c < 2; ++c) {
        const uint32_t col = static_cast<uint32_t>(64 * chain + 32 * c);
        uint32_t oa[32], ob[32];
        QMK_TMEM_LD32(oa, tmem_o0 + lane_base + col);
        if (two) QMK_TMEM_LD32(ob, tmem_o0 + 128u + lane_base + col);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (t < T) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint32_t packed[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              float v0 = __uint_as_float(oa[i + 2 * k]) * fa, v1 = __uint_as_float(oa[i + 2 * k + 1]) * fa;
              if (two) {
                v0 = fmaf(__uint_as_float(ob[i + 2 * k]), fb, v0);
                v1 = fmaf(__uint_as_float(ob[i + 2 * k + 1]), fb, v1);
              }
              const __half2 h = __floats2half2_rn(v0, v1);
              packed[k] = *reinterpret_cast<const uint32_t *>(&h);
            }
            *reinterpret_cast<uint4 *>(orow + c * 32 + i) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
          }
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

}  // namespace qmk_attn
#endif  // QMK_ATTENTION_TCGEN05_CUH_
