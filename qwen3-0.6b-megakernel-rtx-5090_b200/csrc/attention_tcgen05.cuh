// Causal attention of a prefill chunk on the sm_100a tensor cores (tcgen05.mma, accumulators in TMEM).
//
// One CTA per (128-query tile, query head); keys and values come from the fp16 cache in tiles of 64 rows through a
// two-stage ring fed by 3-D tiled TMA loads (no multicast; rows past the end of the sequence are outside the tensor
// map's extent and arrive as zeros).  Per key tile:
//   S[128 x 64]  = Q[128 x 128] . K_tile^T          tcgen05.mma, A and B K-major (128-byte swizzle), fp32 in TMEM
//   P            = exp2(S - m) with the causal mask  four warps, one query row per thread (tcgen05.ld), P rounded to
//                                                    fp16 and stored to shared memory as the next A operand
//   O[128 x 128] += P[128 x 64] . V_tile[64 x 128]   tcgen05.mma, B read MN-major straight from the [key][dim] rows
// The running row maximum is only raised when it grew by more than 2^8 (P stays below 256, far inside fp16), so the
// accumulator in TMEM is rescaled a handful of times per row instead of once per tile; the row sums follow the same
// stale maximum and the final division makes the result exact again.  One thread feeds the K and V rings (two
// stages each; a K slot is free again as soon as its S product is done, a V slot after its P . V), one thread issues
// every MMA.  S is double-buffered in TMEM: the product for tile j + 1 is issued before the thread waits for P of tile
// j, so the softmax warps find their next tile ready and only wait (for "O has taken tile j", one commit) before they
// overwrite P or rescale O.  Two CTAs share an SM (112 KB of shared memory, 256 TMEM columns each): one's softmax
// runs under the other's MMAs.  Every wait is bounded (status 4).
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
constexpr int THREADS = 192;                     // warp 0 loads, warp 1 issues MMAs, warps 2..5 own the 128 query rows
constexpr uint32_t Q_BYTES = TQ * D * 2;         // two [128 x 64] swizzled tiles
constexpr uint32_t KV_STAGE_BYTES = 2 * TK * D * 2;   // K tile (two [64 x 64] halves of the head dimension), then the V tile
constexpr uint32_t P_BYTES = TQ * TK * 2;
constexpr int STAGES = 2;
constexpr uint32_t OFF_KV = Q_BYTES, OFF_P = OFF_KV + STAGES * KV_STAGE_BYTES, OFF_BARS = OFF_P + P_BYTES;
constexpr size_t SMEM_BYTES = OFF_BARS + 128;
constexpr uint32_t TMEM_COLS = 256;              // S buffers in columns [0, 64) and [64, 128), O in [128, 256)
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

// qr: fp32 [T][16 heads][128] (normalised, rotated queries of the chunk; query t sits at position pos0 + t and sees
// cache rows 0 .. pos0 + t).  map_k / map_v: 3-D maps {128 dims, pos0 + T rows, layers x 8 kv heads} of the fp16
// caches, boxes of {64, 64, 1}, 128-byte swizzle.  out: fp16 [T][2048].  grid = ceil(T / 128) * 16 CTAs in one
// dimension; `first_wave` = CTAs that start at once with one CTA per SM (the SM count).
//
// Work per CTA grows with the position of its query tile (causal: tile i sees 2 (i + 1) key tiles of 64).  CTAs are
// therefore numbered so that the block scheduler, which hands them out in order, gives every SM one heavy and one
// light tile: ids below `first_wave` take the (tile, head) pairs from the heaviest down, the ids after that take the
// remaining pairs from the LIGHTEST up - SM k's second CTA (id first_wave + k) is the lighter the heavier its first.
__global__ void __launch_bounds__(THREADS, 2)
causal_attention_tc(const float *qr, const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                    int layer_head0, __half *out, int T, int pos0, float scale, unsigned int *status,
                    unsigned long long budget_ns, int first_wave) {
  using namespace qmk_gemm;
  extern __shared__ __align__(1024) unsigned char attn_smem[];
  const uint32_t base = s32(attn_smem);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int total = static_cast<int>(gridDim.x), id = static_cast<int>(blockIdx.x);
  const int rank = id < first_wave ? id : total - 1 - (id - first_wave);     // position in the heaviest-first order
  const int head = rank % NQ, g = head >> 1;
  const int q0 = (total / NQ - 1 - rank / NQ) * TQ;
  const int last_q = (q0 + TQ < T ? q0 + TQ : T) - 1;                                        // last live query of the tile
  const int ntiles = (pos0 + last_q) / TK + 1;                                              // key tiles it can see
  const uint32_t bars = base + OFF_BARS;
  auto k_full = [&](int s) { return bars + 8u * s; };
  auto k_empty = [&](int s) { return bars + 8u * (2 + s); };
  auto v_full = [&](int s) { return bars + 8u * (4 + s); };
  auto v_empty = [&](int s) { return bars + 8u * (6 + s); };
  auto s_full = [&](int b) { return bars + 8u * (8 + b); };
  const uint32_t p_ready = bars + 8u * 10, pv_done = bars + 8u * 11;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(attn_smem + OFF_BARS + 8 * 12);
  static_assert(STAGES == 2, "barrier layout above");
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

  if ((base & 1023u) != 0u) {   // the swizzled tiles need a 1024-byte aligned window: report instead of computing garbage
    if (threadIdx.x == 0) atomicCAS(status, 0u, 5u);
    return;
  }
  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_k)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_v)) : "memory");
    for (int s = 0; s < STAGES; ++s) {
      bar_init(k_full(s), 1); bar_init(k_empty(s), 1); bar_init(v_full(s), 1); bar_init(v_empty(s), 1); bar_init(s_full(s), 1);
    }
    bar_init(p_ready, 4);      // one arrival per softmax warp
    bar_init(pv_done, 1);
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
  if (warp >= 2) {
    // Q tile: fp32 -> fp16 (times scale * log2 e, so that the softmax is an exp2), stored as two [128 x 64] tiles in
    // the K-major 128-byte-swizzled layout: row r, 16-byte segment s of a tile at r * 128 + ((s ^ (r & 7)) << 4)
    const float sc = scale * 1.4426950408889634f;
    const int w = warp - 2;
    for (int r = w; r < TQ; r += 4) {
      const int t = q0 + r;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (t < T) v = *reinterpret_cast<const float4 *>(qr + (static_cast<size_t>(t) * NQ + head) * D + 4 * lane);
      const __half2 lo = __floats2half2_rn(v.x * sc, v.y * sc), hi = __floats2half2_rn(v.z * sc, v.w * sc);
      const int d = 4 * lane, tile = d >> 6, seg = (d & 63) >> 3, within = (d & 7) * 2;
      const uint32_t addr = base + tile * (TQ * 128) + r * 128 + (((seg ^ (r & 7)) << 4)) + within;
      asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(addr), "r"(*reinterpret_cast<const uint32_t *>(&lo)),
                   "r"(*reinterpret_cast<const uint32_t *>(&hi)) : "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_o = tmem_base + 128u;   // S buffer b at tmem_base + 64 b

  if (warp == 0) {
    if (lane == 0) {                       // ---- producer: K and V tiles of 64 rows, each ring on its own barriers
      int issued = 0;
      for (int j = 0; j < ntiles; ++j) {
        const int s = j % STAGES;
        const uint32_t dst = base + OFF_KV + s * KV_STAGE_BYTES;
        if (j >= STAGES && !bar_wait(k_empty(s), ((j / STAGES) - 1) & 1, abort_flag, status, budget_ns)) break;
        if (*abort_flag) break;
        bar_expect_tx(k_full(s), KV_STAGE_BYTES / 2);
        tma_load_3d(dst, &map_k, 0, j * TK, layer_head0 + g, k_full(s));
        tma_load_3d(dst + TK * 128, &map_k, 64, j * TK, layer_head0 + g, k_full(s));
        if (j >= STAGES && !bar_wait(v_empty(s), ((j / STAGES) - 1) & 1, abort_flag, status, budget_ns)) { issued = 2 * j + 1; break; }
        bar_expect_tx(v_full(s), KV_STAGE_BYTES / 2);
        tma_load_3d(dst + 2 * TK * 128, &map_v, 0, j * TK, layer_head0 + g, v_full(s));
        tma_load_3d(dst + 3 * TK * 128, &map_v, 64, j * TK, layer_head0 + g, v_full(s));
        issued = 2 * j + 2;
      }
      if (*abort_flag) {                   // copies already issued must land before the CTA may exit
        // `issued` counts half-tiles in issue order (K of tile 0, V of tile 0, K of tile 1, ...): wait for the last four
        for (int h = (issued > 2 * STAGES ? issued - 2 * STAGES : 0); h < issued; ++h) {
          const int jj = h >> 1;
          const uint32_t bar = (h & 1) ? v_full(jj % STAGES) : k_full(jj % STAGES);
          const unsigned long long t0 = gtime();
          while (!bar_try(bar, (jj / STAGES) & 1)) {
            if (gtime() - t0 > (budget_ns > 2000000ull ? budget_ns : 2000000ull)) break;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {                       // ---- MMA issuer
      bool ok = true;
      // S_j = Q . K_j^T into S buffer j mod 2: two 64-wide halves of the head dimension, four K = 16 steps each
      auto issue_s = [&](int j) {
        const uint32_t kt = base + OFF_KV + (j % STAGES) * KV_STAGE_BYTES;
        const uint32_t ts = tmem_base + 64u * static_cast<uint32_t>(j & 1);
#pragma unroll
        for (int kb = 0; kb < 2; ++kb) {
          const uint64_t da = smem_desc_sw128(base + kb * (TQ * 128));
          const uint64_t db = smem_desc_sw128(kt + kb * (TK * 128));
#pragma unroll
          for (int i = 0; i < 4; ++i) mma_f16_ss(ts, da + 2u * i, db + 2u * i, (kb > 0 || i > 0) ? 1u : 0u, IDESC_S);
        }
        mma_commit(s_full(j & 1));
        mma_commit(k_empty(j % STAGES));   // the K slot can be refilled as soon as this product is done
      };
      ok = bar_wait(k_full(0), 0, abort_flag, status, budget_ns);
      if (ok) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        issue_s(0);
      }
      for (int j = 0; j < ntiles && ok; ++j) {
        if (j + 1 < ntiles) {
          // next tile's scores first: its S buffer was last read for tile j - 1, whose P this thread has already
          // waited for, and the softmax warps find it ready when they are done with tile j
          ok = bar_wait(k_full((j + 1) % STAGES), ((j + 1) / STAGES) & 1, abort_flag, status, budget_ns);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          issue_s(j + 1);
        }
        ok = bar_wait(p_ready, j & 1, abort_flag, status, budget_ns) &&
             bar_wait(v_full(j % STAGES), (j / STAGES) & 1, abort_flag, status, budget_ns);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        // O += P . V_j: four steps of 16 keys; V rows are [key][dim], i.e. MN-major for the B operand
        const uint32_t vt = base + OFF_KV + (j % STAGES) * KV_STAGE_BYTES + 2 * TK * 128;
        const uint64_t dp = smem_desc_sw128(base + OFF_P);
#pragma unroll
        for (int i = 0; i < 4; ++i)
          mma_f16_ss(tmem_o, dp + 2u * i, smem_desc_mn_sw128(vt + i * 16 * 128, TK * 128), (j > 0 || i > 0) ? 1u : 0u, IDESC_PV);
        mma_commit(pv_done);               // O has taken tile j: P may be overwritten, O rescaled (or, at the end, read)
        mma_commit(v_empty(j % STAGES));
      }
    }
  } else {                                 // ---- softmax: thread = query row = TMEM lane
    const int quarter = warp & 3, row = quarter * 32 + lane;
    const int qpos = pos0 + q0 + row;      // (rows past T compute on zeros and are not stored)
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < ntiles && ok; ++j) {
      ok = __all_sync(0xffffffffu, bar_wait(s_full(j & 1), (j >> 1) & 1, abort_flag, status, budget_ns));
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t tmem_s = tmem_base + 64u * static_cast<uint32_t>(j & 1);
      uint32_t s0[32], s1[32];
      QMK_TMEM_LD32(s0, tmem_s + lane_base);
      QMK_TMEM_LD32(s1, tmem_s + lane_base + 32u);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      const int k0 = j * TK;
      const bool diagonal = k0 + TK - 1 > pos0 + q0;        // some key of the tile is ahead of some query of the CTA
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
      // raise the maximum in use only when it is far behind (first tile: always; key 0 is visible to every query)
      const bool raise = mx > m_used + RESCALE_THRESHOLD;
      const float m_new = raise ? mx : m_used;
      const float alpha = raise ? exp2f(m_used - m_new) : 1.0f;     // first tile: exp2(-inf) = 0, l and O are empty
      if (j > 0) {   // P of tile j - 1 must have been consumed, and O must be at rest, before either is touched
        ok = __all_sync(0xffffffffu, bar_wait(pv_done, (j - 1) & 1, abort_flag, status, budget_ns));
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      }
      if (j > 0 && __any_sync(0xffffffffu, raise)) {
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
      // P = exp2(S - m), fp16, into the swizzled A tile: row `row`, eight 16-byte segments of eight keys
      const uint32_t prow = base + OFF_P + static_cast<uint32_t>(row) * 128u;
      const uint32_t x = static_cast<uint32_t>(row & 7);
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int seg = 0; seg < 8; ++seg) {
        uint32_t packed[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int c = seg * 8 + 2 * i;
          const float a = fast_exp2(__uint_as_float(c < 32 ? s0[c] : s1[c - 32]) - m_used);
          const float b = fast_exp2(__uint_as_float(c + 1 < 32 ? s0[c + 1] : s1[c + 1 - 32]) - m_used);
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
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(p_ready) : "memory");
    }
    ok = ok && __all_sync(0xffffffffu, bar_wait(pv_done, (ntiles - 1) & 1, abort_flag, status, budget_ns));
    if (ok) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const float inv = 1.0f / l;
      const int t = q0 + row;
      __half *orow = out + static_cast<size_t>(t < T ? t : 0) * (NQ * D) + head * D;
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        uint32_t o[32];
        QMK_TMEM_LD32(o, tmem_o + lane_base + static_cast<uint32_t>(c * 32));
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (t < T) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint32_t packed[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const __half2 h = __floats2half2_rn(__uint_as_float(o[i + 2 * k]) * inv, __uint_as_float(o[i + 2 * k + 1]) * inv);
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
