// C[M x N] (fp32) = A[M x K] (fp16, row-major) * B[N x K]^T (fp16, row-major) on the sm_100a tensor cores.
//
// One CTA per 128 x BN output tile (BN = 128, or 64 when 128-wide tiles would leave most SMs idle),
// warp-specialised:
//   warp 0   : one thread streams 128 x 64 tiles of A and BN x 64 tiles of B with tiled TMA loads (128-byte
//              swizzle) into a 4-stage shared-memory ring (full/empty mbarriers);
//   warp 1   : allocates BN TMEM columns, then one thread issues tcgen05.mma (M 128, N BN, K 16; four per
//              64-wide K block) with shared-memory matrix descriptors, commits each stage back to the
//              producer and finally commits the accumulator to the epilogue;
//   warps 2-5: read the fp32 accumulator from TMEM (tcgen05.ld, each warp its own 32-lane quarter) and store
//              it to global memory.
// Every mbarrier wait is bounded by a clock budget; a wait that runs out sets *status = 4 and all roles
// leave their loops (outstanding copies are given the same budget to land, TMEM is freed) so that the
// context survives.  No cluster multicast anywhere.
//
// Shapes: M, N multiples of 128, K a multiple of 64 (the callers pad the token dimension).
#ifndef QMK_GEMM_TCGEN05_CUH_
#define QMK_GEMM_TCGEN05_CUH_

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace qmk_gemm {

constexpr int BM = 128, BK = 64;                 // BK * 2 bytes = one 128-byte swizzle row; the N tile (128 or 64) is a template parameter
// Ring depth per N-tile variant: as many stages as fit in ~192 KB (a skinny M = 128 problem is bound by the
// latency of its K loop, so the whole K extent of a 1024-wide matrix is in flight at once).
constexpr int stages_for(int bn) { return bn == 32 ? 10 : bn == 64 ? 8 : 6; }
constexpr int MAX_GROUPS = 3;   // matrices sharing one A operand that one launch can multiply (q/k/v, gate/up)
constexpr int THREADS = 192;
constexpr uint32_t TILE_A_BYTES = BM * BK * 2;   // 16 KB
constexpr uint32_t stage_bytes_for(int bn) { return TILE_A_BYTES + static_cast<uint32_t>(bn) * BK * 2; }
constexpr size_t smem_bytes_for(int bn) {
  return 1024 /* alignment slack */ + static_cast<size_t>(stages_for(bn)) * stage_bytes_for(bn) + 256;
}

__device__ __forceinline__ uint32_t s32(const void *p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ unsigned long long gtime() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void bar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void bar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool bar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: false when the budget ran out or another role already gave up.
__device__ __forceinline__ bool bar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, unsigned int *status,
                                         unsigned long long budget_ns) {
  if (bar_try(bar, parity)) return true;
  const unsigned long long t0 = gtime();
  uint32_t it = 0;
  for (;;) {
    if (bar_try(bar, parity)) return true;
    if ((++it & 63u) == 0u) {
      if (*abort_flag) return false;
      if (gtime() - t0 > budget_ns) {
        *abort_flag = 1;
        atomicCAS(status, 0u, 4u);
        return false;
      }
    }
  }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int c0, int c1, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar)
      : "memory");
}
// Shared-memory matrix descriptor of a K-major tile stored as rows of 128 bytes with the 128-byte swizzle:
// 8-row groups are 1024 bytes apart (stride byte offset), version 1 (sm_100), layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
  return static_cast<uint64_t>((addr & 0x3FFFFu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor: fp32 accumulator, fp16 A and B, both K-major, N >> 3 at bit 17, M >> 4 at bit 24.
constexpr uint32_t idesc_for(int bn) {
  return (1u << 4) | (static_cast<uint32_t>(bn >> 3) << 17) | (static_cast<uint32_t>(BM >> 4) << 24);
}

__device__ __forceinline__ void mma_f16_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t accumulate,
                                           uint32_t IDESC) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t"
      "}\n"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(IDESC), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
      : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// Up to three B matrices (same K) against one A in one launch: blockIdx.x counts the N tiles of group 0, then of
// group 1, then of group 2; C_g is [M x N_g].
struct Groups {
  float *C[MAX_GROUPS];
  int N[MAX_GROUPS];
  // Split-K (single group only): gridDim.z CTAs share an output tile, CTA z multiplies K blocks
  // [z * kblocks_per_split, (z + 1) * kblocks_per_split) and writes its partial sums to C + z * split_stride
  // (floats); the consumer adds the partial matrices in a fixed order.  0 = no split.
  int kblocks_per_split;
  size_t split_stride;
  // Bytes one A box brings in (0 = the whole 128 x 64 tile).  A map whose box has fewer than 128 rows fills only
  // the first rows of the tile; the MMA still reads all 128, so output rows past the box are garbage and the
  // caller must not store them (kernel argument M <= box rows).
  uint32_t a_box_bytes;
};

// FUSE (BN = 32 or 64): B0 is the gate matrix and B1 the up matrix of a SwiGLU MLP; the CTA keeps two accumulators
// (gate tile in TMEM columns [0, BN), up tile in [BN, 2 BN)) and its epilogue writes fp16 silu(gate) * up to
// groups.C[0] (reinterpreted as __half [M x N]) instead of two fp32 matrices.
template <int BN, bool FUSE = false>
__global__ void __launch_bounds__(THREADS, 1)
gemm_f16_tn_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b0,
                   const __grid_constant__ CUtensorMap map_b1, const __grid_constant__ CUtensorMap map_b2,
                   const Groups groups, int M, int K, unsigned int *status, unsigned long long budget_ns,
                   int selftest_no_loads) {
  static_assert(BN == 32 || BN == 64 || BN == 128, "N tiles of 32, 64 or 128 columns");
  static_assert(!FUSE || BN <= 64, "the fused SwiGLU epilogue keeps two accumulators of at most 64 columns");
  constexpr int SB = FUSE ? 2 * BN : BN;          // B rows held per stage / accumulator columns
  constexpr int STAGES = stages_for(SB);
  constexpr uint32_t STAGE_BYTES = stage_bytes_for(SB);
  // which matrix this CTA works on
  int tile = blockIdx.x, grp = 0;
  if (!FUSE && tile >= groups.N[0] / BN) { tile -= groups.N[0] / BN; grp = 1; }
  if (!FUSE && grp == 1 && tile >= groups.N[1] / BN) { tile -= groups.N[1] / BN; grp = 2; }
  const CUtensorMap *map_b = grp == 0 ? &map_b0 : grp == 1 ? &map_b1 : &map_b2;
  float *C = grp == 0 ? groups.C[0] : grp == 1 ? groups.C[1] : groups.C[2];
  const int N = grp == 0 ? groups.N[0] : grp == 1 ? groups.N[1] : groups.N[2];
  extern __shared__ unsigned char gemm_smem_raw[];
  const uint32_t raw = s32(gemm_smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;                 // swizzled tiles need 1024-byte alignment
  unsigned char *aligned = gemm_smem_raw + (base - raw);
  const uint32_t bars = base + STAGES * STAGE_BYTES;            // full[STAGES], empty[STAGES], acc_full, then scratch
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(aligned + STAGES * STAGE_BYTES + 8 * (2 * STAGES + 1));
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = tile * BN, m0 = blockIdx.y * BM;
  const int kblocks = groups.kblocks_per_split > 0 ? groups.kblocks_per_split : K / BK;
  const int kb0 = groups.kblocks_per_split > 0 ? static_cast<int>(blockIdx.z) * groups.kblocks_per_split : 0;
  constexpr uint32_t TILE_B_BYTES = BN * BK * 2;
  constexpr uint32_t TMEM_COLS = SB;             // fp32 accumulator(s): 128 lanes x SB columns (a power of two >= 32)
  auto full = [&](int s) { return bars + 8u * s; };
  auto empty = [&](int s) { return bars + 8u * (STAGES + s); };
  const uint32_t acc_full = bars + 8u * (2 * STAGES);

  // the first fill of the ring needs no free-slot wait: thread 0 issues it before the CTA-wide barrier below, so
  // that the first TMA round trip overlaps the TMEM allocation
  const int prologue = selftest_no_loads ? 0 : (kblocks < STAGES ? kblocks : STAGES);
  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_a)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map_b)) : "memory");
    if (FUSE) asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_b1)) : "memory");
    for (int s = 0; s < STAGES; ++s) { bar_init(full(s), 1); bar_init(empty(s), 1); }
    bar_init(acc_full, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    for (int kb = 0; kb < prologue; ++kb) {
      bar_expect_tx(full(kb), (groups.a_box_bytes ? groups.a_box_bytes : TILE_A_BYTES) + (FUSE ? 2 : 1) * TILE_B_BYTES);
      tma_load_2d(base + kb * STAGE_BYTES, &map_a, (kb0 + kb) * BK, m0, full(kb));
      tma_load_2d(base + kb * STAGE_BYTES + TILE_A_BYTES, map_b, (kb0 + kb) * BK, n0, full(kb));
      if (FUSE) tma_load_2d(base + kb * STAGE_BYTES + TILE_A_BYTES + TILE_B_BYTES, &map_b1, (kb0 + kb) * BK, n0, full(kb));
    }
  }
  if (warp == 1) {   // the whole warp allocates; the address lands in shared memory
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s32(tmem_slot)), "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {                       // ---- producer
      int issued = prologue;
      // self test of the bounded waits: the loads are never issued, so the MMA thread's first wait runs out
      for (int kb = prologue; kb < (selftest_no_loads ? 0 : kblocks); ++kb) {
        const int s = kb % STAGES;
        if (kb >= STAGES && !bar_wait(empty(s), ((kb / STAGES) - 1) & 1, abort_flag, status, budget_ns)) break;
        if (*abort_flag) break;
        bar_expect_tx(full(s), (groups.a_box_bytes ? groups.a_box_bytes : TILE_A_BYTES) + (FUSE ? 2 : 1) * TILE_B_BYTES);
        tma_load_2d(base + s * STAGE_BYTES, &map_a, (kb0 + kb) * BK, m0, full(s));
        tma_load_2d(base + s * STAGE_BYTES + TILE_A_BYTES, map_b, (kb0 + kb) * BK, n0, full(s));
        if (FUSE) tma_load_2d(base + s * STAGE_BYTES + TILE_A_BYTES + TILE_B_BYTES, &map_b1, (kb0 + kb) * BK, n0, full(s));
        issued = kb + 1;
      }
      // after an abort the copies already issued must land before the CTA can exit
      if (*abort_flag) {
        for (int kb = (issued > STAGES ? issued - STAGES : 0); kb < issued; ++kb) {
          const unsigned long long t0 = gtime();
          while (!bar_try(full(kb % STAGES), (kb / STAGES) & 1)) {
            if (gtime() - t0 > (budget_ns > 2000000ull ? budget_ns : 2000000ull)) break;   // landing takes microseconds
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {                       // ---- MMA issuer
      bool ok = true;
      for (int kb = 0; kb < kblocks && ok; ++kb) {
        const int s = kb % STAGES;
        ok = bar_wait(full(s), (kb / STAGES) & 1, abort_flag, status, budget_ns);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint64_t da = smem_desc_sw128(base + s * STAGE_BYTES);
        const uint64_t db = smem_desc_sw128(base + s * STAGE_BYTES + TILE_A_BYTES);
#pragma unroll
        for (int j = 0; j < BK / 16; ++j) {  // 16 halves = 32 bytes = 2 descriptor address units per K step
          // FUSE: the up tile follows the gate tile in shared memory (BN more rows of the same 8-row-group layout),
          // so one MMA of N = 2 BN covers both and leaves gate in columns [0, BN), up in [BN, 2 BN)
          mma_f16_ss(tmem_base, da + 2u * j, db + 2u * j, (kb > 0 || j > 0) ? 1u : 0u, idesc_for(SB));
        }
        mma_commit(empty(s));               // the stage is free once these MMAs have read it
      }
      if (ok) mma_commit(acc_full);         // accumulator complete
    }
  } else {                                 // ---- epilogue: warps 2..5 own TMEM lanes 32 * (warp % 4) ..
    const int quarter = warp & 3;
    // warp-uniform outcome: the TMEM loads below are warp-wide instructions
    const bool ok = __all_sync(0xffffffffu, bar_wait(acc_full, 0, abort_flag, status, budget_ns));
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (ok && FUSE) {
      const int row = m0 + quarter * 32 + lane;
      __half *arow = reinterpret_cast<__half *>(C) + static_cast<size_t>(row) * N + n0;
#pragma unroll 1
      for (int c = 0; c < BN / 16; ++c) {     // 16 columns of the gate tile and the same 16 of the up tile per pass
        uint32_t g[16], u[16];
        const uint32_t tg = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(c * 16);
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
            "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
            : "=r"(g[0]), "=r"(g[1]), "=r"(g[2]), "=r"(g[3]), "=r"(g[4]), "=r"(g[5]), "=r"(g[6]), "=r"(g[7]), "=r"(g[8]),
              "=r"(g[9]), "=r"(g[10]), "=r"(g[11]), "=r"(g[12]), "=r"(g[13]), "=r"(g[14]), "=r"(g[15])
            : "r"(tg)
            : "memory");
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
            "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
            : "=r"(u[0]), "=r"(u[1]), "=r"(u[2]), "=r"(u[3]), "=r"(u[4]), "=r"(u[5]), "=r"(u[6]), "=r"(u[7]), "=r"(u[8]),
              "=r"(u[9]), "=r"(u[10]), "=r"(u[11]), "=r"(u[12]), "=r"(u[13]), "=r"(u[14]), "=r"(u[15])
            : "r"(tg + BN)
            : "memory");
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (row < M) {
          uint32_t packed[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float g0 = __uint_as_float(g[2 * i]), g1 = __uint_as_float(g[2 * i + 1]);
            const __half2 h = __floats2half2_rn(g0 / (1.0f + expf(-g0)) * __uint_as_float(u[2 * i]),
                                                g1 / (1.0f + expf(-g1)) * __uint_as_float(u[2 * i + 1]));
            packed[i] = *reinterpret_cast<const uint32_t *>(&h);
          }
          *reinterpret_cast<uint4 *>(arow + c * 16) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
          *reinterpret_cast<uint4 *>(arow + c * 16 + 8) = make_uint4(packed[4], packed[5], packed[6], packed[7]);
        }
      }
    } else if (ok) {
      const int row = m0 + quarter * 32 + lane;
      float *crow = C + static_cast<size_t>(blockIdx.z) * groups.split_stride + static_cast<size_t>(row) * N + n0;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(c * 32);
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
            "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
            "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
              "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
              "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
              "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
            : "r"(taddr)
            : "memory");
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (row < M) {
#pragma unroll
          for (int i = 0; i < 32; i += 4)
            *reinterpret_cast<float4 *>(crow + c * 32 + i) =
                make_float4(__uint_as_float(r[i]), __uint_as_float(r[i + 1]), __uint_as_float(r[i + 2]),
                            __uint_as_float(r[i + 3]));
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

}  // namespace qmk_gemm
#endif  // QMK_GEMM_TCGEN05_CUH_
