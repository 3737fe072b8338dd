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
//
// Packed weights (template parameter WQ): B may stay in its packed form in global memory - WQ 1: FP8-E4M3 rows
// with an fp32 row scale in a 16-byte trailer; WQ 2: NVFP4 rows (two e2m1 values per byte, one e4m3 scale per 16
// values behind them, the fp32 tensor scale in the trailer).  The producer then brings the PACKED K block into a raw
// area of the stage (half or a quarter of the fp16 bytes cross HBM and L2), warps 2-5 - idle until the epilogue
// otherwise - expand it to the fp16, 128-byte-swizzled tile the MMA descriptors expect (e4m3 and e2m1 x block scale
// are exact in fp16), fence the writes towards the async proxy and arrive on the stage's `full` barrier; the fp32
// row / tensor scale multiplies the accumulator in the epilogue.  The activations stay fp16 and the accumulation fp32,
// so the products are those of the dequantised matrix: tcgen05's own narrow kinds (f8f6f4, mxf4nvf4) would need the
// ACTIVATIONS in 8 or 4 bits as well, which a greedy decoder checked token by token cannot afford.
#ifndef QMK_GEMM_TCGEN05_CUH_
#define QMK_GEMM_TCGEN05_CUH_

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace qmk_gemm {

constexpr int BM = 128, BK = 64;                 // BK * 2 bytes = one 128-byte swizzle row; the N tile (128 or 64) is a template parameter
// Ring depth per N-tile variant: as many stages as fit in ~192 KB (a skinny M = 128 problem is bound by the
// latency of its K loop, so the whole K extent of a 1024-wide matrix is in flight at once).
constexpr int stages_for(int bn, int wq = 0) {
  return wq ? (bn == 32 ? 8 : bn == 64 ? 6 : bn == 128 ? 4 : 2) : (bn == 32 ? 10 : bn == 64 ? 8 : bn == 128 ? 6 : 4);
}
constexpr int MAX_GROUPS = 3;   // matrices sharing one A operand that one launch can multiply (q/k/v, gate/up)
constexpr int THREADS = 192;                     // fp16 weights: producer warp, MMA warp, four epilogue warps
constexpr int THREADS_PACKED = 320;              // packed weights: four more warps that only expand K blocks
constexpr int threads_for(int wq) { return wq ? THREADS_PACKED : THREADS; }
constexpr uint32_t TILE_A_BYTES = BM * BK * 2;   // 16 KB
// Packed K block of one B row: 64 e4m3 bytes, or 32 bytes of e2m1 pairs
constexpr uint32_t raw_row_bytes(int wq) { return wq == 1 ? 64u : wq == 2 ? 32u : 0u; }
constexpr uint32_t stage_bytes_for(int bn, int wq = 0) {
  return TILE_A_BYTES + static_cast<uint32_t>(bn) * BK * 2 + static_cast<uint32_t>(bn) * raw_row_bytes(wq);
}
// Per-row scales kept in shared memory for the whole tile: the fp32 row / tensor scale, and for NVFP4 the block
// scales of the CTA's K range (one byte per 16 values; K <= 3072 -> 192 bytes, rows 196 bytes apart against bank
// conflicts).
constexpr int MAX_K_PACKED = 3072;
constexpr uint32_t BS_PITCH = MAX_K_PACKED / 16 + 4;
constexpr uint32_t scale_bytes_for(int bn, int wq) {
  return wq == 0 ? 0u : static_cast<uint32_t>(bn) * 4u + (wq == 2 ? static_cast<uint32_t>(bn) * BS_PITCH : 0u);
}
constexpr int MAX_STAGES = 16;
constexpr uint32_t BARRIER_BYTES = 640;   // full[16], empty[16], acc_full, raw_full[16], a_full[16], TMEM address, abort flag
constexpr size_t smem_bytes_for(int bn, int wq = 0) {
  return 1024 /* alignment slack */ + static_cast<size_t>(stages_for(bn, wq)) * stage_bytes_for(bn, wq) + BARRIER_BYTES +
         scale_bytes_for(bn, wq);
}
// Ring depth of a launch: the compile-time depth above (one CTA per SM, ~200 KB: a skinny problem wants its whole K
// extent in flight), or as many stages as fit `budget_bytes` - with about 96 KB two CTAs share an SM and the epilogue
// of one (TMEM -> registers -> global) runs under the main loop of the other, which is what a multi-wave prefill GEMM
// wants (measured on 2048 prompt tokens: 7.9 -> 6.8 ms per pass).
struct RingGeometry { int stages; uint32_t ring_bytes; size_t smem_bytes; };
inline RingGeometry ring_geometry(int sb, int wq, uint32_t budget_bytes) {
  RingGeometry g;
  g.stages = stages_for(sb, wq);
  if (budget_bytes > 0) {
    const int fit = static_cast<int>(budget_bytes / stage_bytes_for(sb, wq));
    if (fit < g.stages) g.stages = fit < 2 ? 2 : fit;
  }
  g.ring_bytes = static_cast<uint32_t>(g.stages) * stage_bytes_for(sb, wq);
  g.smem_bytes = 1024 + static_cast<size_t>(g.ring_bytes) + BARRIER_BYTES + scale_bytes_for(sb, wq);
  return g;
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
// Programmatic dependent launch (see prefill_kernels.cuh): no-ops unless the launch carries the attribute.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

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
  // Packed weights (WQ != 0): base of every group's packed matrix, bytes between rows, offset of the block scales
  // (NVFP4) and of the fp32 scale (the trailer) inside a row.
  const unsigned char *braw[MAX_GROUPS];
  uint32_t raw_pitch, raw_bs_off, raw_scale_off;
  // Ring geometry (ring_geometry()): stages and bytes from the ring's start to the barriers.
  int stages;
  uint32_t ring_bytes;
  // Greedy pick fused into the epilogue (single group, no split-K; null = off): instead of storing its part of the
  // row, every thread keeps the largest value and its column (lowest column on ties) and writes one pair per row
  // and N tile - amax_val / amax_idx [row][gridDim.x]; a small kernel then reduces gridDim.x pairs per row instead of
  // reading the whole row of logits, which is never written.
  float *amax_val;
  int *amax_idx;
  // Plain epilogue, no split-K: 1 = the C matrices are fp16 [M x N_g] (the pointers are reinterpreted), half the
  // store burst of a launch whose CTAs all reach their epilogue together.
  int out_f16;
};

// Eight e2m1 values of one 32-bit word (element 2 i in the low nibble of byte i) -> four half2 registers.
__device__ __forceinline__ void e2m1x8_to_half2x4(uint32_t word, uint32_t (&out)[4]) {
  asm("{\n\t"
      ".reg .b8 b0, b1, b2, b3;\n\t"
      "mov.b32 {b0, b1, b2, b3}, %4;\n\t"
      "cvt.rn.f16x2.e2m1x2 %0, b0;\n\t"
      "cvt.rn.f16x2.e2m1x2 %1, b1;\n\t"
      "cvt.rn.f16x2.e2m1x2 %2, b2;\n\t"
      "cvt.rn.f16x2.e2m1x2 %3, b3;\n\t"
      "}"
      : "=r"(out[0]), "=r"(out[1]), "=r"(out[2]), "=r"(out[3])
      : "r"(word));
}
__device__ __forceinline__ uint32_t e4m3x2_to_half2_bits(uint32_t two_bytes) {
  const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(two_bytes & 0xFFFFu), __NV_E4M3);
  return static_cast<uint32_t>(h.x) | (static_cast<uint32_t>(h.y) << 16);
}

// FUSE (BN = 32 or 64): B0 is the gate matrix and B1 the up matrix of a SwiGLU MLP; the CTA keeps two accumulators
// (gate tile in TMEM columns [0, BN), up tile in [BN, 2 BN)) and its epilogue writes fp16 silu(gate) * up to
// groups.C[0] (reinterpreted as __half [M x N]) instead of two fp32 matrices.
template <int BN, bool FUSE = false, int WQ = 0>
__global__ void __launch_bounds__(WQ ? THREADS_PACKED : THREADS, 1)
gemm_f16_tn_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b0,
                   const __grid_constant__ CUtensorMap map_b1, const __grid_constant__ CUtensorMap map_b2,
                   const Groups groups, int M, int K, unsigned int *status, unsigned long long budget_ns,
                   int selftest_no_loads) {
  static_assert(BN == 32 || BN == 64 || BN == 128 || BN == 256, "N tiles of 32, 64, 128 or 256 columns");
  static_assert(!FUSE || BN <= 128, "the fused SwiGLU epilogue keeps two accumulators of at most 128 columns (one MMA of N = 256)");
  static_assert(WQ == 0 || (FUSE ? 2 * BN : BN) <= 128, "packed weights: at most 128 B rows per stage (scales live in shared memory)");
  constexpr int SB = FUSE ? 2 * BN : BN;          // B rows held per stage / accumulator columns
  constexpr uint32_t RAW_ROW = raw_row_bytes(WQ);
  const int STAGES = groups.stages;
  constexpr uint32_t STAGE_BYTES = stage_bytes_for(SB, WQ);
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
  const uint32_t bars = base + groups.ring_bytes;               // full[16], empty[16], acc_full, raw_full[16], a_full[16], then scratch
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(aligned + groups.ring_bytes + 8 * (4 * MAX_STAGES + 1));
  float *s_rowscale = reinterpret_cast<float *>(aligned + groups.ring_bytes + BARRIER_BYTES);   // [SB] (WQ != 0)
  unsigned char *s_bs = reinterpret_cast<unsigned char *>(s_rowscale + SB);                // [SB][BS_PITCH] (WQ == 2)
  static_assert(8 * (4 * MAX_STAGES + 1) + 8 <= BARRIER_BYTES, "barriers and scratch fit the bytes reserved behind the ring");
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = tile * BN, m0 = blockIdx.y * BM;
  const int kblocks = groups.kblocks_per_split > 0 ? groups.kblocks_per_split : K / BK;
  const int kb0 = groups.kblocks_per_split > 0 ? static_cast<int>(blockIdx.z) * groups.kblocks_per_split : 0;
  constexpr uint32_t TILE_B_BYTES = BN * BK * 2;
  constexpr uint32_t TMEM_COLS = SB;             // fp32 accumulator(s): 128 lanes x SB columns (a power of two >= 32)
  auto full = [&](int s) { return bars + 8u * s; };
  auto empty = [&](int s) { return bars + 8u * (MAX_STAGES + s); };
  const uint32_t acc_full = bars + 8u * (2 * MAX_STAGES);
  auto raw_full = [&](int s) { return bars + 8u * (2 * MAX_STAGES + 1 + s); };   // packed K block landed
  auto a_full = [&](int s) { return bars + 8u * (3 * MAX_STAGES + 1 + s); };     // packed weights: the A tile landed
  // What the producer's copies of one stage signal.  fp16 weights: A and B complete `full` together.  Packed weights:
  // the packed K block completes `raw_full`, on which the expanding warps wait before they arrive on `full`
  // themselves (one warp per stage), and the A tile completes `a_full` - on its own barrier, because B does not
  // depend on the preceding kernel: the first ring fill of weights is requested AND expanded before that kernel has
  // finished, and when A finally arrives the MMAs start at once.
  auto b_landed = [&](int s) { return WQ ? raw_full(s) : full(s); };
  auto a_landed = [&](int s) { return WQ ? a_full(s) : full(s); };
  constexpr uint32_t TILE_RAW_BYTES = BN * RAW_ROW;
  const uint32_t a_tx = groups.a_box_bytes ? groups.a_box_bytes : TILE_A_BYTES;
  const uint32_t b_tx = (FUSE ? 2u : 1u) * (WQ ? TILE_RAW_BYTES : TILE_B_BYTES);
  constexpr uint32_t TILE_A = TILE_A_BYTES;   // the B tile follows the A tile in a stage
  const int kcol = WQ ? static_cast<int>(RAW_ROW) : BK;          // B-map columns (bytes for packed rows) per K block
  const uint32_t b_dst = WQ ? TILE_A + (FUSE ? 2u : 1u) * TILE_B_BYTES : TILE_A;   // where the B copies land in a stage
  const uint32_t b_dst_step = WQ ? TILE_RAW_BYTES : TILE_B_BYTES;
  // the first fill of the ring needs no free-slot wait: thread 0 issues it before the CTA-wide barrier below, so
  // that the first TMA round trip overlaps the TMEM allocation
  const int prologue = selftest_no_loads ? 0 : (kblocks < STAGES ? kblocks : STAGES);
  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_a)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map_b)) : "memory");
    if (FUSE) asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_b1)) : "memory");
    for (int s = 0; s < STAGES; ++s) {
      bar_init(full(s), WQ ? 2 : 1);      // packed weights: the two warps that expand a stage arrive
      bar_init(empty(s), 1);
      if (WQ) { bar_init(raw_full(s), 1); bar_init(a_full(s), 1); }
    }
    bar_init(acc_full, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    // B is a weight matrix: its first tiles are requested before the wait for the preceding kernel (whose output is
    // A, requested behind the wait below), so the weight stream of this GEMM overlaps that kernel's tail
    for (int kb = 0; kb < prologue; ++kb) {
      bar_expect_tx(b_landed(kb), WQ ? b_tx : a_tx + b_tx);
      tma_load_2d(base + kb * STAGE_BYTES + b_dst, map_b, (kb0 + kb) * kcol, n0, b_landed(kb));
      if (FUSE) tma_load_2d(base + kb * STAGE_BYTES + b_dst + b_dst_step, &map_b1, (kb0 + kb) * kcol, n0, b_landed(kb));
    }
  }
  if (WQ != 0 && warp >= 2 && warp < 6) {
    // scales of this CTA's B rows into shared memory while the first copies are in flight (the CTA-wide barrier below
    // publishes them): the fp32 row / tensor scale of every row and, for NVFP4, the block scales of the K range
    const int ct = static_cast<int>(threadIdx.x) - 64;          // 0..127
    // (selected with conditionals: a run-time index into the kernel parameter would copy the struct to local memory)
    const unsigned char *braw_lo = FUSE ? groups.braw[0] : grp == 0 ? groups.braw[0] : grp == 1 ? groups.braw[1] : groups.braw[2];
    const unsigned char *braw_hi = FUSE ? groups.braw[1] : braw_lo;
    for (int r = ct; r < SB; r += 128) {
      const unsigned char *row = (FUSE && r >= BN ? braw_hi : braw_lo) +
                                 static_cast<size_t>(n0 + (FUSE && r >= BN ? r - BN : r)) * groups.raw_pitch;
      s_rowscale[r] = *reinterpret_cast<const float *>(row + groups.raw_scale_off);
    }
    if (WQ == 2) {                                              // one word (four block scales) per row and K block
      for (int i = ct; i < SB * kblocks; i += 128) {
        const int r = i / kblocks, w = i - r * kblocks;
        const unsigned char *row = (FUSE && r >= BN ? braw_hi : braw_lo) +
                                   static_cast<size_t>(n0 + (FUSE && r >= BN ? r - BN : r)) * groups.raw_pitch;
        *reinterpret_cast<uint32_t *>(s_bs + r * BS_PITCH + 4 * w) =
            *reinterpret_cast<const uint32_t *>(row + groups.raw_bs_off + 4 * (kb0 + w));
      }
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
      pdl_wait();                          // A is the preceding kernel's output
      // Only now may the NEXT kernel of the chain be scheduled (to set itself up and request its weight tiles behind
      // this one): a kernel that let its dependents go before its own predecessor had completed put three kernels in
      // flight at once, and the chunked prefill then produced run-to-run different cache rows - at most two overlap.
      pdl_trigger();
      for (int kb = 0; kb < prologue; ++kb) {
        if (WQ) bar_expect_tx(a_full(kb), a_tx);
        tma_load_2d(base + kb * STAGE_BYTES, &map_a, (kb0 + kb) * BK, m0, a_landed(kb));
      }
      int issued = prologue;
      // self test of the bounded waits: the loads are never issued, so the MMA thread's first wait runs out
      for (int kb = prologue; kb < (selftest_no_loads ? 0 : kblocks); ++kb) {
        const int s = kb % STAGES;
        if (kb >= STAGES && !bar_wait(empty(s), ((kb / STAGES) - 1) & 1, abort_flag, status, budget_ns)) break;
        if (*abort_flag) break;
        bar_expect_tx(b_landed(s), WQ ? b_tx : a_tx + b_tx);
        if (WQ) bar_expect_tx(a_full(s), a_tx);
        tma_load_2d(base + s * STAGE_BYTES, &map_a, (kb0 + kb) * BK, m0, a_landed(s));
        tma_load_2d(base + s * STAGE_BYTES + b_dst, map_b, (kb0 + kb) * kcol, n0, b_landed(s));
        if (FUSE) tma_load_2d(base + s * STAGE_BYTES + b_dst + b_dst_step, &map_b1, (kb0 + kb) * kcol, n0, b_landed(s));
        issued = kb + 1;
      }
      // after an abort the copies already issued must land before the CTA can exit
      if (*abort_flag) {
        for (int kb = (issued > STAGES ? issued - STAGES : 0); kb < issued; ++kb) {
          const unsigned long long t0 = gtime();
          while (!(bar_try(b_landed(kb % STAGES), (kb / STAGES) & 1) && bar_try(a_landed(kb % STAGES), (kb / STAGES) & 1))) {
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
        ok = bar_wait(full(s), (kb / STAGES) & 1, abort_flag, status, budget_ns) &&
             (!WQ || bar_wait(a_full(s), (kb / STAGES) & 1, abort_flag, status, budget_ns));
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint64_t da = smem_desc_sw128(base + s * STAGE_BYTES);
        const uint64_t db = smem_desc_sw128(base + s * STAGE_BYTES + TILE_A);
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
  } else {                                 // ---- warps 2..5: epilogue, each owns TMEM lanes 32 * (warp % 4) ..; packed
                                           //      weights: first they and warps 6..9 expand the K blocks
    const int quarter = warp & 3;
    if (WQ) {
      // Eight warps expand: stage s belongs to the two warps whose (index mod 4) is s mod 4, each takes every other
      // 16-value chunk of it and arrives on `full` (count 2).  The chain wait -> load -> convert -> store -> fence ->
      // arrive is latency, so several chains run side by side; and a warp owns STAGES, not K blocks: it then meets
      // the uses of a stage's barrier in order - a parity wait cannot tell use u from use u - 2, so a warp that
      // reached use u of a stage before anyone had waited for use u - 1 would run ahead on stale data.
      const int cw = warp - 2, part = cw >> 2;
      bool live = !selftest_no_loads;
      for (int kb = 0; kb < kblocks && live; ++kb) {
        const int s = kb % STAGES;
        if ((s & 3) != (cw & 3)) continue;
        live = __all_sync(0xffffffffu, bar_wait(raw_full(s), (kb / STAGES) & 1, abort_flag, status, budget_ns));
        if (!live) break;
        const uint32_t btile = base + s * STAGE_BYTES + TILE_A;
        const uint32_t rawt = base + s * STAGE_BYTES + b_dst;
        // one 16-value chunk per lane and pass: chunk i = row * 4 + quarter of the 64-wide K block; the packed
        // rows are dense, so consecutive lanes read consecutive bytes
#pragma unroll 4
        for (int i = lane + 32 * part; i < SB * 4; i += 64) {
          const int r = i >> 2, c = i & 3;
          uint32_t h[8];
          if (WQ == 1) {
            uint32_t v0, v1, v2, v3;
            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v0), "=r"(v1), "=r"(v2), "=r"(v3) : "r"(rawt + i * 16));
            h[0] = e4m3x2_to_half2_bits(v0); h[1] = e4m3x2_to_half2_bits(v0 >> 16);
            h[2] = e4m3x2_to_half2_bits(v1); h[3] = e4m3x2_to_half2_bits(v1 >> 16);
            h[4] = e4m3x2_to_half2_bits(v2); h[5] = e4m3x2_to_half2_bits(v2 >> 16);
            h[6] = e4m3x2_to_half2_bits(v3); h[7] = e4m3x2_to_half2_bits(v3 >> 16);
          } else {
            uint32_t v0, v1;
            asm volatile("ld.shared.v2.b32 {%0, %1}, [%2];" : "=r"(v0), "=r"(v1) : "r"(rawt + i * 8));
            const uint32_t sb2 = e4m3x2_to_half2_bits(s_bs[r * BS_PITCH + 4 * kb + c]);   // low half = the block's scale
            const __half2 sc = __half2half2(__ushort_as_half(static_cast<unsigned short>(sb2 & 0xFFFFu)));
            uint32_t lo[4], hi[4];
            e2m1x8_to_half2x4(v0, lo);
            e2m1x8_to_half2x4(v1, hi);
#pragma unroll
            for (int j = 0; j < 4; ++j) {       // e2m1 x e4m3 has six significant bits: exact in fp16
              const __half2 a = __hmul2(*reinterpret_cast<const __half2 *>(&lo[j]), sc);
              const __half2 b = __hmul2(*reinterpret_cast<const __half2 *>(&hi[j]), sc);
              h[j] = *reinterpret_cast<const uint32_t *>(&a);
              h[4 + j] = *reinterpret_cast<const uint32_t *>(&b);
            }
          }
          // 128-byte swizzle of the MMA tile: 16-byte segment index XOR (row mod 8)
          const uint32_t rowaddr = btile + static_cast<uint32_t>(r) * 128u;
          const uint32_t x = static_cast<uint32_t>(r & 7);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(rowaddr + (((2u * c) ^ x) << 4)), "r"(h[0]), "r"(h[1]), "r"(h[2]), "r"(h[3]) : "memory");
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(rowaddr + (((2u * c + 1u) ^ x) << 4)), "r"(h[4]), "r"(h[5]), "r"(h[6]), "r"(h[7]) : "memory");
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes before the MMA's async-proxy reads
        __syncwarp();
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(full(s)) : "memory");
      }
    }
    if (warp < 6) {
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
            float g0 = __uint_as_float(g[2 * i]), g1 = __uint_as_float(g[2 * i + 1]);
            float u0 = __uint_as_float(u[2 * i]), u1 = __uint_as_float(u[2 * i + 1]);
            if (WQ) {
              g0 *= s_rowscale[c * 16 + 2 * i]; g1 *= s_rowscale[c * 16 + 2 * i + 1];
              u0 *= s_rowscale[BN + c * 16 + 2 * i]; u1 *= s_rowscale[BN + c * 16 + 2 * i + 1];
            }
            // (hardware exp2 and reciprocal: a few ulp, far inside the fp16 rounding of the result; the exact forms
            // cost about 25 instructions per value and made this epilogue as long as a third of the K loop)
            const __half2 h = __floats2half2_rn(__fdividef(g0, 1.0f + __expf(-g0)) * u0, __fdividef(g1, 1.0f + __expf(-g1)) * u1);
            packed[i] = *reinterpret_cast<const uint32_t *>(&h);
          }
          *reinterpret_cast<uint4 *>(arow + c * 16) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
          *reinterpret_cast<uint4 *>(arow + c * 16 + 8) = make_uint4(packed[4], packed[5], packed[6], packed[7]);
        }
      }
    } else if (ok) {
      const int row = m0 + quarter * 32 + lane;
      float *crow = C + static_cast<size_t>(blockIdx.z) * groups.split_stride + static_cast<size_t>(row) * N + n0;
      __half *hrow = reinterpret_cast<__half *>(C) + static_cast<size_t>(row) * N + n0;   // (out_f16)
      const bool pick = groups.amax_val != nullptr;
      const bool f16 = groups.out_f16 != 0;
      float best = -INFINITY;
      int best_col = 0x7fffffff;
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
        if (row < M && f16) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint32_t packed[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              float a = __uint_as_float(r[i + 2 * k]), b = __uint_as_float(r[i + 2 * k + 1]);
              if (WQ) { a *= s_rowscale[c * 32 + i + 2 * k]; b *= s_rowscale[c * 32 + i + 2 * k + 1]; }
              const __half2 h = __floats2half2_rn(a, b);
              packed[k] = *reinterpret_cast<const uint32_t *>(&h);
            }
            *reinterpret_cast<uint4 *>(hrow + c * 32 + i) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
          }
        } else if (row < M) {
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            float4 o = make_float4(__uint_as_float(r[i]), __uint_as_float(r[i + 1]), __uint_as_float(r[i + 2]),
                                   __uint_as_float(r[i + 3]));
            if (WQ) {
              const float *sc = s_rowscale + c * 32 + i;
              o.x *= sc[0]; o.y *= sc[1]; o.z *= sc[2]; o.w *= sc[3];
            }
            if (pick) {   // increasing columns: strict > keeps the lowest index among equals
              const int col = n0 + c * 32 + i;
              if (o.x > best) { best = o.x; best_col = col; }
              if (o.y > best) { best = o.y; best_col = col + 1; }
              if (o.z > best) { best = o.z; best_col = col + 2; }
              if (o.w > best) { best = o.w; best_col = col + 3; }
            } else {
              *reinterpret_cast<float4 *>(crow + c * 32 + i) = o;
            }
          }
        }
      }
      if (pick && row < M) {
        groups.amax_val[static_cast<size_t>(row) * gridDim.x + blockIdx.x] = best;
        groups.amax_idx[static_cast<size_t>(row) * gridDim.x + blockIdx.x] = best_col;
      }
    }
    }   // warps 2..5
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
