// Batched decode attention on mma.sync (see the comment at the kernel).
#ifndef QMK_DECODE_ATTENTION_MMA_CUH_
#define QMK_DECODE_ATTENTION_MMA_CUH_

#include <cuda.h>
#include "prefill_kernels.cuh"

namespace qmk_pf {

// Decode-step attention for a batch of sequences on the tensor cores, with the per-head preparation fused in.
// grid = (B, 8 kv heads, splits), block = 288 = 8 consumer warps + 1 producer warp; splits, new row, cache write and
// the merge of split sequences as in decode_attention_ring (prefill_kernels.cuh), which this kernel replaces: there
// every lane scored one key with 128 FMAs and the kernel ran at half the DRAM bandwidth because it was bound by
// instruction issue.  Here the old rows arrive as chunks of 16 K rows + 16 V rows - four tiled TMA boxes of 16 rows x
// 128 bytes with the 128-byte swizzle, through per-sequence tensor maps kept in device memory - and a warp handles
// a chunk with 16 mma.sync.m16n8k16: scores = K[16 x 128] . q[128 x 4] (columns: head 0 hi / lo, head 1 hi / lo of
// the fp32 query split into two fp16 numbers), online softmax on the accumulator fragments (log2 domain), then
// out[128 x 4] += V^T[128 x 16] . p[16 x 4] with V read through ldmatrix.trans and p split like q - about 75
// instructions per 16 rows instead of about 400.  Waits are bounded: on a time-out the CTA sets *status = 4 and
// leaves after its copies have landed.
constexpr int DAM_WARPS = 8, DAM_SLOTS = 12, DAM_ROWS = 16;
constexpr int DAM_BOX = DAM_ROWS * 128;                // one box: 16 rows x 64 dims
constexpr int DAM_SLOT_BYTES = 4 * DAM_BOX;            // 8 KB: K dims 0..63, K dims 64..127, V dims 0..63, V dims 64..127
constexpr int DAM_SMEM_BYTES = DAM_SLOTS * DAM_SLOT_BYTES + 2 * DAM_SLOTS * 8 + 16;   // ring, barriers, abort flag + issued counter
constexpr int DAM_QPITCH = 2 * D + 16;                 // bytes between the four query-operand rows (conflict-free ldmatrix)
constexpr float DAM_LO_SCALE = 2048.0f, DAM_LO_INV = 1.0f / 2048.0f;

__device__ __forceinline__ void dam_ldsm_x4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr) : "memory");
}
__device__ __forceinline__ void dam_ldsm_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr) : "memory");
}
// fp32 -> fp16 operand half: the value rounded to fp16 (lo = false) or its scaled remainder (lo = true)
__device__ __forceinline__ __half dam_split(float x, bool lo) {
  const __half h = __float2half_rn(x);
  return lo ? __float2half_rn((x - __half2float(h)) * DAM_LO_SCALE) : h;
}
__device__ __forceinline__ uint32_t dam_pack(__half a, __half b) {
  return static_cast<uint32_t>(__half_as_ushort(a)) | (static_cast<uint32_t>(__half_as_ushort(b)) << 16);
}
__global__ void __launch_bounds__((DAM_WARPS + 1) * 32) decode_attention_mma(
    const float *q, const float *k, const float *v, const __half *q_norm, const __half *k_norm, const float *rope,
    const __half *cos_table, const __half *sin_table, __half *const *k_ptrs, __half *const *v_ptrs, size_t layer_off,
    const int *positions, __half *out, int max_seq_len, float scale, unsigned int *status, unsigned long long budget_ns,
    float *split_part, unsigned int *split_count, const CUtensorMap *kv_maps, int layer_row0) {
  extern __shared__ __align__(128) unsigned char dam_smem[];
  __shared__ __align__(16) float sq[2 * D];
  __shared__ __align__(16) unsigned char s_qf[4 * DAM_QPITCH];   // fp16 query operand: q0 hi, q0 lo, q1 hi, q1 lo
  __shared__ float sknew[D], svnew[D], snew_score[2];
  __shared__ float sm[DAM_WARPS][2], sl[DAM_WARPS][2];
  __shared__ __align__(16) float sacc[DAM_WARPS][2][D];
  uint64_t *full = reinterpret_cast<uint64_t *>(dam_smem + DAM_SLOTS * DAM_SLOT_BYTES);
  uint64_t *empty = full + DAM_SLOTS;
  volatile int *abort_flag = reinterpret_cast<volatile int *>(empty + DAM_SLOTS);
  // Chunks issued so far.  A parity wait can only tell two consecutive uses of a slot apart, and a warp's first
  // chunk may already be a second use (chunk 6 or 7 in slot 0 or 1): consumers wait for "issued" first.
  volatile int *issued_ctr = abort_flag + 1;
  const int b = blockIdx.x, g = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pos = positions[b];
  const int nchunks_all = (pos + DAM_ROWS - 1) / DAM_ROWS;
  // gridDim.z CTAs share a (sequence, kv head): CTA z streams chunks [c_begin, c_end) of the old rows, the last one
  // also folds in the new row; see the merge at the end.
  const int nsplit = gridDim.z, split = blockIdx.z;
  const int c_begin = nchunks_all * split / nsplit, c_end = nchunks_all * (split + 1) / nsplit;
  const int nchunks = c_end - c_begin;        // ring indices below are local: chunk c_begin + i is ring chunk i
  const bool owner = split == nsplit - 1;
  __half *kbase = k_ptrs[b] + layer_off + static_cast<size_t>(g) * max_seq_len * D;
  __half *vbase = v_ptrs[b] + layer_off + static_cast<size_t>(g) * max_seq_len * D;
  auto s32 = [](const void *p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); };
  auto try_wait = [&](uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(s32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
  };
  auto wait = [&](uint64_t *bar, uint32_t parity) {   // bounded
    if (try_wait(bar, parity)) return true;
    unsigned long long t0;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    for (uint32_t it = 1;; ++it) {
      if (try_wait(bar, parity)) return true;
      if ((it & 63u) == 0u) {
        if (*abort_flag) return false;
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        if (t - t0 > budget_ns) { *abort_flag = 1; atomicCAS(status, 0u, 4u); return false; }
      }
    }
  };
  if (threadIdx.x == 0) {
    for (int i = 0; i < DAM_SLOTS; ++i) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s32(full + i)), "r"(1) : "memory");
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s32(empty + i)), "r"(1) : "memory");
    }
    *abort_flag = 0;
    *issued_ctr = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  // The producer streams cache rows written by EARLIER steps, so it starts at once; everyone else reads what the
  // q/k/v GEMM launched just before wrote, and writes (cache row, output, split partials) only after it completed.
  if (warp != DAM_WARPS) {
    pdl_wait();
    if (threadIdx.x == 0) pdl_trigger();   // (after the wait: at most two kernels of a chain overlap)
  }
  if (warp == DAM_WARPS) {            // ---- producer: old rows [0, pos) in chunks of 16
    if (lane == 0) {
      const CUtensorMap *kmap = kv_maps + 2 * b, *vmap = kmap + 1;
      // the maps were written by the host into device memory before this launch
      asm volatile("fence.proxy.tensormap::generic.acquire.sys [%0], 128;" ::"l"(reinterpret_cast<uint64_t>(kmap)) : "memory");
      asm volatile("fence.proxy.tensormap::generic.acquire.sys [%0], 128;" ::"l"(reinterpret_cast<uint64_t>(vmap)) : "memory");
      const int row0 = layer_row0 + g * max_seq_len;   // this head's first row in the sequence's [layer][head][pos] cache
      int issued = 0;
      for (int c = 0; c < nchunks; ++c) {
        const int slot = c % DAM_SLOTS;
        if (c >= DAM_SLOTS && !wait(empty + slot, ((c / DAM_SLOTS) - 1) & 1)) break;
        const int row = row0 + (c_begin + c) * DAM_ROWS;
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(s32(full + slot)), "r"(DAM_SLOT_BYTES) : "memory");
        const uint32_t dst = s32(dam_smem + slot * DAM_SLOT_BYTES);
#pragma unroll
        for (int sub = 0; sub < 4; ++sub)
          asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                       ::"r"(dst + sub * DAM_BOX), "l"(sub < 2 ? kmap : vmap), "r"((sub & 1) * 64), "r"(row), "r"(s32(full + slot))
                       : "memory");
        issued = c + 1;
        __threadfence_block();
        *issued_ctr = issued;
      }
      if (*abort_flag)   // copies already issued must land before the CTA may exit
        for (int c = (issued > DAM_SLOTS ? issued - DAM_SLOTS : 0); c < issued; ++c) {
          unsigned long long t0, t;
          asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
          while (!try_wait(full + c % DAM_SLOTS, (c / DAM_SLOTS) & 1)) {
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
            if (t - t0 > (budget_ns > 2000000ull ? budget_ns : 2000000ull)) break;
          }
        }
    }
  } else if (warp < 4) {              // ---- head preparation
    const float *src = warp < 2 ? q + static_cast<size_t>(b) * QS + (2 * g + warp) * D
                                : (warp == 2 ? k : v) + static_cast<size_t>(b) * KVS + g * D;
    float x[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) x[i] = src[lane + 32 * i];
    if (warp < 3) {
      const __half *nw = warp < 2 ? q_norm : k_norm;
      float ss = x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3];
      ss = warp_sum(ss);
      const float rstd = 1.0f / sqrtf(ss * (1.0f / D) + RMS_EPS);
#pragma unroll
      for (int i = 0; i < 4; ++i) x[i] = x[i] * rstd * __half2float(nw[lane + 32 * i]);
      float c0, s0, c1, s1;
      if (rope) {
        const float *r = rope + static_cast<size_t>(pos) * D;
        c0 = r[lane]; c1 = r[lane + 32]; s0 = r[64 + lane]; s1 = r[64 + lane + 32];
      } else {
        const __half *ct = cos_table + static_cast<size_t>(pos) * D, *st = sin_table + static_cast<size_t>(pos) * D;
        c0 = __half2float(ct[lane]); c1 = __half2float(ct[lane + 32]);
        s0 = __half2float(st[lane]); s1 = __half2float(st[lane + 32]);
      }
      const float r0 = x[0] * c0 - x[2] * s0, r2 = x[0] * s0 + x[2] * c0;
      const float r1 = x[1] * c1 - x[3] * s1, r3 = x[1] * s1 + x[3] * c1;
      x[0] = r0; x[1] = r1; x[2] = r2; x[3] = r3;
    }
    if (warp < 2) {
      __half *qh = reinterpret_cast<__half *>(s_qf + (2 * warp) * DAM_QPITCH);
      __half *ql = reinterpret_cast<__half *>(s_qf + (2 * warp + 1) * DAM_QPITCH);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        sq[warp * D + lane + 32 * i] = x[i];
        qh[lane + 32 * i] = dam_split(x[i], false);
        ql[lane + 32 * i] = dam_split(x[i], true);
      }
    } else {
      float *snew = warp == 2 ? sknew : svnew;
      __half *dst = (warp == 2 ? kbase : vbase) + static_cast<size_t>(pos) * D;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const __half hv = __float2half_rn(x[i]);
        if (owner) dst[lane + 32 * i] = hv;
        snew[lane + 32 * i] = __half2float(hv);
      }
    }
  }
  // the eight consumer warps only: the producer thread must not wait here (it waits for slots they free later)
  if (warp < DAM_WARPS) asm volatile("bar.sync 1, %0;" ::"n"(DAM_WARPS * 32) : "memory");
  const float sc = scale * 1.4426950408889634f;
  if (warp < 2) {   // score of the new row for query head `warp`
    float d = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) d = fmaf(sq[warp * D + lane + 32 * i], sknew[lane + 32 * i], d);
    d = warp_sum(d);
    if (lane == 0) snew_score[warp] = d * sc;
  }
  if (warp < DAM_WARPS) {             // ---- consumers
    const int quad = lane & 3, rowq = lane >> 2;     // accumulator fragment: rows rowq, rowq + 8; columns 2 quad, 2 quad + 1
    float acc[8][4];
#pragma unroll
    for (int t = 0; t < 8; ++t) { acc[t][0] = 0.f; acc[t][1] = 0.f; acc[t][2] = 0.f; acc[t][3] = 0.f; }
    float m = -INFINITY, l = 0.f;                    // running max / sum of this lane's head (quad = head, quads 2, 3 idle)
    uint32_t qf[4][4];                               // query operand fragments of the four 32-dim groups
    {
      const uint32_t q_addr = s32(s_qf + (lane & 3) * DAM_QPITCH) + (lane >> 3) * 16;   // rows 4..7 repeat 0..3
#pragma unroll
      for (int p = 0; p < 4; ++p) dam_ldsm_x4(q_addr + p * 64, qf[p]);
    }
    const int lr = (lane & 7) + ((lane >> 3) & 1) * 8;
    for (int c = warp; c < nchunks; c += DAM_WARPS) {
      const int slot = c % DAM_SLOTS;
      bool mine = true;
      if (*issued_ctr <= c) {           // bounded wait for the producer to reach this chunk
        unsigned long long t0, t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
        for (uint32_t it = 1; *issued_ctr <= c; ++it) {
          if ((it & 63u) == 0u) {
            if (*abort_flag) { mine = false; break; }
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
            if (t - t0 > budget_ns) { *abort_flag = 1; atomicCAS(status, 0u, 4u); mine = false; break; }
          }
        }
      }
      const bool ok = __all_sync(0xffffffffu, mine && wait(full + slot, (c / DAM_SLOTS) & 1));
      const int nrow = min(DAM_ROWS, pos - (c_begin + c) * DAM_ROWS);
      if (ok) {   // warp-uniform
        unsigned char *slot_ptr = dam_smem + slot * DAM_SLOT_BYTES;
        const uint32_t base = s32(slot_ptr);
        if (nrow < DAM_ROWS) {   // rows past the sequence's end hold whatever the cache holds there: p = 0 for them, but 0 x NaN must not happen
          unsigned char *vrows = slot_ptr + 2 * DAM_BOX;
          const int pieces = (DAM_ROWS - nrow) * 8;      // 16-byte pieces per box
          for (int i = lane; i < 2 * pieces; i += 32)
            reinterpret_cast<uint4 *>(vrows + (i >= pieces ? DAM_BOX : 0) + nrow * 128)[i >= pieces ? i - pieces : i] = make_uint4(0u, 0u, 0u, 0u);
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // these stores precede the slot's next tiled copy
          __syncwarp();
        }
        float sc4[4] = {0.f, 0.f, 0.f, 0.f}, sc4b[4] = {0.f, 0.f, 0.f, 0.f};   // two chains of four dependent MMAs instead of one of eight
        const uint32_t k_row = base + lr * 128;                        // this lane's K row in box 0
        const uint32_t k_xor = ((k_row >> 7) & 7u) << 4;               // swizzle of that row (the same in box 1: boxes are 2048 bytes)
        const uint32_t k_off = (lane >> 4) * 16;
#pragma unroll
        for (int p = 0; p < 4; ++p) {
          uint32_t a0[4], a1[4];
          dam_ldsm_x4(k_row + (p >> 1) * DAM_BOX + ((((p & 1) * 64) + k_off) ^ k_xor), a0);
          dam_ldsm_x4(k_row + (p >> 1) * DAM_BOX + ((((p & 1) * 64) + 32 + k_off) ^ k_xor), a1);
          mma_16816(sc4, a0, qf[p][0], qf[p][1]);
          mma_16816(sc4b, a1, qf[p][2], qf[p][3]);
        }
        float s_top = fmaf(sc4[1] + sc4b[1], DAM_LO_INV, sc4[0] + sc4b[0]) * sc, s_bot = fmaf(sc4[3] + sc4b[3], DAM_LO_INV, sc4[2] + sc4b[2]) * sc;
        if (rowq >= nrow) s_top = -INFINITY;
        if (rowq + 8 >= nrow) s_bot = -INFINITY;
        float cm = fmaxf(s_top, s_bot);
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) cm = fmaxf(cm, __shfl_xor_sync(0xffffffffu, cm, o));
        const float mn = fmaxf(m, cm);                    // finite: row 0 of a chunk always exists
        const float corr = exp2f(m - mn);
        const float p_top = exp2f(s_top - mn), p_bot = exp2f(s_bot - mn);
        float ps = p_top + p_bot;
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
        l = fmaf(l, corr, ps);
        m = mn;
        if (__any_sync(0xffffffffu, corr != 1.0f)) {
#pragma unroll
          for (int t = 0; t < 8; ++t) { acc[t][0] *= corr; acc[t][1] *= corr; acc[t][2] *= corr; acc[t][3] *= corr; }
        }
        // p as the B operand: column n = lane / 4 (0: head 0 hi, 1: head 0 lo, 2: head 1 hi, 3: head 1 lo, 4..7: zero),
        // rows 2 quad, 2 quad + 1 (b0) and + 8 (b1); p(head h, row r) lives in lane 4 (r % 8) + h
        const int n = lane >> 2, src_lane = (2 * quad) * 4 + ((n >> 1) & 1);
        const float pta = __shfl_sync(0xffffffffu, p_top, src_lane), ptb = __shfl_sync(0xffffffffu, p_top, src_lane + 4);
        const float pba = __shfl_sync(0xffffffffu, p_bot, src_lane), pbb = __shfl_sync(0xffffffffu, p_bot, src_lane + 4);
        uint32_t b0 = 0u, b1 = 0u;
        if (n < 4) {
          const bool lo = (n & 1) != 0;
          b0 = dam_pack(dam_split(pta, lo), dam_split(ptb, lo));
          b1 = dam_pack(dam_split(pba, lo), dam_split(pbb, lo));
        }
        const uint32_t v_row = base + 2 * DAM_BOX + ((lane & 7) + 8 * (lane >> 4)) * 128;
        const uint32_t v_xor = ((v_row >> 7) & 7u) << 4;
        const uint32_t v_off = ((lane >> 3) & 1) * 16;
#pragma unroll
        for (int t = 0; t < 8; ++t) {
          uint32_t a[4];
          dam_ldsm_x4_trans(v_row + (t >> 2) * DAM_BOX + ((((t & 3) * 32) + v_off) ^ v_xor), a);
          mma_16816(acc[t], a, b0, b1);
        }
      }
      __syncwarp();
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(s32(empty + slot)) : "memory");
      if (!ok) break;
    }
    // this warp's partial state: lanes of quad h hold head h (columns hi, lo of the accumulator fragments)
    if (quad < 2) {
#pragma unroll
      for (int t = 0; t < 8; ++t) {
        sacc[warp][quad][t * 16 + rowq] = fmaf(acc[t][1], DAM_LO_INV, acc[t][0]);
        sacc[warp][quad][t * 16 + rowq + 8] = fmaf(acc[t][3], DAM_LO_INV, acc[t][2]);
      }
      if (rowq == 0) { sm[warp][quad] = m; sl[warp][quad] = l; }
    }
  }
  __syncthreads();
  // This CTA's state per (head, dim): running maximum M, sum L, unnormalised output A.
  float M = -INFINITY, L = 0.f, A = 0.f;
  const int h = (threadIdx.x >> 7) & 1, d = threadIdx.x & (D - 1);
  if (threadIdx.x < 2 * D) {
    if (owner) M = snew_score[h];     // the new row is always there
#pragma unroll
    for (int w = 0; w < DAM_WARPS; ++w) M = fmaxf(M, sm[w][h]);
    if (owner) { L = exp2f(snew_score[h] - M); A = L * svnew[d]; }
#pragma unroll
    for (int w = 0; w < DAM_WARPS; ++w) {
      const float mw = sm[w][h];
      const float s = (mw == -INFINITY) ? 0.f : exp2f(mw - M);
      L = fmaf(sl[w][h], s, L);
      A = fmaf(sacc[w][h][d], s, A);
    }
  }
  if (nsplit == 1) {
    if (threadIdx.x < 2 * D) out[static_cast<size_t>(b) * QS + (2 * g + h) * D + d] = __float2half_rn(A / L);
    return;
  }
  // Split sequence: every CTA leaves (A, M, L) in global memory; the CTA that arrives last (a counter per
  // (sequence, kv head), no waiting) adds the partial states in split order and resets the counter.
  constexpr int PART = 2 * (D + 2);                       // floats per partial state: two heads of A[128], M, L
  float *mine = split_part + (static_cast<size_t>(b * NKV + g) * nsplit + split) * PART;
  if (threadIdx.x < 2 * D) {
    mine[h * (D + 2) + d] = A;
    if (d == 0) { mine[h * (D + 2) + D] = M; mine[h * (D + 2) + D + 1] = L; }
  }
  __threadfence();
  __syncthreads();
  __shared__ unsigned int s_last;
  if (threadIdx.x == 0) s_last = atomicAdd(split_count + b * NKV + g, 1u) == static_cast<unsigned int>(nsplit - 1);
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  if (threadIdx.x < 2 * D) {
    const float *base = split_part + static_cast<size_t>(b * NKV + g) * nsplit * PART + h * (D + 2);
    constexpr int MAX_SPLITS = 8;      // (the host never launches more) all loads first: one L2 round trip
    float ms[MAX_SPLITS], ls[MAX_SPLITS], as[MAX_SPLITS];
#pragma unroll
    for (int sp = 0; sp < MAX_SPLITS; ++sp) {
      const bool have = sp < nsplit;
      ms[sp] = have ? __ldcg(base + sp * PART + D) : -INFINITY;
      ls[sp] = have ? __ldcg(base + sp * PART + D + 1) : 0.f;
      as[sp] = have ? __ldcg(base + sp * PART + d) : 0.f;
    }
    float Mt = -INFINITY;
#pragma unroll
    for (int sp = 0; sp < MAX_SPLITS; ++sp) Mt = fmaxf(Mt, ms[sp]);
    float Lt = 0.f, At = 0.f;
#pragma unroll
    for (int sp = 0; sp < MAX_SPLITS; ++sp) {      // split order
      const float sc2 = (ms[sp] == -INFINITY) ? 0.f : exp2f(ms[sp] - Mt);
      Lt = fmaf(ls[sp], sc2, Lt);
      At = fmaf(as[sp], sc2, At);
    }
    out[static_cast<size_t>(b) * QS + (2 * g + h) * D + d] = __float2half_rn(At / Lt);
  }
  if (threadIdx.x == 0) split_count[b * NKV + g] = 0u;   // ready for the next launch (stream order)
}

}  // namespace qmk_pf
#endif  // QMK_DECODE_ATTENTION_MMA_CUH_
