// Fused single-sequence decode kernel: four cross-CTA hand-overs per layer instead of six.
//
// Included by megakernel_sm100.cu after megakernel_device.cuh (single-sequence build) and built from its parts:
// the same weight/KV ring, tagged exchange words, bounded waits, RMSNorm/row-product routines and attention items.
// What changes is where the O and down projections run.  In megakernel_device.cuh's kernel a layer is
//   QKV rows -> [q|k|v words] -> attention items -> [partials] -> merge -> [attention output, 2048 words to all]
//   -> O rows -> [x1, 1024 words to all] -> gate/up rows -> [activations, 3072 words to all] -> down rows -> [x2 to all]
// i.e. six dependent grid-wide hand-overs, each 1.3-2.5 us on 148 CTAs.  Here the CTA that merges attention
// outputs [e0, e1) multiplies them straight into rows [e0, e1) of a K-major copy of W_o, and the CTA that owns
// gate/up rows [m0, m1) multiplies its activations into rows [m0, m1) of a K-major copy of W_down.  Either way it
// holds 1024 partial sums, which all CTAs add into 1024 global 64-bit accumulators (split-K across the grid):
//   QKV rows -> [q|k|v words] -> attention items -> [partials] -> merge + O slice -> (sum x1) -> gate/up rows +
//   down slice -> (sum x2)
// The 2048-word and the 3072-word broadcasts and two whole phases are gone.
//
// The sums.  An accumulator word is an integer: (sum of fixed-point contributions << 10) + number of
// contributions.  Integer adds commute, so the result does not depend on arrival order (logits stay bit-identical
// run to run), and the word tells by itself when it is complete: use number k of a buffer is complete when the
// low ten bits equal k * contributors (mod 1024), with no separate flag, counter or fence.  Words are never reset
// while a launch runs: every CTA adds the DIFFERENCE between its partial of this use and its partial of the
// previous use (kept in shared memory), so a complete word always holds the current sum.  The host zeroes the
// buffer before each launch.  Fixed point: 2^-28 units in a signed 54-bit field, i.e. |sum| < 3.3e7 to 3.7e-9.
// Reuse is safe with a single buffer per sum: a CTA adds into x1 of layer L+1 only after it saw x2 of layer L
// complete, which every CTA contributes to after it has read x1 of layer L in full (and likewise for x2).
//
// Measured primitive (148 CTAs, chained): one such all-reduce of 1024 values costs 3.3 us, of which 0.9 us is the
// 148 same-address adds draining one after the other; `red_copies` = 2 halves that queue (even and odd CTAs add
// into different copies, readers add the copies).

namespace QMK_NS {
#if QMK_MAX_SEQ == 1

constexpr int RED_CNT_BITS = 10;
constexpr unsigned long long RED_CNT_MASK = (1ull << RED_CNT_BITS) - 1ull;
constexpr float RED_SCALE = 268435456.0f;             // 2^28
constexpr float RED_INV_SCALE = 1.0f / 268435456.0f;
constexpr int RED_MAX_COPIES = 2;
constexpr int RED_BUF_STRIDE = RED_MAX_COPIES * H;    // words of one sum: [copy][1024]
constexpr int RED_X1 = 0, RED_X2 = RED_BUF_STRIDE;
constexpr int RED_WORDS = 2 * RED_BUF_STRIDE;
static_assert(MAX_CTAS < (1 << RED_CNT_BITS), "the contribution count of one use must fit the count field");

// Shared-memory aliases of the fused kernel inside the single-sequence layout: the 3072-float activation vector
// is not needed (activations never leave the CTA), the per-warp attention partials are free outside the attention phase.
constexpr int FF_PREV = F_VEC;                 // [2][1024] this CTA's previous contribution to x1 / x2
constexpr int FF_ATTN = F_VEC + 2 * H;         // [<= 32]   merged attention outputs of this CTA's slice
constexpr int FF_INTER = FF_ATTN + 32;         // [<= 64]   SwiGLU outputs of this CTA's gate/up rows
constexpr int FF_SPLITW = FF_INTER + 64;       // [2][32]   weight of each split of the (at most two) heads of the slice
constexpr int FF_COLPART = F_WPART;            // [3][1024] column partials of the three warp groups
static_assert(FF_SPLITW + 64 <= F_VEC + I, "fused aliases exceed the activation vector");
static_assert(3 * H <= CONS_WARPS * 2 * PART_STRIDE, "column partials exceed the attention partial area");
static_assert(CONS_WARPS == 12, "slice_colgemv maps 12 warps to 3 row groups x 4 column blocks");
constexpr int FUSED_MIN_CTAS = 74;             // below: a slice exceeds the aliases above / a phase exceeds the ring
constexpr int SLICE_ROWS_PER_CHUNK = 4;

__device__ __forceinline__ void red_add_u64(unsigned long long *p, unsigned long long v) {
  asm volatile("red.relaxed.gpu.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

// Contributors to copy r of a sum: CTAs r, r + R, ...
__device__ __forceinline__ uint32_t red_contributors(int ncta, int R, int r) { return static_cast<uint32_t>((ncta - r + R - 1) / R); }

#ifndef QMK_TC_BUILD
// Waits until use number `use` (1-based) of a sum is complete, writes its 1024 fp32 values to shared memory
// and returns this thread's share of the sum of squares.  Every thread polls its own three words; all loads
// of a round are issued before any is looked at.  With two accumulator copies the copies are taken one after
// the other (they complete together; the second pass costs one more L2 round trip) and added as integers.
// which = 0: sum x1 -> s_x1; 1: sum x2 -> s_x (the next layer's input)
__device__ __noinline__ float red_wait_vec(const Params &P, const Ctx c, int which, uint32_t use) {
  constexpr int PT = (H + CONS_THREADS - 1) / CONS_THREADS;   // 3 words per thread and copy
  const unsigned long long *buf = P.red + (which ? RED_X2 : RED_X1);
  float *dst = c.f(which ? F_X : F_X1);
  const int R = P.red_copies;
  QMK_FINE(which ? 44 : 40);
  long long vi[PT];
#pragma unroll
  for (int j = 0; j < PT; ++j) vi[j] = 0;
  uint32_t valid = 0;
#pragma unroll
  for (int j = 0; j < PT; ++j)
    if (c.tid + j * CONS_THREADS < H) valid |= 1u << j;
#pragma unroll 1
  for (int r = 0; r < R; ++r) {
    const unsigned long long base = static_cast<unsigned long long>(use) * red_contributors(c.ncta, R, r);
    const unsigned long long *src = buf + r * H + c.tid;
    unsigned long long w[PT];
#pragma unroll
    for (int j = 0; j < PT; ++j)
      if (valid & (1u << j)) w[j] = ll_load(src + j * CONS_THREADS);
    uint32_t pending = valid;
    unsigned long long t0 = 0;
    uint32_t it = 0;
    for (;;) {
#pragma unroll
      for (int j = 0; j < PT; ++j)
        if ((pending & (1u << j)) && ((w[j] - base) & RED_CNT_MASK) == 0ull) pending &= ~(1u << j);
      if (pending == 0u) break;
      if (P.spin_sleep_ns) __nanosleep(P.spin_sleep_ns);
#pragma unroll
      for (int j = 0; j < PT; ++j)
        if (pending & (1u << j)) w[j] = ll_load(src + j * CONS_THREADS);
      if ((++it & 255u) == 0u) {
        if (c.flags()[0]) break;
        if (ld_relaxed_u32(P.status) != 0u) { c.flags()[0] = 1; break; }
        const unsigned long long t = now_ns();
        if (t0 == 0) t0 = t;
        if (t - t0 > P.timeout_ns) { raise_error(P, c, QMK_ERR_WAIT_TIMEOUT, WHERE_LL); break; }
      }
    }
#pragma unroll
    for (int j = 0; j < PT; ++j)
      if (valid & (1u << j)) vi[j] += static_cast<long long>(w[j] - base) >> RED_CNT_BITS;   // exact
  }
  QMK_FINE(which ? 45 : 41);
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < PT; ++j)
    if (valid & (1u << j)) {
      const float v = static_cast<float>(vi[j]) * RED_INV_SCALE;
      dst[c.tid + j * CONS_THREADS] = v;
      ss = fmaf(v, v, ss);
    }
  return ss;
}

// Eight consecutive K-major weights (one per output column) as fp32.
__device__ __forceinline__ void load_t8(const unsigned char *row, int col8, int wfmt, float (&w)[8]) { load_w8(row, col8, wfmt, w); }

// Split-K slice of a projection whose K-major rows [first, first + nrows) this CTA streamed through the ring in
// chunks of four rows: partial[n] = sum_i act[i] * Wt[first + i][n] for all 1024 outputs n, plus resid[n] for the
// outputs [n0, n1) whose residual this CTA owns, added into the sum at `buf` as the difference to this CTA's
// previous contribution (`prev`, shared memory).  Warp w: row group w / 4 takes chunks g, g + 3, ...; column
// block w % 4 takes outputs [256 (w % 4), +256), eight per lane.
// which = 0: O slice (rows = this CTA's merged attention outputs, residual x, sum x1);
//         1: down slice (rows = its SwiGLU outputs, residual x1, sum x2).
__device__ __noinline__ uint32_t slice_colgemv(const Params &P, Ctx c, int which, int layer) {
  const int wfmt = P.wfmt;
  const SegTab *t = c.segs();
  const int nrows = which ? (t->nseg[K_GU] ? t->nrows[K_GU][0] : 0) : t->e1 - t->e0;
  const float *act = c.f(which ? FF_INTER : FF_ATTN);
  const float *resid = c.f(which ? F_X1 : F_X);
  unsigned long long *buf = P.red + (which ? RED_X2 : RED_X1);
  float *prev = c.f(FF_PREV) + (which ? H : 0);
  const int g = c.warp >> 2, cb = c.warp & 3;
  const int nch = (nrows + SLICE_ROWS_PER_CHUNK - 1) / SLICE_ROWS_PER_CHUNK;
  const int trb = wfmt ? H : 2 * H;                 // bytes of a K-major row
  const int col8 = cb * 32 + c.lane;                // group of eight outputs this lane owns
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  [[maybe_unused]] const int fb = which ? 30 : 20;   // (stamp base of the fine-grained profile build)
  QMK_FINE(fb + 0);
#pragma unroll 1
  for (int ch = g; ch < nch; ch += CONS_WARPS / 4) {
    const uint32_t idx = c.chunk + static_cast<uint32_t>(ch);
    if (__all_sync(0xffffffffu, mbar_wait(P, c, c.full(idx % NSLOTS), (idx / NSLOTS) & 1u, WHERE_FULL, false))) {
      const unsigned char *rows = c.slot(idx);
#pragma unroll
      for (int r = 0; r < SLICE_ROWS_PER_CHUNK; ++r) {
        const int i = ch * SLICE_ROWS_PER_CHUNK + r;
        if (i < nrows) {                              // warp-uniform
          const float a = act[i];
          float w[8];
          load_t8(rows + r * trb, col8, wfmt, w);
#pragma unroll
          for (int q = 0; q < 8; ++q) acc[q] = fmaf(w[q], a, acc[q]);
        }
      }
    }
    __syncwarp();
    if (c.lane == 0) mbar_arrive_n(c.empty(idx % NSLOTS), EMPTY_UNITS / 4);   // four column-block warps per chunk
  }
  if (wfmt) {   // per-output scales of the fp8 matrix: they follow its K rows
    const float *col_scale = reinterpret_cast<const float *>(
        reinterpret_cast<const unsigned char *>(c.layer_rec_t(layer)[which]) + static_cast<size_t>(which ? I : QS) * H);
    const float4 s0 = __ldg(reinterpret_cast<const float4 *>(col_scale) + col8 * 2);
    const float4 s1 = __ldg(reinterpret_cast<const float4 *>(col_scale) + col8 * 2 + 1);
    acc[0] *= s0.x; acc[1] *= s0.y; acc[2] *= s0.z; acc[3] *= s0.w;
    acc[4] *= s1.x; acc[5] *= s1.y; acc[6] *= s1.z; acc[7] *= s1.w;
  }
  QMK_FINE(fb + 1);
  float *colpart = c.f(FF_COLPART);
  {
    float4 *dst = reinterpret_cast<float4 *>(colpart + g * H + col8 * 8);
    dst[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
    dst[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
  }
  cons_sync();
  QMK_FINE(fb + 2);
  const int n0 = t->n0, n1 = t->n1;
  unsigned long long *mine = buf + (c.cta % P.red_copies) * H;
#pragma unroll
  for (int j = 0; j < (H + CONS_THREADS - 1) / CONS_THREADS; ++j) {
    const int n = c.tid + j * CONS_THREADS;
    if (n < H) {
      float v = (colpart[n] + colpart[H + n]) + colpart[2 * H + n];
      if (n >= n0 && n < n1) v += resid[n];
      const long long fx = __float2ll_rn(v * RED_SCALE), fx_prev = __float2ll_rn(prev[n] * RED_SCALE);
      prev[n] = v;
      red_add_u64(mine + n, (static_cast<unsigned long long>(fx - fx_prev) << RED_CNT_BITS) + 1ull);
    }
  }
  QMK_FINE(fb + 3);
  return c.chunk + static_cast<uint32_t>(nch);
}

#endif  // QMK_TC_BUILD

// Combines the S partials of every attention output element this CTA owns into s_attn[e - e0] (shared memory).
// The slice [e0, e1) lies in at most two query heads.  The last two warps fetch the (max, sum) pairs of those
// heads' splits and turn them into one weight per split, exp2(max_s - max) / sum; meanwhile every warp fetches
// the unnormalised outputs of its elements (lanes = splits, up to three elements per warp, all words polled
// together).  After a barrier an element is the weighted sum over its splits.
// act16 (tensor-core build): also leave the outputs as fp16 hi / scaled-lo halves at act16[i] / act16[ACT16_PITCH + i],
// zero from the slice's end up to 32.
constexpr int ACT16_PITCH = 72;                // halves between the hi and the lo row (64 + 8: other banks)
__device__ __noinline__ void merge_slice(const Params &P, const Ctx c, int S, uint32_t tag, __half *act16 = nullptr) {
  float *s_attn = c.f(FF_ATTN), *s_wt = c.f(FF_SPLITW);
  const int e0 = c.segs()->e0, e1 = c.segs()->e1;
  const int h0 = e0 >> 7;
  const int s = min(c.lane, S - 1);
  constexpr int NE = 3;
  static_assert(NE * CONS_WARPS >= (QS + FUSED_MIN_CTAS - 1) / FUSED_MIN_CTAS + 1, "elements per CTA exceed three per warp");
  const unsigned long long *wp[NE];
  uint32_t valid = 0;
#pragma unroll
  for (int q = 0; q < NE; ++q) {
    const int e = min(e0 + c.warp + q * CONS_WARPS, e1 - 1);
    wp[q] = c.llr + LL_PART + static_cast<size_t>((e >> 7) * MAX_SPLITS + s) * PART_STRIDE + (e & (D - 1));
    if (c.lane < S && e0 + c.warp + q * CONS_WARPS < e1) valid |= 1u << q;
  }
  float a[NE];
  QMK_FINE(50);
#ifdef QMK_TC_BUILD
  // the owner split (the last one) also handles the new row: its words arrive last
  ll_sentinel(P, c, c.llr + LL_PART + static_cast<size_t>((min(e0 + c.warp, e1 - 1) >> 7) * MAX_SPLITS + S - 1) * PART_STRIDE +
                        (min(e0 + c.warp, e1 - 1) & (D - 1)), tag);
#endif
  const int hw = h0 + (c.warp - (CONS_WARPS - 2));                // head whose split weights this warp makes (last two warps)
  if (c.warp >= CONS_WARPS - 2 && hw <= ((e1 - 1) >> 7)) {        // warp-uniform
    // outputs and the head's (max, sum) pairs in ONE round of polls (one after the other costs a second L2 round trip)
    const unsigned long long *part = c.llr + LL_PART + static_cast<size_t>(hw * MAX_SPLITS + s) * PART_STRIDE;
    const unsigned long long *wp5[NE + 2] = {wp[0], wp[1], wp[2], part + D, part + D + 1};
    float v5[NE + 2];
    ll_wait_many<NE + 2>(P, c, wp5, valid | (c.lane < S ? (3u << NE) : 0u), tag, v5);
    QMK_FINE(51);
#pragma unroll
    for (int q = 0; q < NE; ++q) a[q] = v5[q];
    const float m = c.lane < S ? v5[NE] : -INFINITY, l = c.lane < S ? v5[NE + 1] : 0.f;
    const float M = warp_max(m);
    const float sc = (m == -INFINITY) ? 0.f : exp2f(m - M);
    const float L = warp_sum(l * sc);
    s_wt[(hw - h0) * 32 + c.lane] = sc / L;
  } else {
    ll_wait_many<NE>(P, c, wp, valid, tag, a);
    QMK_FINE(51);
  }
  cons_sync();
  QMK_FINE(52);
  // the (up to three) weighted sums of this warp side by side: their shuffle chains overlap
  float A[NE];
#pragma unroll
  for (int q = 0; q < NE; ++q) {
    const int e = min(e0 + c.warp + q * CONS_WARPS, e1 - 1);
    const float wgt = s_wt[((e >> 7) - h0) * 32 + c.lane];        // 0 for lanes >= S
    A[q] = (valid & (1u << q)) ? a[q] * wgt : 0.f;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
#pragma unroll
    for (int q = 0; q < NE; ++q) A[q] += __shfl_xor_sync(0xffffffffu, A[q], o);
#pragma unroll
  for (int q = 0; q < NE; ++q) {
    const int e = e0 + c.warp + q * CONS_WARPS;
    if (e < e1 && c.lane == 0) {
      s_attn[e - e0] = A[q];
      if (act16) {
        const __half h = __float2half_rn(A[q]);
        act16[e - e0] = h;
        act16[ACT16_PITCH + e - e0] = __float2half_rn((A[q] - __half2float(h)) * 2048.0f);
      }
    }
  }
  if (act16 && c.tid < 32 && c.tid >= e1 - e0) { act16[c.tid] = __float2half_rn(0.f); act16[ACT16_PITCH + c.tid] = __float2half_rn(0.f); }
}

#ifndef QMK_TC_BUILD
__device__ __forceinline__ bool produce_rows(const Params &P, const Ctx &c, uint32_t &idx, uint64_t pol, const unsigned char *src,
                                             int nrows, int row_bytes) {
#pragma unroll 1
  for (int r = 0; r < nrows; r += SLICE_ROWS_PER_CHUNK) {
    const int nr = min(SLICE_ROWS_PER_CHUNK, nrows - r);
    if (!produce_chunk(P, c, idx, pol, src + static_cast<size_t>(r) * row_bytes, nullptr, static_cast<uint32_t>(nr * row_bytes),
                       P.stream_inflight))
      return false;
  }
  return true;
}

// Producer schedule of the fused kernel.  Per layer: norm vectors, QKV rows, this CTA's old K/V rows, K-major
// O rows [e0, e1), gate/up rows, K-major down rows [m0, m1); per token: LM-head rows.
__device__ __noinline__ void producer_main_fused(const Params &P, const Ctx c) {
  const uint64_t pol = P.l2_evict_first ? l2_evict_first_policy() : l2_evict_normal_policy();
  const SegTab *t = c.segs();
  const int e0 = t->e0, ne = t->e1 - t->e0;
  const int m0 = t->nseg[K_GU] ? t->row0[K_GU][0] : 0, nm = t->nseg[K_GU] ? t->nrows[K_GU][0] : 0;
  const int trb = P.wfmt ? H : 2 * H;
  uint32_t idx = 0;
  bool ok = true;
#pragma unroll 1
  for (int step = 0; ok && step < P.num_steps; ++step) {
#pragma unroll 1
    for (int l = 0; ok && l < P.num_layers; ++l) {
      const unsigned long long *rec = c.layer_rec(l);
      const unsigned long long *rect = c.layer_rec_t(l);
      {
        const uint32_t L = static_cast<uint32_t>(step) * static_cast<uint32_t>(P.num_layers) + static_cast<uint32_t>(l);
        const uint32_t b = L & 1u;
        __half *dst = c.norms(b);
        c.flags()[4 + b] = static_cast<int>(L + 1u);
        mbar_arrive_expect_tx(c.nfull(b), NORM_HALVES * 2);
        bulk_g2s(dst + NB_IN_LN, reinterpret_cast<const void *>(rec[REC_IN_LN]), H * 2, c.nfull(b), l2_evict_normal_policy());
        bulk_g2s(dst + NB_POST_LN, reinterpret_cast<const void *>(rec[REC_POST_LN]), H * 2, c.nfull(b), l2_evict_normal_policy());
        bulk_g2s(dst + NB_QNORM, reinterpret_cast<const void *>(rec[REC_QNORM]), D * 2, c.nfull(b), l2_evict_normal_policy());
        bulk_g2s(dst + NB_KNORM, reinterpret_cast<const void *>(rec[REC_KNORM]), D * 2, c.nfull(b), l2_evict_normal_policy());
      }
      ok = produce_phase(P, c, idx, pol, K_QKV, rec);
      {
        const AttnItem it = attn_item(P, c, 0, 1, CONS_WARPS, P.start_position + step);
        const size_t head_base = (static_cast<size_t>(l) * NKV + it.g) * static_cast<size_t>(P.max_seq_len) * D;
#pragma unroll 1
        for (int r = it.p0; ok && r < it.p1; r += it.rpc) {
          const uint32_t bytes = static_cast<uint32_t>(min(it.rpc, it.p1 - r)) * D * 2;
          const size_t off = (head_base + static_cast<size_t>(r) * D) * 2;
          ok = produce_chunk(P, c, idx, pol, reinterpret_cast<const unsigned char *>(P.k_cache) + off,
                             reinterpret_cast<const unsigned char *>(P.v_cache) + off, bytes, P.stream_inflight);
        }
      }
      if (ok) ok = produce_rows(P, c, idx, pol, reinterpret_cast<const unsigned char *>(rect[0]) + static_cast<size_t>(e0) * trb, ne, trb);
      if (ok) ok = produce_phase(P, c, idx, pol, K_GU, rec);
      if (ok) ok = produce_rows(P, c, idx, pol, reinterpret_cast<const unsigned char *>(rect[1]) + static_cast<size_t>(m0) * trb, nm, trb);
    }
    if (ok && !P.prefill) ok = produce_phase(P, c, idx, pol, K_LM, nullptr);
  }
  c.flags()[2] = static_cast<int>(idx);
}

// Embedding row of `token` -> fp32 residual stream in shared memory (megakernel_5090.cu:825-830); returns this
// thread's share of the sum of squares.
__device__ __noinline__ float embed_row(const Params &P, const Ctx c, int token) {
  float *s_x = c.f(F_X);
  float ss = 0.f;
  const unsigned char *erow = reinterpret_cast<const unsigned char *>(P.embed) +
                              static_cast<size_t>(token) * kind_row_bytes(K_LM, P.wfmt);
  const float escale = P.wfmt ? __ldg(reinterpret_cast<const float *>(erow + H)) : 1.0f;
#pragma unroll
  for (int j = 0; j < (H + CONS_THREADS - 1) / CONS_THREADS; ++j)
    if (c.tid + j * CONS_THREADS < H) {
      const int k = c.tid + j * CONS_THREADS;
      float v;
      if (P.wfmt) {
        const __half_raw hr = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(__ldg(erow + k)), __NV_E4M3);
        v = __half2float(*reinterpret_cast<const __half *>(&hr)) * escale;
      } else {
        v = __half2float(__ldg(reinterpret_cast<const __half *>(erow) + k));
      }
      s_x[k] = v;
      ss = fmaf(v, v, ss);
    }
  return ss;
}

#endif  // QMK_TC_BUILD

// Argmax across the grid (megakernel_5090.cu:1137-1167): every CTA publishes the best (value, row) of its LM-head
// rows (left per warp in s_misc[32..], s_misc[48..]), reads all CTAs' pairs and leaves the winning row, lowest
// index on ties, in s_misc[16].  Entered after a consumer barrier.
__device__ __noinline__ void argmax_exchange(const Params &P, const Ctx c, uint32_t atag) {
  float *s_misc = c.f(F_MISC), *s_amax = c.f(F_AMAX);
  if (c.tid == 0) {
    float best = s_misc[32];
    int best_i = __float_as_int(s_misc[48]);
#pragma unroll 1
    for (int w = 1; w < CONS_WARPS; ++w) {
      const float v = s_misc[32 + w];
      const int vi = __float_as_int(s_misc[48 + w]);
      if (v > best || (v == best && vi < best_i)) { best = v; best_i = vi; }
    }
    ll_publish(P.ll + LL_AMAX + 2 * c.cta, best, atag, 1);
    ll_publish(P.ll + LL_AMAX + 2 * c.cta + 1, __int_as_float(best_i), atag, 1);
    if (P.bmax_vals) P.bmax_vals[c.cta] = best;
    if (P.bmax_idxs) P.bmax_idxs[c.cta] = best_i;
  }
#pragma unroll 1
  for (int i = c.tid; i < 2 * c.ncta; i += CONS_THREADS) s_amax[i] = ll_wait(P, c, c.llr + LL_AMAX + i, atag);
  cons_sync();
  if (c.warp == 0) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
#pragma unroll 1
    for (int k = c.lane; k < c.ncta; k += 32) {
      const float v = s_amax[2 * k];
      const int vi = __float_as_int(s_amax[2 * k + 1]);
      if (v > bv || (v == bv && vi < bi)) { bv = v; bi = vi; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (c.lane == 0) s_misc[16] = __int_as_float(bi);
  }
}

#ifndef QMK_TC_BUILD
__global__ void __launch_bounds__(THREADS, 1) qwen3_decode_megakernel_fused(const __grid_constant__ Params P) {
  extern __shared__ __align__(128) unsigned char smem[];
  Ctx c;
  c.smem = smem;
  c.tid = threadIdx.x;
  c.warp = threadIdx.x >> 5;
  c.lane = threadIdx.x & 31;
  c.cta = blockIdx.x;
  c.ncta = gridDim.x;
  c.chunk = 0;
  c.repl = 1;            // the exchanges that remain have few readers per word: one copy
  c.llr = P.ll;

  if (c.tid == 0) {
    for (int i = 0; i < NSLOTS; ++i) { mbar_init(c.full(i), 1); mbar_init(c.empty(i), EMPTY_UNITS); }
    mbar_init(c.nfull(0), 1);
    mbar_init(c.nfull(1), 1);
    volatile int *fl = c.flags();
    fl[0] = 0; fl[1] = 0; fl[2] = 0; fl[3] = 0; fl[4] = 0; fl[5] = 0; fl[6] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (c.tid == 32) build_segtab(reinterpret_cast<SegTab *>(smem + OFF_SEGS), c.cta, c.ncta, P.vocab);
  {
    const unsigned long long *src = reinterpret_cast<const unsigned long long *>(P.layers);
    unsigned long long *dst = reinterpret_cast<unsigned long long *>(smem + OFF_LAYERS);
    for (int i = c.tid; i < P.num_layers * 12; i += THREADS) dst[i] = src[i];
    const unsigned long long *srct = reinterpret_cast<const unsigned long long *>(P.layers_t);
    unsigned long long *dstt = reinterpret_cast<unsigned long long *>(smem + OFF_LAYERS_T);
    for (int i = c.tid; i < P.num_layers * 2; i += THREADS) dstt[i] = srct[i];
    float *prev = c.f(FF_PREV);
    for (int i = c.tid; i < 2 * H; i += THREADS) prev[i] = 0.f;   // the host zeroed the sums: nothing contributed yet
  }
  __syncthreads();

  if (c.warp == CONS_WARPS) {
    if (c.lane == 0) producer_main_fused(P, c);
    __syncwarp();
  } else {
    float *s_x = c.f(F_X), *s_misc = c.f(F_MISC);
    int token = P.prefill ? P.token_ids[0] : P.first_token;
#pragma unroll 1
    for (int step = 0; step < P.num_steps; ++step) {
      const int pos = P.start_position + step;
      const uint32_t tag_base = (P.seq_base + static_cast<uint32_t>(step)) * 64u;
      if (token < 0 || token >= P.vocab) { if (c.tid == 0) raise_error(P, c, QMK_ERR_BAD_TOKEN, WHERE_TOKEN); token = 0; }
      if (c.tid < D / 2) {
        float cs, sn;
        if (P.rope_from_table) {
          cs = __half2float(P.cos_table[static_cast<size_t>(pos) * D + c.tid]);
          sn = __half2float(P.sin_table[static_cast<size_t>(pos) * D + c.tid]);
        } else {
          cs = __ldg(P.rope + static_cast<size_t>(pos) * D + c.tid);
          sn = __ldg(P.rope + static_cast<size_t>(pos) * D + 64 + c.tid);
        }
        c.f(F_CS)[c.tid] = cs;
        c.f(F_CS)[64 + c.tid] = sn;
      }
      __threadfence();  // acquire side of the KV-row ordering (rows written in earlier steps)
      const int S_step = max(1, min(pos / max(1, P.split_len), min(MAX_SPLITS, max(1, c.ncta / NKV))));  // as attn_item
      float ss = embed_row(P, c, token);
#pragma unroll 1
      for (int layer = 0; layer < P.num_layers; ++layer) {
        const uint32_t tag = tag_base + static_cast<uint32_t>(layer) + 1u;
        const uint32_t Lg = static_cast<uint32_t>(step) * static_cast<uint32_t>(P.num_layers) + static_cast<uint32_t>(layer);
        const __half *nv = c.norms(Lg & 1u);
        const uint32_t use = Lg + 1u;   // uses of each sum in this launch, this layer's included
#ifdef QMK_FINE_PROF
        if (c.tid == 0) c.flags()[8] = (step == P.num_steps - 1 && layer == 5) ? 1 : 0;
#endif
        mbar_wait(P, c, c.nfull(Lg & 1u), (Lg >> 1) & 1u, WHERE_FULL, false);
        // P1: input RMSNorm + fused QKV rows -> q|k|v words
        QMK_STAMP(layer * 12 + 0);
        c.chunk = gemv_k1024<false>(P, c, K_QKV, s_x, ss, nv + NB_IN_LN, P.ll + LL_QKV, tag, nullptr);
        // P2: attention work items -> partials
        QMK_STAMP(layer * 12 + 1);
        c.chunk = attention_phase<true>(P, c, nv, layer, pos, tag);
        // P3: merge of this CTA's output elements, their slice of the O projection, residual -> sum x1
        QMK_STAMP(layer * 12 + 2);
        merge_slice(P, c, S_step, tag);
        QMK_STAMP(layer * 12 + 3);
        cons_sync();
        c.chunk = slice_colgemv(P, c, 0, layer);
        // P4: post-attention RMSNorm, gate/up rows + SwiGLU, their slice of the down projection, residual -> sum x2
        QMK_STAMP(layer * 12 + 4);
        ss = red_wait_vec(P, c, 0, use);
        QMK_STAMP(layer * 12 + 5);
        c.chunk = gemv_k1024<false>(P, c, K_GU, c.f(F_X1), ss, nv + NB_POST_LN, nullptr, tag, nullptr, c.f(FF_INTER));
        QMK_STAMP(layer * 12 + 6);
        cons_sync();
        c.chunk = slice_colgemv(P, c, 1, layer);
        QMK_STAMP(layer * 12 + 7);
        ss = red_wait_vec(P, c, 1, use);
        QMK_STAMP(layer * 12 + 8);
        if (cons_any(c.flags()[0] != 0)) break;
      }
      if (cons_any(c.flags()[0] != 0)) break;
      if (P.prefill) {
        if (step + 1 < P.num_steps) token = P.token_ids[step + 1];
        continue;
      }
      QMK_STAMP(P.num_layers * 12 + 0);
      c.chunk = gemv_k1024<false>(P, c, K_LM, s_x, ss, P.final_norm, nullptr, 0u,
                                  P.logits_out ? P.logits_out + static_cast<size_t>(step) * P.vocab : nullptr);
      QMK_STAMP(P.num_layers * 12 + 1);
      cons_sync();
      argmax_exchange(P, c, tag_base + 63u);
      const bool aborted = cons_any(c.flags()[0] != 0);
      QMK_STAMP(P.num_layers * 12 + 2);
      token = __float_as_int(s_misc[16]);
      if (aborted) break;
      if (c.cta == 0 && c.tid == 0) {
        if (P.output_log) P.output_log[step] = token;
        if (P.output_token) *P.output_token = token;
      }
      if (token == P.eos) break;
    }
    if (c.tid == 0) { c.flags()[3] = static_cast<int>(c.chunk); c.flags()[1] = 1; }
  }
  __syncthreads();
  if (c.tid == CONS_THREADS) {   // bulk copies issued but never consumed must land before the CTA exits
    const uint32_t issued = static_cast<uint32_t>(c.flags()[2]);
#pragma unroll 1
    for (uint32_t i = (issued > NSLOTS ? issued - NSLOTS : 0u); i < issued; ++i) {
      uint64_t *bar = c.full(i % NSLOTS);
      const uint32_t parity = (i / NSLOTS) & 1u;
      const unsigned long long t0 = now_ns();
      while (!mbar_try_wait(bar, parity)) {
        if (now_ns() - t0 > P.timeout_ns) { raise_error(P, c, QMK_ERR_WAIT_TIMEOUT, WHERE_DRAIN); break; }
      }
    }
    for (uint32_t b = 0; b < 2; ++b) {
      const int v = c.flags()[4 + b];
      if (v == 0) continue;
      const uint32_t parity = ((static_cast<uint32_t>(v) - 1u) >> 1) & 1u;
      const unsigned long long t0 = now_ns();
      while (!mbar_try_wait(c.nfull(b), parity)) {
        if (now_ns() - t0 > P.timeout_ns) { raise_error(P, c, QMK_ERR_WAIT_TIMEOUT, WHERE_DRAIN); break; }
      }
    }
  }
}

#endif  // QMK_TC_BUILD

#endif  // QMK_MAX_SEQ == 1
}  // namespace QMK_NS
