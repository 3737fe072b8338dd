// Fused single-sequence decode kernel whose row products run on the tensor cores (fp16 weights).
//
// Same layer structure as megakernel_fused.cuh (four cross-CTA hand-overs per layer, integer all-reduced residual
// sums) and the same attention items, merge and exchange code.  What changes is how a CTA multiplies its weight
// rows with the activation vector.  Measured with cycle stamps, every phase of the CUDA-core version ran at 10-20
// cycles per instruction per warp: a phase executes once per layer, the layer's code (150 KB) does not stay in the
// 32 KB an SM can loop in at full fetch rate, and a 1024-wide fp16 row costs 68 instructions per warp (one
// convert and one FMA per weight).  So the goal here is few instructions:
//   * a 16-row x 16-input tile of weights is one ldmatrix.x4 and one mma.sync.m16n8k16; the activation vector is
//     the B operand with its fp32 value split over two fp16 columns (hi = fp16(x), lo = fp16((x - hi) * 2048); the
//     row result is acc_hi + acc_lo / 2048, exact products, fp32 accumulation, relative error ~2^-22), i.e. about
//     5 instructions per row instead of 68;
//   * RMSNorm is applied once per CTA (each thread normalises the three values it fetched, the hi/lo halves go to
//     shared memory) instead of once per warp;
//   * the producer is one loop over four-row chunks for every tensor.
// Ring chunk = four consecutive rows of one matrix, each copied by its own cp.async.bulk to a 2064-byte pitch (and
// chunks in odd slots start 64 bytes in), so that the eight row addresses of an ldmatrix phase fall into different
// banks (2048-byte pitch: 8-way conflict).  Cache chunks (16 K rows + 16 V rows) arrive as four tiled TMA boxes of
// 16 rows x 128 bytes with the 128-byte swizzle, which does the same for 256-byte rows with 4 copies instead of 32
// (one bulk copy per padded 256-byte row was tried: the copy engine takes ~30 cycles per copy whatever its size,
// and 480 copies per layer made the attention phase slower than the CUDA-core loop).
// CTAs own whole chunks: rows of the fused q|k|v matrix, of gate/up and of the LM head are split in units of four.

namespace QMK_NS {
#if QMK_MAX_SEQ == 1 && defined(QMK_TC_BUILD)

constexpr int TC_MIN_CTAS = 96;                // smallest grid: <= 2 attention outputs per warp to merge, O / down slices of <= 32 rows
static_assert(TC_MIN_CTAS >= FUSED_MIN_CTAS, "the tensor-core kernel shares the fused kernel's slice layout");
static_assert(4 * ((I / 4 + TC_MIN_CTAS - 1) / TC_MIN_CTAS) <= 32, "slice_cols takes two k-steps");
constexpr int ROW_PITCH = 2 * H + 16;          // bytes between the rows of a chunk in shared memory
constexpr int CH_ROWS = 4;
constexpr int ODD_SLOT_SKEW = 64;              // weight rows of chunks in odd slots start four 16-byte bank groups later
static_assert(SLOT_BYTES >= ODD_SLOT_SKEW + CH_ROWS * ROW_PITCH, "a slot holds four padded rows");
static_assert(SLOT_BYTES % 128 == 0 && NSLOTS % 2 == 0, "swizzled boxes need 128-byte aligned slots; slot parity = chunk parity");
static_assert(EMPTY_UNITS == 12, "1, 2, 3, 4, 6 or 12 warps share a chunk");
constexpr float LO_SCALE = 2048.0f, LO_INV = 1.0f / 2048.0f;
// Cache chunk in a slot: four boxes of 16 rows x 128 bytes: K dims 0..63, K dims 64..127, V dims 0..63, V dims 64..127.
// Within a box the 16-byte piece j of row r sits at piece j ^ ((address >> 7) & 7) (128-byte swizzle on address bits).
constexpr int KV_BOX = KV_ROWS_PER_CHUNK * 128;
constexpr int KV_V_OFF = 2 * KV_BOX;
constexpr int KV_PITCH = 2 * D + 16;           // pitch of the four query-operand rows (plain padded rows)
static_assert(SLOT_BYTES >= 4 * KV_BOX, "a slot holds the four boxes of a cache chunk");
constexpr int QKV_CHUNKS = QKV_ROWS / CH_ROWS, GU_CHUNKS = I / CH_ROWS;
constexpr int KPAIRS = H / 32;                 // pairs of 16-input k-steps in a row

// Extra shared memory of this kernel, behind the single-sequence layout.
// Normalised activations as the B operand of the row products, in MMA fragment order: 128 bytes per pair of
// k-steps (32 inputs) = [hi: 4 lanes x 16 bytes][lo: 4 lanes x 16 bytes]; the 16 bytes of lane kq are the halves
// {b0, b1} of the first k-step (inputs 2kq, 2kq+1, 2kq+8, 2kq+9) and of the second (the same + 16).  Lanes 0..7 of a
// warp fetch a pair's operand with ONE 128-byte wavefront (ldmatrix.x4 over plain hi / lo rows takes four; the row
// products are bound by shared-memory bandwidth, where that is a third of the traffic).
constexpr size_t OFF_XF = (SMEM_BYTES + 127) / 128 * 128;
constexpr size_t OFF_PART = OFF_XF + 4 * H;                    // fp32 tile partials [2][12 tasks][16 rows]
constexpr size_t OFF_QF = OFF_PART + 2 * 12 * 16 * 4;           // fp16 query operand [4: q0 hi, q0 lo, q1 hi, q1 lo][128], rows at KV_PITCH
constexpr size_t OFF_ACT16 = OFF_QF + 4 * KV_PITCH;            // fp16 hi row, scaled-lo row of a slice's activations (merge / gate-up outputs)
constexpr size_t OFF_TCTAB = OFF_ACT16 + ((2 * ACT16_PITCH * 2 + 15) / 16) * 16;
struct alignas(16) TileTask { int active, first, valid, p0, p1, units, pad0, pad1; };   // see build_tile_tasks
struct alignas(16) TcTab {
  int q0, nq, g0, ng, lm0, nlm;    // first chunk / chunks of this CTA: q|k|v rows, gate (= up) rows, LM-head rows
  int nkb_qkv, nkb_gu;             // warps per tile in the two row-product phases
  TileTask qkv[12], gu[12];        // each warp's tile task in those phases
};
constexpr size_t TC_SMEM_BYTES = OFF_TCTAB + sizeof(TcTab);
static_assert(TC_SMEM_BYTES <= 232448, "over the 227 KB shared-memory limit of one CTA");
static_assert(OFF_XF % 128 == 0 && OFF_QF % 16 == 0, "operand rows are 16-byte aligned, a pair's 128 bytes one wavefront");
// Byte offset in the fragment-order array of input i's hi (lo = 0) or lo (1) half.
__device__ __forceinline__ int xf_offset(int i, int lo) {
  const int kk = i & 31, rem = kk & 15, r8 = rem & 7;
  return (i >> 5) * 128 + lo * 64 + (r8 >> 1) * 16 + ((kk >> 4) * 4 + (rem >> 3) * 2 + (r8 & 1)) * 2;
}

__device__ __forceinline__ const TcTab *tctab(const Ctx &c) { return reinterpret_cast<const TcTab *>(c.smem + OFF_TCTAB); }
__device__ __forceinline__ float *tc_part(const Ctx &c) { return reinterpret_cast<float *>(c.smem + OFF_PART); }

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr) : "memory");
}
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr) : "memory");
}
// fp32 -> fp16 operand half: the value rounded to fp16 (lo = false) or its scaled remainder (lo = true)
__device__ __forceinline__ __half split_half(float x, bool lo) {
  const __half h = __float2half_rn(x);
  return lo ? __float2half_rn((x - __half2float(h)) * LO_SCALE) : h;
}
__device__ __forceinline__ uint32_t pack_half2(__half a, __half b) {
  return static_cast<uint32_t>(__half_as_ushort(a)) | (static_cast<uint32_t>(__half_as_ushort(b)) << 16);
}

// Activation operand of k-step pair p for this lane: column n = lane / 4 of B is the hi vector (n = 0), the lo vector
// (n = 1) or zero; {x, y} = fragments of the first k-step, {z, w} of the second.
__device__ __forceinline__ uint4 b_pair(const Ctx &c, int p) {
  return c.lane < 8 ? *reinterpret_cast<const uint4 *>(c.smem + OFF_XF + p * 128 + c.lane * 16) : make_uint4(0u, 0u, 0u, 0u);
}

// Shared-window address of row 0 of the weight chunk with ring index idx.
__device__ __forceinline__ uint32_t weight_rows(const Ctx &c, uint32_t idx) {
  return smem_u32(c.slot(idx)) + (idx & 1u) * ODD_SLOT_SKEW;
}
__device__ __forceinline__ void tma_box_2d(uint32_t dst, const void *map, int c0, int c1, uint64_t *bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(smem_u32(bar)) : "memory");
}

// One warp: rows of the 16-row tile that starts at ring chunk `first` (valid rows <= 16), k-step pairs [p0, p1).
// Leaves the 16 row sums of that k range in part[0..15] and hands the tile's chunks back with `units` each.
// Lanes 0..3 each wait for one of the tile's chunks (the vote that follows orders the copied bytes before every
// lane's loads); two accumulators halve the chain of dependent MMAs.
__device__ __forceinline__ void tile_task(const Params &P, const Ctx &c, uint32_t first, int valid_rows, int p0, int p1,
                                          float *part, int units, int fslot = 70) {
  const int nch = (valid_rows + CH_ROWS - 1) / CH_ROWS;
  bool ok = true;
  if (c.lane < nch) {
    const uint32_t idx = first + static_cast<uint32_t>(c.lane);
    ok = mbar_wait(P, c, c.full(idx % NSLOTS), (idx / NSLOTS) & 1u, WHERE_FULL, false);
  }
  ok = __all_sync(0xffffffffu, ok);
  QMK_FINE(fslot + 1);
  int lr = (c.lane & 7) + ((c.lane >> 3) & 1) * 8;      // tile row whose address this lane supplies
  if (lr >= valid_rows) lr = 0;                         // rows past the end repeat row 0 (their sums are not used)
  const uint32_t a_addr = weight_rows(c, first + static_cast<uint32_t>(lr >> 2)) + (lr & 3) * ROW_PITCH + (c.lane >> 4) * 16;
  float acc0[4] = {0.f, 0.f, 0.f, 0.f}, acc1[4] = {0.f, 0.f, 0.f, 0.f};
  if (ok) {
#pragma unroll 2
    for (int p = p0; p < p1; ++p) {
      uint32_t a0[4], a1[4];
      const uint4 b = b_pair(c, p);
      ldsm_x4(a_addr + p * 64, a0);
      ldsm_x4(a_addr + p * 64 + 32, a1);
      mma_16816(acc0, a0, b.x, b.y);
      mma_16816(acc1, a1, b.z, b.w);
    }
  }
  QMK_FINE(fslot + 5);
  __syncwarp();
  if (c.lane < nch) mbar_arrive_n(c.empty((first + static_cast<uint32_t>(c.lane)) % NSLOTS), static_cast<uint32_t>(units));
  if ((c.lane & 3) == 0) {
    part[c.lane >> 2] = fmaf(acc0[1] + acc1[1], LO_INV, acc0[0] + acc1[0]);
    part[(c.lane >> 2) + 8] = fmaf(acc0[3] + acc1[3], LO_INV, acc0[2] + acc1[2]);
  }
}

// Per-warp work of a layer phase, fixed for the launch (computed once: the integer divisions behind it cost more
// than the MMAs).  Phase rows = `groups` runs of `nch` consecutive chunks (q|k|v: one run; gate/up: the gate rows'
// chunks, then the up rows'); tiles of 16 rows; when there are fewer tiles than warps, nkb warps share a tile's
// 1024 inputs.  Grids of at least FUSED_MIN_CTAS CTAs have at most 6 tiles per phase: one task per warp.
__device__ inline void build_tile_tasks(TileTask *tasks, int *nkb_out, int groups, int nch) {
  const int tpg = (nch + 3) >> 2, T = groups * tpg;
  const int nkb = T >= CONS_WARPS ? 1 : CONS_WARPS / T;   // 12, 6, 4, 3, 2, 2, 1: divides EMPTY_UNITS
  *nkb_out = nkb;
  for (int w = 0; w < CONS_WARPS; ++w) {
    TileTask &t = tasks[w];
    t.active = w < T * nkb ? 1 : 0;
    const int tile = w / nkb, kb = w - tile * nkb, grp = tile / tpg, tt = tile - grp * tpg;
    t.first = grp * nch + tt * 4;
    t.valid = min(16, (nch - tt * 4) * CH_ROWS);
    t.p0 = (KPAIRS * kb) / nkb;
    t.p1 = (KPAIRS * (kb + 1)) / nkb;
    t.units = EMPTY_UNITS / nkb;
    t.pad0 = t.pad1 = 0;
  }
}
__device__ __forceinline__ void run_tile_task(const Params &P, const Ctx &c, const TileTask *tasks, int fslot) {
  const int4 a = reinterpret_cast<const int4 *>(tasks + c.warp)[0], b = reinterpret_cast<const int4 *>(tasks + c.warp)[1];
  // a = {active, first, valid, p0}, b = {p1, units, -, -}
  if (a.x) tile_task(P, c, c.chunk + static_cast<uint32_t>(a.y), a.z, a.w, b.x, tc_part(c) + c.warp * 16, b.y, fslot);
}

// q|k|v rows of this CTA -> exchange words (megakernel_5090.cu:251-302).
__device__ __noinline__ uint32_t qkv_phase(const Params &P, Ctx c, uint32_t tag) {
  const TcTab *t = tctab(c);
  const int nch = t->nq, nkb = t->nkb_qkv;
  QMK_FINE(0);
  run_tile_task(P, c, t->qkv, 0);
  QMK_FINE(2);
  cons_sync();
  if (c.tid < nch * CH_ROWS) {
    const int r = c.tid;
    const float *p = tc_part(c) + (r >> 4) * nkb * 16 + (r & 15);
    float v = 0.f;
#pragma unroll
    for (int kb = 0; kb < CONS_WARPS; ++kb)
      if (kb < nkb) v += p[kb * 16];
    ll_store(P.ll + LL_QKV + t->q0 * CH_ROWS + r, v, tag);
  }
  QMK_FINE(4);
  return c.chunk + static_cast<uint32_t>(nch);
}

// gate/up rows of this CTA -> silu(gate) * up in shared memory (megakernel_5090.cu:653-685, SiLU in fp32).
__device__ __noinline__ uint32_t gateup_phase(const Params &P, Ctx c) {
  const TcTab *t = tctab(c);
  const int nch = t->ng, nkb = t->nkb_gu;
  QMK_FINE(10);
  run_tile_task(P, c, t->gu, 10);
  QMK_FINE(12);
  cons_sync();
  if (c.tid < nch * CH_ROWS) {
    const int r = c.tid, tpg = (nch + 3) >> 2;
    const float *pg = tc_part(c) + (r >> 4) * nkb * 16 + (r & 15);
    const float *pu = pg + tpg * nkb * 16;
    float g = 0.f, u = 0.f;
#pragma unroll
    for (int kb = 0; kb < CONS_WARPS / 2; ++kb)
      if (kb < nkb) { g += pg[kb * 16]; u += pu[kb * 16]; }
    const float a = g / (1.0f + expf(-g)) * u;
    c.f(FF_INTER)[r] = a;
    __half *act16 = reinterpret_cast<__half *>(c.smem + OFF_ACT16);
    act16[r] = split_half(a, false);
    act16[ACT16_PITCH + r] = split_half(a, true);
  } else if (c.tid < 64) {   // rows past the slice multiply stale bytes: zero activations
    __half *act16 = reinterpret_cast<__half *>(c.smem + OFF_ACT16);
    act16[c.tid] = __float2half_rn(0.f);
    act16[ACT16_PITCH + c.tid] = __float2half_rn(0.f);
  }
  QMK_FINE(14);
  return c.chunk + static_cast<uint32_t>(2 * nch);
}

// Attention work item (kv head g, split s) of this CTA on the tensor cores.  Same contract as attention_phase
// (megakernel_device.cuh): old cache rows [p0, p1) arrive as ring chunks of 16 K rows + 16 V rows (272-byte pitch),
// warp w takes chunks w, w + 12, ...; the last split also normalises, rotates and stores the new K/V row and folds
// it in; unnormalised partials (acc[128], max, sum per query head) are published for the merge.
// Per chunk: scores = K[16 x 128] . q[128 x 4] (columns: head 0 hi/lo, head 1 hi/lo of the fp32 query) as 8 MMAs,
// online softmax on the accumulator fragments (log2 domain), then out[128 x 4] += V^T[128 x 16] . p[16 x 4] as 8
// MMAs with V read through ldmatrix.trans and p split into hi/lo fp16 columns like q: ~75 instructions per 16
// rows where the CUDA-core loop needs ~480.
__device__ __noinline__ uint32_t attention_tc(const Params &P, Ctx c, const __half *nv, int layer, int pos, uint32_t tag) {
  const AttnItem it = attn_item(P, c, 0, 1, CONS_WARPS, pos);
  float *s_q = c.f(F_Q), *s_knew = c.f(F_KNEW), *s_vnew = c.f(F_VNEW), *s_wpart = c.f(F_WPART), *s_misc = c.f(F_MISC);
  const float *s_cs = c.f(F_CS);
  const unsigned long long *qkv = c.llr + LL_QKV;
  if (!it.active) return c.chunk;
  const int S = it.S, g = it.g, s = it.s;
  const bool owner = (s == S - 1);
  const int nrows_item = it.p1 - it.p0;
  const size_t head_base = (static_cast<size_t>(layer) * NKV + g) * static_cast<size_t>(P.max_seq_len) * D;

  QMK_FINE(60);
  // (1) head preparation: warps 0,1 = the two query heads; owner: warp 2 = K, warp 3 = V
  if (c.warp < 2 || (owner && c.warp < 4)) {
    const int w = c.warp, lane = c.lane;
    const unsigned long long *src = (w < 2) ? qkv + (2 * g + w) * D : (w == 2) ? qkv + QS + g * D : qkv + QS + KVS + g * D;
    float nw[4] = {1.f, 1.f, 1.f, 1.f};
    if (w < 3) {
      const __half *nwp = nv + ((w < 2) ? NB_QNORM : NB_KNORM);   // shared memory
#pragma unroll
      for (int i = 0; i < 4; ++i) nw[i] = __half2float(nwp[lane + 32 * i]);
    }
    float v[4];
    {
      const unsigned long long *wp[4] = {src + lane, src + lane + 32, src + lane + 64, src + lane + 96};
      // (a sentinel poll first, as in the residual-sum wait, costs its extra round trip here: 4.05 -> 4.34 us)
      ll_wait_many<4>(P, c, wp, 0xfu, tag, v);
    }
    if (w < 3) {
      float ss = v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3];
      ss = warp_sum(ss);
      const float rstd = 1.0f / sqrtf(ss * (1.0f / D) + RMS_EPS);
#pragma unroll
      for (int i = 0; i < 4; ++i) v[i] = v[i] * rstd * nw[i];
      // rotate-half: element i pairs with i+64 and both use frequency i (i < 64)
      const float c0 = s_cs[lane], s0 = s_cs[64 + lane];
      const float c1 = s_cs[lane + 32], s1 = s_cs[64 + lane + 32];
      const float r0 = v[0] * c0 - v[2] * s0, r2 = v[0] * s0 + v[2] * c0;
      const float r1 = v[1] * c1 - v[3] * s1, r3 = v[1] * s1 + v[3] * c1;
      v[0] = r0; v[1] = r1; v[2] = r2; v[3] = r3;
    }
    if (w < 2) {
      __half *qh = reinterpret_cast<__half *>(c.smem + OFF_QF + (2 * w) * KV_PITCH);
      __half *ql = reinterpret_cast<__half *>(c.smem + OFF_QF + (2 * w + 1) * KV_PITCH);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        s_q[w * D + lane + 32 * i] = v[i];
        qh[lane + 32 * i] = split_half(v[i], false);
        ql[lane + 32 * i] = split_half(v[i], true);
      }
    } else {
      // the new row takes part in this step's attention as the fp16 value the cache will hold
      float *snew = (w == 2) ? s_knew : s_vnew;
#pragma unroll
      for (int i = 0; i < 4; ++i) snew[lane + 32 * i] = __half2float(__float2half_rn(v[i]));
    }
  }
  QMK_FINE(61);
  cons_sync();
  QMK_FINE(62);

  const float sc_log2 = P.attn_scale * 1.4426950408889634f;
  if (owner && c.warp < 2) {   // score of the new row
    float d = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) d = fmaf(s_q[c.warp * D + c.lane + 32 * i], s_knew[c.lane + 32 * i], d);
    d = warp_sum(d);
    if (c.lane == 0) s_misc[c.warp] = d * sc_log2;
  }

  // (2) stream the old rows
  const int quad = c.lane & 3, rowq = c.lane >> 2;     // accumulator fragment: rows rowq, rowq + 8; columns 2 quad, 2 quad + 1
  float acc[8][4];
#pragma unroll
  for (int t = 0; t < 8; ++t) { acc[t][0] = 0.f; acc[t][1] = 0.f; acc[t][2] = 0.f; acc[t][3] = 0.f; }
  float m = -INFINITY, l = 0.f;                        // running max / sum of this lane's head (quad = head, quads 2, 3 idle)
  uint32_t qf[4][4];                                   // query operand fragments of the four 32-input pairs
  {
    const uint32_t q_addr = smem_u32(c.smem + OFF_QF + (c.lane & 3) * KV_PITCH) + (c.lane >> 3) * 16;   // rows 4..7 repeat 0..3
#pragma unroll
    for (int p = 0; p < 4; ++p) ldsm_x4(q_addr + p * 64, qf[p]);
  }
  const int lr = (c.lane & 7) + ((c.lane >> 3) & 1) * 8;
  const bool pass_gate = it.nchunks > NSLOTS;   // see attention_phase
#pragma unroll 1
  for (int j0 = 0; j0 < it.nchunks; j0 += CONS_WARPS) {
    const int j = j0 + c.warp;
    if (j >= it.nchunks) {
      if (pass_gate) cons_sync();
      continue;
    }
    const uint32_t idx = c.chunk + static_cast<uint32_t>(j);
    const int nrow = min(KV_ROWS_PER_CHUNK, nrows_item - j * KV_ROWS_PER_CHUNK);
    if (__all_sync(0xffffffffu, mbar_wait(P, c, c.full(idx % NSLOTS), (idx / NSLOTS) & 1u, WHERE_FULL, false))) {
      const uint32_t base = smem_u32(c.slot(idx));
      if (nrow < KV_ROWS_PER_CHUNK) {   // rows past the item's end hold other rows of the cache: p = 0 for them, but 0 x NaN must not happen
        unsigned char *vrows = c.slot(idx) + KV_V_OFF;
        const int pieces = (KV_ROWS_PER_CHUNK - nrow) * 8;      // 16-byte pieces per box
        for (int i = c.lane; i < 2 * pieces; i += 32)
          reinterpret_cast<uint4 *>(vrows + (i >= pieces ? KV_BOX : 0) + nrow * 128)[i >= pieces ? i - pieces : i] = make_uint4(0u, 0u, 0u, 0u);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // these stores precede the slot's next tiled copy
        __syncwarp();
      }
      float sc[4] = {0.f, 0.f, 0.f, 0.f}, sc2[4] = {0.f, 0.f, 0.f, 0.f};   // two chains of four dependent MMAs instead of one of eight
      const uint32_t k_row = base + lr * 128;                        // this lane's K row in box 0
      const uint32_t k_xor = ((k_row >> 7) & 7u) << 4;               // swizzle of that row (the same in box 1: boxes are 2048 bytes)
      const uint32_t k_off = (c.lane >> 4) * 16;
#pragma unroll
      for (int p = 0; p < 4; ++p) {
        uint32_t a0[4], a1[4];
        ldsm_x4(k_row + (p >> 1) * KV_BOX + ((((p & 1) * 64) + k_off) ^ k_xor), a0);
        ldsm_x4(k_row + (p >> 1) * KV_BOX + ((((p & 1) * 64) + 32 + k_off) ^ k_xor), a1);
        mma_16816(sc, a0, qf[p][0], qf[p][1]);
        mma_16816(sc2, a1, qf[p][2], qf[p][3]);
      }
      float s_top = fmaf(sc[1] + sc2[1], LO_INV, sc[0] + sc2[0]) * sc_log2, s_bot = fmaf(sc[3] + sc2[3], LO_INV, sc[2] + sc2[2]) * sc_log2;
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
      const int n = c.lane >> 2, src_lane = (2 * quad) * 4 + ((n >> 1) & 1);
      const float pta = __shfl_sync(0xffffffffu, p_top, src_lane), ptb = __shfl_sync(0xffffffffu, p_top, src_lane + 4);
      const float pba = __shfl_sync(0xffffffffu, p_bot, src_lane), pbb = __shfl_sync(0xffffffffu, p_bot, src_lane + 4);
      uint32_t b0 = 0u, b1 = 0u;
      if (n < 4) {
        const bool lo = (n & 1) != 0;
        b0 = pack_half2(split_half(pta, lo), split_half(ptb, lo));
        b1 = pack_half2(split_half(pba, lo), split_half(pbb, lo));
      }
      const uint32_t v_row = base + KV_V_OFF + ((c.lane & 7) + 8 * (c.lane >> 4)) * 128;
      const uint32_t v_xor = ((v_row >> 7) & 7u) << 4;
      const uint32_t v_off = ((c.lane >> 3) & 1) * 16;
#pragma unroll
      for (int t = 0; t < 8; ++t) {
        uint32_t a[4];
        ldsm_x4_trans(v_row + (t >> 2) * KV_BOX + ((((t & 3) * 32) + v_off) ^ v_xor), a);
        mma_16816(acc[t], a, b0, b1);
      }
    }
    __syncwarp();
    if (c.lane == 0) mbar_arrive_n(c.empty(idx % NSLOTS), EMPTY_UNITS);
    if (pass_gate) cons_sync();
  }
  c.chunk += static_cast<uint32_t>(it.nchunks);
  QMK_FINE(63);
  // (3) this warp's partial state -> shared memory: lanes of quad h hold head h (columns hi, lo)
  if (quad < 2) {
    float *wp = s_wpart + (c.warp * 2 + quad) * PART_STRIDE;
#pragma unroll
    for (int t = 0; t < 8; ++t) {
      wp[t * 16 + rowq] = fmaf(acc[t][1], LO_INV, acc[t][0]);
      wp[t * 16 + rowq + 8] = fmaf(acc[t][3], LO_INV, acc[t][2]);
    }
    if (rowq == 0) { wp[D] = m; wp[D + 1] = l; }
  }
  QMK_FINE(64);
  cons_sync();
  QMK_FINE(65);
  // (4) merge the warps (+ the new row).  First the 2 x 13 weights exp2(max_w - max) and the head's (max, sum), by
  // warps 0 and 1 (one head each, lane = contributing warp, lane 12 = the new row); then every (head, dim) is a
  // weighted sum of 13 independent loads (a running max + rescale per thread took 1180 cycles here).
  float *s_scale = c.f(FF_SPLITW);                       // [2][16], free between the merges
  if (c.warp < 2) {
    const int h = c.warp;
    float mw = -INFINITY, lw = 0.f;
    if (c.lane < CONS_WARPS) {
      mw = s_wpart[(c.lane * 2 + h) * PART_STRIDE + D];
      lw = s_wpart[(c.lane * 2 + h) * PART_STRIDE + D + 1];
    } else if (c.lane == CONS_WARPS && owner) {
      mw = s_misc[h];
      lw = 1.f;
    }
    const float M = warp_max(mw);
    const float scw = (mw == -INFINITY) ? 0.f : exp2f(mw - M);
    const float L = warp_sum(lw * scw);
    if (c.lane < 16) s_scale[h * 16 + c.lane] = scw;
    if (c.lane == 0) {
      unsigned long long *part = P.ll + LL_PART + static_cast<size_t>((2 * g + h) * MAX_SPLITS + s) * PART_STRIDE;
      ll_store(part + D, M, tag);
      ll_store(part + D + 1, L, tag);
    }
  }
  cons_sync();
  if (c.tid < 2 * D) {
    const int h = c.tid >> 7, d = c.tid & (D - 1);
    float A = s_vnew[d] * s_scale[h * 16 + CONS_WARPS];   // 0 weight unless this CTA owns the new row
#pragma unroll
    for (int w = 0; w < CONS_WARPS; ++w) A = fmaf(s_wpart[(w * 2 + h) * PART_STRIDE + d], s_scale[h * 16 + w], A);
    ll_store(P.ll + LL_PART + static_cast<size_t>((2 * g + h) * MAX_SPLITS + s) * PART_STRIDE + d, A, tag);
  }
  QMK_FINE(66);
  // New K,V row -> cache (megakernel_5090.cu:392-397), off the critical path.  The fence orders the row before the
  // exchange words this CTA publishes later; readers fence once per step.
  if (owner && (c.warp == 2 || c.warp == 3)) {
    __half *cache = ((c.warp == 2) ? P.k_cache : P.v_cache) + head_base + static_cast<size_t>(pos) * D;
    const float *snew = (c.warp == 2) ? s_knew : s_vnew;
#pragma unroll
    for (int i = 0; i < 4; ++i) cache[c.lane + 32 * i] = __float2half_rn(snew[c.lane + 32 * i]);
    __threadfence();
  }
  return c.chunk;
}

// 1 / sqrt(mean of squares + eps) over the 1024 values whose squares the consumer threads hold in `ss`; one barrier.
// (rsqrt.approx: 2 ulp; the sum's order is fixed.)
__device__ __forceinline__ float block_rstd(const Ctx &c, float ss) {
  ss = warp_sum(ss);
  float *red = c.f(F_RED);
  if (c.lane == 0) red[c.warp] = ss;
  cons_sync();
  const float4 r0 = reinterpret_cast<const float4 *>(red)[0], r1 = reinterpret_cast<const float4 *>(red)[1],
               r2 = reinterpret_cast<const float4 *>(red)[2];
  const float tot = (((r0.x + r0.y) + (r0.z + r0.w)) + ((r1.x + r1.y) + (r1.z + r1.w))) + ((r2.x + r2.y) + (r2.z + r2.w));
  return rsqrtf(tot * (1.0f / H) + RMS_EPS);
}

// fp32 vector value -> residual stream (fp32) and the hi/lo fp16 halves of its RMS-normalised form.
__device__ __forceinline__ void store_normalised(const Ctx &c, int n, float v, float rstd, float w, float *dst) {
  dst[n] = v;
  const float xn = v * rstd * w;
  *reinterpret_cast<__half *>(c.smem + OFF_XF + xf_offset(n, 0)) = split_half(xn, false);
  *reinterpret_cast<__half *>(c.smem + OFF_XF + xf_offset(n, 1)) = split_half(xn, true);
}

// Waits until use number `use` (1-based) of a sum is complete (see megakernel_fused.cuh), writes the 1024 values
// to shared memory (which = 0: x1; 1: x, the next input) and RMS-normalises them with `norm_w` (fp16[1024], shared
// or global) into the hi/lo halves the tile products read.  emit: CTA 0 also writes the reference-signature outputs
// (final-norm result fp32, last hidden state fp16).  Ends with a consumer barrier.
__device__ __noinline__ void red_wait_norm(const Params &P, const Ctx c, int which, uint32_t use, const __half *norm_w, int emit) {
  constexpr int PT = (H + CONS_THREADS - 1) / CONS_THREADS;
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
    {
      // one lane per warp watches one word until it is complete, then the warp fetches its words: 32x fewer polls
      // hitting the lines the adds are draining into, at the price of one more L2 round trip at the end (measured at
      // 4096-token context: 1714 -> 1784 tok/s; one lane per CTA + a barrier: the same; a pause between polls: slower)
      if (c.lane == 0) {
        uint32_t n = 0;
        while (((ll_load(src) - base) & RED_CNT_MASK) != 0ull) {
          if ((++n & 1023u) == 0u && (c.flags()[0] || ld_relaxed_u32(P.status) != 0u)) break;   // the full wait below reports time-outs
          if (n > (1u << 22)) break;
        }
      }
      __syncwarp();
    }
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
  float v[PT], ss = 0.f;
#pragma unroll
  for (int j = 0; j < PT; ++j) {
    v[j] = (valid & (1u << j)) ? static_cast<float>(vi[j]) * RED_INV_SCALE : 0.f;
    ss = fmaf(v[j], v[j], ss);
  }
  const float rstd = block_rstd(c, ss);
#pragma unroll
  for (int j = 0; j < PT; ++j)
    if (valid & (1u << j)) {
      const int n = c.tid + j * CONS_THREADS;
      const float w = __half2float(norm_w[n]);
      store_normalised(c, n, v[j], rstd, w, dst);
      if (emit && c.cta == 0) {
        if (P.normalized_out) P.normalized_out[n] = v[j] * rstd * w;
        if (P.hidden_out) P.hidden_out[n] = __float2half_rn(v[j]);
      }
    }
  cons_sync();
  QMK_FINE(which ? 46 : 42);
}

// Embedding row of `token` (megakernel_5090.cu:825-830) -> residual stream, normalised with layer 0's input norm.
__device__ __noinline__ void embed_norm(const Params &P, const Ctx c, int token, const __half *norm_w) {
  constexpr int PT = (H + CONS_THREADS - 1) / CONS_THREADS;
  const __half *erow = P.embed + static_cast<size_t>(token) * H;
  float v[PT], ss = 0.f;
#pragma unroll
  for (int j = 0; j < PT; ++j) {
    const int n = c.tid + j * CONS_THREADS;
    v[j] = n < H ? __half2float(__ldg(erow + n)) : 0.f;
    ss = fmaf(v[j], v[j], ss);
  }
  const float rstd = block_rstd(c, ss);
#pragma unroll
  for (int j = 0; j < PT; ++j) {
    const int n = c.tid + j * CONS_THREADS;
    if (n < H) store_normalised(c, n, v[j], rstd, __half2float(norm_w[n]), c.f(F_X));
  }
  cons_sync();
}

// Split-K slice of the O (which = 0) or down (1) projection (see slice_colgemv of megakernel_fused.cuh) on the
// tensor cores: partial[n] = sum_i act[i] * Wt[first + i][n] with the K-major rows as the A operand read through
// ldmatrix.trans (tile = 16 outputs x 16 rows, at most two k-steps: slices of at most 32 rows), the slice's
// activations as B (hi / lo columns, from act16).  Warp w takes output tiles w, w + 12, ... over ALL rows of the
// slice, so a partial is complete when it leaves the warp: after each pair of tiles the 32 sums are spread over
// the 32 lanes (four shuffles) and every lane adds its one output into the residual sum - no staging in shared
// memory, no barrier, and the adds of early tiles drain while later tiles are computed.
__device__ __noinline__ uint32_t slice_cols(const Params &P, Ctx c, int which) {
  const SegTab *t = c.segs();
  const int nrows = which ? tctab(c)->ng * CH_ROWS : t->e1 - t->e0;
  const float *resid = c.f(which ? F_X1 : F_X);
  float *prev = c.f(FF_PREV) + (which ? H : 0);
  unsigned long long *mine = P.red + (which ? RED_X2 : RED_X1) + (c.cta % P.red_copies) * H;
  const int nch = (nrows + CH_ROWS - 1) / CH_ROWS;
  const bool two = nrows > 16;
  [[maybe_unused]] const int fb = which ? 30 : 20;
  QMK_FINE(fb + 0);
  bool ok = true;
  if (c.lane < nch) {
    const uint32_t idx = c.chunk + static_cast<uint32_t>(c.lane);
    ok = mbar_wait(P, c, c.full(idx % NSLOTS), (idx / NSLOTS) & 1u, WHERE_FULL, false);
  }
  ok = __all_sync(0xffffffffu, ok);
  if (ok) {
    // B: the slice's activations; row n of B^T = hi (even n) / lo (odd n) vector; one ldmatrix.x4 = two k-steps
    uint32_t bq[4];
    ldsm_x4(smem_u32(c.smem + OFF_ACT16) + (c.lane & 1) * (ACT16_PITCH * 2) + (c.lane >> 3) * 16, bq);
    // A: this lane's row of each k-step (rows past the slice repeat row 0: their activations are zero)
    uint32_t arow[2];
#pragma unroll
    for (int ks = 0; ks < 2; ++ks) {
      int row = ks * 16 + (c.lane & 7) + 8 * (c.lane >> 4);
      if (row >= nrows) row = 0;
      arow[ks] = weight_rows(c, c.chunk + static_cast<uint32_t>(row >> 2)) + (row & 3) * ROW_PITCH + ((c.lane >> 3) & 1) * 16;
    }
    const int n0 = t->n0, n1 = t->n1;
    const int src = (c.lane & 7) * 4;                 // lane that holds this lane's output row (fragment row = lane / 4)
#pragma unroll 1
    for (int t0 = c.warp; t0 < H / 16; t0 += 2 * CONS_WARPS) {
      float acc[2][4];
      uint32_t a[2][4], a2[2][4];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int tile = min(t0 + u * CONS_WARPS, H / 16 - 1);   // past the end: repeat a valid tile, not added
        acc[u][0] = 0.f; acc[u][1] = 0.f; acc[u][2] = 0.f; acc[u][3] = 0.f;
        ldsm_x4_trans(arow[0] + tile * 32, a[u]);
        if (two) ldsm_x4_trans(arow[1] + tile * 32, a2[u]);
      }
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        mma_16816(acc[u], a[u], bq[0], bq[1]);
        if (two) mma_16816(acc[u], a2[u], bq[2], bq[3]);
      }
      // lanes of quad 0 hold (hi, lo) sums of rows lane / 4 and lane / 4 + 8 of both tiles; lane L takes output
      // L % 16 of tile L / 16
      const float s0 = __shfl_sync(0xffffffffu, fmaf(acc[0][1], LO_INV, acc[0][0]), src);
      const float s1 = __shfl_sync(0xffffffffu, fmaf(acc[0][3], LO_INV, acc[0][2]), src);
      const float s2 = __shfl_sync(0xffffffffu, fmaf(acc[1][1], LO_INV, acc[1][0]), src);
      const float s3 = __shfl_sync(0xffffffffu, fmaf(acc[1][3], LO_INV, acc[1][2]), src);
      const int tile = t0 + (c.lane >> 4) * CONS_WARPS;
      if (tile < H / 16) {
        const int n = tile * 16 + (c.lane & 15);
        float v = (c.lane & 16) ? ((c.lane & 8) ? s3 : s2) : ((c.lane & 8) ? s1 : s0);
        if (n >= n0 && n < n1) v += resid[n];
        const long long fx = __float2ll_rn(v * RED_SCALE), fx_prev = __float2ll_rn(prev[n] * RED_SCALE);
        prev[n] = v;
        red_add_u64(mine + n, (static_cast<unsigned long long>(fx - fx_prev) << RED_CNT_BITS) + 1ull);
      }
    }
  }
  __syncwarp();
  if (c.lane < nch) mbar_arrive_n(c.empty((c.chunk + static_cast<uint32_t>(c.lane)) % NSLOTS), EMPTY_UNITS / CONS_WARPS);
  QMK_FINE(fb + 3);
  return c.chunk + static_cast<uint32_t>(nch);
}

// Tied LM head + per-CTA argmax (megakernel_5090.cu:1024-1132).  One 16-row tile per round, its 1024 inputs split
// over the twelve warps; the partial sums go through a double-buffered shared array, so one barrier per round;
// threads 0..15 finish one row each and keep a running (max, lowest index).  A round consumes four of the ring's
// twenty chunks, which leaves sixteen in flight (the stream needs bandwidth x latency = ~130 KB per SM in flight;
// rounds of three tiles left eight and ran at 3.4 TB/s).  Leaves the per-warp results that argmax_exchange()
// expects in s_misc[32..43] / s_misc[48..59].
__device__ __noinline__ uint32_t lm_head_tc(const Params &P, Ctx c, float *dump) {
  const TcTab *t = tctab(c);
  const int nch = t->nlm, ntiles = (nch + 3) >> 2;
  float *part = tc_part(c), *s_misc = c.f(F_MISC);
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  const int p0 = (KPAIRS * c.warp) / CONS_WARPS, p1 = (KPAIRS * (c.warp + 1)) / CONS_WARPS;
#pragma unroll 1
  for (int tile = 0; tile < ntiles; ++tile) {
    float *pr = part + (tile & 1) * (CONS_WARPS * 16);
    tile_task(P, c, c.chunk + static_cast<uint32_t>(tile * 4), min(16, (nch - tile * 4) * CH_ROWS), p0, p1, pr + c.warp * 16,
              EMPTY_UNITS / CONS_WARPS);
    cons_sync();
    if (c.tid < 16) {
      const int row = tile * 16 + c.tid;
      if (row < nch * CH_ROWS) {
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < CONS_WARPS; ++w) v += pr[w * 16 + c.tid];
        const int o = t->lm0 * CH_ROWS + row;
        if (v > best) { best = v; best_i = o; }     // rows ascend per thread: strict > keeps the lowest index
        if (dump) dump[o] = v;
      }
    }
  }
  if (c.warp == 0) {   // threads 0..15 hold candidates
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
      if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
  }
  if (c.lane == 0) {
    s_misc[32 + c.warp] = c.warp == 0 ? best : -INFINITY;
    s_misc[48 + c.warp] = __int_as_float(c.warp == 0 ? best_i : 0x7fffffff);
  }
  return c.chunk + static_cast<uint32_t>(nch);
}

// ----------------------------------------------------------------------------- producer (one warp)
// The warp issues eight chunks at a time: lanes 4g..4g+3 own chunk g of the group of eight, lane 4g waits for
// the slot and announces the bytes, lane 4g + r copies row r (one cp.async.bulk per row, 2064-byte pitch).  Per
// chunk, wait + announce + copy are ~800 cycles of dependent latency; one chunk at a time capped the stream at
// 19 GB/s per SM (LM head 2.8 TB/s), eight at a time keep that latency off the stream.
// A layer's chunks in ring order: q|k|v rows, this CTA's old K/V rows, K-major O rows [e0, e1), gate rows, up
// rows, K-major down rows; after the last layer the LM-head rows.
// kv_row >= 0 marks a cache chunk: 16 rows of the K and of the V cache from that row on (rows of the caches seen as
// [layers * 8 * max_seq_len][128]); lane r of the group copies box r (K low dims, K high dims, V low, V high).
struct ChunkSrc { const unsigned char *src; size_t src_pitch; uint32_t rows, row_bytes, dst_pitch; int kv_row; };

__device__ __forceinline__ bool tc_issue8(const Params &P, const Ctx &c, uint32_t ci, bool active, const ChunkSrc &d, uint64_t pol) {
  if (__any_sync(0xffffffffu, (c.flags()[0] | c.flags()[1]) != 0)) return false;   // the warp leaves as a whole
  const uint32_t slot = ci % NSLOTS;
  bool ok = true;
  if (active && ci >= NSLOTS) ok = mbar_wait(P, c, c.empty(slot), ((ci / NSLOTS) - 1u) & 1u, WHERE_EMPTY, true);
  if (!__all_sync(0xffffffffu, ok)) return false;
  const int sub = c.lane & 3;
  if (active && sub == 0) mbar_arrive_expect_tx(c.full(slot), d.kv_row >= 0 ? 4u * KV_BOX : d.rows * d.row_bytes);
  __syncwarp();
  if (active && d.kv_row >= 0) {
    tma_box_2d(smem_u32(c.slot(ci)) + sub * KV_BOX, sub < 2 ? static_cast<const void *>(P.kmap) : static_cast<const void *>(P.vmap),
               (sub & 1) * 64, d.kv_row, c.full(slot));
  } else if (active && sub < static_cast<int>(d.rows)) {
    bulk_g2s(c.slot(ci) + (ci & 1u) * ODD_SLOT_SKEW + sub * d.dst_pitch, d.src + sub * d.src_pitch, d.row_bytes, c.full(slot), pol);
  }
  return true;
}
// Four rows of a row-major fp16 matrix with 1024 inputs, starting at `row`.
__device__ __forceinline__ ChunkSrc matrix_chunk(const void *base, int row, int rows) {
  ChunkSrc d;
  d.src = reinterpret_cast<const unsigned char *>(base) + static_cast<size_t>(row) * (2 * H);
  d.src_pitch = 2 * H;
  d.rows = static_cast<uint32_t>(rows);
  d.row_bytes = 2 * H;
  d.dst_pitch = ROW_PITCH;
  d.kv_row = -1;
  return d;
}

__device__ __noinline__ void producer_main_tc(const Params &P, const Ctx c) {
  const uint64_t pol = P.l2_evict_first ? l2_evict_first_policy() : l2_evict_normal_policy();
  const SegTab *t = c.segs();
  const TcTab *tt = tctab(c);
  const int grp = c.lane >> 2;
  const int nq = tt->nq, ng = tt->ng, ne = t->e1 - t->e0, no = (ne + CH_ROWS - 1) / CH_ROWS;
  uint32_t idx = 0, issued = 0;   // first chunk of the current layer / chunks issued so far
  bool ok = true;
#pragma unroll 1
  for (int step = 0; ok && step < P.num_steps; ++step) {
    const AttnItem it = attn_item(P, c, 0, 1, CONS_WARPS, P.start_position + step);
    const int s1 = nq, s2 = s1 + it.nchunks, s3 = s2 + no, s4 = s3 + ng, s5 = s4 + ng, per_layer = s5 + ng;
#pragma unroll 1
    for (int l = 0; ok && l < P.num_layers; ++l) {
      const unsigned long long *rec = c.layer_rec(l);
      const unsigned long long *rect = c.layer_rec_t(l);
      if (c.lane == 0) {   // this layer's norm vectors (see producer_main)
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
      __syncwarp();
#pragma unroll 1
      for (int j0 = 0; ok && j0 < per_layer; j0 += 8) {
        const int j = j0 + grp;
        ChunkSrc d = matrix_chunk(nullptr, 0, 0);
        if (j < s1) {            // q|k|v: a chunk lies in one tensor (2048 and 3072 are multiples of 4)
          const int row = (tt->q0 + j) * CH_ROWS;
          const int sel = row < QS ? 0 : row < QS + KVS ? 1 : 2;
          d = matrix_chunk(reinterpret_cast<const void *>(rec[REC_WQ + sel]), row - (sel == 0 ? 0 : sel == 1 ? QS : QS + KVS), CH_ROWS);
        } else if (j < s2) {     // old K rows (lane 4g) and V rows (lane 4g + 1) of the attention item
          d.kv_row = (l * NKV + it.g) * P.max_seq_len + it.p0 + (j - s1) * it.rpc;
        } else if (j < s3) {
          const int r = (j - s2) * CH_ROWS;
          d = matrix_chunk(reinterpret_cast<const void *>(rect[0]), t->e0 + r, min(CH_ROWS, ne - r));
        } else if (j < s4) {
          d = matrix_chunk(reinterpret_cast<const void *>(rec[REC_GATE]), (tt->g0 + j - s3) * CH_ROWS, CH_ROWS);
        } else if (j < s5) {
          d = matrix_chunk(reinterpret_cast<const void *>(rec[REC_UP]), (tt->g0 + j - s4) * CH_ROWS, CH_ROWS);
        } else if (j < per_layer) {
          d = matrix_chunk(reinterpret_cast<const void *>(rect[1]), (tt->g0 + j - s5) * CH_ROWS, CH_ROWS);
        }
        ok = tc_issue8(P, c, idx + static_cast<uint32_t>(j), j < per_layer, d, pol);   // issues all eight or none
        if (ok) issued = idx + static_cast<uint32_t>(min(j0 + 8, per_layer));
      }
      idx += static_cast<uint32_t>(per_layer);
    }
    if (!P.prefill) {
#pragma unroll 1
      for (int j0 = 0; ok && j0 < tt->nlm; j0 += 8) {
        const int j = j0 + grp;
        const ChunkSrc d = matrix_chunk(P.lm_head, (tt->lm0 + j) * CH_ROWS, CH_ROWS);
        ok = tc_issue8(P, c, idx + static_cast<uint32_t>(j), j < tt->nlm, d, pol);
        if (ok) issued = idx + static_cast<uint32_t>(min(j0 + 8, tt->nlm));
      }
      idx += static_cast<uint32_t>(tt->nlm);
    }
  }
  if (c.lane == 0) c.flags()[2] = static_cast<int>(issued);
}

__global__ void __launch_bounds__(THREADS, 1) qwen3_decode_megakernel_tc(const __grid_constant__ Params P) {
  extern __shared__ __align__(128) unsigned char smem[];
  Ctx c;
  c.smem = smem;
  c.tid = threadIdx.x;
  c.warp = threadIdx.x >> 5;
  c.lane = threadIdx.x & 31;
  c.cta = blockIdx.x;
  c.ncta = gridDim.x;
  c.chunk = 0;
  c.repl = 1;
  c.llr = P.ll;

  if (c.tid == 0) {
    for (int i = 0; i < NSLOTS; ++i) { mbar_init(c.full(i), 1); mbar_init(c.empty(i), EMPTY_UNITS); }
    mbar_init(c.nfull(0), 1);
    mbar_init(c.nfull(1), 1);
    volatile int *fl = c.flags();
    fl[0] = 0; fl[1] = 0; fl[2] = 0; fl[3] = 0; fl[4] = 0; fl[5] = 0; fl[6] = 0; fl[8] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (c.tid == 32) {
    build_segtab(reinterpret_cast<SegTab *>(smem + OFF_SEGS), c.cta, c.ncta, P.vocab);
    TcTab *tt = reinterpret_cast<TcTab *>(smem + OFF_TCTAB);
    int a, b;
    split_rows(QKV_CHUNKS, c.ncta, c.cta, a, b); tt->q0 = a; tt->nq = b - a;
    split_rows(GU_CHUNKS, c.ncta, c.cta, a, b); tt->g0 = a; tt->ng = b - a;
    split_rows(P.vocab / CH_ROWS, c.ncta, c.cta, a, b); tt->lm0 = a; tt->nlm = b - a;
    build_tile_tasks(tt->qkv, &tt->nkb_qkv, 1, tt->nq);
    build_tile_tasks(tt->gu, &tt->nkb_gu, 2, tt->ng);
  }
  {
    const unsigned long long *src = reinterpret_cast<const unsigned long long *>(P.layers);
    unsigned long long *dst = reinterpret_cast<unsigned long long *>(smem + OFF_LAYERS);
    for (int i = c.tid; i < P.num_layers * 12; i += THREADS) dst[i] = src[i];
    const unsigned long long *srct = reinterpret_cast<const unsigned long long *>(P.layers_t);
    unsigned long long *dstt = reinterpret_cast<unsigned long long *>(smem + OFF_LAYERS_T);
    for (int i = c.tid; i < P.num_layers * 2; i += THREADS) dstt[i] = srct[i];
    float *prev = c.f(FF_PREV);
    for (int i = c.tid; i < 2 * H; i += THREADS) prev[i] = 0.f;
  }
  __syncthreads();

  if (c.warp == CONS_WARPS) {
    producer_main_tc(P, c);
    __syncwarp();
  } else {
    float *s_misc = c.f(F_MISC);
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
      {
        const uint32_t L0 = static_cast<uint32_t>(step) * static_cast<uint32_t>(P.num_layers);
        mbar_wait(P, c, c.nfull(L0 & 1u), (L0 >> 1) & 1u, WHERE_FULL, false);
        embed_norm(P, c, token, c.norms(L0 & 1u) + NB_IN_LN);
      }
#pragma unroll 1
      for (int layer = 0; layer < P.num_layers; ++layer) {
        const uint32_t tag = tag_base + static_cast<uint32_t>(layer) + 1u;
        const uint32_t Lg = static_cast<uint32_t>(step) * static_cast<uint32_t>(P.num_layers) + static_cast<uint32_t>(layer);
        const __half *nv = c.norms(Lg & 1u);
        const uint32_t use = Lg + 1u;
#ifdef QMK_FINE_PROF
        if (c.tid == 0) c.flags()[8] = (step == P.num_steps - 1 && layer == 5) ? 1 : 0;
#endif
        QMK_STAMP(layer * 12 + 0);
        c.chunk = qkv_phase(P, c, tag);
        QMK_STAMP(layer * 12 + 1);
        c.chunk = attention_tc(P, c, nv, layer, pos, tag);
        QMK_STAMP(layer * 12 + 2);
        merge_slice(P, c, S_step, tag, reinterpret_cast<__half *>(c.smem + OFF_ACT16));
        QMK_STAMP(layer * 12 + 3);
        cons_sync();
        c.chunk = slice_cols(P, c, 0);
        QMK_STAMP(layer * 12 + 4);
        red_wait_norm(P, c, 0, use, nv + NB_POST_LN, 0);
        QMK_STAMP(layer * 12 + 5);
        c.chunk = gateup_phase(P, c);
        QMK_STAMP(layer * 12 + 6);
        cons_sync();
        c.chunk = slice_cols(P, c, 1);
        QMK_STAMP(layer * 12 + 7);
        const bool last = layer == P.num_layers - 1;
        if (!last) mbar_wait(P, c, c.nfull((Lg + 1u) & 1u), ((Lg + 1u) >> 1) & 1u, WHERE_FULL, false);
        // the next consumer of x: the following layer's input norm, or the final norm before the LM head (a prefill
        // pass ends here: any vector will do)
        const __half *next_norm = !last ? c.norms((Lg + 1u) & 1u) + NB_IN_LN : P.prefill ? nv + NB_IN_LN : P.final_norm;
        red_wait_norm(P, c, 1, use, next_norm, (last && !P.prefill) ? 1 : 0);
        QMK_STAMP(layer * 12 + 8);
        if (cons_any(c.flags()[0] != 0)) break;
      }
      if (cons_any(c.flags()[0] != 0)) break;
      if (P.prefill) {
        if (step + 1 < P.num_steps) token = P.token_ids[step + 1];
        continue;
      }
      QMK_STAMP(P.num_layers * 12 + 0);
      c.chunk = lm_head_tc(P, c, P.logits_out ? P.logits_out + static_cast<size_t>(step) * P.vocab : nullptr);
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

#endif  // QMK_MAX_SEQ == 1 && QMK_TC_BUILD
}  // namespace QMK_NS
