// Device code of the persistent decode megakernel.  Included once per build variant with
//   QMK_NS       namespace of this variant
//   QMK_MAX_SEQ  how many sequences one launch can interleave (sizes the shared-memory activations,
//                and with them the depth of the weight/KV ring)
// See megakernel_sm100.cu for the design notes.
#ifndef QMK_NS
#error "define QMK_NS and QMK_MAX_SEQ before including megakernel_device.cuh"
#endif

namespace QMK_NS {

using qmkp::LayerW;
using qmkp::Params;


constexpr int H = 1024;          // hidden
constexpr int I = 3072;          // MLP intermediate
constexpr int NQ = 16;           // query heads
constexpr int NKV = 8;           // kv heads
constexpr int D = 128;           // head dim
constexpr int QS = NQ * D;       // 2048
constexpr int KVS = NKV * D;     // 1024
constexpr int QKV_ROWS = QS + 2 * KVS;  // 4096
constexpr float RMS_EPS = 1e-6f;

#ifndef QMK_CONS_WARPS
#define QMK_CONS_WARPS 12
#endif
// Math warps per CTA, a multiple of 4 (rows-per-chunk divides it).  12 + the producer warp puts at
// most 4 warps on each SM sub-partition, which allows 128 registers per thread and a spill-free
// kernel; 16 + 1 caps registers at 96 and spills.
constexpr int CONS_WARPS = QMK_CONS_WARPS;
constexpr int CONS_THREADS = CONS_WARPS * 32;   // 384 math threads
constexpr int THREADS = CONS_THREADS + 32;      // + 1 producer warp
// Ring geometry.  The tensor-core build (QMK_TC_BUILD) overrides it: slots hold four weight rows padded to
// 2064 bytes, and a slot is freed by 12 arrival units (1, 2, 3, 4, 6 or 12 warps share a chunk there).
#ifdef QMK_SLOT_BYTES
constexpr int SLOT_BYTES = QMK_SLOT_BYTES;
#else
constexpr int SLOT_BYTES = 8192;
#endif
#ifdef QMK_NSLOTS
constexpr int NSLOTS = QMK_NSLOTS;
#elif QMK_MAX_SEQ == 1
constexpr int NSLOTS = 21;
#else
constexpr int NSLOTS = 13;       // every sequence keeps its own activations in shared memory: a shorter ring
#endif
static_assert(NSLOTS >= CONS_WARPS, "a group of chunks (up to one per warp) must fit in the ring");
#ifdef QMK_EMPTY_UNITS
constexpr int EMPTY_UNITS = QMK_EMPTY_UNITS;
#else
constexpr int EMPTY_UNITS = 4;   // single-sequence build: arrival units that free a ring slot (rows-per-chunk is 4, 2 or 1)
#endif
constexpr int SLOT_HALF = (SLOT_BYTES / 2) & ~15;   // second source of a two-source chunk (V rows, up rows)
constexpr int MAX_SPLITS = 24;   // attention work items per kv head (<= grid / 8)
constexpr int MAX_CTAS = 256;
constexpr int MAX_LAYERS = 48;
constexpr int PART_STRIDE = D + 2;  // acc[128], max, sum
constexpr int PROF_STRIDE = 768;    // timestamp slots per CTA: 12 per layer + 8 for the LM head

// Exchange buffers, in 8-byte words.
constexpr int LL_QKV = 0;
constexpr int LL_ATTN = LL_QKV + QKV_ROWS;
constexpr int LL_X1 = LL_ATTN + QS;
constexpr int LL_INTER = LL_X1 + H;
constexpr int LL_X2 = LL_INTER + I;
constexpr int LL_AMAX = LL_X2 + H;
constexpr int LL_PART = LL_AMAX + 2 * MAX_CTAS;
constexpr int LL_WORDS = LL_PART + NQ * MAX_SPLITS * PART_STRIDE;
constexpr int MAX_REPL = 4;      // the allocated exchange area holds up to 4 copies
// Exchange area layout: [copy][sequence][LL_WORDS]; the single-sequence build has one sequence per copy.
constexpr int LL_REPL_STRIDE = QMK_MAX_SEQ * LL_WORDS;

__constant__ float c_inv_freq[D / 2];

// ----------------------------------------------------------------------------- PTX helpers
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_n(uint64_t *bar, uint32_t n) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(n) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ uint64_t l2_evict_normal_policy() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_normal.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
// Bulk (non-tensor, non-multicast) TMA copy global -> this CTA's shared memory.
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, uint32_t bytes, uint64_t *bar, uint64_t pol) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
      ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(pol)
      : "memory");
}
__device__ __forceinline__ unsigned long long now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void cons_sync() { asm volatile("bar.sync 1, %0;" ::"n"(CONS_THREADS) : "memory"); }

// Consumer barrier that also ORs a predicate over all math threads (same result everywhere).
__device__ __forceinline__ bool cons_any(bool pred) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 q, %1, 0;\n\t"
      "barrier.cta.red.or.pred p, 1, %2, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(r)
      : "r"(static_cast<uint32_t>(pred)), "n"(CONS_THREADS)
      : "memory");
  return r != 0;
}

__device__ __forceinline__ void ll_store(unsigned long long *p, float v, uint32_t tag) {
  unsigned long long w = (static_cast<unsigned long long>(tag) << 32) | __float_as_uint(v);
  asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
// Publishes one exchange word to all `repl` copies of the area.
__device__ __forceinline__ void ll_publish(unsigned long long *p, float v, uint32_t tag, int repl) {
  ll_store(p, v, tag);
  if (repl > 1) {
    ll_store(p + LL_REPL_STRIDE, v, tag);
    if (repl > 2) { ll_store(p + 2 * LL_REPL_STRIDE, v, tag); ll_store(p + 3 * LL_REPL_STRIDE, v, tag); }
  }
}
__device__ __forceinline__ unsigned long long ll_load(const unsigned long long *p) {
  unsigned long long w;
  asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
  return w;
}
__device__ __forceinline__ unsigned int ld_relaxed_u32(const unsigned int *p) {
  unsigned int w;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(w) : "l"(p) : "memory");
  return w;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// ----------------------------------------------------------------------------- per-CTA state
// Everything below is force-inlined into the one kernel and keeps its state in registers or in
// shared memory at fixed offsets.  The kernel must compile to (next to) no stack frame: with 222 KB
// of shared memory carved out, L1 is ~30 KB for 416 threads, so any per-thread local memory
// (escaping structs, dynamically indexed local arrays, spills) turns every touch into an L2
// round trip on the critical path.  build.py reads ptxas' report and fails the build when a decode
// megakernel's frame exceeds 16 bytes (they have 0 to 8).

constexpr size_t SMEM_RING = static_cast<size_t>(NSLOTS) * SLOT_BYTES;
// fp32 regions (offsets in floats from the end of the ring)
#if QMK_MAX_SEQ == 1
constexpr int F_X = 0;                       // residual stream / layer input      [1024]
constexpr int F_X1 = F_X + H;                // residual after attention           [1024]
constexpr int F_VEC = F_X1 + H;              // attention output / MLP activations [3072]
constexpr int F_RED = F_VEC + I;             // block reduction scratch            [32]
constexpr int F_Q = F_RED + 32;              // rotated query heads                [2][128]
constexpr int F_KNEW = F_Q + 2 * D;          // new K row (fp16-rounded)           [128]
constexpr int F_VNEW = F_KNEW + D;           // new V row (fp16-rounded)           [128]
constexpr int F_WPART = F_VNEW + D;          // per-warp attention partials        [12][2][130]
constexpr int F_CS = F_WPART + CONS_WARPS * 2 * PART_STRIDE;  // cos[64], sin[64] of this position
constexpr int F_AMAX = F_CS + 2 * (D / 2);   // argmax partials of all CTAs        [2*256]
constexpr int F_MISC = F_AMAX + 2 * MAX_CTAS;  // [0,1] new-row scores, [16] token, [32..47]/[48..63] warp argmax
constexpr int F_END = F_MISC + 64;
#else
// Multi-sequence build: one block of G_END floats per sequence (= per warp group), then the per-warp
// attention partials of all twelve math warps.
constexpr int G_X = 0;                       // residual stream / layer input      [1024]
constexpr int G_X1 = G_X + H;                // residual after attention           [1024]
constexpr int G_VEC = G_X1 + H;              // attention output / MLP activations [3072]
constexpr int G_AMAX = G_VEC;                // argmax partials of all CTAs [2*256]: the LM head does not use G_VEC
constexpr int G_RED = G_VEC + I;             // group reduction scratch            [32]
constexpr int G_Q = G_RED + 32;              // rotated query heads                [2][128]
constexpr int G_KNEW = G_Q + 2 * D;          // new K row (fp16-rounded)           [128]
constexpr int G_VNEW = G_KNEW + D;           // new V row (fp16-rounded)           [128]
constexpr int G_CS = G_VNEW + D;             // cos[64], sin[64] of this sequence's position
constexpr int G_MISC = G_CS + 2 * (D / 2);   // [0,1] new-row scores, [16] token, [32..47]/[48..63] warp argmax
constexpr int G_END = G_MISC + 64;
constexpr int F_WPART = QMK_MAX_SEQ * G_END; // per-warp attention partials        [12][2][130]
constexpr int F_END = F_WPART + CONS_WARPS * 2 * PART_STRIDE;
static_assert(2 * MAX_CTAS <= I, "argmax partials alias the activation vector");
#endif
constexpr size_t OFF_FULL = SMEM_RING + static_cast<size_t>(F_END) * 4;   // mbarriers: full[NSLOTS]
constexpr size_t OFF_EMPTY = OFF_FULL + NSLOTS * 8;                       //            empty[NSLOTS]
constexpr size_t OFF_NFULL = OFF_EMPTY + NSLOTS * 8;   // mbarriers of the two norm-vector buffers
constexpr size_t OFF_FLAGS = OFF_NFULL + 16;           // int[16]: 0 abort, 1 stop, 2 issued chunks (at exit), 3 consumed chunks,
                                                       // 4/5 norm-buffer fills, 6 issued chunks (running)
constexpr size_t OFF_LAYERS = OFF_FLAGS + 64;          // copy of the layer pointer table, 12 x u64 per layer
// Norm vectors of a layer (fp16): in_ln[1024] | post_ln[1024] | q_norm[128] | k_norm[128]; two buffers,
// layer parity selects one.  The producer copies them in when it starts a layer's weights.
constexpr int NORM_HALVES = 2 * H + 2 * D;
constexpr int NB_IN_LN = 0, NB_POST_LN = H, NB_QNORM = 2 * H, NB_KNORM = 2 * H + D;
constexpr size_t OFF_NORMS = OFF_LAYERS + MAX_LAYERS * sizeof(LayerW);
constexpr size_t OFF_SEGS = OFF_NORMS + 2 * NORM_HALVES * 2;
constexpr int NKIND = 5;
enum Kind { K_QKV = 0, K_O = 1, K_GU = 2, K_DOWN = 3, K_LM = 4 };
// Row slices this CTA owns in every phase, computed once per launch (shared memory).
struct SegTab {
  int nseg[NKIND];
  int tsel[NKIND][3];    // pointer slot within the 12-pointer layer record (K_LM: unused)
  int row0[NKIND][3];    // first row within that tensor
  int nrows[NKIND][3];
  int out0[NKIND][3];    // index of the first output element
  int e0, e1;            // attention outputs this CTA merges when KV is split
  int n0, n1;            // fused kernel: outputs of the hidden vector whose residual this CTA adds into the sums
  int long_phase;        // some projection phase (QKV .. down) has more chunks here than the ring has slots
};
constexpr size_t OFF_LAYERS_T = OFF_SEGS + ((sizeof(SegTab) + 63) / 64) * 64;   // fused kernel: K-major pointers, 2 x u64 per layer
constexpr size_t SMEM_BYTES = OFF_LAYERS_T + MAX_LAYERS * sizeof(qmkp::LayerT);
static_assert((I + CONS_THREADS - 1) / CONS_THREADS <= 8, "poll_vec handles at most 8 words per thread");
static_assert(SMEM_BYTES <= 232448, "over the 227 KB shared-memory limit of one CTA");
static_assert(OFF_FULL % 8 == 0 && OFF_LAYERS % 16 == 0 && OFF_NORMS % 16 == 0, "shared-memory alignment");

struct Ctx {
  int repl;                        // copies of the exchange area (kept in a register for the publish path)
  const unsigned long long *llr;   // the copy of the exchange area this CTA polls
  unsigned char *smem;
  int tid, warp, lane, cta, ncta;
  uint32_t chunk;   // consumer-side running chunk index (uniform over consumer threads)
#if QMK_MAX_SEQ > 1
  // Multi-sequence build: the math warps are split into one group per sequence.
  int seq;                         // sequence (= group) of this warp
  int gw, gwarp, gtid, gthreads;   // warps per group; this warp / thread within its group; threads per group
  unsigned long long *llw;         // copy 0 of this sequence's exchange area (publish target)
  __device__ __forceinline__ float *g(int off) const {
    return reinterpret_cast<float *>(smem + SMEM_RING) + seq * G_END + off;
  }
#endif
  __device__ __forceinline__ float *f(int off) const { return reinterpret_cast<float *>(smem + SMEM_RING) + off; }
  __device__ __forceinline__ uint64_t *full(uint32_t slot) const { return reinterpret_cast<uint64_t *>(smem + OFF_FULL) + slot; }
  __device__ __forceinline__ uint64_t *empty(uint32_t slot) const { return reinterpret_cast<uint64_t *>(smem + OFF_EMPTY) + slot; }
  __device__ __forceinline__ uint64_t *nfull(uint32_t b) const { return reinterpret_cast<uint64_t *>(smem + OFF_NFULL) + b; }
  __device__ __forceinline__ __half *norms(uint32_t b) const { return reinterpret_cast<__half *>(smem + OFF_NORMS) + b * NORM_HALVES; }
  __device__ __forceinline__ volatile int *flags() const { return reinterpret_cast<volatile int *>(smem + OFF_FLAGS); }
  __device__ __forceinline__ const unsigned long long *layer_rec(int l) const {
    return reinterpret_cast<const unsigned long long *>(smem + OFF_LAYERS) + l * 12;
  }
  __device__ __forceinline__ const unsigned long long *layer_rec_t(int l) const {
    return reinterpret_cast<const unsigned long long *>(smem + OFF_LAYERS_T) + l * 2;
  }
  __device__ __forceinline__ const SegTab *segs() const { return reinterpret_cast<const SegTab *>(smem + OFF_SEGS); }
  __device__ __forceinline__ unsigned char *slot(uint32_t idx) const { return smem + static_cast<size_t>(idx % NSLOTS) * SLOT_BYTES; }
};

enum { WHERE_LL = 1, WHERE_FULL = 2, WHERE_EMPTY = 3, WHERE_DRAIN = 4, WHERE_TOKEN = 5 };
// pointer slots of the layer record (megakernel_5090.cu:91-104)
enum { REC_IN_LN = 0, REC_WQ = 1, REC_WK = 2, REC_WV = 3, REC_QNORM = 4, REC_KNORM = 5, REC_WO = 6, REC_POST_LN = 7,
       REC_GATE = 8, REC_UP = 9, REC_DOWN = 10 };

__device__ __forceinline__ void raise_error(const Params &P, const Ctx &c, int code, int where) {
  if (atomicCAS(P.status, 0u, static_cast<unsigned>(code)) == 0u) {
    P.status[1] = static_cast<unsigned>(where);
    P.status[2] = static_cast<unsigned>(c.cta);
  }
  c.flags()[0] = 1;
}

// Wait for an exchange word to carry `tag`.  The fast path is one load; the spin looks at the abort
// flag, the global status and the clock only every 256 polls.  Returns garbage after an abort.
__device__ __forceinline__ unsigned long long ll_spin(const Params &P, const Ctx &c, const unsigned long long *p, uint32_t tag) {
  unsigned long long t0 = 0;
  uint32_t it = 0;
  for (;;) {
    const unsigned long long w = ll_load(p);
    if (static_cast<uint32_t>(w >> 32) == tag) return w;
    if (P.spin_sleep_ns) __nanosleep(P.spin_sleep_ns);
    if ((++it & 255u) == 0u) {
      if (c.flags()[0]) return 0ull;
      if (ld_relaxed_u32(P.status) != 0u) { c.flags()[0] = 1; return 0ull; }
      const unsigned long long t = now_ns();
      if (t0 == 0) t0 = t;
      if (t - t0 > P.timeout_ns) { raise_error(P, c, QMK_ERR_WAIT_TIMEOUT, WHERE_LL); return 0ull; }
    }
  }
}
__device__ __forceinline__ float ll_wait(const Params &P, const Ctx &c, const unsigned long long *p, uint32_t tag) {
  unsigned long long w = ll_load(p);
  if (static_cast<uint32_t>(w >> 32) != tag) w = ll_spin(P, c, p, tag);
  return __uint_as_float(static_cast<uint32_t>(w));
}

// One lane of the warp watches ONE word until it carries `tag`; the warp then goes on to its full wait.  Polls of
// every lane on every word slow the very stores (and adds) they wait for; while most of the wait is spent here,
// the lines see 1/32 of the polls.  Bounded: gives up silently, the full wait that follows reports time-outs.
__device__ __forceinline__ void ll_sentinel(const Params &P, const Ctx &c, const unsigned long long *p, uint32_t tag) {
  if (c.lane == 0) {
    uint32_t n = 0;
    while (static_cast<uint32_t>(ll_load(p) >> 32) != tag) {
      if ((++n & 1023u) == 0u && (c.flags()[0] || ld_relaxed_u32(P.status) != 0u)) break;
      if (n > (1u << 22)) break;
    }
  }
  __syncwarp();
}

// Waits for NW exchange words at once: every pass re-loads ALL words still missing before looking at
// any of them, so the whole set completes one L2 round trip after its last word lands (polling them
// one after the other costs a round trip per word that was stale in the first pass).
// `valid` masks the words this thread really owns.  Values are garbage after an abort.
template <int NW>
__device__ __forceinline__ void ll_wait_many(const Params &P, const Ctx &c, const unsigned long long *const (&p)[NW],
                                             uint32_t valid, uint32_t tag, float (&out)[NW]) {
  unsigned long long w[NW];
#pragma unroll
  for (int j = 0; j < NW; ++j)
    if (valid & (1u << j)) w[j] = ll_load(p[j]);
  uint32_t pending = valid;
  unsigned long long t0 = 0;
  uint32_t it = 0;
  for (;;) {
#pragma unroll
    for (int j = 0; j < NW; ++j)
      if ((pending & (1u << j)) && static_cast<uint32_t>(w[j] >> 32) == tag) pending &= ~(1u << j);
    if (pending == 0u) break;
    if (P.spin_sleep_ns) __nanosleep(P.spin_sleep_ns);
#pragma unroll
    for (int j = 0; j < NW; ++j)
      if (pending & (1u << j)) w[j] = ll_load(p[j]);
    if ((++it & 255u) == 0u) {
      if (c.flags()[0]) break;
      if (ld_relaxed_u32(P.status) != 0u) { c.flags()[0] = 1; break; }
      const unsigned long long t = now_ns();
      if (t0 == 0) t0 = t;
      if (t - t0 > P.timeout_ns) { raise_error(P, c, QMK_ERR_WAIT_TIMEOUT, WHERE_LL); break; }
    }
  }
#pragma unroll
  for (int j = 0; j < NW; ++j) out[j] = __uint_as_float(static_cast<uint32_t>(w[j]));
}

// Wait on an mbarrier phase with the same bounds.  Returns false after an abort (or, for the
// producer, after the consumers said stop).
__device__ __forceinline__ bool mbar_wait(const Params &P, const Ctx &c, uint64_t *bar, uint32_t parity, int where, bool producer) {
  if (mbar_try_wait(bar, parity)) return true;
  unsigned long long t0 = 0;
  uint32_t it = 0;
  for (;;) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++it & 31u) == 0u) {
      if (c.flags()[0]) return false;
      if (producer && c.flags()[1]) return false;
      if (ld_relaxed_u32(P.status) != 0u) { c.flags()[0] = 1; return false; }
      const unsigned long long t = now_ns();
      if (t0 == 0) t0 = t;
      // the producer may legitimately wait as long as any consumer does: 4x budget
      if (t - t0 > (producer ? 4 * P.timeout_ns : P.timeout_ns)) { raise_error(P, c, QMK_ERR_WAIT_TIMEOUT, where); return false; }
    }
  }
}
// Waits until ring chunk `idx` has landed in its slot.  A parity wait can only tell two consecutive
// uses of a slot apart: asked about use n while use n-1 is still in flight, it answers for use n-2 and
// says "complete".  So the wait first makes sure the producer has issued chunk `idx` (flags()[6] counts
// issued chunks): from then on the slot's barrier is in use n and the parity is unambiguous.  Warps
// that jump ahead in the ring (a group skipping another sequence's cache rows) depend on this.
// Only the multi-sequence build needs the counter.  The single-sequence kernel's warps never skip chunks: a
// phase with more chunks than ring slots is walked in passes with a CTA barrier between them (see pass_gate),
// which orders the previous use of every slot before the wait, and its hot loops stay free of the check.
#ifndef QMK_ISSUED_CHECK
#define QMK_ISSUED_CHECK (QMK_MAX_SEQ > 1)
#endif
#ifndef QMK_ISSUED_FENCE
#define QMK_ISSUED_FENCE 1
#endif
// `seen` caches the last value read of the counter (it only grows): the producer usually runs a ring ahead,
// so one read covers the next several chunks.  Callers keep it in a local and start it at 0.
__device__ __forceinline__ bool chunk_wait(const Params &P, const Ctx &c, uint32_t idx, uint32_t &seen) {
  volatile int *fl = c.flags();
  if (QMK_ISSUED_CHECK && seen <= idx) {
    seen = static_cast<uint32_t>(fl[6]);
    if (seen <= idx) {
      unsigned long long t0 = 0;
      uint32_t it = 0;
      for (;;) {
        seen = static_cast<uint32_t>(fl[6]);
        if (seen > idx) break;
        if ((++it & 31u) == 0u) {
          if (fl[0]) return false;
          if (ld_relaxed_u32(P.status) != 0u) { fl[0] = 1; return false; }
          const unsigned long long t = now_ns();
          if (t0 == 0) t0 = t;
          if (t - t0 > P.timeout_ns) { raise_error(P, c, QMK_ERR_WAIT_TIMEOUT, WHERE_FULL); return false; }
        }
      }
    }
  }
  return mbar_wait(P, c, c.full(idx % NSLOTS), (idx / NSLOTS) & 1u, WHERE_FULL, false);
}
// The whole warp takes the same branch afterwards (shuffles follow).
__device__ __forceinline__ bool wait_full(const Params &P, const Ctx &c, uint32_t idx, uint32_t &seen) {
  return __all_sync(0xffffffffu, chunk_wait(P, c, idx, seen));
}

// Rows [r0, r1) of an n-row matrix owned by CTA `cta` of `ncta` (launch-time only: 64-bit divisions).
__host__ __device__ __forceinline__ void split_rows(int n, int ncta, int cta, int &r0, int &r1) {
  r0 = static_cast<int>((static_cast<long long>(n) * cta) / ncta);
  r1 = static_cast<int>((static_cast<long long>(n) * (cta + 1)) / ncta);
}
__device__ __forceinline__ constexpr int kind_k(int kind) { return kind == K_O ? QS : kind == K_DOWN ? I : H; }
// Bytes of one weight row.  fp16: K halves.  fp8: K e4m3 bytes followed by a 16-byte trailer whose first
// four bytes are the row's fp32 scale (the trailer keeps rows 16-byte aligned for bulk copies and brings
// the scale into shared memory with the row).
constexpr int FP8_TRAILER = 16;
__device__ __forceinline__ constexpr int kind_row_bytes(int kind, int wfmt) {
  return wfmt ? kind_k(kind) + FP8_TRAILER : kind_k(kind) * 2;
}
__host__ __device__ __forceinline__ constexpr int kind_rpc(int kind) { return (kind == K_QKV || kind == K_LM) ? 4 : kind == K_DOWN ? 1 : 2; }

// Thread 0, once per launch.
__host__ __device__ inline void build_segtab(SegTab *t, int cta, int ncta, int vocab) {
  int r0, r1;
  for (int k = 0; k < NKIND; ++k) t->nseg[k] = 0;
  split_rows(QKV_ROWS, ncta, cta, r0, r1);
  const int lo[3] = {0, QS, QS + KVS}, hi[3] = {QS, QS + KVS, QKV_ROWS};
  for (int i = 0; i < 3; ++i) {
    const int a = max(r0, lo[i]), b = min(r1, hi[i]);
    if (a < b) {
      const int n = t->nseg[K_QKV]++;
      t->tsel[K_QKV][n] = REC_WQ + i; t->row0[K_QKV][n] = a - lo[i]; t->nrows[K_QKV][n] = b - a; t->out0[K_QKV][n] = a;
    }
  }
  const int rows[NKIND] = {0, H, I, H, vocab};
  const int rec[NKIND] = {0, REC_WO, REC_GATE, REC_DOWN, 0};
  for (int k = K_O; k <= K_LM; ++k) {
    split_rows(rows[k], ncta, cta, r0, r1);
    if (r0 < r1) { t->nseg[k] = 1; t->tsel[k][0] = rec[k]; t->row0[k][0] = r0; t->nrows[k][0] = r1 - r0; t->out0[k][0] = r0; }
  }
  split_rows(QS, ncta, cta, t->e0, t->e1);
  split_rows(H, ncta, cta, t->n0, t->n1);
  t->long_phase = 0;
  for (int k = K_QKV; k <= K_DOWN; ++k) {
    const int rpc = kind_rpc(k);
    int chunks = 0;
    for (int s = 0; s < t->nseg[k]; ++s) chunks += (t->nrows[k][s] + rpc - 1) / rpc;
    if (chunks > NSLOTS) t->long_phase = 1;
  }
}

// Weight rows of segment s of phase `kind` (layer record `rec` in shared memory, or the LM head).
__device__ __forceinline__ const unsigned char *seg_src(const SegTab *t, int kind, int s, const unsigned long long *rec,
                                                        const __half *lm_head, int which_up, int wfmt) {
  const unsigned long long base = (kind == K_LM) ? reinterpret_cast<unsigned long long>(lm_head)
                                                 : rec[t->tsel[kind][s] + which_up];
  return reinterpret_cast<const unsigned char *>(base) + static_cast<size_t>(t->row0[kind][s]) * kind_row_bytes(kind, wfmt);
}

// Attention work item of this CTA at position `pos`: kv head g, split s of S, old cache rows [p0, p1).
// Both the producer (to stream the rows) and the consumers (to use them) call this.
constexpr int KV_ROWS_PER_CHUNK = 16;   // at most 16 K rows (4 KB) + 16 V rows (4 KB) per ring slot
struct AttnItem { int S, g, s, p0, p1, nchunks, rpc; bool active; };
// Entry b of a per-sequence launch-parameter array.  Written as selects on purpose: indexing a kernel
// parameter array with a run-time value makes the compiler copy the array to the thread's stack.
template <typename T>
__device__ __forceinline__ T per_seq(const T (&arr)[qmkp::MAX_SEQ], int b) {
  static_assert(qmkp::MAX_SEQ == 4, "written out for four entries");
  return b == 0 ? arr[0] : b == 1 ? arr[1] : b == 2 ? arr[2] : arr[3];
}
// `b` of `nseq` sequences: each sequence's items start at a different CTA so that short contexts (few
// items per sequence) land on different SMs.  `gw` = math warps that share the item's rows.
__device__ __forceinline__ AttnItem attn_item(const Params &P, const Ctx &c, int b, int nseq, int gw, int pos) {
  AttnItem it;
  const int S_max = min(MAX_SPLITS, max(1, c.ncta / NKV));
  it.S = max(1, min(pos / max(1, P.split_len), S_max));
  int local = c.cta;
  if (nseq > 1) {
    local -= (b * c.ncta) / nseq;
    if (local < 0) local += c.ncta;
  }
  it.active = local < NKV * it.S;
  it.g = local % NKV;
  it.s = local / NKV;
  // old rows [p0, p1) of [0, pos); pos * S < 2^31, 32-bit division
  it.p0 = it.active ? static_cast<int>(static_cast<unsigned>(pos * it.s) / static_cast<unsigned>(it.S)) : 0;
  it.p1 = it.active ? static_cast<int>(static_cast<unsigned>(pos * (it.s + 1)) / static_cast<unsigned>(it.S)) : 0;
  // Rows per chunk chosen so that every warp gets the same number of (equally long) chunks: with a fixed
  // 16 rows per chunk, 15 chunks over 12 warps left three warps with twice the work of the others.
  const int rows = it.p1 - it.p0;
  const int rounds = max(1, (rows + gw * KV_ROWS_PER_CHUNK - 1) / (gw * KV_ROWS_PER_CHUNK));
  it.rpc = min(KV_ROWS_PER_CHUNK, max(1, (rows + gw * rounds - 1) / (gw * rounds)));
#ifdef QMK_TC_BUILD
  it.rpc = KV_ROWS_PER_CHUNK;   // tensor-core build: a chunk is one 16-row MMA tile
#endif
  it.nchunks = (rows + it.rpc - 1) / it.rpc;
  return it;
}

// Debug build only (-DQMK_FINE_PROF): cycle stamps inside the phases of ONE layer (flags()[8] != 0 marks it),
// written by thread 0 to slots 400 + i of its CTA's profile row.
#ifdef QMK_FINE_PROF
#define QMK_FINE(i)                                                                               \
  do {                                                                                            \
    if (P.prof && c.tid == 0 && c.flags()[8])                                                     \
      P.prof[static_cast<size_t>(c.cta) * PROF_STRIDE + 400 + (i)] = static_cast<unsigned long long>(clock64()); \
  } while (0)
#else
#define QMK_FINE(i) do { } while (0)
#endif

// ----------------------------------------------------------------------------- producer (one thread)
__device__ __forceinline__ bool produce_chunk(const Params &P, const Ctx &c, uint32_t &idx, uint64_t pol,
                                              const unsigned char *src, const unsigned char *src2, uint32_t bytes,
                                              int inflight) {
  const uint32_t slot = idx % NSLOTS;
  if (c.flags()[0] | c.flags()[1]) return false;
  if (idx >= NSLOTS && !mbar_wait(P, c, c.empty(slot), ((idx / NSLOTS) - 1u) & 1u, WHERE_EMPTY, true)) return false;
  if (inflight > 0 && idx >= static_cast<uint32_t>(inflight)) {   // pacing: chunk idx - inflight must have landed
    const uint32_t prev = idx - static_cast<uint32_t>(inflight);
    if (!mbar_wait(P, c, c.full(prev % NSLOTS), (prev / NSLOTS) & 1u, WHERE_EMPTY, true)) return false;
  }
  unsigned char *dst = c.slot(idx);
  mbar_arrive_expect_tx(c.full(slot), src2 ? 2 * bytes : bytes);
  bulk_g2s(dst, src, bytes, c.full(slot), pol);
  if (src2) bulk_g2s(dst + SLOT_HALF, src2, bytes, c.full(slot), pol);
  ++idx;
#if QMK_ISSUED_CHECK
#if QMK_ISSUED_FENCE
  __threadfence_block();          // the barrier's new use is visible before the count that announces it
#endif
  c.flags()[6] = static_cast<int>(idx);
#endif
  return true;
}

__device__ __forceinline__ bool produce_phase(const Params &P, const Ctx &c, uint32_t &idx, uint64_t pol, int kind,
                                              const unsigned long long *rec) {
  const SegTab *t = c.segs();
  const int rb = kind_row_bytes(kind, P.wfmt), rpc = kind_rpc(kind);
  const int n = t->nseg[kind];
  for (int s = 0; s < n; ++s) {
    const unsigned char *src = seg_src(t, kind, s, rec, P.lm_head, 0, P.wfmt);
    const unsigned char *src2 = (kind == K_GU) ? seg_src(t, kind, s, rec, P.lm_head, 1, P.wfmt) : nullptr;
    const int nrows = t->nrows[kind][s];
#pragma unroll 1
    for (int r = 0; r < nrows; r += rpc) {
      const int nr = min(rpc, nrows - r);
      const size_t off = static_cast<size_t>(r) * rb;
      if (!produce_chunk(P, c, idx, pol, src + off, src2 ? src2 + off : nullptr, static_cast<uint32_t>(nr * rb),
                         kind == K_LM ? 0 : P.stream_inflight))
        return false;
    }
  }
  return true;
}

#ifndef QMK_PRODUCER_INLINE
#define QMK_PRODUCER_INLINE 0
#endif
#if QMK_PRODUCER_INLINE
__device__ __forceinline__
#else
// Not inlined: inside the kernel its loops raise the register pressure of the consumer path (kernel-level spills).
__device__ __noinline__
#endif
void producer_main(const Params &P, const Ctx c) {
  const uint64_t pol = P.l2_evict_first ? l2_evict_first_policy() : l2_evict_normal_policy();
  uint32_t idx = 0;
  bool ok = true;
  const int nseq = (QMK_MAX_SEQ > 1) ? P.nseq : 1;
#pragma unroll 1
  for (int step = 0; ok && step < P.num_steps; ++step) {
#pragma unroll 1
    for (int l = 0; ok && l < P.num_layers; ++l) {
      const unsigned long long *rec = c.layer_rec(l);
      {  // this layer's norm vectors -> shared memory.  The buffer of layer L-2 is free: the ring holds fewer
         // chunks than one layer has, so the math is at least in layer L-1 when this point is reached.
        const uint32_t L = static_cast<uint32_t>(step) * static_cast<uint32_t>(P.num_layers) + static_cast<uint32_t>(l);
        const uint32_t b = L & 1u;
        __half *dst = c.norms(b);
        c.flags()[4 + b] = static_cast<int>(L + 1u);   // for the exit drain
        mbar_arrive_expect_tx(c.nfull(b), NORM_HALVES * 2);
        bulk_g2s(dst + NB_IN_LN, reinterpret_cast<const void *>(rec[REC_IN_LN]), H * 2, c.nfull(b), l2_evict_normal_policy());
        bulk_g2s(dst + NB_POST_LN, reinterpret_cast<const void *>(rec[REC_POST_LN]), H * 2, c.nfull(b), l2_evict_normal_policy());
        bulk_g2s(dst + NB_QNORM, reinterpret_cast<const void *>(rec[REC_QNORM]), D * 2, c.nfull(b), l2_evict_normal_policy());
        bulk_g2s(dst + NB_KNORM, reinterpret_cast<const void *>(rec[REC_KNORM]), D * 2, c.nfull(b), l2_evict_normal_policy());
      }
      ok = produce_phase(P, c, idx, pol, K_QKV, rec);
#pragma unroll 1
      for (int b = 0; ok && b < nseq; ++b) {  // this CTA's range of old K/V rows of each sequence's attention item
        const AttnItem it = attn_item(P, c, b, nseq, CONS_WARPS / nseq, per_seq(P.start_positions, b) + step);
        const size_t head_base = (static_cast<size_t>(l) * NKV + it.g) * static_cast<size_t>(P.max_seq_len) * D;
#pragma unroll 1
        for (int r = it.p0; ok && r < it.p1; r += it.rpc) {
          const uint32_t bytes = static_cast<uint32_t>(min(it.rpc, it.p1 - r)) * D * 2;
          const size_t off = (head_base + static_cast<size_t>(r) * D) * 2;
          ok = produce_chunk(P, c, idx, pol, reinterpret_cast<const unsigned char *>(per_seq(P.k_caches, b)) + off,
                             reinterpret_cast<const unsigned char *>(per_seq(P.v_caches, b)) + off, bytes, P.stream_inflight);
        }
      }
#pragma unroll 1
      for (int kind = K_O; ok && kind <= K_DOWN; ++kind) ok = produce_phase(P, c, idx, pol, kind, rec);
    }
    if (ok && !P.prefill) ok = produce_phase(P, c, idx, pol, K_LM, nullptr);
  }
  c.flags()[2] = static_cast<int>(idx);
}

// ----------------------------------------------------------------------------- consumer math
// Eight consecutive weights of a row in shared memory as fp32: `idx8` counts groups of eight.
__device__ __forceinline__ void load_w8(const unsigned char *row, int idx8, int wfmt, float (&w)[8]) {
  if (wfmt == 0) {
    const uint4 v = reinterpret_cast<const uint4 *>(row)[idx8];
    const __half2 *h = reinterpret_cast<const __half2 *>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __half22float2(h[i]);
      w[2 * i] = f.x;
      w[2 * i + 1] = f.y;
    }
  } else {
    const uint2 v = reinterpret_cast<const uint2 *>(row)[idx8];
    const unsigned short *p = reinterpret_cast<const unsigned short *>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(p[i]), __NV_E4M3);
      const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&hr));
      w[2 * i] = f.x;
      w[2 * i + 1] = f.y;
    }
  }
}
// Packed FMAs pay in the multi-sequence build, where the row products are the limit (3 sequences 1879 -> 1924 tok/s,
// 4 sequences with FP8 rows 2143 -> 2234); the single-sequence kernel measured the same within its run-to-run spread.
#ifndef QMK_PACKED_FMA
#define QMK_PACKED_FMA (QMK_MAX_SEQ > 1)
#endif
// acc + sum w[i] a[i].  Packed form: four fma.rn.f32x2 (even and odd terms accumulate in the two halves of a
// register pair) and one add instead of eight scalar FMAs; the order of the sum is fixed either way.
__device__ __forceinline__ float dot8f(const float (&w)[8], const float *a, float acc) {
#if QMK_PACKED_FMA
  float2 s2 = make_float2(acc, 0.f);
#pragma unroll
  for (int i = 0; i < 4; ++i) s2 = __ffma2_rn(make_float2(w[2 * i], w[2 * i + 1]), make_float2(a[2 * i], a[2 * i + 1]), s2);
  return s2.x + s2.y;
#else
#pragma unroll
  for (int i = 0; i < 8; ++i) acc = fmaf(w[i], a[i], acc);
  return acc;
#endif
}
// fp32 scale of an fp8 row (1 for fp16 rows): first word of the trailer behind the K weights
__device__ __forceinline__ float row_scale(const unsigned char *row, int k, int wfmt) {
  return wfmt ? *reinterpret_cast<const float *>(row + k) : 1.0f;
}
__device__ __forceinline__ float dot8(const uint4 w, const float *a, float acc) {
  const __half2 *h = reinterpret_cast<const __half2 *>(&w);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __half22float2(h[i]);
    acc = fmaf(f.x, a[2 * i], acc);
    acc = fmaf(f.y, a[2 * i + 1], acc);
  }
  return acc;
}
// Sums four per-lane values over the warp with 6 shuffles instead of 20: lanes trade halves of their
// value set (xor 16, xor 8) and then finish one value each (xor 4, 2, 1).  Afterwards every lane with
// (lane >> 3) == r holds the complete sum of value r.  The tree is fixed, so results are deterministic.
__device__ __forceinline__ float warp_reduce_scatter4(float v0, float v1, float v2, float v3, int lane) {
  const bool hi16 = (lane & 16) != 0;
  // keep values {0,1} in lanes 0..15 and {2,3} in lanes 16..31
  float k0 = hi16 ? v2 : v0, k1 = hi16 ? v3 : v1;
  const float s0 = hi16 ? v0 : v2, s1 = hi16 ? v1 : v3;
  k0 += __shfl_xor_sync(0xffffffffu, s0, 16);
  k1 += __shfl_xor_sync(0xffffffffu, s1, 16);
  const bool hi8 = (lane & 8) != 0;
  float k = hi8 ? k1 : k0;
  const float sd = hi8 ? k0 : k1;
  k += __shfl_xor_sync(0xffffffffu, sd, 8);
  k += __shfl_xor_sync(0xffffffffu, k, 4);
  k += __shfl_xor_sync(0xffffffffu, k, 2);
  k += __shfl_xor_sync(0xffffffffu, k, 1);
  return k;
}

// RMSNorm of the fp32 vector x in shared memory (`ss` = this thread's share of sum x^2) into
// per-lane registers: a[j*8+i] = x[k] * rstd * w[k], k = j*256 + lane*8 + i.
__device__ __forceinline__ void norm_apply(const Ctx &c, const float *x, float tot, const __half *norm_w, float (&a)[32]) {
  uint4 wn[4];
  // The norm weights are loaded after the barrier of the sum on purpose: issued before it (while the
  // CTA is still polling exchange words) the same loads measured ~100 us/token slower.
#pragma unroll
  for (int j = 0; j < 4; ++j) wn[j] = *reinterpret_cast<const uint4 *>(norm_w + j * 256 + c.lane * 8);
  const float rstd = 1.0f / sqrtf(tot * (1.0f / H) + RMS_EPS);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int k = j * 256 + c.lane * 8;
    const float4 x0 = *reinterpret_cast<const float4 *>(x + k);
    const float4 x1 = *reinterpret_cast<const float4 *>(x + k + 4);
    const float xs[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
    const __half2 *h = reinterpret_cast<const __half2 *>(&wn[j]);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 wf = __half22float2(h[i]);
      a[j * 8 + 2 * i] = xs[2 * i] * rstd * wf.x;
      a[j * 8 + 2 * i + 1] = xs[2 * i + 1] * rstd * wf.y;
    }
  }
}

// This CTA's rows of one projection, streamed through the ring.  Warp w takes row (w % RPC) of chunk
// (w / RPC) of each group of CONS_WARPS/RPC chunks; NB groups are handled per pass so that a warp
// loads, multiplies and reduces all its rows of a layer phase together (one pass per layer phase), and
// hands each slot back when its row is done.
//   K_QKV : out[row] = W.a                       K_GU  : out[row] = silu(Wg.a) * (Wu.a)
//   K_O / K_DOWN : out[row] = W.act + resid[row] (activations in shared memory)
//   K_LM  : running (max, argmax) in best / best_i, optional logits dump
__device__ __forceinline__ float row_partial_regs(const unsigned char *row, const float (&a)[32], int lane, int wfmt) {
  float acc[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float w[8];
    load_w8(row, j * 32 + lane, wfmt, w);
    acc[j] = dot8f(w, &a[j * 8], 0.f);
  }
  // every lane multiplies its partial by the row scale (1 for fp16): the sum over lanes is scaled once
  return ((acc[0] + acc[1]) + (acc[2] + acc[3])) * row_scale(row, H, wfmt);
}
#if QMK_MAX_SEQ == 1
// ----------------------------------------------------------------------------- single-sequence math
// sum over the consumer threads; contains one consumer barrier
__device__ __forceinline__ float block_sum(const Ctx &c, float v) {
  v = warp_sum(v);
  float *red = c.f(F_RED);
  if (c.lane == 0) red[c.warp] = v;
  cons_sync();
  float t = 0.f;
#pragma unroll
  for (int i = 0; i < CONS_WARPS; ++i) t += red[i];
  return t;
}

#ifndef QMK_TC_BUILD
// Polls N exchange words into shared memory as fp32; returns this thread's sum of squares.
// All loads are issued before the first one is looked at.
// One shared (non-inlined) copy: the kernel's per-layer code has to stay small enough for the
// instruction cache, and this routine has five call sites.  Arguments are scalars / by value, so it
// needs no stack.  n <= 8 * CONS_THREADS.
__device__ __noinline__ float poll_vec(const Params &P, const Ctx c, const unsigned long long *buf, int n, uint32_t tag,
                                       float *dst) {
  constexpr int PT = 8;
  const unsigned long long *p[PT];
  uint32_t valid = 0;
#pragma unroll
  for (int j = 0; j < PT; ++j) {
    p[j] = buf + c.tid + j * CONS_THREADS;
    if (c.tid + j * CONS_THREADS < n) valid |= 1u << j;
  }
  float v[PT];
  ll_wait_many<PT>(P, c, p, valid, tag, v);
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < PT; ++j)
    if (valid & (1u << j)) {
      dst[c.tid + j * CONS_THREADS] = v[j];
      ss = fmaf(v[j], v[j], ss);
    }
  return ss;
}

__device__ __forceinline__ void norm_to_regs(const Ctx &c, const float *x, float ss, const __half *norm_w, float (&a)[32]) {
  const float tot = block_sum(c, ss);  // the barrier inside also publishes x
  norm_apply(c, x, tot, norm_w, a);
}

// K = 1024 phases (fused QKV, gate/up, LM head): RMSNorm of x into registers, then this CTA's rows.
// One shared non-inlined copy (runtime `kind`); returns the advanced chunk counter.  For K_LM each warp
// leaves its running (max, argmax) in s_misc[32 + warp] / s_misc[48 + warp].
// GATED: see the comment at the waits below; the barrier inside the pass loop costs ~2.5 % of a decode step
// even when it is never taken, hence a separate copy (and kernel entry point) for grids that need it.
template <bool GATED>
__device__ __noinline__ uint32_t gemv_k1024(const Params &P, Ctx c, int kind, const float *x, float ss,
                                            const __half *norm_w, unsigned long long *out, uint32_t tag, float *dump,
                                            float *local_out = nullptr) {
  const int wfmt = P.wfmt;
  float a[32];
  [[maybe_unused]] const int fb = kind == K_QKV ? 0 : 10;   // (stamp base of the fine-grained profile build)
  QMK_FINE(fb + 0);
  norm_to_regs(c, x, ss, norm_w, a);
  QMK_FINE(fb + 1);
  if (kind == K_LM && c.cta == 0 && c.warp == 0 && (P.normalized_out || P.hidden_out)) {  // reference-signature outputs
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int k = j * 256 + c.lane * 8 + i;
        if (P.normalized_out) P.normalized_out[k] = a[j * 8 + i];
        if (P.hidden_out) P.hidden_out[k] = __float2half_rn(x[k]);
      }
  }
  constexpr int NB = 3;                                 // rows per warp and pass (warp_reduce_scatter4 takes up to 4)
  const int rsh = kind == K_GU ? 1 : 2;                 // log2(rows per chunk)
  const int RPC = 1 << rsh, G = CONS_WARPS >> rsh;
  const SegTab *t = c.segs();
  const int sub = c.warp & (RPC - 1), wch = c.warp >> rsh;
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  const int n = t->nseg[kind];
  // A parity wait is exact only when the slot's previous use (NSLOTS chunks back) has landed: (a) the phase
  // has at most NSLOTS chunks on this CTA, so that use belongs to an earlier phase, which every warp finished
  // before the barrier that opened this one; (b) LM head: one segment, NB * G = 9 chunks per pass and
  // NSLOTS = 2 * 9 + G, so that use is a chunk this very warp consumed two passes ago; (c) otherwise
  // (GATED: reduced grids, where some phase is longer than the ring) a barrier after every pass: a pass
  // has fewer chunks than the ring, so that use lies in an earlier pass.
  static_assert(NSLOTS == 21 && NB * (CONS_WARPS >> 2) == 9, "case (b) above is written for these values");
  static_assert(NB * (CONS_WARPS >> 1) <= NSLOTS, "case (c): a pass must fit the ring");
  const bool pass_gate = GATED && kind != K_LM;
  for (int s = 0; s < n; ++s) {
    const int nrows = t->nrows[kind][s];
    const int out0 = t->out0[kind][s];
    const int nchunks = (nrows + RPC - 1) >> rsh;
#pragma unroll 1
    for (int c0 = 0; c0 < nchunks; c0 += NB * G) {
      float v[NB], u[NB];
      bool valid[NB];
      bool ok = true;
      // one combined wait for the (up to) NB chunks of this warp, then all the math
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        const int ch = c0 + b * G + wch;
        valid[b] = ch < nchunks && ((ch << rsh) + sub) < nrows;          // warp-uniform
        if (valid[b]) {
          const uint32_t idx = c.chunk + static_cast<uint32_t>(ch);
          ok &= mbar_wait(P, c, c.full(idx % NSLOTS), (idx / NSLOTS) & 1u, WHERE_FULL, false);
        }
      }
      ok = __all_sync(0xffffffffu, ok);   // the whole warp takes the same branch (shuffles follow)
      if (kind != K_LM) QMK_FINE(fb + 2);
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        v[b] = 0.f;
        u[b] = 0.f;
        if (valid[b] && ok) {
          const uint32_t idx = c.chunk + static_cast<uint32_t>(c0 + b * G + wch);
          const unsigned char *p = c.slot(idx) + sub * kind_row_bytes(K_QKV, wfmt);
          v[b] = row_partial_regs(p, a, c.lane, wfmt);
          if (kind == K_GU) u[b] = row_partial_regs(p + SLOT_HALF, a, c.lane, wfmt);
        }
      }
      // The rows are in registers now: hand the slots back BEFORE publishing (mbarrier.arrive has
      // release semantics and would otherwise wait for the global stores).  The RPC warps mapped to a
      // chunk each return EMPTY_UNITS/RPC units, whether or not their row exists (a short last chunk).
      if (kind != K_LM) QMK_FINE(fb + 3);
      __syncwarp();
      if (c.lane == 0) {
#pragma unroll
        for (int b = 0; b < NB; ++b) {
          const int ch = c0 + b * G + wch;
          if (ch < nchunks) mbar_arrive_n(c.empty((c.chunk + static_cast<uint32_t>(ch)) % NSLOTS), EMPTY_UNITS >> rsh);
        }
      }
      // lanes 0-7 end up with row b = 0, lanes 8-15 with b = 1, lanes 16-23 with b = 2
      float r = warp_reduce_scatter4(v[0], v[1], v[2], 0.f, c.lane);
      if (kind == K_GU) {
        const float ur = warp_reduce_scatter4(u[0], u[1], u[2], 0.f, c.lane);
        r = r / (1.0f + expf(-r)) * ur;   // SiLU(gate) * up in fp32 (megakernel_5090.cu:681-684 does it in fp16)
      }
      const int mb = c.lane >> 3;                                   // which of the NB rows this lane holds
      const bool mine = ok && (c.lane & 7) == 0 && mb < NB && ((mb == 0 && valid[0]) || (mb == 1 && valid[1]) || (mb == 2 && valid[2]));
      if (mine) {
        const int o = out0 + ((c0 + mb * G + wch) << rsh) + sub;
        if (kind == K_LM) {
          if (r > best || (r == best && o < best_i)) { best = r; best_i = o; }
          if (dump) dump[o] = r;
        } else if (local_out) {
          local_out[o - out0] = r;                                  // fused kernel: the row's result stays in this CTA
        } else {
          ll_publish(out + o, r, tag, c.repl);                      // one store instruction covers the NB rows
        }
      }
      if (pass_gate) cons_sync();
      if (kind != K_LM) QMK_FINE(fb + 4);
    }
    c.chunk += static_cast<uint32_t>(nchunks);
  }
  if (kind == K_LM) {   // lanes 0, 8 and 16 each tracked their own rows
#pragma unroll
    for (int o = 16; o >= 8; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
      if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    if (c.lane == 0) { c.f(F_MISC)[32 + c.warp] = best; c.f(F_MISC)[48 + c.warp] = __int_as_float(best_i); }
  }
  return c.chunk;
}

// O (K = 2048) and down (K = 3072) projections: out[row] = W.act + resid[row], activations and residual
// in shared memory.  One shared non-inlined copy; returns the advanced chunk counter.
template <bool GATED>
__device__ __noinline__ uint32_t gemv_wide(const Params &P, Ctx c, int kind, const float *act, const float *resid,
                                           unsigned long long *out, uint32_t tag) {
  const int rsh = kind == K_O ? 1 : 0;
  const int wfmt = P.wfmt;
  const int RPC = 1 << rsh, G = CONS_WARPS >> rsh, K = kind == K_O ? QS : I, rb = kind_row_bytes(kind, wfmt);
  const int kiters = K / 256;    // 256 weights per warp pass: 8 or 12
  const SegTab *t = c.segs();
  const int sub = c.warp & (RPC - 1), wch = c.warp >> rsh;
  const int n = t->nseg[kind];
  // plain parity waits; GATED (some phase longer than the ring) puts a barrier after every pass of G chunks,
  // see gemv_k1024
  constexpr bool pass_gate = GATED;
  for (int s = 0; s < n; ++s) {
    const int nrows = t->nrows[kind][s];
    const int out0 = t->out0[kind][s];
    const int nchunks = (nrows + RPC - 1) >> rsh;
#pragma unroll 1
    for (int c0 = 0; c0 < nchunks; c0 += G) {
      const int ch = c0 + wch;
      const int row = (ch << rsh) + sub;
      float part = 0.f;
      bool have = false;
      if (ch < nchunks && row < nrows) {            // warp-uniform
        const uint32_t idx = c.chunk + static_cast<uint32_t>(ch);
        if (__all_sync(0xffffffffu, mbar_wait(P, c, c.full(idx % NSLOTS), (idx / NSLOTS) & 1u, WHERE_FULL, false))) {
          const unsigned char *wrow = c.slot(idx) + sub * rb;
          float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
          for (int j = 0; j < kiters; j += 4) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const int k = (j + q) * 256 + c.lane * 8;
              const float4 a0 = *reinterpret_cast<const float4 *>(act + k);
              const float4 a1 = *reinterpret_cast<const float4 *>(act + k + 4);
              const float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
              float wv[8];
              load_w8(wrow, (j + q) * 32 + c.lane, wfmt, wv);
              acc[q] = dot8f(wv, av, acc[q]);
            }
          }
          part = ((acc[0] + acc[1]) + (acc[2] + acc[3])) * row_scale(wrow, K, wfmt);
          have = true;
        }
      }
      __syncwarp();   // slot first, then the stores (see gemv_k1024)
      if (c.lane == 0 && ch < nchunks)
        mbar_arrive_n(c.empty((c.chunk + static_cast<uint32_t>(ch)) % NSLOTS), EMPTY_UNITS >> rsh);
      if (have) {
        const int o = out0 + row;
        const float r = warp_sum(part) + resid[o];
        if (c.lane == 0) ll_publish(out + o, r, tag, c.repl);
      }
      if (pass_gate) cons_sync();
    }
    c.chunk += static_cast<uint32_t>(nchunks);
  }
  return c.chunk;
}

#endif  // QMK_TC_BUILD
// ----------------------------------------------------------------------------- attention
// Work item (kv head g, split s) on CTA g + 8*s: old cache rows [p0, p1); the last split also
// normalises/rotates/stores the new K,V row and folds it in.  Writes either the final head
// outputs (one split) or unnormalised partials.
// FUSED: unnormalised partials also when there is one split (the merge follows in every case).
template <bool FUSED>
__device__ __noinline__ uint32_t attention_phase(const Params &P, Ctx c, const __half *nv, int layer, int pos,
                                                 uint32_t tag) {
  const AttnItem it = attn_item(P, c, 0, 1, CONS_WARPS, pos);
  float *s_q = c.f(F_Q), *s_knew = c.f(F_KNEW), *s_vnew = c.f(F_VNEW), *s_wpart = c.f(F_WPART), *s_misc = c.f(F_MISC);
  const float *s_cs = c.f(F_CS);
  const unsigned long long *qkv = c.llr + LL_QKV;
  if (!it.active) return c.chunk;
  const int S = it.S, g = it.g, s = it.s;
  const bool owner = (s == S - 1);
  const int p0 = it.p0, p1 = it.p1;
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
#pragma unroll
      for (int i = 0; i < 4; ++i) s_q[w * D + lane + 32 * i] = v[i];
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
  // score of the new row (owner only), by warps 0 and 1
  if (owner && c.warp < 2) {
    float d = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) d = fmaf(s_q[c.warp * D + c.lane + 32 * i], s_knew[c.lane + 32 * i], d);
    d = warp_sum(d);
    if (c.lane == 0) s_misc[c.warp] = d * sc_log2;
  }

  // (2) stream old rows: 16 lanes per row (8 dims each), 2 rows per warp pass, 32 rows per CTA pass.
  // (8 lanes x 16 dims needs 32 more registers and spilled; spills cost an L2 round trip here.)
  const int grp = c.lane >> 4, seg = c.lane & 15;
  float q0[8], q1[8], a0[8], a1[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    q0[i] = s_q[seg * 8 + i];
    q1[i] = s_q[D + seg * 8 + i];
    a0[i] = 0.f;
    a1[i] = 0.f;
  }
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  // The two row groups of a warp can run different trip counts: shuffles inside the loop name
  // only the 16 lanes of the group.
  const uint32_t grp_mask = 0xffffu << (grp * 16);
  // Old rows arrive through the ring in chunks of 16 K rows + 16 V rows; warp w takes chunks
  // w, w + CONS_WARPS, ... and hands each slot back when done.  Plain parity waits: an item with more chunks
  // than ring slots (more than 336 rows: contexts past 6000 tokens, or reduced grids) puts a barrier after
  // every pass of CONS_WARPS chunks, see gemv_k1024.
  const bool pass_gate = it.nchunks > NSLOTS;
#pragma unroll 1
  for (int j0 = 0; j0 < it.nchunks; j0 += CONS_WARPS) {
    const int j = j0 + c.warp;
    if (j >= it.nchunks) {
      if (pass_gate) cons_sync();
      continue;
    }
    const uint32_t idx = c.chunk + static_cast<uint32_t>(j);
    const int nrow = min(it.rpc, (p1 - p0) - j * it.rpc);
    if (__all_sync(0xffffffffu, mbar_wait(P, c, c.full(idx % NSLOTS), (idx / NSLOTS) & 1u, WHERE_FULL, false))) {
      const unsigned char *kslot = c.slot(idx) + seg * 16;
#pragma unroll 2
      for (int r = grp; r < nrow; r += 2) {
        const uint4 k0 = *reinterpret_cast<const uint4 *>(kslot + r * (D * 2));
        const uint4 v0 = *reinterpret_cast<const uint4 *>(kslot + SLOT_HALF + r * (D * 2));
        float d0 = dot8(k0, q0, 0.f), d1 = dot8(k0, q1, 0.f);
#pragma unroll
        for (int o = 1; o < 16; o <<= 1) {
          d0 += __shfl_xor_sync(grp_mask, d0, o);
          d1 += __shfl_xor_sync(grp_mask, d1, o);
        }
        d0 *= sc_log2;
        d1 *= sc_log2;
        const float n0 = fmaxf(m0, d0), n1 = fmaxf(m1, d1);
        const float cr0 = exp2f(m0 - n0), cr1 = exp2f(m1 - n1);
        const float e0 = exp2f(d0 - n0), e1 = exp2f(d1 - n1);
        m0 = n0; m1 = n1;
        l0 = fmaf(l0, cr0, e0);
        l1 = fmaf(l1, cr1, e1);
        const __half2 *h = reinterpret_cast<const __half2 *>(&v0);
        // packed fp32 multiply / FMA (two dims per instruction); at 4096-token contexts +1.6 % on one GPU, no
        // difference on another (the kernel's build-to-build spread is of that size)
        const float2 cr0p = make_float2(cr0, cr0), cr1p = make_float2(cr1, cr1), e0p = make_float2(e0, e0), e1p = make_float2(e1, e1);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = __half22float2(h[i]);
          const float2 r0 = __ffma2_rn(make_float2(a0[2 * i], a0[2 * i + 1]), cr0p, __fmul2_rn(e0p, f));
          const float2 r1 = __ffma2_rn(make_float2(a1[2 * i], a1[2 * i + 1]), cr1p, __fmul2_rn(e1p, f));
          a0[2 * i] = r0.x; a0[2 * i + 1] = r0.y;
          a1[2 * i] = r1.x; a1[2 * i + 1] = r1.y;
        }
      }
    }
    __syncwarp();
    if (c.lane == 0) mbar_arrive_n(c.empty(idx % NSLOTS), EMPTY_UNITS);
    if (pass_gate) cons_sync();
  }
  c.chunk += static_cast<uint32_t>(it.nchunks);
  QMK_FINE(63);
  // (3) merge the 2 row groups of the warp (rows differ, dims match for equal `seg`)
  __syncwarp();
  {
    const int o = 16;
    const float om0 = __shfl_xor_sync(0xffffffffu, m0, o), om1 = __shfl_xor_sync(0xffffffffu, m1, o);
    const float ol0 = __shfl_xor_sync(0xffffffffu, l0, o), ol1 = __shfl_xor_sync(0xffffffffu, l1, o);
    const float n0 = fmaxf(m0, om0), n1 = fmaxf(m1, om1);
    const float sa0 = (m0 == -INFINITY) ? 0.f : exp2f(m0 - n0), sb0 = (om0 == -INFINITY) ? 0.f : exp2f(om0 - n0);
    const float sa1 = (m1 == -INFINITY) ? 0.f : exp2f(m1 - n1), sb1 = (om1 == -INFINITY) ? 0.f : exp2f(om1 - n1);
    l0 = l0 * sa0 + ol0 * sb0;
    l1 = l1 * sa1 + ol1 * sb1;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float oa0 = __shfl_xor_sync(0xffffffffu, a0[i], o), oa1 = __shfl_xor_sync(0xffffffffu, a1[i], o);
      a0[i] = a0[i] * sa0 + oa0 * sb0;
      a1[i] = a1[i] * sa1 + oa1 * sb1;
    }
    m0 = n0; m1 = n1;
  }
  if (grp == 0) {
    float *w0 = s_wpart + (c.warp * 2 + 0) * PART_STRIDE, *w1 = s_wpart + (c.warp * 2 + 1) * PART_STRIDE;
#pragma unroll
    for (int i = 0; i < 8; ++i) { w0[seg * 8 + i] = a0[i]; w1[seg * 8 + i] = a1[i]; }
    if (seg == 0) { w0[D] = m0; w0[D + 1] = l0; w1[D] = m1; w1[D + 1] = l1; }
  }
  QMK_FINE(64);
  cons_sync();
  QMK_FINE(65);
  // (4) merge the 16 warps (+ the new row) per (head, dim)
  if (c.tid < 2 * D) {
    const int h = c.tid >> 7, d = c.tid & (D - 1);
    float M = owner ? s_misc[h] : -INFINITY;
    for (int w = 0; w < CONS_WARPS; ++w) M = fmaxf(M, s_wpart[(w * 2 + h) * PART_STRIDE + D]);
    float L = 0.f, A = 0.f;
    if (M != -INFINITY) {
      for (int w = 0; w < CONS_WARPS; ++w) {
        const float *wp = s_wpart + (w * 2 + h) * PART_STRIDE;
        const float mw = wp[D];
        const float sc = (mw == -INFINITY) ? 0.f : exp2f(mw - M);
        L = fmaf(wp[D + 1], sc, L);
        A = fmaf(wp[d], sc, A);
      }
      if (owner) {
        const float sc = exp2f(s_misc[h] - M);
        L += sc;
        A = fmaf(s_vnew[d], sc, A);
      }
    }
    const int hq = 2 * g + h;
    if (!FUSED && S == 1) {
      ll_publish(P.ll + LL_ATTN + hq * D + d, A / L, tag, c.repl);
    } else {
      unsigned long long *part = P.ll + LL_PART + static_cast<size_t>(hq * MAX_SPLITS + s) * PART_STRIDE;
      ll_publish(part + d, A, tag, c.repl);
      if (d == 0) { ll_publish(part + D, M, tag, c.repl); ll_publish(part + D + 1, L, tag, c.repl); }
    }
  }
  QMK_FINE(66);
  // New K,V row -> cache (megakernel_5090.cu:392-397), off the critical path.  The fence orders
  // the row before the exchange words this CTA publishes later; readers fence once per step.
  if (owner && (c.warp == 2 || c.warp == 3)) {
    __half *cache = ((c.warp == 2) ? P.k_cache : P.v_cache) + head_base + static_cast<size_t>(pos) * D;
    const float *snew = (c.warp == 2) ? s_knew : s_vnew;
#pragma unroll
    for (int i = 0; i < 4; ++i) cache[c.lane + 32 * i] = __float2half_rn(snew[c.lane + 32 * i]);
    __threadfence();
  }
  return c.chunk;
}

#define QMK_STAMP(slot)                                                                           \
  do {                                                                                            \
    if (P.prof && c.tid == 0 && step == P.num_steps - 1)                                          \
      P.prof[static_cast<size_t>(c.cta) * PROF_STRIDE + (slot)] = now_ns();                       \
  } while (0)

#ifndef QMK_TC_BUILD
// Combines the S partials of each attention output element this CTA owns (S > 1 only).
__device__ __noinline__ void attention_merge(const Params &P, const Ctx c, int S, uint32_t tag) {
  const int e0 = c.segs()->e0, e1 = c.segs()->e1;
#pragma unroll 1
  for (int e = e0 + c.warp; e < e1; e += CONS_WARPS) {
    const int hq = e >> 7, d = e & (D - 1);
    float a = 0.f, m = -INFINITY, l = 0.f;
    if (c.lane < S) {
      const unsigned long long *part = c.llr + LL_PART + static_cast<size_t>(hq * MAX_SPLITS + c.lane) * PART_STRIDE;
      const unsigned long long *wp[3] = {part + d, part + D, part + D + 1};
      float v3[3];
      ll_wait_many<3>(P, c, wp, 0x7u, tag, v3);
      a = v3[0]; m = v3[1]; l = v3[2];
    }
    const float M = warp_max(m);
    const float sc = (m == -INFINITY) ? 0.f : exp2f(m - M);
    const float L = warp_sum(l * sc), A = warp_sum(a * sc);
    if (c.lane == 0) ll_publish(P.ll + LL_ATTN + e, A / L, tag, c.repl);
  }
}

// ----------------------------------------------------------------------------- the kernel
// GATED: the grid is so small (below ~74 CTAs) that a projection phase has more chunks on a CTA than the ring
// has slots; the host picks the entry point with grid_has_long_phase().
template <bool GATED>
__device__ __forceinline__ void decode_body(const Params &P) {
  extern __shared__ __align__(128) unsigned char smem[];
  Ctx c;
  c.smem = smem;
  c.tid = threadIdx.x;
  c.warp = threadIdx.x >> 5;
  c.lane = threadIdx.x & 31;
  c.cta = blockIdx.x;
  c.ncta = gridDim.x;
  c.chunk = 0;
  c.repl = max(1, P.repl);
  c.llr = P.ll + static_cast<size_t>(c.cta % c.repl) * LL_REPL_STRIDE;

  if (c.tid == 0) {
    for (int i = 0; i < NSLOTS; ++i) { mbar_init(c.full(i), 1); mbar_init(c.empty(i), EMPTY_UNITS); }
    mbar_init(c.nfull(0), 1);
    mbar_init(c.nfull(1), 1);
    volatile int *fl = c.flags();
    fl[0] = 0; fl[1] = 0; fl[2] = 0; fl[3] = 0; fl[4] = 0; fl[5] = 0; fl[6] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (c.tid == 32) build_segtab(reinterpret_cast<SegTab *>(smem + OFF_SEGS), c.cta, c.ncta, P.vocab);
  {  // layer pointer table -> shared memory (12 pointers per layer)
    const unsigned long long *src = reinterpret_cast<const unsigned long long *>(P.layers);
    unsigned long long *dst = reinterpret_cast<unsigned long long *>(smem + OFF_LAYERS);
    for (int i = c.tid; i < P.num_layers * 12; i += THREADS) dst[i] = src[i];
  }
  __syncthreads();

  if (c.warp == CONS_WARPS) {
    if (c.lane == 0) producer_main(P, c);
    __syncwarp();   // the warp meets the block barrier below as a whole
  } else {
    float *s_x = c.f(F_X), *s_x1 = c.f(F_X1), *s_vec = c.f(F_VEC), *s_misc = c.f(F_MISC), *s_amax = c.f(F_AMAX);
    int token = P.prefill ? P.token_ids[0] : P.first_token;
#pragma unroll 1
    for (int step = 0; step < P.num_steps; ++step) {
      const int pos = P.start_position + step;
      const uint32_t tag_base = (P.seq_base + static_cast<uint32_t>(step)) * 64u;
      if (token < 0 || token >= P.vocab) { if (c.tid == 0) raise_error(P, c, QMK_ERR_BAD_TOKEN, WHERE_TOKEN); token = 0; }
      // cos/sin of this position (fp32 angles, or the caller's fp16 table row)
      if (c.tid < D / 2) {
        float cs, sn;
        if (P.rope_from_table) {
          cs = __half2float(P.cos_table[static_cast<size_t>(pos) * D + c.tid]);
          sn = __half2float(P.sin_table[static_cast<size_t>(pos) * D + c.tid]);
        } else {   // fp32 table (sincosf's large-argument path would put a stack frame into this kernel)
          cs = __ldg(P.rope + static_cast<size_t>(pos) * D + c.tid);
          sn = __ldg(P.rope + static_cast<size_t>(pos) * D + 64 + c.tid);
        }
        c.f(F_CS)[c.tid] = cs;
        c.f(F_CS)[64 + c.tid] = sn;
      }
      __threadfence();  // acquire side of the KV-row ordering (rows written in earlier steps)
      const int S_step = max(1, min(pos / max(1, P.split_len), min(MAX_SPLITS, max(1, c.ncta / NKV))));  // as attn_item
      // embedding row -> fp32 residual stream (megakernel_5090.cu:825-830)
      float ss = 0.f;
      {
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
            s_x[c.tid + j * CONS_THREADS] = v;
            ss = fmaf(v, v, ss);
          }
      }
#pragma unroll 1
      for (int layer = 0; layer < P.num_layers; ++layer) {
        const unsigned long long *rec = c.layer_rec(layer);
        const uint32_t tag = tag_base + static_cast<uint32_t>(layer) + 1u;
        const uint32_t Lg = static_cast<uint32_t>(step) * static_cast<uint32_t>(P.num_layers) + static_cast<uint32_t>(layer);
        const __half *nv = c.norms(Lg & 1u);
        mbar_wait(P, c, c.nfull(Lg & 1u), (Lg >> 1) & 1u, WHERE_FULL, false);
        // P1: input RMSNorm + fused QKV rows
        QMK_STAMP(layer * 12 + 0);
        c.chunk = gemv_k1024<GATED>(P, c, K_QKV, s_x, ss, nv + NB_IN_LN, P.ll + LL_QKV, tag, nullptr);
        // P2/P3: attention work items, then merge of split partials
        QMK_STAMP(layer * 12 + 1);
        c.chunk = attention_phase<false>(P, c, nv, layer, pos, tag);
        QMK_STAMP(layer * 12 + 2);
        if (S_step > 1) attention_merge(P, c, S_step, tag);
        QMK_STAMP(layer * 12 + 3);
        // P4: O-proj + residual
        poll_vec(P, c, c.llr + LL_ATTN, QS, tag, s_vec);
        QMK_STAMP(layer * 12 + 4);
        cons_sync();
        c.chunk = gemv_wide<GATED>(P, c, K_O, s_vec, s_x, P.ll + LL_X1, tag);
        // P5: post-attention RMSNorm + gate/up + SwiGLU
        QMK_STAMP(layer * 12 + 5);
        ss = poll_vec(P, c, c.llr + LL_X1, H, tag, s_x1);
        QMK_STAMP(layer * 12 + 6);
        c.chunk = gemv_k1024<GATED>(P, c, K_GU, s_x1, ss, nv + NB_POST_LN, P.ll + LL_INTER, tag, nullptr);
        // P6: down-proj + residual
        QMK_STAMP(layer * 12 + 7);
        poll_vec(P, c, c.llr + LL_INTER, I, tag, s_vec);
        QMK_STAMP(layer * 12 + 8);
        cons_sync();
        c.chunk = gemv_wide<GATED>(P, c, K_DOWN, s_vec, s_x1, P.ll + LL_X2, tag);
        // next layer's input (in prefill mode the last layer's output is not needed)
        QMK_STAMP(layer * 12 + 9);
        if (!(P.prefill && layer == P.num_layers - 1)) ss = poll_vec(P, c, c.llr + LL_X2, H, tag, s_x);
        QMK_STAMP(layer * 12 + 10);
        if (cons_any(c.flags()[0] != 0)) break;
      }
      if (cons_any(c.flags()[0] != 0)) break;
      if (P.prefill) {
        if (step + 1 < P.num_steps) token = P.token_ids[step + 1];
        continue;
      }
      // final RMSNorm + tied LM head + argmax (megakernel_5090.cu:921-947, 1024-1167)
      QMK_STAMP(P.num_layers * 12 + 0);
      c.chunk = gemv_k1024<false>(P, c, K_LM, s_x, ss, P.final_norm, nullptr, 0u,
                                  P.logits_out ? P.logits_out + static_cast<size_t>(step) * P.vocab : nullptr);
      QMK_STAMP(P.num_layers * 12 + 1);
      cons_sync();
      const uint32_t atag = tag_base + 63u;
      if (c.tid == 0) {
        float best = s_misc[32];
        int best_i = __float_as_int(s_misc[48]);
#pragma unroll 1
        for (int w = 1; w < CONS_WARPS; ++w) {
          const float v = s_misc[32 + w];
          const int vi = __float_as_int(s_misc[48 + w]);
          if (v > best || (v == best && vi < best_i)) { best = v; best_i = vi; }
        }
        ll_publish(P.ll + LL_AMAX + 2 * c.cta, best, atag, c.repl);
        ll_publish(P.ll + LL_AMAX + 2 * c.cta + 1, __int_as_float(best_i), atag, c.repl);
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
      const bool aborted = cons_any(c.flags()[0] != 0);
      QMK_STAMP(P.num_layers * 12 + 2);
      token = __float_as_int(s_misc[16]);
      if (aborted) break;
      if (c.cta == 0 && c.tid == 0) {
        if (P.output_log) P.output_log[step] = token;   // the EOS token is logged too (megakernel_5090.cu:785-787)
        if (P.output_token) *P.output_token = token;
      }
      if (token == P.eos) break;
    }
    if (c.tid == 0) { c.flags()[3] = static_cast<int>(c.chunk); c.flags()[1] = 1; }
  }
  __syncthreads();
  // Bulk copies issued but never consumed (early stop, abort) must land before the CTA exits.
  if (c.tid == CONS_THREADS) {
    // Every slot's latest fill is checked (already-landed phases answer at once), so this also
    // covers chunks the consumers skipped after an abort.
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
    for (uint32_t b = 0; b < 2; ++b) {   // norm-vector copies
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

__global__ void __launch_bounds__(THREADS, 1) qwen3_decode_megakernel(const __grid_constant__ Params P) {
  decode_body<false>(P);
}
__global__ void __launch_bounds__(THREADS, 1) qwen3_decode_megakernel_small_grid(const __grid_constant__ Params P) {
  decode_body<true>(P);
}
// Host side: which of the two a grid of `ncta` CTAs needs (the same row split the kernel computes).
inline bool grid_has_long_phase(int ncta) {
  SegTab t;
  for (int cta = 0; cta < ncta; ++cta) {
    build_segtab(&t, cta, ncta, 0);
    if (t.long_phase) return true;
  }
  return false;
}
#endif  // QMK_TC_BUILD

#endif  // QMK_MAX_SEQ == 1

}  // namespace QMK_NS
