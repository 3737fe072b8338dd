// Persistent batch-1 decode megakernel for Qwen3-0.6B on B200 (sm_100a), and its C ABI.
//
// One cooperative launch of one CTA per SM runs `num_steps` tokens end to end:
// embedding, 28 x {RMSNorm, QKV, QK-norm + RoPE, split-KV GQA attention, O-proj,
// RMSNorm, SwiGLU, down-proj}, final RMSNorm, tied LM head, argmax, token feedback.
// It replaces the reference's per-token launch sequence
// (Tools/megakernel/megakernel_5090.cu:796-1167, 1398-1432).
//
// Design (why it looks nothing like the reference's kernel):
//  * Weights never wait for activations.  Every CTA owns a fixed row slice of every
//    matrix ([out,in] row-major, so a slice is one contiguous byte range); a producer
//    warp streams those slices HBM -> shared memory with cp.async.bulk into an
//    mbarrier ring and runs ahead of the math across phase, layer and token
//    boundaries.  HBM stays busy while consumer warps wait for activations.
//  * No grid barriers.  Activations cross CTAs as 8-byte words {fp32 value, 32-bit
//    tag}; a 64-bit store is single-copy atomic, so a consumer that sees the tag of
//    this (token, layer) has the value.  One L2 round trip per exchange replaces
//    arrive + poll + fence + reload (the reference: 226 counter barriers per token,
//    megakernel_5090.cu:108-135).
//  * fp32 residual stream and activations; fp16 only for weights and the KV cache.
//  * Attention is split over (kv head, KV range) work items on all SMs, both query
//    heads of a GQA pair share each K/V byte, partial (max, sum, acc) merged after.
//  * LM head + argmax (lowest index wins ties) + token feedback are phases of the
//    same launch, so a whole request is one kernel.
//  * Every wait is bounded; on a timeout the kernel records a status word, all CTAs
//    drain, in-flight bulk copies are awaited, and the launch returns normally.

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>
#include <math.h>
#include <mutex>
#include <string>

#include "../../include/qwen_megakernel.h"

namespace qmk {

constexpr int H = 1024;          // hidden
constexpr int I = 3072;          // MLP intermediate
constexpr int NQ = 16;           // query heads
constexpr int NKV = 8;           // kv heads
constexpr int D = 128;           // head dim
constexpr int QS = NQ * D;       // 2048
constexpr int KVS = NKV * D;     // 1024
constexpr int QKV_ROWS = QS + 2 * KVS;  // 4096
constexpr float RMS_EPS = 1e-6f;

constexpr int CONS_WARPS = 16;
constexpr int CONS_THREADS = CONS_WARPS * 32;   // 512 math threads
constexpr int THREADS = CONS_THREADS + 32;      // + 1 producer warp
constexpr int SLOT_BYTES = 8192;
constexpr int NSLOTS = 22;
static_assert(NSLOTS >= CONS_WARPS, "a group of chunks (up to one per warp) must fit in the ring");
constexpr int MAX_SPLITS = 24;   // attention work items per kv head (<= grid / 8)
constexpr int MAX_CTAS = 256;
constexpr int PART_STRIDE = D + 2;  // acc[128], max, sum

// Exchange buffers, in 8-byte words.
constexpr int LL_QKV = 0;
constexpr int LL_ATTN = LL_QKV + QKV_ROWS;
constexpr int LL_X1 = LL_ATTN + QS;
constexpr int LL_INTER = LL_X1 + H;
constexpr int LL_X2 = LL_INTER + I;
constexpr int LL_AMAX = LL_X2 + H;
constexpr int LL_PART = LL_AMAX + 2 * MAX_CTAS;
constexpr int LL_WORDS = LL_PART + NQ * MAX_SPLITS * PART_STRIDE;

// Same binary layout as the reference's per-layer pointer record
// (megakernel_5090.cu:91-104): 11 fp16 pointers + 1 pad = 96 bytes.
struct __align__(16) LayerW {
  const __half *in_ln, *wq, *wk, *wv, *q_norm, *k_norm, *wo, *post_ln, *w_gate, *w_up, *w_down;
  const void *pad;
};

struct Params {
  const __half *embed;
  const LayerW *layers;
  const __half *final_norm;
  const __half *lm_head;
  const __half *cos_table, *sin_table;
  __half *k_cache, *v_cache;
  unsigned long long *ll;
  unsigned int *status;          // [0] code, [1] where, [2] cta
  const int *token_ids;          // prefill: device array of num_steps tokens
  int *output_log;               // decode: token per step (may be null)
  int *output_token;             // decode: last token (may be null)
  float *normalized_out;         // fp32[1024] final-norm output of the last step (may be null)
  __half *hidden_out;            // fp16[1024] last hidden state (may be null)
  float *bmax_vals;              // per-CTA argmax partials (may be null)
  int *bmax_idxs;
  float *logits_out;             // debug dump (may be null)
  unsigned long long timeout_ns;
  int first_token, num_steps, num_layers, start_position, max_seq_len, vocab;
  int eos, prefill, rope_from_table, split_len;
  unsigned int seq_base;
  float attn_scale;
};

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

// Consumer barrier that also ORs a predicate over all 512 threads (same result everywhere).
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

// ----------------------------------------------------------------------------- per-CTA context
struct Ctx {
  unsigned char *ring;
  uint64_t *full, *empty;
  float *s_x, *s_x1, *s_vec, *s_red, *s_q, *s_knew, *s_vnew, *s_wpart, *s_cs, *s_misc;
  volatile int *s_flags;  // [0] abort, [1] stop, [2] issued chunks, [3] consumed chunks
  unsigned int *status;
  unsigned long long timeout_ns;
  int tid, warp, lane, cta, ncta;
  uint32_t chunk;  // consumer-side running chunk index (uniform over consumer threads)
};

enum { WHERE_LL = 1, WHERE_FULL = 2, WHERE_EMPTY = 3, WHERE_DRAIN = 4, WHERE_TOKEN = 5 };

__device__ __noinline__ void raise_error(Ctx &c, int code, int where) {
  if (atomicCAS(c.status, 0u, static_cast<unsigned>(code)) == 0u) {
    c.status[1] = static_cast<unsigned>(where);
    c.status[2] = static_cast<unsigned>(c.cta);
  }
  c.s_flags[0] = 1;
}

// Slow path of an exchange-word wait: spin until the tag shows up, another CTA reported
// an error, or the time budget is gone.  Returns the word (garbage after an abort).
__device__ __noinline__ unsigned long long ll_spin(const unsigned long long *p, uint32_t tag, Ctx &c) {
  const unsigned long long t0 = now_ns();
  uint32_t it = 0;
  for (;;) {
    unsigned long long w = ll_load(p);
    if (static_cast<uint32_t>(w >> 32) == tag) return w;
    if ((++it & 63u) == 0u) {
      if (c.s_flags[0]) return 0ull;
      if (ld_relaxed_u32(c.status) != 0u) { c.s_flags[0] = 1; return 0ull; }
      if (now_ns() - t0 > c.timeout_ns) { raise_error(c, QMK_ERR_WAIT_TIMEOUT, WHERE_LL); return 0ull; }
    }
  }
}
__device__ __forceinline__ float ll_wait(const unsigned long long *p, uint32_t tag, Ctx &c) {
  unsigned long long w = ll_load(p);
  if (static_cast<uint32_t>(w >> 32) != tag) w = ll_spin(p, tag, c);
  return __uint_as_float(static_cast<uint32_t>(w));
}

// Wait on an mbarrier phase with the same bounds.  Returns false after an abort.
__device__ __noinline__ bool mbar_spin(uint64_t *bar, uint32_t parity, Ctx &c, int where, bool watch_stop) {
  const unsigned long long t0 = now_ns();
  uint32_t it = 0;
  for (;;) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++it & 15u) == 0u) {
      if (c.s_flags[0]) return false;
      if (watch_stop && c.s_flags[1]) return false;
      if (ld_relaxed_u32(c.status) != 0u) { c.s_flags[0] = 1; return false; }
      // the producer may legitimately wait as long as any consumer does: 4x budget
      if (now_ns() - t0 > (watch_stop ? 4 * c.timeout_ns : c.timeout_ns)) {
        raise_error(c, QMK_ERR_WAIT_TIMEOUT, where);
        return false;
      }
    }
  }
}
__device__ __forceinline__ bool wait_full(Ctx &c, uint32_t idx) {
  uint64_t *bar = c.full + (idx % NSLOTS);
  uint32_t parity = (idx / NSLOTS) & 1u;
  bool ok = mbar_try_wait(bar, parity);
  if (!ok) ok = mbar_spin(bar, parity, c, WHERE_FULL, false);
  return __all_sync(0xffffffffu, ok);   // the whole warp takes the same branch (shuffles follow)
}

// Rows [r0, r1) of an n-row matrix owned by this CTA.
__device__ __forceinline__ void split_rows(int n, int ncta, int cta, int &r0, int &r1) {
  r0 = static_cast<int>((static_cast<long long>(n) * cta) / ncta);
  r1 = static_cast<int>((static_cast<long long>(n) * (cta + 1)) / ncta);
}

// A contiguous run of weight rows one CTA streams and multiplies.
struct Seg {
  const unsigned char *src;   // first row
  const unsigned char *src2;  // second matrix (up_proj rows) for the gate/up phase, else null
  int nrows;
  int out0;                   // index of the first output element
};

enum Phase { PH_QKV = 0, PH_O = 1, PH_GU = 2, PH_DOWN = 3, PH_LM = 4 };
template <int PH> struct PhaseCfg;
template <> struct PhaseCfg<PH_QKV> { static constexpr int K = H, RPC = 4; };
template <> struct PhaseCfg<PH_O> { static constexpr int K = QS, RPC = 2; };
template <> struct PhaseCfg<PH_GU> { static constexpr int K = H, RPC = 2; };   // 2 gate + 2 up rows
template <> struct PhaseCfg<PH_DOWN> { static constexpr int K = I, RPC = 1; };
template <> struct PhaseCfg<PH_LM> { static constexpr int K = H, RPC = 4; };

// Row slices of one phase for this CTA.  Used verbatim by the producer and the consumers,
// which is what keeps their chunk sequences identical.
template <int PH>
__device__ __forceinline__ int phase_segs(const LayerW &lw, const __half *lm_head, int vocab, int cta, int ncta,
                                          Seg segs[3]) {
  int r0, r1, n = 0;
  if (PH == PH_QKV) {
    split_rows(QKV_ROWS, ncta, cta, r0, r1);
    const __half *base[3] = {lw.wq, lw.wk, lw.wv};
    const int lo[3] = {0, QS, QS + KVS}, hi[3] = {QS, QS + KVS, QKV_ROWS};
#pragma unroll
    for (int t = 0; t < 3; ++t) {
      int a = max(r0, lo[t]), b = min(r1, hi[t]);
      if (a < b) {
        segs[n].src = reinterpret_cast<const unsigned char *>(base[t] + static_cast<size_t>(a - lo[t]) * H);
        segs[n].src2 = nullptr;
        segs[n].nrows = b - a;
        segs[n].out0 = a;
        ++n;
      }
    }
  } else if (PH == PH_O) {
    split_rows(H, ncta, cta, r0, r1);
    if (r0 < r1) { segs[0] = {reinterpret_cast<const unsigned char *>(lw.wo + static_cast<size_t>(r0) * QS), nullptr, r1 - r0, r0}; n = 1; }
  } else if (PH == PH_GU) {
    split_rows(I, ncta, cta, r0, r1);
    if (r0 < r1) {
      segs[0] = {reinterpret_cast<const unsigned char *>(lw.w_gate + static_cast<size_t>(r0) * H),
                 reinterpret_cast<const unsigned char *>(lw.w_up + static_cast<size_t>(r0) * H), r1 - r0, r0};
      n = 1;
    }
  } else if (PH == PH_DOWN) {
    split_rows(H, ncta, cta, r0, r1);
    if (r0 < r1) { segs[0] = {reinterpret_cast<const unsigned char *>(lw.w_down + static_cast<size_t>(r0) * I), nullptr, r1 - r0, r0}; n = 1; }
  } else {
    split_rows(vocab, ncta, cta, r0, r1);
    if (r0 < r1) { segs[0] = {reinterpret_cast<const unsigned char *>(lm_head + static_cast<size_t>(r0) * H), nullptr, r1 - r0, r0}; n = 1; }
  }
  return n;
}

// ----------------------------------------------------------------------------- producer
struct Producer {
  Ctx &c;
  uint64_t pol;
  uint32_t idx;
  __device__ bool issue(const unsigned char *src, const unsigned char *src2, uint32_t bytes) {
    const uint32_t slot = idx % NSLOTS;
    if (c.s_flags[0] | c.s_flags[1]) return false;
    if (idx >= NSLOTS) {
      const uint32_t parity = ((idx / NSLOTS) - 1u) & 1u;
      if (!mbar_try_wait(c.empty + slot, parity) && !mbar_spin(c.empty + slot, parity, c, WHERE_EMPTY, true)) return false;
    }
    unsigned char *dst = c.ring + static_cast<size_t>(slot) * SLOT_BYTES;
    mbar_arrive_expect_tx(c.full + slot, src2 ? 2 * bytes : bytes);
    bulk_g2s(dst, src, bytes, c.full + slot, pol);
    if (src2) bulk_g2s(dst + SLOT_BYTES / 2, src2, bytes, c.full + slot, pol);
    ++idx;
    return true;
  }
  template <int PH>
  __device__ bool phase(const LayerW &lw, const __half *lm_head, int vocab) {
    constexpr int RB = PhaseCfg<PH>::K * 2, RPC = PhaseCfg<PH>::RPC;
    Seg segs[3];
    const int n = phase_segs<PH>(lw, lm_head, vocab, c.cta, c.ncta, segs);
    for (int s = 0; s < n; ++s)
      for (int r = 0; r < segs[s].nrows; r += RPC) {
        const int nr = min(RPC, segs[s].nrows - r);
        if (!issue(segs[s].src + static_cast<size_t>(r) * RB, segs[s].src2 ? segs[s].src2 + static_cast<size_t>(r) * RB : nullptr,
                   static_cast<uint32_t>(nr) * RB))
          return false;
      }
    return true;
  }
};

__device__ void producer_main(const Params &P, Ctx &c) {
  Producer pr{c, l2_evict_first_policy(), 0u};
  LayerW none{};
  bool ok = true;
  for (int step = 0; ok && step < P.num_steps; ++step) {
    for (int l = 0; ok && l < P.num_layers; ++l) {
      const LayerW lw = P.layers[l];
      ok = pr.phase<PH_QKV>(lw, nullptr, 0) && pr.phase<PH_O>(lw, nullptr, 0) && pr.phase<PH_GU>(lw, nullptr, 0) &&
           pr.phase<PH_DOWN>(lw, nullptr, 0);
    }
    if (ok && !P.prefill) ok = pr.phase<PH_LM>(none, P.lm_head, P.vocab);
  }
  c.s_flags[2] = static_cast<int>(pr.idx);
}

// ----------------------------------------------------------------------------- consumer math
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
// Row of K=1024 fp16 weights in shared memory times activations held in registers
// (lane owns k = j*256 + lane*8 + i).
__device__ __forceinline__ float row_dot_regs(const unsigned char *row, const float (&a)[32], int lane) {
  const uint4 *w = reinterpret_cast<const uint4 *>(row);
  float acc[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) acc[j] = dot8(w[j * 32 + lane], &a[j * 8], 0.f);
  return warp_sum((acc[0] + acc[1]) + (acc[2] + acc[3]));
}
// Row of K fp16 weights in shared memory times fp32 activations in shared memory.
template <int K>
__device__ __forceinline__ float row_dot_smem(const unsigned char *row, const float *act, int lane) {
  const uint4 *w = reinterpret_cast<const uint4 *>(row);
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int j = 0; j < K / 256; ++j) {
    const int k = j * 256 + lane * 8;
    const float4 a0 = *reinterpret_cast<const float4 *>(act + k);
    const float4 a1 = *reinterpret_cast<const float4 *>(act + k + 4);
    const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
    acc[j & 3] = dot8(w[j * 32 + lane], a, acc[j & 3]);
  }
  return warp_sum((acc[0] + acc[1]) + (acc[2] + acc[3]));
}

// sum over the 512 consumer threads; contains one consumer barrier
__device__ __forceinline__ float block_sum(Ctx &c, float v) {
  v = warp_sum(v);
  if (c.lane == 0) c.s_red[c.warp] = v;
  cons_sync();
  float t = 0.f;
#pragma unroll
  for (int i = 0; i < CONS_WARPS; ++i) t += c.s_red[i];
  return t;
}

// Polls N exchange words into shared memory as fp32; returns this thread's sum of squares.
template <int N>
__device__ __forceinline__ float poll_vec(const unsigned long long *buf, uint32_t tag, float *dst, Ctx &c) {
  constexpr int PT = N / CONS_THREADS;
  unsigned long long w[PT];
#pragma unroll
  for (int j = 0; j < PT; ++j) w[j] = ll_load(buf + c.tid + j * CONS_THREADS);
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < PT; ++j) {
    if (static_cast<uint32_t>(w[j] >> 32) != tag) w[j] = ll_spin(buf + c.tid + j * CONS_THREADS, tag, c);
    const float v = __uint_as_float(static_cast<uint32_t>(w[j]));
    dst[c.tid + j * CONS_THREADS] = v;
    ss = fmaf(v, v, ss);
  }
  return ss;
}

// RMSNorm of the vector in `src` (sum of squares `ss` per thread) into per-lane registers.
__device__ __forceinline__ void norm_to_regs(Ctx &c, const float *src, float ss, const uint4 (&wn)[4], float (&a)[32]) {
  const float tot = block_sum(c, ss);  // barrier inside also publishes `src`
  const float rstd = 1.0f / sqrtf(tot * (1.0f / H) + RMS_EPS);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int k = j * 256 + c.lane * 8;
    const float4 x0 = *reinterpret_cast<const float4 *>(src + k);
    const float4 x1 = *reinterpret_cast<const float4 *>(src + k + 4);
    const float x[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
    const __half2 *h = reinterpret_cast<const __half2 *>(&wn[j]);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 wf = __half22float2(h[i]);
      a[j * 8 + 2 * i] = x[2 * i] * rstd * wf.x;
      a[j * 8 + 2 * i + 1] = x[2 * i + 1] * rstd * wf.y;
    }
  }
}
__device__ __forceinline__ void load_norm_w(const __half *w, int lane, uint4 (&wn)[4]) {
#pragma unroll
  for (int j = 0; j < 4; ++j) wn[j] = __ldg(reinterpret_cast<const uint4 *>(w + j * 256 + lane * 8));
}

// Walks this CTA's chunks of one phase.  Warp w takes row (w % RPC) of chunk (w / RPC) of each
// group of 16/RPC chunks; `fn(row_ptr, row_ptr2, out_index)` runs on the whole warp.
// Every warp releases every chunk of the group (the empty barriers count 16 arrivals).
template <int PH, typename Fn>
__device__ __forceinline__ void consume_phase(Ctx &c, const LayerW &lw, const __half *lm_head, int vocab, Fn fn) {
  constexpr int RB = PhaseCfg<PH>::K * 2, RPC = PhaseCfg<PH>::RPC, G = CONS_WARPS / RPC;
  Seg segs[3];
  const int n = phase_segs<PH>(lw, lm_head, vocab, c.cta, c.ncta, segs);
  for (int s = 0; s < n; ++s) {
    const int nrows = segs[s].nrows;
    const int nchunks = (nrows + RPC - 1) / RPC;
    for (int c0 = 0; c0 < nchunks; c0 += G) {
      const int ch = c0 + c.warp / RPC;
      const int row = ch * RPC + (c.warp % RPC);
      if (ch < nchunks && row < nrows) {
        const uint32_t idx = c.chunk + static_cast<uint32_t>(ch);
        if (wait_full(c, idx)) {
          const unsigned char *p = c.ring + static_cast<size_t>(idx % NSLOTS) * SLOT_BYTES + (c.warp % RPC) * RB;
          fn(p, p + SLOT_BYTES / 2, segs[s].out0 + row);
        }
      }
      __syncwarp();
      if (c.lane == 0) {
        const int last = min(G, nchunks - c0);
        for (int j = 0; j < last; ++j) mbar_arrive(c.empty + ((c.chunk + static_cast<uint32_t>(c0 + j)) % NSLOTS));
      }
    }
    c.chunk += static_cast<uint32_t>(nchunks);
  }
}

// ----------------------------------------------------------------------------- attention
// Work item (kv head g, split s) on CTA g + 8*s: old cache rows [p0, p1); the last split also
// normalises/rotates/stores the new K,V row and folds it in.  Writes either the final head
// outputs (one split) or unnormalised partials.
__device__ void attention_phase(const Params &P, Ctx &c, const LayerW &lw, int layer, int pos, int S, uint32_t tag) {
  const unsigned long long *qkv = P.ll + LL_QKV;
  if (c.cta >= NKV * S) return;
  const int g = c.cta % NKV, s = c.cta / NKV;
  const bool owner = (s == S - 1);
  const int p0 = static_cast<int>((static_cast<long long>(pos) * s) / S);
  const int p1 = static_cast<int>((static_cast<long long>(pos) * (s + 1)) / S);
  const size_t head_base = (static_cast<size_t>(layer) * NKV + g) * static_cast<size_t>(P.max_seq_len) * D;

  // (1) head preparation: warps 0,1 = the two query heads; owner: warp 2 = K, warp 3 = V
  if (c.warp < 2 || (owner && c.warp < 4)) {
    const int w = c.warp, lane = c.lane;
    const unsigned long long *src = (w < 2) ? qkv + (2 * g + w) * D : (w == 2) ? qkv + QS + g * D : qkv + QS + KVS + g * D;
    float nw[4] = {1.f, 1.f, 1.f, 1.f};
    if (w < 3) {
      const __half *nwp = (w < 2) ? lw.q_norm : lw.k_norm;
#pragma unroll
      for (int i = 0; i < 4; ++i) nw[i] = __half2float(__ldg(nwp + lane + 32 * i));
    }
    float v[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = ll_wait(src + lane + 32 * i, tag, c);
    if (w < 3) {
      float ss = v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3];
      ss = warp_sum(ss);
      const float rstd = 1.0f / sqrtf(ss * (1.0f / D) + RMS_EPS);
#pragma unroll
      for (int i = 0; i < 4; ++i) v[i] = v[i] * rstd * nw[i];
      // rotate-half: element i pairs with i+64 and both use frequency i (i < 64)
      const float c0 = c.s_cs[lane], s0 = c.s_cs[64 + lane];
      const float c1 = c.s_cs[lane + 32], s1 = c.s_cs[64 + lane + 32];
      const float r0 = v[0] * c0 - v[2] * s0, r2 = v[0] * s0 + v[2] * c0;
      const float r1 = v[1] * c1 - v[3] * s1, r3 = v[1] * s1 + v[3] * c1;
      v[0] = r0; v[1] = r1; v[2] = r2; v[3] = r3;
    }
    if (w < 2) {
#pragma unroll
      for (int i = 0; i < 4; ++i) c.s_q[w * D + lane + 32 * i] = v[i];
    } else {
      // the new row takes part in this step's attention as the fp16 value the cache will hold
      float *snew = (w == 2) ? c.s_knew : c.s_vnew;
#pragma unroll
      for (int i = 0; i < 4; ++i) snew[lane + 32 * i] = __half2float(__float2half_rn(v[i]));
    }
  }
  cons_sync();

  const float sc_log2 = P.attn_scale * 1.4426950408889634f;
  // score of the new row (owner only), by warps 0 and 1
  if (owner && c.warp < 2) {
    float d = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) d = fmaf(c.s_q[c.warp * D + c.lane + 32 * i], c.s_knew[c.lane + 32 * i], d);
    d = warp_sum(d);
    if (c.lane == 0) c.s_misc[c.warp] = d * sc_log2;
  }

  // (2) stream old rows: 8 lanes per row (16 dims each), 4 rows per warp pass, 64 rows per CTA pass
  const int grp = c.lane >> 3, seg = c.lane & 7;
  float q0[16], q1[16], a0[16], a1[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    q0[i] = c.s_q[seg * 16 + i];
    q1[i] = c.s_q[D + seg * 16 + i];
    a0[i] = 0.f;
    a1[i] = 0.f;
  }
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  // Row groups of one warp can run different trip counts: shuffles inside the loop name only
  // the 8 lanes of the group.
  const uint32_t grp_mask = 0xffu << (grp * 8);
  const __half *kb = P.k_cache + head_base + seg * 16;
  const __half *vb = P.v_cache + head_base + seg * 16;
  for (int p = p0 + c.warp * 4 + grp; p < p1; p += CONS_WARPS * 4) {
    const uint4 *kp = reinterpret_cast<const uint4 *>(kb + static_cast<size_t>(p) * D);
    const uint4 *vp = reinterpret_cast<const uint4 *>(vb + static_cast<size_t>(p) * D);
    const uint4 k0 = __ldcg(kp), k1 = __ldcg(kp + 1), v0 = __ldcg(vp), v1 = __ldcg(vp + 1);
    float d0 = dot8(k0, q0, 0.f), d1 = dot8(k0, q1, 0.f);
    d0 = dot8(k1, q0 + 8, d0);
    d1 = dot8(k1, q1 + 8, d1);
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) {
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
    float vf[16];
    {
      const __half2 *h = reinterpret_cast<const __half2 *>(&v0);
      const __half2 *h2 = reinterpret_cast<const __half2 *>(&v1);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(h[i]), f2 = __half22float2(h2[i]);
        vf[2 * i] = f.x; vf[2 * i + 1] = f.y; vf[8 + 2 * i] = f2.x; vf[8 + 2 * i + 1] = f2.y;
      }
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      a0[i] = fmaf(a0[i], cr0, e0 * vf[i]);
      a1[i] = fmaf(a1[i], cr1, e1 * vf[i]);
    }
  }
  // (3) merge the 4 row groups of the warp (rows differ, dims match for equal `seg`)
  __syncwarp();
#pragma unroll
  for (int o = 8; o <= 16; o <<= 1) {
    const float om0 = __shfl_xor_sync(0xffffffffu, m0, o), om1 = __shfl_xor_sync(0xffffffffu, m1, o);
    const float ol0 = __shfl_xor_sync(0xffffffffu, l0, o), ol1 = __shfl_xor_sync(0xffffffffu, l1, o);
    const float n0 = fmaxf(m0, om0), n1 = fmaxf(m1, om1);
    const float sa0 = (m0 == -INFINITY) ? 0.f : exp2f(m0 - n0), sb0 = (om0 == -INFINITY) ? 0.f : exp2f(om0 - n0);
    const float sa1 = (m1 == -INFINITY) ? 0.f : exp2f(m1 - n1), sb1 = (om1 == -INFINITY) ? 0.f : exp2f(om1 - n1);
    l0 = l0 * sa0 + ol0 * sb0;
    l1 = l1 * sa1 + ol1 * sb1;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float oa0 = __shfl_xor_sync(0xffffffffu, a0[i], o), oa1 = __shfl_xor_sync(0xffffffffu, a1[i], o);
      a0[i] = a0[i] * sa0 + oa0 * sb0;
      a1[i] = a1[i] * sa1 + oa1 * sb1;
    }
    m0 = n0; m1 = n1;
  }
  if (grp == 0) {
    float *w0 = c.s_wpart + (c.warp * 2 + 0) * PART_STRIDE, *w1 = c.s_wpart + (c.warp * 2 + 1) * PART_STRIDE;
#pragma unroll
    for (int i = 0; i < 16; ++i) { w0[seg * 16 + i] = a0[i]; w1[seg * 16 + i] = a1[i]; }
    if (seg == 0) { w0[D] = m0; w0[D + 1] = l0; w1[D] = m1; w1[D + 1] = l1; }
  }
  cons_sync();
  // (4) merge the 16 warps (+ the new row) per (head, dim)
  if (c.tid < 2 * D) {
    const int h = c.tid >> 7, d = c.tid & (D - 1);
    float M = owner ? c.s_misc[h] : -INFINITY;
    for (int w = 0; w < CONS_WARPS; ++w) M = fmaxf(M, c.s_wpart[(w * 2 + h) * PART_STRIDE + D]);
    float L = 0.f, A = 0.f;
    if (M != -INFINITY) {
      for (int w = 0; w < CONS_WARPS; ++w) {
        const float *wp = c.s_wpart + (w * 2 + h) * PART_STRIDE;
        const float mw = wp[D];
        const float sc = (mw == -INFINITY) ? 0.f : exp2f(mw - M);
        L = fmaf(wp[D + 1], sc, L);
        A = fmaf(wp[d], sc, A);
      }
      if (owner) {
        const float sc = exp2f(c.s_misc[h] - M);
        L += sc;
        A = fmaf(c.s_vnew[d], sc, A);
      }
    }
    const int hq = 2 * g + h;
    if (S == 1) {
      ll_store(P.ll + LL_ATTN + hq * D + d, A / L, tag);
    } else {
      unsigned long long *part = P.ll + LL_PART + static_cast<size_t>(hq * MAX_SPLITS + s) * PART_STRIDE;
      ll_store(part + d, A, tag);
      if (d == 0) { ll_store(part + D, M, tag); ll_store(part + D + 1, L, tag); }
    }
  }
  // New K,V row -> cache (megakernel_5090.cu:392-397), off the critical path.  The fence orders
  // the row before the exchange words this CTA publishes later; readers fence once per step.
  if (owner && (c.warp == 2 || c.warp == 3)) {
    __half *cache = ((c.warp == 2) ? P.k_cache : P.v_cache) + head_base + static_cast<size_t>(pos) * D;
    const float *snew = (c.warp == 2) ? c.s_knew : c.s_vnew;
#pragma unroll
    for (int i = 0; i < 4; ++i) cache[c.lane + 32 * i] = __float2half_rn(snew[c.lane + 32 * i]);
    __threadfence();
  }
}

// Combines the S partials of each attention output element this CTA owns (S > 1 only).
__device__ void attention_merge(const Params &P, Ctx &c, int S, uint32_t tag) {
  int e0, e1;
  split_rows(QS, c.ncta, c.cta, e0, e1);
  for (int e = e0 + c.warp; e < e1; e += CONS_WARPS) {
    const int hq = e >> 7, d = e & (D - 1);
    float a = 0.f, m = -INFINITY, l = 0.f;
    if (c.lane < S) {
      const unsigned long long *part = P.ll + LL_PART + static_cast<size_t>(hq * MAX_SPLITS + c.lane) * PART_STRIDE;
      a = ll_wait(part + d, tag, c);
      m = ll_wait(part + D, tag, c);
      l = ll_wait(part + D + 1, tag, c);
    }
    const float M = warp_max(m);
    const float sc = (m == -INFINITY) ? 0.f : exp2f(m - M);
    const float L = warp_sum(l * sc), A = warp_sum(a * sc);
    if (c.lane == 0) ll_store(P.ll + LL_ATTN + e, A / L, tag);
  }
}

// ----------------------------------------------------------------------------- the kernel
constexpr size_t SMEM_RING = static_cast<size_t>(NSLOTS) * SLOT_BYTES;
constexpr size_t SMEM_FLOATS = H + H + I + 32 + 2 * D + D + D + CONS_WARPS * 2 * PART_STRIDE + 2 * (D / 2) + 2 * MAX_CTAS + 64;
constexpr size_t SMEM_BYTES = SMEM_RING + SMEM_FLOATS * 4 + 2 * NSLOTS * 8 + 64;

__global__ void __launch_bounds__(THREADS, 1) qwen3_decode_megakernel(const __grid_constant__ Params P) {
  extern __shared__ __align__(128) unsigned char smem[];
  Ctx c;
  c.ring = smem;
  float *f = reinterpret_cast<float *>(smem + SMEM_RING);
  c.s_x = f;            f += H;
  c.s_x1 = f;           f += H;
  c.s_vec = f;          f += I;
  c.s_red = f;          f += 32;
  c.s_q = f;            f += 2 * D;
  c.s_knew = f;         f += D;
  c.s_vnew = f;         f += D;
  c.s_wpart = f;        f += CONS_WARPS * 2 * PART_STRIDE;
  c.s_cs = f;           f += 2 * (D / 2);
  float *s_amax = f;    f += 2 * MAX_CTAS;
  c.s_misc = f;         f += 64;   // [0,1] new-row scores, [16] token, [32..47]/[48..63] warp argmax
  c.full = reinterpret_cast<uint64_t *>(f);
  c.empty = c.full + NSLOTS;
  c.s_flags = reinterpret_cast<volatile int *>(c.empty + NSLOTS);
  c.status = P.status;
  c.timeout_ns = P.timeout_ns;
  c.tid = threadIdx.x;
  c.warp = threadIdx.x >> 5;
  c.lane = threadIdx.x & 31;
  c.cta = blockIdx.x;
  c.ncta = gridDim.x;
  c.chunk = 0;

  if (c.tid == 0) {
    for (int i = 0; i < NSLOTS; ++i) { mbar_init(c.full + i, 1); mbar_init(c.empty + i, CONS_WARPS); }
    c.s_flags[0] = 0; c.s_flags[1] = 0; c.s_flags[2] = 0; c.s_flags[3] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  if (c.warp == CONS_WARPS) {
    if (c.lane == 0) producer_main(P, c);
    __syncwarp();   // the warp meets the block barrier below as a whole
  } else {
    const int S_max = min(MAX_SPLITS, max(1, c.ncta / NKV));
    int token = P.prefill ? P.token_ids[0] : P.first_token;
    LayerW none{};
    for (int step = 0; step < P.num_steps; ++step) {
      const int pos = P.start_position + step;
      const uint32_t tag_base = (P.seq_base + static_cast<uint32_t>(step)) * 64u;
      if (token < 0 || token >= P.vocab) { if (c.tid == 0) raise_error(c, QMK_ERR_BAD_TOKEN, WHERE_TOKEN); token = 0; }
      // cos/sin of this position (fp32 angles, or the caller's fp16 table row)
      if (c.tid < D / 2) {
        float cs, sn;
        if (P.rope_from_table) {
          cs = __half2float(P.cos_table[static_cast<size_t>(pos) * D + c.tid]);
          sn = __half2float(P.sin_table[static_cast<size_t>(pos) * D + c.tid]);
        } else {
          sincosf(static_cast<float>(pos) * c_inv_freq[c.tid], &sn, &cs);
        }
        c.s_cs[c.tid] = cs;
        c.s_cs[64 + c.tid] = sn;
      }
      __threadfence();  // acquire side of the KV-row ordering (rows written in earlier steps)
      int S = pos / max(1, P.split_len);
      S = max(1, min(S, S_max));
      // embedding row -> fp32 residual stream (megakernel_5090.cu:825-830)
      float ss = 0.f;
      {
        const __half *row = P.embed + static_cast<size_t>(token) * H;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const float v = __half2float(__ldg(row + c.tid + j * CONS_THREADS));
          c.s_x[c.tid + j * CONS_THREADS] = v;
          ss = fmaf(v, v, ss);
        }
      }
      for (int layer = 0; layer < P.num_layers; ++layer) {
        const LayerW lw = P.layers[layer];
        const uint32_t tag = tag_base + static_cast<uint32_t>(layer) + 1u;
        uint4 wn[4];
        float a[32];
        // P1: input RMSNorm + fused QKV rows
        load_norm_w(lw.in_ln, c.lane, wn);
        norm_to_regs(c, c.s_x, ss, wn, a);
        consume_phase<PH_QKV>(c, lw, nullptr, 0, [&](const unsigned char *row, const unsigned char *, int out) {
          const float v = row_dot_regs(row, a, c.lane);
          if (c.lane == 0) ll_store(P.ll + LL_QKV + out, v, tag);
        });
        // P2/P3: attention work items, then merge of split partials
        attention_phase(P, c, lw, layer, pos, S, tag);
        if (S > 1) attention_merge(P, c, S, tag);
        // P4: O-proj + residual
        poll_vec<QS>(P.ll + LL_ATTN, tag, c.s_vec, c);
        load_norm_w(lw.post_ln, c.lane, wn);
        cons_sync();
        consume_phase<PH_O>(c, lw, nullptr, 0, [&](const unsigned char *row, const unsigned char *, int out) {
          const float v = row_dot_smem<QS>(row, c.s_vec, c.lane) + c.s_x[out];
          if (c.lane == 0) ll_store(P.ll + LL_X1 + out, v, tag);
        });
        // P5: post-attention RMSNorm + gate/up + SwiGLU
        ss = poll_vec<H>(P.ll + LL_X1, tag, c.s_x1, c);
        norm_to_regs(c, c.s_x1, ss, wn, a);
        consume_phase<PH_GU>(c, lw, nullptr, 0, [&](const unsigned char *grow, const unsigned char *urow, int out) {
          const float gv = row_dot_regs(grow, a, c.lane);
          const float uv = row_dot_regs(urow, a, c.lane);
          if (c.lane == 0) ll_store(P.ll + LL_INTER + out, gv / (1.0f + expf(-gv)) * uv, tag);
        });
        // P6: down-proj + residual
        poll_vec<I>(P.ll + LL_INTER, tag, c.s_vec, c);
        cons_sync();
        consume_phase<PH_DOWN>(c, lw, nullptr, 0, [&](const unsigned char *row, const unsigned char *, int out) {
          const float v = row_dot_smem<I>(row, c.s_vec, c.lane) + c.s_x1[out];
          if (c.lane == 0) ll_store(P.ll + LL_X2 + out, v, tag);
        });
        // next layer's input (in prefill mode the last layer's output is not needed)
        if (!(P.prefill && layer == P.num_layers - 1)) ss = poll_vec<H>(P.ll + LL_X2, tag, c.s_x, c);
        if (cons_any(c.s_flags[0] != 0)) break;
      }
      if (cons_any(c.s_flags[0] != 0)) break;
      if (P.prefill) {
        if (step + 1 < P.num_steps) token = P.token_ids[step + 1];
        continue;
      }
      // final RMSNorm + tied LM head + argmax (megakernel_5090.cu:921-947, 1024-1167)
      {
        uint4 wn[4];
        float a[32];
        load_norm_w(P.final_norm, c.lane, wn);
        norm_to_regs(c, c.s_x, ss, wn, a);
        if (c.cta == 0 && c.warp == 0) {
#pragma unroll
          for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              if (P.normalized_out) P.normalized_out[j * 256 + c.lane * 8 + i] = a[j * 8 + i];
              if (P.hidden_out) P.hidden_out[j * 256 + c.lane * 8 + i] = __float2half_rn(c.s_x[j * 256 + c.lane * 8 + i]);
            }
        }
        float best = -INFINITY;
        int best_i = 0x7fffffff;
        float *dump = P.logits_out ? P.logits_out + static_cast<size_t>(step) * P.vocab : nullptr;
        consume_phase<PH_LM>(c, none, P.lm_head, P.vocab, [&](const unsigned char *row, const unsigned char *, int out) {
          const float v = row_dot_regs(row, a, c.lane);
          if (v > best || (v == best && out < best_i)) { best = v; best_i = out; }
          if (dump && c.lane == 0) dump[out] = v;
        });
        if (c.lane == 0) { c.s_misc[32 + c.warp] = best; c.s_misc[48 + c.warp] = __int_as_float(best_i); }
        cons_sync();
        const uint32_t atag = tag_base + 63u;
        if (c.tid == 0) {
          for (int w = 1; w < CONS_WARPS; ++w) {
            const float v = c.s_misc[32 + w];
            const int vi = __float_as_int(c.s_misc[48 + w]);
            if (v > best || (v == best && vi < best_i)) { best = v; best_i = vi; }
          }
          ll_store(P.ll + LL_AMAX + 2 * c.cta, best, atag);
          ll_store(P.ll + LL_AMAX + 2 * c.cta + 1, __int_as_float(best_i), atag);
          if (P.bmax_vals) P.bmax_vals[c.cta] = best;
          if (P.bmax_idxs) P.bmax_idxs[c.cta] = best_i;
        }
        if (c.tid < 2 * c.ncta) s_amax[c.tid] = ll_wait(P.ll + LL_AMAX + c.tid, atag, c);
        cons_sync();
        if (c.warp == 0) {
          float bv = -INFINITY;
          int bi = 0x7fffffff;
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
          if (c.lane == 0) c.s_misc[16] = __int_as_float(bi);
        }
        const bool aborted = cons_any(c.s_flags[0] != 0);
        token = __float_as_int(c.s_misc[16]);
        if (aborted) break;
        if (c.cta == 0 && c.tid == 0) {
          if (P.output_log) P.output_log[step] = token;   // the EOS token is logged too (megakernel_5090.cu:785-787)
          if (P.output_token) *P.output_token = token;
        }
        if (token == P.eos) break;
      }
    }
    if (c.tid == 0) { c.s_flags[3] = static_cast<int>(c.chunk); c.s_flags[1] = 1; }
  }
  __syncthreads();
  // Bulk copies issued but never consumed (early stop, abort) must land before the CTA exits.
  if (c.tid == CONS_THREADS) {
    // Every slot's latest fill is checked (already-landed phases answer at once), so this also
    // covers chunks the consumers skipped after an abort.
    const uint32_t issued = static_cast<uint32_t>(c.s_flags[2]);
    for (uint32_t i = (issued > NSLOTS ? issued - NSLOTS : 0u); i < issued; ++i) {
      uint64_t *bar = c.full + (i % NSLOTS);
      const uint32_t parity = (i / NSLOTS) & 1u;
      const unsigned long long t0 = now_ns();
      while (!mbar_try_wait(bar, parity)) {
        if (now_ns() - t0 > c.timeout_ns) { raise_error(c, QMK_ERR_WAIT_TIMEOUT, WHERE_DRAIN); break; }
      }
    }
  }
}

// Bounded-wait self test: waits for a tag nothing writes.
__global__ void wait_timeout_probe(unsigned long long *word, unsigned int *status, unsigned long long budget_ns) {
  __shared__ int flags[4];
  if (threadIdx.x == 0) {
    flags[0] = 0;
    Ctx c{};
    c.s_flags = flags;
    c.status = status;
    c.timeout_ns = budget_ns;
    c.cta = blockIdx.x;
    ll_wait(word, 0xfffffff0u, c);
  }
}

}  // namespace qmk

// ============================================================================= host side
namespace {

using qmk::Params;

struct Engine {
  bool ready = false;
  int device = -1;
  int num_sms = 0;
  int grid = 0;
  unsigned long long *ll = nullptr;
  unsigned int *status = nullptr;       // device
  unsigned int *status_host = nullptr;  // pinned
  int *tok_dev = nullptr;
  int tok_cap = 0;
  uint32_t seq = 0;
  int last_status = 0;
  std::string last_error;
  // options
  int vocab = 151936;
  int rope_from_table = 0;
  int split_len = 128;
  int max_ctas = 0;
  int timeout_ms = 2000;
  float *logits_out = nullptr;
  bool inv_freq_set = false;
};

constexpr int MAX_DEVICES = 16;
Engine g_engines[MAX_DEVICES];
std::mutex g_mutex;

Engine *current_engine_unlocked() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return nullptr;
  Engine *e = &g_engines[dev];
  e->device = dev;
  return e;
}

void clear_error(Engine *e) {
  e->last_status = QMK_OK;
  e->last_error.clear();
}

int fail(Engine *e, int code, const std::string &msg) {
  if (e) { e->last_status = code; e->last_error = msg; }
  fprintf(stderr, "[qwen_megakernel] error %d: %s\n", code, msg.c_str());
  return code;
}

#define QMK_CUDA(e, call)                                                                         \
  do {                                                                                            \
    cudaError_t err__ = (call);                                                                   \
    if (err__ != cudaSuccess)                                                                     \
      return fail(e, QMK_ERR_CUDA, std::string(#call) + ": " + cudaGetErrorString(err__));        \
  } while (0)

int ensure_ready(Engine *e) {
  if (e->ready) return QMK_OK;
  cudaDeviceProp prop;
  QMK_CUDA(e, cudaGetDeviceProperties(&prop, e->device));
  if (prop.major < 10) return fail(e, QMK_ERR_CUDA, "this library is built for sm_100a only");
  e->num_sms = prop.multiProcessorCount;
  QMK_CUDA(e, cudaFuncSetAttribute(qmk::qwen3_decode_megakernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   static_cast<int>(qmk::SMEM_BYTES)));
  int per_sm = 0;
  QMK_CUDA(e, cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, qmk::qwen3_decode_megakernel, qmk::THREADS,
                                                            qmk::SMEM_BYTES));
  if (per_sm < 1) return fail(e, QMK_ERR_NOT_RESIDENT, "megakernel does not fit on an SM");
  e->grid = e->num_sms;
  if (e->grid > qmk::MAX_CTAS) e->grid = qmk::MAX_CTAS;
  QMK_CUDA(e, cudaMalloc(&e->ll, sizeof(unsigned long long) * qmk::LL_WORDS));
  QMK_CUDA(e, cudaMemset(e->ll, 0, sizeof(unsigned long long) * qmk::LL_WORDS));
  QMK_CUDA(e, cudaMalloc(&e->status, 16));
  QMK_CUDA(e, cudaMemset(e->status, 0, 16));
  QMK_CUDA(e, cudaHostAlloc(&e->status_host, 16, cudaHostAllocDefault));
  memset(e->status_host, 0, 16);
  if (!e->inv_freq_set) {
    float inv[qmk::D / 2];
    for (int i = 0; i < qmk::D / 2; ++i) inv[i] = static_cast<float>(1.0 / pow(1.0e6, (2.0 * i) / qmk::D));
    QMK_CUDA(e, cudaMemcpyToSymbol(qmk::c_inv_freq, inv, sizeof(inv)));
  }
  e->seq = 0;
  e->ready = true;
  return QMK_OK;
}

int grid_for(const Engine *e) {
  int g = e->grid;
  if (e->max_ctas > 0 && e->max_ctas < g) g = e->max_ctas;
  return g;
}

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Common launch path.  `P` arrives with the per-call fields set.
int launch(Engine *e, Params &P, cudaStream_t stream, bool synchronize) {
  if (P.num_steps <= 0) return QMK_OK;
  if (!P.embed || !P.layers || !P.k_cache || !P.v_cache || (!P.prefill && (!P.final_norm || !P.lm_head)))
    return fail(e, QMK_ERR_BAD_ARGUMENT, "null weight or cache pointer");
  if (!aligned16(P.embed) || !aligned16(P.layers) || !aligned16(P.k_cache) || !aligned16(P.v_cache) ||
      (P.lm_head && !aligned16(P.lm_head)))
    return fail(e, QMK_ERR_BAD_ARGUMENT, "weight, cache and layer-table pointers must be 16-byte aligned");
  if (P.num_layers < 1 || P.num_layers > 60) return fail(e, QMK_ERR_BAD_ARGUMENT, "num_layers must be in [1, 60]");
  if (P.start_position < 0 || P.start_position + P.num_steps > P.max_seq_len)
    return fail(e, QMK_ERR_POSITION, "start_position + steps exceeds max_seq_len");
  if (e->rope_from_table && (!P.cos_table || !P.sin_table))
    return fail(e, QMK_ERR_BAD_ARGUMENT, "rope_from_table needs cos/sin tables");
  int rc = ensure_ready(e);
  if (rc != QMK_OK) return rc;

  // Tags are (sequence number * 64 + layer); restart the sequence before it can wrap.
  if (static_cast<unsigned long long>(e->seq) + static_cast<unsigned long long>(P.num_steps) >= (1ull << 26)) {
    QMK_CUDA(e, cudaMemsetAsync(e->ll, 0, sizeof(unsigned long long) * qmk::LL_WORDS, stream));
    e->seq = 0;
  }
  QMK_CUDA(e, cudaMemsetAsync(e->status, 0, 16, stream));
  P.ll = e->ll;
  P.status = e->status;
  P.seq_base = e->seq;
  P.vocab = e->vocab;
  P.rope_from_table = e->rope_from_table;
  P.split_len = e->split_len;
  P.timeout_ns = static_cast<unsigned long long>(e->timeout_ms) * 1000000ull;
  P.logits_out = P.prefill ? nullptr : e->logits_out;
  e->seq += static_cast<uint32_t>(P.num_steps);

  void *args[] = {&P};
  const int grid = grid_for(e);
  cudaError_t err = cudaLaunchCooperativeKernel(reinterpret_cast<const void *>(qmk::qwen3_decode_megakernel), dim3(grid),
                                                dim3(qmk::THREADS), args, qmk::SMEM_BYTES, stream);
  if (err == cudaErrorCooperativeLaunchTooLarge)
    return fail(e, QMK_ERR_NOT_RESIDENT, "persistent grid cannot be co-resident on this device");
  if (err != cudaSuccess) return fail(e, QMK_ERR_CUDA, std::string("cudaLaunchCooperativeKernel: ") + cudaGetErrorString(err));
  e->last_status = QMK_OK;
  e->last_error.clear();
  if (synchronize) {
    QMK_CUDA(e, cudaMemcpyAsync(e->status_host, e->status, 16, cudaMemcpyDeviceToHost, stream));
    QMK_CUDA(e, cudaStreamSynchronize(stream));
    if (e->status_host[0] != 0) {
      char buf[160];
      snprintf(buf, sizeof(buf), "device status %u (where %u, cta %u)", e->status_host[0], e->status_host[1],
               e->status_host[2]);
      return fail(e, static_cast<int>(e->status_host[0]), buf);
    }
  }
  return QMK_OK;
}

Params base_params(const void *embed, const LDGLayerWeight *layers, const void *final_norm, const void *lm_head,
                   const void *cos_table, const void *sin_table, void *k_cache, void *v_cache, int num_layers,
                   int start_position, int max_seq_len, float attn_scale) {
  Params P;
  memset(&P, 0, sizeof(P));
  P.embed = static_cast<const __half *>(embed);
  P.layers = reinterpret_cast<const qmk::LayerW *>(layers);
  P.final_norm = static_cast<const __half *>(final_norm);
  P.lm_head = static_cast<const __half *>(lm_head);
  P.cos_table = static_cast<const __half *>(cos_table);
  P.sin_table = static_cast<const __half *>(sin_table);
  P.k_cache = static_cast<__half *>(k_cache);
  P.v_cache = static_cast<__half *>(v_cache);
  P.num_layers = num_layers;
  P.start_position = start_position;
  P.max_seq_len = max_seq_len;
  P.attn_scale = attn_scale;
  P.eos = -1;
  return P;
}

}  // namespace

extern "C" {

int qmk_abi_version(void) { return 2; }

int qmk_configure(int vocab_size, int rope_from_table, int split_len, int max_ctas, int timeout_ms) {
  std::lock_guard<std::mutex> lock(g_mutex);
  Engine *e = current_engine_unlocked();
  if (!e) return QMK_ERR_CUDA;
  if (vocab_size == 0 || split_len == 0 || timeout_ms == 0) return fail(e, QMK_ERR_BAD_ARGUMENT, "zero option value");
  if (vocab_size > 0) e->vocab = vocab_size;
  if (rope_from_table >= 0) e->rope_from_table = rope_from_table ? 1 : 0;
  if (split_len > 0) e->split_len = split_len;
  if (max_ctas > 0 && max_ctas < qmk::NKV) return fail(e, QMK_ERR_BAD_ARGUMENT, "max_ctas must be 0 or >= 8");
  if (max_ctas >= 0) e->max_ctas = max_ctas;
  if (timeout_ms > 0) e->timeout_ms = timeout_ms;
  return QMK_OK;
}

int qmk_set_inv_freq(const float *inv_freq64) {
  std::lock_guard<std::mutex> lock(g_mutex);
  Engine *e = current_engine_unlocked();
  if (!e || !inv_freq64) return QMK_ERR_BAD_ARGUMENT;
  QMK_CUDA(e, cudaMemcpyToSymbol(qmk::c_inv_freq, inv_freq64, sizeof(float) * (qmk::D / 2)));
  e->inv_freq_set = true;
  return QMK_OK;
}

int qmk_set_logits_dump(float *logits_out) {
  std::lock_guard<std::mutex> lock(g_mutex);
  Engine *e = current_engine_unlocked();
  if (!e) return QMK_ERR_CUDA;
  e->logits_out = logits_out;
  return QMK_OK;
}

int qmk_decode(int input_token_id, int *output_token_id, const void *embed_weight, const LDGLayerWeight *layer_weights,
               const void *final_norm_weight, const void *lm_head_weight, const void *cos_table, const void *sin_table,
               void *k_cache, void *v_cache, void *hidden_buffer, void *g_normalized, void *block_max_vals,
               void *block_max_idxs, int num_layers, int position, int max_seq_len, float attn_scale,
               cudaStream_t stream) {
  std::lock_guard<std::mutex> lock(g_mutex);
  Engine *e = current_engine_unlocked();
  if (!e) return QMK_ERR_CUDA;
  clear_error(e);
  Params P = base_params(embed_weight, layer_weights, final_norm_weight, lm_head_weight, cos_table, sin_table, k_cache,
                         v_cache, num_layers, position, max_seq_len, attn_scale);
  P.first_token = input_token_id;
  P.num_steps = 1;
  P.output_token = output_token_id;
  P.hidden_out = static_cast<__half *>(hidden_buffer);
  P.normalized_out = static_cast<float *>(g_normalized);
  P.bmax_vals = static_cast<float *>(block_max_vals);
  P.bmax_idxs = static_cast<int *>(block_max_idxs);
  return launch(e, P, stream, false);
}

int qmk_generate(int first_token_id, int num_steps, const void *embed_weight, const LDGLayerWeight *layer_weights,
                 const void *final_norm_weight, const void *lm_head_weight, const void *cos_table,
                 const void *sin_table, void *k_cache, void *v_cache, void *hidden_buffer, void *g_normalized,
                 void *block_max_vals, void *block_max_idxs, int *output_log, int num_layers, int start_position,
                 int max_seq_len, float attn_scale, int eos_token_id, int synchronize, cudaStream_t stream) {
  std::lock_guard<std::mutex> lock(g_mutex);
  Engine *e = current_engine_unlocked();
  if (!e) return QMK_ERR_CUDA;
  clear_error(e);
  if (num_steps > 0 && !output_log) return fail(e, QMK_ERR_BAD_ARGUMENT, "output_log is null");
  Params P = base_params(embed_weight, layer_weights, final_norm_weight, lm_head_weight, cos_table, sin_table, k_cache,
                         v_cache, num_layers, start_position, max_seq_len, attn_scale);
  P.first_token = first_token_id;
  P.num_steps = num_steps;
  P.output_log = output_log;
  P.eos = eos_token_id;
  P.hidden_out = static_cast<__half *>(hidden_buffer);
  P.normalized_out = static_cast<float *>(g_normalized);
  P.bmax_vals = static_cast<float *>(block_max_vals);
  P.bmax_idxs = static_cast<int *>(block_max_idxs);
  return launch(e, P, stream, synchronize != 0);
}

int qmk_prefill(const int *token_ids_host, int num_tokens, const void *embed_weight,
                const LDGLayerWeight *layer_weights, const void *final_norm_weight, const void *cos_table,
                const void *sin_table, void *k_cache, void *v_cache, int num_layers, int start_position,
                int max_seq_len, float attn_scale, cudaStream_t stream) {
  std::lock_guard<std::mutex> lock(g_mutex);
  Engine *e = current_engine_unlocked();
  if (!e) return QMK_ERR_CUDA;
  clear_error(e);
  if (num_tokens <= 0) return QMK_OK;
  if (!token_ids_host) return fail(e, QMK_ERR_BAD_ARGUMENT, "token_ids is null");
  for (int i = 0; i < num_tokens; ++i)
    if (token_ids_host[i] < 0 || token_ids_host[i] >= e->vocab)
      return fail(e, QMK_ERR_BAD_TOKEN, "prompt token outside [0, vocab)");
  if (num_tokens > e->tok_cap) {  // grow-only staging, as the reference keeps (megakernel_5090.cu:1303-1307)
    if (e->tok_dev) cudaFree(e->tok_dev);
    e->tok_dev = nullptr;
    e->tok_cap = 0;
    int cap = 1024;
    while (cap < num_tokens) cap *= 2;
    QMK_CUDA(e, cudaMalloc(&e->tok_dev, sizeof(int) * cap));
    e->tok_cap = cap;
  }
  QMK_CUDA(e, cudaMemcpyAsync(e->tok_dev, token_ids_host, sizeof(int) * num_tokens, cudaMemcpyHostToDevice, stream));
  Params P = base_params(embed_weight, layer_weights, final_norm_weight, nullptr, cos_table, sin_table, k_cache, v_cache,
                         num_layers, start_position, max_seq_len, attn_scale);
  P.prefill = 1;
  P.num_steps = num_tokens;
  P.token_ids = e->tok_dev;
  return launch(e, P, stream, true);
}

int qmk_sync_status(void) {
  std::lock_guard<std::mutex> lock(g_mutex);
  Engine *e = current_engine_unlocked();
  if (!e) return QMK_ERR_CUDA;
  if (!e->ready) return e->last_status;
  QMK_CUDA(e, cudaDeviceSynchronize());
  QMK_CUDA(e, cudaMemcpy(e->status_host, e->status, 16, cudaMemcpyDeviceToHost));
  if (e->status_host[0] != 0) {
    char buf[160];
    snprintf(buf, sizeof(buf), "device status %u (where %u, cta %u)", e->status_host[0], e->status_host[1],
             e->status_host[2]);
    return fail(e, static_cast<int>(e->status_host[0]), buf);
  }
  return e->last_status;
}

const char *qmk_last_error(void) {
  std::lock_guard<std::mutex> lock(g_mutex);
  Engine *e = current_engine_unlocked();
  return e ? e->last_error.c_str() : "no CUDA device";
}

int qmk_num_ctas(void) {
  std::lock_guard<std::mutex> lock(g_mutex);
  Engine *e = current_engine_unlocked();
  if (!e || ensure_ready(e) != QMK_OK) return -1;
  return grid_for(e);
}

long long qmk_scratch_bytes(void) { return static_cast<long long>(sizeof(unsigned long long)) * qmk::LL_WORDS + 16; }

int qmk_selftest_wait_timeout(int budget_us) {
  std::lock_guard<std::mutex> lock(g_mutex);
  Engine *e = current_engine_unlocked();
  if (!e) return QMK_ERR_CUDA;
  int rc = ensure_ready(e);
  if (rc != QMK_OK) return rc;
  if (budget_us < 1 || budget_us > 1000000) return fail(e, QMK_ERR_BAD_ARGUMENT, "budget_us must be in [1, 1e6]");
  QMK_CUDA(e, cudaMemset(e->status, 0, 16));
  qmk::wait_timeout_probe<<<1, 32>>>(e->ll + qmk::LL_AMAX, e->status, static_cast<unsigned long long>(budget_us) * 1000ull);
  QMK_CUDA(e, cudaGetLastError());
  QMK_CUDA(e, cudaDeviceSynchronize());
  QMK_CUDA(e, cudaMemcpy(e->status_host, e->status, 16, cudaMemcpyDeviceToHost));
  const int code = static_cast<int>(e->status_host[0]);
  QMK_CUDA(e, cudaMemset(e->status, 0, 16));
  return code;
}

// ---- reference-signature entry points (qwen_ops.cpp:9-39) ------------------------------------
void launch_ldg_decode_direct(int input_token_id, int *output_token_id, const void *embed_weight,
                              const LDGLayerWeight *layer_weights, const void *final_norm_weight,
                              const void *lm_head_weight, const void *cos_table, const void *sin_table, void *k_cache,
                              void *v_cache, void *hidden_buffer, void *g_activations, void *g_residual, void *g_q,
                              void *g_k, void *g_v, void *g_attn_out, void *g_mlp_intermediate, void *g_normalized,
                              void *block_max_vals, void *block_max_idxs, int num_layers, int position,
                              int max_seq_len, float attn_scale, cudaStream_t stream) {
  (void)g_activations; (void)g_residual; (void)g_q; (void)g_k; (void)g_v; (void)g_attn_out; (void)g_mlp_intermediate;
  qmk_decode(input_token_id, output_token_id, embed_weight, layer_weights, final_norm_weight, lm_head_weight, cos_table,
             sin_table, k_cache, v_cache, hidden_buffer, g_normalized, block_max_vals, block_max_idxs, num_layers,
             position, max_seq_len, attn_scale, stream);
}

void launch_ldg_decode_persistent(int input_token_id, int *output_token_id, const void *embed_weight,
                                  const LDGLayerWeight *layer_weights, const void *final_norm_weight,
                                  const void *lm_head_weight, const void *cos_table, const void *sin_table,
                                  void *k_cache, void *v_cache, void *hidden_buffer, void *g_activations,
                                  void *g_residual, void *g_q, void *g_k, void *g_v, void *g_attn_out,
                                  void *g_mlp_intermediate, void *g_normalized, void *block_max_vals,
                                  void *block_max_idxs, int num_layers, int position, int max_seq_len,
                                  float attn_scale, cudaStream_t stream) {
  launch_ldg_decode_direct(input_token_id, output_token_id, embed_weight, layer_weights, final_norm_weight,
                           lm_head_weight, cos_table, sin_table, k_cache, v_cache, hidden_buffer, g_activations,
                           g_residual, g_q, g_k, g_v, g_attn_out, g_mlp_intermediate, g_normalized, block_max_vals,
                           block_max_idxs, num_layers, position, max_seq_len, attn_scale, stream);
}

void launch_ldg_generate_nosync(int first_token_id, int num_steps, const void *embed_weight,
                                const LDGLayerWeight *layer_weights, const void *final_norm_weight,
                                const void *lm_head_weight, const void *cos_table, const void *sin_table,
                                void *k_cache, void *v_cache, void *hidden_buffer, void *g_activations,
                                void *g_residual, void *g_q, void *g_k, void *g_v, void *g_attn_out,
                                void *g_mlp_intermediate, void *g_normalized, void *block_max_vals,
                                void *block_max_idxs, int *output_log, int num_layers, int start_position,
                                int max_seq_len, float attn_scale, int eos_token_id, cudaStream_t stream) {
  (void)g_activations; (void)g_residual; (void)g_q; (void)g_k; (void)g_v; (void)g_attn_out; (void)g_mlp_intermediate;
  qmk_generate(first_token_id, num_steps, embed_weight, layer_weights, final_norm_weight, lm_head_weight, cos_table,
               sin_table, k_cache, v_cache, hidden_buffer, g_normalized, block_max_vals, block_max_idxs, output_log,
               num_layers, start_position, max_seq_len, attn_scale, eos_token_id, 1, stream);
}

void launch_ldg_prefill(const int *token_ids, int num_tokens, const void *embed_weight,
                        const LDGLayerWeight *layer_weights, const void *final_norm_weight, const void *lm_head_weight,
                        const void *cos_table, const void *sin_table, void *k_cache, void *v_cache,
                        void *hidden_buffer, void *g_activations, void *g_residual, void *g_q, void *g_k, void *g_v,
                        void *g_attn_out, void *g_mlp_intermediate, void *g_normalized, void *block_max_vals,
                        void *block_max_idxs, int num_layers, int start_position, int max_seq_len, float attn_scale,
                        cudaStream_t stream) {
  (void)lm_head_weight; (void)hidden_buffer; (void)g_activations; (void)g_residual; (void)g_q; (void)g_k; (void)g_v;
  (void)g_attn_out; (void)g_mlp_intermediate; (void)g_normalized; (void)block_max_vals; (void)block_max_idxs;
  qmk_prefill(token_ids, num_tokens, embed_weight, layer_weights, final_norm_weight, cos_table, sin_table, k_cache,
              v_cache, num_layers, start_position, max_seq_len, attn_scale, stream);
}

}  // extern "C"
