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
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>
#include <stdlib.h>
#include <math.h>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/qwen_megakernel.h"

#include "megakernel_params.h"

#define QMK_NS qmk
#define QMK_MAX_SEQ 1
#include "megakernel_device.cuh"
#include "megakernel_fused.cuh"
#include "megakernel_batch.h"
#include "megakernel_tc.h"
#include "prefill_sm100.h"
#include "engine_internal.h"

namespace qmk {

// fp32 rotary factors for positions [0, n): angle = float(pos) * inv_freq[i], as the oracle computes them.
__global__ void rope_table_kernel(float *table, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n * (D / 2)) return;
  const int pos = i / (D / 2), f = i % (D / 2);
  float sn, cs;
  sincosf(static_cast<float>(pos) * c_inv_freq[f], &sn, &cs);
  table[static_cast<size_t>(pos) * D + f] = cs;
  table[static_cast<size_t>(pos) * D + 64 + f] = sn;
}

// Bounded-wait self test: waits for a tag nothing writes.
__global__ void wait_timeout_probe(const __grid_constant__ Params P, unsigned long long *word) {
  extern __shared__ __align__(128) unsigned char smem[];
  if (threadIdx.x == 0) {
    Ctx c;
    c.smem = smem;
    c.tid = c.warp = c.lane = 0;
    c.cta = blockIdx.x;
    c.ncta = gridDim.x;
    c.chunk = 0;
    c.repl = 1;
    c.llr = word;
    c.flags()[0] = 0;
    ll_wait(P, c, word, 0xfffffff0u);
  }
}

// ---- K-major copies of W_o and W_down for the fused kernel ------------------------------------------------
// One launch both checks and (re)builds them, so that nothing on the host has to wait for the answer: CTA group
// (layer, matrix) hashes 256 sampled 16-byte pieces of the caller's matrix (and its address), compares the hash
// with the one stored when the copy was made, and transposes again when they differ.  The hashes live in two
// arrays used in turn (read `parity`, write `parity ^ 1`), so that the CTA that stores the new hash cannot change
// what the other CTAs of its group compare against.  A change confined to unsampled elements goes unnoticed:
// callers that edit weights in place call qmk_invalidate_weights().
constexpr int PREP_SUB = 16;      // CTAs per matrix
struct PrepArgs {
  const LayerW *layers;           // the caller's table (device)
  const qmkp::LayerT *out;        // destinations (device)
  unsigned long long *fp;         // [2][2 * num_layers] hashes
  int num_layers, wfmt, parity, force;
};
__global__ void __launch_bounds__(256) kmajor_prepare_kernel(const PrepArgs a) {
  __shared__ unsigned long long s_hash;
  __shared__ int s_redo;
  __shared__ unsigned short tile16[32][33];
  __shared__ unsigned char tile8[32][33];
  const int m = blockIdx.y, l = m >> 1, which = m & 1, t = threadIdx.x;
  const int K = which ? I : QS;                       // inputs of the projection = rows of the K-major copy
  const unsigned char *src = reinterpret_cast<const unsigned char *>(which ? a.layers[l].w_down : a.layers[l].wo);
  unsigned char *dst = reinterpret_cast<unsigned char *>(const_cast<void *>(which ? a.out[l].wd_t : a.out[l].wo_t));
  const size_t in_row = a.wfmt ? static_cast<size_t>(K) + FP8_TRAILER : static_cast<size_t>(K) * 2;
  const size_t n16 = in_row * H / 16;
  if (t == 0) s_hash = reinterpret_cast<unsigned long long>(src) * 0x9E3779B97F4A7C15ull;
  __syncthreads();
  {
    const size_t per = n16 / 256;
    const size_t i16 = static_cast<size_t>(t) * per + (static_cast<size_t>(t) * 37u) % per;
    const uint4 v = __ldg(reinterpret_cast<const uint4 *>(src) + i16);
    unsigned long long h = (static_cast<unsigned long long>(v.x) << 32 | v.y) * 0xD6E8FEB86659FD93ull;
    h ^= (static_cast<unsigned long long>(v.z) << 32 | v.w) * 0xA0761D6478BD642Full;
    h = (h ^ (h >> 29)) * (2ull * static_cast<unsigned long long>(t) + 1ull);
    atomicAdd(&s_hash, h);
  }
  __syncthreads();
  const unsigned long long hash = s_hash;
  const int M = 2 * a.num_layers;
  if (t == 0) {
    s_redo = (a.force || a.fp[static_cast<size_t>(a.parity) * M + m] != hash) ? 1 : 0;
    if (blockIdx.x == 0) a.fp[static_cast<size_t>(a.parity ^ 1) * M + m] = hash;
  }
  __syncthreads();
  if (!s_redo) return;
  const int tx = t & 31, ty = t >> 5;                 // 32 x 8 threads, four rows each per tile
  const int ntiles = (H / 32) * (K / 32);
  for (int tile = blockIdx.x; tile < ntiles; tile += PREP_SUB) {
    const int tn = tile % (H / 32), tk = tile / (H / 32);
    if (a.wfmt == 0) {
      const unsigned short *in = reinterpret_cast<const unsigned short *>(src);
      unsigned short *out = reinterpret_cast<unsigned short *>(dst);
#pragma unroll
      for (int i = 0; i < 4; ++i) tile16[ty + 8 * i][tx] = in[static_cast<size_t>(tn * 32 + ty + 8 * i) * K + tk * 32 + tx];
      __syncthreads();
#pragma unroll
      for (int i = 0; i < 4; ++i) out[static_cast<size_t>(tk * 32 + ty + 8 * i) * H + tn * 32 + tx] = tile16[tx][ty + 8 * i];
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i) tile8[ty + 8 * i][tx] = src[static_cast<size_t>(tn * 32 + ty + 8 * i) * in_row + tk * 32 + tx];
      __syncthreads();
#pragma unroll
      for (int i = 0; i < 4; ++i) dst[static_cast<size_t>(tk * 32 + ty + 8 * i) * H + tn * 32 + tx] = tile8[tx][ty + 8 * i];
    }
    __syncthreads();
  }
  if (a.wfmt && blockIdx.x == 0) {                    // per-output scales follow the K rows
    float *sc = reinterpret_cast<float *>(dst + static_cast<size_t>(K) * H);
    for (int n = t; n < H; n += 256) sc[n] = *reinterpret_cast<const float *>(src + static_cast<size_t>(n) * in_row + K);
  }
}

// ---- scratch for the allocation-free entry point (qmk_generate_static) ----------------------
// Some callers cannot allocate device memory once they are running: a serving process that gave all
// free HBM to its own cache pool at start-up (a later cudaMalloc simply fails), or a loop that cannot
// afford cudaMalloc's device-wide synchronisation.  For them the megakernel's scratch lives in this
// fixed array, which every process that loads the library holds on every GPU it touches until exit:
// the exchange words, an fp32 rotary table for STATIC_MAX_POSITIONS positions, and the status words.
constexpr int STATIC_MAX_POSITIONS = 2048;
constexpr size_t STATIC_LL_BYTES = sizeof(unsigned long long) * LL_WORDS;
constexpr size_t STATIC_ROPE_BYTES = sizeof(float) * D * STATIC_MAX_POSITIONS;
constexpr size_t STATIC_SCRATCH_BYTES = STATIC_LL_BYTES + STATIC_ROPE_BYTES + 64;   // 1,542,208 B
static __device__ __align__(256) unsigned char g_static_scratch[STATIC_SCRATCH_BYTES];

}  // namespace qmk

// ============================================================================= host side
namespace {

using qmkp::Params;

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
  float *rope = nullptr;   // fp32 rotary table for positions [0, rope_cap)
  int rope_cap = 0;
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
  unsigned long long *prof = nullptr;
  int spin_sleep_ns = 600;   // measured: 745 -> 695 us/token; without a pause the polls delay the stores they wait for
  int l2_evict_first = 1;
  int wfmt = 0;              // 0 fp16, 1 fp8-e4m3 rows with scale trailer
  int repl = 4;              // measured: 835 -> 752 us/token at short context, 1152 -> 1061 at 4096
  int stream_inflight = 0;   // measured: pacing the stream changes nothing
  bool inv_freq_set = false;
  float inv_freq[qmk::D / 2] = {};   // host copy of what c_inv_freq holds (when inv_freq_set)
  // fused single-sequence kernel (megakernel_fused.cuh)
  int fused = 2;             // 0: always the unfused kernel; 1: fused, CUDA-core row products; 2: fused, tensor-core row products (fp16 weights)
  int red_copies = 1;
  int decode_attn_mma = 1;   // batched decode: attention on mma.sync (0: the CUDA-core ring kernel)
  int prefill_attn_tc = 1;   // chunked prefill: attention on tcgen05 (0: the mma.sync kernel)
  int step_overlap = 1;      // batched decode: kernels of a step launched as programmatic dependents of one another
  int fused_sleep_ns = 0;    // measured at 4096-token context: 600 ns 1224 tok/s, 200 ns 1259, 0 ns 1305 (few pollers per word)
  unsigned long long *red = nullptr;   // the two residual sums
  struct Prepared {          // K-major copies of W_o / W_down of one caller table
    const void *table = nullptr;
    int num_layers = 0, wfmt = 0, parity = 0, force = 1;
    unsigned char *buf = nullptr;
    qmkp::LayerT *tbl = nullptr;
    unsigned long long *fp = nullptr;
    unsigned long long last_use = 0;
  };
  std::vector<Prepared> prepared;
  unsigned long long use_clock = 0;
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

// One allocation serves both builds of the kernel: [copy][sequence][LL_WORDS] words.
size_t exchange_bytes() {
  size_t words = static_cast<size_t>(qmk::LL_WORDS) * qmk::MAX_REPL;
  if (qmk_batch::exchange_words() > words) words = qmk_batch::exchange_words();
  return words * sizeof(unsigned long long);
}

int ensure_ready(Engine *e) {
  if (e->ready) return QMK_OK;
  cudaDeviceProp prop;
  QMK_CUDA(e, cudaGetDeviceProperties(&prop, e->device));
  if (prop.major < 10) return fail(e, QMK_ERR_CUDA, "this library is built for sm_100a only");
  e->num_sms = prop.multiProcessorCount;
  QMK_CUDA(e, cudaFuncSetAttribute(qmk::qwen3_decode_megakernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   static_cast<int>(qmk::SMEM_BYTES)));
  QMK_CUDA(e, cudaFuncSetAttribute(qmk::qwen3_decode_megakernel_small_grid, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   static_cast<int>(qmk::SMEM_BYTES)));
  QMK_CUDA(e, cudaFuncSetAttribute(qmk::wait_timeout_probe, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   static_cast<int>(qmk::SMEM_BYTES)));
  QMK_CUDA(e, cudaFuncSetAttribute(qmk::qwen3_decode_megakernel_fused, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   static_cast<int>(qmk::SMEM_BYTES)));
  int per_sm = 0;
  QMK_CUDA(e, cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, qmk::qwen3_decode_megakernel, qmk::THREADS,
                                                            qmk::SMEM_BYTES));
  if (per_sm < 1) return fail(e, QMK_ERR_NOT_RESIDENT, "megakernel does not fit on an SM");
  e->grid = e->num_sms;
  if (e->grid > qmk::MAX_CTAS) e->grid = qmk::MAX_CTAS;
  QMK_CUDA(e, cudaFuncSetAttribute(qmk_batch::kernel(), cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   static_cast<int>(qmk_batch::smem_bytes())));
  QMK_CUDA(e, cudaFuncSetAttribute(qmk_fused_tc::kernel(), cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   static_cast<int>(qmk_fused_tc::smem_bytes())));
  QMK_CUDA(e, cudaMalloc(&e->ll, exchange_bytes()));
  QMK_CUDA(e, cudaMemset(e->ll, 0, exchange_bytes()));
  QMK_CUDA(e, cudaMalloc(&e->status, 16));
  QMK_CUDA(e, cudaMemset(e->status, 0, 16));
  QMK_CUDA(e, cudaMalloc(&e->red, sizeof(unsigned long long) * qmk::RED_WORDS));
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

// Entry point of the single-sequence kernel for a grid of `grid` CTAs: small grids, where a projection phase
// has more ring chunks on a CTA than the ring has slots, take the copy with a barrier between passes.
const void *single_sequence_kernel(int grid) {
  static signed char cache[qmk::MAX_CTAS + 1];   // 0 unknown, 1 plain, 2 small grid (a race stores the same value)
  if (grid < 1 || grid > qmk::MAX_CTAS) grid = qmk::MAX_CTAS;
  if (cache[grid] == 0) cache[grid] = qmk::grid_has_long_phase(grid) ? 2 : 1;
  return cache[grid] == 2 ? reinterpret_cast<const void *>(qmk::qwen3_decode_megakernel_small_grid)
                          : reinterpret_cast<const void *>(qmk::qwen3_decode_megakernel);
}

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// fp32 rotary table covering positions [0, max_seq_len): grow-only, like the token staging buffer.
int ensure_rope(Engine *e, int max_seq_len, cudaStream_t stream) {
  if (e->rope_from_table || max_seq_len <= e->rope_cap) return QMK_OK;
  if (e->rope) cudaFree(e->rope);
  e->rope = nullptr;
  e->rope_cap = 0;
  int cap = 2048;
  while (cap < max_seq_len) cap *= 2;
  QMK_CUDA(e, cudaMalloc(&e->rope, sizeof(float) * qmk::D * cap));
  qmk::rope_table_kernel<<<(cap * (qmk::D / 2) + 255) / 256, 256, 0, stream>>>(e->rope, cap);
  QMK_CUDA(e, cudaGetLastError());
  // the table is shared by launches on other streams (overlapped prefill): it is complete before it is published
  QMK_CUDA(e, cudaStreamSynchronize(stream));
  e->rope_cap = cap;
  return QMK_OK;
}

// Bytes of the K-major copies of one layer: O rows then down rows (fp8: each followed by 1024 fp32 scales).
size_t kmajor_o_bytes(int wfmt) {
  const size_t b = wfmt ? static_cast<size_t>(qmk::QS) * qmk::H + qmk::H * 4 : static_cast<size_t>(qmk::QS) * qmk::H * 2;
  return (b + 255) / 256 * 256;
}
size_t kmajor_d_bytes(int wfmt) {
  const size_t b = wfmt ? static_cast<size_t>(qmk::I) * qmk::H + qmk::H * 4 : static_cast<size_t>(qmk::I) * qmk::H * 2;
  return (b + 255) / 256 * 256;
}
void free_prepared(Engine::Prepared &p) {
  if (p.buf) cudaFree(p.buf);
  if (p.tbl) cudaFree(p.tbl);
  if (p.fp) cudaFree(p.fp);
  p = Engine::Prepared();
}
constexpr size_t MAX_PREPARED = 4;   // weight sets kept per device (a 28-layer fp16 set is 294 MB)

// Finds or creates the K-major copies for the caller's layer table and enqueues the check-and-rebuild kernel.
int ensure_prepared(Engine *e, const Params &P, int wfmt, cudaStream_t stream, Engine::Prepared **out) {
  Engine::Prepared *hit = nullptr;
  for (auto &p : e->prepared)
    if (p.table == P.layers && p.num_layers == P.num_layers && p.wfmt == wfmt) hit = &p;
  if (!hit) {
    if (e->prepared.size() >= MAX_PREPARED) {   // drop the set used longest ago
      size_t victim = 0;
      for (size_t i = 1; i < e->prepared.size(); ++i)
        if (e->prepared[i].last_use < e->prepared[victim].last_use) victim = i;
      QMK_CUDA(e, cudaDeviceSynchronize());
      free_prepared(e->prepared[victim]);
      e->prepared.erase(e->prepared.begin() + static_cast<long>(victim));
    }
    Engine::Prepared p;
    p.table = P.layers;
    p.num_layers = P.num_layers;
    p.wfmt = wfmt;
    const size_t ob = kmajor_o_bytes(wfmt), db = kmajor_d_bytes(wfmt);
    QMK_CUDA(e, cudaMalloc(&p.buf, (ob + db) * P.num_layers));
    QMK_CUDA(e, cudaMalloc(&p.tbl, sizeof(qmkp::LayerT) * P.num_layers));
    QMK_CUDA(e, cudaMalloc(&p.fp, sizeof(unsigned long long) * 4 * P.num_layers));
    QMK_CUDA(e, cudaMemsetAsync(p.fp, 0, sizeof(unsigned long long) * 4 * P.num_layers, stream));
    std::vector<qmkp::LayerT> host(P.num_layers);
    for (int l = 0; l < P.num_layers; ++l) {
      host[l].wo_t = p.buf + (ob + db) * l;
      host[l].wd_t = p.buf + (ob + db) * l + ob;
    }
    QMK_CUDA(e, cudaMemcpyAsync(p.tbl, host.data(), sizeof(qmkp::LayerT) * P.num_layers, cudaMemcpyHostToDevice, stream));
    QMK_CUDA(e, cudaStreamSynchronize(stream));   // `host` goes out of scope
    e->prepared.push_back(p);
    hit = &e->prepared.back();
  }
  hit->last_use = ++e->use_clock;
  qmk::PrepArgs a;
  a.layers = P.layers;
  a.out = hit->tbl;
  a.fp = hit->fp;
  a.num_layers = P.num_layers;
  a.wfmt = wfmt;
  a.parity = hit->parity;
  a.force = hit->force;
  qmk::kmajor_prepare_kernel<<<dim3(qmk::PREP_SUB, 2 * P.num_layers), 256, 0, stream>>>(a);
  QMK_CUDA(e, cudaGetLastError());
  hit->parity ^= 1;
  hit->force = 0;
  *out = hit;
  return QMK_OK;
}

// The producer code shared by both builds reads per-sequence entries: entry 0 mirrors the scalar fields.
void mirror_sequence0(Params &P) {
  P.nseq = 1;
  P.first_tokens[0] = P.first_token;
  P.start_positions[0] = P.start_position;
  P.k_caches[0] = P.k_cache;
  P.v_caches[0] = P.v_cache;
  P.output_logs[0] = P.output_log;
}

// Common launch path.  `P` arrives with the per-call fields set; `batch` selects the multi-sequence
// build (per-sequence entries filled by the caller) instead of the single-sequence kernel.
int launch(Engine *e, Params &P, cudaStream_t stream, bool synchronize, bool batch = false) {
  if (P.num_steps <= 0) return QMK_OK;
  if (!batch) mirror_sequence0(P);
  if (!P.embed || !P.layers || (!P.prefill && (!P.final_norm || !P.lm_head)))
    return fail(e, QMK_ERR_BAD_ARGUMENT, "null weight or cache pointer");
  if (!aligned16(P.embed) || !aligned16(P.layers) || (P.lm_head && !aligned16(P.lm_head)))
    return fail(e, QMK_ERR_BAD_ARGUMENT, "weight, cache and layer-table pointers must be 16-byte aligned");
  if (P.num_layers < 1 || P.num_layers > qmk::MAX_LAYERS)
    return fail(e, QMK_ERR_BAD_ARGUMENT, "num_layers must be in [1, 48]");
  for (int b = 0; b < P.nseq; ++b) {
    if (!P.k_caches[b] || !P.v_caches[b]) return fail(e, QMK_ERR_BAD_ARGUMENT, "null weight or cache pointer");
    if (!aligned16(P.k_caches[b]) || !aligned16(P.v_caches[b]))
      return fail(e, QMK_ERR_BAD_ARGUMENT, "weight, cache and layer-table pointers must be 16-byte aligned");
    if (P.start_positions[b] < 0 || P.start_positions[b] + P.num_steps > P.max_seq_len)
      return fail(e, QMK_ERR_POSITION, "start_position + steps exceeds max_seq_len");
  }
  if (e->rope_from_table && (!P.cos_table || !P.sin_table))
    return fail(e, QMK_ERR_BAD_ARGUMENT, "rope_from_table needs cos/sin tables");
  if (e->wfmt == 2)
    return fail(e, QMK_ERR_BAD_ARGUMENT,
                "NVFP4 rows are read by the tensor-core entry points only (qmk_prefill_chunked, qmk_decode_batched)");
  int rc = ensure_ready(e);
  if (rc != QMK_OK) return rc;

  // Tags are (sequence number * 64 + layer); restart the sequence before it can wrap.
  if (static_cast<unsigned long long>(e->seq) + static_cast<unsigned long long>(P.num_steps) >= (1ull << 26)) {
    QMK_CUDA(e, cudaMemsetAsync(e->ll, 0, exchange_bytes(), stream));
    e->seq = 0;
  }
  rc = ensure_rope(e, P.max_seq_len, stream);
  if (rc != QMK_OK) return rc;
  P.rope = e->rope;
  QMK_CUDA(e, cudaMemsetAsync(e->status, 0, 16, stream));
  P.ll = e->ll;
  P.status = e->status;
  P.seq_base = e->seq;
  P.vocab = e->vocab;
  P.rope_from_table = e->rope_from_table;
  P.split_len = e->split_len;
  P.timeout_ns = static_cast<unsigned long long>(e->timeout_ms) * 1000000ull;
  P.logits_out = P.prefill ? nullptr : e->logits_out;
  P.prof = e->prof;
  P.spin_sleep_ns = e->spin_sleep_ns;
  P.l2_evict_first = e->l2_evict_first;
  P.repl = e->repl;
  P.wfmt = e->wfmt;
  P.stream_inflight = e->stream_inflight;
  e->seq += static_cast<uint32_t>(P.num_steps);

  void *args[] = {&P};
  const int grid = grid_for(e);
  const void *kernel = batch ? qmk_batch::kernel() : single_sequence_kernel(grid);
  size_t smem = qmk::SMEM_BYTES;
  if (!batch && e->fused && grid >= qmk::FUSED_MIN_CTAS &&
      kernel == reinterpret_cast<const void *>(qmk::qwen3_decode_megakernel)) {
    // fused kernel: O and down projections as split-K slices of K-major copies, two all-reduced residual sums
    Engine::Prepared *prep = nullptr;
    rc = ensure_prepared(e, P, e->wfmt, stream, &prep);
    if (rc != QMK_OK) return rc;
    QMK_CUDA(e, cudaMemsetAsync(e->red, 0, sizeof(unsigned long long) * qmk::RED_WORDS, stream));
    P.layers_t = prep->tbl;
    P.red = e->red;
    P.red_copies = e->red_copies;
    P.spin_sleep_ns = e->fused_sleep_ns;
    kernel = reinterpret_cast<const void *>(qmk::qwen3_decode_megakernel_fused);
    // row products on the tensor cores: fp16 weights, rows owned in units of four
    if (e->fused >= 2 && e->wfmt == 0 && P.vocab % 4 == 0 && grid >= qmk_fused_tc::min_ctas()) {
      // tiled-copy descriptors of the caller's caches (host-side encode, a few microseconds)
      std::string merr;
      const uint64_t kv_rows = static_cast<uint64_t>(P.num_layers) * qmk::NKV * static_cast<uint64_t>(P.max_seq_len);
      rc = qmk_tc::make_map_f16(reinterpret_cast<CUtensorMap *>(P.kmap), P.k_cache, kv_rows, qmk::D, 16, &merr);
      if (rc == QMK_OK) rc = qmk_tc::make_map_f16(reinterpret_cast<CUtensorMap *>(P.vmap), P.v_cache, kv_rows, qmk::D, 16, &merr);
      if (rc != QMK_OK) return fail(e, rc, "KV cache tensor map: " + merr);
      kernel = qmk_fused_tc::kernel();
      smem = qmk_fused_tc::smem_bytes();
    }
  }
  cudaError_t err =
      batch ? cudaLaunchCooperativeKernel(kernel, dim3(grid), dim3(qmk_batch::threads()), args,
                                          qmk_batch::smem_bytes(), stream)
            : cudaLaunchCooperativeKernel(kernel, dim3(grid), dim3(qmk::THREADS), args, smem, stream);
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

namespace qmk_internal {
int prefill_env(int max_seq_len, cudaStream_t stream, PrefillEnv *out) {
  std::lock_guard<std::mutex> lock(g_mutex);
  Engine *e = current_engine_unlocked();
  if (!e) return QMK_ERR_CUDA;
  clear_error(e);
  int rc = ensure_ready(e);
  if (rc == QMK_OK) rc = ensure_rope(e, max_seq_len, stream);
  if (rc != QMK_OK) return rc;
  out->rope = e->rope;
  out->vocab = e->vocab;
  out->timeout_ms = e->timeout_ms;
  out->wfmt = e->wfmt;
  out->rope_from_table = e->rope_from_table;
  out->logits_out = e->logits_out;
  out->pdl = e->step_overlap;
  out->attn_tc = e->prefill_attn_tc;
  out->attn_mma = e->decode_attn_mma;
  return QMK_OK;
}
int report(int code, const std::string &msg) {
  std::lock_guard<std::mutex> lock(g_mutex);
  return fail(current_engine_unlocked(), code, msg);
}
}  // namespace qmk_internal

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
  // callers re-apply their options before every op: the same frequencies again cost nothing
  if (e->inv_freq_set && memcmp(e->inv_freq, inv_freq64, sizeof(e->inv_freq)) == 0) return QMK_OK;
  QMK_CUDA(e, cudaDeviceSynchronize());   // no launch may still be reading the old table
  QMK_CUDA(e, cudaMemcpyToSymbol(qmk::c_inv_freq, inv_freq64, sizeof(float) * (qmk::D / 2)));
  memcpy(e->inv_freq, inv_freq64, sizeof(e->inv_freq));
  e->inv_freq_set = true;
  e->rope_cap = 0;   // rebuilt with the new frequencies at the next launch
  return QMK_OK;
}

int qmk_set_logits_dump(float *logits_out) {
  std::lock_guard<std::mutex> lock(g_mutex);
  Engine *e = current_engine_unlocked();
  if (!e) return QMK_ERR_CUDA;
  e->logits_out = logits_out;
  return QMK_OK;
}

int qmk_set_weight_format(int format) {
  std::lock_guard<std::mutex> lock(g_mutex);
  Engine *e = current_engine_unlocked();
  if (!e) return QMK_ERR_CUDA;
  if (format < 0 || format > 2)
    return fail(e, QMK_ERR_BAD_ARGUMENT, "weight format must be 0 (fp16), 1 (fp8-e4m3 rows) or 2 (nvfp4 rows)");
  e->wfmt = format;
  return QMK_OK;
}

int qmk_set_prefill_attention(int tensor_core) {
  std::lock_guard<std::mutex> lock(g_mutex);
  Engine *e = current_engine_unlocked();
  if (!e) return QMK_ERR_CUDA;
  if (tensor_core >= 0) e->prefill_attn_tc = tensor_core ? 1 : 0;
  return QMK_OK;
}

int qmk_set_decode_attention(int tensor_core) {
  std::lock_guard<std::mutex> lock(g_mutex);
  Engine *e = current_engine_unlocked();
  if (!e) return QMK_ERR_CUDA;
  if (tensor_core >= 0) e->decode_attn_mma = tensor_core ? 1 : 0;
  return QMK_OK;
}

int qmk_set_step_overlap(int enabled) {
  std::lock_guard<std::mutex> lock(g_mutex);
  Engine *e = current_engine_unlocked();
  if (!e) return QMK_ERR_CUDA;
  if (enabled >= 0) e->step_overlap = enabled ? 1 : 0;
  return QMK_OK;
}

int qmk_set_tuning2(int repl, int stream_inflight) {
  std::lock_guard<std::mutex> lock(g_mutex);
  Engine *e = current_engine_unlocked();
  if (!e) return QMK_ERR_CUDA;
  if (repl == 1 || repl == 2 || repl == 4) e->repl = repl;
  else if (repl >= 0) return fail(e, QMK_ERR_BAD_ARGUMENT, "repl must be 1, 2 or 4");
  if (stream_inflight >= 0) e->stream_inflight = stream_inflight > qmk::NSLOTS ? qmk::NSLOTS : stream_inflight;
  return QMK_OK;
}

int qmk_set_tuning(int spin_sleep_ns, int l2_evict_first) {
  std::lock_guard<std::mutex> lock(g_mutex);
  Engine *e = current_engine_unlocked();
  if (!e) return QMK_ERR_CUDA;
  if (spin_sleep_ns >= 0) e->spin_sleep_ns = e->fused_sleep_ns = spin_sleep_ns > 10000 ? 10000 : spin_sleep_ns;
  if (l2_evict_first >= 0) e->l2_evict_first = l2_evict_first ? 1 : 0;
  return QMK_OK;
}

int qmk_set_fused(int fused, int red_copies) {
  std::lock_guard<std::mutex> lock(g_mutex);
  Engine *e = current_engine_unlocked();
  if (!e) return QMK_ERR_CUDA;
  if (fused > 2) return fail(e, QMK_ERR_BAD_ARGUMENT, "fused must be 0, 1 or 2");
  if (fused >= 0) e->fused = fused;
  if (red_copies == 1 || red_copies == 2) e->red_copies = red_copies;
  else if (red_copies >= 0) return fail(e, QMK_ERR_BAD_ARGUMENT, "red_copies must be 1 or 2");
  return QMK_OK;
}

int qmk_invalidate_weights(void) {
  std::lock_guard<std::mutex> lock(g_mutex);
  Engine *e = current_engine_unlocked();
  if (!e) return QMK_ERR_CUDA;
  for (auto &p : e->prepared) p.force = 1;
  return QMK_OK;
}

int qmk_release_weights(const LDGLayerWeight *layer_weights) {
  std::lock_guard<std::mutex> lock(g_mutex);
  Engine *e = current_engine_unlocked();
  if (!e) return QMK_ERR_CUDA;
  for (size_t i = 0; i < e->prepared.size();) {
    if (layer_weights == nullptr || e->prepared[i].table == layer_weights) {
      QMK_CUDA(e, cudaDeviceSynchronize());
      free_prepared(e->prepared[i]);
      e->prepared.erase(e->prepared.begin() + static_cast<long>(i));
    } else {
      ++i;
    }
  }
  return QMK_OK;
}

int qmk_set_profile_buffer(unsigned long long *timestamps) {
  std::lock_guard<std::mutex> lock(g_mutex);
  Engine *e = current_engine_unlocked();
  if (!e) return QMK_ERR_CUDA;
  e->prof = timestamps;
  return QMK_OK;
}

}  // extern "C"

namespace {
int decode_unlocked(int input_token_id, int *output_token_id, const void *embed_weight, const LDGLayerWeight *layer_weights,
                    const void *final_norm_weight, const void *lm_head_weight, const void *cos_table, const void *sin_table,
                    void *k_cache, void *v_cache, void *hidden_buffer, void *g_normalized, void *block_max_vals,
                    void *block_max_idxs, int num_layers, int position, int max_seq_len, float attn_scale,
                    cudaStream_t stream) {
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

int generate_unlocked(int first_token_id, int num_steps, const void *embed_weight, const LDGLayerWeight *layer_weights,
                      const void *final_norm_weight, const void *lm_head_weight, const void *cos_table,
                      const void *sin_table, void *k_cache, void *v_cache, void *hidden_buffer, void *g_normalized,
                      void *block_max_vals, void *block_max_idxs, int *output_log, int num_layers, int start_position,
                      int max_seq_len, float attn_scale, int eos_token_id, int synchronize, cudaStream_t stream) {
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
}  // namespace

extern "C" {

int qmk_decode(int input_token_id, int *output_token_id, const void *embed_weight, const LDGLayerWeight *layer_weights,
               const void *final_norm_weight, const void *lm_head_weight, const void *cos_table, const void *sin_table,
               void *k_cache, void *v_cache, void *hidden_buffer, void *g_normalized, void *block_max_vals,
               void *block_max_idxs, int num_layers, int position, int max_seq_len, float attn_scale,
               cudaStream_t stream) {
  std::lock_guard<std::mutex> lock(g_mutex);
  return decode_unlocked(input_token_id, output_token_id, embed_weight, layer_weights, final_norm_weight, lm_head_weight,
                         cos_table, sin_table, k_cache, v_cache, hidden_buffer, g_normalized, block_max_vals, block_max_idxs,
                         num_layers, position, max_seq_len, attn_scale, stream);
}

int qmk_generate(int first_token_id, int num_steps, const void *embed_weight, const LDGLayerWeight *layer_weights,
                 const void *final_norm_weight, const void *lm_head_weight, const void *cos_table,
                 const void *sin_table, void *k_cache, void *v_cache, void *hidden_buffer, void *g_normalized,
                 void *block_max_vals, void *block_max_idxs, int *output_log, int num_layers, int start_position,
                 int max_seq_len, float attn_scale, int eos_token_id, int synchronize, cudaStream_t stream) {
  std::lock_guard<std::mutex> lock(g_mutex);
  return generate_unlocked(first_token_id, num_steps, embed_weight, layer_weights, final_norm_weight, lm_head_weight,
                           cos_table, sin_table, k_cache, v_cache, hidden_buffer, g_normalized, block_max_vals,
                           block_max_idxs, output_log, num_layers, start_position, max_seq_len, attn_scale, eos_token_id,
                           synchronize, stream);
}

int qmk_generate_batch(int num_sequences, const int *first_token_ids, const int *start_positions, int num_steps,
                       const void *embed_weight, const LDGLayerWeight *layer_weights, const void *final_norm_weight,
                       const void *lm_head_weight, const void *cos_table, const void *sin_table, void *const *k_caches,
                       void *const *v_caches, int *const *output_logs, int num_layers, int max_seq_len, float attn_scale,
                       int synchronize, cudaStream_t stream) {
  std::lock_guard<std::mutex> lock(g_mutex);
  Engine *e = current_engine_unlocked();
  if (!e) return QMK_ERR_CUDA;
  clear_error(e);
  if (num_sequences < 1 || num_sequences > qmkp::MAX_SEQ)
    return fail(e, QMK_ERR_BAD_ARGUMENT, "qmk_generate_batch: num_sequences must be 1, 2, 3 or 4");
  if (!first_token_ids || !start_positions || !k_caches || !v_caches || !output_logs)
    return fail(e, QMK_ERR_BAD_ARGUMENT, "qmk_generate_batch: null array argument");
  Params P = base_params(embed_weight, layer_weights, final_norm_weight, lm_head_weight, cos_table, sin_table, nullptr,
                         nullptr, num_layers, 0, max_seq_len, attn_scale);
  P.num_steps = num_steps;
  P.nseq = num_sequences;
  for (int b = 0; b < num_sequences; ++b) {
    if (num_steps > 0 && !output_logs[b]) return fail(e, QMK_ERR_BAD_ARGUMENT, "output_log is null");
    if (first_token_ids[b] < 0 || first_token_ids[b] >= e->vocab)
      return fail(e, QMK_ERR_BAD_TOKEN, "first token outside [0, vocab)");
    for (int a = 0; a < b; ++a)
      if (k_caches[a] == k_caches[b] || v_caches[a] == v_caches[b] || output_logs[a] == output_logs[b])
        return fail(e, QMK_ERR_BAD_ARGUMENT, "qmk_generate_batch: two sequences share a cache or an output log");
    P.first_tokens[b] = first_token_ids[b];
    P.start_positions[b] = start_positions[b];
    P.k_caches[b] = static_cast<__half *>(k_caches[b]);
    P.v_caches[b] = static_cast<__half *>(v_caches[b]);
    P.output_logs[b] = output_logs[b];
  }
  for (int b = num_sequences; b < qmkp::MAX_SEQ; ++b) {   // unused entries repeat entry 0 (never dereferenced)
    P.first_tokens[b] = P.first_tokens[0];
    P.start_positions[b] = P.start_positions[0];
    P.k_caches[b] = P.k_caches[0];
    P.v_caches[b] = P.v_caches[0];
    P.output_logs[b] = P.output_logs[0];
  }
  return launch(e, P, stream, synchronize != 0, true);
}

}  // extern "C"

namespace {
int prefill_unlocked(const int *token_ids_host, int num_tokens, const void *embed_weight,
                     const LDGLayerWeight *layer_weights, const void *final_norm_weight, const void *cos_table,
                     const void *sin_table, void *k_cache, void *v_cache, int num_layers, int start_position,
                     int max_seq_len, float attn_scale, cudaStream_t stream) {
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

// ---- engine handles ------------------------------------------------------------------------------------------
// The per-device state above (scratch, options) is shared by everything that decodes on a GPU.  A handle is one
// client's view of it: its own options (vocabulary, weight format, RoPE mode and frequencies, grid cap, split length,
// time-out, kernel choice) and its own K-major weight copies.  Every handle call makes the handle's options current
// and runs the op under ONE hold of the lock, so clients with different options can share a GPU from several threads.
}  // namespace

struct qmk_engine {
  int device = 0;
  qmk_engine_config cfg;
  float inv_freq[qmk::D / 2];
  std::vector<const void *> tables;   // layer tables this handle decoded with (their K-major copies die with it)
};

namespace {
int apply_handle_unlocked(qmk_engine *h, const void *table) {
  if (!h) return QMK_ERR_BAD_ARGUMENT;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return QMK_ERR_CUDA;
  if (dev != h->device && cudaSetDevice(h->device) != cudaSuccess) return QMK_ERR_CUDA;
  Engine *e = current_engine_unlocked();
  if (!e) return QMK_ERR_CUDA;
  const qmk_engine_config &c = h->cfg;
  e->vocab = c.vocab_size > 0 ? c.vocab_size : 151936;   // a handle never inherits another client's values
  e->rope_from_table = c.rope_from_table ? 1 : 0;
  if (c.split_len > 0) e->split_len = c.split_len;      // speed / debugging knobs: non-positive leaves qmk_configure's value
  if (c.max_ctas > 0) e->max_ctas = c.max_ctas;
  if (c.timeout_ms > 0) e->timeout_ms = c.timeout_ms;
  e->wfmt = c.weight_format;
  if (c.fused >= 0) e->fused = c.fused;   // a speed knob, not a property of the weights: negative leaves qmk_set_fused's value
  if ((!e->inv_freq_set || memcmp(e->inv_freq, h->inv_freq, sizeof(h->inv_freq)) != 0)) {
    QMK_CUDA(e, cudaDeviceSynchronize());   // no launch may still be reading the old table
    QMK_CUDA(e, cudaMemcpyToSymbol(qmk::c_inv_freq, h->inv_freq, sizeof(h->inv_freq)));
    memcpy(e->inv_freq, h->inv_freq, sizeof(h->inv_freq));
    e->inv_freq_set = true;
    e->rope_cap = 0;
  }
  if (table) {
    bool seen = false;
    for (const void *t : h->tables) seen |= (t == table);
    if (!seen) h->tables.push_back(table);
  }
  return QMK_OK;
}
}  // namespace

extern "C" {

int qmk_prefill(const int *token_ids_host, int num_tokens, const void *embed_weight,
                const LDGLayerWeight *layer_weights, const void *final_norm_weight, const void *cos_table,
                const void *sin_table, void *k_cache, void *v_cache, int num_layers, int start_position,
                int max_seq_len, float attn_scale, cudaStream_t stream) {
  std::lock_guard<std::mutex> lock(g_mutex);
  return prefill_unlocked(token_ids_host, num_tokens, embed_weight, layer_weights, final_norm_weight, cos_table, sin_table,
                          k_cache, v_cache, num_layers, start_position, max_seq_len, attn_scale, stream);
}

int qmk_engine_create(const qmk_engine_config *config, qmk_engine **out) {
  if (!config || !out) return QMK_ERR_BAD_ARGUMENT;
  if (config->weight_format < 0 || config->weight_format > 2) return QMK_ERR_BAD_ARGUMENT;
  if (config->fused > 2 || (config->max_ctas > 0 && config->max_ctas < qmk::NKV)) return QMK_ERR_BAD_ARGUMENT;
  int ndev = 0;
  if (cudaGetDeviceCount(&ndev) != cudaSuccess || config->device < 0 || config->device >= ndev || config->device >= MAX_DEVICES)
    return QMK_ERR_CUDA;
  qmk_engine *h = new qmk_engine();
  h->device = config->device;
  h->cfg = *config;
  if (config->inv_freq64) {
    memcpy(h->inv_freq, config->inv_freq64, sizeof(h->inv_freq));
  } else {   // the library's default: theta = 1e6
    for (int i = 0; i < qmk::D / 2; ++i) h->inv_freq[i] = static_cast<float>(1.0 / pow(1.0e6, (2.0 * i) / qmk::D));
  }
  h->cfg.inv_freq64 = nullptr;   // copied: the caller's array need not outlive the call
  *out = h;
  return QMK_OK;
}

int qmk_engine_destroy(qmk_engine *h) {
  if (!h) return QMK_OK;
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    int prev = 0;
    cudaGetDevice(&prev);
    if (cudaSetDevice(h->device) == cudaSuccess) {
      Engine *e = current_engine_unlocked();
      if (e) {
        for (size_t i = 0; i < e->prepared.size();) {
          bool mine = false;
          for (const void *t : h->tables) mine |= (t == e->prepared[i].table);
          if (mine) {
            cudaDeviceSynchronize();
            free_prepared(e->prepared[i]);
            e->prepared.erase(e->prepared.begin() + static_cast<long>(i));
          } else {
            ++i;
          }
        }
      }
      cudaSetDevice(prev);
    }
  }
  delete h;
  return QMK_OK;
}

int qmk_engine_apply(qmk_engine *h) {
  std::lock_guard<std::mutex> lock(g_mutex);
  return apply_handle_unlocked(h, nullptr);
}

int qmk_engine_decode(qmk_engine *h, int input_token_id, int *output_token_id, const void *embed_weight,
                      const LDGLayerWeight *layer_weights, const void *final_norm_weight, const void *lm_head_weight,
                      const void *cos_table, const void *sin_table, void *k_cache, void *v_cache, void *hidden_buffer,
                      void *g_normalized, void *block_max_vals, void *block_max_idxs, int num_layers, int position,
                      int max_seq_len, float attn_scale, cudaStream_t stream) {
  std::lock_guard<std::mutex> lock(g_mutex);
  const int rc = apply_handle_unlocked(h, layer_weights);
  if (rc != QMK_OK) return rc;
  return decode_unlocked(input_token_id, output_token_id, embed_weight, layer_weights, final_norm_weight, lm_head_weight,
                         cos_table, sin_table, k_cache, v_cache, hidden_buffer, g_normalized, block_max_vals, block_max_idxs,
                         num_layers, position, max_seq_len, attn_scale, stream);
}

int qmk_engine_generate(qmk_engine *h, int first_token_id, int num_steps, const void *embed_weight,
                        const LDGLayerWeight *layer_weights, const void *final_norm_weight, const void *lm_head_weight,
                        const void *cos_table, const void *sin_table, void *k_cache, void *v_cache, void *hidden_buffer,
                        void *g_normalized, void *block_max_vals, void *block_max_idxs, int *output_log, int num_layers,
                        int start_position, int max_seq_len, float attn_scale, int eos_token_id, int synchronize,
                        cudaStream_t stream) {
  std::lock_guard<std::mutex> lock(g_mutex);
  const int rc = apply_handle_unlocked(h, layer_weights);
  if (rc != QMK_OK) return rc;
  return generate_unlocked(first_token_id, num_steps, embed_weight, layer_weights, final_norm_weight, lm_head_weight,
                           cos_table, sin_table, k_cache, v_cache, hidden_buffer, g_normalized, block_max_vals,
                           block_max_idxs, output_log, num_layers, start_position, max_seq_len, attn_scale, eos_token_id,
                           synchronize, stream);
}

int qmk_engine_prefill(qmk_engine *h, const int *token_ids_host, int num_tokens, const void *embed_weight,
                       const LDGLayerWeight *layer_weights, const void *final_norm_weight, const void *cos_table,
                       const void *sin_table, void *k_cache, void *v_cache, int num_layers, int start_position,
                       int max_seq_len, float attn_scale, cudaStream_t stream) {
  std::lock_guard<std::mutex> lock(g_mutex);
  const int rc = apply_handle_unlocked(h, layer_weights);
  if (rc != QMK_OK) return rc;
  return prefill_unlocked(token_ids_host, num_tokens, embed_weight, layer_weights, final_norm_weight, cos_table, sin_table,
                          k_cache, v_cache, num_layers, start_position, max_seq_len, attn_scale, stream);
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
  // a copy per calling thread, taken under the lock: another thread's next call may rewrite the engine's string
  static thread_local std::string mine;
  std::lock_guard<std::mutex> lock(g_mutex);
  Engine *e = current_engine_unlocked();
  mine = e ? e->last_error : std::string("no CUDA device");
  return mine.c_str();
}

int qmk_num_ctas(void) {
  std::lock_guard<std::mutex> lock(g_mutex);
  Engine *e = current_engine_unlocked();
  if (!e || ensure_ready(e) != QMK_OK) return -1;
  return grid_for(e);
}

long long qmk_scratch_bytes(void) {
  return static_cast<long long>(exchange_bytes()) + 16;
}

int qmk_selftest_wait_timeout(int budget_us) {
  std::lock_guard<std::mutex> lock(g_mutex);
  Engine *e = current_engine_unlocked();
  if (!e) return QMK_ERR_CUDA;
  int rc = ensure_ready(e);
  if (rc != QMK_OK) return rc;
  if (budget_us < 1 || budget_us > 1000000) return fail(e, QMK_ERR_BAD_ARGUMENT, "budget_us must be in [1, 1e6]");
  QMK_CUDA(e, cudaMemset(e->status, 0, 16));
  Params P;
  memset(&P, 0, sizeof(P));
  P.status = e->status;
  P.timeout_ns = static_cast<unsigned long long>(budget_us) * 1000ull;
  qmk::wait_timeout_probe<<<1, 32, qmk::SMEM_BYTES>>>(P, e->ll + qmk::LL_AMAX);
  QMK_CUDA(e, cudaGetLastError());
  QMK_CUDA(e, cudaDeviceSynchronize());
  QMK_CUDA(e, cudaMemcpy(e->status_host, e->status, 16, cudaMemcpyDeviceToHost));
  const int code = static_cast<int>(e->status_host[0]);
  QMK_CUDA(e, cudaMemset(e->status, 0, 16));
  return code;
}

// ---- allocation-free variant ------------------------------------------------------------------
// Same kernel and same results as qmk_generate, but nothing here (or below it) calls cudaMalloc,
// cudaFree, cudaHostAlloc or any other allocating routine: the scratch is qmk::g_static_scratch.
// In host code that name is only a stand-in for the device array, not an address a kernel can use,
// so the first call on each device (with that device current) asks the runtime for the real device
// address with cudaGetSymbolAddress and keeps it.  That first call also opts the kernel into its
// shared-memory size; make it before any stream capture starts.
// All calls on a device share the one array and it keeps what the previous call left in it: the
// status words are cleared and the rotary table is rebuilt at the start of every call, the exchange
// words are told apart by their tags (and cleared when the tag sequence restarts).  Two calls that
// overlap on the GPU (two qmk_generate_static calls on different streams of one device) would race on
// the array; keep them on one stream.  (qmk_generate has its own, allocated, scratch.)
struct StaticState {
  bool ready = false;
  unsigned char *base = nullptr;   // device address of qmk::g_static_scratch on this device
  int grid = 0;
  uint32_t seq = 0;
};
StaticState g_static[MAX_DEVICES];

int qmk_generate_static(int first_token_id, int num_steps, const void *embed_weight,
                        const LDGLayerWeight *layer_weights, const void *final_norm_weight,
                        const void *lm_head_weight, void *k_cache, void *v_cache, void *g_normalized,
                        int *output_log, int num_layers, int start_position, int max_seq_len, float attn_scale,
                        int eos_token_id, cudaStream_t stream) {
  std::lock_guard<std::mutex> lock(g_mutex);
  Engine *e = current_engine_unlocked();
  if (!e) return QMK_ERR_CUDA;
  clear_error(e);
  if (num_steps <= 0) return QMK_OK;
  if (!output_log || !embed_weight || !layer_weights || !final_norm_weight || !lm_head_weight || !k_cache || !v_cache)
    return fail(e, QMK_ERR_BAD_ARGUMENT, "qmk_generate_static: null pointer argument");
  if (e->wfmt == 2) return fail(e, QMK_ERR_BAD_ARGUMENT, "qmk_generate_static reads fp16 or FP8-E4M3 rows, not NVFP4");
  if (!aligned16(embed_weight) || !aligned16(layer_weights) || !aligned16(lm_head_weight) || !aligned16(k_cache) ||
      !aligned16(v_cache))
    return fail(e, QMK_ERR_BAD_ARGUMENT, "weight, cache and layer-table pointers must be 16-byte aligned");
  if (num_layers < 1 || num_layers > qmk::MAX_LAYERS)
    return fail(e, QMK_ERR_BAD_ARGUMENT, "num_layers must be in [1, 48]");
  if (max_seq_len > qmk::STATIC_MAX_POSITIONS) {
    char buf[160];
    snprintf(buf, sizeof(buf), "qmk_generate_static: max_seq_len %d exceeds the static scratch limit of %d positions",
             max_seq_len, qmk::STATIC_MAX_POSITIONS);
    return fail(e, QMK_ERR_BAD_ARGUMENT, buf);
  }
  if (start_position < 0 || start_position + num_steps > max_seq_len)
    return fail(e, QMK_ERR_POSITION, "start_position + steps exceeds max_seq_len");

  StaticState &st = g_static[e->device];
  if (!st.ready) {   // once per device, with that device current
    cudaDeviceProp prop;
    QMK_CUDA(e, cudaGetDeviceProperties(&prop, e->device));
    if (prop.major < 10) return fail(e, QMK_ERR_CUDA, "this library is built for sm_100a only");
    QMK_CUDA(e, cudaFuncSetAttribute(qmk::qwen3_decode_megakernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     static_cast<int>(qmk::SMEM_BYTES)));
    QMK_CUDA(e, cudaFuncSetAttribute(qmk::qwen3_decode_megakernel_small_grid, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     static_cast<int>(qmk::SMEM_BYTES)));
    void *dev_ptr = nullptr;
    QMK_CUDA(e, cudaGetSymbolAddress(&dev_ptr, qmk::g_static_scratch));
    st.base = static_cast<unsigned char *>(dev_ptr);
    st.grid = prop.multiProcessorCount < qmk::MAX_CTAS ? prop.multiProcessorCount : qmk::MAX_CTAS;
    if (!e->inv_freq_set && !e->ready) {   // same default frequencies as the allocating path (theta = 1e6)
      float inv[qmk::D / 2];
      for (int i = 0; i < qmk::D / 2; ++i) inv[i] = static_cast<float>(1.0 / pow(1.0e6, (2.0 * i) / qmk::D));
      QMK_CUDA(e, cudaMemcpyToSymbol(qmk::c_inv_freq, inv, sizeof(inv)));
    }
    QMK_CUDA(e, cudaMemsetAsync(st.base, 0, qmk::STATIC_SCRATCH_BYTES, stream));
    st.seq = 0;
    st.ready = true;
  }
  unsigned long long *ll = reinterpret_cast<unsigned long long *>(st.base);
  float *rope = reinterpret_cast<float *>(st.base + qmk::STATIC_LL_BYTES);
  unsigned int *status = reinterpret_cast<unsigned int *>(st.base + qmk::STATIC_LL_BYTES + qmk::STATIC_ROPE_BYTES);
  if (static_cast<unsigned long long>(st.seq) + static_cast<unsigned long long>(num_steps) >= (1ull << 26)) {
    QMK_CUDA(e, cudaMemsetAsync(ll, 0, qmk::STATIC_LL_BYTES, stream));   // tags restart from zero
    st.seq = 0;
  }
  QMK_CUDA(e, cudaMemsetAsync(status, 0, 16, stream));
  // rebuilt every call: picks up a qmk_set_inv_freq made since the last one
  qmk::rope_table_kernel<<<(qmk::STATIC_MAX_POSITIONS * (qmk::D / 2) + 255) / 256, 256, 0, stream>>>(
      rope, qmk::STATIC_MAX_POSITIONS);
  QMK_CUDA(e, cudaGetLastError());

  Params P = base_params(embed_weight, layer_weights, final_norm_weight, lm_head_weight, nullptr, nullptr, k_cache,
                         v_cache, num_layers, start_position, max_seq_len, attn_scale);
  P.first_token = first_token_id;
  P.num_steps = num_steps;
  P.output_log = output_log;
  P.eos = eos_token_id;
  P.normalized_out = static_cast<float *>(g_normalized);
  P.ll = ll;
  P.rope = rope;
  P.status = status;
  P.seq_base = st.seq;
  P.vocab = e->vocab;
  P.rope_from_table = 0;
  P.split_len = e->split_len;
  P.timeout_ns = static_cast<unsigned long long>(e->timeout_ms) * 1000000ull;
  P.logits_out = e->logits_out;
  P.spin_sleep_ns = e->spin_sleep_ns;
  P.l2_evict_first = e->l2_evict_first;
  P.repl = 1;                 // the fixed array holds one copy of the exchange area
  mirror_sequence0(P);
  P.wfmt = e->wfmt;
  P.stream_inflight = e->stream_inflight;
  st.seq += static_cast<uint32_t>(num_steps);
  int grid = st.grid;
  if (e->max_ctas > 0 && e->max_ctas < grid) grid = e->max_ctas;
  void *args[] = {&P};
  cudaError_t err = cudaLaunchCooperativeKernel(single_sequence_kernel(grid), dim3(grid), dim3(qmk::THREADS), args,
                                                qmk::SMEM_BYTES, stream);
  if (err == cudaErrorCooperativeLaunchTooLarge)
    return fail(e, QMK_ERR_NOT_RESIDENT, "persistent grid cannot be co-resident on this device");
  if (err != cudaSuccess) return fail(e, QMK_ERR_CUDA, std::string("cudaLaunchCooperativeKernel: ") + cudaGetErrorString(err));
  unsigned int host_status[4] = {0, 0, 0, 0};   // plain host memory: no pinned allocation on this path
  QMK_CUDA(e, cudaMemcpyAsync(host_status, status, 16, cudaMemcpyDeviceToHost, stream));
  QMK_CUDA(e, cudaStreamSynchronize(stream));
  if (host_status[0] != 0) {
    char buf[160];
    snprintf(buf, sizeof(buf), "device status %u (where %u, cta %u)", host_status[0], host_status[1], host_status[2]);
    return fail(e, static_cast<int>(host_status[0]), buf);
  }
  return QMK_OK;
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
