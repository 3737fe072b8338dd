// Row-wise CUDA kernels of the chunked prefill (everything between the tensor-core GEMMs).  One chunk holds
// `T` prompt tokens of one sequence at positions pos0 .. pos0 + T - 1.  Activations are row-major
// [token][feature]; fp32 wherever the decode kernel keeps fp32 (residual stream, norm statistics, softmax),
// fp16 only as GEMM operands and in the KV cache.
#ifndef QMK_PREFILL_KERNELS_CUH_
#define QMK_PREFILL_KERNELS_CUH_

#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace qmk_pf {

// Programmatic dependent launch: the kernels of a decode step are launched with the stream-serialisation attribute,
// so kernel n + 1 may be scheduled as soon as every CTA of kernel n has executed pdl_trigger(); pdl_wait() then blocks
// until kernel n has COMPLETED and its writes are visible.  Whatever a kernel does before pdl_wait() - barrier and
// TMEM set-up, tensor-map prefetch, streaming weights or cache rows no kernel of the step writes - overlaps its
// predecessor.  Every kernel of the chain waits before its first dependent read and before any global write, and
// triggers only AFTER its own wait: kernel n + 1 then starts no earlier than the completion of kernel n - 1, so at
// most two kernels are in flight.  (With the trigger in front of the wait three and more overlapped, and although
// every kernel still waited for its predecessor the prefill chain produced run-to-run different results.)  Without
// the launch attribute both are no-ops.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

constexpr int H = 1024, I = 3072, NQ = 16, NKV = 8, D = 128, QS = NQ * D, KVS = NKV * D;
constexpr float RMS_EPS = 1e-6f;

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

// x[t][:] = embedding row of token t as fp32.  grid = T, block = 256.  `wq`: 0 fp16 rows; 1 FP8-E4M3 rows (H bytes,
// then a 16-byte trailer with the fp32 row scale); 2 NVFP4 rows (H / 2 bytes of e2m1 pairs, low nibble first, H / 16
// e4m3 block scales, then the trailer with the fp32 tensor scale).
__global__ void embed_rows(const int *tokens, const void *embed, int wq, float *x) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  float *out = x + static_cast<size_t>(t) * H;
  if (wq == 0) {
    const __half *row = static_cast<const __half *>(embed) + static_cast<size_t>(tokens[t]) * H;
    for (int k = threadIdx.x; k < H; k += blockDim.x) out[k] = __half2float(row[k]);
  } else if (wq == 1) {
    const unsigned char *row = static_cast<const unsigned char *>(embed) + static_cast<size_t>(tokens[t]) * (H + 16);
    const float scale = *reinterpret_cast<const float *>(row + H);
    for (int k = threadIdx.x; k < H; k += blockDim.x)
      out[k] = scale * __half2float(__half(__nv_cvt_fp8_to_halfraw(row[k], __NV_E4M3)));
  } else {
    constexpr int PITCH = H / 2 + H / 16 + 16;
    const unsigned char *row = static_cast<const unsigned char *>(embed) + static_cast<size_t>(tokens[t]) * PITCH;
    const float scale = *reinterpret_cast<const float *>(row + H / 2 + H / 16);
    for (int k = threadIdx.x; k < H; k += blockDim.x) {
      const unsigned int code = (row[k >> 1] >> ((k & 1) * 4)) & 0xFu;
      const unsigned int m = code & 7u;
      const float mag = m < 2u ? 0.5f * static_cast<float>(m) : static_cast<float>(2u + (m & 1u)) * static_cast<float>(1u << ((m >> 1) - 1u)) * 0.5f;
      const float bs = __half2float(__half(__nv_cvt_fp8_to_halfraw(row[H / 2 + (k >> 4)], __NV_E4M3)));
      out[k] = scale * bs * ((code & 8u) ? -mag : mag);
    }
  }
}

// Residual add + RMSNorm: x[t] += add[t] (if add), y[t] = fp16(x[t] * rstd * w).  grid = T, block = 256.
// `add` may come as `nparts` (<= 4) partial matrices `part_stride` floats apart (split-K GEMM output): they are
// added in index order.
__global__ void add_rmsnorm_rows(float *x, const float *add, int nparts, size_t part_stride, const __half *w, __half *y) {
  __shared__ float red[8];
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x, k0 = 4 * threadIdx.x;        // four consecutive elements per thread: 16-byte accesses
  float *xr = x + static_cast<size_t>(t) * H;
  constexpr int MAX_PARTS = 4;   // all loads of a thread are issued before the first add (one L2 round trip)
  float4 v = *reinterpret_cast<const float4 *>(xr + k0);
  float4 part[MAX_PARTS];
#pragma unroll
  for (int p = 0; p < MAX_PARTS; ++p)
    part[p] = (add && p < nparts) ? *reinterpret_cast<const float4 *>(add + p * part_stride + static_cast<size_t>(t) * H + k0)
                                  : make_float4(0.f, 0.f, 0.f, 0.f);
  const uint2 wraw = *reinterpret_cast<const uint2 *>(w + k0);
#pragma unroll
  for (int p = 0; p < MAX_PARTS; ++p)
    if (add && p < nparts) { v.x += part[p].x; v.y += part[p].y; v.z += part[p].z; v.w += part[p].w; }   // index order, as the split-K contract says
  float ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, v.w * v.w)));
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) tot += red[i];
  const float rstd = 1.0f / sqrtf(tot * (1.0f / H) + RMS_EPS);
  if (add) *reinterpret_cast<float4 *>(xr + k0) = v;
  const __half2 w01 = *reinterpret_cast<const __half2 *>(&wraw.x), w23 = *reinterpret_cast<const __half2 *>(&wraw.y);
  const __half2 y01 = __floats2half2_rn(v.x * rstd * __low2float(w01), v.y * rstd * __high2float(w01));
  const __half2 y23 = __floats2half2_rn(v.z * rstd * __low2float(w23), v.w * rstd * __high2float(w23));
  uint2 out;
  out.x = *reinterpret_cast<const uint32_t *>(&y01);
  out.y = *reinterpret_cast<const uint32_t *>(&y23);
  *reinterpret_cast<uint2 *>(y + static_cast<size_t>(t) * H + k0) = out;
}

// The same for long chunks: one WARP per row (grid = ceil(T / 8), block = 256), eight 16-byte pieces per lane, every
// load of the lane issued before the first add.  The block-per-row form above keeps one piece per thread in flight
// and needs two waves of blocks for 2048 rows; it spent its 7 us waiting, not copying.  (The sum of squares is added
// in another order than above: results agree to rounding, not bit for bit.)
__global__ void __launch_bounds__(256)
add_rmsnorm_rows_wide(float *x, const float *add, int nparts, size_t part_stride, const __half *w, __half *y, int T) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (t >= T) return;
  constexpr int PIECES = H / 128;                // pieces of four floats per lane
  constexpr int MAX_PARTS = 2;
  float *xr = x + static_cast<size_t>(t) * H;
  float4 v[PIECES], part[MAX_PARTS][PIECES];
  uint2 wraw[PIECES];
#pragma unroll
  for (int i = 0; i < PIECES; ++i) v[i] = *reinterpret_cast<const float4 *>(xr + 4 * (lane + 32 * i));
#pragma unroll
  for (int p = 0; p < MAX_PARTS; ++p)
#pragma unroll
    for (int i = 0; i < PIECES; ++i)
      part[p][i] = (add && p < nparts)
                       ? *reinterpret_cast<const float4 *>(add + p * part_stride + static_cast<size_t>(t) * H + 4 * (lane + 32 * i))
                       : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
  for (int i = 0; i < PIECES; ++i) wraw[i] = *reinterpret_cast<const uint2 *>(w + 4 * (lane + 32 * i));
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < PIECES; ++i) {
#pragma unroll
    for (int p = 0; p < MAX_PARTS; ++p)
      if (add && p < nparts) { v[i].x += part[p][i].x; v[i].y += part[p][i].y; v[i].z += part[p][i].z; v[i].w += part[p][i].w; }   // index order
    ss = fmaf(v[i].x, v[i].x, fmaf(v[i].y, v[i].y, fmaf(v[i].z, v[i].z, fmaf(v[i].w, v[i].w, ss))));
  }
  ss = warp_sum(ss);
  const float rstd = 1.0f / sqrtf(ss * (1.0f / H) + RMS_EPS);
#pragma unroll
  for (int i = 0; i < PIECES; ++i) {
    if (add) *reinterpret_cast<float4 *>(xr + 4 * (lane + 32 * i)) = v[i];
    const __half2 w01 = *reinterpret_cast<const __half2 *>(&wraw[i].x), w23 = *reinterpret_cast<const __half2 *>(&wraw[i].y);
    const __half2 y01 = __floats2half2_rn(v[i].x * rstd * __low2float(w01), v[i].y * rstd * __high2float(w01));
    const __half2 y23 = __floats2half2_rn(v[i].z * rstd * __low2float(w23), v[i].w * rstd * __high2float(w23));
    uint2 out;
    out.x = *reinterpret_cast<const uint32_t *>(&y01);
    out.y = *reinterpret_cast<const uint32_t *>(&y23);
    *reinterpret_cast<uint2 *>(y + static_cast<size_t>(t) * H + 4 * (lane + 32 * i)) = out;
  }
}

// Per head: RMSNorm over 128 with q_norm / k_norm, rotate-half RoPE at position pos0 + t.  Query heads stay
// fp32 (qr[t][head][128]); K (normalised, rotated) and V go to the fp16 cache rows of this layer.
// grid = T, block = 256 = 8 warps; warp w handles query heads w and w + 8, K head w and V head w, with the loads of
// all four issued before the first is used (the kernel is a few dependent round trips per warp: with one head per warp
// and four blocks per token it spent 13 us on seven waves of blocks at 2048 tokens).
// in_f16: q / k / v hold fp16 (the projection's epilogue stored halves) instead of fp32.
// q_f16_scale != 0: the rotated queries are stored as fp16 times that factor (same [t][head][128] layout in halves).
// Packed prompts (row_info != null): row t belongs to sequence row_info[t].x at position row_info[t].y (negative:
// a padding row, nothing to do), whose K / V caches start at kv_ptrs[2 seq], kv_ptrs[2 seq + 1]; the layer's rows
// begin `layer_off` halves into each.
__global__ void __launch_bounds__(256)
qk_norm_rope_cache(const float *q, const float *k, const float *v, int in_f16, const __half *q_norm,
                   const __half *k_norm, const float *rope, const __half *cos_table,
                   const __half *sin_table, float *qr, __half *k_cache_layer, __half *v_cache_layer,
                   int pos0, int max_seq_len, const int2 *row_info, const unsigned long long *kv_ptrs, size_t layer_off,
                   float q_f16_scale) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x, w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int pos = pos0 + t;
  if (row_info != nullptr) {
    const int2 info = row_info[t];
    if (info.y < 0) return;
    pos = info.y;
    k_cache_layer = reinterpret_cast<__half *>(kv_ptrs[2 * info.x]) + layer_off;
    v_cache_layer = reinterpret_cast<__half *>(kv_ptrs[2 * info.x + 1]) + layer_off;
  }
  const int d0 = 4 * lane;                      // four consecutive dims per lane: 16-byte accesses
  auto pack4 = [](float a, float b, float c, float d) {
    const __half2 lo = __floats2half2_rn(a, b), hi = __floats2half2_rn(c, d);
    uint2 o;
    o.x = *reinterpret_cast<const uint32_t *>(&lo);
    o.y = *reinterpret_cast<const uint32_t *>(&hi);
    return o;
  };
  auto load4 = [&](const float *m, size_t idx) {   // four consecutive values from element idx of an fp32 or fp16 matrix
    if (!in_f16) return *reinterpret_cast<const float4 *>(m + idx);
    const uint2 raw = *reinterpret_cast<const uint2 *>(reinterpret_cast<const __half *>(m) + idx);
    const __half2 a = *reinterpret_cast<const __half2 *>(&raw.x), b = *reinterpret_cast<const __half2 *>(&raw.y);
    return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
  };
  auto unpack4 = [](uint2 raw) {
    const __half2 a = *reinterpret_cast<const __half2 *>(&raw.x), b = *reinterpret_cast<const __half2 *>(&raw.y);
    return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
  };
  // ---- every load first
  float4 x[3];                                  // query heads w and w + 8, K head w
  x[0] = load4(q, static_cast<size_t>(t) * QS + w * D + d0);
  x[1] = load4(q, static_cast<size_t>(t) * QS + (w + 8) * D + d0);
  x[2] = load4(k, static_cast<size_t>(t) * KVS + w * D + d0);
  const float4 vv = load4(v, static_cast<size_t>(t) * KVS + w * D + d0);
  const float4 wq4 = unpack4(*reinterpret_cast<const uint2 *>(q_norm + d0));
  const float4 wk4 = unpack4(*reinterpret_cast<const uint2 *>(k_norm + d0));
  // element i pairs with i + 64 and both use frequency i (i < 64): lanes 0..15 hold the low halves, lane + 16 the
  // partners; the frequencies of this lane's dims are those of dims (d0 mod 64) ..
  const int f0 = d0 & 63;
  float4 cs, sn;
  if (rope) {
    const float *r = rope + static_cast<size_t>(pos) * D;
    cs = *reinterpret_cast<const float4 *>(r + f0);
    sn = *reinterpret_cast<const float4 *>(r + 64 + f0);
  } else {
    cs = unpack4(*reinterpret_cast<const uint2 *>(cos_table + static_cast<size_t>(pos) * D + f0));
    sn = unpack4(*reinterpret_cast<const uint2 *>(sin_table + static_cast<size_t>(pos) * D + f0));
  }
  // ---- V head: plain copy to the cache
  *reinterpret_cast<uint2 *>(v_cache_layer + (static_cast<size_t>(w) * max_seq_len + pos) * D + d0) = pack4(vv.x, vv.y, vv.z, vv.w);
#pragma unroll
  for (int h = 0; h < 3; ++h) {
    const float4 nw = h < 2 ? wq4 : wk4;
    float4 a = x[h];
    float ss = fmaf(a.x, a.x, fmaf(a.y, a.y, fmaf(a.z, a.z, a.w * a.w)));
    ss = warp_sum(ss);
    const float rstd = 1.0f / sqrtf(ss * (1.0f / D) + RMS_EPS);
    a.x = a.x * rstd * nw.x; a.y = a.y * rstd * nw.y; a.z = a.z * rstd * nw.z; a.w = a.w * rstd * nw.w;
    float4 o;   // the partner's normalised values
    o.x = __shfl_xor_sync(0xffffffffu, a.x, 16); o.y = __shfl_xor_sync(0xffffffffu, a.y, 16);
    o.z = __shfl_xor_sync(0xffffffffu, a.z, 16); o.w = __shfl_xor_sync(0xffffffffu, a.w, 16);
    float4 r;
    if (lane < 16) {    // low half: lo * cos - hi * sin
      r = make_float4(a.x * cs.x - o.x * sn.x, a.y * cs.y - o.y * sn.y, a.z * cs.z - o.z * sn.z, a.w * cs.w - o.w * sn.w);
    } else {            // high half: lo * sin + hi * cos
      r = make_float4(o.x * sn.x + a.x * cs.x, o.y * sn.y + a.y * cs.y, o.z * sn.z + a.z * cs.z, o.w * sn.w + a.w * cs.w);
    }
    if (h < 2 && q_f16_scale != 0.f)   // fp16 queries, pre-scaled: the tcgen05 attention kernel takes them by TMA as they are
      *reinterpret_cast<uint2 *>(reinterpret_cast<__half *>(qr) + (static_cast<size_t>(t) * NQ + w + 8 * h) * D + d0) =
          pack4(r.x * q_f16_scale, r.y * q_f16_scale, r.z * q_f16_scale, r.w * q_f16_scale);
    else if (h < 2)
      *reinterpret_cast<float4 *>(qr + (static_cast<size_t>(t) * NQ + w + 8 * h) * D + d0) = r;
    else
      *reinterpret_cast<uint2 *>(k_cache_layer + (static_cast<size_t>(w) * max_seq_len + pos) * D + d0) = pack4(r.x, r.y, r.z, r.w);
  }
}

// Causal attention of the chunk's queries over cache rows [0, pos0 + t] (the chunk's own rows are already in the
// cache), on the tensor cores: mma.sync m16n8k16, fp16 operands, fp32 accumulate and softmax.
// grid = (ceil(T / 32), 8 kv heads), block = 128 = 4 warps.  A CTA takes 32 query tokens x the two query heads
// of its kv head; warp w works on head (w & 1) and tokens t0 + 16 * (w >> 1) + 0..15 (one 16-row MMA tile).
// Keys go through shared memory in tiles of 64 rows of K and of V (row pitch 272 bytes: conflict-free for the
// 32-bit B-fragment loads of K and for ldmatrix.trans on V), two stages filled with cp.async so that the next tile
// arrives while this one is multiplied (dynamic shared memory: ATM_SMEM_BYTES).  Per key tile and warp: S = Q K^T (64 MMAs),
// online softmax on the accumulator fragments, P (as fp16 A fragments, straight from the S registers) times V
// (64 MMAs).  q is scaled by scale * log2(e) before it is rounded to fp16, so the softmax runs on exp2.
// (64 query tokens per CTA, 8 warps, measured slower: 7.9 against 7.3 ms for a 2048-token prefill)
constexpr int ATM_Q = 32, ATM_KEYS = 64, ATM_PITCH = D + 8;   // halves per K / V row in shared memory
constexpr int ATM_THREADS = ATM_Q * 4;                          // 2 heads x (ATM_Q / 16) query groups, one warp each
constexpr int ATM_STAGE_HALVES = 2 * ATM_KEYS * ATM_PITCH;      // one stage: a K tile and a V tile
constexpr int ATM_SMEM_BYTES = 2 * ATM_STAGE_HALVES * 2;        // two stages, 69,632 bytes

__device__ __forceinline__ uint32_t pack_half2(float a, float b) {
  const __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<const uint32_t *>(&h);
}
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__global__ void __launch_bounds__(ATM_THREADS) causal_attention_mma(const float *qr, const __half *k_cache_layer,
                                                            const __half *v_cache_layer, __half *out, int T, int pos0,
                                                            int max_seq_len, float scale) {
  pdl_wait();
  pdl_trigger();
  // two stages of (K tile, V tile): the next 64 keys are fetched with cp.async while this tile is multiplied
  extern __shared__ __align__(16) unsigned char atm_smem[];
  __half *const tiles = reinterpret_cast<__half *>(atm_smem);
  const int g = blockIdx.y, t0 = (gridDim.x - 1 - blockIdx.x) * ATM_Q;   // longest tiles first
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = warp & 1, tw = t0 + 16 * (warp >> 1);     // this warp's head and first token
  const int gr = lane >> 2, qd = lane & 3;                // fragment row within 8, quad lane
  const int tok_lo = tw + gr, tok_hi = tw + gr + 8;       // the two query rows this lane holds
  const float sc = scale * 1.4426950408889634f;

  // Q fragments (A operand), 8 k-steps of 16 dims
  uint32_t qa[8][4];
  {
    const float *q_lo = qr + (static_cast<size_t>(min(tok_lo, T - 1)) * NQ + 2 * g + h) * D;
    const float *q_hi = qr + (static_cast<size_t>(min(tok_hi, T - 1)) * NQ + 2 * g + h) * D;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      const int d = ks * 16 + qd * 2;
      const float2 l0 = *reinterpret_cast<const float2 *>(q_lo + d), l1 = *reinterpret_cast<const float2 *>(q_lo + d + 8);
      const float2 h0 = *reinterpret_cast<const float2 *>(q_hi + d), h1 = *reinterpret_cast<const float2 *>(q_hi + d + 8);
      qa[ks][0] = pack_half2(l0.x * sc, l0.y * sc);
      qa[ks][1] = pack_half2(h0.x * sc, h0.y * sc);
      qa[ks][2] = pack_half2(l1.x * sc, l1.y * sc);
      qa[ks][3] = pack_half2(h1.x * sc, h1.y * sc);
    }
  }
  float o[16][4];
#pragma unroll
  for (int dt = 0; dt < 16; ++dt) { o[dt][0] = 0.f; o[dt][1] = 0.f; o[dt][2] = 0.f; o[dt][3] = 0.f; }
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
  // rows beyond the chunk see no key at all
  const int lim_lo = tok_lo < T ? pos0 + tok_lo : -1, lim_hi = tok_hi < T ? pos0 + tok_hi : -1;
  const int warp_last = pos0 + min(tw + 15, T - 1);                   // highest key this warp needs (tw < T or unused)
  const int cta_last = pos0 + min(t0 + ATM_Q - 1, T - 1);
  const __half *kbase = k_cache_layer + static_cast<size_t>(g) * max_seq_len * D;
  const __half *vbase = v_cache_layer + static_cast<size_t>(g) * max_seq_len * D;

  auto fetch_tile = [&](int k0, int stage) {   // rows past the last key this CTA needs are zero-filled
    __half *dk = tiles + stage * ATM_STAGE_HALVES, *dv = dk + ATM_KEYS * ATM_PITCH;
    for (int i = threadIdx.x; i < ATM_KEYS * (D / 8); i += ATM_THREADS) {
      const int j = i >> 4, c = i & 15;
      const bool in = k0 + j <= cta_last;
      const size_t off = static_cast<size_t>(in ? k0 + j : 0) * D + c * 8;
      const uint32_t bytes = in ? 16u : 0u;
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(dk + j * ATM_PITCH + c * 8))),
                   "l"(kbase + off), "r"(bytes) : "memory");
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(dv + j * ATM_PITCH + c * 8))),
                   "l"(vbase + off), "r"(bytes) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  fetch_tile(0, 0);
  int stage = 0;
  for (int k0 = 0; k0 <= cta_last; k0 += ATM_KEYS, stage ^= 1) {
    // the other stage was last read in the previous iteration, which ended with a barrier
    const bool more = k0 + ATM_KEYS <= cta_last;
    if (more) {
      fetch_tile(k0 + ATM_KEYS, stage ^ 1);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    const __half *sk = tiles + stage * ATM_STAGE_HALVES, *sv = sk + ATM_KEYS * ATM_PITCH;
    if (tw >= T || k0 > warp_last) {   // warp-uniform: nothing (more) to do for this warp in this tile
      __syncthreads();
      continue;
    }

    // S = Q K^T for 64 keys: 8 n-tiles of 8 keys
    float sacc[8][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      sacc[nt][0] = 0.f; sacc[nt][1] = 0.f; sacc[nt][2] = 0.f; sacc[nt][3] = 0.f;
      const __half *krow = sk + (nt * 8 + gr) * ATM_PITCH + qd * 2;
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        const uint32_t b0 = *reinterpret_cast<const uint32_t *>(krow + ks * 16);
        const uint32_t b1 = *reinterpret_cast<const uint32_t *>(krow + ks * 16 + 8);
        mma_16816(sacc[nt], qa[ks], b0, b1);
      }
    }
    // causal mask + row maxima (a row lives in the 4 lanes of a quad)
    float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      const int key = k0 + nt * 8 + qd * 2;
      if (key > lim_lo) sacc[nt][0] = -INFINITY;
      if (key + 1 > lim_lo) sacc[nt][1] = -INFINITY;
      if (key > lim_hi) sacc[nt][2] = -INFINITY;
      if (key + 1 > lim_hi) sacc[nt][3] = -INFINITY;
      mx_lo = fmaxf(mx_lo, fmaxf(sacc[nt][0], sacc[nt][1]));
      mx_hi = fmaxf(mx_hi, fmaxf(sacc[nt][2], sacc[nt][3]));
    }
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
    const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
    const float ref_lo = (mn_lo == -INFINITY) ? 0.f : mn_lo, ref_hi = (mn_hi == -INFINITY) ? 0.f : mn_hi;   // fully masked rows
    const float c_lo = exp2f(m_lo - ref_lo), c_hi = exp2f(m_hi - ref_hi);
    m_lo = mn_lo; m_hi = mn_hi;
    float sum_lo = 0.f, sum_hi = 0.f;
    uint32_t pa[4][4];   // P as A fragments: 4 key-steps of 16 keys
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      const float p0 = exp2f(sacc[nt][0] - ref_lo), p1 = exp2f(sacc[nt][1] - ref_lo);
      const float p2 = exp2f(sacc[nt][2] - ref_hi), p3 = exp2f(sacc[nt][3] - ref_hi);
      sum_lo += p0 + p1;
      sum_hi += p2 + p3;
      pa[nt >> 1][(nt & 1) * 2 + 0] = pack_half2(p0, p1);
      pa[nt >> 1][(nt & 1) * 2 + 1] = pack_half2(p2, p3);
    }
    sum_lo += __shfl_xor_sync(0xffffffffu, sum_lo, 1);
    sum_lo += __shfl_xor_sync(0xffffffffu, sum_lo, 2);
    sum_hi += __shfl_xor_sync(0xffffffffu, sum_hi, 1);
    sum_hi += __shfl_xor_sync(0xffffffffu, sum_hi, 2);
    l_lo = l_lo * c_lo + sum_lo;
    l_hi = l_hi * c_hi + sum_hi;
#pragma unroll
    for (int dt = 0; dt < 16; ++dt) { o[dt][0] *= c_lo; o[dt][1] *= c_lo; o[dt][2] *= c_hi; o[dt][3] *= c_hi; }
    // O += P V: B fragments of V through ldmatrix.trans (4 8x8 matrices: keys 0-7 / 8-15 of the step x two dim tiles)
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      const int mi = lane >> 3;
      const __half *vrow = sv + (kk * 16 + (mi & 1) * 8 + (lane & 7)) * ATM_PITCH + (mi >> 1) * 8;
#pragma unroll
      for (int dp = 0; dp < 8; ++dp) {
        uint32_t b0, b1, b2, b3;
        const uint32_t addr = static_cast<uint32_t>(__cvta_generic_to_shared(vrow + dp * 16));
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                     : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3)
                     : "r"(addr));
        mma_16816(o[2 * dp], pa[kk], b0, b1);
        mma_16816(o[2 * dp + 1], pa[kk], b2, b3);
      }
    }
    __syncthreads();   // this stage is free for the fetch of the iteration after next
  }
  if (tw < T) {
    const float inv_lo = l_lo > 0.f ? 1.0f / l_lo : 0.f, inv_hi = l_hi > 0.f ? 1.0f / l_hi : 0.f;
#pragma unroll
    for (int dt = 0; dt < 16; ++dt) {
      const int d = (2 * g + h) * D + dt * 8 + qd * 2;
      if (tok_lo < T)
        *reinterpret_cast<__half2 *>(out + static_cast<size_t>(tok_lo) * QS + d) = __floats2half2_rn(o[dt][0] * inv_lo, o[dt][1] * inv_lo);
      if (tok_hi < T)
        *reinterpret_cast<__half2 *>(out + static_cast<size_t>(tok_hi) * QS + d) = __floats2half2_rn(o[dt][2] * inv_hi, o[dt][3] * inv_hi);
    }
  }
}

// Decode-step attention for a batch of sequences, with the per-head preparation fused in.  grid = (B, 8 kv
// heads, splits), block = 288 = 8 consumer warps + 1 producer warp.  With splits > 1 the old rows of a sequence are
// divided among `splits` CTAs, which leave their softmax states in `split_part`; the CTA that arrives last at the
// counter in `split_count` adds them up in split order (no CTA waits for another).  CTA (sequence b, kv head g) first normalises and
// rotates the two query heads and the K head of row b of the q / k / v GEMM outputs (warps 0-2; warp 3 takes V),
// writes the new K and V rows to sequence b's cache at positions[b], and then attends over the old rows
// [0, positions[b]) plus the new row from shared memory (the fp16-rounded values, i.e. what later steps read).
// The old rows are streamed by one producer thread with bulk copies (cp.async.bulk, 32 K rows + 32 V rows per
// 16 KB ring slot, full / empty mbarriers): the bytes in flight then do not depend on how many loads the compiler
// keeps in registers (a version with per-lane global loads ran at 43 % of DRAM bandwidth with 64 sequences and
// was 7-30 % slower at every batch size).  The consumer warps take slots round-robin; lane j scores key j reading
// its K row in a lane-rotated order (word (d + j) mod 64 at step d), which makes the 256-byte row pitch
// conflict-free; V rows are read by all lanes together; probabilities travel by shuffle; every lane owns 4 output
// dims; the warps' partial softmax states and the new row are merged through shared memory.
// Waits are bounded: on a time-out the CTA sets *status = 4 and leaves after its copies have landed.
constexpr int DAR_WARPS = 8, DAR_SLOTS = 6, DAR_ROWS = 32;
constexpr int DAR_SLOT_BYTES = 2 * DAR_ROWS * D * 2;   // 16 KB: K rows then V rows
constexpr int DAR_SMEM_BYTES = DAR_SLOTS * DAR_SLOT_BYTES + 2 * DAR_SLOTS * 8 + 16;   // ring, barriers, abort flag + issued counter
__global__ void __launch_bounds__((DAR_WARPS + 1) * 32) decode_attention_ring(
    const float *q, const float *k, const float *v, const __half *q_norm, const __half *k_norm, const float *rope,
    const __half *cos_table, const __half *sin_table, __half *const *k_ptrs, __half *const *v_ptrs, size_t layer_off,
    const int *positions, __half *out, int max_seq_len, float scale, unsigned int *status, unsigned long long budget_ns,
    float *split_part, unsigned int *split_count) {
  extern __shared__ __align__(128) unsigned char dar_smem[];
  __shared__ __align__(16) float sq[2 * D];
  __shared__ float sknew[D], svnew[D], snew_score[2];
  __shared__ float sm[DAR_WARPS][2], sl[DAR_WARPS][2];
  __shared__ __align__(16) float sacc[DAR_WARPS][2][D];
  uint64_t *full = reinterpret_cast<uint64_t *>(dar_smem + DAR_SLOTS * DAR_SLOT_BYTES);
  uint64_t *empty = full + DAR_SLOTS;
  volatile int *abort_flag = reinterpret_cast<volatile int *>(empty + DAR_SLOTS);
  // Chunks issued so far.  A parity wait can only tell two consecutive uses of a slot apart, and a warp's first
  // chunk may already be a second use (chunk 6 or 7 in slot 0 or 1): consumers wait for "issued" first.
  volatile int *issued_ctr = abort_flag + 1;
  const int b = blockIdx.x, g = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pos = positions[b];
  const int nchunks_all = (pos + DAR_ROWS - 1) / DAR_ROWS;
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
    for (int i = 0; i < DAR_SLOTS; ++i) {
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
  if (warp != DAR_WARPS) {
    pdl_wait();
    if (threadIdx.x == 0) pdl_trigger();   // (after the wait: at most two kernels of a chain overlap)
  }
  if (warp == DAR_WARPS) {            // ---- producer: old rows [0, pos) in chunks of 32
    if (lane == 0) {
      int issued = 0;
      for (int c = 0; c < nchunks; ++c) {
        const int slot = c % DAR_SLOTS;
        if (c >= DAR_SLOTS && !wait(empty + slot, ((c / DAR_SLOTS) - 1) & 1)) break;
        const int cg = c_begin + c;          // chunk index within the sequence
        const uint32_t bytes = static_cast<uint32_t>(min(DAR_ROWS, pos - cg * DAR_ROWS)) * D * 2;
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(s32(full + slot)), "r"(2 * bytes) : "memory");
        unsigned char *dst = dar_smem + slot * DAR_SLOT_BYTES;
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                     ::"r"(s32(dst)), "l"(kbase + static_cast<size_t>(cg) * DAR_ROWS * D), "r"(bytes), "r"(s32(full + slot)) : "memory");
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                     ::"r"(s32(dst + DAR_SLOT_BYTES / 2)), "l"(vbase + static_cast<size_t>(cg) * DAR_ROWS * D), "r"(bytes),
                     "r"(s32(full + slot)) : "memory");
        issued = c + 1;
        __threadfence_block();
        *issued_ctr = issued;
      }
      if (*abort_flag)   // copies already issued must land before the CTA may exit
        for (int c = (issued > DAR_SLOTS ? issued - DAR_SLOTS : 0); c < issued; ++c) {
          unsigned long long t0, t;
          asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
          while (!try_wait(full + c % DAR_SLOTS, (c / DAR_SLOTS) & 1)) {
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
#pragma unroll
      for (int i = 0; i < 4; ++i) sq[warp * D + lane + 32 * i] = x[i];
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
  if (warp < DAR_WARPS) asm volatile("bar.sync 1, %0;" ::"n"(DAR_WARPS * 32) : "memory");
  const float sc = scale * 1.4426950408889634f;
  if (warp < 2) {   // score of the new row for query head `warp`
    float d = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) d = fmaf(sq[warp * D + lane + 32 * i], sknew[lane + 32 * i], d);
    d = warp_sum(d);
    if (lane == 0) snew_score[warp] = d * sc;
  }
  if (warp < DAR_WARPS) {             // ---- consumers
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    float a0[4] = {0.f, 0.f, 0.f, 0.f}, a1[4] = {0.f, 0.f, 0.f, 0.f};
    for (int c = warp; c < nchunks; c += DAR_WARPS) {
      const int slot = c % DAR_SLOTS;
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
      const bool ok = __all_sync(0xffffffffu, mine && wait(full + slot, (c / DAR_SLOTS) & 1));
      const int nrow = min(DAR_ROWS, pos - (c_begin + c) * DAR_ROWS);
      float sa = -INFINITY, sb = -INFINITY;
      const unsigned char *sk = dar_smem + slot * DAR_SLOT_BYTES, *sv = sk + DAR_SLOT_BYTES / 2;
      if (ok && lane < nrow) {
        const uint32_t *krow = reinterpret_cast<const uint32_t *>(sk + lane * (D * 2));
        // packed fp32 FMAs (two lanes per instruction): even and odd dims accumulate separately
        float2 sa2 = make_float2(0.f, 0.f), sb2 = make_float2(0.f, 0.f);
#pragma unroll 16
        for (int d = 0; d < D / 2; ++d) {
          const int w = (d + lane) & (D / 2 - 1);      // lane-rotated word index: conflict-free at a 256-byte pitch
          const uint32_t kw = krow[w];
          const float2 kf = __half22float2(*reinterpret_cast<const __half2 *>(&kw));
          const float2 qa = *reinterpret_cast<const float2 *>(sq + 2 * w);
          const float2 qb = *reinterpret_cast<const float2 *>(sq + D + 2 * w);
          sa2 = __ffma2_rn(qa, kf, sa2);
          sb2 = __ffma2_rn(qb, kf, sb2);
        }
        sa = (sa2.x + sa2.y) * sc; sb = (sb2.x + sb2.y) * sc;
      }
      if (ok) {   // warp-uniform
        const float na = fmaxf(m0, warp_max(sa)), nb = fmaxf(m1, warp_max(sb));   // row 0 of a chunk always exists
        const float ca = exp2f(m0 - na), cb = exp2f(m1 - nb);
        const float pa = exp2f(sa - na), pb = exp2f(sb - nb);
        l0 = l0 * ca + warp_sum(pa);
        l1 = l1 * cb + warp_sum(pb);
        m0 = na; m1 = nb;
        float2 a0l = make_float2(a0[0] * ca, a0[1] * ca), a0h = make_float2(a0[2] * ca, a0[3] * ca);
        float2 a1l = make_float2(a1[0] * cb, a1[1] * cb), a1h = make_float2(a1[2] * cb, a1[3] * cb);
#pragma unroll 8
        for (int j = 0; j < nrow; ++j) {
          const float pja = __shfl_sync(0xffffffffu, pa, j), pjb = __shfl_sync(0xffffffffu, pb, j);
          const uint2 vv = *reinterpret_cast<const uint2 *>(sv + j * (D * 2) + lane * 8);
          const float2 v01 = __half22float2(*reinterpret_cast<const __half2 *>(&vv.x));
          const float2 v23 = __half22float2(*reinterpret_cast<const __half2 *>(&vv.y));
          const float2 pa2 = make_float2(pja, pja), pb2 = make_float2(pjb, pjb);
          a0l = __ffma2_rn(pa2, v01, a0l); a0h = __ffma2_rn(pa2, v23, a0h);
          a1l = __ffma2_rn(pb2, v01, a1l); a1h = __ffma2_rn(pb2, v23, a1h);
        }
        a0[0] = a0l.x; a0[1] = a0l.y; a0[2] = a0h.x; a0[3] = a0h.y;
        a1[0] = a1l.x; a1[1] = a1l.y; a1[2] = a1h.x; a1[3] = a1h.y;
      }
      __syncwarp();
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(s32(empty + slot)) : "memory");
      if (!ok) break;
    }
    if (lane == 0) { sm[warp][0] = m0; sm[warp][1] = m1; sl[warp][0] = l0; sl[warp][1] = l1; }
#pragma unroll
    for (int d = 0; d < 4; ++d) { sacc[warp][0][lane * 4 + d] = a0[d]; sacc[warp][1][lane * 4 + d] = a1[d]; }
  }
  __syncthreads();
  // This CTA's state per (head, dim): running maximum M, sum L, unnormalised output A.
  float M = -INFINITY, L = 0.f, A = 0.f;
  const int h = (threadIdx.x >> 7) & 1, d = threadIdx.x & (D - 1);
  if (threadIdx.x < 2 * D) {
    if (owner) M = snew_score[h];     // the new row is always there
#pragma unroll
    for (int w = 0; w < DAR_WARPS; ++w) M = fmaxf(M, sm[w][h]);
    if (owner) { L = exp2f(snew_score[h] - M); A = L * svnew[d]; }
#pragma unroll
    for (int w = 0; w < DAR_WARPS; ++w) {
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

// Greedy pick per row: tokens[b] = argmax(logits[b][:]) (lowest index on ties), logged at
// log_ptrs[b][positions[b] - start_positions[b]] (= the step index, kept out of the arguments so that one
// captured graph serves every step); the sequence's position advances by one.  grid = B, block = 1024.
__global__ void __launch_bounds__(1024) argmax_rows(const float *logits, int vocab, int *tokens, int *const *log_ptrs,
                                                    const int *start_positions, int *positions) {
  __shared__ float sv[32];
  __shared__ int si[32];
  pdl_wait();
  pdl_trigger();
  const int b = blockIdx.x;
  const float *row = logits + static_cast<size_t>(b) * vocab;
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  for (int i = threadIdx.x; i < vocab; i += 1024) {
    const float v = row[i];
    if (v > best) { best = v; best_i = i; }      // increasing i per thread: strict > keeps the lowest index
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
  }
  if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = best; si[threadIdx.x >> 5] = best_i; }
  __syncthreads();
  if (threadIdx.x < 32) {
    best = sv[threadIdx.x];
    best_i = si[threadIdx.x];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
      if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    if (threadIdx.x == 0) {
      tokens[b] = best_i;
      const int pos = positions[b];
      if (log_ptrs[b]) log_ptrs[b][pos - start_positions[b]] = best_i;
      positions[b] = pos + 1;
    }
  }
}

// The same pick from the per-tile (value, column) pairs the LM-head GEMM's epilogue leaves behind (`ntiles` pairs
// per row, tiles in increasing column order): no row of logits is ever written or read.  grid = B, block = 256.
__global__ void __launch_bounds__(256) argmax_pairs(const float *val, const int *idx, int ntiles, int *tokens, int *const *log_ptrs,
                                                    const int *start_positions, int *positions) {
  __shared__ float sv[8];
  __shared__ int si[8];
  pdl_wait();
  pdl_trigger();
  const int b = blockIdx.x;
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  for (int t = threadIdx.x; t < ntiles; t += 256) {
    const float v = val[static_cast<size_t>(b) * ntiles + t];
    const int i = idx[static_cast<size_t>(b) * ntiles + t];
    if (v > best) { best = v; best_i = i; }      // increasing columns per thread: strict > keeps the lowest index
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
  }
  if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = best; si[threadIdx.x >> 5] = best_i; }
  __syncthreads();
  if (threadIdx.x < 32) {
    best = threadIdx.x < 8 ? sv[threadIdx.x] : -INFINITY;
    best_i = threadIdx.x < 8 ? si[threadIdx.x] : 0x7fffffff;
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
      if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    if (threadIdx.x == 0) {
      tokens[b] = best_i;
      const int pos = positions[b];
      if (log_ptrs[b]) log_ptrs[b][pos - start_positions[b]] = best_i;
      positions[b] = pos + 1;
    }
  }
}

}  // namespace qmk_pf
#endif  // QMK_PREFILL_KERNELS_CUH_
