// Row-wise CUDA kernels of the chunked prefill (everything between the tensor-core GEMMs).  One chunk holds
// `T` prompt tokens of one sequence at positions pos0 .. pos0 + T - 1.  Activations are row-major
// [token][feature]; fp32 wherever the decode kernel keeps fp32 (residual stream, norm statistics, softmax),
// fp16 only as GEMM operands and in the KV cache.
#ifndef QMK_PREFILL_KERNELS_CUH_
#define QMK_PREFILL_KERNELS_CUH_

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace qmk_pf {

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

// x[t][:] = embedding row of token t (fp16 -> fp32).  grid = T, block = 256.
__global__ void embed_rows(const int *tokens, const __half *embed, float *x) {
  const int t = blockIdx.x;
  const __half *row = embed + static_cast<size_t>(tokens[t]) * H;
  for (int k = threadIdx.x; k < H; k += blockDim.x) x[static_cast<size_t>(t) * H + k] = __half2float(row[k]);
}

// Residual add + RMSNorm: x[t] += add[t] (if add), y[t] = fp16(x[t] * rstd * w).  grid = T, block = 256.
__global__ void add_rmsnorm_rows(float *x, const float *add, const __half *w, __half *y) {
  __shared__ float red[8];
  const int t = blockIdx.x;
  float *xr = x + static_cast<size_t>(t) * H;
  float v[4];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int k = threadIdx.x + j * 256;
    v[j] = xr[k] + (add ? add[static_cast<size_t>(t) * H + k] : 0.f);
    ss = fmaf(v[j], v[j], ss);
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) tot += red[i];
  const float rstd = 1.0f / sqrtf(tot * (1.0f / H) + RMS_EPS);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int k = threadIdx.x + j * 256;
    if (add) xr[k] = v[j];
    y[static_cast<size_t>(t) * H + k] = __float2half_rn(v[j] * rstd * __half2float(w[k]));
  }
}

// Per head: RMSNorm over 128 with q_norm / k_norm, rotate-half RoPE at position pos0 + t.  Query heads stay
// fp32 (qr[t][head][128]); K (normalised, rotated) and V go to the fp16 cache rows of this layer.
// grid = (T, 4), block = 256 = 8 warps; warp w of block y handles head slot y * 8 + w of 32:
// 0..15 query heads, 16..23 K heads, 24..31 V heads.
__global__ void qk_norm_rope_cache(const float *q, const float *k, const float *v, const __half *q_norm,
                                   const __half *k_norm, const float *rope, const __half *cos_table,
                                   const __half *sin_table, float *qr, __half *k_cache_layer, __half *v_cache_layer,
                                   int pos0, int max_seq_len) {
  const int t = blockIdx.x, slot = blockIdx.y * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  const int pos = pos0 + t;
  if (slot >= 24) {   // V head: plain copy to the cache
    const int g = slot - 24;
    const float *src = v + static_cast<size_t>(t) * KVS + g * D;
    __half *dst = v_cache_layer + (static_cast<size_t>(g) * max_seq_len + pos) * D;
#pragma unroll
    for (int i = 0; i < 4; ++i) dst[lane + 32 * i] = __float2half_rn(src[lane + 32 * i]);
    return;
  }
  const bool is_q = slot < 16;
  const int head = is_q ? slot : slot - 16;
  const float *src = is_q ? q + static_cast<size_t>(t) * QS + head * D : k + static_cast<size_t>(t) * KVS + head * D;
  const __half *nw = is_q ? q_norm : k_norm;
  float x[4];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    x[i] = src[lane + 32 * i];
    ss = fmaf(x[i], x[i], ss);
  }
  ss = warp_sum(ss);
  const float rstd = 1.0f / sqrtf(ss * (1.0f / D) + RMS_EPS);
#pragma unroll
  for (int i = 0; i < 4; ++i) x[i] = x[i] * rstd * __half2float(nw[lane + 32 * i]);
  // element i pairs with i + 64 and both use frequency i (i < 64): lane holds i = lane, lane + 32
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
  if (is_q) {
    float *dst = qr + (static_cast<size_t>(t) * NQ + head) * D;
    dst[lane] = r0; dst[lane + 32] = r1; dst[lane + 64] = r2; dst[lane + 96] = r3;
  } else {
    __half *dst = k_cache_layer + (static_cast<size_t>(head) * max_seq_len + pos) * D;
    dst[lane] = __float2half_rn(r0); dst[lane + 32] = __float2half_rn(r1);
    dst[lane + 64] = __float2half_rn(r2); dst[lane + 96] = __float2half_rn(r3);
  }
}

// Causal attention of the chunk's queries over cache rows [0, pos0 + t] (the chunk's own rows are already
// in the cache).  grid = (ceil(T / 16), 8 kv heads), block = 256 = 8 warps.  A CTA takes 16 query tokens x the
// two query heads of its kv head; a warp takes 2 tokens and works on both heads of a token together (they
// share every K and V row).  Query tiles are handed out last-first: the longest ones start first.  Keys go through shared memory in tiles of 32: lane j scores key j, and every
// lane owns 4 of the 128 output dims.  Online softmax in fp32, base-2 exponent.
constexpr int ATT_Q = 16, ATT_KEYS = 32;
constexpr int ATT_KPITCH = D + 2;   // halves per K row in shared memory: an odd number of 32-bit words
__global__ void __launch_bounds__(256) causal_attention(const float *qr, const __half *k_cache_layer,
                                                        const __half *v_cache_layer, __half *out, int T, int pos0,
                                                        int max_seq_len, float scale) {
  __shared__ __align__(16) __half sk[ATT_KEYS * ATT_KPITCH];
  __shared__ __align__(16) __half sv[ATT_KEYS * D];
  __shared__ __align__(16) float sq[ATT_Q * 2 * D];   // [token][head-in-pair][128]
  __shared__ float sp[8][2][ATT_KEYS];                 // probabilities of the two heads, per warp
  const int g = blockIdx.y, t0 = (gridDim.x - 1 - blockIdx.x) * ATT_Q;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nq = min(ATT_Q, T - t0);
  for (int i = threadIdx.x; i < ATT_Q * 2 * D; i += 256) {
    const int tk = i / (2 * D), h = (i / D) & 1, d = i % D, tok = t0 + tk;
    sq[i] = (tok < T) ? qr[(static_cast<size_t>(tok) * NQ + 2 * g + h) * D + d] : 0.f;
  }
  const float sc = scale * 1.4426950408889634f;
  constexpr int TPW = 2;   // tokens per warp
  float m[TPW][2], l[TPW][2], acc[TPW][2][4];
#pragma unroll
  for (int r = 0; r < TPW; ++r)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      m[r][h] = -INFINITY; l[r][h] = 0.f;
#pragma unroll
      for (int d = 0; d < 4; ++d) acc[r][h][d] = 0.f;
    }
  const int last_key = pos0 + t0 + nq - 1;   // highest key any query of this CTA may see
  const __half *kbase = k_cache_layer + static_cast<size_t>(g) * max_seq_len * D;
  const __half *vbase = v_cache_layer + static_cast<size_t>(g) * max_seq_len * D;
  for (int k0 = 0; k0 <= last_key; k0 += ATT_KEYS) {
    __syncthreads();   // previous tile fully used (also orders the sq fill before the first use)
    for (int i = threadIdx.x; i < ATT_KEYS * (D / 8); i += 256) {
      const int j = i / (D / 8), c = i % (D / 8);
      uint4 kv = make_uint4(0, 0, 0, 0), vv = make_uint4(0, 0, 0, 0);
      if (k0 + j <= last_key) {
        kv = *reinterpret_cast<const uint4 *>(kbase + static_cast<size_t>(k0 + j) * D + c * 8);
        vv = *reinterpret_cast<const uint4 *>(vbase + static_cast<size_t>(k0 + j) * D + c * 8);
      }
      uint32_t *kd = reinterpret_cast<uint32_t *>(sk + j * ATT_KPITCH + c * 8);
      kd[0] = kv.x; kd[1] = kv.y; kd[2] = kv.z; kd[3] = kv.w;
      *reinterpret_cast<uint4 *>(sv + j * D + c * 8) = vv;
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < TPW; ++r) {
      const int tk = warp * TPW + r, tok = t0 + tk;
      if (tok >= T) continue;                       // warp-uniform
      const int limit = pos0 + tok;                 // last visible key of this query token
      if (k0 > limit) continue;                     // warp-uniform
      const float2 *qa = reinterpret_cast<const float2 *>(sq + (tk * 2 + 0) * D);
      const float2 *qb = reinterpret_cast<const float2 *>(sq + (tk * 2 + 1) * D);
      const __half2 *krow = reinterpret_cast<const __half2 *>(sk + lane * ATT_KPITCH);
      float sa = 0.f, sb = 0.f;
#pragma unroll 16
      for (int d = 0; d < D / 2; ++d) {
        const float2 kf = __half22float2(krow[d]);
        const float2 a = qa[d], b = qb[d];
        sa = fmaf(a.x, kf.x, sa); sa = fmaf(a.y, kf.y, sa);
        sb = fmaf(b.x, kf.x, sb); sb = fmaf(b.y, kf.y, sb);
      }
      const bool vis = (k0 + lane <= limit);
      sa = vis ? sa * sc : -INFINITY;
      sb = vis ? sb * sc : -INFINITY;
      const float ma = fmaxf(m[r][0], warp_max(sa)), mb = fmaxf(m[r][1], warp_max(sb));
      const float ca = exp2f(m[r][0] - ma), cb = exp2f(m[r][1] - mb);   // first tile: exp2f(-inf) = 0
      const float pa = exp2f(sa - ma), pb = exp2f(sb - mb);
      l[r][0] = l[r][0] * ca + warp_sum(pa);
      l[r][1] = l[r][1] * cb + warp_sum(pb);
      m[r][0] = ma; m[r][1] = mb;
      __syncwarp();
      sp[warp][0][lane] = pa;
      sp[warp][1][lane] = pb;
      __syncwarp();
#pragma unroll
      for (int d = 0; d < 4; ++d) { acc[r][0][d] *= ca; acc[r][1][d] *= cb; }
#pragma unroll 8
      for (int j = 0; j < ATT_KEYS; ++j) {
        const float pja = sp[warp][0][j], pjb = sp[warp][1][j];
        const uint2 vv = *reinterpret_cast<const uint2 *>(sv + j * D + lane * 4);
        const float2 v01 = __half22float2(*reinterpret_cast<const __half2 *>(&vv.x));
        const float2 v23 = __half22float2(*reinterpret_cast<const __half2 *>(&vv.y));
        acc[r][0][0] = fmaf(pja, v01.x, acc[r][0][0]); acc[r][0][1] = fmaf(pja, v01.y, acc[r][0][1]);
        acc[r][0][2] = fmaf(pja, v23.x, acc[r][0][2]); acc[r][0][3] = fmaf(pja, v23.y, acc[r][0][3]);
        acc[r][1][0] = fmaf(pjb, v01.x, acc[r][1][0]); acc[r][1][1] = fmaf(pjb, v01.y, acc[r][1][1]);
        acc[r][1][2] = fmaf(pjb, v23.x, acc[r][1][2]); acc[r][1][3] = fmaf(pjb, v23.y, acc[r][1][3]);
      }
    }
  }
#pragma unroll
  for (int r = 0; r < TPW; ++r) {
    const int tok = t0 + warp * TPW + r;
    if (tok >= T) continue;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const float inv = 1.0f / l[r][h];
      __half *dst = out + static_cast<size_t>(tok) * QS + (2 * g + h) * D + lane * 4;
      *reinterpret_cast<__half2 *>(dst) = __floats2half2_rn(acc[r][h][0] * inv, acc[r][h][1] * inv);
      *reinterpret_cast<__half2 *>(dst + 2) = __floats2half2_rn(acc[r][h][2] * inv, acc[r][h][3] * inv);
    }
  }
}

// act[t][m] = fp16(silu(gate[t][m]) * up[t][m]) in fp32 math.  grid-stride over T * I elements.
__global__ void silu_mul_rows(const float *gate, const float *up, __half *act, size_t n) {
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const float g = gate[i];
    act[i] = __float2half_rn(g / (1.0f + expf(-g)) * up[i]);
  }
}

}  // namespace qmk_pf
#endif  // QMK_PREFILL_KERNELS_CUH_
