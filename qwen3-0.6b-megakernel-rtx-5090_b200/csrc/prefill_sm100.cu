// Tensor-core side of the library: the tcgen05 GEMM and (built on it) the chunked prompt prefill.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <mutex>
#include <algorithm>
#include <string>

#include "../../include/qwen_megakernel.h"
#include "gemm_tcgen05.cuh"
#include "prefill_sm100.h"
#include "prefill_kernels.cuh"
#include "attention_tcgen05.cuh"
#include "decode_attention_mma.cuh"
#include "engine_internal.h"
#include <vector>

namespace qmk_tc {

namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

std::mutex g_mu;
EncodeTiledFn g_encode = nullptr;
bool g_attr_set[16] = {};
int g_sms[16] = {};

// The driver's tensor-map encoder, looked up through the runtime (no link against libcuda).
EncodeTiledFn encoder() {
  if (g_encode) return g_encode;
  void *fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess ||
      q != cudaDriverEntryPointSuccess)
    return nullptr;
  g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  return g_encode;
}

}  // namespace

// Tensor map of a row-major fp16 matrix [rows x cols]: boxes of box_rows x 64 elements, 128-byte swizzle.
int make_map_f16(CUtensorMap *map, const void *ptr, uint64_t rows, uint64_t cols, uint32_t box_rows, std::string *err) {
  EncodeTiledFn enc = encoder();
  if (!enc) { *err = "cuTensorMapEncodeTiled is not available from this driver"; return QMK_ERR_CUDA; }
  if ((reinterpret_cast<uintptr_t>(ptr) & 15u) || (cols * 2) % 16) { *err = "matrix not 16-byte aligned"; return QMK_ERR_BAD_ARGUMENT; }
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {cols * 2};
  const cuuint32_t box[2] = {64, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(ptr), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { *err = "cuTensorMapEncodeTiled failed with code " + std::to_string(static_cast<int>(r)); return QMK_ERR_CUDA; }
  return QMK_OK;
}

// Packed weight rows (weight formats 1 and 2): bytes of values, where the NVFP4 block scales and the 16-byte trailer
// with the fp32 scale sit inside a row, and the bytes between rows.
PackedRow packed_row(int wq, int K) {
  PackedRow r;
  r.data_bytes = wq == 1 ? static_cast<uint32_t>(K) : static_cast<uint32_t>(K) / 2;
  r.bs_off = r.data_bytes;
  r.scale_off = wq == 1 ? r.data_bytes : r.data_bytes + static_cast<uint32_t>(K) / 16;
  r.pitch = r.scale_off + 16;
  return r;
}

// Tensor map of the VALUES of a packed matrix (bytes; scales and trailers stay outside the mapped extent): boxes of
// box_rows rows x one 64-value K block, no swizzle - the expanding warps read it linearly.
int make_map_packed(CUtensorMap *map, const void *ptr, uint64_t rows, int K, uint32_t box_rows, int wq, std::string *err) {
  EncodeTiledFn enc = encoder();
  if (!enc) { *err = "cuTensorMapEncodeTiled is not available from this driver"; return QMK_ERR_CUDA; }
  const PackedRow pr = packed_row(wq, K);
  if ((reinterpret_cast<uintptr_t>(ptr) & 15u) || K % 64 || K > qmk_gemm::MAX_K_PACKED || pr.pitch % 16) {
    *err = "packed matrix: base not 16-byte aligned, or K not a multiple of 64 (NVFP4: of 256, rows must stay 16-byte aligned) up to 3072";
    return QMK_ERR_BAD_ARGUMENT;
  }
  const cuuint64_t dims[2] = {pr.data_bytes, rows};
  const cuuint64_t strides[1] = {pr.pitch};
  const cuuint32_t box[2] = {qmk_gemm::raw_row_bytes(wq), box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(ptr), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { *err = "cuTensorMapEncodeTiled failed with code " + std::to_string(static_cast<int>(r)); return QMK_ERR_CUDA; }
  return QMK_OK;
}
int make_map_b(CUtensorMap *map, const void *ptr, uint64_t rows, int K, uint32_t box_rows, int wq, std::string *err) {
  return wq ? make_map_packed(map, ptr, rows, K, box_rows, wq, err) : make_map_f16(map, ptr, rows, static_cast<uint64_t>(K), box_rows, err);
}

// 3-D tensor map of an fp16 KV cache [heads][max_seq_len][128] of which the first `rows` positions of every head are
// valid: boxes of 64 dims x 64 positions of one head, 128-byte swizzle; positions >= rows read as zeros.
int make_map_kv(CUtensorMap *map, const void *cache, uint64_t rows, uint64_t max_seq_len, uint64_t heads, std::string *err) {
  EncodeTiledFn enc = encoder();
  if (!enc) { *err = "cuTensorMapEncodeTiled is not available from this driver"; return QMK_ERR_CUDA; }
  if (reinterpret_cast<uintptr_t>(cache) & 15u) { *err = "cache not 16-byte aligned"; return QMK_ERR_BAD_ARGUMENT; }
  const cuuint64_t dims[3] = {128, rows, heads};
  const cuuint64_t strides[2] = {256, max_seq_len * 256};
  const cuuint32_t box[3] = {64, 64, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void *>(cache), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { *err = "cuTensorMapEncodeTiled (cache) failed with code " + std::to_string(static_cast<int>(r)); return QMK_ERR_CUDA; }
  return QMK_OK;
}

// Width of the N tiles for C[M x N] = A[M x K] * B[N x K]^T (M, N multiples of 128).  `map_b` must have been made
// with that many rows per box.  Skinny problems are bound by how many SMs pull operands at once and by the fixed
// cost of a CTA (launch, barrier and TMEM set-up, pipeline fill, epilogue - worth about 320 columns of streaming in
// the launch lists of decode steps), so: as few waves as possible, then the narrower tile.  `b_tiles` = B tiles a
// CTA multiplies per K block (2 for the fused gate/up kernel, whose widest tile is 64).
static int sm_count() {
  int dev = 0;
  cudaGetDevice(&dev);
  int sms = (dev >= 0 && dev < 16) ? g_sms[dev] : 0;
  if (sms == 0) {
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (dev >= 0 && dev < 16) g_sms[dev] = sms;
  }
  return sms > 0 ? sms : 148;
}
thread_local unsigned int t_ring_budget = 0;   // shared-memory budget of the ring (0 = the compile-time depth, one CTA per SM)
static int pick_box_n(int M, int N, int b_tiles) {
  const int sms = sm_count() * (t_ring_budget ? 2 : 1);   // CTA slots of one wave: rings sized to a budget share an SM in pairs
  int best = 0;
  long best_cost = 0;
  for (int bn = b_tiles == 2 ? 64 : 128; bn >= 32; bn /= 2) {
    const long ctas = static_cast<long>(M / qmk_gemm::BM) * (N / bn);
    const long cost = ((ctas + sms - 1) / sms) * (b_tiles * bn + 320);
    if (best == 0 || cost < best_cost) { best = bn; best_cost = cost; }
  }
  return best;
}
int gemm_sm_count() { return sm_count(); }
int gemm_box_n(int M, int N) { return pick_box_n(M, N, 1); }
int gemm_box_n_fused(int M, int N) { return pick_box_n(M, N, 2); }

// Launches of a decode step carry the programmatic-stream-serialisation attribute (see pdl_wait in
// prefill_kernels.cuh); the step builder switches it on for the calling thread, everything else launches plainly.
thread_local bool t_pdl = false;
PdlScope::PdlScope(bool on) : prev_(t_pdl) { t_pdl = on; }
PdlScope::~PdlScope() { t_pdl = prev_; }
bool pdl_active() { return t_pdl; }

// The kernel for an N tile, epilogue and weight format, and its dynamic shared memory.
using GemmKernel = void (*)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const CUtensorMap, const qmk_gemm::Groups,
                            int, int, unsigned int *, unsigned long long, int);
template <int WQ>
static GemmKernel gemm_kernel_wq(int bn, bool fuse) {
  if (fuse) return bn == 32 ? qmk_gemm::gemm_f16_tn_kernel<32, true, WQ> : qmk_gemm::gemm_f16_tn_kernel<64, true, WQ>;
  return bn == 32 ? qmk_gemm::gemm_f16_tn_kernel<32, false, WQ>
                  : bn == 64 ? qmk_gemm::gemm_f16_tn_kernel<64, false, WQ> : qmk_gemm::gemm_f16_tn_kernel<128, false, WQ>;
}
// (the widest tiles - 256 B rows per stage - exist for fp16 weights only)
static GemmKernel gemm_kernel(int bn, bool fuse, int wq) {
  if (wq == 0 && fuse && bn == 128) return qmk_gemm::gemm_f16_tn_kernel<128, true, 0>;
  if (wq == 0 && !fuse && bn == 256) return qmk_gemm::gemm_f16_tn_kernel<256, false, 0>;
  return wq == 0 ? gemm_kernel_wq<0>(bn, fuse) : wq == 1 ? gemm_kernel_wq<1>(bn, fuse) : gemm_kernel_wq<2>(bn, fuse);
}
static size_t gemm_smem(int bn, bool fuse, int wq) { return qmk_gemm::smem_bytes_for(fuse ? 2 * bn : bn, wq); }

// Opt-in shared-memory size of every tile variant, once per device (outside any stream capture).
int ensure_gemm_attrs(std::string *err) {
  int dev = 0;
  cudaGetDevice(&dev);
  std::lock_guard<std::mutex> lock(g_mu);
  if (dev >= 0 && dev < 16 && !g_attr_set[dev]) {
    cudaError_t e = cudaSuccess;
    for (int wq = 0; wq < 3 && e == cudaSuccess; ++wq)
      for (int fuse = 0; fuse < 2 && e == cudaSuccess; ++fuse)
        for (int bn = 32; bn <= (fuse ? 64 : 128) * (wq == 0 ? 2 : 1) && e == cudaSuccess; bn *= 2)
          e = cudaFuncSetAttribute(reinterpret_cast<const void *>(gemm_kernel(bn, fuse != 0, wq)),
                                   cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(gemm_smem(bn, fuse != 0, wq)));
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(qmk_pf::causal_attention_mma, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               qmk_pf::ATM_SMEM_BYTES);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(qmk_attn::causal_attention_tc, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(qmk_attn::SMEM_BYTES));
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(qmk_pf::decode_attention_ring, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               qmk_pf::DAR_SMEM_BYTES);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(qmk_pf::decode_attention_mma, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               qmk_pf::DAM_SMEM_BYTES);
    if (e != cudaSuccess) { *err = std::string("cudaFuncSetAttribute: ") + cudaGetErrorString(e); return QMK_ERR_CUDA; }
    g_attr_set[dev] = true;
  }
  return QMK_OK;
}

// Packed-weight fields of a launch: row geometry for K and the groups' base pointers.
static bool set_packed(qmk_gemm::Groups *gr, int wq, int K, int ngroups, const void *const *raws, std::string *err) {
  for (int g = 0; g < qmk_gemm::MAX_GROUPS; ++g) gr->braw[g] = nullptr;
  gr->raw_pitch = gr->raw_bs_off = gr->raw_scale_off = 0;
  if (wq == 0) return true;
  if (wq < 0 || wq > 2 || !raws || K > qmk_gemm::MAX_K_PACKED) { *err = "gemm: bad packed-weight arguments"; return false; }
  const PackedRow pr = packed_row(wq, K);
  gr->raw_pitch = pr.pitch;
  gr->raw_bs_off = pr.bs_off;
  gr->raw_scale_off = pr.scale_off;
  for (int g = 0; g < ngroups; ++g) {
    if (!raws[g]) { *err = "gemm: null packed matrix"; return false; }
    gr->braw[g] = static_cast<const unsigned char *>(raws[g]);
  }
  return true;
}

// Ring depth of a launch (see qmk_gemm::ring_geometry): `sb` = B rows per stage; returns the dynamic shared memory.
thread_local float *t_amax_val = nullptr;   // the next single-matrix GEMM of this thread leaves (value, column) pairs here
thread_local int *t_amax_idx = nullptr;
static size_t set_ring(qmk_gemm::Groups *gr, int sb, int wq) {
  const qmk_gemm::RingGeometry g = qmk_gemm::ring_geometry(sb, wq, t_ring_budget);
  gr->stages = g.stages;
  gr->ring_bytes = g.ring_bytes;
  return g.smem_bytes;
}

RingBudgetScope::RingBudgetScope(unsigned int bytes) : prev_(t_ring_budget) { t_ring_budget = bytes; }
RingBudgetScope::~RingBudgetScope() { t_ring_budget = prev_; }
void set_argmax_target(float *val, int *idx) { t_amax_val = val; t_amax_idx = idx; }
thread_local bool t_out_f16 = false;        // the next grouped GEMM of this thread stores fp16
void set_out_f16(bool on) { t_out_f16 = on; }
size_t selftest_ring(qmk_gemm::Groups *gr) { return set_ring(gr, 128, 0); }

// A maps with short boxes (`a_box_rows` < 128 rows per box, a multiple of 8; decode steps with few live rows): one
// row tile only, and the epilogue must stay inside the box.
static bool a_box_ok(int a_box_rows, int M, int *rows, uint32_t *a_box_bytes, std::string *err) {
  *a_box_bytes = 0;
  if (a_box_rows <= 0 || a_box_rows == qmk_gemm::BM) return true;
  if (a_box_rows % 8 || a_box_rows > qmk_gemm::BM || M != qmk_gemm::BM) { *err = "gemm: bad A box"; return false; }
  if (*rows > a_box_rows) *rows = a_box_rows;
  *a_box_bytes = static_cast<uint32_t>(a_box_rows) * qmk_gemm::BK * 2;
  return true;
}

// C_g[M x N_g] fp32 = A[M x K] * B_g[N_g x K]^T for up to three matrices B_g in one launch.  M, N_g multiples of
// 128; K a multiple of 64; every B map made with `box_n` rows per box (gemm_box_n(M, sum of N_g)).
int launch_gemm_grouped(const CUtensorMap &map_a, int ngroups, const CUtensorMap *const *maps_b, float *const *Cs,
                        const int *Ns, int M, int K, int box_n, unsigned int *status, int timeout_ms, cudaStream_t stream,
                        std::string *err, int live_rows, int a_box_rows, int wq, const void *const *raws) {
  bool bad = M <= 0 || K <= 0 || M % qmk_gemm::BM || K % qmk_gemm::BK ||
             (box_n != 32 && box_n != 64 && box_n != 128 && !(box_n == 256 && wq == 0)) ||
             ngroups < 1 || ngroups > qmk_gemm::MAX_GROUPS;
  for (int g = 0; !bad && g < ngroups; ++g) bad = Ns[g] <= 0 || Ns[g] % (box_n > 128 ? box_n : 128);
  if (bad) {
    *err = "gemm: M and N must be multiples of 128 and K a multiple of 64";
    return QMK_ERR_BAD_ARGUMENT;
  }
  const int arc = ensure_gemm_attrs(err);
  if (arc != QMK_OK) return arc;
  qmk_gemm::Groups gr;
  gr.kblocks_per_split = 0;
  gr.split_stride = 0;
  if (!set_packed(&gr, wq, K, ngroups, raws, err)) return QMK_ERR_BAD_ARGUMENT;
  gr.out_f16 = t_out_f16 ? 1 : 0;
  gr.amax_val = ngroups == 1 ? t_amax_val : nullptr;   // (set around the LM-head launch of a decode step only)
  gr.amax_idx = ngroups == 1 ? t_amax_idx : nullptr;
  int tiles = 0;
  for (int g = 0; g < qmk_gemm::MAX_GROUPS; ++g) {
    gr.C[g] = g < ngroups ? Cs[g] : nullptr;
    gr.N[g] = g < ngroups ? Ns[g] : 0;
    tiles += gr.N[g] / box_n;
  }
  const CUtensorMap &b0 = *maps_b[0], &b1 = *maps_b[ngroups > 1 ? 1 : 0], &b2 = *maps_b[ngroups > 2 ? 2 : 0];
  dim3 grid(tiles, M / qmk_gemm::BM);
  const unsigned long long budget = static_cast<unsigned long long>(timeout_ms) * 1000000ull;
  int rows = live_rows > 0 ? live_rows : M;   // rows the epilogue stores (the rest of the tile is padding)
  if (!a_box_ok(a_box_rows, M, &rows, &gr.a_box_bytes, err)) return QMK_ERR_BAD_ARGUMENT;
  const size_t smem = set_ring(&gr, box_n, wq);
  cudaError_t e = launch_kernel(gemm_kernel(box_n, false, wq), grid, dim3(qmk_gemm::threads_for(wq)), smem, stream,
                                map_a, b0, b1, b2, gr, rows, K, status, budget, 0);
  if (e != cudaSuccess) { *err = std::string("gemm launch: ") + cudaGetErrorString(e); return QMK_ERR_CUDA; }
  return QMK_OK;
}

// act[M x N] fp16 = silu(A * Gate^T) * (A * Up^T): the gate/up pair of the MLP with the SwiGLU in the epilogue.
// Both maps made with `box_n` (64 or 32) rows per box.
int launch_gemm_swiglu(const CUtensorMap &map_a, const CUtensorMap &map_gate, const CUtensorMap &map_up, __half *act, int M,
                       int N, int K, unsigned int *status, int timeout_ms, cudaStream_t stream, std::string *err,
                       int box_n, int live_rows, int a_box_rows, int wq, const void *raw_gate, const void *raw_up) {
  if (M <= 0 || N <= 0 || K <= 0 || M % qmk_gemm::BM || N % 128 || K % qmk_gemm::BK ||
      (box_n != 32 && box_n != 64 && !(box_n == 128 && wq == 0))) {
    *err = "gemm: M and N must be multiples of 128 and K a multiple of 64";
    return QMK_ERR_BAD_ARGUMENT;
  }
  const int arc = ensure_gemm_attrs(err);
  if (arc != QMK_OK) return arc;
  qmk_gemm::Groups gr;
  gr.C[0] = reinterpret_cast<float *>(act); gr.C[1] = nullptr; gr.C[2] = nullptr;
  gr.N[0] = N; gr.N[1] = 0; gr.N[2] = 0;
  gr.kblocks_per_split = 0;
  gr.split_stride = 0;
  const void *raws[2] = {raw_gate, raw_up};
  if (!set_packed(&gr, wq, K, 2, raws, err)) return QMK_ERR_BAD_ARGUMENT;
  gr.amax_val = nullptr;
  gr.out_f16 = 0;
  gr.amax_idx = nullptr;
  int rows = live_rows > 0 ? live_rows : M;
  if (!a_box_ok(a_box_rows, M, &rows, &gr.a_box_bytes, err)) return QMK_ERR_BAD_ARGUMENT;
  const unsigned long long budget = static_cast<unsigned long long>(timeout_ms) * 1000000ull;
  const size_t smem = set_ring(&gr, 2 * box_n, wq);
  cudaError_t e = launch_kernel(gemm_kernel(box_n, true, wq), dim3(N / box_n, M / qmk_gemm::BM), dim3(qmk_gemm::threads_for(wq)),
                                smem, stream, map_a, map_gate, map_up, map_up, gr, rows, K, status, budget, 0);
  if (e != cudaSuccess) { *err = std::string("gemm launch: ") + cudaGetErrorString(e); return QMK_ERR_CUDA; }
  return QMK_OK;
}

// Split-K form for skinny problems (one 128-row tile, long K): `splits` CTAs per output tile, partial matrices
// C + z * M * N.  K / 64 must be a multiple of `splits`.  `map_b` made with `box_n` (64 or 32) rows per box.
int launch_gemm_splitk(const CUtensorMap &map_a, const CUtensorMap &map_b, float *C, int M, int N, int K, int splits,
                       unsigned int *status, int timeout_ms, cudaStream_t stream, std::string *err, int box_n,
                       int live_rows, int a_box_rows, int wq, const void *raw) {
  if (M <= 0 || N <= 0 || K <= 0 || M % qmk_gemm::BM || N % 128 || K % qmk_gemm::BK || splits < 1 ||
      (K / qmk_gemm::BK) % splits || (box_n != 32 && box_n != 64 && box_n != 128 && !(box_n == 256 && wq == 0 && N % 256 == 0))) {
    *err = "gemm: bad split-K shape";
    return QMK_ERR_BAD_ARGUMENT;
  }
  const int arc = ensure_gemm_attrs(err);
  if (arc != QMK_OK) return arc;
  qmk_gemm::Groups gr;
  gr.C[0] = C; gr.C[1] = nullptr; gr.C[2] = nullptr;
  gr.N[0] = N; gr.N[1] = 0; gr.N[2] = 0;
  gr.kblocks_per_split = K / qmk_gemm::BK / splits;
  gr.split_stride = static_cast<size_t>(M) * N;
  if (!set_packed(&gr, wq, K, 1, &raw, err)) return QMK_ERR_BAD_ARGUMENT;
  gr.amax_val = nullptr;
  gr.out_f16 = 0;
  gr.amax_idx = nullptr;
  int rows = live_rows > 0 ? live_rows : M;
  if (!a_box_ok(a_box_rows, M, &rows, &gr.a_box_bytes, err)) return QMK_ERR_BAD_ARGUMENT;
  const unsigned long long budget = static_cast<unsigned long long>(timeout_ms) * 1000000ull;
  const size_t smem = set_ring(&gr, box_n, wq);
  cudaError_t e = launch_kernel(gemm_kernel(box_n, false, wq), dim3(N / box_n, M / qmk_gemm::BM, splits), dim3(qmk_gemm::threads_for(wq)),
                                smem, stream, map_a, map_b, map_b, map_b, gr, rows, K, status, budget, 0);
  if (e != cudaSuccess) { *err = std::string("gemm launch: ") + cudaGetErrorString(e); return QMK_ERR_CUDA; }
  return QMK_OK;
}

int launch_gemm(const CUtensorMap &map_a, const CUtensorMap &map_b, float *C, int M, int N, int K, int box_n,
                unsigned int *status, int timeout_ms, cudaStream_t stream, std::string *err, int live_rows, int a_box_rows,
                int wq, const void *raw) {
  const CUtensorMap *maps[1] = {&map_b};
  float *Cs[1] = {C};
  const int Ns[1] = {N};
  return launch_gemm_grouped(map_a, 1, maps, Cs, Ns, M, K, box_n, status, timeout_ms, stream, err, live_rows, a_box_rows, wq,
                             &raw);
}

}  // namespace qmk_tc

// ----------------------------------------------------------------------------- chunked prefill
namespace {

constexpr unsigned int PREFILL_RING_BYTES = 96 * 1024, GATE_UP_RING_BYTES = 64 * 1024;
constexpr int CHUNK = 4096;         // prompt tokens per pass over the weights (a multiple of the GEMM's 128)
constexpr int MAX_LAYERS = 48;

struct Workspace {                  // per device, allocated on first use, never freed (like the engine's scratch)
  bool ready = false;
  int *tokens = nullptr;
  float *x = nullptr, *q = nullptr, *k = nullptr, *v = nullptr, *qr = nullptr, *o = nullptr, *down = nullptr;
  __half *xn = nullptr, *attn = nullptr, *act = nullptr;
  unsigned int *status = nullptr;
  CUtensorMap map_xn, map_attn, map_act, map_qh;
  // batched decode: per-sequence state and the logits of one step
  int *positions = nullptr, *start_positions = nullptr;
  cudaStream_t gstream = nullptr;        // capture needs a non-default stream
  cudaEvent_t ev_in = nullptr, ev_out = nullptr;
  // One captured decode step per batch size (a serving loop's live count changes from round to round and
  // instantiating ~200 nodes costs tens of milliseconds); entry B is valid while its key matches.
  cudaGraphExec_t step_graph[129] = {};
  unsigned long long step_key[129][12] = {};
  unsigned long long graph_epoch = 1;    // bumped whenever tensor maps baked into the graphs are rebuilt
  __half **k_ptrs = nullptr, **v_ptrs = nullptr;
  CUtensorMap *kv_maps = nullptr;        // [128][2]: tiled-copy descriptors of every sequence's K and V cache (decode_attention_mma)
  unsigned char *packed = nullptr;       // tables of a packed prefill (row info, attention items, per-sequence descriptors and cache pointers)
  int **log_ptrs = nullptr;
  float *split_part = nullptr;            // partial attention states of split sequences (decode_attention_ring)
  unsigned int *split_count = nullptr;    // arrival counters, one per (sequence, kv head); zero between launches
  float *logits = nullptr;
  int logits_vocab = 0;
  float *amax_val = nullptr;              // [128][vocab / 128] pairs of the LM-head epilogue's greedy pick
  int *amax_idx = nullptr;
  const void *lm_ptr = nullptr;
  int lm_wq = 0;
  CUtensorMap map_lm;
  // A-operand maps that expose only the live rows: the rest of the 128-row box is zero-filled by the TMA unit
  // without being read, which cuts the activation traffic of a small batch by 128 / rows
  int a_rows = 0;
  CUtensorMap map_xn_b, map_attn_b, map_act_b;
  // weight maps of the layer table seen last (rebuilt when the table's contents change)
  unsigned long long table[MAX_LAYERS * 12] = {};
  int table_layers = 0;
  int table_wq = 0;                    // weight format the maps below were made for
  CUtensorMap wmap[MAX_LAYERS][7][3];  // q, k, v, o, gate, up, down; boxes of 64, 128 and (fp16 weights) 256 rows
  CUtensorMap wmap32[MAX_LAYERS][7];   // the same matrices in boxes of 32 rows (decode steps: more, smaller tiles)
};
// Prefill and batched decode keep separate workspaces and locks: a serving loop prefills the next request on one
// stream (and thread) while a decode step of the live sequences runs on another.
Workspace g_ws[16], g_ws_decode[16];
std::mutex g_ws_mu, g_ws_decode_mu;

#define PF_CUDA(call)                                                                             \
  do {                                                                                            \
    cudaError_t err__ = (call);                                                                   \
    if (err__ != cudaSuccess)                                                                     \
      return qmk_internal::report(QMK_ERR_CUDA, std::string(#call) + ": " + cudaGetErrorString(err__)); \
  } while (0)

// `rows`: activation rows the buffers hold (CHUNK for prefill, one 128-row tile for the batched decode)
int ensure_workspace(Workspace &w, int rows) {
  if (w.ready) return QMK_OK;
  using namespace qmk_pf;
  const size_t C = static_cast<size_t>(rows);
  PF_CUDA(cudaMalloc(&w.tokens, sizeof(int) * C));
  PF_CUDA(cudaMalloc(&w.x, sizeof(float) * C * H));
  PF_CUDA(cudaMalloc(&w.q, sizeof(float) * C * QS));
  PF_CUDA(cudaMalloc(&w.k, sizeof(float) * C * KVS));
  PF_CUDA(cudaMalloc(&w.v, sizeof(float) * C * KVS));
  PF_CUDA(cudaMalloc(&w.qr, sizeof(float) * C * QS));
  PF_CUDA(cudaMalloc(&w.o, sizeof(float) * 2 * C * H));      // (two split-K partial matrices of a prefill chunk)
  PF_CUDA(cudaMalloc(&w.down, sizeof(float) * 2 * C * H));
  PF_CUDA(cudaMalloc(&w.xn, sizeof(__half) * C * H));
  PF_CUDA(cudaMalloc(&w.attn, sizeof(__half) * C * QS));
  PF_CUDA(cudaMalloc(&w.act, sizeof(__half) * C * I));
  PF_CUDA(cudaMalloc(&w.status, 16));
  // GEMM operand rows beyond a short chunk are read (and ignored): they must hold finite numbers
  PF_CUDA(cudaMemset(w.xn, 0, sizeof(__half) * C * H));
  PF_CUDA(cudaMemset(w.attn, 0, sizeof(__half) * C * QS));
  PF_CUDA(cudaMemset(w.act, 0, sizeof(__half) * C * I));
  PF_CUDA(cudaMemset(w.qr, 0, sizeof(float) * C * QS));
  std::string err;
  int rc = qmk_tc::make_map_f16(&w.map_xn, w.xn, C, H, qmk_gemm::BM, &err);
  if (rc == QMK_OK) rc = qmk_tc::make_map_f16(&w.map_attn, w.attn, C, QS, qmk_gemm::BM, &err);
  if (rc == QMK_OK) rc = qmk_tc::make_map_f16(&w.map_act, w.act, C, I, qmk_gemm::BM, &err);
  // the rotated queries as fp16 (the first half of the fp32 buffer), read by the attention kernel in 128-row boxes
  if (rc == QMK_OK) rc = qmk_tc::make_map_f16(&w.map_qh, w.qr, C, QS, qmk_gemm::BM, &err);
  if (rc != QMK_OK) return qmk_internal::report(rc, err);
  w.ready = true;
  return QMK_OK;
}

// Tensor maps of the seven projection matrices of every layer.  The layer table lives in device memory
// (the reference's packed pointer records): it is read back and the maps are rebuilt only when it changed.
int ensure_weight_maps(Workspace &w, const LDGLayerWeight *layers_dev, int num_layers, int wq, cudaStream_t stream) {
  using namespace qmk_pf;
  std::vector<unsigned long long> host(static_cast<size_t>(num_layers) * 12);
  PF_CUDA(cudaMemcpyAsync(host.data(), layers_dev, host.size() * 8, cudaMemcpyDeviceToHost, stream));
  PF_CUDA(cudaStreamSynchronize(stream));
  if (w.table_layers == num_layers && w.table_wq == wq && memcmp(host.data(), w.table, host.size() * 8) == 0) return QMK_OK;
  // record order: in_ln, wq, wk, wv, q_norm, k_norm, wo, post_ln, gate, up, down, pad
  static const int slot[7] = {1, 2, 3, 6, 8, 9, 10};
  static const int rows[7] = {QS, KVS, KVS, H, I, I, H};
  static const int cols[7] = {H, H, H, QS, H, H, I};
  std::string err;
  for (int l = 0; l < num_layers; ++l)
    for (int j = 0; j < 7; ++j) {
      const void *ptr = reinterpret_cast<const void *>(host[static_cast<size_t>(l) * 12 + slot[j]]);
      if (!ptr) return qmk_internal::report(QMK_ERR_BAD_ARGUMENT, "prefill: null weight pointer in the layer table");
      {
        const int rc = qmk_tc::make_map_b(&w.wmap32[l][j], ptr, rows[j], cols[j], 32, wq, &err);
        if (rc != QMK_OK) return qmk_internal::report(rc, err);
      }
      for (int b = 0; b < (wq == 0 ? 3 : 2); ++b) {
        const int rc = qmk_tc::make_map_b(&w.wmap[l][j][b], ptr, rows[j], cols[j], 64 << b, wq, &err);
        if (rc != QMK_OK) return qmk_internal::report(rc, err);
      }
    }
  memcpy(w.table, host.data(), host.size() * 8);
  w.table_layers = num_layers;
  w.table_wq = wq;
  ++w.graph_epoch;   // captured decode steps hold the old maps
  return QMK_OK;
}

}  // namespace

namespace {
// Several prompts in one pass: sequence s holds lens[s] tokens (concatenated in token_ids_host) and owns the caches
// k_caches[s] / v_caches[s]; every sequence starts at position 0.
struct PackedSeqs {
  int num_seqs;
  const int *lens;
  void *const *k_caches, *const *v_caches;
};
constexpr int MAX_PACKED_SEQS = 64;
constexpr size_t PK_ROWS_OFF = 0, PK_ITEMS_OFF = 32768, PK_MAPS_OFF = 49152, PK_PTRS_OFF = 65536, PK_BYTES = 66560;

int prefill_impl(const int *token_ids_host, int num_tokens, const void *embed_weight, const LDGLayerWeight *layer_weights,
                 const void *cos_table, const void *sin_table, void *k_cache, void *v_cache, int num_layers,
                 int start_position, int max_seq_len, float attn_scale, cudaStream_t stream, const PackedSeqs *pk) {
  using namespace qmk_pf;
  if (num_tokens <= 0) return QMK_OK;
  qmk_internal::PrefillEnv env;
  int rc = qmk_internal::prefill_env(max_seq_len, stream, &env);
  if (rc != QMK_OK) return rc;
  if (!token_ids_host || !embed_weight || !layer_weights || (!pk && (!k_cache || !v_cache)))
    return qmk_internal::report(QMK_ERR_BAD_ARGUMENT, "prefill: null pointer argument");
  const int wq = env.wfmt;   // 0 fp16, 1 FP8-E4M3 rows, 2 NVFP4 rows: packed matrices are expanded inside the GEMM
  if (num_layers < 1 || num_layers > MAX_LAYERS)
    return qmk_internal::report(QMK_ERR_BAD_ARGUMENT, "num_layers must be in [1, 48]");
  if (!pk && (start_position < 0 || start_position + num_tokens > max_seq_len))
    return qmk_internal::report(QMK_ERR_POSITION, "start_position + steps exceeds max_seq_len");
  if (pk) {
    if (pk->num_seqs < 1 || pk->num_seqs > MAX_PACKED_SEQS || !pk->lens || !pk->k_caches || !pk->v_caches || start_position != 0)
      return qmk_internal::report(QMK_ERR_BAD_ARGUMENT, "packed prefill: 1 to 64 sequences, each from position 0");
    int total = 0;
    for (int s = 0; s < pk->num_seqs; ++s) {
      if (pk->lens[s] < 1 || !pk->k_caches[s] || !pk->v_caches[s])
        return qmk_internal::report(QMK_ERR_BAD_ARGUMENT, "packed prefill: empty sequence or null cache");
      if (pk->lens[s] > max_seq_len) return qmk_internal::report(QMK_ERR_POSITION, "a prompt exceeds max_seq_len");
      total += pk->lens[s];
    }
    if (total != num_tokens) return qmk_internal::report(QMK_ERR_BAD_ARGUMENT, "packed prefill: lengths do not add up to num_tokens");
  }
  if (env.rope_from_table && (!cos_table || !sin_table))
    return qmk_internal::report(QMK_ERR_BAD_ARGUMENT, "rope_from_table needs cos/sin tables");
  for (int i = 0; i < num_tokens; ++i)
    if (token_ids_host[i] < 0 || token_ids_host[i] >= env.vocab)
      return qmk_internal::report(QMK_ERR_BAD_TOKEN, "prompt token outside [0, vocab)");
  int dev = 0;
  PF_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 16) return qmk_internal::report(QMK_ERR_CUDA, "device index out of range");
  std::lock_guard<std::mutex> lock(g_ws_mu);
  Workspace &w = g_ws[dev];
  rc = ensure_workspace(w, CHUNK);
  if (rc == QMK_OK) rc = ensure_weight_maps(w, layer_weights, num_layers, wq, stream);
  if (rc != QMK_OK) return rc;
  // ---- packed prompts: rows = the sequences one after the other, each padded to whole 128-row tiles
  std::vector<int> padded_tokens;
  std::vector<unsigned char> pk_host;
  int pk_items = 0;
  if (pk) {
    if (!env.attn_tc) return qmk_internal::report(QMK_ERR_BAD_ARGUMENT, "packed prefill needs the tcgen05 attention kernel");
    if (!w.packed) PF_CUDA(cudaMalloc(&w.packed, PK_BYTES));
    pk_host.assign(PK_BYTES, 0);
    int2 *rows = reinterpret_cast<int2 *>(pk_host.data() + PK_ROWS_OFF);
    int4 *items = reinterpret_cast<int4 *>(pk_host.data() + PK_ITEMS_OFF);
    CUtensorMap *maps = reinterpret_cast<CUtensorMap *>(pk_host.data() + PK_MAPS_OFF);
    unsigned long long *ptrs = reinterpret_cast<unsigned long long *>(pk_host.data() + PK_PTRS_OFF);
    int total_rows = 0;
    for (int s = 0; s < pk->num_seqs; ++s) total_rows += (pk->lens[s] + qmk_gemm::BM - 1) / qmk_gemm::BM * qmk_gemm::BM;
    if (total_rows > CHUNK) return qmk_internal::report(QMK_ERR_BAD_ARGUMENT, "packed prefill: more than 4096 padded rows");
    padded_tokens.assign(total_rows, 0);
    for (int i = 0; i < total_rows; ++i) rows[i] = make_int2(0, -1);
    std::vector<std::pair<int, int4>> order;   // (key tiles, item)
    std::string merr;
    int row0 = 0, tok0 = 0;
    for (int s = 0; s < pk->num_seqs; ++s) {
      const int len = pk->lens[s];
      for (int i = 0; i < len; ++i) {
        padded_tokens[row0 + i] = token_ids_host[tok0 + i];
        rows[row0 + i] = make_int2(s, i);
      }
      ptrs[2 * s] = reinterpret_cast<unsigned long long>(pk->k_caches[s]);
      ptrs[2 * s + 1] = reinterpret_cast<unsigned long long>(pk->v_caches[s]);
      int mrc = qmk_tc::make_map_kv(&maps[2 * s], pk->k_caches[s], static_cast<uint64_t>(len), static_cast<uint64_t>(max_seq_len),
                                    static_cast<uint64_t>(num_layers) * NKV, &merr);
      if (mrc == QMK_OK)
        mrc = qmk_tc::make_map_kv(&maps[2 * s + 1], pk->v_caches[s], static_cast<uint64_t>(len), static_cast<uint64_t>(max_seq_len),
                                  static_cast<uint64_t>(num_layers) * NKV, &merr);
      if (mrc != QMK_OK) return qmk_internal::report(mrc, merr);
      for (int qt = 0; qt * qmk_attn::TQ < len; ++qt) {
        const int last = (qt + 1) * qmk_attn::TQ < len ? (qt + 1) * qmk_attn::TQ - 1 : len - 1;
        for (int h = 0; h < NQ; ++h)
          order.push_back({last / qmk_attn::TK + 1, make_int4(s, row0 + qt * qmk_attn::TQ, qt * qmk_attn::TQ, h | (len << 8))});
      }
      row0 += (len + qmk_gemm::BM - 1) / qmk_gemm::BM * qmk_gemm::BM;
      tok0 += len;
    }
    std::stable_sort(order.begin(), order.end(), [](const auto &a, const auto &b) { return a.first > b.first; });   // longest job first
    pk_items = static_cast<int>(order.size());
    for (int i = 0; i < pk_items; ++i) items[i] = order[i].second;
    PF_CUDA(cudaMemcpyAsync(w.packed, pk_host.data(), PK_BYTES, cudaMemcpyHostToDevice, stream));
    token_ids_host = padded_tokens.data();
    num_tokens = total_rows;
  }
  std::vector<unsigned long long> rec(w.table, w.table + static_cast<size_t>(num_layers) * 12);
  const float *rope = env.rope_from_table ? nullptr : env.rope;
  const __half *cosv = static_cast<const __half *>(cos_table), *sinv = static_cast<const __half *>(sin_table);
  const size_t layer_stride = static_cast<size_t>(NKV) * max_seq_len * D;
  PF_CUDA(cudaMemsetAsync(w.status, 0, 16, stream));
  std::string err;
  // weight matrix j of layer l in boxes of `box_n` rows
  auto wmap_for = [&](int l, int j, int box_n) -> const CUtensorMap & {
    return box_n == 32 ? w.wmap32[l][j] : w.wmap[l][j][box_n == 64 ? 0 : box_n == 128 ? 1 : 2];
  };
  static const int rec_slot[7] = {1, 2, 3, 6, 8, 9, 10};   // q, k, v, o, gate, up, down inside a layer record
  auto wptr = [&](int l, int j) { return reinterpret_cast<const void *>(rec[static_cast<size_t>(l) * 12 + rec_slot[j]]); };
  auto gemm = [&](const CUtensorMap &a, int l, int j, float *c, int M, int N, int K, int live) {
    const int box_n = qmk_tc::gemm_box_n(M, N);
    return qmk_tc::launch_gemm(a, wmap_for(l, j, box_n), c, M, N, K, box_n, w.status, env.timeout_ms, stream, &err, live, 0,
                               wq, wptr(l, j));
  };
  // several matrices against the same activations in one launch (q/k/v)
  auto gemm_group = [&](const CUtensorMap &a, int l, int n, const int *js, float *const *cs, const int *ns, int M, int K,
                        int live) {
    int total = 0;
    for (int i = 0; i < n; ++i) total += ns[i];
    // Long chunks of fp16 weights: 256-wide tiles (one MMA of N = 256 per K step; a third fewer operand bytes per
    // flop than 128-wide ones - these GEMMs are bound by the L2 -> shared-memory feed).  Measured on the q/k/v shape at
    // 2048 rows: 28.8 -> 26.5 us.
    const int box_n = (wq == 0 && M >= 1024 && total / 256 * (M / qmk_gemm::BM) >= qmk_tc::gemm_sm_count()) ? 256
                                                                                                           : qmk_tc::gemm_box_n(M, total);
    const CUtensorMap *maps[3];
    const void *raws[3] = {nullptr, nullptr, nullptr};
    for (int i = 0; i < n; ++i) { maps[i] = &wmap_for(l, js[i], box_n); raws[i] = wptr(l, js[i]); }
    return qmk_tc::launch_gemm_grouped(a, n, maps, cs, ns, M, K, box_n, w.status, env.timeout_ms, stream, &err, live, 0, wq,
                                       raws);
  };
  if ((rc = qmk_tc::ensure_gemm_attrs(&err)) != QMK_OK) return qmk_internal::report(rc, err);
  for (int c0 = 0; c0 < num_tokens; c0 += CHUNK) {
    const int T = (num_tokens - c0 < CHUNK) ? num_tokens - c0 : CHUNK;
    const int M = (T + qmk_gemm::BM - 1) / qmk_gemm::BM * qmk_gemm::BM;
    const int pos0 = start_position + c0;
    // The O and down projections have only 1024 output columns: with 128-wide tiles a long chunk gives 128 CTAs for
    // 148 SMs (296 slots with two CTAs per SM) and a K loop of 32 / 48 blocks.  K split in two doubles the CTAs and
    // halves the loop; the partial matrices are added by the residual + RMSNorm kernel that follows anyway.
    // Short chunks: four splits (M = 512: 32 tiles x 4 = 128 CTAs with K loops of 8 / 12 blocks; unsplit, the narrowest
    // tiles gave 128 CTAs with loops of 32 / 48 blocks of N = 32 MMAs and these two products were 41 % of the pass).
    const int od_splits = wq != 0 ? 1 : M >= 1024 ? 2 : 4;
    const size_t od_stride = od_splits > 1 ? static_cast<size_t>(M) * H : 0;
    auto gemm_od = [&](const CUtensorMap &a, int l, int j, float *c, int Mrows, int K, int live) {
      if (od_splits == 1) return gemm(a, l, j, c, Mrows, H, K, live);
      // 256-wide tiles, one CTA per SM with the whole ring: the main loops are bound by shared-memory traffic (TMA
      // writes + MMA operand reads), and a 256-wide tile moves a quarter fewer bytes per flop than a 128-wide one
      // (2048 tokens: 4.12 -> 4.07 ms per pass, same box); shorter chunks would leave SMs without a tile
      if (Mrows >= 2048) {
        qmk_tc::RingBudgetScope whole(0);
        return qmk_tc::launch_gemm_splitk(a, wmap_for(l, j, 256), c, Mrows, H, K, od_splits, w.status, env.timeout_ms, stream, &err,
                                          256, live, 0, wq, wptr(l, j));
      }
      return qmk_tc::launch_gemm_splitk(a, wmap_for(l, j, 128), c, Mrows, H, K, od_splits, w.status, env.timeout_ms, stream, &err, 128,
                                        live, 0, wq, wptr(l, j));
    };
    CUtensorMap map_kc, map_vc;   // the caches up to this chunk's last position, all layers
    memset(&map_kc, 0, sizeof(map_kc));
    memset(&map_vc, 0, sizeof(map_vc));
    if (env.attn_tc && !pk) {
      rc = qmk_tc::make_map_kv(&map_kc, k_cache, static_cast<uint64_t>(pos0 + T), static_cast<uint64_t>(max_seq_len),
                               static_cast<uint64_t>(num_layers) * NKV, &err);
      if (rc == QMK_OK)
        rc = qmk_tc::make_map_kv(&map_vc, v_cache, static_cast<uint64_t>(pos0 + T), static_cast<uint64_t>(max_seq_len),
                                 static_cast<uint64_t>(num_layers) * NKV, &err);
      if (rc != QMK_OK) break;
    }
    PF_CUDA(cudaMemcpyAsync(w.tokens, token_ids_host + c0, sizeof(int) * T, cudaMemcpyHostToDevice, stream));
    // Programmatic dependent launch for the GEMMs only: their set-up and first ring fill of WEIGHT tiles run under the
    // tail of the kernel before them (every kernel here lasts 2-6 us longer than its CTAs run; 2048 tokens 4.11 -> 3.81
    // ms).  The row kernels and the attention kernel launch plainly: with EVERY kernel of this chain launched as a
    // programmatic dependent, a decode launched after the prefill had returned produced run-to-run different logits
    // although every cache row compared bit-identical afterwards - unexplained; the attribute on the GEMMs alone never
    // showed it (128 prefill + decode cycles compared bit for bit, and the test that found it runs every time).
    qmk_tc::PdlScope pdl_scope(false);
    const bool pdl_gemm = env.pdl != 0;
    qmk_tc::RingBudgetScope ring_scope(PREFILL_RING_BYTES);   // two GEMM CTAs per SM: one's epilogue under the other's main loop
    {
      qmk_tc::PdlScope first(false);            // (follows a copy, not a kernel)
      PF_CUDA(qmk_tc::launch_kernel(embed_rows, dim3(T), dim3(256), 0, stream, w.tokens, embed_weight, wq, w.x));
    }
    // residual add (+ split-K partials) and RMSNorm: a warp per row for long chunks, a block per row for short ones
    auto norm_rows = [&](const float *add, const __half *g) {
      if (T >= 256 && od_splits <= 2)
        return qmk_tc::launch_kernel(add_rmsnorm_rows_wide, dim3((T + 7) / 8), dim3(256), 0, stream, w.x, add, od_splits, od_stride, g,
                                     w.xn, T);
      return qmk_tc::launch_kernel(add_rmsnorm_rows, dim3(T), dim3(256), 0, stream, w.x, add, od_splits, od_stride, g, w.xn);
    };
    for (int l = 0; l < num_layers; ++l) {
      const unsigned long long *r = rec.data() + static_cast<size_t>(l) * 12;
      __half *kc = pk ? nullptr : static_cast<__half *>(k_cache) + l * layer_stride;
      __half *vc = pk ? nullptr : static_cast<__half *>(v_cache) + l * layer_stride;
      PF_CUDA(norm_rows(l > 0 ? w.down : nullptr, reinterpret_cast<const __half *>(r[0])));
      {
        const int js[3] = {0, 1, 2};
        float *const cs[3] = {w.q, w.k, w.v};
        const int ns[3] = {QS, KVS, KVS};
        // fp16 q / k / v: every CTA of this launch reaches its epilogue at the same time, and the burst of stores set
        // its length (9.8 of 26 us at 2048 rows with fp32); the consumer below rounds to fp16 anyway
        qmk_tc::set_out_f16(true);
        {
          qmk_tc::PdlScope g(pdl_gemm);
          rc = gemm_group(w.map_xn, l, 3, js, cs, ns, M, H, T);
        }
        qmk_tc::set_out_f16(false);
        if (rc != QMK_OK) break;
      }
      // (Folding this kernel into the q/k/v GEMM's epilogue - one 128-wide N tile is one head - was built and measured
      // slower: 128 threads per CTA walking TMEM eight columns at a time lose to 2300 x 4 fully parallel CTAs.)
      PF_CUDA(qmk_tc::launch_kernel(qk_norm_rope_cache, dim3(T), dim3(256), 0, stream, w.q, w.k, w.v, 1,
                                    reinterpret_cast<const __half *>(r[4]), reinterpret_cast<const __half *>(r[5]), rope, cosv, sinv,
                                    w.qr, kc, vc, pos0, max_seq_len,
                                    pk ? reinterpret_cast<const int2 *>(w.packed + PK_ROWS_OFF) : nullptr,
                                    pk ? reinterpret_cast<const unsigned long long *>(w.packed + PK_PTRS_OFF) : nullptr,
                                    static_cast<size_t>(l) * layer_stride,
                                    env.attn_tc ? attn_scale * 1.4426950408889634f : 0.f));
      if (l == num_layers - 1) break;   // the cache is complete; nothing downstream of the last layer is kept
      if (env.attn_tc)
        PF_CUDA(qmk_tc::launch_kernel(qmk_attn::causal_attention_tc, dim3(pk ? pk_items : (T + qmk_attn::TQ - 1) / qmk_attn::TQ * NQ),
                                      dim3(qmk_attn::THREADS), qmk_attn::SMEM_BYTES, stream, w.map_qh, map_kc, map_vc, l * NKV, w.attn, T,
                                      pos0, attn_scale, w.status, static_cast<unsigned long long>(env.timeout_ms) * 1000000ull,
                                      pk ? reinterpret_cast<const int4 *>(w.packed + PK_ITEMS_OFF) : nullptr,
                                      pk ? reinterpret_cast<const CUtensorMap *>(w.packed + PK_MAPS_OFF) : nullptr));
      else
        PF_CUDA(qmk_tc::launch_kernel(causal_attention_mma, dim3((T + ATM_Q - 1) / ATM_Q, NKV), dim3(ATM_THREADS), ATM_SMEM_BYTES, stream,
                                      w.qr, kc, vc, w.attn, T, pos0, max_seq_len, attn_scale));
      {
        qmk_tc::PdlScope g(pdl_gemm);
        rc = gemm_od(w.map_attn, l, 3, w.o, M, QS, T);
      }
      if (rc != QMK_OK) break;
      PF_CUDA(norm_rows(w.o, reinterpret_cast<const __half *>(r[7])));
      {
        const int box_gu = qmk_tc::gemm_box_n_fused(M, I);
        // three of these CTAs per SM instead of two: their epilogue (two TMEM reads, SiLU, fp16 pack) is the long part
        qmk_tc::RingBudgetScope gu_scope(M >= 1024 ? GATE_UP_RING_BYTES : PREFILL_RING_BYTES);
        {
          qmk_tc::PdlScope g(pdl_gemm);
          rc = qmk_tc::launch_gemm_swiglu(w.map_xn, wmap_for(l, 4, box_gu), wmap_for(l, 5, box_gu), w.act, M, I, H, w.status,
                                          env.timeout_ms, stream, &err, box_gu, T, 0, wq, wptr(l, 4), wptr(l, 5));
        }
        if (rc != QMK_OK) break;
      }
      {
        qmk_tc::PdlScope g(pdl_gemm);
        rc = gemm_od(w.map_act, l, 6, w.down, M, I, T);
      }
      if (rc != QMK_OK) break;
    }
    if (rc != QMK_OK) break;
    PF_CUDA(cudaGetLastError());     // (the next chunk's token copy is stream-ordered behind this chunk's kernels)
  }
  if (rc != QMK_OK) return qmk_internal::report(rc, err);
  unsigned int host_status[4] = {0, 0, 0, 0};
  PF_CUDA(cudaMemcpyAsync(host_status, w.status, 16, cudaMemcpyDeviceToHost, stream));
  PF_CUDA(cudaStreamSynchronize(stream));
  if (host_status[0] != 0)
    return qmk_internal::report(static_cast<int>(host_status[0]) == 5 ? QMK_ERR_CUDA : static_cast<int>(host_status[0]),
                                host_status[0] == 5 ? "prefill: dynamic shared memory of the attention kernel is not 1024-byte aligned"
                                                    : "prefill: a bounded device wait ran out");
  return QMK_OK;
}
}  // namespace

extern "C" int qmk_prefill_chunked(const int *token_ids_host, int num_tokens, const void *embed_weight,
                                   const LDGLayerWeight *layer_weights, const void *cos_table, const void *sin_table,
                                   void *k_cache, void *v_cache, int num_layers, int start_position, int max_seq_len,
                                   float attn_scale, cudaStream_t stream) {
  return prefill_impl(token_ids_host, num_tokens, embed_weight, layer_weights, cos_table, sin_table, k_cache, v_cache, num_layers,
                      start_position, max_seq_len, attn_scale, stream, nullptr);
}

extern "C" int qmk_prefill_packed(const int *token_ids_host, int num_seqs, const int *seq_lens, const void *embed_weight,
                                  const LDGLayerWeight *layer_weights, const void *cos_table, const void *sin_table,
                                  void *const *k_caches, void *const *v_caches, int num_layers, int max_seq_len, float attn_scale,
                                  cudaStream_t stream) {
  if (num_seqs <= 0) return QMK_OK;
  if (!seq_lens) return qmk_internal::report(QMK_ERR_BAD_ARGUMENT, "packed prefill: null lengths");
  long total = 0;
  for (int s = 0; s < num_seqs && s < MAX_PACKED_SEQS; ++s) total += seq_lens[s] > 0 ? seq_lens[s] : 0;
  const PackedSeqs pk = {num_seqs, seq_lens, k_caches, v_caches};
  return prefill_impl(token_ids_host, static_cast<int>(total), embed_weight, layer_weights, cos_table, sin_table, nullptr, nullptr,
                      num_layers, 0, max_seq_len, attn_scale, stream, &pk);
}

// ----------------------------------------------------------------------------- batched decode on the GEMM path
namespace {
unsigned int __float_as_uint_host(float f) {
  unsigned int u;
  memcpy(&u, &f, 4);
  return u;
}

constexpr int MAX_BATCH = 128;      // one 128-row GEMM tile of sequences

constexpr int MAX_ATTN_SPLITS = 8;
int ensure_decode_workspace(Workspace &w, const void *lm_head, int vocab, int wq) {
  if (!w.positions) {
    PF_CUDA(cudaMalloc(&w.positions, sizeof(int) * MAX_BATCH));
    PF_CUDA(cudaMalloc(&w.start_positions, sizeof(int) * MAX_BATCH));
    PF_CUDA(cudaStreamCreateWithFlags(&w.gstream, cudaStreamNonBlocking));
    PF_CUDA(cudaEventCreateWithFlags(&w.ev_in, cudaEventDisableTiming));
    PF_CUDA(cudaEventCreateWithFlags(&w.ev_out, cudaEventDisableTiming));
    PF_CUDA(cudaMalloc(&w.k_ptrs, sizeof(void *) * MAX_BATCH));
    PF_CUDA(cudaMalloc(&w.v_ptrs, sizeof(void *) * MAX_BATCH));
    PF_CUDA(cudaMalloc(&w.log_ptrs, sizeof(void *) * MAX_BATCH));
    PF_CUDA(cudaMalloc(&w.kv_maps, sizeof(CUtensorMap) * 2 * MAX_BATCH));
    PF_CUDA(cudaMalloc(&w.split_part, sizeof(float) * MAX_BATCH * qmk_pf::NKV * MAX_ATTN_SPLITS * 2 * (qmk_pf::D + 2)));
    PF_CUDA(cudaMalloc(&w.split_count, sizeof(unsigned int) * MAX_BATCH * qmk_pf::NKV));
    PF_CUDA(cudaMemset(w.split_count, 0, sizeof(unsigned int) * MAX_BATCH * qmk_pf::NKV));
  }
  if (w.logits_vocab < vocab) {
    if (w.logits) cudaFree(w.logits);
    w.logits = nullptr;
    w.logits_vocab = 0;
    PF_CUDA(cudaMalloc(&w.logits, sizeof(float) * static_cast<size_t>(MAX_BATCH) * vocab));
    if (w.amax_val) cudaFree(w.amax_val);
    if (w.amax_idx) cudaFree(w.amax_idx);
    w.amax_val = nullptr;
    w.amax_idx = nullptr;
    PF_CUDA(cudaMalloc(&w.amax_val, sizeof(float) * static_cast<size_t>(MAX_BATCH) * (vocab / 128)));
    PF_CUDA(cudaMalloc(&w.amax_idx, sizeof(int) * static_cast<size_t>(MAX_BATCH) * (vocab / 128)));
    w.logits_vocab = vocab;
    w.lm_ptr = nullptr;
  }
  if (w.lm_ptr != lm_head || w.lm_wq != wq) {
    std::string err;
    const int rc = qmk_tc::make_map_b(&w.map_lm, lm_head, vocab, qmk_pf::H, 128, wq, &err);
    if (rc != QMK_OK) return qmk_internal::report(rc, err);
    w.lm_ptr = lm_head;
    w.lm_wq = wq;
    ++w.graph_epoch;
  }
  return QMK_OK;
}
}  // namespace

extern "C" int qmk_decode_batched(int num_sequences, const int *first_token_ids, const int *start_positions, int num_steps,
                                  const void *embed_weight, const LDGLayerWeight *layer_weights,
                                  const void *final_norm_weight, const void *lm_head_weight, const void *cos_table,
                                  const void *sin_table, void *const *k_caches, void *const *v_caches,
                                  int *const *output_logs, int num_layers, int max_seq_len, float attn_scale,
                                  cudaStream_t stream) {
  using namespace qmk_pf;
  if (num_steps <= 0) return QMK_OK;
  qmk_internal::PrefillEnv env;
  int rc = qmk_internal::prefill_env(max_seq_len, stream, &env);
  if (rc != QMK_OK) return rc;
  if (num_sequences < 1 || num_sequences > MAX_BATCH)
    return qmk_internal::report(QMK_ERR_BAD_ARGUMENT, "qmk_decode_batched: num_sequences must be in [1, 128]");
  if (!first_token_ids || !start_positions || !k_caches || !v_caches || !output_logs || !embed_weight || !layer_weights ||
      !final_norm_weight || !lm_head_weight)
    return qmk_internal::report(QMK_ERR_BAD_ARGUMENT, "qmk_decode_batched: null pointer argument");
  const int wq = env.wfmt;   // packed FP8 / NVFP4 matrices stay packed in HBM and are expanded inside the GEMMs
  if (env.vocab % 128 != 0)
    return qmk_internal::report(QMK_ERR_BAD_ARGUMENT, "qmk_decode_batched needs a vocabulary that is a multiple of 128");
  if (num_layers < 1 || num_layers > MAX_LAYERS)
    return qmk_internal::report(QMK_ERR_BAD_ARGUMENT, "num_layers must be in [1, 48]");
  if (env.rope_from_table && (!cos_table || !sin_table))
    return qmk_internal::report(QMK_ERR_BAD_ARGUMENT, "rope_from_table needs cos/sin tables");
  const int B = num_sequences;
  for (int b = 0; b < B; ++b) {
    if (!k_caches[b] || !v_caches[b] || !output_logs[b])
      return qmk_internal::report(QMK_ERR_BAD_ARGUMENT, "qmk_decode_batched: null cache or log pointer");
    if (start_positions[b] < 0 || start_positions[b] + num_steps > max_seq_len)
      return qmk_internal::report(QMK_ERR_POSITION, "start_position + steps exceeds max_seq_len");
    if (first_token_ids[b] < 0 || first_token_ids[b] >= env.vocab)
      return qmk_internal::report(QMK_ERR_BAD_TOKEN, "first token outside [0, vocab)");
    for (int a = 0; a < b; ++a)
      if (k_caches[a] == k_caches[b] || v_caches[a] == v_caches[b] || output_logs[a] == output_logs[b])
        return qmk_internal::report(QMK_ERR_BAD_ARGUMENT, "qmk_decode_batched: two sequences share a cache or an output log");
  }
  int dev = 0;
  PF_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 16) return qmk_internal::report(QMK_ERR_CUDA, "device index out of range");
  std::lock_guard<std::mutex> lock(g_ws_decode_mu);
  Workspace &w = g_ws_decode[dev];
  rc = ensure_workspace(w, 512);   // room for the split-K partial matrices (4 x 128 rows)
  if (rc == QMK_OK) rc = ensure_weight_maps(w, layer_weights, num_layers, wq, stream);
  if (rc == QMK_OK) rc = ensure_decode_workspace(w, lm_head_weight, env.vocab, wq);
  if (rc != QMK_OK) return rc;
  std::vector<unsigned long long> rec(w.table, w.table + static_cast<size_t>(num_layers) * 12);
  const float *rope = env.rope_from_table ? nullptr : env.rope;
  const __half *cosv = static_cast<const __half *>(cos_table), *sinv = static_cast<const __half *>(sin_table);
  const size_t layer_stride = static_cast<size_t>(NKV) * max_seq_len * D;
  PF_CUDA(cudaMemsetAsync(w.status, 0, 16, stream));
  // (the attention kernels leave their arrival counters at zero; a call that failed half-way may not have)
  PF_CUDA(cudaMemsetAsync(w.split_count, 0, sizeof(unsigned int) * MAX_BATCH * NKV, stream));
  PF_CUDA(cudaMemcpyAsync(w.tokens, first_token_ids, sizeof(int) * B, cudaMemcpyHostToDevice, stream));
  PF_CUDA(cudaMemcpyAsync(w.positions, start_positions, sizeof(int) * B, cudaMemcpyHostToDevice, stream));
  PF_CUDA(cudaMemcpyAsync(w.start_positions, start_positions, sizeof(int) * B, cudaMemcpyHostToDevice, stream));
  PF_CUDA(cudaMemcpyAsync(w.k_ptrs, k_caches, sizeof(void *) * B, cudaMemcpyHostToDevice, stream));
  PF_CUDA(cudaMemcpyAsync(w.v_ptrs, v_caches, sizeof(void *) * B, cudaMemcpyHostToDevice, stream));
  PF_CUDA(cudaMemcpyAsync(w.log_ptrs, output_logs, sizeof(void *) * B, cudaMemcpyHostToDevice, stream));
  std::string err;
  std::vector<CUtensorMap> host_maps;
  if (env.attn_mma) {   // per-sequence descriptors of the whole [layer][kv head][position] caches, boxes of 16 rows x 64 dims
    host_maps.resize(2 * static_cast<size_t>(B));
    const uint64_t cache_rows = static_cast<uint64_t>(num_layers) * NKV * static_cast<uint64_t>(max_seq_len);
    for (int b = 0; b < B && rc == QMK_OK; ++b) {
      rc = qmk_tc::make_map_f16(&host_maps[2 * b], k_caches[b], cache_rows, D, 16, &err);
      if (rc == QMK_OK) rc = qmk_tc::make_map_f16(&host_maps[2 * b + 1], v_caches[b], cache_rows, D, 16, &err);
    }
    if (rc != QMK_OK) return qmk_internal::report(rc, err);
    PF_CUDA(cudaMemcpyAsync(w.kv_maps, host_maps.data(), sizeof(CUtensorMap) * host_maps.size(), cudaMemcpyHostToDevice, stream));
    PF_CUDA(cudaStreamSynchronize(stream));   // (the pageable host vector must outlive the copy)
  }
  if ((rc = qmk_tc::ensure_gemm_attrs(&err)) != QMK_OK) return qmk_internal::report(rc, err);
  (void)qmk_tc::gemm_box_n(128, 128);   // caches the SM count before any capture
  {
    const int rows = (B + 7) / 8 * 8;
    if (w.a_rows != rows) {
      // boxes of just the live rows: the rest of the 128-row tile in shared memory is never written (nor needed)
      rc = qmk_tc::make_map_f16(&w.map_xn_b, w.xn, rows, H, rows, &err);
      if (rc == QMK_OK) rc = qmk_tc::make_map_f16(&w.map_attn_b, w.attn, rows, QS, rows, &err);
      if (rc == QMK_OK) rc = qmk_tc::make_map_f16(&w.map_act_b, w.act, rows, I, rows, &err);
      if (rc != QMK_OK) return qmk_internal::report(rc, err);
      w.a_rows = rows;   // (graphs captured earlier keep their own copies of the maps they were captured with)
    }
  }
  const int M = qmk_gemm::BM;   // one tile of rows; rows >= B are computed and ignored
  // One decode step for all sequences, enqueued on `s`.  Everything that changes from step to step (tokens,
  // positions) or from call to call (cache and log pointers) lives in device arrays at fixed addresses, so the
  // same sequence of launches - and a graph captured from it - serves every step.
  // The O (K = 2048) and down (K = 3072) projections have only 1024 output columns: K is split four ways and the
  // following RMSNorm adds the partial matrices.
  // N tiles of 32 columns: 128 (q/k/v), 96 (gate/up) and, with K split four ways, 128 CTAs (O, down) per GEMM
  // instead of 64 / 48 / 32-48 with 64-wide tiles; a decode step is bound by how many SMs pull weights at once.
  // The epilogues store only the B live rows of the 128-row tile (the LM head alone would otherwise write
  // 78 MB of padding logits per step).  Measured: 6.5 k -> 7.5 k tok/s at B = 16, 18.3 k -> 21.0 k at B = 64.
  constexpr int TILE_N = 32, O_SPLITS = 4, DOWN_SPLITS = 4;
  const int live = B, a_box = w.a_rows;
  // Few sequences: split every sequence's cache rows over several CTAs so that the attention fills the device
  // (two CTAs fit on an SM): 8 B CTAs otherwise, each streaming a whole sequence through one ring.
  int attn_splits = (2 * qmk_tc::g_sms[dev]) / (B * NKV);   // (gemm_box_n above cached the SM count of this device)
  attn_splits = attn_splits < 1 ? 1 : attn_splits > MAX_ATTN_SPLITS ? MAX_ATTN_SPLITS : attn_splits;
  const size_t PART = static_cast<size_t>(M) * H;
  auto enqueue_step = [&](cudaStream_t s) -> int {
    int r2 = QMK_OK;
    qmk_tc::PdlScope pdl_scope(env.pdl != 0);   // every launch below may start behind its predecessor's tail
    {
      qmk_tc::PdlScope first(false);            // (the first kernel of a step has no predecessor inside the step)
      PF_CUDA(qmk_tc::launch_kernel(embed_rows, dim3(B), dim3(256), 0, s, w.tokens, embed_weight, wq, w.x));
    }
    for (int l = 0; l < num_layers; ++l) {
      const unsigned long long *r = rec.data() + static_cast<size_t>(l) * 12;
      const size_t layer_off = l * layer_stride;
      auto wm = [&](int j) -> const CUtensorMap & { return w.wmap32[l][j]; };
      static const int rec_slot[7] = {1, 2, 3, 6, 8, 9, 10};   // q, k, v, o, gate, up, down inside a layer record
      auto wp = [&](int j) { return reinterpret_cast<const void *>(r[rec_slot[j]]); };
      PF_CUDA(qmk_tc::launch_kernel(add_rmsnorm_rows, dim3(B), dim3(256), 0, s, w.x, l > 0 ? w.down : nullptr, DOWN_SPLITS, PART,
                                    reinterpret_cast<const __half *>(r[0]), w.xn));
      {
        const CUtensorMap *maps[3] = {&wm(0), &wm(1), &wm(2)};
        float *const cs[3] = {w.q, w.k, w.v};
        const int ns[3] = {QS, KVS, KVS};
        const void *raws[3] = {wp(0), wp(1), wp(2)};
        if ((r2 = qmk_tc::launch_gemm_grouped(w.map_xn_b, 3, maps, cs, ns, M, H, TILE_N, w.status, env.timeout_ms, s, &err,
                                              live, a_box, wq, raws)) != QMK_OK)
          return r2;
      }
      if (env.attn_mma)
        PF_CUDA(qmk_tc::launch_kernel(decode_attention_mma, dim3(B, NKV, attn_splits), dim3((DAM_WARPS + 1) * 32), DAM_SMEM_BYTES, s,
                                      w.q, w.k, w.v, reinterpret_cast<const __half *>(r[4]), reinterpret_cast<const __half *>(r[5]),
                                      rope, cosv, sinv, w.k_ptrs, w.v_ptrs, layer_off, w.positions, w.attn, max_seq_len, attn_scale,
                                      w.status, static_cast<unsigned long long>(env.timeout_ms) * 1000000ull, w.split_part,
                                      w.split_count, w.kv_maps, l * NKV * max_seq_len));
      else
        PF_CUDA(qmk_tc::launch_kernel(decode_attention_ring, dim3(B, NKV, attn_splits), dim3((DAR_WARPS + 1) * 32), DAR_SMEM_BYTES, s,
                                      w.q, w.k, w.v, reinterpret_cast<const __half *>(r[4]), reinterpret_cast<const __half *>(r[5]),
                                      rope, cosv, sinv, w.k_ptrs, w.v_ptrs, layer_off, w.positions, w.attn, max_seq_len, attn_scale,
                                      w.status, static_cast<unsigned long long>(env.timeout_ms) * 1000000ull, w.split_part,
                                      w.split_count));
      if ((r2 = qmk_tc::launch_gemm_splitk(w.map_attn_b, wm(3), w.o, M, H, QS, O_SPLITS, w.status, env.timeout_ms, s, &err,
                                           TILE_N, live, a_box, wq, wp(3))) != QMK_OK)
        return r2;
      PF_CUDA(qmk_tc::launch_kernel(add_rmsnorm_rows, dim3(B), dim3(256), 0, s, w.x, w.o, O_SPLITS, PART,
                                    reinterpret_cast<const __half *>(r[7]), w.xn));
      if ((r2 = qmk_tc::launch_gemm_swiglu(w.map_xn_b, wm(4), wm(5), w.act, M, I, H, w.status, env.timeout_ms, s, &err, TILE_N,
                                           live, a_box, wq, wp(4), wp(5))) != QMK_OK)
        return r2;
      if ((r2 = qmk_tc::launch_gemm_splitk(w.map_act_b, wm(6), w.down, M, H, I, DOWN_SPLITS, w.status, env.timeout_ms, s, &err,
                                           TILE_N, live, a_box, wq, wp(6))) != QMK_OK)
        return r2;
    }
    PF_CUDA(qmk_tc::launch_kernel(add_rmsnorm_rows, dim3(B), dim3(256), 0, s, w.x, w.down, DOWN_SPLITS, PART,
                                  static_cast<const __half *>(final_norm_weight), w.xn));
    // Without a logits dump the LM head's epilogue picks the largest logit of each 128-column tile itself and the
    // rows of logits (B x 608 KB per step) are never written
    const bool fused_pick = env.logits_out == nullptr;
    if (fused_pick) qmk_tc::set_argmax_target(w.amax_val, w.amax_idx);
    qmk_tc::RingBudgetScope lm_scope(PREFILL_RING_BYTES);   // 1187 tiles: two CTAs per SM, four waves instead of eight
    r2 = qmk_tc::launch_gemm(w.map_xn_b, w.map_lm, w.logits, M, env.vocab, H, 128, w.status, env.timeout_ms, s, &err, live, a_box,
                             wq, lm_head_weight);
    qmk_tc::set_argmax_target(nullptr, nullptr);
    if (r2 != QMK_OK) return r2;
    if (fused_pick)
      PF_CUDA(qmk_tc::launch_kernel(argmax_pairs, dim3(B), dim3(256), 0, s, w.amax_val, w.amax_idx, env.vocab / 128, w.tokens,
                                    w.log_ptrs, w.start_positions, w.positions));
    else
      PF_CUDA(qmk_tc::launch_kernel(argmax_rows, dim3(B), dim3(1024), 0, s, w.logits, env.vocab, w.tokens, w.log_ptrs,
                                    w.start_positions, w.positions));
    return QMK_OK;
  };

  if (env.logits_out) {
    // debug dump [sequence][step][vocab]: plain launches with a copy after every step
    for (int step = 0; step < num_steps && rc == QMK_OK; ++step) {
      rc = enqueue_step(stream);
      if (rc != QMK_OK) break;
      PF_CUDA(cudaGetLastError());
      for (int b = 0; b < B; ++b)
        PF_CUDA(cudaMemcpyAsync(env.logits_out + (static_cast<size_t>(b) * num_steps + step) * env.vocab,
                                w.logits + static_cast<size_t>(b) * env.vocab, sizeof(float) * env.vocab,
                                cudaMemcpyDeviceToDevice, stream));
    }
  } else {
    // One step costs about 400 launches: capture it once as a CUDA graph (kept while nothing it bakes in
    // changes) and replay it num_steps times.
    const unsigned long long key[12] = {
        w.graph_epoch, static_cast<unsigned long long>(B) | (static_cast<unsigned long long>(wq) << 32), static_cast<unsigned long long>(num_layers),
        static_cast<unsigned long long>(max_seq_len), static_cast<unsigned long long>(env.vocab),
        static_cast<unsigned long long>(__float_as_uint_host(attn_scale)), reinterpret_cast<unsigned long long>(embed_weight),
        reinterpret_cast<unsigned long long>(final_norm_weight), reinterpret_cast<unsigned long long>(lm_head_weight),
        reinterpret_cast<unsigned long long>(rope), reinterpret_cast<unsigned long long>(cos_table),
        reinterpret_cast<unsigned long long>(sin_table) ^ (static_cast<unsigned long long>(env.timeout_ms) << 48) ^
            (static_cast<unsigned long long>(env.pdl != 0) << 63) ^ (static_cast<unsigned long long>(env.attn_mma != 0) << 62)};
    if (memcmp(key, w.step_key[B], sizeof(key)) != 0) {
      if (w.step_graph[B]) { cudaGraphExecDestroy(w.step_graph[B]); w.step_graph[B] = nullptr; }
      w.step_key[B][0] = 0;
      cudaGraph_t graph = nullptr;
      PF_CUDA(cudaStreamBeginCapture(w.gstream, cudaStreamCaptureModeThreadLocal));
      rc = enqueue_step(w.gstream);
      cudaError_t ce = cudaStreamEndCapture(w.gstream, &graph);   // always end the capture, also after an error
      if (rc == QMK_OK && ce != cudaSuccess) { rc = QMK_ERR_CUDA; err = std::string("graph capture: ") + cudaGetErrorString(ce); }
      if (rc == QMK_OK) {
        ce = cudaGraphInstantiate(&w.step_graph[B], graph, 0);
        if (ce != cudaSuccess) { rc = QMK_ERR_CUDA; err = std::string("cudaGraphInstantiate: ") + cudaGetErrorString(ce); }
      }
      if (graph) cudaGraphDestroy(graph);
      if (rc == QMK_OK) memcpy(w.step_key[B], key, sizeof(key));
    }
    if (rc == QMK_OK) {
      PF_CUDA(cudaEventRecord(w.ev_in, stream));          // the graph stream starts after the caller's stream
      PF_CUDA(cudaStreamWaitEvent(w.gstream, w.ev_in, 0));
      for (int step = 0; step < num_steps; ++step) PF_CUDA(cudaGraphLaunch(w.step_graph[B], w.gstream));
      PF_CUDA(cudaEventRecord(w.ev_out, w.gstream));
      PF_CUDA(cudaStreamWaitEvent(stream, w.ev_out, 0));  // ... and the caller's stream continues after it
    }
  }
  if (rc != QMK_OK) return qmk_internal::report(rc, err);
  unsigned int host_status[4] = {0, 0, 0, 0};
  PF_CUDA(cudaMemcpyAsync(host_status, w.status, 16, cudaMemcpyDeviceToHost, stream));
  PF_CUDA(cudaStreamSynchronize(stream));
  if (host_status[0] != 0)
    return qmk_internal::report(static_cast<int>(host_status[0]), "decode_batched: a bounded device wait ran out");
  return QMK_OK;
}

// Bounded-wait self test of the GEMM kernel: one 128 x 128 tile whose loads are never issued.  The MMA thread's
// wait on the first stage runs out after budget_us, every role leaves its loop, TMEM is freed and the kernel
// returns status 4 with the context intact.
extern "C" int qmk_selftest_gemm_wait_timeout(int budget_us) {
  std::string err;
  if (budget_us < 1 || budget_us > 1000000) return qmk_internal::report(QMK_ERR_BAD_ARGUMENT, "budget_us must be in [1, 1e6]");
  int rc = qmk_tc::ensure_gemm_attrs(&err);
  if (rc != QMK_OK) return qmk_internal::report(rc, err);
  __half *ab = nullptr;
  float *c = nullptr;
  unsigned int *status = nullptr;
  PF_CUDA(cudaMalloc(&ab, sizeof(__half) * 128 * 64));
  PF_CUDA(cudaMalloc(&c, sizeof(float) * 128 * 128));
  PF_CUDA(cudaMalloc(&status, 16));
  PF_CUDA(cudaMemset(ab, 0, sizeof(__half) * 128 * 64));
  PF_CUDA(cudaMemset(status, 0, 16));
  CUtensorMap m;
  rc = qmk_tc::make_map_f16(&m, ab, 128, 64, 128, &err);
  if (rc == QMK_OK) {
    qmk_gemm::Groups gr;
    gr.C[0] = c; gr.C[1] = nullptr; gr.C[2] = nullptr;
    gr.N[0] = 128; gr.N[1] = 0; gr.N[2] = 0;
    gr.kblocks_per_split = 0;
    gr.split_stride = 0;
    gr.a_box_bytes = 0;
    for (int g = 0; g < qmk_gemm::MAX_GROUPS; ++g) gr.braw[g] = nullptr;
    gr.raw_pitch = gr.raw_bs_off = gr.raw_scale_off = 0;
    gr.amax_val = nullptr;
    gr.out_f16 = 0;
  gr.out_f16 = 0;
    gr.amax_idx = nullptr;
    const size_t smem = qmk_tc::selftest_ring(&gr);
    qmk_gemm::gemm_f16_tn_kernel<128><<<dim3(1, 1), qmk_gemm::THREADS, smem>>>(
        m, m, m, m, gr, 128, 64, status, static_cast<unsigned long long>(budget_us) * 1000ull, 1);
    unsigned int host[4] = {0, 0, 0, 0};
    cudaError_t e = cudaMemcpy(host, status, 16, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) { rc = QMK_ERR_CUDA; err = std::string("gemm self test: ") + cudaGetErrorString(e); }
    else rc = static_cast<int>(host[0]);
  }
  cudaFree(ab);
  cudaFree(c);
  cudaFree(status);
  if (rc != QMK_OK && rc != QMK_ERR_WAIT_TIMEOUT) return qmk_internal::report(rc, err);
  return rc;
}

extern "C" int qmk_gemm_f16_tn(const void *a, const void *b, float *c, int m, int n, int k, cudaStream_t stream) {
  std::string err;
  CUtensorMap ma, mb;
  unsigned int *status = nullptr;
  int rc = qmk_tc::make_map_f16(&ma, a, m, k, qmk_gemm::BM, &err);
  const int box_n = (m > 0 && n > 0 && m % 128 == 0 && n % 128 == 0) ? qmk_tc::gemm_box_n(m, n) : 128;
  if (rc == QMK_OK) rc = qmk_tc::make_map_f16(&mb, b, n, k, box_n, &err);
  if (rc == QMK_OK && cudaMalloc(&status, 16) != cudaSuccess) { rc = QMK_ERR_CUDA; err = "cudaMalloc failed"; }
  if (rc == QMK_OK) {
    cudaMemsetAsync(status, 0, 16, stream);
    rc = qmk_tc::launch_gemm(ma, mb, c, m, n, k, box_n, status, 2000, stream, &err);
  }
  if (rc == QMK_OK) {
    unsigned int host[4] = {0, 0, 0, 0};
    cudaError_t e = cudaMemcpyAsync(host, status, 16, cudaMemcpyDeviceToHost, stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) { rc = QMK_ERR_CUDA; err = std::string("gemm: ") + cudaGetErrorString(e); }
    else if (host[0] != 0) { rc = static_cast<int>(host[0]); err = "gemm: a bounded device wait ran out"; }
  }
  if (status) cudaFree(status);
  if (rc != QMK_OK) fprintf(stderr, "[qwen_megakernel] error %d: %s\n", rc, err.c_str());
  return rc;
}

// The same GEMM with B in a packed weight format (1: FP8-E4M3 rows, 2: NVFP4 rows).  `mode` 0: C fp32 [m x n];
// mode 1: split-K in four parts, C holds the four partial matrices; mode 2: `b` is a gate matrix and `b2` an up
// matrix, C receives fp16 silu(A gate^T) * (A up^T) - the three forms the decode step uses.
extern "C" int qmk_gemm_packed_tn(const void *a, const void *b, const void *b2, void *c, int m, int n, int k, int weight_format,
                                  int mode, int box_n, cudaStream_t stream) {
  std::string err;
  CUtensorMap ma, mb, mb2;
  unsigned int *status = nullptr;
  if (weight_format < 1 || weight_format > 2 || mode < 0 || mode > 2 || m <= 0 || n <= 0 || m % 128 || n % 128 ||
      (mode == 2 && !b2) || !a || !b || !c) {
    fprintf(stderr, "[qwen_megakernel] error %d: qmk_gemm_packed_tn: bad argument\n", QMK_ERR_BAD_ARGUMENT);
    return QMK_ERR_BAD_ARGUMENT;
  }
  if (box_n <= 0) box_n = mode == 2 ? qmk_tc::gemm_box_n_fused(m, n) : mode == 1 ? 32 : qmk_tc::gemm_box_n(m, n);
  int rc = qmk_tc::make_map_f16(&ma, a, m, k, qmk_gemm::BM, &err);
  if (rc == QMK_OK) rc = qmk_tc::make_map_packed(&mb, b, n, k, box_n, weight_format, &err);
  if (rc == QMK_OK && mode == 2) rc = qmk_tc::make_map_packed(&mb2, b2, n, k, box_n, weight_format, &err);
  if (rc == QMK_OK && cudaMalloc(&status, 16) != cudaSuccess) { rc = QMK_ERR_CUDA; err = "cudaMalloc failed"; }
  if (rc == QMK_OK) {
    cudaMemsetAsync(status, 0, 16, stream);
    if (mode == 0)
      rc = qmk_tc::launch_gemm(ma, mb, static_cast<float *>(c), m, n, k, box_n, status, 2000, stream, &err, 0, 0, weight_format, b);
    else if (mode == 1)
      rc = qmk_tc::launch_gemm_splitk(ma, mb, static_cast<float *>(c), m, n, k, 4, status, 2000, stream, &err, box_n, 0, 0,
                                      weight_format, b);
    else
      rc = qmk_tc::launch_gemm_swiglu(ma, mb, mb2, static_cast<__half *>(c), m, n, k, status, 2000, stream, &err, box_n, 0, 0,
                                      weight_format, b, b2);
  }
  if (rc == QMK_OK) {
    unsigned int host[4] = {0, 0, 0, 0};
    cudaError_t e = cudaMemcpyAsync(host, status, 16, cudaMemcpyDeviceToHost, stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) { rc = QMK_ERR_CUDA; err = std::string("gemm: ") + cudaGetErrorString(e); }
    else if (host[0] != 0) { rc = static_cast<int>(host[0]); err = "gemm: a bounded device wait ran out"; }
  }
  if (status) cudaFree(status);
  if (rc != QMK_OK) fprintf(stderr, "[qwen_megakernel] error %d: %s\n", rc, err.c_str());
  return rc;
}
