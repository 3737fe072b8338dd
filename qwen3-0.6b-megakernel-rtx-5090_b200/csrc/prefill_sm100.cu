// Tensor-core side of the library: the tcgen05 GEMM and (built on it) the chunked prompt prefill.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>
#include <mutex>
#include <string>

#include "../../include/qwen_megakernel.h"
#include "gemm_tcgen05.cuh"
#include "prefill_sm100.h"

namespace qmk_tc {

namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

std::mutex g_mu;
EncodeTiledFn g_encode = nullptr;
bool g_attr_set[16] = {};

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

// C[M x N] fp32 = A[M x K] * B[N x K]^T.  M, N multiples of 128; K a multiple of 64.
int launch_gemm(const CUtensorMap &map_a, const CUtensorMap &map_b, float *C, int M, int N, int K, unsigned int *status,
                int timeout_ms, cudaStream_t stream, std::string *err) {
  if (M <= 0 || N <= 0 || K <= 0 || M % qmk_gemm::BM || N % qmk_gemm::BN || K % qmk_gemm::BK) {
    *err = "gemm: M and N must be multiples of 128 and K a multiple of 64";
    return QMK_ERR_BAD_ARGUMENT;
  }
  int dev = 0;
  cudaGetDevice(&dev);
  {
    std::lock_guard<std::mutex> lock(g_mu);
    if (dev >= 0 && dev < 16 && !g_attr_set[dev]) {
      cudaError_t e = cudaFuncSetAttribute(qmk_gemm::gemm_f16_tn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           static_cast<int>(qmk_gemm::SMEM_BYTES));
      if (e != cudaSuccess) { *err = std::string("cudaFuncSetAttribute: ") + cudaGetErrorString(e); return QMK_ERR_CUDA; }
      g_attr_set[dev] = true;
    }
  }
  dim3 grid(N / qmk_gemm::BN, M / qmk_gemm::BM);
  qmk_gemm::gemm_f16_tn_kernel<<<grid, qmk_gemm::THREADS, qmk_gemm::SMEM_BYTES, stream>>>(
      map_a, map_b, C, M, N, K, status, static_cast<unsigned long long>(timeout_ms) * 1000000ull);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { *err = std::string("gemm launch: ") + cudaGetErrorString(e); return QMK_ERR_CUDA; }
  return QMK_OK;
}

}  // namespace qmk_tc

extern "C" int qmk_gemm_f16_tn(const void *a, const void *b, float *c, int m, int n, int k, cudaStream_t stream) {
  std::string err;
  CUtensorMap ma, mb;
  unsigned int *status = nullptr;
  int rc = qmk_tc::make_map_f16(&ma, a, m, k, qmk_gemm::BM, &err);
  if (rc == QMK_OK) rc = qmk_tc::make_map_f16(&mb, b, n, k, qmk_gemm::BN, &err);
  if (rc == QMK_OK && cudaMalloc(&status, 16) != cudaSuccess) { rc = QMK_ERR_CUDA; err = "cudaMalloc failed"; }
  if (rc == QMK_OK) {
    cudaMemsetAsync(status, 0, 16, stream);
    rc = qmk_tc::launch_gemm(ma, mb, c, m, n, k, status, 2000, stream, &err);
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
