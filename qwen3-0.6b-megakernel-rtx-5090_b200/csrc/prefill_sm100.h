// Internal interface of the tensor-core side (prefill_sm100.cu).
#ifndef QMK_PREFILL_SM100_H_
#define QMK_PREFILL_SM100_H_

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string>

namespace qmk_tc {
// `box_n`: rows per box the B maps were made with (= the N tile: 32, 64 or 128).  `live_rows` (0 = all M): rows of
// the output the epilogue stores; a decode step of B sequences pads its rows to one 128-row tile and needs only
// the first B.  `a_box_rows` (0 = 128): rows per box of the A map when it is shorter than the tile.
int make_map_f16(CUtensorMap *map, const void *ptr, uint64_t rows, uint64_t cols, uint32_t box_rows, std::string *err);
int gemm_box_n(int M, int N);
int gemm_box_n_fused(int M, int N);   // for launch_gemm_swiglu (N = columns of the gate matrix)
int ensure_gemm_attrs(std::string *err);
int launch_gemm_splitk(const CUtensorMap &map_a, const CUtensorMap &map_b, float *C, int M, int N, int K, int splits,
                       unsigned int *status, int timeout_ms, cudaStream_t stream, std::string *err, int box_n = 64,
                       int live_rows = 0, int a_box_rows = 0);
int launch_gemm_swiglu(const CUtensorMap &map_a, const CUtensorMap &map_gate, const CUtensorMap &map_up, __half *act, int M,
                       int N, int K, unsigned int *status, int timeout_ms, cudaStream_t stream, std::string *err,
                       int box_n = 64, int live_rows = 0, int a_box_rows = 0);
int launch_gemm_grouped(const CUtensorMap &map_a, int ngroups, const CUtensorMap *const *maps_b, float *const *Cs,
                        const int *Ns, int M, int K, int box_n, unsigned int *status, int timeout_ms, cudaStream_t stream,
                        std::string *err, int live_rows = 0, int a_box_rows = 0);
int launch_gemm(const CUtensorMap &map_a, const CUtensorMap &map_b, float *C, int M, int N, int K, int box_n,
                unsigned int *status, int timeout_ms, cudaStream_t stream, std::string *err, int live_rows = 0, int a_box_rows = 0);
}  // namespace qmk_tc

#endif  // QMK_PREFILL_SM100_H_
