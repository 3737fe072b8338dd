// Internal interface of the tensor-core side (prefill_sm100.cu).
#ifndef QMK_PREFILL_SM100_H_
#define QMK_PREFILL_SM100_H_

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string>

namespace qmk_tc {
// While one is alive on a thread, launch_kernel() on that thread adds the programmatic-stream-serialisation attribute.
class PdlScope {
 public:
  explicit PdlScope(bool on);
  ~PdlScope();
 private:
  bool prev_;
};
bool pdl_active();
}  // namespace qmk_tc
namespace qmk_gemm { struct Groups; }
namespace qmk_tc {
void set_out_f16(bool on);                     // calling thread: the next grouped GEMM stores fp16 matrices
void set_argmax_target(float *val, int *idx);   // calling thread: the next single-matrix GEMM picks per tile instead of storing
// While one is alive on a thread, GEMM launches of that thread size their rings to `bytes` of shared memory (0 = full depth).
class RingBudgetScope {
 public:
  explicit RingBudgetScope(unsigned int bytes);
  ~RingBudgetScope();
 private:
  unsigned int prev_;
};
size_t selftest_ring(qmk_gemm::Groups *gr);   // ring geometry of the bounded-wait self test's one-tile launch
template <typename... KArgs, typename... Args>
cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args &&...args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_active() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// `box_n`: rows per box the B maps were made with (= the N tile: 32, 64 or 128).  `live_rows` (0 = all M): rows of
// the output the epilogue stores; a decode step of B sequences pads its rows to one 128-row tile and needs only
// the first B.  `a_box_rows` (0 = 128): rows per box of the A map when it is shorter than the tile.
// `wq`: weight format of B - 0 fp16 (maps from make_map_f16), 1 FP8-E4M3 rows, 2 NVFP4 rows (maps from make_map_packed;
// the launch also needs the matrices' base pointers, `raw...`, for the scales inside the rows).
struct PackedRow { uint32_t data_bytes, bs_off, scale_off, pitch; };
PackedRow packed_row(int wq, int K);
int make_map_packed(CUtensorMap *map, const void *ptr, uint64_t rows, int K, uint32_t box_rows, int wq, std::string *err);
int make_map_b(CUtensorMap *map, const void *ptr, uint64_t rows, int K, uint32_t box_rows, int wq, std::string *err);
int make_map_kv(CUtensorMap *map, const void *cache, uint64_t rows, uint64_t max_seq_len, uint64_t heads, std::string *err);
int make_map_f16(CUtensorMap *map, const void *ptr, uint64_t rows, uint64_t cols, uint32_t box_rows, std::string *err);
int gemm_sm_count();
int gemm_box_n(int M, int N);
int gemm_box_n_fused(int M, int N);   // for launch_gemm_swiglu (N = columns of the gate matrix)
int ensure_gemm_attrs(std::string *err);
int launch_gemm_splitk(const CUtensorMap &map_a, const CUtensorMap &map_b, float *C, int M, int N, int K, int splits,
                       unsigned int *status, int timeout_ms, cudaStream_t stream, std::string *err, int box_n = 64,
                       int live_rows = 0, int a_box_rows = 0, int wq = 0, const void *raw = nullptr);
int launch_gemm_swiglu(const CUtensorMap &map_a, const CUtensorMap &map_gate, const CUtensorMap &map_up, __half *act, int M,
                       int N, int K, unsigned int *status, int timeout_ms, cudaStream_t stream, std::string *err,
                       int box_n = 64, int live_rows = 0, int a_box_rows = 0, int wq = 0, const void *raw_gate = nullptr,
                       const void *raw_up = nullptr);
int launch_gemm_grouped(const CUtensorMap &map_a, int ngroups, const CUtensorMap *const *maps_b, float *const *Cs,
                        const int *Ns, int M, int K, int box_n, unsigned int *status, int timeout_ms, cudaStream_t stream,
                        std::string *err, int live_rows = 0, int a_box_rows = 0, int wq = 0, const void *const *raws = nullptr);
int launch_gemm(const CUtensorMap &map_a, const CUtensorMap &map_b, float *C, int M, int N, int K, int box_n,
                unsigned int *status, int timeout_ms, cudaStream_t stream, std::string *err, int live_rows = 0, int a_box_rows = 0,
                int wq = 0, const void *raw = nullptr);
}  // namespace qmk_tc

#endif  // QMK_PREFILL_SM100_H_
