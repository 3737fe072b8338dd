// What the tensor-core side (prefill_sm100.cu) needs from the per-device engine state kept in
// megakernel_sm100.cu: options set through qmk_configure and the fp32 rotary table.
#ifndef QMK_ENGINE_INTERNAL_H_
#define QMK_ENGINE_INTERNAL_H_

#include <cuda_runtime.h>
#include <string>

namespace qmk_internal {
struct PrefillEnv {
  const float *rope;      // fp32 [position][cos 64 | sin 64] covering max_seq_len (null in table mode)
  int vocab;
  int timeout_ms;
  int wfmt;               // 0 fp16 weights, 1 fp8 rows, 2 nvfp4 rows
  int rope_from_table;
  float *logits_out;      // debug dump set through qmk_set_logits_dump (may be null)
  int attn_mma;           // 1: batched decode attention on mma.sync (decode_attention_mma), 0: the CUDA-core ring kernel
  int attn_tc;            // 1: prefill attention on tcgen05 (causal_attention_tc), 0: on mma.sync (causal_attention_mma)
  int pdl;                // 1: kernels of a decode step / prefill pass are launched as programmatic dependents of one another
};
// Engine of the current device, created on first use; clears its last error.
int prefill_env(int max_seq_len, cudaStream_t stream, PrefillEnv *out);
// Records an error on the current device's engine (qmk_last_error) and returns `code`.
int report(int code, const std::string &msg);
}  // namespace qmk_internal

#endif  // QMK_ENGINE_INTERNAL_H_
