// Multi-sequence build of the persistent decode megakernel for sm_100a: the same producer, ring and
// exchange code as megakernel_sm100.cu, compiled with room for four sequences' activations in shared
// memory, plus the group-per-sequence consumer code of megakernel_batch.cuh.
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <math.h>

#include "../../include/qwen_megakernel.h"

#include "megakernel_params.h"

#define QMK_NS qmkb
#define QMK_MAX_SEQ 4
#include "megakernel_device.cuh"
#include "megakernel_batch.cuh"
#include "megakernel_batch.h"

static_assert(QMK_MAX_SEQ == qmkp::MAX_SEQ, "Params carries MAX_SEQ per-sequence entries");

namespace qmk_batch {
const void *kernel() { return reinterpret_cast<const void *>(qmkb::qwen3_decode_batch_megakernel); }
size_t smem_bytes() { return qmkb::SMEM_BYTES; }
int threads() { return qmkb::THREADS; }
size_t exchange_words() { return static_cast<size_t>(qmkb::LL_REPL_STRIDE) * qmkb::MAX_REPL; }
}  // namespace qmk_batch
