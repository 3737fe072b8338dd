// Tensor-core build of the fused single-sequence decode megakernel for sm_100a: the exchange, attention and
// reduction code of megakernel_device.cuh / megakernel_fused.cuh compiled for a ring of 18 slots (four padded
// weight rows, or sixteen K rows and sixteen V rows as swizzled 128-byte boxes), plus the mma.sync row products, producer and kernel of megakernel_tc.cuh.
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <math.h>

#include "../../include/qwen_megakernel.h"

#include "megakernel_params.h"

#define QMK_NS qmkt
#define QMK_MAX_SEQ 1
#define QMK_TC_BUILD 1
#define QMK_NSLOTS 18
#define QMK_SLOT_BYTES 8832
#define QMK_EMPTY_UNITS 12
#include "megakernel_device.cuh"
#include "megakernel_fused.cuh"
#include "megakernel_tc.cuh"
#include "megakernel_tc.h"

namespace qmk_fused_tc {
const void *kernel() { return reinterpret_cast<const void *>(qmkt::qwen3_decode_megakernel_tc); }
size_t smem_bytes() { return qmkt::TC_SMEM_BYTES; }
int threads() { return qmkt::THREADS; }
int min_ctas() { return qmkt::TC_MIN_CTAS; }
}  // namespace qmk_fused_tc
