// Host-visible handle of the tensor-core build of the fused single-sequence decode megakernel (megakernel_tc_sm100.cu).
#ifndef QMK_MEGAKERNEL_TC_H_
#define QMK_MEGAKERNEL_TC_H_

#include <stddef.h>

namespace qmk_fused_tc {
const void *kernel();          // __global__ entry, launched cooperatively with one Params argument
size_t smem_bytes();           // dynamic shared memory of one CTA
int threads();                 // threads per CTA
int min_ctas();                // smallest grid the kernel's shared-memory slices are sized for
}  // namespace qmk_fused_tc

#endif  // QMK_MEGAKERNEL_TC_H_
