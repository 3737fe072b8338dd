// Host-visible handle of the multi-sequence build of the decode megakernel (megakernel_batch_sm100.cu).
#ifndef QMK_MEGAKERNEL_BATCH_H_
#define QMK_MEGAKERNEL_BATCH_H_

#include <stddef.h>

namespace qmk_batch {
const void *kernel();          // __global__ entry, launched cooperatively with one Params argument
size_t smem_bytes();           // dynamic shared memory of one CTA
int threads();                 // threads per CTA
size_t exchange_words();       // 8-byte words of exchange area the kernel addresses (copies x sequences)
}  // namespace qmk_batch

#endif  // QMK_MEGAKERNEL_BATCH_H_
