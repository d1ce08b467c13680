// Tensor-core (tcgen05) path of the quantized batched matmul. Placeholder until
// the kernel lands: reports "shape not covered" so routing uses the CUDA-core path.
#include "lc_internal.h"

int lc_qgemm_tcgen05(int, bool, lc_kernels *, lc_batch *, const lc_buf *, const lc_buf *, lc_buf *, uint32_t,
                     uint32_t, uint32_t) {
    return -1;
}
