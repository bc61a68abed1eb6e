// Dequantize + tensor-core GEMM for prefill (m >= 64).  Placeholder until the tcgen05 kernel
// lands: reports HLQ_ERR_UNSUPPORTED so that callers fail loudly instead of silently taking
// another path.
#include "hlq_internal.h"

namespace hlq {
int launch_dequant_gemm(const hlq_weight *, int, const void *, int, void *, int, void *, size_t,
                        cudaStream_t) {
    return HLQ_ERR_UNSUPPORTED;
}
}  // namespace hlq
