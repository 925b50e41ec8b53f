#include "qb_internal.h"
bool qb_gemm_tc_supported(const qb_weight *, uint32_t) { return false; }
int qb_launch_gemm_tc(qb_ctx *, const qb_weight *, const int8_t *, const float *, uint32_t, float *, uint32_t) {
    return qb_fail(QB_ERR_UNSUPPORTED, "tensor-core GEMM not built");
}
