// placeholder until the tcgen05 kernel lands
#include "common.cuh"
namespace nslq {
bool ternary_gemm_supported(const void *, const void *, int64_t, int64_t, int64_t) { return false; }
int ternary_gemm_dispatch(const uint8_t *, const int8_t *, const float *, const int32_t *, int64_t, int64_t,
                          int64_t, float, void *, int, int32_t *, const float *, const float *, cudaStream_t)
{ return fail(NSLQ_ERR_UNSUPPORTED, "tcgen05 GEMM not built"); }
}
