// Reference-named entry point of the fused-map demonstration (FStarLang/kuiper
// dist/Kuiper_Example_Fused_GEMM.cu:29-43: one thread per output element, sqrtf(A) * B summed in
// f32), forwarded to the tensor-core GEMM with the square root applied to the staged A tiles.
#include "Kuiper_Example_Fused_GEMM.h"
#include "compat_common.h"

void Kuiper_Example_Fused_GEMM_gemm_sqrt_fused(uint32_t m, uint32_t n, uint32_t k, half *gA, half *gB, half *gC) {
    KPR_GUARD(n % 8U == 0U);
    KPR_GUARD(k % 8U == 0U);
    klas_compat::finish(klas_b200_gemm_tc_fused(KLAS_F16, KLAS_F16, KLAS_B_ROW_MAJOR, 1, m, k, n, gA, gB, NULL, gC, 1.0f,
                                                0.0f, KLAS_MAP_SQRT, KLAS_MAP_ID, KLAS_COMB_NEW, NULL, NULL),
                        "Kuiper_Example_Fused_GEMM_gemm_sqrt_fused", true);
}
