/* Kuiper_Example_Fused_GEMM.h -- prototype of the reference's fused-map demonstration
 * (FStarLang/kuiper dist/Kuiper_Example_Fused_GEMM.h:9-15), served by libklas_b200.so through
 * the Kuiper_Example_Fused_GEMM compatibility object.  C++ linkage, as in the reference. */
#ifndef Kuiper_Example_Fused_GEMM_H
#define Kuiper_Example_Fused_GEMM_H

#include <kuiper.h>

/* C <- sqrt(A) @ B; A m x k, B k x n, C m x n, all fp16 row-major on the device; fp32
 * accumulation.  Here n and k must be multiples of 8 (the tensor-core path's 16-byte rows). */
void
Kuiper_Example_Fused_GEMM_gemm_sqrt_fused(uint32_t m, uint32_t n, uint32_t k, half *gA, half *gB, half *gC);

#define Kuiper_Example_Fused_GEMM_H_DEFINED
#endif /* Kuiper_Example_Fused_GEMM_H */
