/* Klas_GEMM_TensorCore2D_To.h -- prototypes of the reference's Klas_GEMM_TensorCore2D_To entry points (FStarLang/kuiper dist/Klas_GEMM_TensorCore2D_To.h),
 * served by libklas_b200.so through the Klas_GEMM_TensorCore2D_To compatibility object.  C++ linkage, as in the reference. */
#ifndef Klas_GEMM_TensorCore2D_To_H
#define Klas_GEMM_TensorCore2D_To_H

#include <kuiper.h>
#include "klas_signatures.h"

#define KLAS_ENTRY(name, params, ...) void name params;
#define KLAS_TC2D_INSTANCE KLAS_TC2D_TO_INSTANCE
#include "grids/tc2d.inc"
#undef KLAS_TC2D_INSTANCE
#undef KLAS_ENTRY

#define Klas_GEMM_TensorCore2D_To_H_DEFINED
#endif /* Klas_GEMM_TensorCore2D_To_H */
