/* Klas_GEMM_TensorCore.h -- prototypes of the reference's Klas_GEMM_TensorCore entry points (FStarLang/kuiper dist/Klas_GEMM_TensorCore.h),
 * served by libklas_b200.so through the Klas_GEMM_TensorCore compatibility object.  C++ linkage, as in the reference. */
#ifndef Klas_GEMM_TensorCore_H
#define Klas_GEMM_TensorCore_H

#include <kuiper.h>
#include "klas_signatures.h"

#define KLAS_ENTRY(name, params, ...) void name params;
KLAS_TC1D_ENTRIES(KLAS_TC1D_ENTRY)
#undef KLAS_ENTRY

#define Klas_GEMM_TensorCore_H_DEFINED
#endif /* Klas_GEMM_TensorCore_H */
