/* Klas_GEMM_Naive3.h -- prototypes of the reference's Klas_GEMM_Naive3 entry points (FStarLang/kuiper dist/Klas_GEMM_Naive3.h),
 * served by libklas_b200.so through the Klas_GEMM_Naive3 compatibility object.  C++ linkage, as in the reference. */
#ifndef Klas_GEMM_Naive3_H
#define Klas_GEMM_Naive3_H

#include <kuiper.h>
#include "klas_signatures.h"

#define KLAS_ENTRY(name, params, ...) void name params;
KLAS_NAIVE3_TYPES(KLAS_NAIVE3_ENTRIES, Naive3)
#undef KLAS_ENTRY

#define Klas_GEMM_Naive3_H_DEFINED
#endif /* Klas_GEMM_Naive3_H */
