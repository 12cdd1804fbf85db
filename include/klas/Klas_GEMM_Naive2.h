/* Klas_GEMM_Naive2.h -- prototypes of the reference's Klas_GEMM_Naive2 entry points (FStarLang/kuiper dist/Klas_GEMM_Naive2.h),
 * served by libklas_b200.so through the Klas_GEMM_Naive2 compatibility object.  C++ linkage, as in the reference. */
#ifndef Klas_GEMM_Naive2_H
#define Klas_GEMM_Naive2_H

#include <kuiper.h>
#include "klas_signatures.h"

#define KLAS_ENTRY(name, params, ...) void name params;
KLAS_NUM_TYPES(KLAS_NAIVE_ENTRIES, Naive2)
KLAS_NAIVE_BATCHED_ENTRIES(Naive2)
#undef KLAS_ENTRY

#define Klas_GEMM_Naive2_H_DEFINED
#endif /* Klas_GEMM_Naive2_H */
