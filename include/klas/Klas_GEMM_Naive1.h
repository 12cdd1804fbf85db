/* Klas_GEMM_Naive1.h -- prototypes of the reference's Klas_GEMM_Naive1 entry points (FStarLang/kuiper dist/Klas_GEMM_Naive1.h),
 * served by libklas_b200.so through the Klas_GEMM_Naive1 compatibility object.  C++ linkage, as in the reference. */
#ifndef Klas_GEMM_Naive1_H
#define Klas_GEMM_Naive1_H

#include <kuiper.h>
#include "klas_signatures.h"

#define KLAS_ENTRY(name, params, ...) void name params;
KLAS_NUM_TYPES(KLAS_NAIVE_ENTRIES, Naive1)
KLAS_NAIVE_BATCHED_ENTRIES(Naive1)
#undef KLAS_ENTRY

#define Klas_GEMM_Naive1_H_DEFINED
#endif /* Klas_GEMM_Naive1_H */
