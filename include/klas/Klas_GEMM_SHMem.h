/* Klas_GEMM_SHMem.h -- prototypes of the reference's Klas_GEMM_SHMem entry points (FStarLang/kuiper dist/Klas_GEMM_SHMem.h),
 * served by libklas_b200.so through the Klas_GEMM_SHMem compatibility object.  C++ linkage, as in the reference. */
#ifndef Klas_GEMM_SHMem_H
#define Klas_GEMM_SHMem_H

#include <kuiper.h>
#include "klas_signatures.h"

#define KLAS_ENTRY(name, params, ...) void name params;
KLAS_NUM_TYPES(KLAS_TILED_ENTRIES, SHMem)
#undef KLAS_ENTRY

#define Klas_GEMM_SHMem_H_DEFINED
#endif /* Klas_GEMM_SHMem_H */
