/* Klas_GEMM_Tiled.h -- prototypes of the reference's Klas_GEMM_Tiled entry points (FStarLang/kuiper dist/Klas_GEMM_Tiled.h),
 * served by libklas_b200.so through the Klas_GEMM_Tiled compatibility object.  C++ linkage, as in the reference. */
#ifndef Klas_GEMM_Tiled_H
#define Klas_GEMM_Tiled_H

#include <kuiper.h>
#include "klas_signatures.h"

#define KLAS_ENTRY(name, params, ...) void name params;
KLAS_NUM_TYPES(KLAS_TILED_ENTRIES, Tiled)
#undef KLAS_ENTRY

#define Klas_GEMM_Tiled_H_DEFINED
#endif /* Klas_GEMM_Tiled_H */
