/* Klas_GEMM_BlockTiling2D.h -- prototypes of the reference's Klas_GEMM_BlockTiling2D entry points (FStarLang/kuiper dist/Klas_GEMM_BlockTiling2D.h),
 * served by libklas_b200.so through the Klas_GEMM_BlockTiling2D compatibility object.  C++ linkage, as in the reference. */
#ifndef Klas_GEMM_BlockTiling2D_H
#define Klas_GEMM_BlockTiling2D_H

#include <kuiper.h>
#include "klas_signatures.h"

#define KLAS_ENTRY(name, params, ...) void name params;
#include "grids/bt2d.inc"
#undef KLAS_ENTRY

#define Klas_GEMM_BlockTiling2D_H_DEFINED
#endif /* Klas_GEMM_BlockTiling2D_H */
