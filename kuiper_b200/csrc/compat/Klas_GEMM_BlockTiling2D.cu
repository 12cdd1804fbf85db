// Reference-named entry points of Klas_GEMM_BlockTiling2D (FStarLang/kuiper dist/Klas_GEMM_BlockTiling2D.h), forwarded to the C ABI.
// Link this object wherever the reference links its own Klas_GEMM_BlockTiling2D.o (nvcc.mk:22-26).
#include "Klas_GEMM_BlockTiling2D.h"
#undef KLAS_ENTRY
#include "compat_common.h"

#include "grids/bt2d.inc"
