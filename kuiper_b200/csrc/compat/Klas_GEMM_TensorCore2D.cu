// Reference-named entry points of Klas_GEMM_TensorCore2D (FStarLang/kuiper dist/Klas_GEMM_TensorCore2D.h), forwarded to the C ABI.
// Link this object wherever the reference links its own Klas_GEMM_TensorCore2D.o (nvcc.mk:22-26).
#include "Klas_GEMM_TensorCore2D.h"
#undef KLAS_ENTRY
#include "compat_common.h"

#define KLAS_TC2D_INSTANCE KLAS_TC2D_PLAIN_INSTANCE
#include "grids/tc2d.inc"
