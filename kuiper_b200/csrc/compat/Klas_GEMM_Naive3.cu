// Reference-named entry points of Klas_GEMM_Naive3 (FStarLang/kuiper dist/Klas_GEMM_Naive3.h), forwarded to the C ABI.
// Link this object wherever the reference links its own Klas_GEMM_Naive3.o (nvcc.mk:22-26).
#include "Klas_GEMM_Naive3.h"
#undef KLAS_ENTRY
#include "compat_common.h"

KLAS_NAIVE3_TYPES(KLAS_NAIVE3_ENTRIES, Naive3)
