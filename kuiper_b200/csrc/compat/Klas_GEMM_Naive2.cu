// Reference-named entry points of Klas_GEMM_Naive2 (FStarLang/kuiper dist/Klas_GEMM_Naive2.h), forwarded to the C ABI.
// Link this object wherever the reference links its own Klas_GEMM_Naive2.o (nvcc.mk:22-26).
#include "Klas_GEMM_Naive2.h"
#undef KLAS_ENTRY
#include "compat_common.h"

KLAS_NUM_TYPES(KLAS_NAIVE_ENTRIES, Naive2)
KLAS_NAIVE_BATCHED_ENTRIES(Naive2)
