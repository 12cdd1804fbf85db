// Reference-named entry points of Klas_GEMM_Naive1 (FStarLang/kuiper dist/Klas_GEMM_Naive1.h), forwarded to the C ABI.
// Link this object wherever the reference links its own Klas_GEMM_Naive1.o (nvcc.mk:22-26).
#include "Klas_GEMM_Naive1.h"
#undef KLAS_ENTRY
#include "compat_common.h"

KLAS_NUM_TYPES(KLAS_NAIVE_ENTRIES, Naive1)
KLAS_NAIVE_BATCHED_ENTRIES(Naive1)
