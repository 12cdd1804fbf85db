// Reference-named entry points of Klas_GEMM_SHMem (FStarLang/kuiper dist/Klas_GEMM_SHMem.h), forwarded to the C ABI.
// Link this object wherever the reference links its own Klas_GEMM_SHMem.o (nvcc.mk:22-26).
#include "Klas_GEMM_SHMem.h"
#undef KLAS_ENTRY
#include "compat_common.h"

KLAS_NUM_TYPES(KLAS_TILED_ENTRIES, SHMem)
