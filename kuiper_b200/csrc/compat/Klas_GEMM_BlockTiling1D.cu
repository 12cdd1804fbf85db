// Reference-named entry points of Klas_GEMM_BlockTiling1D (FStarLang/kuiper dist/Klas_GEMM_BlockTiling1D.h), forwarded to the C ABI.
// Link this object wherever the reference links its own Klas_GEMM_BlockTiling1D.o (nvcc.mk:22-26).
#include "Klas_GEMM_BlockTiling1D.h"
#undef KLAS_ENTRY
#include "compat_common.h"

KLAS_NUM_TYPES(KLAS_BT1D_ENTRIES, BlockTiling1D)
