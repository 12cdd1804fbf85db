// Reference-named entry points of Klas_SPMM (FStarLang/kuiper dist/Klas_SPMM.h), forwarded to the C ABI.
// Link this object wherever the reference links its own Klas_SPMM.o (nvcc.mk:22-26).
#include "Klas_SPMM.h"
#undef KLAS_ENTRY
#include "compat_common.h"

KLAS_SPMM_FIXED_ENTRIES
#include "grids/spmm.inc"
