// Reference-named entry points of Klas_GEMM_TensorCore (FStarLang/kuiper dist/Klas_GEMM_TensorCore.h), forwarded to the C ABI.
// Link this object wherever the reference links its own Klas_GEMM_TensorCore.o (nvcc.mk:22-26).
#include "Klas_GEMM_TensorCore.h"
#undef KLAS_ENTRY
#include "compat_common.h"

KLAS_TC1D_ENTRIES(KLAS_TC1D_ENTRY)
