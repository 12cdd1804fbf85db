// Reference-named entry points of Klas_RowSoftmax (FStarLang/kuiper dist/Klas_RowSoftmax.h), forwarded to the C ABI.
// Link this object wherever the reference links its own Klas_RowSoftmax.o (nvcc.mk:22-26).
#include "Klas_RowSoftmax.h"
#undef KLAS_ENTRY
#undef KLAS_RENTRY
#include "compat_common.h"

KLAS_ROWSOFTMAX_ENTRIES
