// Reference-named entry points of Klas_RowScale (FStarLang/kuiper dist/Klas_RowScale.h), forwarded to the C ABI.
// Link this object wherever the reference links its own Klas_RowScale.o (nvcc.mk:22-26).
#include "Klas_RowScale.h"
#undef KLAS_ENTRY
#undef KLAS_RENTRY
#include "compat_common.h"

KLAS_ROWSCALE_TYPES(KLAS_ROWSCALE_ENTRIES)
