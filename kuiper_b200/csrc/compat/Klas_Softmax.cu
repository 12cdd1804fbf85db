// Reference-named entry points of Klas_Softmax (FStarLang/kuiper dist/Klas_Softmax.h), forwarded to the C ABI.
// Link this object wherever the reference links its own Klas_Softmax.o (nvcc.mk:22-26).
#include "Klas_Softmax.h"
#undef KLAS_ENTRY
#undef KLAS_RENTRY
#include "compat_common.h"

KLAS_SOFTMAX_TYPES(KLAS_SOFTMAX_ENTRIES, Softmax, softmax)
