// Reference-named entry points of Klas_LogSoftmax (FStarLang/kuiper dist/Klas_LogSoftmax.h), forwarded to the C ABI.
// Link this object wherever the reference links its own Klas_LogSoftmax.o (nvcc.mk:22-26).
#include "Klas_LogSoftmax.h"
#undef KLAS_ENTRY
#undef KLAS_RENTRY
#include "compat_common.h"

KLAS_SOFTMAX_TYPES(KLAS_SOFTMAX_ENTRIES, LogSoftmax, log_softmax)
