// Reference-named entry points of Klas_HReduce (FStarLang/kuiper dist/Klas_HReduce.h), forwarded to the C ABI.
// Link this object wherever the reference links its own Klas_HReduce.o (nvcc.mk:22-26).
#include "Klas_HReduce.h"
#undef KLAS_ENTRY
#undef KLAS_RENTRY
#include "compat_common.h"

KLAS_HREDUCE_ENTRIES
