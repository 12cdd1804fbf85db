// Reference-named entry points of Klas_AtomicReduce (FStarLang/kuiper dist/Klas_AtomicReduce.h), forwarded to the C ABI.
// Link this object wherever the reference links its own Klas_AtomicReduce.o (nvcc.mk:22-26).
#include "Klas_AtomicReduce.h"
#undef KLAS_ENTRY
#undef KLAS_RENTRY
#include "compat_common.h"

KLAS_ATOMICREDUCE_ENTRIES
