/* Klas_AtomicReduce.h -- prototypes of the reference's Klas_AtomicReduce entry points (FStarLang/kuiper dist/Klas_AtomicReduce.h),
 * served by libklas_b200.so through the Klas_AtomicReduce compatibility object.  C++ linkage, as in the reference. */
#ifndef Klas_AtomicReduce_H
#define Klas_AtomicReduce_H

#include <kuiper.h>
#include "klas_signatures.h"

#define KLAS_ENTRY(name, params, ...) void name params;
#define KLAS_RENTRY(ret, name, params, ...) ret name params;
KLAS_ATOMICREDUCE_ENTRIES
#undef KLAS_ENTRY
#undef KLAS_RENTRY

#define Klas_AtomicReduce_H_DEFINED
#endif /* Klas_AtomicReduce_H */
