/* Klas_HReduce.h -- prototypes of the reference's Klas_HReduce entry points (FStarLang/kuiper dist/Klas_HReduce.h),
 * served by libklas_b200.so through the Klas_HReduce compatibility object.  C++ linkage, as in the reference. */
#ifndef Klas_HReduce_H
#define Klas_HReduce_H

#include <kuiper.h>
#include "klas_signatures.h"

#define KLAS_ENTRY(name, params, ...) void name params;
#define KLAS_RENTRY(ret, name, params, ...) ret name params;
KLAS_HREDUCE_ENTRIES
#undef KLAS_ENTRY
#undef KLAS_RENTRY

#define Klas_HReduce_H_DEFINED
#endif /* Klas_HReduce_H */
