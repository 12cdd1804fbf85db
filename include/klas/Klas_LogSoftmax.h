/* Klas_LogSoftmax.h -- prototypes of the reference's Klas_LogSoftmax entry points (FStarLang/kuiper dist/Klas_LogSoftmax.h),
 * served by libklas_b200.so through the Klas_LogSoftmax compatibility object.  C++ linkage, as in the reference. */
#ifndef Klas_LogSoftmax_H
#define Klas_LogSoftmax_H

#include <kuiper.h>
#include "klas_signatures.h"

#define KLAS_ENTRY(name, params, ...) void name params;
#define KLAS_RENTRY(ret, name, params, ...) ret name params;
KLAS_SOFTMAX_TYPES(KLAS_SOFTMAX_ENTRIES, LogSoftmax, log_softmax)
#undef KLAS_ENTRY
#undef KLAS_RENTRY

#define Klas_LogSoftmax_H_DEFINED
#endif /* Klas_LogSoftmax_H */
