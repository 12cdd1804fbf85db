/* Klas_Softmax.h -- prototypes of the reference's Klas_Softmax entry points (FStarLang/kuiper dist/Klas_Softmax.h),
 * served by libklas_b200.so through the Klas_Softmax compatibility object.  C++ linkage, as in the reference. */
#ifndef Klas_Softmax_H
#define Klas_Softmax_H

#include <kuiper.h>
#include "klas_signatures.h"

#define KLAS_ENTRY(name, params, ...) void name params;
#define KLAS_RENTRY(ret, name, params, ...) ret name params;
KLAS_SOFTMAX_TYPES(KLAS_SOFTMAX_ENTRIES, Softmax, softmax)
#undef KLAS_ENTRY
#undef KLAS_RENTRY

#define Klas_Softmax_H_DEFINED
#endif /* Klas_Softmax_H */
