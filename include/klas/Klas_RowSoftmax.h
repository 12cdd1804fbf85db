/* Klas_RowSoftmax.h -- prototypes of the reference's Klas_RowSoftmax entry points (FStarLang/kuiper dist/Klas_RowSoftmax.h),
 * served by libklas_b200.so through the Klas_RowSoftmax compatibility object.  C++ linkage, as in the reference. */
#ifndef Klas_RowSoftmax_H
#define Klas_RowSoftmax_H

#include <kuiper.h>
#include "klas_signatures.h"

#define KLAS_ENTRY(name, params, ...) void name params;
#define KLAS_RENTRY(ret, name, params, ...) ret name params;
KLAS_ROWSOFTMAX_ENTRIES
#undef KLAS_ENTRY
#undef KLAS_RENTRY

#define Klas_RowSoftmax_H_DEFINED
#endif /* Klas_RowSoftmax_H */
