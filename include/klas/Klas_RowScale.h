/* Klas_RowScale.h -- prototypes of the reference's Klas_RowScale entry points (FStarLang/kuiper dist/Klas_RowScale.h),
 * served by libklas_b200.so through the Klas_RowScale compatibility object.  C++ linkage, as in the reference. */
#ifndef Klas_RowScale_H
#define Klas_RowScale_H

#include <kuiper.h>
#include "klas_signatures.h"

#define KLAS_ENTRY(name, params, ...) void name params;
#define KLAS_RENTRY(ret, name, params, ...) ret name params;
KLAS_ROWSCALE_TYPES(KLAS_ROWSCALE_ENTRIES)
#undef KLAS_ENTRY
#undef KLAS_RENTRY

#define Klas_RowScale_H_DEFINED
#endif /* Klas_RowScale_H */
