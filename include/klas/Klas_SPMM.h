/* Klas_SPMM.h -- prototypes of the reference's Klas_SPMM entry points (FStarLang/kuiper dist/Klas_SPMM.h),
 * served by libklas_b200.so through the Klas_SPMM compatibility object.  C++ linkage, as in the reference. */
#ifndef Klas_SPMM_H
#define Klas_SPMM_H

#include <kuiper.h>
#include "klas_signatures.h"

/* CSR matrix handed to the SpMM entry points BY VALUE; all three arrays are device pointers
 * (dist/Klas_SPMM.h:7-12,21-26).  row_off has rows+1 entries, row_off[0] = 0, row_off[rows] = nnz;
 * column indices are sorted inside each row. */
typedef struct Kuiper_Sparse_Matrix_smatrix__uint32_t_s {
    uint32_t nnz;
    uint32_t *elems;
    uint32_t *col_ind;
    uint32_t *row_off;
} Kuiper_Sparse_Matrix_smatrix__uint32_t;

typedef struct Kuiper_Sparse_Matrix_smatrix__float_s {
    uint32_t nnz;
    float *elems;
    uint32_t *col_ind;
    uint32_t *row_off;
} Kuiper_Sparse_Matrix_smatrix__float;

#define KLAS_ENTRY(name, params, ...) void name params;
KLAS_SPMM_FIXED_ENTRIES
#include "grids/spmm.inc"
#undef KLAS_ENTRY

#define Klas_SPMM_H_DEFINED
#endif /* Klas_SPMM_H */
