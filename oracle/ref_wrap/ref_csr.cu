// Test-side wrapper: exposes the reference's host-side CSR preparation, compiled unmodified from
// test/spmm_common.c.inc (sparsify_f32 / sparsify_u32: lines 73-137; mk_row_indices: 139-157), to the
// parity tests through a C ABI.  Not part of the product.
// Compile with: -I <kuiper>/include -I <kuiper>/test -I <kuiper>/dist
#include <inttypes.h>
#include <math.h>
const char *progname_csr = "ref_csr";
#include "spmm_common.c.inc"

// Returns nnz; copies the arrays out when the destinations are given (row_off has rows + 1 slots).
extern "C" uint32_t ref_sparsify_f32(float *M, int rows, int cols, uint32_t *row_off, float *elems, uint32_t *col_ind) {
    smatrix_f32_t s = sparsify_f32(M, rows, cols);
    memcpy(row_off, s.row_off, sizeof(uint32_t) * (rows + 1));
    if (elems) memcpy(elems, s.elems, sizeof(float) * s.nnz);
    if (col_ind) memcpy(col_ind, s.col_ind, sizeof(uint32_t) * s.nnz);
    const uint32_t nnz = s.nnz;
    free(s.elems);
    free(s.col_ind);
    free(s.row_off);
    return nnz;
}

extern "C" uint32_t ref_sparsify_u32(uint32_t *M, int rows, int cols, uint32_t *row_off, uint32_t *elems, uint32_t *col_ind) {
    smatrix_u32_t s = sparsify_u32(M, rows, cols);
    memcpy(row_off, s.row_off, sizeof(uint32_t) * (rows + 1));
    if (elems) memcpy(elems, s.elems, sizeof(uint32_t) * s.nnz);
    if (col_ind) memcpy(col_ind, s.col_ind, sizeof(uint32_t) * s.nnz);
    const uint32_t nnz = s.nnz;
    free(s.elems);
    free(s.col_ind);
    free(s.row_off);
    return nnz;
}

extern "C" void ref_mk_row_indices(int rows, uint32_t *row_off, uint32_t *out) {
    smatrix_u32_t s;
    s.nnz = row_off[rows];
    s.elems = NULL;
    s.col_ind = NULL;
    s.row_off = row_off;
    uint32_t *ri = mk_row_indices(rows, s);
    memcpy(out, ri, sizeof(uint32_t) * rows);
    free(ri);
}
