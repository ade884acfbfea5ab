/* Seeded synthetic CSR matrices with the shape statistics of the benchmark configurations (host code only, no
 * CUDA): libmx_synth.so.  The reference evaluates on SuiteSparse files (data/all_url.log) that are not available
 * offline; these generators stand in for them.  The library is separate from libmatxtract_b200.so so that a process
 * which only needs inputs (a CPU baseline run, a test of the oracle) maps nothing of the GPU library.
 * No counterpart in the reference.
 */
#ifndef MX_SYNTH_H
#define MX_SYNTH_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* value types, same numbering as mx_capi.h */
enum { MX_SYNTH_FP64 = 0, MX_SYNTH_FP16 = 1 };
enum { MX_SYNTH_UNIFORM = 0, MX_SYNTH_POWERLAW = 1, MX_SYNTH_BLOCK = 2, MX_SYNTH_HOTCOL = 3 };
typedef struct {
    int kind;
    int64_t n;            /* square dimension */
    uint64_t seed;
    double mean_len;      /* UNIFORM: Poisson mean; HOTCOL: mean row length (1 + geometric) */
    double zipf_s;        /* POWERLAW: exponent of the row-length law */
    double alpha;         /* POWERLAW: length = clip(ceil(alpha * K), 1, max_len) */
    int64_t max_len;      /* POWERLAW: clip */
    double local_frac;    /* POWERLAW: share of a row's columns within +-local_halfwidth of the row index */
    int64_t local_halfwidth; /* POWERLAW: columns; BLOCK: block columns */
    int blocks_per_row;   /* BLOCK: dense 8x8 blocks per block row */
    double hot_col_frac;  /* HOTCOL: share of columns that are hot */
    double hot_nnz_frac;  /* HOTCOL: share of entries drawn from the hot columns */
    int normal_values;    /* values ~ N(0,1) instead of U(-1,1) */
} mx_synth_params;
/* Row pointers (relative to row_begin) of rows [row_begin, row_end); row_ptr_out has row_end-row_begin+1 ints. */
int mx_synth_row_lengths(const mx_synth_params *p, int64_t row_begin, int64_t row_end, int *row_ptr_out);
int mx_synth_fill(const mx_synth_params *p, int dtype, int64_t row_begin, int64_t row_end, const int *row_ptr,
                  int *col_ind, void *val);
int mx_synth_vector(uint64_t seed, int dtype, int64_t begin, int64_t end, void *x);

#ifdef __cplusplus
}
#endif
#endif /* MX_SYNTH_H */
