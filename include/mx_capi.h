/* C ABI of the B200 MatXtract SpMV library (libmatxtract_b200.so).
 *
 * This is the layer the C++ host API (include/MatXtract.h) and the command-line drivers call CUDA
 * through, and what a foreign-language binding (ctypes, cgo, JNI ...) would bind.  Plain C types only;
 * every function returns an int status (MX_OK = 0), never throws and never exits the process.
 * Host buffers belong to the caller; device buffers belong to the handle.  One thread per handle.
 *
 * Each entry point names the reference interface it replaces (paths relative to the reference project).
 */
#ifndef MX_CAPI_H
#define MX_CAPI_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
    MX_OK = 0,
    MX_ERR_INVALID = 1,  /* bad argument (null pointer, negative size ...) */
    MX_ERR_CUDA = 2,     /* a CUDA runtime call failed; see mx_last_error_string */
    MX_ERR_TAU = 3,      /* tau_c < tau_r, or a threshold that no prefix of the ranking reaches */
    MX_ERR_STATE = 4,    /* call order: no matrix uploaded, no partition built ... */
    MX_ERR_OVERFLOW = 5, /* a count does not fit the reference's int32 index type */
    MX_ERR_TIMEOUT = 6,  /* a bounded device-side wait ran out */
    MX_ERR_NOMEM = 7,
    MX_ERR_NO_DEVICE = 8, /* no CUDA device: there is no CPU fallback */
    MX_ERR_TOO_LARGE = 9  /* the matrix exceeds the fixed scratch of mx_csr_spmv_static */
};

/* Value type of a handle.  The reference fixes it at compile time (-Dfp64, include/common.h:53-70):
 * MX_FP64 = double values, 8x4 fragments, 32-bit bitmaps; MX_FP16 = half values, 8x8 fragments, 64-bit bitmaps. */
enum { MX_FP64 = 0, MX_FP16 = 1 };

typedef struct mx_handle_s *mx_handle_t;

int mx_version(void);
const char *mx_status_string(int status);

/* ---- handle --------------------------------------------------------------------------------------- */
int mx_create(mx_handle_t *h, int device, int dtype);
int mx_destroy(mx_handle_t h);
const char *mx_last_error_string(mx_handle_t h);
/* The CUDA stream (cudaStream_t) all work of this handle is issued on. */
void *mx_stream(mx_handle_t h);
int mx_sync(mx_handle_t h);

/* Uploads a host CSR matrix (replaces the per-call cudaMalloc + cudaMemcpy of every reference wrapper,
 * e.g. src/spmv_kernel/cdSpMV.cu:407-418).  Any previous matrix and partition of the handle is dropped.  The reference
 * trusts its inputs (unchecked copies, include/common.h:81-90); here one pass on the device checks that row_ptr never
 * decreases and that every column index lies in [0, n_cols) before any kernel uses them as addresses: a matrix that
 * fails is refused with MX_ERR_INVALID and the handle is left without a matrix. */
int mx_upload_csr(mx_handle_t h, int n_rows, int n_cols, int nnz, const int *row_ptr, const int *col_ind,
                  const void *val);

/* ---- extraction (preprocessing) ------------------------------------------------------------------- */
typedef struct {
    int dCols, nnzColD, sCols, nnzColS; /* tau_c cut,  test/test_autotc_spmv.cpp:1131-1145 */
    int dRows, nnzRowD, sRows, nnzRowS; /* tau_r cut,  test/test_autotc_spmv.cpp:1249-1269 */
    int chunkNum, totalFrags;           /* 8-row panels and fragments, :1354,:1375 */
    int nnzCD;                          /* residual CSR entries, :1477 */
    int fragK;                          /* 4 (FP64) or 8 (FP16) */
    double tc_nnz_ratio;                /* nnzRowD / (totalFrags * 8 * fragK), :1376 */
    float preprocess_ms;                /* device time of the whole extraction */
    int active;                         /* 0 when tau = (0,0): no extraction, the residual is the input CSR (:1106,:1638) */
    float tuning_ms;                    /* host time of the plan-time tuners (timed trial products), not in preprocess_ms */
} mx_partition_stats;

/* Runs the cascaded extraction on the device: column histogram and tau_c hot-column selection, row
 * ranking inside the hot columns and tau_r hot-row selection, dense 8xK tile construction, residual CSR
 * compaction.  Replaces the host pipeline inside main() of test/test_autotc_spmv.cpp:1119-1421,1486-1492
 * and its three cuSPARSE transposes (utilities/csr2csc.cpp).  tau_c and tau_r are converted to float
 * exactly as the reference does (:1103-1104); tau_c < tau_r is rejected (:1064-1069) with MX_ERR_TAU.
 * The reference assumes a square matrix; a rectangular row slab (rows < cols, one GPU's share of a
 * row-partitioned matrix) is accepted as well and is extracted on its own. */
int mx_partition(mx_handle_t h, double tau_c, double tau_r, mx_partition_stats *stats);
int mx_partition_stats_get(mx_handle_t h, mx_partition_stats *stats);
/* Extraction of one row slab of a matrix that is spread over several GPUs, with the reference's rankings taken over
 * the WHOLE matrix (the reference ranks all columns and all rows of its one matrix, test/test_autotc_spmv.cpp:1122-1141,
 * 1240-1267): the slabs' hot columns are then the whole matrix's hot columns (same dCols, same xperm on every GPU) and
 * the slabs' hot rows together are the whole matrix's hot rows.  The caller supplies what needs an exchange:
 *   1. mx_col_counts on every slab, summed over the slabs                      -> global_col_counts_dev, global_nnz
 *   2. mx_row_counts_in_hot_columns on every slab, concatenated in row order   -> the whole matrix's row counts
 *   3. mx_rank_cut(counts, n_rows, (int)((float)global_nnz * (float)tau_r))     -> out[2], out[3] = the row cut
 *   4. mx_partition_global on every slab with that cut and the slab's first global row index.
 * mx_mg_partition does these steps itself.  All *_dev pointers are device memory on the handle's GPU. */
int mx_col_counts(mx_handle_t h, int *counts_dev /* [n_cols] */);
int mx_row_counts_in_hot_columns(mx_handle_t h, double tau_c, const int *global_col_counts_dev, long long global_nnz,
                                 int *row_counts_dev /* [n_rows] */);
/* counts ranked descending (ties: lower index first); out = {k, sum, count of the k-th, index of the k-th} for the
 * smallest prefix k >= 1 whose sum reaches threshold; k = 0 when none does. */
int mx_rank_cut(mx_handle_t h, const int *counts_dev, int n, long long threshold, long long out[4]);
int mx_partition_global(mx_handle_t h, double tau_c, double tau_r, const int *global_col_counts_dev,
                        long long global_nnz, int row_cut_count, long long row_cut_index, long long row_offset,
                        mx_partition_stats *stats);
/* The int32 limit of the fragment format (the reference's indT, include/common.h:79, indexes both the fragments and
 * the fragK x-index slots of each, test/test_autotc_spmv.cpp:1384-1404): MX_OK when `total_frags` fragments can be
 * indexed, MX_ERR_OVERFLOW when not.  mx_partition applies this rule to the fragment total (taken in 64 bits on the
 * device) and fails with MX_ERR_OVERFLOW instead of wrapping.  Host-only. */
int mx_fragment_count_status(long long total_frags, int dtype);
/* Shape of the matrix the handle holds (uploaded, or restored by mx_load_partition). */
int mx_dims(mx_handle_t h, int *n_rows, int *n_cols, int *nnz);

/* Stores / restores a partition so that the extraction is paid once per matrix (successor of the reference's
 * `<matrix>_preprocessed[_fp16].dat` dump, test/tcpreprocess.cpp:1208-1255, which held the fragment format only).
 * The file holds every array of mx_partition_arrays plus the counts; it is enough to multiply: mx_load_partition
 * needs no uploaded matrix (and drops one that is there), builds the execution plans and leaves the handle ready for
 * mx_spmv.  A loaded handle cannot be re-extracted with other taus (the original CSR is not in the file). */
int mx_save_partition(mx_handle_t h, const char *path);
/* Every array of the file ends up as addresses in the kernels, so the whole file is read and checked on the host
 * before anything is uploaded (pointer arrays monotone and ending at their counts, row ids distinct and in range,
 * xperm a permutation, column ids in range, value counts equal to the bitmaps' population counts); a file that fails
 * is refused with MX_ERR_INVALID and the handle is left empty. */
int mx_load_partition(mx_handle_t h, const char *path, mx_partition_stats *stats);
/* The loader's check alone, without a GPU: MX_OK, or MX_ERR_INVALID with what is wrong in msg (if msg != NULL). */
int mx_check_partition_file(const char *path, int dtype, char *msg, int msg_len);

/* Searches (tau_c, tau_r) on the device instead of the reference's 20-run Bayesian search through the command-line
 * driver (ML/bayes_opt.py:153-163): every valid point of the grid {0, 1/grid, ..., 1}^2 with tau_c >= tau_r is
 * extracted and its product timed (3 warm + 10 timed); the fastest is left installed in the handle.
 * ms_plain is the time of tau = (0,0). */
int mx_autotune_tau(mx_handle_t h, int grid, double *tau_c, double *tau_r, float *ms_best, float *ms_plain);

/* Host destinations for the arrays of the partition, in the reference's layout; a NULL member is skipped.
 * Sizes follow from mx_partition_stats (K = fragK). */
typedef struct {
    int *xperm;      /* [n_cols]  x_CD[i] = x[xperm[i]]; first dCols entries = hot columns in rank order */
    int *rId;        /* [dRows]   original row of hot row i */
    int *rowPtr_dd;  /* [dRows+1] core-dense block as CSR, column ids = density ranks */
    int *colInd_dd;  /* [nnzRowD] */
    void *val_dd;    /* [nnzRowD] */
    int *chunkPtr;   /* [chunkNum+1] */
    int *AToX;       /* [totalFrags*K] sparse_AToX_index */
    int *fragPtr;    /* [totalFrags+1] */
    void *fragBit;   /* [totalFrags] uint32 (FP64) or uint64 (FP16) */
    void *tcVal;     /* [nnzRowD] */
    int *rowPtr_CD;  /* [n_rows+1] residual CSR */
    int *colInd_CD;  /* [nnzCD] */
    void *val_CD;    /* [nnzCD] */
} mx_partition_arrays;
int mx_download_partition(mx_handle_t h, const mx_partition_arrays *out);

/* ---- execution ------------------------------------------------------------------------------------ */
/* y = A x with x and y DEVICE pointers in the matrix's original column / row order; asynchronous on the
 * handle's stream.  Runs the tile kernel on the core-dense block and the CSR kernel on the residual; the
 * second produces the final y, so there is no merge pass and no host scatter
 * (replaces test/test_autotc_spmv.cpp:1507-1559). */
int mx_spmv(mx_handle_t h, const void *x_dev, void *y_dev);
/* Row-partitioned product across the GPUs of one box with the y all-gather fused into the kernel (the reference is
 * single-GPU; this is the multi-GPU exchange step).  This handle owns the row slab [row_offset, row_offset + n_rows)
 * of the whole matrix; y_peers[g] is a DEVICE pointer, valid on this GPU, to the full-length y of GPU g (peer-mapped
 * memory, e.g. a symmetric-memory buffer; y_peers must include this GPU's own buffer; n_peers <= 8).  Every finished
 * row is stored into all n_peers buffers with plain stores over NVLink while the rest of the kernel is still
 * computing.  The caller runs a barrier across the GPUs afterwards (every y is complete once all GPUs have passed it);
 * nothing in the kernels waits on another GPU. */
int mx_spmv_peers(mx_handle_t h, const void *x_dev, void *const *y_peers, int n_peers, long long row_offset);
/* mx_spmv_peers with the rows sent through NVSwitch multicast: y_multicast is the multicast address of the same
 * buffers (every GPU's y bound to one NVLink multicast object, e.g. torch symmetric memory's multicast_ptr).  Each
 * 8-byte row - or aligned pair of adjacent 2-byte rows - leaves the GPU as ONE multimem.st that the switch writes
 * into every GPU's copy; rows that cannot be paired fall back to the peer stores of mx_spmv_peers.  Same barrier
 * obligation afterwards.  No counterpart in the reference. */
int mx_spmv_multicast(mx_handle_t h, const void *x_dev, void *const *y_peers, int n_peers, void *y_multicast,
                      long long row_offset);
/* The unfused alternative for small slabs: after mx_spmv wrote this GPU's rows into its own full-length y
 * (y_peers[self] + row_offset), copy those rows into the same place of every other GPU's y with 16-byte peer stores.
 * table_dev: 64 bytes of device memory the call may use (the peers' row addresses).  Followed, like mx_spmv_peers, by
 * the caller's barrier across the GPUs. */
int mx_peer_push(int dtype, void *const *y_peers, int n_peers, int self, long long row_offset, long long n_rows,
                 void *table_dev, void *stream);
/* ---- multi-GPU: one process drives several GPUs of one box (no counterpart in the reference, which is single-GPU) -- */
/* Rows are cut into n_devices contiguous slabs of equal non-zero count, bounds[g] = lower_bound(row_ptr, g*nnz/G);
 * x is replicated, every GPU extracts and multiplies its own slab (rows_g x all columns) through a handle of its own,
 * and every GPU ends a product with the whole y.  The exchange of y is either MX_MG_EXCHANGE_PEER (default where the
 * GPUs can address each other's memory): the SpMV kernels store their finished rows into every GPU's buffer over
 * NVLink (mx_spmv_peers) and the GPUs then wait for each other's CUDA events in stream order - nothing spins; or
 * MX_MG_EXCHANGE_NCCL: every GPU writes its own rows and NCCL broadcasts the slabs (ncclCommInitAll; libnccl.so.2 is
 * bound at run time).  One host thread per mx_mg_t.  Devices must be distinct. */
typedef struct mx_mg_s *mx_mg_t;
enum { MX_MG_EXCHANGE_PEER = 0, MX_MG_EXCHANGE_NCCL = 1 };
/* devices = NULL: GPUs 0 .. n_devices-1.  n_devices <= 8. */
int mx_mg_create(mx_mg_t *mg, int n_devices, const int *devices, int dtype);
int mx_mg_destroy(mx_mg_t mg);
const char *mx_mg_last_error_string(mx_mg_t mg);
int mx_mg_set_exchange(mx_mg_t mg, int mode);
/* The nnz-balanced row boundaries alone (host code, no GPU): bounds has n_parts + 1 entries. */
int mx_mg_partition_rows(const int *row_ptr, int n_rows, int n_parts, int *bounds);
/* Cuts the host CSR matrix with mx_mg_partition_rows and uploads slab g to GPU g (validated like mx_upload_csr). */
int mx_mg_upload_csr(mx_mg_t mg, int n_rows, int n_cols, int nnz, const int *row_ptr, const int *col_ind,
                     const void *val);
/* Extraction on every slab; per_device (may be NULL) receives n_devices stats.  With more than one GPU and tau != (0,0)
 * the rankings are those of the whole matrix (column counts summed over the GPUs, row counts gathered, one cut):
 * see mx_partition_global. */
int mx_mg_partition(mx_mg_t mg, double tau_c, double tau_r, mx_partition_stats *per_device);
/* on != 0: every slab ranks its own columns and rows (mx_partition per slab) instead of the whole matrix's */
int mx_mg_set_local_ranking(mx_mg_t mg, int on);
int mx_mg_bounds(mx_mg_t mg, int *bounds); /* n_devices + 1 entries */
int mx_mg_devices(mx_mg_t mg);
mx_handle_t mx_mg_handle(mx_mg_t mg, int g); /* the handle of slab g, e.g. for mx_set_dd_executor */
/* y = A x with HOST x (n_cols values) and y (n_rows values): x to every GPU, product + exchange, y from GPU 0. */
int mx_mg_spmv(mx_mg_t mg, const void *x_host, void *y_host);
/* The whole y as GPU g holds it after the last product (every GPU holds the same). */
int mx_mg_download_y(mx_mg_t mg, int g, void *y_host);
/* warm + iters products on device-resident copies of x; *ms_per_spmv = device time of the slowest GPU / iters. */
int mx_mg_spmv_timed(mx_mg_t mg, const void *x_host, int warm, int iters, float *ms_per_spmv);

/* Same with HOST pointers: copies x in, runs, copies y out, synchronises.  (Products enqueued with
 * mx_spmv_host_async that are still in flight are waited for first: they share the staging buffers.) */
int mx_spmv_host(mx_handle_t h, const void *x_host, void *y_host);
/* A sequence of products with HOST pointers, pipelined: the call enqueues "copy x in, multiply, copy y out" and
 * returns; the copy in, the kernels and the copy out of consecutive calls run on three streams over two sets of
 * device buffers, so that the transfers of one product overlap the kernels of its neighbours (PCIe carries both
 * directions at once).  x_host and y_host should be page-locked (pageable memory works but does not overlap) and
 * must stay valid, x unmodified and y unread, until mx_host_sync returns.  Any number of calls may precede one
 * mx_host_sync; results are identical to mx_spmv_host.  Mirrors the reference's per-call cudaMemcpy in / out of
 * every wrapper (src/spmv_kernel/cdSpMV.cu:405-420,483-486), which it issues synchronously around each product. */
int mx_spmv_host_async(mx_handle_t h, const void *x_host, void *y_host);
/* Waits for every product enqueued with mx_spmv_host_async (and for the handle's stream). */
int mx_host_sync(mx_handle_t h);
/* Timing loop on the device: `warm` untimed and `iters` timed repetitions (the reference uses 200 and
 * 4000, src/spmv_kernel/cdSpMV.cu:454-455).  ms_tile / ms_resid time each half alone, as the reference's
 * "MatXtract time = tcTime + cdTime" does (:1564); ms_total times the real back-to-back sequence. */
int mx_spmv_timed(mx_handle_t h, const void *x_dev, void *y_dev, int warm, int iters, float *ms_tile,
                  float *ms_resid, float *ms_total);
/* Structure features of the uploaded matrix: the statistics of its non-zeros-per-row and non-zeros-per-column
 * distributions that the reference's tau predictor takes as input (ML/extract_features.cpp:19-93; CSV columns
 * rowMean ... rowHot90, colMean ... colHot90 of :112-119), computed on the device.  top[] = k-th largest count / mean
 * for k = 1,2,3,4,5,10,50,100,200,300; hot[] = fraction of rows (columns) that holds 10 %, 20 %, ... 90 % of the
 * non-zeros when taken in descending order. */
typedef struct {
    double mean, std_dev;
    long long min, max;
    double p_ratio;
    double top[10];
    double hot[9];
} mx_dist_features;
typedef struct {
    long long rows, cols, nnz;
    mx_dist_features row, col;
} mx_matrix_features;
int mx_features(mx_handle_t h, mx_matrix_features *out);
/* Matrix Market coordinate file -> host CSR with the result of the reference's mmio_allinone
 * (utilities/mmio.cpp:1547-1713: rows in file order, `symmetric`/`hermitian` storage mirrored, pattern = 1, complex =
 * real part, double -> value type in one rounding), parsed by `threads` host threads (<= 0: all).  Host-only: works
 * without a GPU.  row_ptr / col_ind / val are malloc'ed; release them with free() or mx_host_free().  Returns 0 or
 * the reference's codes: -1 cannot open, -2 banner, -4 size line / entries, -5 more than INT_MAX stored entries or
 * out of memory, -3 bad argument. */
int mx_read_matrix_market(const char *path, int dtype, int threads, int *rows, int *cols, int *nnz, int *is_symmetric,
                          int **row_ptr, int **col_ind, void **val);
void mx_host_free(void *p);
/* L2 prefetch distance (in tiles of the CSR kernel; 0 = off) that mx_partition settled on, by timing, for the
 * residual half and for the core-dense block when that runs as CSR.  MX_RESID_PREFETCH=<tiles> in the environment
 * forces a distance.  No counterpart in the reference. */
int mx_csr_prefetch(mx_handle_t h, int *resid_tiles, int *dd_tiles);
/* Measurement aid (no counterpart in the reference): times a pass over the uploaded CSR that streams its column
 * indices and values and gathers x for every non-zero but has no row logic and writes nothing.  *ms is the floor
 * that the matrix's own index pattern sets for a kernel that visits the non-zeros in CSR order on this GPU; an
 * SpMV time is to be read against it when the gathers, not HBM, bound the product. */
int mx_stream_gather_floor(mx_handle_t h, const void *x_dev, int warm, int iters, float *ms);
/* Executor of the core-dense block.  The reference switches between its "dense-unfold" fragment kernel and its
 * "sparse-encode" kernel on nnz and the fragment fill ratio, with thresholds tuned on another GPU
 * (test/test_autotc_spmv.cpp:1507,1518).  Here: MX_DD_TILE = the tensor-core fragment kernel (du_tcspmv_*),
 * MX_DD_SE = the tensor-core sparse-encode kernel (se_tcspmv_*: length-sorted rows in zero-padded 8-row slabs, built
 * on the device), MX_DD_CSR = the CUDA-core CSR kernel on the same entries, MX_DD_AUTO (default) = mx_partition times
 * the block through all three on the device and keeps the fastest (mx_dd_executor_times reports the three times, 0
 * where one was not timed).  The partition arrays do not depend on the choice. */
enum { MX_DD_AUTO = 0, MX_DD_TILE = 1, MX_DD_CSR = 2, MX_DD_SE = 3 };
#define MX_DD_AUTO_FILL 0.25 /* starting guess before the timing: fragments at least this full go to MX_DD_TILE */
int mx_set_dd_executor(mx_handle_t h, int mode);
int mx_dd_executor(mx_handle_t h); /* the one in use: MX_DD_TILE, MX_DD_CSR or MX_DD_SE */
int mx_dd_executor_times(mx_handle_t h, float *ms_tile, float *ms_csr, float *ms_se);
/* Column numbering used for EXECUTION (the partition arrays, and what mx_download_partition returns, always use the
 * reference's numbering).  MX_COLSPACE_PERMUTED: hot columns first in density-rank order, as the reference executes
 * (x is permuted on the device at every product; pays when few hot columns carry much of the matrix).
 * MX_COLSPACE_ORIGINAL: the same entries with their original column ids (x is read directly; keeps the matrix's own
 * locality).  MX_COLSPACE_AUTO (default): mx_partition times both on the device and keeps the faster. */
enum { MX_COLSPACE_AUTO = 0, MX_COLSPACE_PERMUTED = 1, MX_COLSPACE_ORIGINAL = 2 };
int mx_set_column_space(mx_handle_t h, int mode);
/* the one in use; optionally the two timings (ms per product) of the last automatic choice */
int mx_column_space(mx_handle_t h, float *ms_permuted, float *ms_original);
/* Hot-column prefix of x in shared memory.  In the permuted numbering the first dCols entries of x are the densest
 * columns in rank order (what tau_c selects, test/test_autotc_spmv.cpp:1122-1141); when the CSR kernels run in that
 * numbering, a persistent variant copies as long a prefix of them as fits one SM's shared memory (1-D bulk copies)
 * and serves every gather of those columns from there instead of L1 / L2.  MX_HOT_AUTO (default): mx_partition
 * times the product with and without it and keeps the faster; MX_HOT_OFF / MX_HOT_ON force it.  mx_hot_prefix reports
 * the prefix length in use (0 = off) and the two timings of the last choice.  The partition arrays do not depend on
 * it.  The reference gathers x from global memory in every kernel (src/spmv_kernel/cdSpMV.cu:282-300). */
enum { MX_HOT_AUTO = 0, MX_HOT_OFF = 1, MX_HOT_ON = 2 };
int mx_set_hot_prefix(mx_handle_t h, int mode);
int mx_hot_prefix(mx_handle_t h, int *hot_cols, float *ms_with, float *ms_without);
/* Column-slab execution of the plain CSR product (tau = (0,0)) for a matrix whose x is far larger than the L2 cache.
 * A CSR-ordered kernel then pays one 64-byte DRAM burst per gathered x value.  The matrix is split into its BAND (the
 * entries within 65,536 columns of the diagonal: one CSR pass over all rows, whose gathers walk x almost
 * sequentially) and its FAR entries, cut into vertical slabs, each stored as its own CSR over its non-empty rows and
 * multiplied in a pass that adds into y while gathering from an x range that L2 holds.  count = -1 (default): when x
 * exceeds L2, mx_partition builds the slabs for x ranges of 96 / 64 / 32 MB, times the product each way and keeps the
 * fastest; 0 = never; k >= 2 = always k slabs.  FP64 only (the passes accumulate in the value type); rows must have
 * ascending column ids (otherwise the plain kernel stays).  mx_column_slabs reports the slab count in use (0 = plain
 * kernel) and the timings.  For a row slab of a larger square matrix, mx_set_row_offset (before mx_partition) tells
 * where its diagonal lies; mx_spmv_peers then runs the far passes first, accumulating locally, and the band pass
 * last, storing the finished rows into every GPU's y from its epilogue.  The reference has one CSR kernel over the
 * whole matrix (src/spmv_kernel/cdSpMV.cu:395-491). */
int mx_set_row_offset(mx_handle_t h, long long first_global_row);
int mx_set_column_slabs(mx_handle_t h, int count);
int mx_column_slabs(mx_handle_t h, int *count, float *ms_plain, float *ms_slabbed);
/* Number of kernel launches one mx_spmv issues for the current matrix / partition. */
int mx_spmv_launches(mx_handle_t h);
/* Device error word of the last kernels (0 = none). */
int mx_device_error(mx_handle_t h, int *err);

/* ---- stateless mirrors of include/MatXtract.h (host pointers in and out, synchronous) -------------- */
/* cdspmv (include/MatXtract.h:3-5, src/spmv_kernel/cdSpMV.cu:395-491): y += A x on the CUDA cores; y is in/out. */
int mx_cdspmv(int dtype, const void *csrVal, const int *csrRowPtr, const int *csrColInd, const void *x, void *y,
              int rowA, int colA, int nnzA, int warm, int iters, double *ms_per_spmv, double *pre_ms);
/* du_tcspmv_fp64 / du_tcspmv_fp16_v2 (include/MatXtract.h:7-9,26-28): fragment-format SpMV on the tensor cores.
 * FP64: y is in/out (the reference preloads it and adds, du_tcSpMV_fp64.cu:296,334); FP16: y is overwritten
 * (du_tcSpMV_fp16_v2.cu:150,187). */
int mx_du_tcspmv(int dtype, const int *chunkPtr, const int *fragPtr, const void *fragBit, const void *tcVal,
                 int n_vals, const int *sparse_AToX_index, const void *x, void *y, int dRows, int dCols, int warm,
                 int iters, double *ms_per_spmv);
/* se_tcspmv_fp64 / se_tcspmv_fp16 (include/MatXtract.h:14-15,30-31; src/spmv_kernel/se_tcSpMV_fp64.cu:496-1496):
 * SpMV of the core-dense block given as CSR through the sparse-encode layout, which is built on the device.  NUM =
 * warps per CTA, threshold = fill an 8-row slab needs to be stored for the tensor cores (the rest of its rows goes to
 * the CUDA-core tail), block_longest = length from which a row is split across work units; values <= 0 (threshold
 * < 0) select the reference's defaults 4 / 0.75 / 256 (test/test_autotc_spmv.cpp:1501-1503).  y[i] is the result for
 * input row order_rid[i] (rows sorted by length, longest first); the caller un-permutes (:1542). */
int mx_se_tcspmv(int dtype, const void *csrVal, const int *csrRowPtr, const int *csrColIdx, const void *x, void *y,
                 int *order_rid, int rowA, int colA, int nnzA, int NUM, double threshold, int block_longest, int warm,
                 int iters, double *ms_per_spmv);

/* ---- allocation-free CSR SpMV (no counterpart in the reference: every reference wrapper allocates) ---------- */
/* y = A x for a CSR matrix that is already on the device, for callers that must not allocate device memory at call
 * time: code running inside a fixed memory arena, a real-time loop that may not block on the driver's allocator, a
 * process whose memory budget was fixed at start-up.  The call performs no cudaMalloc / cudaFree and uses no library
 * routine that allocates; all pointers are DEVICE pointers supplied by the caller (y is overwritten).  The scratch the
 * kernels need lives in a fixed array inside the library image (MX_STATIC_SCRATCH_BYTES per GPU, held until the
 * process exits), which bounds the problem: at most MX_STATIC_MAX_ROWS rows and MX_STATIC_MAX_NNZ non-zeros, else
 * MX_ERR_TOO_LARGE.  All calls share that array: do not let two calls overlap on the GPU (they would race on it).
 * The call synchronises `stream` once (it reads one count back).  The first call on a device looks up the array's
 * device address; make that first call before starting any stream capture.  The looked-up address is kept for the
 * life of the process and is not valid after a cudaDeviceReset of that device.  `stream` is a cudaStream_t (NULL =
 * the default stream). */
#define MX_STATIC_MAX_ROWS (1 << 20)
#define MX_STATIC_MAX_NNZ (1 << 26)
#define MX_STATIC_SCRATCH_BYTES (24u << 20)
int mx_csr_spmv_static(int dtype, int n_rows, int n_cols, int nnz, const int *row_ptr_dev, const int *col_ind_dev,
                       const void *val_dev, const void *x_dev, void *y_dev, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* MX_CAPI_H */
