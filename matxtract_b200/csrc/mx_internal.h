// Internal declarations shared by the translation units of libmatxtract_b200.so.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

#include "mx_capi.h"

namespace mx {

// ------------------------------------------------------------------------------------------------
// Residual CSR kernel geometry: a tile is RESID_THREADS * IPT consecutive non-zeros.
#ifndef MX_RESID_THREADS
#define MX_RESID_THREADS 128
#endif
#ifndef MX_RESID_IPT_FP64
#define MX_RESID_IPT_FP64 16
#endif
#ifndef MX_RESID_IPT_FP16
#define MX_RESID_IPT_FP16 16
#endif
#ifndef MX_RESID_MINBLOCKS_FP64
#define MX_RESID_MINBLOCKS_FP64 6  // 80 registers per thread: 16 doubles of values + 16 products in flight
#endif
#ifndef MX_RESID_MINBLOCKS_FP16
#define MX_RESID_MINBLOCKS_FP16 (1024 / MX_RESID_THREADS)
#endif
constexpr int RESID_THREADS = MX_RESID_THREADS;
template <typename V>
struct ResidCfg;
template <>
struct ResidCfg<double> {
    static constexpr int IPT = MX_RESID_IPT_FP64;  // A/B on the block matrix: 8 -> 16 raises 4.7 to 5.5 TB/s
    static constexpr int MINBLOCKS = MX_RESID_MINBLOCKS_FP64;
};
template <>
struct ResidCfg<__half> {
    static constexpr int IPT = MX_RESID_IPT_FP16;
    static constexpr int MINBLOCKS = MX_RESID_MINBLOCKS_FP16;
};

// Device error word bits: DEVERR_INPUT = an uploaded matrix failed the index check; DEVERR_TILE_RANGE = a bounded wait
// of the tile kernel on its bulk copies ran out.
enum : int { DEVERR_INPUT = 1, DEVERR_TILE_RANGE = 2 };

// Plan + buffers of the residual CSR kernel for one CSR matrix that lives on the device.
struct ResidPlan {
    int n_rows = 0, n_cols = 0, nnz = 0;
    const int *row_ptr = nullptr;  // [n_rows+1]
    const int *col_ind = nullptr;  // [nnz]
    const void *val = nullptr;     // [nnz]
    int tile_nnz = 0, num_tiles = 0;
    int prefetch_tiles = 0;          // L2 prefetch distance of the CSR kernel in tiles (0: off)
    int hot_cols = 0;                // > 0: x[0, hot_cols) is the hot-column prefix of a permuted x; the persistent kernel
                                     // keeps it in shared memory (a multiple of 16 bytes of values)
    int *dev_err = nullptr;          // device error word for bounded waits (may be null)
    bool dense_row_ends = false;     // a tile closes hundreds of rows: the plain product marks row ends with bytes and
                                     // a scan instead of shared-memory atomics (the column-slab passes)
    int m_rows = 0, n_empty = 0;     // non-empty / empty rows
    const int *c_ptr = nullptr;      // [m_rows+1] row pointers of the non-empty rows (= row_ptr when none is empty)
    int *c_ptr_own = nullptr;        // storage of c_ptr when it is not row_ptr
    int *nz_row = nullptr;           // [m_rows] k-th non-empty row -> row index (null: identity)
    int *empty_row = nullptr;        // [n_empty]
    int *tile_row = nullptr;   // [num_tiles+1] non-empty rows whose end lies at or before the tile's first non-zero
    void *carry = nullptr;     // [num_tiles] accumulate-type partial of the tile's unfinished last row
    void *head = nullptr;      // [num_tiles] accumulate-type partial of a first row that began in an earlier tile
};

// Column-slab execution of one CSR matrix (col_slabs.cu): the band around the diagonal as one CSR over all rows, the
// far entries cut into vertical slabs of `width` columns, each a CSR of its own over its non-empty rows and multiplied
// in a pass of its own, so that the x range a pass gathers from stays resident in L2.  A pass writes one partial sum
// per non-empty row of its slab, densely; a last kernel adds every row's partial sums in slab order.  Owned.
constexpr int COMBINE_ROWS = 2048;  // rows whose sums one CTA of the combining kernel holds in shared memory
struct ColSlabs {
    int count = 0, width = 0, halo = 0;
    long long row_offset = 0;    // global index of the matrix's first row (a row slab of a larger square matrix)
    bool has_band = false;       // row slabs only: the entries near the diagonal as a pass of their own
    ResidPlan near;              // the band; its arrays:
    int *near_row_ptr = nullptr, *near_col = nullptr;
    void *near_val = nullptr;
    ResidPlan *plans = nullptr;  // [count] host array; every plan owns its row tables, the struct owns col/val
    int **col = nullptr;         // [count] host array of device pointers
    void **val = nullptr;        // [count]
    void **part = nullptr;       // [count] host array: partial sums (value type) of slab k's non-empty rows, in row order
    unsigned short **row_in_block = nullptr;  // [count] host array: for slab k's i-th non-empty row, its index inside
                                              // its block of COMBINE_ROWS consecutive rows
    int *block_base = nullptr;   // [ceil(n_rows / COMBINE_ROWS) + 1][count]: non-empty rows of slab k before the block
    int n_rows = 0;
    // the band once more as `band_chunks` row ranges of equal non-zero count, each with a plan of its own (views into
    // near_col / near_val with rebased row pointers): through mx_spmv_peers the ranges are multiplied one after the
    // other and every finished range is copied to the other GPUs from a second stream while the next is computed
    int band_chunks = 0;
    ResidPlan *chunk_plans = nullptr;  // [band_chunks]
    int *chunk_row_ptr = nullptr;      // storage of the rebased row pointers
    int *chunk_rows = nullptr;         // host [band_chunks + 1] row boundaries
    static constexpr int SEND_STREAMS = 2;  // concurrent engine copies to one destination (or stream 0: the copy kernel)
    cudaStream_t send_stream[SEND_STREAMS] = {};
    cudaEvent_t send_done[SEND_STREAMS] = {};  // a stream's copies have all been issued and finished
    cudaEvent_t *chunk_done = nullptr;         // [band_chunks]: the range's rows are final
};

// Plain CSR on the device (non-owning view).
struct CsrDev {
    int n_rows = 0, n_cols = 0, nnz = 0;
    const int *row_ptr = nullptr;
    const int *col_ind = nullptr;
    const void *val = nullptr;
};

// Tile-format matrix on the device (layout of the reference's fragment format).
struct TileArrays {
    int dRows = 0, dCols = 0, chunkNum = 0, totalFrags = 0, nvals = 0;
    int *chunkPtr = nullptr;  // [chunkNum+1]
    int *AToX = nullptr;      // [totalFrags*K]
    int *fragPtr = nullptr;   // [totalFrags+1]
    void *fragBit = nullptr;  // [totalFrags] uint32 / uint64
    void *tcVal = nullptr;    // [nvals]
};

// Execution plan of the tile kernel over a TileArrays: a panel with many fragments is cut into several
// work segments.
struct TilePlan {
    TileArrays A;  // view, not owned
    int numSegs = 0, numMultiSegs = 0;
    bool allFull = false;           // every fragment completely filled: the streaming kernel (no bitmap decode) applies
    bool useFull = false;           // ... and is in use (the plan-time tuner times it against the staged kernel)
    int *segPanel = nullptr;        // [numSegs]
    int *segBegin = nullptr;        // [numSegs] fragment range of segment s = [segBegin[s], segEnd[s])
    int *segEnd = nullptr;          // [numSegs]
    int *segSlot = nullptr;         // [numSegs] slot in `partial` (-1: the panel has one segment, write directly)
    int *panelFirstSeg = nullptr;   // [chunkNum+1]
    void *partial = nullptr;        // [numMultiSegs][8] accumulate-type partial sums
    unsigned *panelCount = nullptr; // [chunkNum] arrival counters of split panels (self-resetting)
    // CTAs own runs of consecutive segments sized by the bytes they stage in shared memory
    int numCtas = 0, stageBytes = 0;  // grid size; largest stage (dynamic shared memory per CTA)
    void *ctaDesc = nullptr;          // [numCtas] descriptors
    void *segDesc = nullptr;          // [numSegs] packed {panel, first fragment, end fragment, slot}
};

// Sparse-encode layout of a CSR block (se_spmv.cu): rows sorted by length, 8-row blocks of zero-padded 8xK slabs for
// the tensor cores, irregular tails as CSR.  Owned.
struct SePlan {
    int n_rows = 0, n_cols = 0, nnz = 0;
    // the reference's tuning knobs (test/test_autotc_spmv.cpp:1501-1503): warps per CTA, the fill a slab needs to be
    // stored for the tensor cores, and the length from which a row is "long"
    int warps_per_cta = 4;
    double threshold = 0.75;
    int block_longest = 256;
    int nLong = 0, numBlocks = 0, numSlabs = 0, numUnits = 0, tailNnz = 0;
    int *order = nullptr;     // [n_rows] sorted position -> input row
    int *outRow = nullptr;    // [n_rows] sorted position -> index the row's result is written to
    int *slabPtr = nullptr;   // [numBlocks+1]
    int *unitPtr = nullptr;   // [numBlocks+1] work units (<= 64 slabs each) of every block
    void *unitDesc = nullptr; // [numUnits] int4 {block, first slab, end slab, 0}
    void *slabVal = nullptr;  // [numSlabs * 8K] values in MMA operand order
    int *slabCol = nullptr;   // [numSlabs * 8K] their column ids
    int *tailPtr = nullptr;   // [n_rows+1] irregular tails, by sorted position
    void *tailVal = nullptr;
    int *tailCol = nullptr;
    void *partial = nullptr;  // [numUnits][8] accumulate-type diagonal sums
};

// Everything the extraction produces, on the device (owned).
struct PartArrays {
    int *xperm = nullptr;        // [n_cols]
    int *rId = nullptr;          // [dRows]
    uint32_t *hotmask = nullptr; // [ceil(n_rows/32)] bit r set when row r is hot
    int *rowPtr_dd = nullptr, *colInd_dd = nullptr;
    void *val_dd = nullptr;
    int *rowPtr_CD = nullptr, *colInd_CD = nullptr;
    void *val_CD = nullptr;
    TileArrays tiles;
};

// ---- launchers (each returns the cudaError_t of its launches) ----
cudaError_t resid_plan_build(int dtype, ResidPlan &plan, cudaStream_t s);
cudaError_t resid_plan_finish(int dtype, ResidPlan &plan, cudaStream_t s);
void resid_plan_free(ResidPlan &plan, cudaStream_t s);
// y[r] = sum_r (+ y_in[r] when accumulate) (+ ytile[r] for rows flagged in hotmask).  ytile is of the
// accumulate type (float for FP16, double for FP64); hotmask has one bit per row.
// chained: the launch directly follows, on the same stream, the CSR launches of the same product's core-dense block
// (which do not write x); the kernel's first wave may then start while they drain.  Measured: -9 % on the power-law
// benchmark shape.  Behind the tensor-core tile kernel the same overlap costs 13 %, so it is not used there.
cudaError_t resid_spmv(int dtype, const ResidPlan &plan, const void *x, void *y, const void *ytile,
                       const uint32_t *hotmask, bool accumulate, cudaStream_t s, bool chained = false);
// carrier[row_map[r]] = sum_r in the accumulate type: runs the core-dense block as CSR (low-fill dispatch)
cudaError_t resid_spmv_to_carrier(int dtype, const ResidPlan &plan, const void *x, void *carrier, const int *row_map,
                                  cudaStream_t s);
// y_peer[g][row_offset + r] = row r for every g < n_peers (peer-mapped full-length y of every GPU): fused all-gather.
// mc_y (optional): the NVLink multicast address of the same buffers; rows then go out as one multicast store each.
cudaError_t resid_spmv_peers(int dtype, const ResidPlan &plan, const void *x, void *const *peers, int n_peers,
                             long long row_offset, const void *ytile, const uint32_t *hotmask, cudaStream_t s,
                             bool chained = false, void *mc_y = nullptr);
int resid_launches(const ResidPlan &plan);
// largest hot-column prefix (columns, rounded down to 16 bytes of values) the persistent CSR kernel can hold in shared
// memory for this value type; 0 when `d_cols` is too small to be worth a persistent launch
int resid_hot_cols_budget(int dtype, int d_cols);
// Splits A (rows with ascending column ids) into its band and `count` column slabs of far entries; row_offset = global
// index of A's first row; *status = MX_ERR_INVALID when a row is not sorted.
cudaError_t col_slabs_build(int dtype, const CsrDev &A, int count, long long row_offset, ColSlabs &out, int *status,
                            cudaStream_t s);
void col_slabs_free(ColSlabs &S, cudaStream_t s);
int col_slabs_launches(const ColSlabs &S);
// y = A x (value type): the band pass writes every row (without a band y is cleared), every slab adds its part.
cudaError_t col_slabs_spmv(int dtype, const ColSlabs &S, const void *x, void *y, size_t y_bytes, cudaStream_t s);
// one GPU's share of a row-partitioned product: the far passes' sums are combined into this GPU's rows of
// peers[self], the band follows in row ranges, and every finished range is sent to the other GPUs' buffers from
// other streams; on return the stream s is ordered after the last send
cudaError_t col_slabs_spmv_peers(int dtype, const ColSlabs &S, const void *x, void *const *peers, int n_peers, int self,
                                 long long row_offset, cudaStream_t s);

// rows [row_offset, row_offset + n_rows) of peers[self] -> the same rows of every other buffer (16-byte stores over
// NVLink by a copy kernel on a third of the SMs; byte stores for ragged ends)
cudaError_t peer_push_rows(int dtype, void *const *peers, int n_peers, int self, long long row_offset, long long n_rows,
                           cudaStream_t s);
cudaError_t tile_plan_build(int dtype, TilePlan &plan, cudaStream_t s);
void tile_plan_free(TilePlan &plan, cudaStream_t s);
// out[row_map ? row_map[i] : i] (accumulate type when out_is_acc, else value type) = tile row i result.
cudaError_t tile_spmv(int dtype, const TilePlan &plan, const void *x_d, void *out, const int *row_map,
                      bool out_is_acc, bool accumulate, int *dev_err, cudaStream_t s);
int tile_launches(const TilePlan &plan);

// Builds the sparse-encode layout of the CSR block (rowPtr, colInd, val) with P.n_rows / n_cols / nnz and the knobs
// set; row_map (may be null) sends the result of input row i to out[row_map[i]] instead of its sorted position.
cudaError_t se_plan_build(int dtype, SePlan &P, const int *rowPtr, const int *colInd, const void *val,
                          const int *row_map, cudaStream_t s);
void se_plan_free(SePlan &P, cudaStream_t s);
// out[outRow[r]] (accumulate type when out_is_acc, else value type) = result of sorted row r
cudaError_t se_spmv(int dtype, const SePlan &P, const void *x, void *out, bool out_is_acc, bool accumulate,
                    cudaStream_t s);
int se_launches(const SePlan &P);

// Rankings of a matrix whose rows are spread over several GPUs (see partition.cu).
struct GlobalRanking {
    const int *col_counts = nullptr;  // [n_cols] column counts of the whole matrix (device)
    long long nnz = 0;                // its non-zero count
    bool has_row_cut = false;         // hot rows = those above the whole matrix's row cut:
    int row_cut_count = 0;            //   count of the last hot row of the whole matrix's ranking
    long long row_cut_index = 0;      //   and its (global) row index
    long long row_offset = 0;         // global index of this slab's first row
};
cudaError_t partition_run(int dtype, const CsrDev &A, float tau_c, float tau_r, PartArrays &P, mx_partition_stats &st,
                          int *status, cudaStream_t s, const GlobalRanking *G = nullptr);
// per-row count of entries inside the hot columns (the tau_c cut of G's or the slab's own column counts)
cudaError_t partition_row_counts(int dtype, const CsrDev &A, float tau_c, const GlobalRanking *G, int *row_counts,
                                 int *status, cudaStream_t s);
cudaError_t column_counts(const CsrDev &A, int *counts, cudaStream_t s);
cudaError_t rank_cut(const int *counts, int n, int threshold, long long out[4], cudaStream_t s);
cudaError_t tiles_from_dd(int dtype, int dRows, int nnzRowD, const int *rowPtr_dd, const int *colInd_dd,
                          const void *val_dd, TileArrays &T, int *status, cudaStream_t s);
// sets DEVERR_INPUT in *dev_err when row_ptr decreases anywhere or a column index is outside [0, n_cols)
cudaError_t validate_csr(int n_rows, int n_cols, int nnz, const int *row_ptr, const int *col_ind, int *dev_err,
                         cudaStream_t s);
// MX_OK when `total_frags` fragments of K columns can be indexed with int32 (fragment ids and x-index slots)
int fragment_count_status(long long total_frags, int K);
// bit r set for every r in rId (a stored partition carries rId, not the bitmap)
cudaError_t hotmask_from_rid(const int *rId, int dRows, int n_rows, uint32_t **hotmask, cudaStream_t s);
// every buffer of the library comes from the stream-ordered pool: allocate and free on the stream that uses it
void part_arrays_free(PartArrays &P, cudaStream_t s);
void tile_arrays_free(TileArrays &T, cudaStream_t s);

// out[i] = map[in[i]]
cudaError_t map_indices(const int *in, const int *map, int *out, long long n, cudaStream_t s);
// x_perm[i] = x[perm[i]]
cudaError_t matrix_features(const CsrDev &A, mx_matrix_features &out, cudaStream_t s);
cudaError_t stream_gather_pass(int dtype, const int *col_ind, const void *val, const void *x, float *sink, int nnz,
                               cudaStream_t s);
cudaError_t gather_vector(int dtype, const void *x, const int *perm, void *x_perm, int n, cudaStream_t s);

inline size_t val_bytes(int dtype) { return dtype == MX_FP64 ? 8 : 2; }
inline size_t acc_bytes(int dtype) { return dtype == MX_FP64 ? 8 : 4; }
inline int frag_k(int dtype) { return dtype == MX_FP64 ? 4 : 8; }
inline size_t bit_bytes(int dtype) { return dtype == MX_FP64 ? 4 : 8; }

}  // namespace mx
