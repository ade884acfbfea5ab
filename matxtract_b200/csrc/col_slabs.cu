// Column-slab execution of a CSR SpMV whose x does not fit the L2 cache.
//
// A CSR-ordered kernel gathers x[col] for every non-zero.  When x is much larger than L2 (a 64M-column FP64 vector is
// 512 MB) and the columns of a row are spread over the whole range, every such gather is a DRAM access that moves a
// whole 64-byte burst for 8 useful bytes: measured on the 1e9-non-zero power-law matrix, the kernel moves 3-4x the
// matrix's own bytes.  Here the matrix is split in two:
//   * the BAND: the entries of every row whose column lies within COL_SLAB_HALO of the row's own index.  Their
//     gathers walk x almost sequentially whatever its size, so the band is one ordinary CSR pass over all rows;
//   * the FAR entries, cut into vertical slabs of `width` columns, each stored as its own CSR over its non-empty
//     rows.  One pass per slab streams that slab's entries and gathers from an x range that stays in L2.
// A pass is the ordinary CSR kernel (resid_kernel) over the slab's NON-EMPTY rows as if they were a dense row space:
// it writes one partial sum per such row into a buffer of its own, sequentially, and reads nothing but the slab and
// x.  (Adding into y instead made every pass read and write the whole of y, a sector at a time, through a row-index
// table: on the 1e9-non-zero shape 8 GB of the product's 28 GB of DRAM traffic.)  A last kernel (k_combine) adds every
// row's partial sums in slab order - the same order of additions as accumulating pass by pass, without atomics and
// bit-reproducible: a CTA holds the sums of a block of rows in shared memory and streams, slab by slab, the block's
// contiguous share of the slab's partial sums with a 2-byte row index each.  A whole (square) matrix has no band: its
// near-diagonal entries stay in the slabs.  One GPU's share of a row-partitioned matrix has one: the combined far
// sums land in its own rows, the band follows in row ranges and every finished range is sent to the other GPUs from
// other streams, so that the exchange overlaps the band, about half of the work.
// The reference has no counterpart: it runs one CSR kernel over the whole matrix (src/spmv_kernel/cdSpMV.cu:395-491).
#include <algorithm>

#include "device_prims.cuh"
#include "mx_internal.h"

namespace mx {
namespace {

#define CS_TRY(call)                      \
    do {                                  \
        cudaError_t e_ = (call);          \
        if (e_ != cudaSuccess) return e_; \
    } while (0)

inline int nblk(long long n, int b = 256) { return (int)((n + b - 1) / b); }

constexpr int COL_SLAB_HALO = 1 << 16;  // columns on either side of the diagonal that count as the band
constexpr int MAX_COL_SLABS = 64;       // mx_set_column_slabs accepts at most this many
constexpr int BAND_CHUNKS = 4;          // row ranges of the band whose sends overlap the next range's kernels (2 GPUs,
                                        // 2.79 ms of kernels: 2 ranges 3.02 ms, 4: 2.97, 8: 3.01)

// first position in [lo, hi) whose column is >= c
__device__ __forceinline__ int lower_col(const int *__restrict__ col, int lo, int hi, int c) {
    while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (__ldg(col + mid) < c)
            lo = mid + 1;
        else
            hi = mid;
    }
    return lo;
}

__global__ void k_rows_sorted(const int *__restrict__ row_ptr, const int *__restrict__ col, int n, int *__restrict__ bad) {
    const int r = (int)(((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5), lane = threadIdx.x & 31;
    if (r >= n) return;
    bool b = false;
    for (int e = row_ptr[r] + 1 + lane, end = row_ptr[r + 1]; e < end; e += 32) b |= __ldg(col + e) <= __ldg(col + e - 1);
    if (__any_sync(0xffffffffu, b) && lane == 0) *bad = 1;
}

// the band of every row: entries whose column lies within `halo` of the row's own (global) index
__global__ void k_near_ranges(const int *__restrict__ row_ptr, const int *__restrict__ col, int n, long long row_offset,
                              int halo, int *__restrict__ nlo, int *__restrict__ nlen) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r > n) return;
    int a = 0, l = 0;
    if (r < n) {
        const int b = row_ptr[r], e = row_ptr[r + 1];
        const long long g = row_offset + r;
        const long long c0 = g - halo, c1 = g + halo + 1;  // [c0, c1)
        a = lower_col(col, b, e, (int)max(c0, 0LL));
        l = lower_col(col, a, e, (int)min(c1, 2147483647LL)) - a;
    }
    nlo[r] = a;
    nlen[r] = l;
}

// the part of every row that falls into columns [c0, c1) and is NOT in the row's band: at most two ranges of the
// (sorted) row, [lo1, lo1 + len1) left of the band and [lo2, lo2 + len2) right of it
__global__ void k_far_ranges(const int *__restrict__ row_ptr, const int *__restrict__ col, const int *__restrict__ nlo,
                             const int *__restrict__ nlen, int n, int c0, int c1, int *__restrict__ lo1,
                             int *__restrict__ len1, int *__restrict__ lo2, int *__restrict__ len2,
                             int *__restrict__ len, int *__restrict__ flag) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r > n) return;
    int a1 = 0, l1 = 0, a2 = 0, l2 = 0;
    if (r < n) {
        const int b = row_ptr[r], e = row_ptr[r + 1];
        const int p0 = lower_col(col, b, e, c0), p1 = lower_col(col, p0, e, c1);
        const int w0 = nlo[r], w1 = w0 + nlen[r];
        a1 = p0;
        l1 = max(0, min(p1, w0) - p0);
        a2 = max(p0, w1);
        l2 = max(0, p1 - a2);
    }
    lo1[r] = a1, len1[r] = l1, lo2[r] = a2, len2[r] = l2;
    len[r] = l1 + l2;
    flag[r] = l1 + l2 > 0;
}

// copies entries [a, a + l) of the source arrays to [o, o + l): short ranges by their lane, long ones by the warp
template <typename V>
__device__ __forceinline__ void copy_ranges(const int *__restrict__ col, const V *__restrict__ val, int a, int l, int o,
                                            int lane, int *__restrict__ ocol, V *__restrict__ oval) {
    if (l > 0 && l < 32)
        for (int j = 0; j < l; ++j) {
            ocol[o + j] = __ldg(col + a + j);
            oval[o + j] = val[a + j];
        }
    unsigned big = __ballot_sync(0xffffffffu, l >= 32);
    while (big) {
        const int src = __ffs(big) - 1;
        big &= big - 1;
        const int sa = __shfl_sync(0xffffffffu, a, src), sl = __shfl_sync(0xffffffffu, l, src),
                  so = __shfl_sync(0xffffffffu, o, src);
        for (int j = lane; j < sl; j += 32) {
            ocol[so + j] = __ldg(col + sa + j);
            oval[so + j] = val[sa + j];
        }
    }
}

// one lane per row (a warp per 32 rows): the row's band -> the near matrix (row pointers = off)
template <typename V>
__global__ void k_near_copy(const int *__restrict__ col, const V *__restrict__ val, const int *__restrict__ nlo,
                            const int *__restrict__ nlen, const int *__restrict__ off, int n, int *__restrict__ ocol,
                            V *__restrict__ oval) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x, lane = threadIdx.x & 31;
    int a = 0, l = 0, o = 0;
    if (r < n) a = nlo[r], l = nlen[r], o = off[r];
    copy_ranges<V>(col, val, a, l, o, lane, ocol, oval);
}

// one lane per row: the row's far entries inside the slab -> the slab's CSR over its non-empty rows
template <typename V>
__global__ void k_far_copy(const int *__restrict__ col, const V *__restrict__ val, const int *__restrict__ lo1,
                           const int *__restrict__ len1, const int *__restrict__ lo2, const int *__restrict__ len2,
                           const int *__restrict__ pos, const int *__restrict__ off, int n, int m_rows, int nnz_slab,
                           int *__restrict__ c_ptr, int *__restrict__ ocol,
                           V *__restrict__ oval) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x, lane = threadIdx.x & 31;
    int a1 = 0, l1 = 0, a2 = 0, l2 = 0, o = 0;
    if (r < n) {
        a1 = lo1[r], l1 = len1[r], a2 = lo2[r], l2 = len2[r], o = off[r];
        if (l1 + l2 > 0) {
            const int k = pos[r];
            c_ptr[k] = o;
        }
    }
    if (r == 0) c_ptr[m_rows] = nnz_slab;
    copy_ranges<V>(col, val, a1, l1, o, lane, ocol, oval);
    copy_ranges<V>(col, val, a2, l2, o + l1, lane, ocol, oval);
}

// row boundaries that cut the band into `chunks` ranges of equal non-zero count: bounds[c] = lower_bound(rp, c*nnz/chunks)
__global__ void k_chunk_bounds(const int *__restrict__ rp, int n, int chunks, int *__restrict__ bounds) {
    const int c = threadIdx.x;
    if (c > chunks) return;
    const long long target = (long long)rp[n] * c / chunks;
    int lo = 0, hi = n;
    while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (rp[mid] < target)
            lo = mid + 1;
        else
            hi = mid;
    }
    bounds[c] = c == chunks ? n : lo;
    bounds[chunks + 1 + c] = rp[c == chunks ? n : lo];
}
// out[i] = rp[r0 + i] - rp[r0], i in [0, len]
__global__ void k_rebase(const int *__restrict__ rp, int r0, int len, int *__restrict__ out) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i <= len) out[i] = rp[r0 + i] - rp[r0];
}

// slab k of the combining kernel's tables: flag[r] = the row has entries in the slab, pos = exclusive scan of flag.
// The i-th non-empty row of the slab records where it sits inside its block of COMBINE_ROWS rows; every block records
// how many of the slab's non-empty rows precede it (one entry more than blocks: the total).
__global__ void k_row_in_block(const int *__restrict__ flag, const int *__restrict__ pos, int n, int k, int count,
                               unsigned short *__restrict__ row_in_block, int *__restrict__ block_base) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r > n) return;
    if (r < n && flag[r]) row_in_block[pos[r]] = (unsigned short)(r % COMBINE_ROWS);
    if (r % COMBINE_ROWS == 0 || r == n) block_base[(size_t)((r + COMBINE_ROWS - 1) / COMBINE_ROWS) * count + k] = pos[r];
}

// y[r] = sum over the slabs, in slab order, of the partial sum of row r (where the row has entries in the slab).
// A CTA owns COMBINE_ROWS consecutive rows and keeps their sums in shared memory.  Slab by slab it streams the block's
// share of the slab's partial sums - a contiguous range, because a pass writes them in row order - together with each
// one's row index inside the block (2 bytes) and adds it to that row's sum; a row occurs at most once per slab, so
// the adds of one slab never collide, and a barrier separates the slabs: every row adds its partial sums in slab
// order, the same additions in the same order as accumulating pass by pass, without atomics.  Coalesced loads, about
// eight instructions per partial sum.  (First version: one lane per row, a presence bit per (row, slab) and a warp
// ballot per slab to find each row's partial sum: 180-350 instructions per 32 rows, issue-bound, 0.95 ms of a 5.5 ms
// product on the 1e9-non-zero shape with 12 slabs.  Column slabs exist for FP64 only: the passes and this kernel add
// in the value type.)
struct PartTable {
    const double *p[MAX_COL_SLABS];          // partial sums of every slab (kernel parameters: constant bank)
    const unsigned short *row[MAX_COL_SLABS]; // their rows' indices inside their blocks
};
__global__ void __launch_bounds__(256) k_combine(const __grid_constant__ PartTable part,
                                                 const int *__restrict__ block_base, int count, int n,
                                                 double *__restrict__ y) {
    __shared__ double acc[COMBINE_ROWS];
    const int tid = threadIdx.x;
    const long long r0 = (long long)blockIdx.x * COMBINE_ROWS;
    for (int i = tid; i < COMBINE_ROWS; i += 256) acc[i] = 0.0;
    const int *bb = block_base + (size_t)blockIdx.x * count;
    __syncthreads();
    for (int k = 0; k < count; ++k) {
        const int lo = __ldg(bb + k), len = __ldg(bb + count + k) - lo;
        const double *__restrict__ p = part.p[k] + lo;
        const unsigned short *__restrict__ row = part.row[k] + lo;
        int i = tid;
        for (; i + 768 < len; i += 1024) {  // four independent loads in flight per thread
            const double v0 = __ldg(p + i), v1 = __ldg(p + i + 256), v2 = __ldg(p + i + 512), v3 = __ldg(p + i + 768);
            const int q0 = __ldg(row + i), q1 = __ldg(row + i + 256), q2 = __ldg(row + i + 512), q3 = __ldg(row + i + 768);
            acc[q0] += v0, acc[q1] += v1, acc[q2] += v2, acc[q3] += v3;
        }
        for (; i < len; i += 256) acc[__ldg(row + i)] += __ldg(p + i);
        __syncthreads();
    }
    for (int i = tid; i < COMBINE_ROWS && r0 + i < n; i += 256) y[r0 + i] = acc[i];
}

template <typename V>
cudaError_t build_t(const CsrDev &A, int count, long long row_offset, ColSlabs &out, int *status, cudaStream_t s) {
    constexpr int dtype = sizeof(V) == 8 ? MX_FP64 : MX_FP16;
    const int n = A.n_rows;
    const size_t n1 = (size_t)n + 1;
    *status = MX_OK;
    TempBuf tmp;
    int *nlo = nullptr, *nlen = nullptr, *lo1 = nullptr, *len1 = nullptr, *lo2 = nullptr, *len2 = nullptr, *len = nullptr,
        *flag = nullptr, *pos = nullptr, *off = nullptr, *bad = nullptr;
    struct Guard {
        cudaStream_t s;
        int **p[11];
        ~Guard() {
            for (int **q : p)
                if (*q) cudaFreeAsync(*q, s);
        }
    } guard{s, {&nlo, &nlen, &lo1, &len1, &lo2, &len2, &len, &flag, &pos, &off, &bad}};
    CS_TRY(cudaMallocAsync(&bad, sizeof(int), s));
    CS_TRY(cudaMemsetAsync(bad, 0, sizeof(int), s));
    if (n > 0) k_rows_sorted<<<nblk((long long)n * 32), 256, 0, s>>>(A.row_ptr, A.col_ind, n, bad);
    int hbad = 0;
    CS_TRY(cudaMemcpyAsync(&hbad, bad, sizeof(int), cudaMemcpyDeviceToHost, s));
    CS_TRY(cudaStreamSynchronize(s));
    if (hbad) {
        *status = MX_ERR_INVALID;
        return cudaSuccess;
    }
    for (int **q : {&nlo, &nlen, &lo1, &len1, &lo2, &len2, &len, &flag, &pos, &off})
        CS_TRY(cudaMallocAsync(q, n1 * sizeof(int), s));
    int width = (int)(((long long)A.n_cols + count - 1) / count);
    width = (width + 15) & ~15;
    out.count = count;
    out.width = width;
    out.halo = COL_SLAB_HALO;
    out.row_offset = row_offset;
    out.n_rows = n;
    out.plans = new ResidPlan[count];
    out.col = new int *[count]();
    out.val = new void *[count]();
    out.part = new void *[count]();
    out.row_in_block = new unsigned short *[count]();
    const size_t blocks = ((size_t)n + COMBINE_ROWS - 1) / COMBINE_ROWS;
    CS_TRY(cudaMallocAsync(&out.block_base, (blocks + 1) * count * sizeof(int), s));
    // ---- the band: a CSR over all rows.  Only a row slab of a larger matrix (one GPU's share) has one: its band
    //      pass is what sends the finished rows to the other GPUs.  A whole matrix keeps its near-diagonal entries in
    //      the slabs (one pass over y fewer: measured 6.40 against 6.56 ms on the 1e9-nnz shape). ----
    out.has_band = n < A.n_cols;
    if (!out.has_band) {
        CS_TRY(cudaMemsetAsync(nlo, 0, n1 * sizeof(int), s));
        CS_TRY(cudaMemsetAsync(nlen, 0, n1 * sizeof(int), s));
    } else {
        k_near_ranges<<<nblk(n1), 256, 0, s>>>(A.row_ptr, A.col_ind, n, row_offset, out.halo, nlo, nlen);
    }
    if (out.has_band) {
        CS_TRY(cudaMallocAsync(&out.near_row_ptr, n1 * sizeof(int), s));
        CS_TRY(exclusive_sum(tmp, nlen, out.near_row_ptr, (int)n1, s));
        int nnz_near = 0;
        CS_TRY(cudaMemcpyAsync(&nnz_near, out.near_row_ptr + n, sizeof(int), cudaMemcpyDeviceToHost, s));
        CS_TRY(cudaStreamSynchronize(s));
        CS_TRY(cudaMallocAsync(&out.near_col, (size_t)std::max(nnz_near, 1) * sizeof(int), s));
        CS_TRY(cudaMallocAsync(&out.near_val, (size_t)std::max(nnz_near, 1) * sizeof(V), s));
        k_near_copy<V><<<nblk(std::max(n, 1)), 256, 0, s>>>(A.col_ind, (const V *)A.val, nlo, nlen, out.near_row_ptr, n,
                                                            out.near_col, (V *)out.near_val);
        CS_TRY(cudaGetLastError());
        out.near.n_rows = n;
        out.near.n_cols = A.n_cols;
        out.near.nnz = nnz_near;
        out.near.row_ptr = out.near_row_ptr;
        out.near.col_ind = out.near_col;
        out.near.val = out.near_val;
        CS_TRY(resid_plan_build(dtype, out.near, s));
        out.near.prefetch_tiles = 0;
        // the band once more in row ranges of equal non-zero count (each at least a few waves of tiles long)
        const int chunks = (int)std::max<long long>(1, std::min<long long>(BAND_CHUNKS, nnz_near / (1 << 19)));
        int *dbounds = nullptr, hb[2 * (BAND_CHUNKS + 1)];
        CS_TRY(cudaMallocAsync(&dbounds, sizeof(hb), s));
        k_chunk_bounds<<<1, BAND_CHUNKS + 1, 0, s>>>(out.near_row_ptr, n, chunks, dbounds);
        CS_TRY(cudaMemcpyAsync(hb, dbounds, sizeof(int) * 2 * (chunks + 1), cudaMemcpyDeviceToHost, s));
        CS_TRY(cudaStreamSynchronize(s));
        CS_TRY(cudaFreeAsync(dbounds, s));
        out.band_chunks = chunks;
        out.chunk_plans = new ResidPlan[chunks];
        out.chunk_rows = new int[chunks + 1];
        out.chunk_done = new cudaEvent_t[chunks]();
        CS_TRY(cudaMallocAsync(&out.chunk_row_ptr, ((size_t)n + chunks) * sizeof(int), s));
        for (int i = 0; i < ColSlabs::SEND_STREAMS; ++i) {
            CS_TRY(cudaStreamCreateWithFlags(&out.send_stream[i], cudaStreamNonBlocking));
            CS_TRY(cudaEventCreateWithFlags(&out.send_done[i], cudaEventDisableTiming));
        }
        for (int c = 0; c <= chunks; ++c) out.chunk_rows[c] = hb[c];
        for (int c = 0; c < chunks; ++c) CS_TRY(cudaEventCreateWithFlags(&out.chunk_done[c], cudaEventDisableTiming));
        for (int c = 0; c < chunks; ++c) {
            const int r0 = hb[c], len = hb[c + 1] - r0, e0 = hb[chunks + 1 + c], e1 = hb[chunks + 1 + c + 1];
            int *rp = out.chunk_row_ptr + r0 + c;
            k_rebase<<<nblk((long long)len + 1), 256, 0, s>>>(out.near_row_ptr, r0, len, rp);
            ResidPlan &P = out.chunk_plans[c];
            P.n_rows = len;
            P.n_cols = A.n_cols;
            P.nnz = e1 - e0;
            P.row_ptr = rp;
            P.col_ind = out.near_col + e0;
            P.val = static_cast<const char *>(out.near_val) + (size_t)e0 * sizeof(V);
            CS_TRY(resid_plan_build(dtype, P, s));
            P.prefetch_tiles = 0;
        }
    }
    // ---- the far entries, one slab of columns at a time ----
    for (int k = 0; k < count; ++k) {
        const long long c0 = std::min<long long>((long long)k * width, A.n_cols), c1 = std::min<long long>(c0 + width, A.n_cols);
        k_far_ranges<<<nblk(n1), 256, 0, s>>>(A.row_ptr, A.col_ind, nlo, nlen, n, (int)c0, (int)c1, lo1, len1, lo2, len2,
                                              len, flag);
        CS_TRY(exclusive_sum(tmp, flag, pos, (int)n1, s));
        CS_TRY(exclusive_sum(tmp, len, off, (int)n1, s));
        int m_rows = 0, nnz_slab = 0;
        CS_TRY(cudaMemcpyAsync(&m_rows, pos + n, sizeof(int), cudaMemcpyDeviceToHost, s));
        CS_TRY(cudaMemcpyAsync(&nnz_slab, off + n, sizeof(int), cudaMemcpyDeviceToHost, s));
        CS_TRY(cudaStreamSynchronize(s));
        ResidPlan &P = out.plans[k];
        P.n_rows = n;
        P.n_cols = A.n_cols;
        P.nnz = nnz_slab;
        P.m_rows = m_rows;
        P.n_empty = 0;  // rows without entries in this slab are not touched by its pass
        P.dense_row_ends = (long long)m_rows * 16 >= nnz_slab;  // 128 or more row ends per tile of 2048 non-zeros
        CS_TRY(cudaMallocAsync(&P.c_ptr_own, ((size_t)m_rows + 1) * sizeof(int), s));
        CS_TRY(cudaMallocAsync(&out.part[k], (size_t)std::max(m_rows, 1) * sizeof(V), s));
        CS_TRY(cudaMallocAsync(&out.row_in_block[k], (size_t)std::max(m_rows, 1) * sizeof(unsigned short), s));
        k_row_in_block<<<nblk(n1), 256, 0, s>>>(flag, pos, n, k, count, out.row_in_block[k], out.block_base);
        CS_TRY(cudaMallocAsync(&out.col[k], (size_t)std::max(nnz_slab, 1) * sizeof(int), s));
        CS_TRY(cudaMallocAsync(&out.val[k], (size_t)std::max(nnz_slab, 1) * sizeof(V), s));
        k_far_copy<V><<<nblk(std::max(n, 1)), 256, 0, s>>>(A.col_ind, (const V *)A.val, lo1, len1, lo2, len2, pos, off, n,
                                                           m_rows, nnz_slab, P.c_ptr_own, out.col[k],
                                                           (V *)out.val[k]);
        CS_TRY(cudaGetLastError());
        P.c_ptr = P.c_ptr_own;
        P.row_ptr = nullptr;
        P.col_ind = out.col[k];
        P.val = out.val[k];
        CS_TRY(resid_plan_finish(dtype, P, s));
    }
    CS_TRY(cudaStreamSynchronize(s));
    return cudaSuccess;
}

}  // namespace

cudaError_t col_slabs_build(int dtype, const CsrDev &A, int count, long long row_offset, ColSlabs &out, int *status,
                            cudaStream_t s) {
    if (count < 1) count = 1;
    cudaError_t e = dtype == MX_FP64 ? build_t<double>(A, count, row_offset, out, status, s)
                                     : build_t<__half>(A, count, row_offset, out, status, s);
    if (e != cudaSuccess || *status != MX_OK) col_slabs_free(out, s);
    return e;
}

void col_slabs_free(ColSlabs &S, cudaStream_t s) {
    for (int k = 0; k < S.count; ++k) {
        if (S.plans) resid_plan_free(S.plans[k], s);
        if (S.col && S.col[k]) cudaFreeAsync(S.col[k], s);
        if (S.val && S.val[k]) cudaFreeAsync(S.val[k], s);
        if (S.part && S.part[k]) cudaFreeAsync(S.part[k], s);
        if (S.row_in_block && S.row_in_block[k]) cudaFreeAsync(S.row_in_block[k], s);
    }
    if (S.block_base) cudaFreeAsync(S.block_base, s);
    resid_plan_free(S.near, s);
    for (cudaStream_t q : S.send_stream)
        if (q) cudaStreamSynchronize(q);
    for (int c = 0; c < S.band_chunks; ++c) resid_plan_free(S.chunk_plans[c], s);
    if (S.chunk_done)
        for (int c = 0; c < S.band_chunks; ++c)
            if (S.chunk_done[c]) cudaEventDestroy(S.chunk_done[c]);
    for (int i = 0; i < ColSlabs::SEND_STREAMS; ++i) {
        if (S.send_done[i]) cudaEventDestroy(S.send_done[i]);
        if (S.send_stream[i]) cudaStreamDestroy(S.send_stream[i]);
    }
    if (S.chunk_row_ptr) cudaFreeAsync(S.chunk_row_ptr, s);
    delete[] S.chunk_plans;
    delete[] S.chunk_rows;
    delete[] S.chunk_done;
    for (void *p : {(void *)S.near_row_ptr, (void *)S.near_col, S.near_val})
        if (p) cudaFreeAsync(p, s);
    delete[] S.plans;
    delete[] S.col;
    delete[] S.val;
    delete[] S.part;
    delete[] S.row_in_block;
    S = ColSlabs();
}

int col_slabs_launches(const ColSlabs &S) {
    int n = (S.has_band ? resid_launches(S.near) : 0) + 1;  // + the combining kernel (mx_spmv; mx_spmv_peers runs the band
                                                            // in ranges and adds one send per range)
    for (int k = 0; k < S.count; ++k)
        if (S.plans[k].nnz > 0) n += resid_launches(S.plans[k]);
    return n;
}

namespace {

// the slab passes: pass k writes the partial sums of slab k's non-empty rows to S.part[k] (its row space is the
// compressed one: the plan has no row-index table); each pass is chained behind its predecessor
cudaError_t far_passes(int dtype, const ColSlabs &S, const void *x, cudaStream_t s, bool &first) {
    cudaError_t e = cudaSuccess;
    for (int k = 0; k < S.count && e == cudaSuccess; ++k)
        if (S.plans[k].nnz > 0) {
            e = resid_spmv(dtype, S.plans[k], x, S.part[k], nullptr, nullptr, /*accumulate=*/false, s, /*chained=*/!first);
            first = false;
        }
    return e;
}

cudaError_t combine(int dtype, const ColSlabs &S, void *y, cudaStream_t s) {
    if (S.n_rows <= 0) return cudaSuccess;
    const int grid = (S.n_rows + COMBINE_ROWS - 1) / COMBINE_ROWS;
    if (dtype != MX_FP64) return cudaErrorNotSupported;
    if (S.count > MAX_COL_SLABS) return cudaErrorInvalidValue;
    PartTable T{};
    for (int k = 0; k < S.count; ++k) {
        T.p[k] = static_cast<const double *>(S.part[k]);
        T.row[k] = S.row_in_block[k];
    }
    k_combine<<<grid, 256, 0, s>>>(T, S.block_base, S.count, S.n_rows, (double *)y);
    return cudaGetLastError();
}

}  // namespace

// y = A x on one GPU: one pass per slab, then the rows' partial sums are added in slab order.  (A matrix with a band
// - a row slab of a larger matrix multiplied without peers - adds the band last, in the CSR kernel's accumulate mode.)
cudaError_t col_slabs_spmv(int dtype, const ColSlabs &S, const void *x, void *y, size_t y_bytes, cudaStream_t s) {
    (void)y_bytes;
    bool first = true;
    cudaError_t e = far_passes(dtype, S, x, s, first);
    if (e == cudaSuccess) e = combine(dtype, S, y, s);
    if (e == cudaSuccess && S.has_band)
        e = resid_spmv(dtype, S.near, x, y, nullptr, nullptr, /*accumulate=*/true, s, /*chained=*/true);
    return e;
}

// The same product as one GPU's share of a row-partitioned matrix: the far passes' partial sums are combined into
// this GPU's rows of its own full-length buffer; the band follows in row ranges of equal non-zero count (the CSR
// kernel's accumulate mode), and as soon as a range is finished its rows are sent to the other GPUs' buffers from
// other streams while the next range is computed - by the copy engines when there is one destination, by a small copy
// kernel when there are several (see below).  The exchange thus overlaps the band, about half of the work.  Measured
// before this: the rows stored to the peers from the band kernel's own epilogue - once the stores of all SMs saturate
// NVLink they back up into the SMs and stall the gathers behind them (4 GPUs: 2.56 ms against 2.23 ms for kernels
// followed by one copy).
cudaError_t col_slabs_spmv_peers(int dtype, const ColSlabs &S, const void *x, void *const *peers, int n_peers, int self,
                                 long long row_offset, cudaStream_t s) {
    if (!S.has_band || S.band_chunks < 1) return cudaErrorNotSupported;  // without a band the caller sends the rows
    const size_t vb = val_bytes(dtype);
    char *y_own = static_cast<char *>(peers[self]) + (size_t)row_offset * vb;
    bool first = true;
    cudaError_t e = far_passes(dtype, S, x, s, first);
    if (e == cudaSuccess) e = combine(dtype, S, y_own, s);
    // How a finished range leaves.  One destination (2 GPUs): two copies by the copy engines, each on a stream of its
    // own (one engine moves about 330 GB/s over NVLink; they take no SM from the band: 2.97 ms against 3.04 ms with
    // the copy kernel, 2.79 ms of kernels).  Several destinations: one launch of the copy kernel on a third of the
    // SMs, which keeps all links busy at once (4 GPUs, 1.49 ms of kernels: 2.10 ms against 2.17 ms with one engine
    // copy per destination).
    const int nd = n_peers - 1;
    const bool by_kernel = nd >= 2;
    const int parts = 2, used = by_kernel ? 1 : std::min(ColSlabs::SEND_STREAMS, std::max(nd * parts, 0));
    for (int c = 0; c < S.band_chunks && e == cudaSuccess; ++c) {
        const int r0 = S.chunk_rows[c], len = S.chunk_rows[c + 1] - r0;
        if (len <= 0) continue;
        if (S.chunk_plans[c].nnz > 0)
            e = resid_spmv(dtype, S.chunk_plans[c], x, y_own + (size_t)r0 * vb, nullptr, nullptr, /*accumulate=*/true, s);
        if (nd <= 0) continue;
        if (e == cudaSuccess) e = cudaEventRecord(S.chunk_done[c], s);
        for (int i = 0; i < used && e == cudaSuccess; ++i) e = cudaStreamWaitEvent(S.send_stream[i], S.chunk_done[c], 0);
        if (by_kernel) {
            if (e == cudaSuccess) e = peer_push_rows(dtype, peers, n_peers, self, row_offset + r0, len, S.send_stream[0]);
            continue;
        }
        int k = 0;
        for (int g = 0; g < n_peers && e == cudaSuccess; ++g) {
            if (g == self) continue;
            for (int q = 0; q < parts && e == cudaSuccess; ++q, ++k) {
                const size_t a = (size_t)len * q / parts, b = (size_t)len * (q + 1) / parts;
                if (b > a)
                    e = cudaMemcpyAsync(static_cast<char *>(peers[g]) + ((size_t)(row_offset + r0) + a) * vb,
                                        y_own + ((size_t)r0 + a) * vb, (b - a) * vb, cudaMemcpyDeviceToDevice,
                                        S.send_stream[k % ColSlabs::SEND_STREAMS]);
            }
        }
    }
    for (int i = 0; i < used && e == cudaSuccess; ++i) {  // the caller's stream continues after the last copy
        e = cudaEventRecord(S.send_done[i], S.send_stream[i]);
        if (e == cudaSuccess) e = cudaStreamWaitEvent(s, S.send_done[i], 0);
    }
    return e;
}

}  // namespace mx
