// Column-slab execution of a CSR SpMV whose x does not fit the L2 cache.
//
// A CSR-ordered kernel gathers x[col] for every non-zero.  When x is much larger than L2 (a 64M-column FP64 vector is
// 512 MB) and the columns of a row are spread over the whole range, every such gather is a DRAM access that moves a
// whole 64-byte burst for 8 useful bytes: measured on the 1e9-non-zero power-law matrix, the kernel moves 3-4x the
// matrix's own bytes.  Here the matrix is cut into vertical slabs of `width` columns, each stored as its own CSR over
// its non-empty rows.  One pass per slab streams that slab's entries and gathers from a 32 MB range of x that stays in
// L2; the price is that y is read and written once per pass instead of once.  The passes are the ordinary CSR kernel
// (resid_kernel) in its accumulate mode, so the arithmetic stays free of atomics and bit-reproducible.
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

// the part of every row that falls into columns [c0, c1): start in the source arrays, length, non-empty flag
__global__ void k_slab_ranges(const int *__restrict__ row_ptr, const int *__restrict__ col, int n, int c0, int c1,
                              int *__restrict__ lo, int *__restrict__ len, int *__restrict__ flag) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r > n) return;
    int a = 0, l = 0;
    if (r < n) {
        const int b = row_ptr[r], e = row_ptr[r + 1];
        a = lower_col(col, b, e, c0);
        l = lower_col(col, a, e, c1) - a;
    }
    lo[r] = a;
    len[r] = l;
    flag[r] = l > 0;
}

// one warp per 32 rows: every lane owns a row; short parts are copied by their lane, long ones by the whole warp
template <typename V>
__global__ void k_slab_copy(const int *__restrict__ col, const V *__restrict__ val, const int *__restrict__ lo,
                            const int *__restrict__ len, const int *__restrict__ pos, const int *__restrict__ off, int n,
                            int m_rows, int nnz_slab, int *__restrict__ c_ptr, int *__restrict__ nz_row,
                            int *__restrict__ ocol, V *__restrict__ oval) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x, lane = threadIdx.x & 31;
    int a = 0, l = 0, o = 0;
    if (r < n) {
        a = lo[r];
        l = len[r];
        o = off[r];
        if (l > 0) {
            const int k = pos[r];
            c_ptr[k] = o;
            nz_row[k] = r;
        }
    }
    if (r == 0) c_ptr[m_rows] = nnz_slab;
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

template <typename V>
cudaError_t build_t(const CsrDev &A, int count, ColSlabs &out, int *status, cudaStream_t s) {
    const int n = A.n_rows;
    const size_t n1 = (size_t)n + 1;
    *status = MX_OK;
    TempBuf tmp;
    int *lo = nullptr, *len = nullptr, *flag = nullptr, *pos = nullptr, *off = nullptr, *bad = nullptr;
    struct Guard {
        cudaStream_t s;
        int **p[6];
        ~Guard() {
            for (int **q : p)
                if (*q) cudaFreeAsync(*q, s);
        }
    } guard{s, {&lo, &len, &flag, &pos, &off, &bad}};
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
    CS_TRY(cudaMallocAsync(&lo, n1 * sizeof(int), s));
    CS_TRY(cudaMallocAsync(&len, n1 * sizeof(int), s));
    CS_TRY(cudaMallocAsync(&flag, n1 * sizeof(int), s));
    CS_TRY(cudaMallocAsync(&pos, n1 * sizeof(int), s));
    CS_TRY(cudaMallocAsync(&off, n1 * sizeof(int), s));
    int width = (int)(((long long)A.n_cols + count - 1) / count);
    width = (width + 15) & ~15;
    out.count = count;
    out.width = width;
    out.plans = new ResidPlan[count];
    out.col = new int *[count]();
    out.val = new void *[count]();
    for (int k = 0; k < count; ++k) {
        const long long c0 = (long long)k * width, c1 = std::min<long long>(c0 + width, A.n_cols);
        k_slab_ranges<<<nblk(n1), 256, 0, s>>>(A.row_ptr, A.col_ind, n, (int)std::min<long long>(c0, A.n_cols), (int)c1,
                                               lo, len, flag);
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
        CS_TRY(cudaMallocAsync(&P.c_ptr_own, ((size_t)m_rows + 1) * sizeof(int), s));
        CS_TRY(cudaMallocAsync(&P.nz_row, ((size_t)m_rows + 1) * sizeof(int), s));
        CS_TRY(cudaMallocAsync(&out.col[k], (size_t)(nnz_slab > 0 ? nnz_slab : 1) * sizeof(int), s));
        CS_TRY(cudaMallocAsync(&out.val[k], (size_t)(nnz_slab > 0 ? nnz_slab : 1) * sizeof(V), s));
        k_slab_copy<V><<<nblk(std::max(n, 1)), 256, 0, s>>>(A.col_ind, (const V *)A.val, lo, len, pos, off, n, m_rows,
                                                            nnz_slab, P.c_ptr_own, P.nz_row, out.col[k], (V *)out.val[k]);
        CS_TRY(cudaGetLastError());
        P.c_ptr = P.c_ptr_own;
        P.row_ptr = nullptr;
        P.col_ind = out.col[k];
        P.val = out.val[k];
        CS_TRY(resid_plan_finish(sizeof(V) == 8 ? MX_FP64 : MX_FP16, P, s));
    }
    return cudaSuccess;
}

}  // namespace

cudaError_t col_slabs_build(int dtype, const CsrDev &A, int count, ColSlabs &out, int *status, cudaStream_t s) {
    if (count < 1) count = 1;
    cudaError_t e = dtype == MX_FP64 ? build_t<double>(A, count, out, status, s) : build_t<__half>(A, count, out, status, s);
    if (e != cudaSuccess || *status != MX_OK) col_slabs_free(out, s);
    return e;
}

void col_slabs_free(ColSlabs &S, cudaStream_t s) {
    for (int k = 0; k < S.count; ++k) {
        if (S.plans) resid_plan_free(S.plans[k], s);
        if (S.col && S.col[k]) cudaFreeAsync(S.col[k], s);
        if (S.val && S.val[k]) cudaFreeAsync(S.val[k], s);
    }
    delete[] S.plans;
    delete[] S.col;
    delete[] S.val;
    S = ColSlabs();
}

cudaError_t col_slabs_spmv(int dtype, const ColSlabs &S, const void *x, void *y, size_t y_bytes, cudaStream_t s) {
    cudaError_t e = cudaMemsetAsync(y, 0, y_bytes, s);
    for (int k = 0; k < S.count && e == cudaSuccess; ++k)
        if (S.plans[k].nnz > 0)  // passes after the first are chained: their prologue overlaps the previous pass's tail
            e = resid_spmv(dtype, S.plans[k], x, y, nullptr, nullptr, /*accumulate=*/true, s, /*chained=*/k > 0);
    return e;
}

}  // namespace mx
