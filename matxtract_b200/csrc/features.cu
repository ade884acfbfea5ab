// Structure features of the uploaded matrix, on the device: the 24 statistics of the non-zeros-per-row distribution
// and the same 24 of the non-zeros-per-column distribution that the reference's tau predictor is trained on
// (ML/extract_features.cpp:19-93 computeDistStats, :155-170 how the two distributions are formed).  The reference
// transposes the matrix through cuSPARSE to count the columns and sorts on the host; here: one histogram, one CUB key
// sort per distribution, one scan, exact integer moments, and the nine coverage fractions by binary search with the
// reference's own predicate.  Everything except the standard deviation is bit-identical to the reference's doubles;
// the standard deviation comes from exact integer sums instead of a long-double accumulation (last-bit differences).
#include <algorithm>
#include <cmath>
#include <cstdint>

#include "device_prims.cuh"
#include "mx_internal.h"

namespace mx {
namespace {

#define FCK(call)                         \
    do {                                  \
        cudaError_t e_ = (call);          \
        if (e_ != cudaSuccess) return e_; \
    } while (0)

__global__ void f_row_counts(const int *__restrict__ row_ptr, int n, int *__restrict__ cnt) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) cnt[i] = row_ptr[i + 1] - row_ptr[i];
}
__global__ void f_col_hist(const int *__restrict__ col_ind, int nnz, int *__restrict__ cnt) {
    const int stride = gridDim.x * blockDim.x;
    for (int e = blockIdx.x * blockDim.x + threadIdx.x; e < nnz; e += stride) atomicAdd(cnt + __ldg(col_ind + e), 1);
}

// sum of squares as two 64-bit sums (low and high 32 bits of each square): neither can overflow for n < 2^31
__global__ void f_square_sums(const int *__restrict__ cnt, int n, unsigned long long *__restrict__ out) {
    unsigned long long lo = 0, hi = 0;
    const int stride = gridDim.x * blockDim.x;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const unsigned long long v = (unsigned long long)cnt[i], q = v * v;
        lo += q & 0xffffffffull;
        hi += q >> 32;
    }
    for (int d = 16; d > 0; d >>= 1) {
        lo += __shfl_down_sync(0xffffffffu, lo, d);
        hi += __shfl_down_sync(0xffffffffu, hi, d);
    }
    if ((threadIdx.x & 31) == 0) {
        atomicAdd(out, lo);
        atomicAdd(out + 1, hi);
    }
}

// sorted: counts in descending order, pref: their inclusive prefix sums.  out[0..9] = sorted[k-1] for the reference's
// k list (or -1 past the end), out[10..18] = smallest i+1 with pref[i] / total >= coverage (0 when none),
// out[19] = min, out[20] = max.
__global__ void f_pick(const int *__restrict__ sorted, const long long *__restrict__ pref, int n,
                       long long *__restrict__ out) {
    const int t = threadIdx.x;
    const int topK[10] = {1, 2, 3, 4, 5, 10, 50, 100, 200, 300};
    const double cover[9] = {0.1, 0.2, 0.3, 0.4, 0.5, 0.6, 0.7, 0.8, 0.9};
    if (t < 10) out[t] = topK[t] - 1 < n ? sorted[topK[t] - 1] : -1;
    if (t >= 10 && t < 19) {
        const double total = (double)pref[n - 1], target = cover[t - 10];
        int lo = 0, hi = n;  // first i in [0, n) with the predicate true; the predicate is monotone in i
        while (lo < hi) {
            const int mid = lo + (hi - lo) / 2;
            if ((double)pref[mid] / total >= target)
                hi = mid;
            else
                lo = mid + 1;
        }
        out[t] = lo < n ? lo + 1 : 0;
    }
    if (t == 19) out[19] = sorted[n - 1];
    if (t == 20) out[20] = sorted[0];
}

cudaError_t dist_features(const int *cnt, int n, mx_dist_features &F, cudaStream_t s) {
    F = mx_dist_features{};
    if (n <= 0) return cudaSuccess;  // the reference's empty case: everything 0
    int *sorted = nullptr;
    long long *pref = nullptr, *picks = nullptr;
    unsigned long long *sq = nullptr;
    FCK(cudaMallocAsync(&sorted, sizeof(int) * (size_t)n, s));
    FCK(cudaMallocAsync(&pref, sizeof(long long) * (size_t)n, s));
    FCK(cudaMallocAsync(&picks, sizeof(long long) * 21, s));
    FCK(cudaMallocAsync(&sq, sizeof(unsigned long long) * 2, s));
    cudaError_t e = cudaSuccess;
    long long hp[21];
    unsigned long long hsq[2];
    long long total = 0;
    {
        TempBuf tmp;
        size_t bytes = 0;
        e = cub::DeviceRadixSort::SortKeysDescending(nullptr, bytes, cnt, sorted, n, 0, 32, s);
        if (e == cudaSuccess) e = tmp.reserve(bytes, s);
        if (e == cudaSuccess) e = cub::DeviceRadixSort::SortKeysDescending(tmp.p, bytes, cnt, sorted, n, 0, 32, s);
        if (e == cudaSuccess) e = inclusive_sum(tmp, sorted, pref, n, s);
        if (e == cudaSuccess) e = cudaMemsetAsync(sq, 0, sizeof(unsigned long long) * 2, s);
        if (e == cudaSuccess) {
            f_square_sums<<<std::min((n + 255) / 256, 148 * 8), 256, 0, s>>>(cnt, n, sq);
            f_pick<<<1, 32, 0, s>>>(sorted, pref, n, picks);
            e = cudaGetLastError();
        }
        if (e == cudaSuccess) e = cudaMemcpyAsync(hp, picks, sizeof hp, cudaMemcpyDeviceToHost, s);
        if (e == cudaSuccess) e = cudaMemcpyAsync(hsq, sq, sizeof hsq, cudaMemcpyDeviceToHost, s);
        if (e == cudaSuccess) e = cudaMemcpyAsync(&total, pref + (n - 1), sizeof total, cudaMemcpyDeviceToHost, s);
        if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    }
    cudaFreeAsync(sorted, s);
    cudaFreeAsync(pref, s);
    cudaFreeAsync(picks, s);
    cudaFreeAsync(sq, s);
    if (e != cudaSuccess) return e;
    // the reference's arithmetic on these integers (ML/extract_features.cpp:41-89)
    const double mean = (double)total / n;
    // variance = (n * sum(v^2) - (sum v)^2) / n^2, numerator exact in 128-bit integers
    const unsigned __int128 sumsq = ((unsigned __int128)hsq[1] << 32) + hsq[0];
    const unsigned __int128 num = (unsigned __int128)n * sumsq - (unsigned __int128)total * (unsigned __int128)total;
    const long double var = (long double)num / ((long double)n * (long double)n);
    F.mean = mean;
    F.std_dev = std::sqrt((double)var);
    F.min = hp[19];
    F.max = hp[20];
    F.p_ratio = F.min > 0 ? (double)F.max / (double)F.min : 0.0;
    for (int i = 0; i < 10; ++i) F.top[i] = (hp[i] >= 0 && mean > 0) ? (double)hp[i] / mean : 0.0;
    for (int i = 0; i < 9; ++i) F.hot[i] = hp[10 + i] > 0 ? (double)hp[10 + i] / n : 0.0;
    return cudaSuccess;
}

}  // namespace

cudaError_t matrix_features(const CsrDev &A, mx_matrix_features &out, cudaStream_t s) {
    out = mx_matrix_features{};
    out.rows = A.n_rows;
    out.cols = A.n_cols;
    out.nnz = A.nnz;
    const int n = std::max(A.n_rows, A.n_cols);
    if (n <= 0) return cudaSuccess;
    int *cnt = nullptr;
    FCK(cudaMallocAsync(&cnt, sizeof(int) * (size_t)n, s));
    cudaError_t e = cudaSuccess;
    if (A.n_rows > 0) {
        f_row_counts<<<(A.n_rows + 255) / 256, 256, 0, s>>>(A.row_ptr, A.n_rows, cnt);
        e = cudaGetLastError();
        if (e == cudaSuccess) e = dist_features(cnt, A.n_rows, out.row, s);
    }
    if (e == cudaSuccess && A.n_cols > 0) {
        e = cudaMemsetAsync(cnt, 0, sizeof(int) * (size_t)A.n_cols, s);
        if (e == cudaSuccess && A.nnz > 0) {
            f_col_hist<<<std::min((A.nnz + 255) / 256, 148 * 16), 256, 0, s>>>(A.col_ind, A.nnz, cnt);
            e = cudaGetLastError();
        }
        if (e == cudaSuccess) e = dist_features(cnt, A.n_cols, out.col, s);
    }
    cudaFreeAsync(cnt, s);
    return e;
}

}  // namespace mx
