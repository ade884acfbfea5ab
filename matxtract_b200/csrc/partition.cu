// Cascaded compute-density extraction on the device.  Replaces the host pipeline in main() of the
// reference driver (test/test_autotc_spmv.cpp:1119-1421 and merge2CSR_opt :129-250) together with its three
// cuSPARSE transposes (utilities/csr2csc.cpp).  Every output array is bit-identical to what that pipeline
// produces; the route is different — nothing is transposed:
//
//   1. column histogram (atomics)                               <- csr2csc + count loop          (:1119-1129)
//   2. stable descending radix sort of (count, column)          <- glibc qsort, ties keep index  (:1130)
//   3. inclusive scan + first prefix >= (int)(nnz * tau_c)      <- serial prefix loop            (:1131-1141)
//   4. column map: D column -> density rank, S column -> dCols + (its index among S columns)   (:1147-1221)
//   5. per-row count of D entries (warp per row)                <- csc2csr of the D part         (:1234-1247)
//   6. stable descending sort of rows, scan, tau_r cut, rId, hot-row bitmap                     (:1248-1267)
//   7. row pointers of the core-dense block dd and of the residual A_CD by two scans           (:1271-1345, :167-189)
//   8. one pass over the input scatters every entry to its row segment of dd or A_CD; a segmented sort
//      then orders each segment (S entries by new column id, then D entries by rank), which is the order
//      the reference gets from its stable transposes                                             (:213-246)
//   9. tiles from dd: segmented sort of each 8-row panel's column ids, head flags + scan give every entry
//      its slot in the panel's sorted unique list -> chunkPtr, sparse_AToX_index, bitmaps (atomicOr),
//      fragPtr (popcount scan), packed values                                                    (:502-585, :1369-1404, :718-978)
#include <algorithm>
#include <vector>

#include "device_prims.cuh"
#include "mx_internal.h"

namespace mx {
namespace {

#define PCK(call)                        \
    do {                                 \
        cudaError_t e_ = (call);         \
        if (e_ != cudaSuccess) return e_; \
    } while (0)

template <typename T>
cudaError_t dalloc(T **p, size_t n, cudaStream_t s) {
    return cudaMallocAsync((void **)p, (n > 0 ? n : 1) * sizeof(T), s);
}
// scratch buffers of one run, taken from the stream-ordered pool (no device-wide synchronisation per buffer) and
// released on every exit path
struct Scratch {
    cudaStream_t s;
    std::vector<void *> bufs;
    explicit Scratch(cudaStream_t stream) : s(stream) {}
    template <typename T>
    cudaError_t alloc(T **p, size_t n) {
        cudaError_t e = cudaMallocAsync((void **)p, (n > 0 ? n : 1) * sizeof(T), s);
        if (e == cudaSuccess) bufs.push_back(*p);
        return e;
    }
    ~Scratch() {
        for (void *b : bufs) cudaFreeAsync(b, s);
    }
};

__global__ void k_col_hist(const int *__restrict__ col_ind, int nnz, int *__restrict__ cnt) {
    int stride = gridDim.x * blockDim.x;
    for (int e = blockIdx.x * blockDim.x + threadIdx.x; e < nnz; e += stride) atomicAdd(cnt + __ldg(col_ind + e), 1);
}
__global__ void k_iota(int *p, int n) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) p[i] = i;
}
__global__ void k_fill(int *p, int n, int v) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) p[i] = v;
}
// smallest k >= 1 (k <= bound) with pref[k-1] >= T; out = {k, pref[k-1]}, left {0,0} when none
__global__ void k_find_cut(const int *__restrict__ pref, int bound, int T, int *__restrict__ out) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= bound) return;
    if (pref[i] >= T && (i == 0 || pref[i - 1] < T)) {
        out[0] = i + 1;
        out[1] = pref[i];
    }
}
__global__ void k_mark_rank(const int *__restrict__ colOrder, int dCols, int *__restrict__ rankOf,
                            int *__restrict__ isS) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= dCols) return;
    int c = colOrder[i];
    rankOf[c] = i;
    isS[c] = 0;
}
__global__ void k_colmap(const int *__restrict__ isS, const int *__restrict__ sidx, const int *__restrict__ rankOf,
                         int dCols, int n_cols, int *__restrict__ colMap, int *__restrict__ xperm) {
    int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= n_cols) return;
    int m = isS[j] ? dCols + sidx[j] : rankOf[j];
    colMap[j] = m;
    xperm[m] = j;
}
__global__ void k_row_count_d(const int *__restrict__ row_ptr, const int *__restrict__ col_ind,
                              const int *__restrict__ colMap, int dCols, int n_rows, int *__restrict__ rowCntD) {
    int r = (int)(((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5), lane = threadIdx.x & 31;
    if (r >= n_rows) return;
    int c = 0;
    for (int e = row_ptr[r] + lane, end = row_ptr[r + 1]; e < end; e += 32)
        c += __ldg(colMap + __ldg(col_ind + e)) < dCols;
    for (int d = 16; d; d >>= 1) c += __shfl_xor_sync(0xffffffffu, c, d);
    if (lane == 0) rowCntD[r] = c;
}
__global__ void k_mark_hot(const int *__restrict__ rowOrder, int dRows, int *__restrict__ hotPos,
                           uint32_t *__restrict__ hotmask, int *__restrict__ rId) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= dRows) return;
    int r = rowOrder[i];
    rId[i] = r;
    hotPos[r] = i;
    atomicOr(hotmask + (r >> 5), 1u << (r & 31));
}
__global__ void k_res_len(const int *__restrict__ row_ptr, const int *__restrict__ rowCntD,
                          const int *__restrict__ hotPos, int n_rows, int *__restrict__ resLen) {
    int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r > n_rows) return;
    resLen[r] = r < n_rows ? (row_ptr[r + 1] - row_ptr[r]) - (hotPos[r] >= 0 ? rowCntD[r] : 0) : 0;
}
__global__ void k_scatter(const int *__restrict__ row_ptr, const int *__restrict__ col_ind,
                          const int *__restrict__ colMap, const int *__restrict__ hotPos,
                          const int *__restrict__ rowPtr_dd, const int *__restrict__ rowPtr_CD, int dCols, int sCols,
                          int n_rows, int *__restrict__ Kdd, int *__restrict__ Pdd, int *__restrict__ Kcd,
                          int *__restrict__ Pcd) {
    int r = (int)(((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5), lane = threadIdx.x & 31;
    if (r >= n_rows) return;
    const int start = row_ptr[r], end = row_ptr[r + 1], hp = hotPos[r];
    const bool hot = hp >= 0;
    const int ddBase = hot ? rowPtr_dd[hp] : 0, cdBase = rowPtr_CD[r];
    const unsigned lt = (1u << lane) - 1u;
    int nd = 0, nc = 0;
    for (int e0 = start; e0 < end; e0 += 32) {
        const int e = e0 + lane;
        const bool valid = e < end;
        const int c = valid ? __ldg(colMap + __ldg(col_ind + e)) : 0;
        const bool isD = valid && c < dCols, toDD = isD && hot, toCD = valid && !toDD;
        const unsigned mDD = __ballot_sync(0xffffffffu, toDD), mCD = __ballot_sync(0xffffffffu, toCD);
        if (toDD) {
            int pos = ddBase + nd + __popc(mDD & lt);
            Kdd[pos] = c;
            Pdd[pos] = e;
        }
        if (toCD) {
            int pos = cdBase + nc + __popc(mCD & lt);
            Kcd[pos] = isD ? c + sCols : c - dCols;  // ascending: S entries by new id, then D entries by rank
            Pcd[pos] = e;
        }
        nd += __popc(mDD);
        nc += __popc(mCD);
    }
}
template <typename V>
__global__ void k_finalize_cd(const int *__restrict__ K, const int *__restrict__ P, const V *__restrict__ val, int n,
                              int dCols, int sCols, int *__restrict__ colInd, V *__restrict__ oval) {
    int q = blockIdx.x * blockDim.x + threadIdx.x;
    if (q >= n) return;
    int k = K[q];
    colInd[q] = k < sCols ? dCols + k : k - sCols;
    oval[q] = val[P[q]];
}
template <typename V>
__global__ void k_gather_vals(const int *__restrict__ P, const V *__restrict__ val, int n, V *__restrict__ oval) {
    int q = blockIdx.x * blockDim.x + threadIdx.x;
    if (q < n) oval[q] = val[P[q]];
}

// ---- tiles from dd ----
__global__ void k_panel_off(const int *__restrict__ rowPtr_dd, int dRows, int chunkNum, int *__restrict__ panelOff) {
    int p = blockIdx.x * blockDim.x + threadIdx.x;
    if (p <= chunkNum) panelOff[p] = rowPtr_dd[min(p * 8, dRows)];
}
__global__ void k_expand_rows(const int *__restrict__ rowPtr_dd, int dRows, int *__restrict__ rowOf) {
    int r = (int)(((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5), lane = threadIdx.x & 31;
    if (r >= dRows) return;
    for (int e = rowPtr_dd[r] + lane, end = rowPtr_dd[r + 1]; e < end; e += 32) rowOf[e] = r;
}
// head[q] = 1 when sorted column q starts a new distinct column inside its panel
__global__ void k_heads(const int *__restrict__ sortedCol, const int *__restrict__ srcIdx,
                        const int *__restrict__ rowOf, int n, int *__restrict__ head) {
    int q = blockIdx.x * blockDim.x + threadIdx.x;
    if (q >= n) return;
    int h = 1;
    if (q > 0) {
        int p = rowOf[srcIdx[q]] >> 3, pp = rowOf[srcIdx[q - 1]] >> 3;
        h = (p != pp) || (sortedCol[q] != sortedCol[q - 1]);
    }
    head[q] = h;
}
__global__ void k_frag_count(const int *__restrict__ panelOff, const int *__restrict__ H, int chunkNum, int K,
                             int *__restrict__ nf) {
    int p = blockIdx.x * blockDim.x + threadIdx.x;
    if (p > chunkNum) return;
    int c = 0;
    if (p < chunkNum) {
        int b = panelOff[p], e = panelOff[p + 1];
        if (e > b) {
            int uniq = H[e - 1] - H[b] + 1;
            c = (uniq + K - 1) / K;
        }
    }
    nf[p] = c;
}
template <typename B>
__global__ void k_atox_bits(const int *__restrict__ sortedCol, const int *__restrict__ srcIdx,
                            const int *__restrict__ rowOf, const int *__restrict__ head, const int *__restrict__ H,
                            const int *__restrict__ panelOff, const int *__restrict__ chunkPtr, int n, int K,
                            int *__restrict__ AToX, B *__restrict__ fragBit, int *__restrict__ entFrag,
                            int *__restrict__ entBit) {
    int q = blockIdx.x * blockDim.x + threadIdx.x;
    if (q >= n) return;
    const int row = rowOf[srcIdx[q]], p = row >> 3;
    const int s = H[q] - H[panelOff[p]];
    const int f = chunkPtr[p] + s / K, bit = (row & 7) * K + s % K;
    if (head[q]) AToX[(size_t)chunkPtr[p] * K + s] = sortedCol[q];
    if constexpr (sizeof(B) == 8)
        atomicOr(reinterpret_cast<unsigned long long *>(fragBit) + f, 1ull << bit);
    else
        atomicOr(reinterpret_cast<unsigned *>(fragBit) + f, 1u << bit);
    entFrag[q] = f;
    entBit[q] = bit;
}
template <typename B>
__global__ void k_popc(const B *__restrict__ fragBit, int n, int *__restrict__ cnt) {
    int f = blockIdx.x * blockDim.x + threadIdx.x;
    if (f > n) return;
    cnt[f] = f < n ? (sizeof(B) == 8 ? __popcll((unsigned long long)fragBit[f]) : __popc((unsigned)fragBit[f])) : 0;
}
template <typename V, typename B>
__global__ void k_tile_vals(const int *__restrict__ srcIdx, const int *__restrict__ entFrag,
                            const int *__restrict__ entBit, const B *__restrict__ fragBit,
                            const int *__restrict__ fragPtr, const V *__restrict__ val_dd, int n,
                            V *__restrict__ tcVal) {
    int q = blockIdx.x * blockDim.x + threadIdx.x;
    if (q >= n) return;
    const int f = entFrag[q], bit = entBit[q];
    const B bm = fragBit[f];
    int below;
    if constexpr (sizeof(B) == 8)
        below = __popcll((unsigned long long)bm & ((1ull << bit) - 1ull));
    else
        below = __popc((unsigned)bm & ((1u << bit) - 1u));
    tcVal[fragPtr[f] + below] = val_dd[srcIdx[q]];
}

cudaError_t seg_sort_pairs(TempBuf &tmp, const int *kin, int *kout, const int *vin, int *vout, int n, int nseg,
                           const int *offsets, cudaStream_t s) {
    if (n <= 0 || nseg <= 0) return cudaSuccess;
    size_t bytes = 0;
    PCK(cub::DeviceSegmentedSort::SortPairs(nullptr, bytes, kin, kout, vin, vout, n, nseg, offsets, offsets + 1, s));
    PCK(tmp.reserve(bytes, s));
    return cub::DeviceSegmentedSort::SortPairs(tmp.p, bytes, kin, kout, vin, vout, n, nseg, offsets, offsets + 1, s);
}

cudaError_t sort_desc_pairs(TempBuf &tmp, const int *kin, int *kout, const int *vin, int *vout, int n,
                            cudaStream_t s) {
    if (n <= 0) return cudaSuccess;
    size_t bytes = 0;
    PCK(cub::DeviceRadixSort::SortPairsDescending(nullptr, bytes, kin, kout, vin, vout, n, 0, 32, s));
    PCK(tmp.reserve(bytes, s));
    return cub::DeviceRadixSort::SortPairsDescending(tmp.p, bytes, kin, kout, vin, vout, n, 0, 32, s);
}

struct ToLongLong {
    __host__ __device__ long long operator()(int v) const { return (long long)v; }
};

inline int nblk(long long n, int b = 256) { return (int)((n + b - 1) / b); }

template <typename V, typename B>
cudaError_t tiles_from_dd_t(int dRows, int nnzRowD, const int *rowPtr_dd, const int *colInd_dd, const V *val_dd,
                            TileArrays &T, int *status, cudaStream_t s) {
    constexpr int K = sizeof(B) == 8 ? 8 : 4;
    *status = MX_OK;
    TempBuf tmp;
    Scratch sc(s);
    const int chunkNum = (dRows + 7) / 8;
    T.dRows = dRows;
    T.chunkNum = chunkNum;
    T.nvals = nnzRowD;
    int *panelOff = nullptr, *rowOf = nullptr, *iota = nullptr, *sortedCol = nullptr, *srcIdx = nullptr,
        *head = nullptr, *H = nullptr, *nf = nullptr, *entFrag = nullptr, *entBit = nullptr, *pc = nullptr;
    PCK(sc.alloc(&panelOff, (size_t)chunkNum + 1));
    PCK(sc.alloc(&rowOf, (size_t)nnzRowD));
    PCK(sc.alloc(&iota, (size_t)nnzRowD));
    PCK(sc.alloc(&sortedCol, (size_t)nnzRowD));
    PCK(sc.alloc(&srcIdx, (size_t)nnzRowD));
    PCK(sc.alloc(&head, (size_t)nnzRowD));
    PCK(sc.alloc(&H, (size_t)nnzRowD));
    PCK(sc.alloc(&nf, (size_t)chunkNum + 1));
    PCK(dalloc(&T.chunkPtr, (size_t)chunkNum + 1, s));
    k_panel_off<<<nblk(chunkNum + 1), 256, 0, s>>>(rowPtr_dd, dRows, chunkNum, panelOff);
    if (nnzRowD > 0) {
        k_expand_rows<<<nblk((long long)dRows * 32), 256, 0, s>>>(rowPtr_dd, dRows, rowOf);
        k_iota<<<nblk(nnzRowD), 256, 0, s>>>(iota, nnzRowD);
        PCK(seg_sort_pairs(tmp, colInd_dd, sortedCol, iota, srcIdx, nnzRowD, chunkNum, panelOff, s));
        k_heads<<<nblk(nnzRowD), 256, 0, s>>>(sortedCol, srcIdx, rowOf, nnzRowD, head);
        PCK(inclusive_sum(tmp, head, H, nnzRowD, s));
    }
    k_frag_count<<<nblk(chunkNum + 1), 256, 0, s>>>(panelOff, H, chunkNum, K, nf);
    // the fragment total is taken in 64 bits first: the int32 scan below is only meaningful when it fits
    long long *total64 = nullptr, htotal = 0;
    PCK(sc.alloc(&total64, 1));
    {
        size_t bytes = 0;
        cub::TransformInputIterator<long long, ToLongLong, const int *> it(nf, ToLongLong());
        PCK(cub::DeviceReduce::Sum(nullptr, bytes, it, total64, chunkNum + 1, s));
        PCK(tmp.reserve(bytes, s));
        PCK(cub::DeviceReduce::Sum(tmp.p, bytes, it, total64, chunkNum + 1, s));
    }
    PCK(cudaMemcpyAsync(&htotal, total64, sizeof(long long), cudaMemcpyDeviceToHost, s));
    PCK(cudaStreamSynchronize(s));
    int totalFrags = 0;
    if (fragment_count_status(htotal, K) != MX_OK) {
        *status = MX_ERR_OVERFLOW;
        PCK(cudaMemsetAsync(T.chunkPtr, 0, ((size_t)chunkNum + 1) * sizeof(int), s));
    } else {
        totalFrags = (int)htotal;
        PCK(exclusive_sum(tmp, nf, T.chunkPtr, chunkNum + 1, s));
    }
    T.totalFrags = totalFrags;
    PCK(dalloc(&T.AToX, (size_t)totalFrags * K + 8, s));  // +slack: bulk copies round up to 16 bytes
    PCK(dalloc((B **)&T.fragBit, (size_t)totalFrags + 8, s));
    PCK(dalloc(&T.fragPtr, (size_t)totalFrags + 1 + 8, s));
    PCK(dalloc((V **)&T.tcVal, (size_t)nnzRowD + 16, s));
    PCK(sc.alloc(&pc, (size_t)totalFrags + 1));
    PCK(sc.alloc(&entFrag, (size_t)nnzRowD));
    PCK(sc.alloc(&entBit, (size_t)nnzRowD));
    PCK(cudaMemsetAsync(T.AToX, 0, (size_t)totalFrags * K * sizeof(int), s));
    PCK(cudaMemsetAsync(T.fragBit, 0, (size_t)totalFrags * sizeof(B), s));
    if (*status == MX_OK && nnzRowD > 0) {
        k_atox_bits<B><<<nblk(nnzRowD), 256, 0, s>>>(sortedCol, srcIdx, rowOf, head, H, panelOff, T.chunkPtr, nnzRowD, K,
                                                     T.AToX, (B *)T.fragBit, entFrag, entBit);
    }
    k_popc<B><<<nblk(totalFrags + 1), 256, 0, s>>>((const B *)T.fragBit, totalFrags, pc);
    PCK(exclusive_sum(tmp, pc, T.fragPtr, totalFrags + 1, s));
    if (*status == MX_OK && nnzRowD > 0) {
        k_tile_vals<V, B><<<nblk(nnzRowD), 256, 0, s>>>(srcIdx, entFrag, entBit, (const B *)T.fragBit, T.fragPtr, val_dd,
                                                        nnzRowD, (V *)T.tcVal);
    }
    PCK(cudaGetLastError());
    PCK(cudaStreamSynchronize(s));
    return cudaSuccess;
}

// rows that are hot under a GLOBAL row cut: count above the cut's, or equal and not after the cut's row
__global__ void k_count_hot_global(const int *__restrict__ rowCntD, int n_rows, int cutCount, long long cutRow,
                                   long long rowOffset, int *__restrict__ out) {
    int r = blockIdx.x * blockDim.x + threadIdx.x;
    bool hot = false;
    if (r < n_rows) {
        const int c = rowCntD[r];
        hot = c > cutCount || (c == cutCount && rowOffset + r <= cutRow);
    }
    const unsigned m = __ballot_sync(0xffffffffu, hot);
    if ((threadIdx.x & 31) == 0 && m) atomicAdd(out, __popc(m));
}

// G (may be null): the rankings of a matrix whose rows are spread over several GPUs.  col_counts = column counts of
// the WHOLE matrix, nnz = its non-zero count (the tau thresholds are fractions of it); with has_row_cut the hot rows
// are those above the whole matrix's row cut.  rows_only_out: stop after the per-row counts inside the hot columns and
// copy them there (what the caller all-gathers to find the global row cut).
template <typename V, typename B>
cudaError_t partition_t(const CsrDev &A, float tau_c, float tau_r, PartArrays &P, mx_partition_stats &st, int *status,
                        cudaStream_t s, const GlobalRanking *G, int *rows_only_out) {
    *status = MX_OK;
    const int R = A.n_rows, C = A.n_cols, nnz = A.nnz;
    const int nnzCut = G ? (int)G->nnz : nnz;  // what the tau fractions refer to
    TempBuf tmp;
    Scratch sc(s);
    int *colCnt = nullptr, *iota = nullptr, *sortedCnt = nullptr, *colOrder = nullptr, *pref = nullptr, *cut = nullptr,
        *rankOf = nullptr, *isS = nullptr, *sidx = nullptr, *colMap = nullptr, *rowCntD = nullptr,
        *sortedRCnt = nullptr, *rowOrder = nullptr, *hotPos = nullptr, *resLen = nullptr, *Kdd = nullptr,
        *Pdd = nullptr, *Kcd = nullptr, *Pcd = nullptr, *Pdd2 = nullptr, *Kcd2 = nullptr,
        *Pcd2 = nullptr;
    const int N = R > C ? R : C;
    PCK(sc.alloc(&colCnt, (size_t)C));
    PCK(sc.alloc(&iota, (size_t)N));
    PCK(sc.alloc(&sortedCnt, (size_t)C));
    PCK(sc.alloc(&colOrder, (size_t)C));
    PCK(sc.alloc(&pref, (size_t)N));
    PCK(sc.alloc(&cut, 2));
    // 1-3: column histogram, ranking, tau_c cut
    if (G && G->col_counts) {
        PCK(cudaMemcpyAsync(colCnt, G->col_counts, (size_t)C * sizeof(int), cudaMemcpyDeviceToDevice, s));
    } else {
        PCK(cudaMemsetAsync(colCnt, 0, (size_t)C * sizeof(int), s));
        if (nnz > 0) k_col_hist<<<std::min(nblk(nnz), 148 * 16), 256, 0, s>>>(A.col_ind, nnz, colCnt);
    }
    k_iota<<<nblk(N), 256, 0, s>>>(iota, N);
    PCK(sort_desc_pairs(tmp, colCnt, sortedCnt, iota, colOrder, C, s));
    PCK(inclusive_sum(tmp, sortedCnt, pref, C, s));
    const int dColsNnz = nnzCut * tau_c;  // int * float -> float product, truncated (reference :1131)
    int hcut[2] = {0, 0};
    PCK(cudaMemsetAsync(cut, 0, 2 * sizeof(int), s));
    // the reference scans the first rowA ranked columns (square matrix); a slab ranked on its own scans min(rows,
    // cols), a slab ranked with the whole matrix's counts scans like the whole (square) matrix
    const int colBound = G ? C : std::min(R, C);
    k_find_cut<<<nblk(colBound), 256, 0, s>>>(pref, colBound, dColsNnz, cut);
    PCK(cudaMemcpyAsync(hcut, cut, 2 * sizeof(int), cudaMemcpyDeviceToHost, s));
    PCK(cudaStreamSynchronize(s));
    const int dCols = hcut[0];
    int nnzColD = hcut[1];  // with global counts: of the whole matrix; the local figure follows from the row counts
    if (dCols == 0) {
        *status = MX_ERR_TAU;
        return cudaSuccess;
    }
    const int sCols = C - dCols;
    // 4: column map
    PCK(sc.alloc(&rankOf, (size_t)C));
    PCK(sc.alloc(&isS, (size_t)C));
    PCK(sc.alloc(&sidx, (size_t)C));
    PCK(sc.alloc(&colMap, (size_t)C));
    PCK(dalloc(&P.xperm, (size_t)C, s));
    k_fill<<<nblk(C), 256, 0, s>>>(isS, C, 1);
    k_mark_rank<<<nblk(dCols), 256, 0, s>>>(colOrder, dCols, rankOf, isS);
    PCK(exclusive_sum(tmp, isS, sidx, C, s));
    k_colmap<<<nblk(C), 256, 0, s>>>(isS, sidx, rankOf, dCols, C, colMap, P.xperm);
    // 5-6: row ranking inside D, tau_r cut
    PCK(sc.alloc(&rowCntD, (size_t)R));
    PCK(sc.alloc(&sortedRCnt, (size_t)R));
    PCK(sc.alloc(&rowOrder, (size_t)R));
    k_row_count_d<<<nblk((long long)R * 32), 256, 0, s>>>(A.row_ptr, A.col_ind, colMap, dCols, R, rowCntD);
    if (rows_only_out) {
        PCK(cudaMemcpyAsync(rows_only_out, rowCntD, (size_t)R * sizeof(int), cudaMemcpyDeviceToDevice, s));
        PCK(cudaStreamSynchronize(s));
        cudaFreeAsync(P.xperm, s);
        P.xperm = nullptr;
        return cudaSuccess;
    }
    PCK(sort_desc_pairs(tmp, rowCntD, sortedRCnt, iota, rowOrder, R, s));
    PCK(inclusive_sum(tmp, sortedRCnt, pref, R, s));
    if (G) {  // entries of THIS slab inside the hot columns
        if (R > 0) PCK(cudaMemcpyAsync(&nnzColD, pref + R - 1, sizeof(int), cudaMemcpyDeviceToHost, s));
        else nnzColD = 0;
    }
    int dRows = 0, nnzRowD = 0;
    if (G && G->has_row_cut) {
        // the whole matrix's ranking restricted to this slab is this slab's own ranking, so its hot rows are a prefix
        // of the local order: count them (at least one row, like the reference's cut)
        PCK(cudaMemsetAsync(cut, 0, 2 * sizeof(int), s));
        k_count_hot_global<<<nblk(std::max(R, 1)), 256, 0, s>>>(rowCntD, R, G->row_cut_count, G->row_cut_index,
                                                                 G->row_offset, cut);
        PCK(cudaMemcpyAsync(hcut, cut, sizeof(int), cudaMemcpyDeviceToHost, s));
        PCK(cudaStreamSynchronize(s));
        dRows = std::max(1, std::min(hcut[0], R));
        PCK(cudaMemcpyAsync(&nnzRowD, pref + dRows - 1, sizeof(int), cudaMemcpyDeviceToHost, s));
        PCK(cudaStreamSynchronize(s));
    } else {
        const int dRowsNnz = nnzCut * tau_r;  // fraction of the TOTAL nnz (reference :1249)
        PCK(cudaMemsetAsync(cut, 0, 2 * sizeof(int), s));
        k_find_cut<<<nblk(R), 256, 0, s>>>(pref, R, dRowsNnz, cut);
        PCK(cudaMemcpyAsync(hcut, cut, 2 * sizeof(int), cudaMemcpyDeviceToHost, s));
        PCK(cudaStreamSynchronize(s));
        dRows = hcut[0], nnzRowD = hcut[1];
    }
    if (dRows == 0) {
        *status = MX_ERR_TAU;
        return cudaSuccess;
    }
    const int nnzColS = nnz - nnzColD;
    const int sRows = R - dRows, nnzRowS = nnzColD - nnzRowD, nnzCD = nnzColS + nnzRowS;
    PCK(sc.alloc(&hotPos, (size_t)R));
    PCK(dalloc(&P.rId, (size_t)dRows, s));
    PCK(dalloc(&P.hotmask, (size_t)(R + 31) / 32, s));
    PCK(cudaMemsetAsync(P.hotmask, 0, ((size_t)(R + 31) / 32) * sizeof(uint32_t), s));
    k_fill<<<nblk(R), 256, 0, s>>>(hotPos, R, -1);
    k_mark_hot<<<nblk(dRows), 256, 0, s>>>(rowOrder, dRows, hotPos, P.hotmask, P.rId);
    // 7: row pointers of dd (lengths = the first dRows sorted counts) and of the residual
    PCK(dalloc(&P.rowPtr_dd, (size_t)dRows + 1, s));
    PCK(dalloc(&P.rowPtr_CD, (size_t)R + 1, s));
    PCK(sc.alloc(&resLen, (size_t)R + 1));
    PCK(exclusive_sum(tmp, sortedRCnt, P.rowPtr_dd, dRows, s));
    PCK(cudaMemcpyAsync(P.rowPtr_dd + dRows, &nnzRowD, sizeof(int), cudaMemcpyHostToDevice, s));
    k_res_len<<<nblk(R + 1), 256, 0, s>>>(A.row_ptr, rowCntD, hotPos, R, resLen);
    PCK(exclusive_sum(tmp, resLen, P.rowPtr_CD, R + 1, s));
    // 8: scatter + segmented sort + finalize
    PCK(sc.alloc(&Kdd, (size_t)nnzRowD));
    PCK(sc.alloc(&Pdd, (size_t)nnzRowD));
    PCK(sc.alloc(&Kcd, (size_t)nnzCD));
    PCK(sc.alloc(&Pcd, (size_t)nnzCD));
    PCK(sc.alloc(&Pdd2, (size_t)nnzRowD));
    PCK(sc.alloc(&Kcd2, (size_t)nnzCD));
    PCK(sc.alloc(&Pcd2, (size_t)nnzCD));
    PCK(dalloc(&P.colInd_dd, (size_t)nnzRowD, s));
    PCK(dalloc(&P.colInd_CD, (size_t)nnzCD, s));
    PCK(dalloc((V **)&P.val_dd, (size_t)nnzRowD, s));
    PCK(dalloc((V **)&P.val_CD, (size_t)nnzCD, s));
    k_scatter<<<nblk((long long)R * 32), 256, 0, s>>>(A.row_ptr, A.col_ind, colMap, hotPos, P.rowPtr_dd, P.rowPtr_CD,
                                                      dCols, sCols, R, Kdd, Pdd, Kcd, Pcd);
    PCK(seg_sort_pairs(tmp, Kdd, P.colInd_dd, Pdd, Pdd2, nnzRowD, dRows, P.rowPtr_dd, s));
    PCK(seg_sort_pairs(tmp, Kcd, Kcd2, Pcd, Pcd2, nnzCD, R, P.rowPtr_CD, s));
    if (nnzRowD > 0)
        k_gather_vals<V><<<nblk(nnzRowD), 256, 0, s>>>(Pdd2, (const V *)A.val, nnzRowD, (V *)P.val_dd);
    if (nnzCD > 0)
        k_finalize_cd<V><<<nblk(nnzCD), 256, 0, s>>>(Kcd2, Pcd2, (const V *)A.val, nnzCD, dCols, sCols, P.colInd_CD,
                                                     (V *)P.val_CD);
    PCK(cudaGetLastError());
    // 9: tiles
    int tstatus = MX_OK;
    PCK((tiles_from_dd_t<V, B>(dRows, nnzRowD, P.rowPtr_dd, P.colInd_dd, (const V *)P.val_dd, P.tiles, &tstatus, s)));
    P.tiles.dCols = dCols;
    *status = tstatus;
    st.dCols = dCols;
    st.nnzColD = nnzColD;
    st.sCols = sCols;
    st.nnzColS = nnzColS;
    st.dRows = dRows;
    st.nnzRowD = nnzRowD;
    st.sRows = sRows;
    st.nnzRowS = nnzRowS;
    st.chunkNum = P.tiles.chunkNum;
    st.totalFrags = P.tiles.totalFrags;
    st.nnzCD = nnzCD;
    st.fragK = sizeof(B) == 8 ? 8 : 4;
    st.tc_nnz_ratio = (double)nnzRowD / ((double)P.tiles.totalFrags * 8 * st.fragK);
    st.active = 1;
    PCK(cudaStreamSynchronize(s));
    return cudaSuccess;
}

}  // namespace

// The reference indexes fragments, and the K x-index slots of every fragment, with its int32 index type
// (sparse_AToX_index[chunkPtr[p] * fragK + s], test/test_autotc_spmv.cpp:1384-1404): a panel decomposition whose slot
// count does not fit is refused rather than wrapped.
int fragment_count_status(long long total_frags, int K) {
    if (total_frags < 0 || total_frags + 1 > 2147483647LL || total_frags * K > 2147483647LL) return MX_ERR_OVERFLOW;
    return MX_OK;
}

cudaError_t partition_run(int dtype, const CsrDev &A, float tau_c, float tau_r, PartArrays &P, mx_partition_stats &st,
                          int *status, cudaStream_t s, const GlobalRanking *G) {
    if (dtype == MX_FP64) return partition_t<double, uint32_t>(A, tau_c, tau_r, P, st, status, s, G, nullptr);
    return partition_t<__half, uint64_t>(A, tau_c, tau_r, P, st, status, s, G, nullptr);
}

cudaError_t partition_row_counts(int dtype, const CsrDev &A, float tau_c, const GlobalRanking *G, int *row_counts,
                                 int *status, cudaStream_t s) {
    PartArrays P;
    mx_partition_stats st{};
    if (dtype == MX_FP64) return partition_t<double, uint32_t>(A, tau_c, 0.f, P, st, status, s, G, row_counts);
    return partition_t<__half, uint64_t>(A, tau_c, 0.f, P, st, status, s, G, row_counts);
}

cudaError_t column_counts(const CsrDev &A, int *counts, cudaStream_t s) {
    PCK(cudaMemsetAsync(counts, 0, (size_t)A.n_cols * sizeof(int), s));
    if (A.nnz > 0) k_col_hist<<<std::min(nblk(A.nnz), 148 * 16), 256, 0, s>>>(A.col_ind, A.nnz, counts);
    return cudaGetLastError();
}

// The cut of a ranking: counts sorted descending (ties: lower index first), k = smallest prefix whose sum reaches
// `threshold` (at least 1); out = {k, prefix sum, count of the k-th element, index of the k-th element}; k = 0 when no
// prefix reaches it.
cudaError_t rank_cut(const int *counts, int n, int threshold, long long out[4], cudaStream_t s) {
    out[0] = out[1] = out[2] = out[3] = 0;
    if (n <= 0) return cudaSuccess;
    TempBuf tmp;
    Scratch sc(s);
    int *iota = nullptr, *sorted = nullptr, *order = nullptr, *pref = nullptr, *cut = nullptr;
    PCK(sc.alloc(&iota, (size_t)n));
    PCK(sc.alloc(&sorted, (size_t)n));
    PCK(sc.alloc(&order, (size_t)n));
    PCK(sc.alloc(&pref, (size_t)n));
    PCK(sc.alloc(&cut, 2));
    k_iota<<<nblk(n), 256, 0, s>>>(iota, n);
    PCK(sort_desc_pairs(tmp, counts, sorted, iota, order, n, s));
    PCK(inclusive_sum(tmp, sorted, pref, n, s));
    PCK(cudaMemsetAsync(cut, 0, 2 * sizeof(int), s));
    k_find_cut<<<nblk(n), 256, 0, s>>>(pref, n, threshold, cut);
    int hcut[2] = {0, 0};
    PCK(cudaMemcpyAsync(hcut, cut, 2 * sizeof(int), cudaMemcpyDeviceToHost, s));
    PCK(cudaStreamSynchronize(s));
    if (hcut[0] == 0) return cudaSuccess;
    int c = 0, idx = 0;
    PCK(cudaMemcpyAsync(&c, sorted + hcut[0] - 1, sizeof(int), cudaMemcpyDeviceToHost, s));
    PCK(cudaMemcpyAsync(&idx, order + hcut[0] - 1, sizeof(int), cudaMemcpyDeviceToHost, s));
    PCK(cudaStreamSynchronize(s));
    out[0] = hcut[0], out[1] = hcut[1], out[2] = c, out[3] = idx;
    return cudaSuccess;
}

cudaError_t tiles_from_dd(int dtype, int dRows, int nnzRowD, const int *rowPtr_dd, const int *colInd_dd,
                          const void *val_dd, TileArrays &T, int *status, cudaStream_t s) {
    if (dtype == MX_FP64)
        return tiles_from_dd_t<double, uint32_t>(dRows, nnzRowD, rowPtr_dd, colInd_dd, (const double *)val_dd, T,
                                                 status, s);
    return tiles_from_dd_t<__half, uint64_t>(dRows, nnzRowD, rowPtr_dd, colInd_dd, (const __half *)val_dd, T, status,
                                             s);
}

// index check of an uploaded matrix: grid-stride over the row pointers and the column indices
__global__ void k_validate_csr(const int *__restrict__ row_ptr, const int *__restrict__ col_ind, int n_rows, int n_cols,
                               int nnz, int *__restrict__ dev_err) {
    const long long stride = (long long)gridDim.x * blockDim.x, t0 = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    bool bad = false;
    for (long long r = t0; r < n_rows; r += stride) bad |= __ldg(row_ptr + r + 1) < __ldg(row_ptr + r);
    for (long long e = t0; e < nnz; e += stride) {
        const int c = __ldg(col_ind + e);
        bad |= c < 0 || c >= n_cols;
    }
    if (__any_sync(0xffffffffu, bad) && (threadIdx.x & 31) == 0) atomicOr(dev_err, DEVERR_INPUT);
}

cudaError_t validate_csr(int n_rows, int n_cols, int nnz, const int *row_ptr, const int *col_ind, int *dev_err,
                         cudaStream_t s) {
    const long long work = std::max<long long>(n_rows, nnz);
    if (work <= 0) return cudaSuccess;
    const int grid = (int)std::min<long long>((work + 255) / 256, 148 * 16);
    k_validate_csr<<<grid, 256, 0, s>>>(row_ptr, col_ind, n_rows, n_cols, nnz, dev_err);
    return cudaGetLastError();
}

__global__ void k_hotmask_from_rid(const int *__restrict__ rId, int dRows, uint32_t *__restrict__ hotmask) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= dRows) return;
    int r = rId[i];
    atomicOr(hotmask + (r >> 5), 1u << (r & 31));
}

cudaError_t hotmask_from_rid(const int *rId, int dRows, int n_rows, uint32_t **hotmask, cudaStream_t s) {
    const size_t words = ((size_t)n_rows + 31) / 32;
    cudaError_t e = cudaMallocAsync((void **)hotmask, (words > 0 ? words : 1) * sizeof(uint32_t), s);
    if (e != cudaSuccess) return e;
    if ((e = cudaMemsetAsync(*hotmask, 0, (words > 0 ? words : 1) * sizeof(uint32_t), s)) != cudaSuccess) return e;
    if (dRows > 0) k_hotmask_from_rid<<<(dRows + 255) / 256, 256, 0, s>>>(rId, dRows, *hotmask);
    return cudaGetLastError();
}

void part_arrays_free(PartArrays &P, cudaStream_t s) {
    void *bufs[] = {P.xperm, P.rId, P.hotmask, P.rowPtr_dd, P.colInd_dd, P.val_dd, P.rowPtr_CD, P.colInd_CD, P.val_CD};
    for (void *b : bufs)
        if (b) cudaFreeAsync(b, s);
    tile_arrays_free(P.tiles, s);
    P = PartArrays();
}

void tile_arrays_free(TileArrays &T, cudaStream_t s) {
    void *bufs[] = {T.chunkPtr, T.AToX, T.fragPtr, T.fragBit, T.tcVal};
    for (void *b : bufs)
        if (b) cudaFreeAsync(b, s);
    T = TileArrays();
}

}  // namespace mx
