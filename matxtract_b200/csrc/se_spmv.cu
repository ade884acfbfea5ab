// "Sparse-encode" executor of the core-dense block — the B200 counterpart of the reference's se_tcspmv_fp64 /
// se_tcspmv_fp16 (src/spmv_kernel/se_tcSpMV_fp64.cu:496-1170 host re-encoding, :87-493 kernel, :62-84 long-row sum;
// FP16 twin src/spmv_kernel/se_tcSpMV_fp16.cu), which the reference runs on the block when its fragments are poorly
// filled (test/test_autotc_spmv.cpp:1507,1518).
//
// The idea kept from that path: rows are bucketed by length and their entries are laid out so that a tensor-core MMA
// computes eight row sums at once with NO bitmap decode — A holds 8 rows x K consecutive entries, B holds, in column
// j, the x values gathered for row j's entries, and the row sums are the diagonal of the product.  Every lane loads
// one (FP64) or four (FP16) stored slots — value and column id, both coalesced — gathers x for its own slots, and
// issues the MMA.  What is different here: the layout is BUILT ON THE DEVICE (the reference re-encodes on the host
// with serial loops and per-block malloc), long rows are cut into bounded work units whose partial sums are added in
// a fixed order (no atomics, bit-reproducible), and FP16 accumulates in FP32.
//
// Layout (rows sorted by length, longest first; order[] maps a sorted position to the input row):
//   * long rows (length >= block_longest): one block per row; its entries are dealt K at a time to the 8 MMA rows,
//     8K entries per "slab"; the row's result is the sum of the 8 diagonal entries;
//   * all other rows: blocks of 8 consecutive sorted rows; slab k of a block holds entries [kK, kK+K) of each of its
//     rows, zero-padded; slabs are stored while their fill is >= threshold * 8K (the reference's rule,
//     se_tcSpMV_fp64.cu:1070-1083), what is left of the rows is the block's irregular tail, kept as CSR and added on
//     the CUDA cores by the finishing kernel (rows of 1-2 entries are all tail when threshold > 0.5);
//   * K = 4 for FP64 (mma.m8n8k4.f64), K = 16 for FP16 (mma.m16n8k16, f32 accumulate, upper 8 A rows zero).
#include <algorithm>

#include "device_prims.cuh"
#include "mx_internal.h"

namespace mx {
namespace {

#define SCK_(call)                        \
    do {                                  \
        cudaError_t e_ = (call);          \
        if (e_ != cudaSuccess) return e_; \
    } while (0)

constexpr int SE_SEG = 64;  // slabs per work unit

template <typename V>
struct SeCfg;
template <>
struct SeCfg<double> {
    static constexpr int K = 4;
    using A = double;
};
template <>
struct SeCfg<__half> {
    static constexpr int K = 16;
    using A = float;
};

// position of entry p (0..K-1) of MMA row i inside a slab's storage: the slot a lane loads for the MMA operand
template <int K>
__host__ __device__ __forceinline__ int slab_slot(int i, int p) {
    if constexpr (K == 4) {
        return i * 4 + p;  // lane 4i+p holds A[i][p] and B[p][i]
    } else {
        // m16n8k16: lane (g = i, t) holds A[g][2t], A[g][2t+1] (a0) and A[g][2t+8], A[g][2t+9] (a2): 4 slots per lane
        const int t = (p & 7) >> 1, j = (p & 1) + 2 * (p >> 3);
        return (4 * i + t) * 4 + j;
    }
}

__global__ void k_se_row_len(const int *__restrict__ rowPtr, int n, int *__restrict__ len, int *__restrict__ iota) {
    int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r < n) {
        len[r] = rowPtr[r + 1] - rowPtr[r];
        iota[r] = r;
    }
}

// number of leading entries of the descending array that are >= bound
__global__ void k_se_count_ge(const int *__restrict__ sortedLen, int n, int bound, int *__restrict__ out) {
    int lo = 0, hi = n;
    while (lo < hi) {
        int mid = (lo + hi) >> 1;
        if (sortedLen[mid] >= bound)
            lo = mid + 1;
        else
            hi = mid;
    }
    *out = lo;
}

template <int K>
__global__ void k_se_block_shape(const int *__restrict__ sortedLen, int n, int nLong, int numBlocks, double threshold,
                                 int *__restrict__ nslab, int *__restrict__ nunit) {
    int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b > numBlocks) return;
    int ns = 0;
    const double need = threshold * 8 * K;
    if (b < nLong) {
        const int L = sortedLen[b], rem = L % (8 * K);
        ns = L / (8 * K) + ((rem > 0 && (double)rem >= need) ? 1 : 0);
    } else if (b < numBlocks) {
        const int r0 = nLong + (b - nLong) * 8, r1 = min(r0 + 8, n);
        for (int k = 0;; ++k) {  // rows are sorted, so the fill only falls with k
            int fill = 0;
            for (int r = r0; r < r1; ++r) fill += min(K, max(0, sortedLen[r] - K * k));
            if (fill == 0 || (double)fill < need) break;
            ++ns;
        }
    }
    nslab[b] = ns;
    nunit[b] = (ns + SE_SEG - 1) / SE_SEG;
}

template <int K>
__global__ void k_se_tail_len(const int *__restrict__ sortedLen, const int *__restrict__ nslab, int n, int nLong,
                              int *__restrict__ tlen) {
    int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r > n) return;
    int t = 0;
    if (r < n) {
        const int L = sortedLen[r];
        const int kept = r < nLong ? nslab[r] * 8 * K : nslab[nLong + (r - nLong) / 8] * K;
        t = L - min(L, kept);
    }
    tlen[r] = t;
}

// one warp per block: writes the block's slabs (zero-padded) and the tails of its rows
template <typename V, int K>
__global__ void k_se_fill(const int *__restrict__ rowPtr, const int *__restrict__ colInd, const V *__restrict__ val,
                          const int *__restrict__ order, const int *__restrict__ slabPtr,
                          const int *__restrict__ tailPtr, int n, int nLong, int numBlocks, V *__restrict__ slabVal,
                          int *__restrict__ slabCol, V *__restrict__ tailVal, int *__restrict__ tailCol) {
    const int b = (int)(((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5), lane = threadIdx.x & 31;
    if (b >= numBlocks) return;
    const int s0 = slabPtr[b], ns = slabPtr[b + 1] - s0;
    constexpr int SLOTS = 8 * K;
    if (b < nLong) {
        const int ir = order[b], base = rowPtr[ir], L = rowPtr[ir + 1] - base;
        for (int s = 0; s < ns; ++s)
            for (int q = lane; q < SLOTS; q += 32) {  // q-th entry of the slab = entry q % K of MMA row q / K
                const int e = s * SLOTS + q;
                const size_t at = (size_t)(s0 + s) * SLOTS + slab_slot<K>(q / K, q % K);
                slabVal[at] = e < L ? val[base + e] : V(0);
                slabCol[at] = e < L ? colInd[base + e] : 0;
            }
        const int kept = min(L, ns * SLOTS), t0 = tailPtr[b];
        for (int e = kept + lane; e < L; e += 32) {
            tailVal[t0 + e - kept] = val[base + e];
            tailCol[t0 + e - kept] = colInd[base + e];
        }
    } else {
        const int r0 = nLong + (b - nLong) * 8;
        for (int i = 0; i < 8; ++i) {
            const int r = r0 + i;
            int base = 0, L = 0;
            if (r < n) {
                const int ir = order[r];
                base = rowPtr[ir];
                L = rowPtr[ir + 1] - base;
            }
            for (int e = lane; e < ns * K; e += 32) {
                const size_t at = (size_t)(s0 + e / K) * SLOTS + slab_slot<K>(i, e % K);
                slabVal[at] = e < L ? val[base + e] : V(0);
                slabCol[at] = e < L ? colInd[base + e] : 0;
            }
            if (r < n) {
                const int kept = min(L, ns * K), t0 = tailPtr[r];
                for (int e = kept + lane; e < L; e += 32) {
                    tailVal[t0 + e - kept] = val[base + e];
                    tailCol[t0 + e - kept] = colInd[base + e];
                }
            }
        }
    }
}

__global__ void k_se_units(const int *__restrict__ slabPtr, const int *__restrict__ unitPtr, int numBlocks,
                           int4 *__restrict__ unitDesc) {
    int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= numBlocks) return;
    const int s0 = slabPtr[b], s1 = slabPtr[b + 1], u0 = unitPtr[b], nu = unitPtr[b + 1] - u0;
    for (int u = 0; u < nu; ++u) unitDesc[u0 + u] = make_int4(b, s0 + u * SE_SEG, min(s1, s0 + (u + 1) * SE_SEG), 0);
}

__global__ void k_se_out_rows(const int *__restrict__ order, const int *__restrict__ row_map, int n,
                              int *__restrict__ outRow) {
    int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r < n) outRow[r] = row_map ? row_map[order[r]] : r;
}

__device__ __forceinline__ double ld_stream(const double *p) {
    double r;
    asm volatile("ld.global.nc.L1::no_allocate.f64 %0, [%1];" : "=d"(r) : "l"(p));
    return r;
}
__device__ __forceinline__ int ld_stream(const int *p) {
    int r;
    asm volatile("ld.global.nc.L1::no_allocate.s32 %0, [%1];" : "=r"(r) : "l"(p));
    return r;
}
__device__ __forceinline__ uint2 ld_stream(const uint2 *p) {
    uint2 r;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(r.x), "=r"(r.y) : "l"(p));
    return r;
}
__device__ __forceinline__ int4 ld_stream(const int4 *p) {
    int4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.s32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(p));
    return r;
}

// one warp per work unit: the slabs of the unit through the tensor cores, the 8 diagonal sums to partial[unit][0..7]
__global__ void se_kernel_fp64(const double *__restrict__ x, const double *__restrict__ slabVal,
                               const int *__restrict__ slabCol, const int4 *__restrict__ unitDesc, int numUnits,
                               double *__restrict__ partial) {
    const int u = (int)(((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5), lane = threadIdx.x & 31;
    if (u >= numUnits) return;
    const int4 d = __ldg(unitDesc + u);
    double c0 = 0.0, c1 = 0.0, e0 = 0.0, e1 = 0.0;  // two independent accumulator chains
    int s = d.y;
#pragma unroll 4
    for (; s + 1 < d.z; s += 2) {
        const size_t at = (size_t)s * 32 + lane;
        const double aA = ld_stream(slabVal + at), aB = ld_stream(slabVal + at + 32);
        const int cA = ld_stream(slabCol + at), cB = ld_stream(slabCol + at + 32);
        const double bA = __ldg(x + cA), bB = __ldg(x + cB);
        asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0,%1}, {%2}, {%3}, {%0,%1};"
                     : "+d"(c0), "+d"(c1)
                     : "d"(aA), "d"(bA));
        asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0,%1}, {%2}, {%3}, {%0,%1};"
                     : "+d"(e0), "+d"(e1)
                     : "d"(aB), "d"(bB));
    }
    if (s < d.z) {
        const size_t at = (size_t)s * 32 + lane;
        const double aA = ld_stream(slabVal + at);
        const double bA = __ldg(x + ld_stream(slabCol + at));
        asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0,%1}, {%2}, {%3}, {%0,%1};"
                     : "+d"(c0), "+d"(c1)
                     : "d"(aA), "d"(bA));
    }
    // lane l holds C[l/4][2(l%4)] and C[l/4][2(l%4)+1]: the diagonal entry of row m = l/4 sits where l%4 == m/2
    const int m = lane >> 2;
    if ((lane & 3) == (m >> 1)) partial[(size_t)u * 8 + m] = (m & 1) ? (c1 + e1) : (c0 + e0);
}

__global__ void se_kernel_fp16(const __half *__restrict__ x, const __half *__restrict__ slabVal,
                               const int *__restrict__ slabCol, const int4 *__restrict__ unitDesc, int numUnits,
                               float *__restrict__ partial) {
    const int u = (int)(((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5), lane = threadIdx.x & 31;
    if (u >= numUnits) return;
    const int4 d = __ldg(unitDesc + u);
    float c0 = 0.f, c1 = 0.f, c2 = 0.f, c3 = 0.f;
#pragma unroll 2
    for (int s = d.y; s < d.z; ++s) {
        const size_t at = (size_t)s * 128 + lane * 4;  // this lane's 4 slots
        const uint2 a = ld_stream(reinterpret_cast<const uint2 *>(slabVal + at));
        const int4 c = ld_stream(reinterpret_cast<const int4 *>(slabCol + at));
        const unsigned b0 = (unsigned)__half_as_ushort(__ldg(x + c.x)) | ((unsigned)__half_as_ushort(__ldg(x + c.y)) << 16);
        const unsigned b1 = (unsigned)__half_as_ushort(__ldg(x + c.z)) | ((unsigned)__half_as_ushort(__ldg(x + c.w)) << 16);
        const unsigned zero = 0u;  // A rows 8-15 are not used
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+f"(c0), "+f"(c1), "+f"(c2), "+f"(c3)
            : "r"(a.x), "r"(zero), "r"(a.y), "r"(zero), "r"(b0), "r"(b1));
    }
    // lane (g, t) holds C[g][2t], C[g][2t+1]: the diagonal entry of row g sits where t == g/2
    const int g = lane >> 2;
    if ((lane & 3) == (g >> 1)) partial[(size_t)u * 8 + g] = (g & 1) ? c1 : c0;
}

__device__ __forceinline__ void se_put(double *o, double v) { *o = v; }
__device__ __forceinline__ void se_put(float *o, float v) { *o = v; }
__device__ __forceinline__ void se_put(__half *o, float v) { *o = __float2half_rn(v); }
__device__ __forceinline__ double se_get(const double *o) { return *o; }
__device__ __forceinline__ float se_get(const float *o) { return *o; }
__device__ __forceinline__ float se_get(const __half *o) { return __half2float(*o); }
__device__ __forceinline__ double se_acc(double v) { return v; }
__device__ __forceinline__ float se_acc(__half v) { return __half2float(v); }

// one thread per sorted row: the partial sums of its block's units in unit order, then its irregular tail
template <typename V, typename OutT, bool ACCUM>
__global__ void se_finish_kernel(const V *__restrict__ x, const typename SeCfg<V>::A *__restrict__ partial,
                                 const int *__restrict__ unitPtr, const int *__restrict__ tailPtr,
                                 const V *__restrict__ tailVal, const int *__restrict__ tailCol,
                                 const int *__restrict__ outRow, int n, int nLong, OutT *__restrict__ out) {
    using A = typename SeCfg<V>::A;
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= n) return;
    A sum = A(0);
    if (r < nLong) {
        for (int u = unitPtr[r], u1 = unitPtr[r + 1]; u < u1; ++u)
#pragma unroll
            for (int i = 0; i < 8; ++i) sum += partial[(size_t)u * 8 + i];
    } else {
        const int b = nLong + (r - nLong) / 8, i = (r - nLong) & 7;
        for (int u = unitPtr[b], u1 = unitPtr[b + 1]; u < u1; ++u) sum += partial[(size_t)u * 8 + i];
    }
    for (int e = tailPtr[r], e1 = tailPtr[r + 1]; e < e1; ++e) sum += se_acc(tailVal[e]) * se_acc(__ldg(x + tailCol[e]));
    const int o = outRow[r];
    if (ACCUM) sum += (A)se_get(out + o);
    se_put(out + o, sum);
}

inline int nblk(long long n, int b = 256) { return (int)((n + b - 1) / b); }

template <typename V>
cudaError_t se_plan_build_t(SePlan &P, const int *rowPtr, const int *colInd, const V *val, const int *row_map,
                            cudaStream_t s) {
    constexpr int K = SeCfg<V>::K;
    const int n = P.n_rows;
    TempBuf tmp;
    int *len = nullptr, *iota = nullptr, *sortedLen = nullptr, *nslab = nullptr, *nunit = nullptr, *tlen = nullptr,
        *cnt = nullptr;
    auto release = [&]() {
        for (int *p : {len, iota, sortedLen, nslab, nunit, tlen, cnt})
            if (p) cudaFreeAsync(p, s);
    };
    auto fail = [&](cudaError_t e) {
        release();
        return e;
    };
#define SE_TRY(call)                            \
    do {                                        \
        cudaError_t e_ = (call);                \
        if (e_ != cudaSuccess) return fail(e_); \
    } while (0)
    const size_t n1 = (size_t)n + 1;
    SE_TRY(cudaMallocAsync(&len, n1 * sizeof(int), s));
    SE_TRY(cudaMallocAsync(&iota, n1 * sizeof(int), s));
    SE_TRY(cudaMallocAsync(&sortedLen, n1 * sizeof(int), s));
    SE_TRY(cudaMallocAsync(&cnt, sizeof(int), s));
    SE_TRY(cudaMallocAsync(&P.order, n1 * sizeof(int), s));
    SE_TRY(cudaMallocAsync(&P.outRow, n1 * sizeof(int), s));
    if (n > 0) {
        k_se_row_len<<<nblk(n), 256, 0, s>>>(rowPtr, n, len, iota);
        size_t bytes = 0;  // stable: rows of equal length keep their input order
        SE_TRY(cub::DeviceRadixSort::SortPairsDescending(nullptr, bytes, len, sortedLen, iota, P.order, n, 0, 32, s));
        SE_TRY(tmp.reserve(bytes, s));
        SE_TRY(cub::DeviceRadixSort::SortPairsDescending(tmp.p, bytes, len, sortedLen, iota, P.order, n, 0, 32, s));
        k_se_out_rows<<<nblk(n), 256, 0, s>>>(P.order, row_map, n, P.outRow);
    }
    k_se_count_ge<<<1, 1, 0, s>>>(sortedLen, n, P.block_longest, cnt);
    SE_TRY(cudaMemcpyAsync(&P.nLong, cnt, sizeof(int), cudaMemcpyDeviceToHost, s));
    SE_TRY(cudaStreamSynchronize(s));
    P.numBlocks = P.nLong + (n - P.nLong + 7) / 8;
    const size_t nb1 = (size_t)P.numBlocks + 1;
    SE_TRY(cudaMallocAsync(&nslab, nb1 * sizeof(int), s));
    SE_TRY(cudaMallocAsync(&nunit, nb1 * sizeof(int), s));
    SE_TRY(cudaMallocAsync(&tlen, n1 * sizeof(int), s));
    SE_TRY(cudaMallocAsync(&P.slabPtr, nb1 * sizeof(int), s));
    SE_TRY(cudaMallocAsync(&P.unitPtr, nb1 * sizeof(int), s));
    SE_TRY(cudaMallocAsync(&P.tailPtr, n1 * sizeof(int), s));
    k_se_block_shape<K><<<nblk(nb1), 256, 0, s>>>(sortedLen, n, P.nLong, P.numBlocks, P.threshold, nslab, nunit);
    k_se_tail_len<K><<<nblk(n1), 256, 0, s>>>(sortedLen, nslab, n, P.nLong, tlen);
    SE_TRY(exclusive_sum(tmp, nslab, P.slabPtr, (int)nb1, s));
    SE_TRY(exclusive_sum(tmp, nunit, P.unitPtr, (int)nb1, s));
    SE_TRY(exclusive_sum(tmp, tlen, P.tailPtr, (int)n1, s));
    int totals[3] = {0, 0, 0};
    SE_TRY(cudaMemcpyAsync(&totals[0], P.slabPtr + P.numBlocks, sizeof(int), cudaMemcpyDeviceToHost, s));
    SE_TRY(cudaMemcpyAsync(&totals[1], P.unitPtr + P.numBlocks, sizeof(int), cudaMemcpyDeviceToHost, s));
    SE_TRY(cudaMemcpyAsync(&totals[2], P.tailPtr + n, sizeof(int), cudaMemcpyDeviceToHost, s));
    SE_TRY(cudaStreamSynchronize(s));
    P.numSlabs = totals[0];
    P.numUnits = totals[1];
    P.tailNnz = totals[2];
    const size_t slots = (size_t)P.numSlabs * 8 * K;
    SE_TRY(cudaMallocAsync(&P.slabVal, (slots > 0 ? slots : 1) * sizeof(V), s));
    SE_TRY(cudaMallocAsync(&P.slabCol, (slots > 0 ? slots : 1) * sizeof(int), s));
    SE_TRY(cudaMallocAsync(&P.tailVal, (size_t)(P.tailNnz > 0 ? P.tailNnz : 1) * sizeof(V), s));
    SE_TRY(cudaMallocAsync(&P.tailCol, (size_t)(P.tailNnz > 0 ? P.tailNnz : 1) * sizeof(int), s));
    SE_TRY(cudaMallocAsync(&P.unitDesc, (size_t)(P.numUnits > 0 ? P.numUnits : 1) * sizeof(int4), s));
    SE_TRY(cudaMallocAsync(&P.partial, (size_t)(P.numUnits > 0 ? P.numUnits : 1) * 8 * sizeof(typename SeCfg<V>::A), s));
    if (P.numBlocks > 0) {
        k_se_fill<V, K><<<nblk((long long)P.numBlocks * 32), 256, 0, s>>>(
            rowPtr, colInd, val, P.order, P.slabPtr, P.tailPtr, n, P.nLong, P.numBlocks, (V *)P.slabVal, P.slabCol,
            (V *)P.tailVal, P.tailCol);
        k_se_units<<<nblk(P.numBlocks), 256, 0, s>>>(P.slabPtr, P.unitPtr, P.numBlocks, (int4 *)P.unitDesc);
    }
    SE_TRY(cudaGetLastError());
    SE_TRY(cudaStreamSynchronize(s));
#undef SE_TRY
    release();
    return cudaSuccess;
}

}  // namespace

cudaError_t se_plan_build(int dtype, SePlan &P, const int *rowPtr, const int *colInd, const void *val,
                          const int *row_map, cudaStream_t s) {
    if (P.warps_per_cta < 1) P.warps_per_cta = 1;
    if (P.warps_per_cta > 16) P.warps_per_cta = 16;
    if (P.block_longest < 5) P.block_longest = 5;  // rows of 1-4 entries are never "long"
    if (!(P.threshold >= 0.0)) P.threshold = 0.0;
    if (P.threshold > 1.0) P.threshold = 1.0;
    if (dtype == MX_FP64) return se_plan_build_t<double>(P, rowPtr, colInd, (const double *)val, row_map, s);
    return se_plan_build_t<__half>(P, rowPtr, colInd, (const __half *)val, row_map, s);
}

void se_plan_free(SePlan &P, cudaStream_t s) {
    void *bufs[] = {P.order, P.outRow, P.slabPtr, P.unitPtr, P.unitDesc, P.slabVal, P.slabCol,
                    P.tailPtr, P.tailVal, P.tailCol, P.partial};
    for (void *b : bufs)
        if (b) cudaFreeAsync(b, s);
    const int w = P.warps_per_cta, bl = P.block_longest;
    const double th = P.threshold;
    P = SePlan();
    P.warps_per_cta = w;
    P.block_longest = bl;
    P.threshold = th;
}

int se_launches(const SePlan &P) { return P.n_rows > 0 ? (P.numUnits > 0 ? 2 : 1) : 0; }

cudaError_t se_spmv(int dtype, const SePlan &P, const void *x, void *out, bool out_is_acc, bool accumulate,
                    cudaStream_t s) {
    if (P.n_rows <= 0) return cudaSuccess;
    const int threads = P.warps_per_cta * 32;
    if (P.numUnits > 0) {
        const int grid = (int)(((long long)P.numUnits * 32 + threads - 1) / threads);
        if (dtype == MX_FP64)
            se_kernel_fp64<<<grid, threads, 0, s>>>((const double *)x, (const double *)P.slabVal, P.slabCol,
                                                    (const int4 *)P.unitDesc, P.numUnits, (double *)P.partial);
        else
            se_kernel_fp16<<<grid, threads, 0, s>>>((const __half *)x, (const __half *)P.slabVal, P.slabCol,
                                                    (const int4 *)P.unitDesc, P.numUnits, (float *)P.partial);
    }
    const int fg = (P.n_rows + 255) / 256;
#define SE_FIN(VT, OT, AC)                                                                                       \
    se_finish_kernel<VT, OT, AC><<<fg, 256, 0, s>>>((const VT *)x, (const SeCfg<VT>::A *)P.partial, P.unitPtr,    \
                                                    P.tailPtr, (const VT *)P.tailVal, P.tailCol, P.outRow,       \
                                                    P.n_rows, P.nLong, (OT *)out)
    if (dtype == MX_FP64) {
        if (accumulate)
            SE_FIN(double, double, true);
        else
            SE_FIN(double, double, false);
    } else if (out_is_acc) {
        SE_FIN(__half, float, false);
    } else if (accumulate) {
        SE_FIN(__half, __half, true);
    } else {
        SE_FIN(__half, __half, false);
    }
#undef SE_FIN
    return cudaGetLastError();
}

}  // namespace mx
