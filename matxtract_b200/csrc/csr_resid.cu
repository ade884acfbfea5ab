// Residual ("cold") CSR SpMV on the CUDA cores — the B200 counterpart of the reference's cdspmv
// (src/spmv_kernel/cdSpMV.cu:244-392 kernel, :395-491 wrapper).
//
// Work is split by non-zeros, not by rows: a tile is THREADS*IPT consecutive non-zeros, so a power-law
// row of 100 000 entries and a thousand rows of 4 entries cost the same.  Per tile:
//   A. every thread loads its own IPT consecutive column indices and values with 128-bit read-only loads
//      (evict-first, so the stream does not displace x from L1), gathers x through the read-only path
//      and keeps the IPT products in registers — no shared-memory transposition;
//   B. it then walks the row ends that fall inside its products (the tile's slice of the row pointers
//      sits in shared memory as 16-bit offsets) and drops finished row sums into shared memory; sums of
//      rows that cross threads are joined by a key-segmented scan over the tile (warp shuffles), so no
//      atomics are used and the result is bit-reproducible;
//   C. a coalesced epilogue stores one row per thread (adding the tile-kernel contribution of hot rows);
//   D. rows that cross tiles leave a "carry" (tile's unfinished last row) and a "head" (first row that
//      began earlier); a second tiny kernel adds them in tile order.
// Every row of y is stored exactly once; rows that also have a tile-kernel contribution (flagged in
// `hotmask`) add it at that point, so there is no merge pass.
#include <climits>

#include "mx_internal.h"

namespace mx {
namespace {

template <typename V>
struct AccOf;
template <>
struct AccOf<double> {
    using T = double;
};
template <>
struct AccOf<__half> {
    using T = float;
};

__device__ __forceinline__ float to_acc(__half v) { return __half2float(v); }
__device__ __forceinline__ double to_acc(double v) { return v; }
__device__ __forceinline__ void from_acc(double a, double *o) { *o = a; }
__device__ __forceinline__ void from_acc(float a, __half *o) { *o = __float2half_rn(a); }

// How a finished row leaves the kernel.
enum OutMode : int {
    OUT_Y = 0,        // y[r] = sum (+ tile contribution of hot rows)
    OUT_Y_ACCUM = 1,  // y[r] += sum  (the reference's cdspmv adds into y, cdSpMV.cu:418,483)
    OUT_CARRIER = 2   // carrier[row_map[r]] = sum in the accumulate type (core-dense block run as CSR)
};

__global__ void tile_row_kernel(const int *__restrict__ rowPtr, int n_rows, int nnz, int tile_nnz, int num_tiles,
                                int *__restrict__ tile_row) {
    int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t > num_tiles) return;
    if (t == 0) {
        tile_row[0] = 0;
        return;
    }
    long long p = (long long)t * tile_nnz;
    if (p > nnz) p = nnz;
    int lo = 0, hi = n_rows;  // number of rows whose end is <= p
    while (lo < hi) {
        int mid = (lo + hi) >> 1;
        if (rowPtr[mid + 1] <= p)
            lo = mid + 1;
        else
            hi = mid;
    }
    tile_row[t] = lo;
}

template <typename V>
struct RowOut {
    using A = typename AccOf<V>::T;
    V *__restrict__ y;
    A *__restrict__ carrier_out;           // OUT_CARRIER
    const int *__restrict__ row_map;       // OUT_CARRIER
    const A *__restrict__ ytile;           // HAS_TILE: tile-half contribution per row
    const uint32_t *__restrict__ hotmask;  // HAS_TILE: bit r set when row r has one
};

template <typename V, bool HAS_TILE, int MODE>
__device__ __forceinline__ void store_row(const RowOut<V> &o, int r, typename AccOf<V>::T v) {
    if (MODE == OUT_CARRIER) {
        o.carrier_out[o.row_map[r]] = v;
        return;
    }
    if (HAS_TILE) {
        if ((__ldg(o.hotmask + (r >> 5)) >> (r & 31)) & 1u) v += o.ytile[r];
    }
    if (MODE == OUT_Y_ACCUM) v += to_acc(o.y[r]);
    from_acc(v, o.y + r);
}

// 128-bit read-only loads that do not displace the gathered x from L1
__device__ __forceinline__ int4 ldg_stream(const int4 *p) {
    int4 r;
    asm volatile("ld.global.nc.L1::evict_first.v4.s32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(p));
    return r;
}

template <typename V, int IPT, bool HAS_TILE, int MODE>
__global__ void __launch_bounds__(RESID_THREADS)
    resid_kernel(const int *__restrict__ rowPtr, const int *__restrict__ colInd, const V *__restrict__ val,
                 const V *__restrict__ x, RowOut<V> out, const int *__restrict__ tileRow,
                 typename AccOf<V>::T *__restrict__ carry, typename AccOf<V>::T *__restrict__ head, int n_rows,
                 int nnz) {
    using A = typename AccOf<V>::T;
    constexpr int THREADS = RESID_THREADS;
    constexpr int T = THREADS * IPT;
    constexpr int KMAX = T / 2;  // row ends a tile keeps in shared memory (more: slow path through global memory)
    __shared__ unsigned short sEnd[KMAX + 2];
    __shared__ A ysum[KMAX];
    __shared__ A warpVal[THREADS / 32];
    __shared__ int warpKey[THREADS / 32];

    const int t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    const int base = t * T;  // nnz < 2^31, so base fits
    const int cnt = min(T, nnz - base);
    const int a = tid * IPT;

    // ---- this thread's IPT consecutive column indices and values (blocked, 128-bit loads) ----
    int c[IPT];
    A v[IPT];
    if (a + IPT <= cnt) {
        const int4 *cp = reinterpret_cast<const int4 *>(colInd + base + a);
#pragma unroll
        for (int q = 0; q < IPT / 4; ++q) {
            int4 cc = ldg_stream(cp + q);
            c[4 * q] = cc.x;
            c[4 * q + 1] = cc.y;
            c[4 * q + 2] = cc.z;
            c[4 * q + 3] = cc.w;
        }
        if constexpr (sizeof(V) == 2) {
            const int4 *vp = reinterpret_cast<const int4 *>(val + base + a);
#pragma unroll
            for (int q = 0; q < IPT / 8; ++q) {
                int4 raw = ldg_stream(vp + q);
                const __half2 *h = reinterpret_cast<const __half2 *>(&raw);
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    float2 f = __half22float2(h[u]);
                    v[8 * q + 2 * u] = f.x;
                    v[8 * q + 2 * u + 1] = f.y;
                }
            }
        } else {
            const int4 *vp = reinterpret_cast<const int4 *>(val + base + a);
#pragma unroll
            for (int q = 0; q < IPT / 2; ++q) {
                int4 raw = ldg_stream(vp + q);
                const double *d = reinterpret_cast<const double *>(&raw);
                v[2 * q] = d[0];
                v[2 * q + 1] = d[1];
            }
        }
    } else {
#pragma unroll
        for (int j = 0; j < IPT; ++j) {
            const bool ok = a + j < cnt;
            c[j] = ok ? __ldg(colInd + base + a + j) : 0;
            v[j] = ok ? to_acc(val[base + a + j]) : A(0);  // past the end: value 0, column 0 (harmless)
        }
    }

    // ---- rows this tile looks at ----
    const int r0 = tileRow[t], rE = tileRow[t + 1];
    const int nEmit = rE - r0;                // rows that end inside this tile
    const int ne = min(rE + 1, n_rows) - r0;  // row ends the walk may compare against
    const bool inSmem = ne <= KMAX;
    if (inSmem) {
        for (int k = tid; k < ne; k += THREADS) sEnd[k] = (unsigned short)min(rowPtr[r0 + 1 + k] - base, 0xFFFF);
        if (tid == 0) sEnd[ne] = 0xFFFF;
    }
    const bool headOpen = (r0 < n_rows) && (rowPtr[r0] < base);  // first row began in an earlier tile

    // ---- products ----
    A p[IPT];
#pragma unroll
    for (int j = 0; j < IPT; ++j) p[j] = v[j] * to_acc(__ldg(x + c[j]));
    __syncthreads();

    auto rowEnd = [&](int k) -> int {
        if (inSmem) return sEnd[k];
        return k < ne ? rowPtr[r0 + 1 + k] - base : INT_MAX;
    };
    int k = 0;  // row (relative to r0) the thread's first product belongs to
    if (tid != 0) {
        int lo = 0, hi = ne;
        while (lo < hi) {
            int mid = (lo + hi) >> 1;
            if (rowEnd(mid) <= a)
                lo = mid + 1;
            else
                hi = mid;
        }
        k = lo;
    }
    A acc = A(0), headAcc = A(0);
    int headK = -1;
    int e = rowEnd(k);
    auto emit = [&]() {
        if (headK < 0) {  // first row this thread finishes: it may have begun in an earlier thread
            headK = k;
            headAcc = acc;
        } else if (inSmem) {
            ysum[k] = acc;
        } else {
            store_row<V, HAS_TILE, MODE>(out, r0 + k, acc);
        }
        acc = A(0);
        ++k;
        e = rowEnd(k);
    };
#pragma unroll
    for (int j = 0; j < IPT; ++j) {
        const int i = a + j;
        if (i < cnt) {
            while (i >= e) emit();
            acc += p[j];
        }
    }
    while (k < nEmit && e <= a + IPT) emit();

    // ---- key-segmented inclusive scan of the (row, partial) tails over the tile ----
    int key = k;
    A sv = acc;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        int k2 = __shfl_up_sync(0xffffffffu, key, d);
        A v2 = __shfl_up_sync(0xffffffffu, sv, d);
        if (lane >= d && k2 == key) sv += v2;
    }
    if (lane == 31) {
        warpKey[w] = key;
        warpVal[w] = sv;
    }
    __syncthreads();
    int ck = -1;  // carry into this warp
    A cv = A(0);
    if (w > 0) {
        ck = warpKey[w - 1];
        for (int u = 0; u < w; ++u)
            if (warpKey[u] == ck) cv += warpVal[u];
    }
    int pk = __shfl_up_sync(0xffffffffu, key, 1);
    A pv = __shfl_up_sync(0xffffffffu, sv, 1);
    if (lane == 0) {
        pk = ck;
        pv = cv;
    } else if (pk == ck) {
        pv += cv;
    }
    if (headK >= 0) {
        A hv = headAcc + (pk == headK ? pv : A(0));
        if (headK == 0 && headOpen)
            head[t] = hv;  // the fix-up kernel finishes rows that span tiles
        else if (inSmem)
            ysum[headK] = hv;
        else
            store_row<V, HAS_TILE, MODE>(out, r0 + headK, hv);
    }
    if (tid == THREADS - 1) carry[t] = sv + (key == ck ? cv : A(0));
    if (!inSmem) return;  // block-uniform
    __syncthreads();
    // ---- coalesced epilogue: one row per thread per pass ----
    for (int q = tid + (headOpen ? 1 : 0); q < nEmit; q += THREADS) store_row<V, HAS_TILE, MODE>(out, r0 + q, ysum[q]);
}

// Rows that span tiles: sum the carries of the tiles the row passed through, in tile order, then the head.
template <typename V, int IPT, bool HAS_TILE, int MODE>
__global__ void resid_fixup_kernel(const int *__restrict__ rowPtr, RowOut<V> out, const int *__restrict__ tileRow,
                                   const typename AccOf<V>::T *__restrict__ carry,
                                   const typename AccOf<V>::T *__restrict__ head, int n_rows, int num_tiles) {
    using A = typename AccOf<V>::T;
    constexpr int T = RESID_THREADS * IPT;
    int t = blockIdx.x * blockDim.x + threadIdx.x + 1;
    if (t >= num_tiles) return;
    int r0 = tileRow[t];
    if (r0 >= n_rows || tileRow[t + 1] <= r0) return;  // no row ends in this tile
    int start = rowPtr[r0];
    if (start >= t * T) return;  // the first row begins inside the tile
    A s = A(0);
    for (int u = start / T; u < t; ++u) s += carry[u];
    s += head[t];
    store_row<V, HAS_TILE, MODE>(out, r0, s);
}

template <typename V>
__global__ void gather_kernel(const V *__restrict__ x, const int *__restrict__ perm, V *__restrict__ out, int n) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = __ldg(x + __ldg(perm + i));
}

template <typename V>
cudaError_t resid_spmv_t(const ResidPlan &P, const void *x, void *y, const void *ytile, const uint32_t *hotmask,
                         int mode, const int *row_map, cudaStream_t s) {
    using A = typename AccOf<V>::T;
    constexpr int IPT = ResidCfg<V>::IPT;
    const bool hasTile = mode != OUT_CARRIER && ytile != nullptr && hotmask != nullptr;
    RowOut<V> out;
    out.y = (V *)y;
    out.carrier_out = (A *)y;
    out.row_map = row_map;
    out.ytile = (const A *)ytile;
    out.hotmask = hotmask;
    dim3 grid(P.num_tiles), block(RESID_THREADS);
    int fgrid = (P.num_tiles - 1 + 127) / 128;
#define MX_LAUNCH(HT, MD)                                                                                          \
    do {                                                                                                           \
        resid_kernel<V, IPT, HT, MD><<<grid, block, 0, s>>>(P.row_ptr, P.col_ind, (const V *)P.val, (const V *)x,  \
                                                            out, P.tile_row, (A *)P.carry, (A *)P.head, P.n_rows,  \
                                                            P.nnz);                                                \
        if (fgrid > 0)                                                                                             \
            resid_fixup_kernel<V, IPT, HT, MD><<<fgrid, 128, 0, s>>>(P.row_ptr, out, P.tile_row,                   \
                                                                     (const A *)P.carry, (const A *)P.head,       \
                                                                     P.n_rows, P.num_tiles);                      \
    } while (0)
    if (mode == OUT_CARRIER)
        MX_LAUNCH(false, OUT_CARRIER);
    else if (hasTile && mode == OUT_Y_ACCUM)
        MX_LAUNCH(true, OUT_Y_ACCUM);
    else if (hasTile)
        MX_LAUNCH(true, OUT_Y);
    else if (mode == OUT_Y_ACCUM)
        MX_LAUNCH(false, OUT_Y_ACCUM);
    else
        MX_LAUNCH(false, OUT_Y);
#undef MX_LAUNCH
    return cudaGetLastError();
}

}  // namespace

cudaError_t resid_plan_build(int dtype, ResidPlan &P, cudaStream_t s) {
    P.tile_nnz = RESID_THREADS * (dtype == MX_FP64 ? ResidCfg<double>::IPT : ResidCfg<__half>::IPT);
    P.num_tiles = P.nnz > 0 ? (int)(((long long)P.nnz + P.tile_nnz - 1) / P.tile_nnz) : 1;
    cudaError_t e;
    if ((e = cudaMalloc(&P.tile_row, sizeof(int) * (size_t)(P.num_tiles + 1))) != cudaSuccess) return e;
    if ((e = cudaMalloc(&P.carry, acc_bytes(dtype) * (size_t)P.num_tiles)) != cudaSuccess) return e;
    if ((e = cudaMalloc(&P.head, acc_bytes(dtype) * (size_t)P.num_tiles)) != cudaSuccess) return e;
    tile_row_kernel<<<(P.num_tiles + 1 + 255) / 256, 256, 0, s>>>(P.row_ptr, P.n_rows, P.nnz, P.tile_nnz, P.num_tiles,
                                                                  P.tile_row);
    return cudaGetLastError();
}

void resid_plan_free(ResidPlan &P) {
    cudaFree(P.tile_row);
    cudaFree(P.carry);
    cudaFree(P.head);
    P.tile_row = nullptr;
    P.carry = P.head = nullptr;
}

int resid_launches(const ResidPlan &P) { return P.num_tiles > 1 ? 2 : 1; }

cudaError_t resid_spmv(int dtype, const ResidPlan &P, const void *x, void *y, const void *ytile,
                       const uint32_t *hotmask, bool accumulate, int *, cudaStream_t s) {
    const int mode = accumulate ? OUT_Y_ACCUM : OUT_Y;
    if (dtype == MX_FP64) return resid_spmv_t<double>(P, x, y, ytile, hotmask, mode, nullptr, s);
    return resid_spmv_t<__half>(P, x, y, ytile, hotmask, mode, nullptr, s);
}

cudaError_t resid_spmv_to_carrier(int dtype, const ResidPlan &P, const void *x, void *carrier, const int *row_map,
                                  cudaStream_t s) {
    if (dtype == MX_FP64) return resid_spmv_t<double>(P, x, carrier, nullptr, nullptr, OUT_CARRIER, row_map, s);
    return resid_spmv_t<__half>(P, x, carrier, nullptr, nullptr, OUT_CARRIER, row_map, s);
}

cudaError_t gather_vector(int dtype, const void *x, const int *perm, void *out, int n, cudaStream_t s) {
    if (n <= 0) return cudaSuccess;
    int grid = (n + 255) / 256;
    if (dtype == MX_FP64)
        gather_kernel<double><<<grid, 256, 0, s>>>((const double *)x, perm, (double *)out, n);
    else
        gather_kernel<__half><<<grid, 256, 0, s>>>((const __half *)x, perm, (__half *)out, n);
    return cudaGetLastError();
}

}  // namespace mx
