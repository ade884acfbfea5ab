// Residual ("cold") CSR SpMV on the CUDA cores — the B200 counterpart of the reference's cdspmv
// (src/spmv_kernel/cdSpMV.cu:244-392 kernel, :395-491 wrapper).
//
// Work is split by non-zeros, not by rows: a tile is THREADS*IPT consecutive non-zeros, so a power-law
// row of 100 000 entries and a thousand rows of 4 entries cost the same.  Per tile:
//   A. every thread loads 4 consecutive column indices (one 128-bit load) and 4 values (64/2x128 bit),
//      gathers x through the read-only path, and writes the products to shared memory;
//   B. every thread then owns IPT consecutive products, walks the row ends that fall inside them and
//      emits finished rows; sums of rows that cross threads are joined by a key-segmented scan over the
//      tile (warp shuffles), so no atomics are used and the result is bit-reproducible;
//   C. rows that cross tiles leave a "carry" (tile's unfinished last row) and a "head" (first row that
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

// 16 bytes of padding after every 16 products: a thread's IPT consecutive products are then read with
// conflict-free 128-bit shared loads, and the 4 products written in phase A stay 16-byte aligned.
template <typename A>
__device__ __forceinline__ int pidx(int i) {
    return i + (i >> 4) * (16 / (int)sizeof(A));
}

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

template <typename V, bool HAS_TILE, bool ACCUM>
__device__ __forceinline__ void store_row(V *__restrict__ y, int r, typename AccOf<V>::T v,
                                          const typename AccOf<V>::T *__restrict__ ytile,
                                          const uint32_t *__restrict__ hotmask) {
    if (HAS_TILE) {
        if ((__ldg(hotmask + (r >> 5)) >> (r & 31)) & 1u) v += ytile[r];
    }
    if (ACCUM) v += to_acc(y[r]);
    from_acc(v, y + r);
}

template <typename V, int IPT, bool HAS_TILE, bool ACCUM>
__global__ void __launch_bounds__(RESID_THREADS)
    resid_kernel(const int *__restrict__ rowPtr, const int *__restrict__ colInd, const V *__restrict__ val,
                 const V *__restrict__ x, V *__restrict__ y, const typename AccOf<V>::T *__restrict__ ytile,
                 const uint32_t *__restrict__ hotmask, const int *__restrict__ tileRow,
                 typename AccOf<V>::T *__restrict__ carry, typename AccOf<V>::T *__restrict__ head, int n_rows,
                 int nnz) {
    using A = typename AccOf<V>::T;
    constexpr int THREADS = RESID_THREADS;
    constexpr int T = THREADS * IPT;
    constexpr int SMAX = T + 8;
    constexpr int PADW = 16 / (int)sizeof(A);
    __shared__ __align__(16) A sp[T + (T / 16) * PADW];
    __shared__ int sEnd[SMAX + 1];
    __shared__ A warpVal[THREADS / 32];
    __shared__ int warpKey[THREADS / 32];

    const int t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    const int base = t * T;  // nnz < 2^31, so base fits
    const int cnt = min(T, nnz - base);
    const int r0 = tileRow[t], rE = tileRow[t + 1];
    const int nEmit = rE - r0;
    const int ne = min(rE + 1, n_rows) - r0;  // row ends this tile may look at
    const bool inSmem = ne <= SMAX;
    if (inSmem) {
        for (int k = tid; k < ne; k += THREADS) sEnd[k] = rowPtr[r0 + 1 + k] - base;
        if (tid == 0) sEnd[ne] = INT_MAX;
    }
    const bool headOpen = (r0 < n_rows) && (rowPtr[r0] < base);

    // ---- phase A: products, striped over the tile in groups of 4 ----
    {
        const int *cbase = colInd + base;
        const V *vbase = val + base;
        int4 c[IPT / 4];
        A v[IPT / 4][4];
#pragma unroll
        for (int j = 0; j < IPT / 4; ++j) {
            const int i = (tid + j * THREADS) * 4;
            if (i + 3 < cnt) {
                c[j] = __ldg(reinterpret_cast<const int4 *>(cbase + i));
                if constexpr (sizeof(V) == 2) {
                    uint2 raw = __ldg(reinterpret_cast<const uint2 *>(vbase + i));
                    __half2 h01 = *reinterpret_cast<__half2 *>(&raw.x), h23 = *reinterpret_cast<__half2 *>(&raw.y);
                    float2 f01 = __half22float2(h01), f23 = __half22float2(h23);
                    v[j][0] = f01.x;
                    v[j][1] = f01.y;
                    v[j][2] = f23.x;
                    v[j][3] = f23.y;
                } else {
                    double2 d01 = __ldg(reinterpret_cast<const double2 *>(vbase + i));
                    double2 d23 = __ldg(reinterpret_cast<const double2 *>(vbase + i + 2));
                    v[j][0] = d01.x;
                    v[j][1] = d01.y;
                    v[j][2] = d23.x;
                    v[j][3] = d23.y;
                }
            } else {
                int cc[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    bool ok = i + q < cnt;
                    cc[q] = ok ? __ldg(cbase + i + q) : 0;
                    v[j][q] = ok ? to_acc(vbase[i + q]) : A(0);
                }
                c[j] = make_int4(cc[0], cc[1], cc[2], cc[3]);
            }
        }
#pragma unroll
        for (int j = 0; j < IPT / 4; ++j) {
            const int i = (tid + j * THREADS) * 4;
            // entries past the end of the matrix have value 0 and column 0: harmless
            A p0 = v[j][0] * to_acc(__ldg(x + c[j].x));
            A p1 = v[j][1] * to_acc(__ldg(x + c[j].y));
            A p2 = v[j][2] * to_acc(__ldg(x + c[j].z));
            A p3 = v[j][3] * to_acc(__ldg(x + c[j].w));
            A *dst = sp + pidx<A>(i);
            if constexpr (sizeof(A) == 4) {
                *reinterpret_cast<float4 *>(dst) = make_float4(p0, p1, p2, p3);
            } else {
                *reinterpret_cast<double2 *>(dst) = make_double2(p0, p1);
                *reinterpret_cast<double2 *>(dst + 2) = make_double2(p2, p3);
            }
        }
    }
    __syncthreads();

    // ---- phase B: each thread owns IPT consecutive products ----
    auto rowEnd = [&](int k) -> int {
        if (inSmem) return sEnd[k];
        return k < ne ? rowPtr[r0 + 1 + k] - base : INT_MAX;
    };
    const int a = tid * IPT;
    A p[IPT];
    {
        const A *src = sp + pidx<A>(a);  // IPT <= 16: the chunk never crosses a padding slot
        if constexpr (sizeof(A) == 4) {
#pragma unroll
            for (int q = 0; q < IPT / 4; ++q) {
                float4 f = *reinterpret_cast<const float4 *>(src + 4 * q);
                p[4 * q] = f.x;
                p[4 * q + 1] = f.y;
                p[4 * q + 2] = f.z;
                p[4 * q + 3] = f.w;
            }
        } else {
#pragma unroll
            for (int q = 0; q < IPT / 2; ++q) {
                double2 d = *reinterpret_cast<const double2 *>(src + 2 * q);
                p[2 * q] = d.x;
                p[2 * q + 1] = d.y;
            }
        }
    }
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
        if (headK < 0) {
            headK = k;
            headAcc = acc;
        } else {
            store_row<V, HAS_TILE, ACCUM>(y, r0 + k, acc, ytile, hotmask);
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
    A v = acc;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        int k2 = __shfl_up_sync(0xffffffffu, key, d);
        A v2 = __shfl_up_sync(0xffffffffu, v, d);
        if (lane >= d && k2 == key) v += v2;
    }
    if (lane == 31) {
        warpKey[w] = key;
        warpVal[w] = v;
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
    A pv = __shfl_up_sync(0xffffffffu, v, 1);
    if (lane == 0) {
        pk = ck;
        pv = cv;
    } else if (pk == ck) {
        pv += cv;
    }
    if (headK >= 0) {
        A hv = headAcc + (pk == headK ? pv : A(0));
        if (headK == 0 && headOpen)
            head[t] = hv;  // the row began in an earlier tile: the fix-up kernel finishes it
        else
            store_row<V, HAS_TILE, ACCUM>(y, r0 + headK, hv, ytile, hotmask);
    }
    if (tid == THREADS - 1) carry[t] = v + (key == ck ? cv : A(0));
}

// Rows that span tiles: sum the carries of the tiles the row passed through, in tile order, then the head.
template <typename V, int IPT, bool HAS_TILE, bool ACCUM>
__global__ void resid_fixup_kernel(const int *__restrict__ rowPtr, V *__restrict__ y,
                                   const typename AccOf<V>::T *__restrict__ ytile,
                                   const uint32_t *__restrict__ hotmask, const int *__restrict__ tileRow,
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
    store_row<V, HAS_TILE, ACCUM>(y, r0, s, ytile, hotmask);
}

template <typename V>
__global__ void gather_kernel(const V *__restrict__ x, const int *__restrict__ perm, V *__restrict__ out, int n) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = __ldg(x + __ldg(perm + i));
}

template <typename V>
cudaError_t resid_spmv_t(const ResidPlan &P, const void *x, void *y, const void *ytile, const uint32_t *hotmask,
                         bool accumulate, cudaStream_t s) {
    using A = typename AccOf<V>::T;
    constexpr int IPT = ResidCfg<V>::IPT;
    const bool hasTile = ytile != nullptr && hotmask != nullptr;
    dim3 grid(P.num_tiles), block(RESID_THREADS);
    int fgrid = (P.num_tiles - 1 + 127) / 128;
#define MX_LAUNCH(HT, AC)                                                                                         \
    do {                                                                                                          \
        resid_kernel<V, IPT, HT, AC><<<grid, block, 0, s>>>(P.row_ptr, P.col_ind, (const V *)P.val, (const V *)x, \
                                                            (V *)y, (const A *)ytile, hotmask, P.tile_row,       \
                                                            (A *)P.carry, (A *)P.head, P.n_rows, P.nnz);         \
        if (fgrid > 0)                                                                                            \
            resid_fixup_kernel<V, IPT, HT, AC><<<fgrid, 128, 0, s>>>(P.row_ptr, (V *)y, (const A *)ytile,        \
                                                                     hotmask, P.tile_row, (const A *)P.carry,   \
                                                                     (const A *)P.head, P.n_rows, P.num_tiles); \
    } while (0)
    if (hasTile) {
        if (accumulate)
            MX_LAUNCH(true, true);
        else
            MX_LAUNCH(true, false);
    } else {
        if (accumulate)
            MX_LAUNCH(false, true);
        else
            MX_LAUNCH(false, false);
    }
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
    if (dtype == MX_FP64) return resid_spmv_t<double>(P, x, y, ytile, hotmask, accumulate, s);
    return resid_spmv_t<__half>(P, x, y, ytile, hotmask, accumulate, s);
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
