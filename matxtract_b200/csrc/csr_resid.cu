// Residual ("cold") CSR SpMV on the CUDA cores — the B200 counterpart of the reference's cdspmv
// (src/spmv_kernel/cdSpMV.cu:244-392 kernel, :395-491 wrapper).
//
// Work is split by non-zeros, not by rows: a tile is THREADS*IPT consecutive non-zeros, so a power-law
// row of 100 000 entries and a thousand rows of 4 entries cost the same.  Per tile:
//   A. lane i of a warp takes non-zero i: column indices and values stream in with coalesced read-only
//      loads (evict-first, so the stream does not displace x from L1) and the x gathers coalesce wherever
//      consecutive non-zeros have consecutive columns (blocked / banded matrices); the products go to a
//      padded shared-memory buffer;
//   B. every thread then owns IPT consecutive products (conflict-free 128-bit shared loads).  The rows that
//      end inside the tile have set one bit each in a shared-memory mask, and recorded the lowest row
//      index per 32-non-zero word (rows without entries are taken out of the row space at plan time, so
//      ends are distinct): a thread reads the IPT bits over its products, knows which row its first bit
//      closes, and a branch-free walk drops finished row sums into shared memory.  What is left after a
//      thread's last closed row is joined to the next closing thread by a flag-segmented warp-shuffle
//      scan — no float atomics, so the result is bit-reproducible;
//   C. a coalesced epilogue stores one row per thread (adding the tile-kernel contribution of hot rows);
//   D. rows that cross tiles leave a "carry" (tile's unfinished last row) and a "head" (first row that
//      began earlier); a second tiny kernel adds them in tile order.
// Every row of y is stored exactly once; rows that also have a tile-kernel contribution (flagged in
// `hotmask`) add it at that point, so there is no merge pass.
#include <algorithm>
#include <climits>
#include <cstdlib>

#include "device_prims.cuh"
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
    OUT_CARRIER = 2,  // carrier[row_map[r]] = sum in the accumulate type (core-dense block run as CSR)
    OUT_Y_PEERS = 3   // y_peer[g][row_offset + r] = sum for every GPU g of the box: the y all-gather, fused
};
__host__ __device__ constexpr bool is_peers(int m) { return m == OUT_Y_PEERS; }
__host__ __device__ constexpr bool is_accum(int m) { return m == OUT_Y_ACCUM; }
constexpr int MAX_PEERS = 8;
constexpr int PEER_VEC_FLAG = 0x100;

// tile_row[t] = number of (non-empty) rows whose end lies at or before the first non-zero of tile t
__global__ void tile_row_kernel(const int *__restrict__ cPtr, int m_rows, int nnz, int tile_nnz, int num_tiles,
                                int *__restrict__ tile_row) {
    int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t > num_tiles) return;
    long long p = (long long)t * tile_nnz;
    if (p > nnz) p = nnz;
    int lo = 0, hi = m_rows;
    while (lo < hi) {
        int mid = (lo + hi) >> 1;
        if (cPtr[mid + 1] <= p)
            lo = mid + 1;
        else
            hi = mid;
    }
    tile_row[t] = lo;
}

// Empty rows are taken out of the kernel's row space once, at plan time.
__global__ void nonempty_flag_kernel(const int *__restrict__ rowPtr, int n_rows, int *__restrict__ flag) {
    int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r <= n_rows) flag[r] = r < n_rows ? (rowPtr[r + 1] > rowPtr[r]) : 0;
}
__global__ void compress_rows_kernel(const int *__restrict__ rowPtr, const int *__restrict__ pos, int n_rows,
                                     int *__restrict__ cPtr, int *__restrict__ nzRow, int *__restrict__ emptyRow) {
    int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= n_rows) return;
    const int k = pos[r];  // non-empty rows before r
    if (rowPtr[r + 1] > rowPtr[r]) {
        nzRow[k] = r;
        cPtr[k + 1] = rowPtr[r + 1];
    } else {
        emptyRow[r - k] = r;
    }
    if (r == 0) cPtr[0] = 0;
}

template <typename V>
struct RowOut {
    using A = typename AccOf<V>::T;
    V *__restrict__ y;
    A *__restrict__ carrier_out;           // OUT_CARRIER
    const int *__restrict__ row_map;       // OUT_CARRIER
    const A *__restrict__ ytile;           // HAS_TILE: tile-half contribution per row
    const uint32_t *__restrict__ hotmask;  // HAS_TILE: bit r set when row r has one
    const int *__restrict__ nzRow;         // k-th non-empty row -> row index (null: no empty rows, identity)
    V *peer_y[MAX_PEERS];                  // OUT_Y_PEERS: every GPU's full-length y (peer-mapped), this GPU's included
    int n_peers;
    long long row_offset;                  // OUT_Y_PEERS: first row of this GPU's slab in the full y
    // OUT_Y_PEERS with multicast stores: carrier_out (unused in that mode) carries the NVLink multicast address of
    // the same y buffers, or null.  A member of its own changed the register allocation of every variant of the
    // kernel (all up to the launch-bound cap) and cost 4 % on the single-GPU product.
    __device__ __forceinline__ V *multicast() const { return reinterpret_cast<V *>(carrier_out); }
    // OUT_Y_PEERS: n_peers carries PEER_VEC_FLAG when every peer buffer is 16-byte aligned (16-byte row vectors allowed)
    __device__ __forceinline__ int peers() const { return n_peers & 0xff; }
    __device__ __forceinline__ bool vec_ok() const { return (n_peers & PEER_VEC_FLAG) != 0; }
};

// one store to a multicast address: the switch writes it into every GPU's copy of the buffer
__device__ __forceinline__ void multicast_store64(double *mc, double v) {
    asm volatile("multimem.st.relaxed.sys.global.f64 [%0], %1;" ::"l"(mc), "d"(v) : "memory");
}
__device__ __forceinline__ void multicast_store32(void *mc, unsigned v) {
    asm volatile("multimem.st.relaxed.sys.global.b32 [%0], %1;" ::"l"(mc), "r"(v) : "memory");
}

// the row's final value: its sum plus what the tile half and (when accumulating) the old y contribute
template <typename V, bool HAS_TILE, int MODE>
__device__ __forceinline__ typename AccOf<V>::T row_value(const RowOut<V> &o, int r, typename AccOf<V>::T v) {
    if (HAS_TILE) {
        if ((__ldg(o.hotmask + (r >> 5)) >> (r & 31)) & 1u) v += o.ytile[r];
    }
    if (is_accum(MODE)) v += to_acc(o.y[r]);
    return v;
}

// plain stores into every GPU's y over NVLink: consecutive rows of a warp make contiguous segments, and the traffic
// overlaps the rest of the kernel (which is bound by x gathers, not by NVLink)
template <typename V>
__device__ __forceinline__ void store_peers(const RowOut<V> &o, int r, typename AccOf<V>::T v) {
#pragma unroll
    for (int g = 0; g < MAX_PEERS; ++g)
        if (g < o.peers()) from_acc(v, o.peer_y[g] + o.row_offset + r);
}

// The y exchange of a tile's finished rows as 16-byte vectors.  `stage[q]` holds the final value (value type) of the
// q-th row that ends in the tile, q in [qb, nEmit); rowOf(q) is its row index in this GPU's slab.  Rows of a tile are
// consecutive unless rows without entries lie between them, so the rows are cut into groups of VEC = 16 / sizeof(V)
// that start at a 16-byte boundary of y; a group whose rows are consecutive leaves as ONE 16-byte store per GPU (a
// warp then writes 512 contiguous bytes per GPU), the ragged head and tail and any group broken by a gap as scalars.
template <typename V, typename RowOf>
__device__ __forceinline__ void store_rows_peers_vec(const RowOut<V> &o, const V *stage, int qb, int nEmit, int tid,
                                                     int nthreads, RowOf rowOf) {
    constexpr int VEC = 16 / (int)sizeof(V);
    const int n = nEmit - qb;
    if (n <= 0) return;
    const long long g0 = o.row_offset + rowOf(qb);
    int lead = (int)((VEC - (g0 & (VEC - 1))) & (VEC - 1));
    if (lead > n) lead = n;
    const int nGroups = (n - lead) / VEC, tail0 = qb + lead + nGroups * VEC;
    for (int i = tid; i < nGroups; i += nthreads) {
        const int qs = qb + lead + i * VEC;
        const int rf = rowOf(qs), rl = rowOf(qs + VEC - 1);
        if (rl - rf == VEC - 1 && ((o.row_offset + rf) & (VEC - 1)) == 0) {
            int4 pk;
            if constexpr (sizeof(V) == 8) {
                const double a = stage[qs], b = stage[qs + 1];
                pk.x = __double2loint(a), pk.y = __double2hiint(a), pk.z = __double2loint(b), pk.w = __double2hiint(b);
            } else {
                unsigned u[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) u[j] = (unsigned)__half_as_ushort(stage[qs + j]);
                pk.x = (int)(u[0] | (u[1] << 16)), pk.y = (int)(u[2] | (u[3] << 16));
                pk.z = (int)(u[4] | (u[5] << 16)), pk.w = (int)(u[6] | (u[7] << 16));
            }
#pragma unroll
            for (int g = 0; g < MAX_PEERS; ++g)
                if (g < o.peers()) *reinterpret_cast<int4 *>(o.peer_y[g] + o.row_offset + rf) = pk;
        } else {
#pragma unroll
            for (int j = 0; j < VEC; ++j) {
                const long long at = o.row_offset + rowOf(qs + j);
#pragma unroll
                for (int g = 0; g < MAX_PEERS; ++g)
                    if (g < o.peers()) o.peer_y[g][at] = stage[qs + j];
            }
        }
    }
    // ragged ends: rows [qb, qb + lead) and [tail0, nEmit)
    const int nEnds = lead + (nEmit - tail0);
    for (int i = tid; i < nEnds; i += nthreads) {
        const int q = i < lead ? qb + i : tail0 + (i - lead);
        const long long at = o.row_offset + rowOf(q);
#pragma unroll
        for (int g = 0; g < MAX_PEERS; ++g)
            if (g < o.peers()) o.peer_y[g][at] = stage[q];
    }
}

template <typename V, bool HAS_TILE, int MODE>
__device__ __forceinline__ void store_row(const RowOut<V> &o, int r, typename AccOf<V>::T v) {
    if (MODE == OUT_CARRIER) {
        o.carrier_out[o.row_map[r]] = v;
        return;
    }
    if (HAS_TILE) {
        if ((__ldg(o.hotmask + (r >> 5)) >> (r & 31)) & 1u) v += o.ytile[r];
    }
    if (is_accum(MODE)) v += to_acc(o.y[r]);
    if (is_peers(MODE)) {
        if constexpr (sizeof(V) == 8) {
            if (o.multicast()) {
                multicast_store64(reinterpret_cast<double *>(o.multicast()) + o.row_offset + r, v);
                return;
            }
        }
        store_peers<V>(o, r, v);  // 2-byte rows cannot be multicast one by one: see store_rows_multicast16
        return;
    }
    from_acc(v, o.y + r);
}

// FP16 rows through the multicast address, called by all 32 lanes of a warp (valid: this lane has a row).  The
// smallest multicast store is 4 bytes, so a lane whose row starts an aligned pair and whose right neighbour holds the
// next row stores both; rows left single go to every GPU with plain 2-byte stores.
__device__ __forceinline__ void store_rows_multicast16(const RowOut<__half> &o, bool valid, int r, float v, int lane) {
    const unsigned h = (unsigned)__half_as_ushort(__float2half_rn(v));
    const unsigned hn = __shfl_down_sync(0xffffffffu, h, 1);
    const int rn = __shfl_down_sync(0xffffffffu, r, 1);
    const bool vn = __shfl_down_sync(0xffffffffu, (int)valid, 1) != 0;
    const bool pack = valid && vn && lane < 31 && rn == r + 1 && (((o.row_offset + r) & 1LL) == 0);
    const bool taken = __shfl_up_sync(0xffffffffu, (int)pack, 1) != 0 && lane > 0;
    if (pack)
        multicast_store32(o.multicast() + o.row_offset + r, h | (hn << 16));
    else if (valid && !taken)
        store_peers<__half>(o, r, v);
}

// read-only loads that do not displace the gathered x from L1 (L2 evict-first / evict-last cache-policy hints on the
// stream and on x were measured too: no effect on any configuration, so they are not used)
__device__ __forceinline__ int ldg_stream(const int *p) {
    int r;
    asm volatile("ld.global.nc.L1::evict_first.s32 %0, [%1];" : "=r"(r) : "l"(p));
    return r;
}
__device__ __forceinline__ float ldg_stream_val(const __half *p) {
    unsigned short r;
    asm volatile("ld.global.nc.L1::evict_first.u16 %0, [%1];" : "=h"(r) : "l"(p));
    return __half2float(__ushort_as_half(r));
}
__device__ __forceinline__ double ldg_stream_val(const double *p) {
    double r;
    asm volatile("ld.global.nc.L1::evict_first.f64 %0, [%1];" : "=d"(r) : "l"(p));
    return r;
}

// 16 bytes of padding after every 16 products: the striped stores of phase A and the 128-bit blocked
// loads of phase B are then both free of bank conflicts.
template <typename A>
__device__ __forceinline__ int pidx(int i) {
    return i + (i >> 4) * (16 / (int)sizeof(A));
}

// Programmatic dependent launch: the kernels of one product are chained so that a kernel's CTAs become resident while
// its predecessor drains.  A chained kernel reads only what no kernel of the product writes (the matrix, x) before
// dep_wait(); everything a predecessor produces, and every global write, comes after it.  Both instructions do
// nothing in a kernel that was launched without the attribute or has no dependent.
__device__ __forceinline__ void dep_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <typename... KArgs, typename... Args>
cudaError_t launch_chained(void (*kernel)(KArgs...), dim3 grid, dim3 block, cudaStream_t s, bool chained, size_t smem,
                           Args... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute at{};
    at.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &at;
    cfg.numAttrs = chained ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// Shared-memory working set of one tile (one per CTA in the one-tile-per-CTA kernel, one per thread group in the
// persistent kernel).
template <typename A, int T, int NW, bool DENSE = false>
struct __align__(16) TileSmem {
    static constexpr int PADW = 16 / (int)sizeof(A);
    A sp[T + (T / 16) * PADW];  // products, padded; reused for the sums of the rows that end in the tile
    // where the tile's rows end, in one of two encodings:
    union {
        struct {
            unsigned sFlag[T / 32];  // bit i set: a row ends after the tile's i-th non-zero
            int sFirst[T / 32];      // lowest row (relative) that ends inside the 32-nnz word
        };
        unsigned char sEnd[DENSE ? T : 16];  // DENSE: one byte per non-zero, 1 = a row ends after it
    };
    A warpTail[NW];
    int warpOpen[NW];
    int warpEnds[NW];  // DENSE: rows that end inside the warp's share of the tile
};

// barrier over the RESID_THREADS threads that work on one tile: the whole CTA, or one group of a persistent CTA
// (named barriers 1..GROUPS)
template <int GROUPS>
__device__ __forceinline__ void tile_sync(int grp) {
    if constexpr (GROUPS == 1)
        __syncthreads();
    else
        asm volatile("bar.sync %0, %1;" ::"r"(grp + 1), "n"(RESID_THREADS) : "memory");
}

// x[c]: from the shared-memory copy of the hot-column prefix when the kernel holds one, else through the read-only path
template <typename V, bool HOTX>
__device__ __forceinline__ V load_x(const V *__restrict__ x, const V *xs, int hotCols, int c) {
    if constexpr (HOTX) {
        if (c < hotCols) return xs[c];
    }
    return __ldg(x + c);
}

// One tile (T consecutive non-zeros) of the product, by the RESID_THREADS threads tid = 0..RESID_THREADS-1.
// DENSE selects how the row ends of a tile are marked.  false: one bit per non-zero in shared words plus the lowest row
// per word, set with two shared-memory atomics per row end - cheapest when a tile closes few rows.  true: one byte per
// non-zero set with plain stores, the row index of a thread's first end from a scan of the threads' end counts - no
// atomics, which serialise on the words neighbouring rows share when a tile closes hundreds of rows (a column-slab
// pass closes ~480 per tile: 3.4 % faster on the 1e9-non-zero shape; 1-3 % slower on the other benchmark shapes).
template <typename V, int IPT, bool HAS_TILE, int MODE, int GROUPS, bool HOTX, bool DENSE = false>
__device__ __forceinline__ void resid_tile(const int t, const int tid, const int grp, const int numTiles,
                                           TileSmem<typename AccOf<V>::T, RESID_THREADS * IPT, RESID_THREADS / 32, DENSE> &sm,
                                           const V *xs, const int hotCols, const int *__restrict__ cPtr,
                                           const int *__restrict__ colInd, const V *__restrict__ val,
                                           const V *__restrict__ x, const RowOut<V> &out,
                                           const int *__restrict__ tileRow, typename AccOf<V>::T *__restrict__ carry,
                                           typename AccOf<V>::T *__restrict__ head, int nnz, int prefetchTiles) {
    using A = typename AccOf<V>::T;
    constexpr int THREADS = RESID_THREADS;
    constexpr int T = THREADS * IPT;
    A *const sp = sm.sp;
    A *const ysum = sp;  // sums of the rows that end in this tile: reuses the buffer once the products are in registers
    unsigned *const sFlag = sm.sFlag;
    int *const sFirst = sm.sFirst;
    A *const warpTail = sm.warpTail;
    int *const warpOpen = sm.warpOpen;
    const int lane = tid & 31, w = tid >> 5;
    const int base = t * T;  // nnz < 2^31, so base fits
    const int cnt = min(T, nnz - base);

    // ---- phase A: lane <-> consecutive non-zeros: coalesced streams, and gathers that coalesce on runs of
    //      consecutive columns (a 4-wide lane mapping and a shared-memory x window were measured: both slower) ----
    int c[IPT];
    A v[IPT];
    const int *cb = colInd + base + tid;
    const V *vb = val + base + tid;
    if (cnt == T) {
#pragma unroll
        for (int j = 0; j < IPT; ++j) {
            c[j] = ldg_stream(cb + j * THREADS);
            v[j] = ldg_stream_val(vb + j * THREADS);
        }
    } else {
#pragma unroll
        for (int j = 0; j < IPT; ++j) {
            const bool ok = tid + j * THREADS < cnt;
            c[j] = ok ? ldg_stream(cb + j * THREADS) : 0;
            v[j] = ok ? ldg_stream_val(vb + j * THREADS) : A(0);  // past the end: value 0, column 0
        }
    }
    if (prefetchTiles > 0) {  // ask L2 for the streams of the tile that a CTA of the next wave will read
        const int tp = t + prefetchTiles;
        if (tp + 1 < numTiles) {
            constexpr int CL = T * 4 / 128, VL = T * (int)sizeof(V) / 128;
            const char *pc = reinterpret_cast<const char *>(colInd + (size_t)tp * T);
            const char *pv = reinterpret_cast<const char *>(val + (size_t)tp * T);
            for (int i = tid; i < CL + VL; i += THREADS) {
                const char *q = i < CL ? pc + i * 128 : pv + (i - CL) * 128;
                asm volatile("prefetch.global.L2 [%0];" ::"l"(q));
            }
        }
    }
    // Everything the later phases need from global memory is requested here, before the first wait: the tile's row
    // range, the ends of its first 2*THREADS rows and the head test travel together with the streams and the
    // gathers instead of forming a chain of dependent round trips between the barriers.
    const int r0 = __ldg(tileRow + t), nEmit = __ldg(tileRow + t + 1) - r0;  // rows that end inside this tile
    const int *ce = cPtr + r0;
    const int headPtr = __ldg(ce);  // < base: the first of those rows began in an earlier tile
    // ends are in [0, cnt): rows are non-empty, so they are distinct
    const int e0 = tid < nEmit ? __ldg(ce + 1 + tid) - base - 1 : -1;
    const int e1 = tid + THREADS < nEmit ? __ldg(ce + 1 + tid + THREADS) - base - 1 : -1;
    if constexpr (DENSE) {
        for (int i = tid; i < T / 16; i += THREADS) reinterpret_cast<uint4 *>(sm.sEnd)[i] = make_uint4(0u, 0u, 0u, 0u);
    } else {
        for (int i = tid; i < T / 32; i += THREADS) {
            sFlag[i] = 0u;
            sFirst[i] = INT_MAX;
        }
    }
#pragma unroll
    for (int j = 0; j < IPT; ++j) sp[pidx<A>(tid + j * THREADS)] = v[j] * to_acc(load_x<V, HOTX>(x, xs, hotCols, c[j]));
    const bool headOpen = headPtr < base;
    const int q0 = tid + (headOpen ? 1 : 0);  // the row this thread stores first in the epilogue
    const int rz = (out.nzRow && q0 < nEmit) ? __ldg(out.nzRow + r0 + q0) : r0 + q0;
    tile_sync<GROUPS>(grp);
    auto mark_end = [&](int e, int row) {  // rows are non-empty, so ends are distinct positions
        if constexpr (DENSE) {
            sm.sEnd[e] = 1;
        } else {
            atomicOr(&sFlag[e >> 5], 1u << (e & 31));
            atomicMin(&sFirst[e >> 5], row);
        }
    };
    if (e0 >= 0) mark_end(e0, tid);
    if (e1 >= 0) mark_end(e1, tid + THREADS);
    for (int kk = tid + 2 * THREADS; kk < nEmit; kk += 4 * THREADS) {  // further row ends, four loads in flight
        int e[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) e[j] = kk + j * THREADS < nEmit ? __ldg(ce + 1 + kk + j * THREADS) - base - 1 : -1;
#pragma unroll
        for (int j = 0; j < 4; ++j)
            if (e[j] >= 0) mark_end(e[j], kk + j * THREADS);
    }
    tile_sync<GROUPS>(grp);

    // ---- phase B: every thread owns IPT consecutive products ----
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
    // mask: bit j set when a row ends at this thread's j-th product; k0: the row (relative to r0) its first bit closes
    unsigned mask = 0u;
    int k0 = 0;
    if constexpr (DENSE) {
#pragma unroll
        for (int q = 0; q < IPT / 4; ++q) {  // four end bytes become four bits with one multiply
            const unsigned wv = reinterpret_cast<const unsigned *>(sm.sEnd + a)[q];
            mask |= (((wv * 0x01020408u) >> 24) & 0xfu) << (4 * q);
        }
        // k0 = row ends before this thread's first product: scan of the threads' counts
        const int myEnds = __popc(mask);
        int endsIncl = myEnds;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int o = __shfl_up_sync(0xffffffffu, endsIncl, d);
            if (lane >= d) endsIncl += o;
        }
        if (lane == 31) sm.warpEnds[w] = endsIncl;
        k0 = endsIncl - myEnds;
    } else {
        const unsigned word = sFlag[a >> 5];
        mask = (word >> (a & 31)) & ((1u << IPT) - 1u);
        k0 = sFirst[a >> 5] + __popc(word & ((1u << (a & 31)) - 1u));
    }
    const bool hasEnd = mask != 0u;
    tile_sync<GROUPS>(grp);  // every product is in registers: the buffer now holds row sums
    if constexpr (DENSE)
        for (int u = 0; u < w; ++u) k0 += sm.warpEnds[u];
    int k = k0;
    A acc = A(0);
#pragma unroll
    for (int j = 0; j < IPT; ++j) {  // branch-free walk: a set bit closes a row
        acc += p[j];
        if ((mask >> j) & 1u) {
            ysum[k] = acc;
            ++k;
            acc = A(0);
        }
    }

    // ---- what a thread has left after its last closed row belongs to a row closed by a later thread:
    //      segmented inclusive scan of these tails; a thread that closed a row starts a new segment ----
    const unsigned hm = __ballot_sync(0xffffffffu, hasEnd);
    const unsigned upto = hm & (0xffffffffu >> (31 - lane));  // lanes <= this one that closed a row
    const int segStart = upto ? 31 - __clz(upto) : 0;
    A sv = acc;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        A o = __shfl_up_sync(0xffffffffu, sv, d);
        if (lane - d >= segStart) sv += o;
    }
    A pv = __shfl_up_sync(0xffffffffu, sv, 1);  // tails left by the lanes before this one
    if (lane == 31) {
        warpTail[w] = sv;
        warpOpen[w] = hm == 0u;
    }
    tile_sync<GROUPS>(grp);
    A cv = A(0);  // tails left by earlier warps for the row that is open at this warp's start
    for (int u = w - 1; u >= 0; --u) {
        cv += warpTail[u];
        if (!warpOpen[u]) break;
    }
    const bool openToWarpStart = (hm & ((1u << lane) - 1u)) == 0u;  // no lane before this one closed a row
    if (lane == 0)
        pv = cv;
    else if (openToWarpStart)
        pv += cv;
    if (hasEnd) ysum[k0] += pv;  // the first row this thread closed began in earlier threads
    dep_wait();  // from here on: global writes, and the tile half's carrier is read
    if (tid == THREADS - 1) carry[t] = sv + (upto == 0u ? cv : A(0));
    tile_sync<GROUPS>(grp);

    // ---- coalesced epilogue: one row per thread per pass ----
    if (headOpen && nEmit > 0 && tid == 0) head[t] = ysum[0];  // the fix-up kernel finishes rows that span tiles
    if constexpr (is_peers(MODE) && sizeof(V) == 2) {
        if (out.multicast()) {  // warp-uniform loop: the lanes of a warp pair up their rows
            for (int qb = headOpen ? 1 : 0; qb < nEmit; qb += THREADS) {
                const int q = qb + tid;
                const bool valid = q < nEmit;
                int r = 0;
                A v = A(0);
                if (valid) {
                    r = q == q0 ? rz : (out.nzRow ? __ldg(out.nzRow + r0 + q) : r0 + q);
                    v = row_value<V, HAS_TILE, MODE>(out, r, ysum[q]);
                }
                store_rows_multicast16(out, valid, r, v, lane);
            }
            return;
        }
    }
    if constexpr (is_peers(MODE)) {
        // plain peer stores: stage the tile's finished rows in the value type, then send 16-byte vectors.  FP64 rows
        // are staged in place; FP16 rows go to the padding tail of the product buffer (T/2 halves), so a tile that
        // closes more rows than that keeps the one-row-per-thread path below.
        constexpr bool IN_PLACE = sizeof(V) == sizeof(A);
        const int qb = headOpen ? 1 : 0;
        if (out.vec_ok() && !out.multicast() && (IN_PLACE || nEmit <= T / 2)) {
            V *stage = IN_PLACE ? reinterpret_cast<V *>(ysum) : reinterpret_cast<V *>(sp + T);
            auto rowOf = [&](int q) { return out.nzRow ? __ldg(out.nzRow + r0 + q) : r0 + q; };
            for (int q = q0; q < nEmit; q += THREADS) {
                const int r = q == q0 ? rz : rowOf(q);
                A v = row_value<V, HAS_TILE, MODE>(out, r, ysum[q]);
                V o;
                from_acc(v, &o);
                stage[q] = o;
            }
            tile_sync<GROUPS>(grp);
            store_rows_peers_vec<V>(out, stage, qb, nEmit, tid, THREADS, rowOf);
            return;
        }
    }
    // One row per thread per round, EB rounds batched: the row indices of a batch are requested together, then
    // everything that depends on them (old y when accumulating, the tile half's carrier, the carrier's destination),
    // then the stores - three dependent round trips per batch instead of per round.  A tile of short rows closes many
    // rows (a column-slab pass: ~700), and one round at a time left the kernel waiting on these chains.
    constexpr int EB = 4;
    for (int qs = q0; qs < nEmit; qs += EB * THREADS) {
        int r[EB], dst[EB];
        A add[EB];
#pragma unroll
        for (int k = 0; k < EB; ++k) {
            const int q = qs + k * THREADS;
            r[k] = q < nEmit ? (q == q0 ? rz : (out.nzRow ? __ldg(out.nzRow + r0 + q) : r0 + q)) : -1;
        }
#pragma unroll
        for (int k = 0; k < EB; ++k) {
            dst[k] = r[k];
            add[k] = A(0);
            if (r[k] >= 0) {
                if (MODE == OUT_CARRIER) {
                    dst[k] = __ldg(out.row_map + r[k]);
                } else {
                    if (HAS_TILE) {
                        if ((__ldg(out.hotmask + (r[k] >> 5)) >> (r[k] & 31)) & 1u) add[k] = out.ytile[r[k]];
                    }
                    if (is_accum(MODE)) add[k] += to_acc(out.y[r[k]]);
                }
            }
        }
#pragma unroll
        for (int k = 0; k < EB; ++k) {
            if (r[k] < 0) continue;
            const A v = ysum[qs + k * THREADS] + add[k];
            if (MODE == OUT_CARRIER) {
                out.carrier_out[dst[k]] = v;
            } else if (is_peers(MODE)) {
                if constexpr (sizeof(V) == 8) {
                    if (out.multicast()) {
                        multicast_store64(reinterpret_cast<double *>(out.multicast()) + out.row_offset + r[k], v);
                        continue;
                    }
                }
                store_peers<V>(out, r[k], v);
            } else {
                from_acc(v, out.y + r[k]);
            }
        }
    }
}


template <typename V, int IPT, bool HAS_TILE, int MODE, bool DENSE = false>
__global__ void __launch_bounds__(RESID_THREADS, ResidCfg<V>::MINBLOCKS)
    resid_kernel(const int *__restrict__ cPtr, const int *__restrict__ colInd, const V *__restrict__ val,
                 const V *__restrict__ x, RowOut<V> out, const int *__restrict__ tileRow,
                 typename AccOf<V>::T *__restrict__ carry, typename AccOf<V>::T *__restrict__ head, int nnz,
                 int prefetchTiles) {
    __shared__ TileSmem<typename AccOf<V>::T, RESID_THREADS * IPT, RESID_THREADS / 32, DENSE> sm;
    dep_release();  // the fix-up launch may become resident; it waits for this grid to finish
    resid_tile<V, IPT, HAS_TILE, MODE, 1, false, DENSE>(blockIdx.x, threadIdx.x, 0, (int)gridDim.x, sm, nullptr, 0,
                                                        cPtr, colInd, val, x, out, tileRow, carry, head, nnz,
                                                        prefetchTiles);
}

// The same product with the hot-column prefix of x in shared memory.  In the extraction's column numbering the first
// dCols entries of x are the densest columns in rank order, so a prefix of them that fits one SM's shared memory can
// serve every gather of those columns without touching L1 or L2.  One persistent CTA per SM copies the prefix once
// (1-D bulk copies completing on an mbarrier, bounded wait) and then its HOTX_GROUPS groups of RESID_THREADS threads
// each run tiles like the CTAs of resid_kernel, synchronising on a named barrier of their own.
template <typename V>
struct HotxCfg;
template <>
struct HotxCfg<__half> {
    static constexpr int GROUPS = 8;  // 1024 threads: the same residency as the one-tile-per-CTA kernel (6 groups measured 40-55 % slower)
};
template <>
struct HotxCfg<double> {
    static constexpr int GROUPS = 4;
};
constexpr int HOTX_SMEM_LIMIT = 227 * 1024;

template <typename V, int IPT, bool HAS_TILE, int MODE>
__global__ void __launch_bounds__(RESID_THREADS *HotxCfg<V>::GROUPS, 1)
    resid_hotx_kernel(const int *__restrict__ cPtr, const int *__restrict__ colInd, const V *__restrict__ val,
                      const V *__restrict__ x, RowOut<V> out, const int *__restrict__ tileRow,
                      typename AccOf<V>::T *__restrict__ carry, typename AccOf<V>::T *__restrict__ head, int nnz,
                      int prefetchTiles, int numTiles, int hotCols, int *__restrict__ devErr) {
    constexpr int GROUPS = HotxCfg<V>::GROUPS;
    using TS = TileSmem<typename AccOf<V>::T, RESID_THREADS * IPT, RESID_THREADS / 32>;
    extern __shared__ __align__(16) unsigned char dyn[];
    uint64_t *bar = reinterpret_cast<uint64_t *>(dyn);  // first 16 bytes
    V *xs = reinterpret_cast<V *>(dyn + 16);
    const uint32_t xbytes = (uint32_t)hotCols * (uint32_t)sizeof(V);  // a multiple of 16 (the host rounds hotCols)
    const int grp = threadIdx.x / RESID_THREADS, tid = threadIdx.x % RESID_THREADS;
    TS &sm = reinterpret_cast<TS *>(dyn + 16 + xbytes)[grp];
    dep_release();
    if (threadIdx.x == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(bar)) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(xbytes) : "memory");
        constexpr uint32_t CHUNK = 32 * 1024;
        for (uint32_t off = 0; off < xbytes; off += CHUNK)
            bulk_g2s(reinterpret_cast<unsigned char *>(xs) + off, reinterpret_cast<const unsigned char *>(x) + off,
                     min(CHUNK, xbytes - off), bar);
    }
    __syncthreads();  // the barrier is initialised before anyone polls it
    if (!mbar_wait_bounded(bar)) {  // never expected; leaves a mark instead of spinning for ever
        if (threadIdx.x == 0 && devErr) atomicOr(devErr, DEVERR_TILE_RANGE);
        return;
    }
    for (int t = blockIdx.x * GROUPS + grp; t < numTiles; t += (int)gridDim.x * GROUPS) {
        resid_tile<V, IPT, HAS_TILE, MODE, GROUPS, true>(t, tid, grp, numTiles, sm, xs, hotCols, cPtr, colInd, val, x,
                                                         out, tileRow, carry, head, nnz, prefetchTiles);
        tile_sync<GROUPS>(grp);  // the group's buffers are free for its next tile
    }
}

// Rows that span tiles: sum the carries of the tiles the row passed through, in tile order, then the head.
// The same launch writes the empty rows (their y is 0, or the tile-half contribution).
template <typename V, int IPT, bool HAS_TILE, int MODE>
__global__ void resid_fixup_kernel(const int *__restrict__ cPtr, RowOut<V> out, const int *__restrict__ tileRow,
                                   const typename AccOf<V>::T *__restrict__ carry,
                                   const typename AccOf<V>::T *__restrict__ head, int m_rows, int num_tiles,
                                   const int *__restrict__ emptyRow, int n_empty) {
    using A = typename AccOf<V>::T;
    constexpr int T = RESID_THREADS * IPT;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    dep_release();
    dep_wait();  // needs every carry and head of the main launch
    if (i < n_empty) store_row<V, HAS_TILE, MODE>(out, emptyRow[i], A(0));
    const int t = i + 1;
    if (t >= num_tiles) return;
    const int r0 = tileRow[t];
    if (r0 >= m_rows || tileRow[t + 1] <= r0) return;  // no row ends in this tile
    const int start = cPtr[r0];
    if (start >= t * T) return;  // the first row begins inside the tile
    A s = A(0);
    for (int u = start / T; u < t; ++u) s += carry[u];
    s += head[t];
    store_row<V, HAS_TILE, MODE>(out, out.nzRow ? out.nzRow[r0] : r0, s);
}

__global__ void map_indices_kernel(const int *__restrict__ in, const int *__restrict__ map, int *__restrict__ out,
                                   long long n) {
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = __ldg(map + __ldg(in + i));
}

// this GPU's finished slab -> the same rows of every other GPU's y over NVLink: 16-byte stores for the part between
// the first and the last 16-byte boundary, single bytes for the ragged ends (a slab cut at an nnz-balanced row boundary
// rarely starts on one).  aligned = every destination has the source's alignment modulo 16; otherwise all by bytes.
__global__ void peer_push_kernel(const unsigned char *__restrict__ src, unsigned char *const *__restrict__ dst_table,
                                 long long nbytes, int aligned) {
    unsigned char *dst = dst_table[blockIdx.y];
    long long head = aligned ? (long long)((16u - (unsigned)((uintptr_t)src & 15u)) & 15u) : nbytes;
    if (head > nbytes) head = nbytes;
    const long long n16 = (nbytes - head) / 16, tail0 = head + n16 * 16;
    const int4 *s16 = reinterpret_cast<const int4 *>(src + head);
    int4 *d16 = reinterpret_cast<int4 *>(dst + head);
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += stride) d16[i] = __ldg(s16 + i);
    if (aligned && blockIdx.x == 0) {
        for (long long i = threadIdx.x; i < head; i += blockDim.x) dst[i] = src[i];
        for (long long i = tail0 + threadIdx.x; i < nbytes; i += blockDim.x) dst[i] = src[i];
    } else if (!aligned) {
        for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nbytes; i += stride) dst[i] = src[i];
    }
}

// the same copy with the destinations passed by value (no table in device memory)
struct PushDst {
    unsigned char *p[MAX_PEERS];
};
// (a small grid, four 16-byte loads in flight per thread: the copy runs beside the CSR kernel of the next row range)
__global__ void __launch_bounds__(256) peer_push_kernel_v(const unsigned char *__restrict__ src, PushDst dst_table,
                                                          long long nbytes, int aligned) {
    unsigned char *dst = dst_table.p[blockIdx.y];
    long long head = aligned ? (long long)((16u - (unsigned)((uintptr_t)src & 15u)) & 15u) : nbytes;
    if (head > nbytes) head = nbytes;
    const long long n16 = (nbytes - head) / 16, tail0 = head + n16 * 16;
    const int4 *s16 = reinterpret_cast<const int4 *>(src + head);
    int4 *d16 = reinterpret_cast<int4 *>(dst + head);
    const long long stride = (long long)gridDim.x * blockDim.x;
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    for (; i + 3 * stride < n16; i += 4 * stride) {
        const int4 a = __ldg(s16 + i), b = __ldg(s16 + i + stride), c = __ldg(s16 + i + 2 * stride),
                   d = __ldg(s16 + i + 3 * stride);
        d16[i] = a, d16[i + stride] = b, d16[i + 2 * stride] = c, d16[i + 3 * stride] = d;
    }
    for (; i < n16; i += stride) d16[i] = __ldg(s16 + i);
    if (aligned && blockIdx.x == 0) {
        for (long long i = threadIdx.x; i < head; i += blockDim.x) dst[i] = src[i];
        for (long long i = tail0 + threadIdx.x; i < nbytes; i += blockDim.x) dst[i] = src[i];
    } else if (!aligned) {
        for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nbytes; i += stride) dst[i] = src[i];
    }
}

template <typename V>
__global__ void gather_kernel(const V *__restrict__ x, const int *__restrict__ perm, V *__restrict__ out, int n) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = __ldg(x + __ldg(perm + i));
}

template <typename V>
size_t hotx_smem_bytes(int hotCols) {
    using TS = TileSmem<typename AccOf<V>::T, RESID_THREADS * ResidCfg<V>::IPT, RESID_THREADS / 32>;
    return 16 + (size_t)hotCols * sizeof(V) + sizeof(TS) * HotxCfg<V>::GROUPS;
}

int hotx_sm_count() {
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    return sms;
}

template <typename V>
cudaError_t resid_spmv_t(const ResidPlan &P, const void *x, void *y, const void *ytile, const uint32_t *hotmask,
                         int mode, const int *row_map, cudaStream_t s, bool chained, void *const *peers = nullptr,
                         int n_peers = 0, long long row_offset = 0, void *mc_y = nullptr) {
    using A = typename AccOf<V>::T;
    constexpr int IPT = ResidCfg<V>::IPT;
    const bool hasTile = mode != OUT_CARRIER && ytile != nullptr && hotmask != nullptr;
    RowOut<V> out;
    out.y = (V *)y;
    out.carrier_out = is_peers(mode) ? (A *)mc_y : (A *)y;
    out.row_map = row_map;
    out.ytile = (const A *)ytile;
    out.hotmask = hotmask;
    out.nzRow = P.nz_row;
    out.n_peers = n_peers;
    out.row_offset = row_offset;
    bool aligned16 = n_peers > 0;
    for (int g = 0; g < MAX_PEERS; ++g) {
        out.peer_y[g] = g < n_peers ? (V *)peers[g] : nullptr;
        if (g < n_peers && ((uintptr_t)peers[g] & 15u) != 0) aligned16 = false;
    }
    if (aligned16) out.n_peers |= PEER_VEC_FLAG;
    dim3 grid(P.num_tiles), block(RESID_THREADS);
    const int fwork = P.num_tiles - 1 > P.n_empty ? P.num_tiles - 1 : P.n_empty;
    const int fgrid = (fwork + 127) / 128;
    cudaError_t le = cudaSuccess;
    // hot-column prefix of x in shared memory (persistent kernel): only where the plan says so and x is 16-byte aligned
    const int hot = (P.hot_cols > 0 && ((uintptr_t)x & 15u) == 0 && !is_accum(mode)) ? P.hot_cols : 0;
#define MX_LAUNCH(HT, MD)                                                                                           \
    do {                                                                                                            \
        if (hot > 0) {                                                                                              \
            auto kern = resid_hotx_kernel<V, IPT, HT, MD>;                                                          \
            const size_t smem = hotx_smem_bytes<V>(hot);                                                            \
            le = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);               \
            if (le == cudaSuccess) {                                                                                \
                const int pgrid = std::min(hotx_sm_count(), (P.num_tiles + HotxCfg<V>::GROUPS - 1) / HotxCfg<V>::GROUPS); \
                le = launch_chained(kern, dim3(pgrid), dim3(RESID_THREADS * HotxCfg<V>::GROUPS), s, chained, smem,  \
                                    P.c_ptr, P.col_ind, (const V *)P.val, (const V *)x, out,                        \
                                    (const int *)P.tile_row, (A *)P.carry, (A *)P.head, P.nnz, P.prefetch_tiles,    \
                                    P.num_tiles, hot, P.dev_err);                                                    \
            }                                                                                                       \
        } else if (P.dense_row_ends && !HT && MD == OUT_Y) {                                                        \
            le = launch_chained(resid_kernel<V, IPT, false, OUT_Y, true>, grid, block, s, chained, 0, P.c_ptr,      \
                                P.col_ind, (const V *)P.val, (const V *)x, out, (const int *)P.tile_row,           \
                                (A *)P.carry, (A *)P.head, P.nnz, P.prefetch_tiles);                                \
        } else {                                                                                                    \
            le = launch_chained(resid_kernel<V, IPT, HT, MD>, grid, block, s, chained, 0, P.c_ptr, P.col_ind,       \
                                (const V *)P.val, (const V *)x, out, (const int *)P.tile_row, (A *)P.carry,        \
                                (A *)P.head, P.nnz, P.prefetch_tiles);                                              \
        }                                                                                                           \
        if (le == cudaSuccess && fgrid > 0)                                                                         \
            le = launch_chained(resid_fixup_kernel<V, IPT, HT, MD>, dim3(fgrid), dim3(128), s, true, 0, P.c_ptr,    \
                                out, (const int *)P.tile_row, (const A *)P.carry, (const A *)P.head, P.m_rows,      \
                                P.num_tiles, (const int *)P.empty_row, P.n_empty);                                  \
    } while (0)
    if (mode == OUT_CARRIER)
        MX_LAUNCH(false, OUT_CARRIER);
    else if (mode == OUT_Y_PEERS && hasTile)
        MX_LAUNCH(true, OUT_Y_PEERS);
    else if (mode == OUT_Y_PEERS)
        MX_LAUNCH(false, OUT_Y_PEERS);
    else if (hasTile && mode == OUT_Y_ACCUM)
        MX_LAUNCH(true, OUT_Y_ACCUM);
    else if (hasTile)
        MX_LAUNCH(true, OUT_Y);
    else if (mode == OUT_Y_ACCUM)
        MX_LAUNCH(false, OUT_Y_ACCUM);
    else
        MX_LAUNCH(false, OUT_Y);
#undef MX_LAUNCH
    return le != cudaSuccess ? le : cudaGetLastError();
}

}  // namespace

// L2 prefetch distance of the CSR kernel, in tiles: one wave of resident CTAs ahead, so that a CTA finds its index and
// value streams in L2 instead of waiting on HBM.  The prefetched window shares L2 with the gathered x: measured on
// this GPU it gains 9 % on a block-structured matrix (x = 12.6 MB) and 2-3 % on a power-law one (x = 4 MB), and loses
// 25 % when x alone (64 MB) already fills the half of L2 that is local to an SM.  So it is on only while x plus the
// window fit into half of L2.  MX_RESID_PREFETCH=<tiles> overrides (0 = off).
static int resid_prefetch_distance(int dtype, int n_cols, int tile_nnz) {
    if (const char *env = getenv("MX_RESID_PREFETCH")) return atoi(env) > 0 ? atoi(env) : 0;
    int dev = 0, sms = 0, l2 = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaDeviceGetAttribute(&l2, cudaDevAttrL2CacheSize, dev);
    const size_t vb = dtype == MX_FP64 ? sizeof(double) : sizeof(__half);
    const int per_sm = dtype == MX_FP64 ? ResidCfg<double>::MINBLOCKS : ResidCfg<__half>::MINBLOCKS;
    const int wave = sms * per_sm;
    const size_t window = (size_t)wave * tile_nnz * (vb + 4), xbytes = (size_t)n_cols * vb;
    return xbytes + window <= (size_t)l2 / 2 ? wave : 0;
}

cudaError_t resid_plan_build(int dtype, ResidPlan &P, cudaStream_t s) {
    P.tile_nnz = RESID_THREADS * (dtype == MX_FP64 ? ResidCfg<double>::IPT : ResidCfg<__half>::IPT);
    P.num_tiles = P.nnz > 0 ? (int)(((long long)P.nnz + P.tile_nnz - 1) / P.tile_nnz) : 1;
    P.prefetch_tiles = resid_prefetch_distance(dtype, P.n_cols, P.tile_nnz);
    cudaError_t e;
    // rows without entries leave the kernel's row space: cPtr = row pointers of the non-empty rows
    int *flag = nullptr, *pos = nullptr;
    const size_t nr = (size_t)P.n_rows + 1;
    if ((e = cudaMallocAsync(&flag, nr * sizeof(int), s)) != cudaSuccess) return e;
    if ((e = cudaMallocAsync(&pos, nr * sizeof(int), s)) != cudaSuccess) return e;
    nonempty_flag_kernel<<<(int)((nr + 255) / 256), 256, 0, s>>>(P.row_ptr, P.n_rows, flag);
    {
        TempBuf tmp;
        if ((e = exclusive_sum(tmp, flag, pos, (int)nr, s)) != cudaSuccess) return e;
        if ((e = cudaMemcpyAsync(&P.m_rows, pos + P.n_rows, sizeof(int), cudaMemcpyDeviceToHost, s)) != cudaSuccess)
            return e;
        if ((e = cudaStreamSynchronize(s)) != cudaSuccess) return e;
    }
    P.n_empty = P.n_rows - P.m_rows;
    if (P.n_empty == 0) {
        P.c_ptr = P.row_ptr;
        P.nz_row = nullptr;
        P.empty_row = nullptr;
    } else {
        if ((e = cudaMallocAsync(&P.c_ptr_own, ((size_t)P.m_rows + 1) * sizeof(int), s)) != cudaSuccess) return e;
        if ((e = cudaMallocAsync(&P.nz_row, ((size_t)P.m_rows + 1) * sizeof(int), s)) != cudaSuccess) return e;
        if ((e = cudaMallocAsync(&P.empty_row, (size_t)P.n_empty * sizeof(int), s)) != cudaSuccess) return e;
        compress_rows_kernel<<<(P.n_rows + 255) / 256, 256, 0, s>>>(P.row_ptr, pos, P.n_rows, P.c_ptr_own, P.nz_row,
                                                                    P.empty_row);
        P.c_ptr = P.c_ptr_own;
    }
    e = resid_plan_finish(dtype, P, s);
    if (flag) cudaFreeAsync(flag, s);
    if (pos) cudaFreeAsync(pos, s);
    return e;
}

// The part of the plan that follows the row compression: per-tile row offsets and the carry / head slots.  Callers
// that already hold the compressed row table (c_ptr, nz_row, m_rows, n_empty) of a matrix call this directly.
cudaError_t resid_plan_finish(int dtype, ResidPlan &P, cudaStream_t s) {
    cudaError_t e;
    if (P.tile_nnz == 0) {
        P.tile_nnz = RESID_THREADS * (dtype == MX_FP64 ? ResidCfg<double>::IPT : ResidCfg<__half>::IPT);
        P.num_tiles = P.nnz > 0 ? (int)(((long long)P.nnz + P.tile_nnz - 1) / P.tile_nnz) : 1;
    }
    if ((e = cudaMallocAsync(&P.tile_row, sizeof(int) * (size_t)(P.num_tiles + 1), s)) != cudaSuccess) return e;
    if ((e = cudaMallocAsync(&P.carry, acc_bytes(dtype) * (size_t)P.num_tiles, s)) != cudaSuccess) return e;
    if ((e = cudaMallocAsync(&P.head, acc_bytes(dtype) * (size_t)P.num_tiles, s)) != cudaSuccess) return e;
    tile_row_kernel<<<(P.num_tiles + 1 + 255) / 256, 256, 0, s>>>(P.c_ptr, P.m_rows, P.nnz, P.tile_nnz, P.num_tiles,
                                                                  P.tile_row);
    e = cudaGetLastError();
    cudaError_t e2 = cudaStreamSynchronize(s);
    return e != cudaSuccess ? e : e2;
}

void resid_plan_free(ResidPlan &P, cudaStream_t s) {
    if (P.tile_row) cudaFreeAsync(P.tile_row, s);
    if (P.carry) cudaFreeAsync(P.carry, s);
    if (P.head) cudaFreeAsync(P.head, s);
    if (P.c_ptr_own) cudaFreeAsync(P.c_ptr_own, s);
    if (P.nz_row) cudaFreeAsync(P.nz_row, s);
    if (P.empty_row) cudaFreeAsync(P.empty_row, s);
    P.tile_row = P.c_ptr_own = P.nz_row = P.empty_row = nullptr;
    P.c_ptr = nullptr;
    P.carry = P.head = nullptr;
}

int resid_hot_cols_budget(int dtype, int d_cols) {
    const size_t fixed = dtype == MX_FP64 ? hotx_smem_bytes<double>(0) : hotx_smem_bytes<__half>(0);
    const size_t vb = val_bytes(dtype);
    long long cols = (long long)((HOTX_SMEM_LIMIT - fixed) / vb);
    if (cols > d_cols) cols = d_cols;
    cols -= cols % (long long)(16 / vb);
    return cols >= 256 ? (int)cols : 0;
}

int resid_launches(const ResidPlan &P) { return (P.num_tiles > 1 || P.n_empty > 0) ? 2 : 1; }

cudaError_t resid_spmv(int dtype, const ResidPlan &P, const void *x, void *y, const void *ytile,
                       const uint32_t *hotmask, bool accumulate, cudaStream_t s, bool chained) {
    const int mode = accumulate ? OUT_Y_ACCUM : OUT_Y;
    if (dtype == MX_FP64) return resid_spmv_t<double>(P, x, y, ytile, hotmask, mode, nullptr, s, chained);
    return resid_spmv_t<__half>(P, x, y, ytile, hotmask, mode, nullptr, s, chained);
}

cudaError_t resid_spmv_peers(int dtype, const ResidPlan &P, const void *x, void *const *peers, int n_peers,
                             long long row_offset, const void *ytile, const uint32_t *hotmask, cudaStream_t s,
                             bool chained, void *mc_y) {
    if (n_peers < 1 || n_peers > MAX_PEERS) return cudaErrorInvalidValue;
    if (dtype == MX_FP64)
        return resid_spmv_t<double>(P, x, peers[0], ytile, hotmask, OUT_Y_PEERS, nullptr, s, chained, peers, n_peers,
                                    row_offset, mc_y);
    return resid_spmv_t<__half>(P, x, peers[0], ytile, hotmask, OUT_Y_PEERS, nullptr, s, chained, peers, n_peers,
                                row_offset, mc_y);
}

cudaError_t peer_push_rows(int dtype, void *const *peers, int n_peers, int self, long long row_offset, long long n_rows,
                           cudaStream_t s) {
    if (n_peers < 1 || n_peers > MAX_PEERS || self < 0 || self >= n_peers) return cudaErrorInvalidValue;
    if (n_peers == 1 || n_rows <= 0) return cudaSuccess;
    const size_t vb = val_bytes(dtype);
    PushDst dst{};
    int nd = 0;
    const unsigned char *src = static_cast<const unsigned char *>(peers[self]) + (size_t)row_offset * vb;
    int aligned = 1;
    for (int g = 0; g < n_peers; ++g)
        if (g != self) {
            dst.p[nd] = static_cast<unsigned char *>(peers[g]) + (size_t)row_offset * vb;
            if ((((uintptr_t)dst.p[nd] ^ (uintptr_t)src) & 15u) != 0) aligned = 0;
            ++nd;
        }
    const long long nbytes = n_rows * (long long)vb;
    const long long units = aligned ? (nbytes + 15) / 16 : nbytes;
    // CTAs over all destinations: a third of the SMs.  Measured on 2 GPUs beside the CSR kernel of the next row range
    // (3.02 ms of kernels + 0.47 ms of copy when run one after the other): 148 CTAs 3.41 ms, 96: 3.34, 48: 3.28,
    // 24: 3.29, 16: 3.30 - the copy alone is no slower with 48 (NVLink-bound), and fewer SMs have the stores that
    // wait for NVLink in front of their gathers.
    const int total = std::max(16, hotx_sm_count() / 3);
    const int gx = (int)std::max<long long>(1, std::min<long long>((units + 255) / 256, (total + nd - 1) / nd));
    peer_push_kernel_v<<<dim3(gx, nd), 256, 0, s>>>(src, dst, nbytes, aligned);
    return cudaGetLastError();
}

cudaError_t resid_spmv_to_carrier(int dtype, const ResidPlan &P, const void *x, void *carrier, const int *row_map,
                                  cudaStream_t s) {
    if (dtype == MX_FP64) return resid_spmv_t<double>(P, x, carrier, nullptr, nullptr, OUT_CARRIER, row_map, s, false);
    return resid_spmv_t<__half>(P, x, carrier, nullptr, nullptr, OUT_CARRIER, row_map, s, false);
}

cudaError_t map_indices(const int *in, const int *map, int *out, long long n, cudaStream_t s) {
    if (n <= 0) return cudaSuccess;
    map_indices_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(in, map, out, n);
    return cudaGetLastError();
}

// The product without its row logic: stream (column, value), gather x, multiply, reduce per thread, write nothing.
// Its duration is the floor that the matrix's own index pattern sets for any kernel that visits the non-zeros in CSR
// order on this GPU (index and value streams from HBM, one gather per non-zero through L1).
template <typename V, int IPT>
__global__ void __launch_bounds__(128) stream_gather_kernel(const int *__restrict__ colInd, const V *__restrict__ val,
                                                            const V *__restrict__ x, float *sink, int nnz) {
    const long long base = (long long)blockIdx.x * 128 * IPT;
    int c[IPT];
    float v[IPT];
#pragma unroll
    for (int j = 0; j < IPT; ++j) {
        const long long i = base + threadIdx.x + j * 128;
        c[j] = i < nnz ? ldg_stream(colInd + i) : 0;
        v[j] = i < nnz ? (float)ldg_stream_val(val + i) : 0.f;
    }
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < IPT; ++j) acc += v[j] * (float)to_acc(__ldg(x + c[j]));
    if (acc == 123456.789f) *sink = acc;  // keeps the loads alive; practically never true
}

cudaError_t stream_gather_pass(int dtype, const int *col_ind, const void *val, const void *x, float *sink, int nnz,
                               cudaStream_t s) {
    if (nnz <= 0) return cudaSuccess;
    constexpr int IPT = 16;
    const int grid = (int)(((long long)nnz + 128 * IPT - 1) / (128 * IPT));
    if (dtype == MX_FP64)
        stream_gather_kernel<double, IPT><<<grid, 128, 0, s>>>(col_ind, (const double *)val, (const double *)x, sink, nnz);
    else
        stream_gather_kernel<__half, IPT><<<grid, 128, 0, s>>>(col_ind, (const __half *)val, (const __half *)x, sink, nnz);
    return cudaGetLastError();
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

// ---------------------------------------------------------------------------------------------------------------
// Allocation-free CSR SpMV.
//
// Some callers of this library run where device memory cannot be requested: a solver that was handed a fixed
// arena and must not touch the allocator, a real-time loop that may not block on the driver's allocation lock, a
// process whose memory budget was fixed at start-up.  For them this entry point computes y = A x for a CSR matrix
// that already lives on the device with NO cudaMalloc / cudaFree (and no library call that allocates): everything the
// kernels need beyond the caller's inputs and output — the compressed row table, the per-tile row offsets and the
// carry / head slots of rows that span tiles — lives in the fixed array below.
//
// The array is part of the library image: every GPU that loads the library holds MX_STATIC_SCRATCH_BYTES of it until
// the process exits.  All calls share it and it keeps what the last call left there, so (a) the slots that a call
// reads before writing are cleared at the start of every call, and (b) two calls that overlap on the GPU (different
// streams, or different host threads) race on it — issue them one after the other.
// In host code `g_static_scratch` is only a stand-in for the device symbol, not a device address: its address is
// looked up once per device with cudaGetSymbolAddress (with that device current) and that pointer is what the kernels
// get.  The first call on a device performs this look-up, so it should happen before any stream capture begins.  The
// address is cached for the life of the process: it does not survive a cudaDeviceReset of that device.  Every call
// also reads one count back and synchronises the stream once.
// ---------------------------------------------------------------------------------------------------------------
namespace mx {
namespace {

constexpr size_t ST_ROWS = MX_STATIC_MAX_ROWS;
// tile slots are sized for the value type with the smaller tile (more tiles per non-zero)
constexpr int ST_MIN_IPT = ResidCfg<double>::IPT < ResidCfg<__half>::IPT ? ResidCfg<double>::IPT : ResidCfg<__half>::IPT;
constexpr size_t ST_TILES = (size_t)MX_STATIC_MAX_NNZ / (RESID_THREADS * ST_MIN_IPT) + 1;
constexpr size_t ST_CUB_TEMP = 1u << 20;
// layout (byte offsets, each region 256-byte aligned)
constexpr size_t st_align(size_t b) { return (b + 255) & ~(size_t)255; }
constexpr size_t ST_OFF_FLAG = 0;
constexpr size_t ST_OFF_POS = ST_OFF_FLAG + st_align((ST_ROWS + 1) * 4);
constexpr size_t ST_OFF_CPTR = ST_OFF_POS + st_align((ST_ROWS + 1) * 4);
constexpr size_t ST_OFF_NZROW = ST_OFF_CPTR + st_align((ST_ROWS + 1) * 4);
constexpr size_t ST_OFF_EMPTY = ST_OFF_NZROW + st_align((ST_ROWS + 1) * 4);
constexpr size_t ST_OFF_TILEROW = ST_OFF_EMPTY + st_align((ST_ROWS + 1) * 4);
constexpr size_t ST_OFF_CARRY = ST_OFF_TILEROW + st_align((ST_TILES + 1) * 4);
constexpr size_t ST_OFF_HEAD = ST_OFF_CARRY + st_align(ST_TILES * 8);
constexpr size_t ST_OFF_TEMP = ST_OFF_HEAD + st_align(ST_TILES * 8);
constexpr size_t ST_TOTAL = ST_OFF_TEMP + ST_CUB_TEMP;
static_assert(ST_TOTAL <= MX_STATIC_SCRATCH_BYTES, "scratch layout exceeds the size stated in mx_capi.h");

static __device__ __align__(256) unsigned char g_static_scratch[MX_STATIC_SCRATCH_BYTES];

constexpr int ST_MAX_DEVICES = 64;
unsigned char *g_static_ptr[ST_MAX_DEVICES] = {};  // device address of g_static_scratch, per device

// once per device, with that device current
cudaError_t static_scratch_address(unsigned char **out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= ST_MAX_DEVICES) return cudaErrorInvalidDevice;
    if (!g_static_ptr[dev]) {
        void *p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess) return e;
        g_static_ptr[dev] = static_cast<unsigned char *>(p);
    }
    *out = g_static_ptr[dev];
    return cudaSuccess;
}

}  // namespace
}  // namespace mx

extern "C" int mx_csr_spmv_static(int dtype, int n_rows, int n_cols, int nnz, const int *row_ptr_dev,
                                  const int *col_ind_dev, const void *val_dev, const void *x_dev, void *y_dev,
                                  void *stream) {
    using namespace mx;
    if ((dtype != MX_FP64 && dtype != MX_FP16) || n_rows < 0 || n_cols < 0 || nnz < 0 || !row_ptr_dev || !x_dev ||
        !y_dev || (nnz > 0 && (!col_ind_dev || !val_dev)))
        return MX_ERR_INVALID;
    if ((size_t)n_rows > ST_ROWS || (long long)nnz > (long long)MX_STATIC_MAX_NNZ) {
        fprintf(stderr,
                "mx_csr_spmv_static: %d rows / %d non-zeros exceed the fixed scratch (at most %d rows, %d non-zeros); "
                "use a handle (mx_create / mx_upload_csr / mx_spmv) for larger matrices\n",
                n_rows, nnz, (int)MX_STATIC_MAX_ROWS, (int)MX_STATIC_MAX_NNZ);
        return MX_ERR_TOO_LARGE;
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    unsigned char *base = nullptr;
    if (static_scratch_address(&base) != cudaSuccess) {
        cudaGetLastError();
        return MX_ERR_CUDA;
    }
    int *flag = reinterpret_cast<int *>(base + ST_OFF_FLAG), *pos = reinterpret_cast<int *>(base + ST_OFF_POS);
    ResidPlan P;
    P.n_rows = n_rows;
    P.n_cols = n_cols;
    P.nnz = nnz;
    P.row_ptr = row_ptr_dev;
    P.col_ind = col_ind_dev;
    P.val = val_dev;
    P.tile_nnz = RESID_THREADS * (dtype == MX_FP64 ? ResidCfg<double>::IPT : ResidCfg<__half>::IPT);
    P.num_tiles = nnz > 0 ? (int)(((long long)nnz + P.tile_nnz - 1) / P.tile_nnz) : 1;
    P.tile_row = reinterpret_cast<int *>(base + ST_OFF_TILEROW);
    P.carry = base + ST_OFF_CARRY;
    P.head = base + ST_OFF_HEAD;
#define STCK(call)                            \
    do {                                      \
        if ((call) != cudaSuccess) {          \
            cudaGetLastError();               \
            return MX_ERR_CUDA;               \
        }                                     \
    } while (0)
    // the array keeps the previous call's contents: clear the slots that are read before they are written
    STCK(cudaMemsetAsync(P.carry, 0, acc_bytes(dtype) * (size_t)P.num_tiles, s));
    STCK(cudaMemsetAsync(P.head, 0, acc_bytes(dtype) * (size_t)P.num_tiles, s));
    // rows without entries leave the kernel's row space (same steps as resid_plan_build, on the fixed array)
    const size_t nr = (size_t)n_rows + 1;
    nonempty_flag_kernel<<<(int)((nr + 255) / 256), 256, 0, s>>>(row_ptr_dev, n_rows, flag);
    size_t temp_bytes = 0;
    STCK(cub::DeviceScan::ExclusiveSum(nullptr, temp_bytes, flag, pos, (int)nr, s));
    if (temp_bytes > ST_CUB_TEMP) return MX_ERR_TOO_LARGE;
    STCK(cub::DeviceScan::ExclusiveSum(base + ST_OFF_TEMP, temp_bytes, flag, pos, (int)nr, s));
    int m_rows = 0;
    STCK(cudaMemcpyAsync(&m_rows, pos + n_rows, sizeof(int), cudaMemcpyDeviceToHost, s));
    STCK(cudaStreamSynchronize(s));
    P.m_rows = m_rows;
    P.n_empty = n_rows - m_rows;
    if (P.n_empty == 0) {
        P.c_ptr = row_ptr_dev;
    } else {
        int *cptr = reinterpret_cast<int *>(base + ST_OFF_CPTR);
        P.nz_row = reinterpret_cast<int *>(base + ST_OFF_NZROW);
        P.empty_row = reinterpret_cast<int *>(base + ST_OFF_EMPTY);
        compress_rows_kernel<<<(n_rows + 255) / 256, 256, 0, s>>>(row_ptr_dev, pos, n_rows, cptr, P.nz_row, P.empty_row);
        P.c_ptr = cptr;
    }
    tile_row_kernel<<<(P.num_tiles + 1 + 255) / 256, 256, 0, s>>>(P.c_ptr, P.m_rows, P.nnz, P.tile_nnz, P.num_tiles,
                                                                  P.tile_row);
    STCK(cudaGetLastError());
    cudaError_t e = dtype == MX_FP64
                        ? resid_spmv_t<double>(P, x_dev, y_dev, nullptr, nullptr, OUT_Y, nullptr, s, false)
                        : resid_spmv_t<__half>(P, x_dev, y_dev, nullptr, nullptr, OUT_Y, nullptr, s, false);
    STCK(e);
#undef STCK
    return MX_OK;
}

// ---------------------------------------------------------------------------------------------------------------
// Slab push: after a product that wrote this GPU's rows into its own full-length y, copy those rows into the same
// place of every other GPU's y.  dst_table is a small device array of the peers' row addresses (filled by the caller
// side below with cudaMemcpyAsync from a host array that lives until the copy has been issued).
// ---------------------------------------------------------------------------------------------------------------
extern "C" int mx_peer_push(int dtype, void *const *y_peers, int n_peers, int self, long long row_offset,
                            long long n_rows, void *table_dev, void *stream) {
    using namespace mx;
    if ((dtype != MX_FP64 && dtype != MX_FP16) || !y_peers || n_peers < 1 || n_peers > MAX_PEERS || self < 0 ||
        self >= n_peers || row_offset < 0 || n_rows < 0 || !table_dev)
        return MX_ERR_INVALID;
    if (n_peers == 1 || n_rows == 0) return MX_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const size_t vb = val_bytes(dtype);
    unsigned char *host_tab[MAX_PEERS];
    int nd = 0;
    for (int g = 0; g < n_peers; ++g)
        if (g != self) host_tab[nd++] = static_cast<unsigned char *>(y_peers[g]) + (size_t)row_offset * vb;
    // pageable source: the runtime stages it before returning, so the stack array may go out of scope
    if (cudaMemcpyAsync(table_dev, host_tab, sizeof(void *) * nd, cudaMemcpyHostToDevice, s) != cudaSuccess) {
        cudaGetLastError();
        return MX_ERR_CUDA;
    }
    const unsigned char *src = static_cast<const unsigned char *>(y_peers[self]) + (size_t)row_offset * vb;
    const long long nbytes = n_rows * (long long)vb;
    int aligned = 1;
    for (int d = 0; d < nd; ++d)
        if ((((uintptr_t)host_tab[d] ^ (uintptr_t)src) & 15u) != 0) aligned = 0;
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const long long units = aligned ? (nbytes + 15) / 16 : nbytes;
    const int gx = (int)std::max<long long>(1, std::min<long long>((units + 255) / 256, sms * 4 / nd + 1));
    peer_push_kernel<<<dim3(gx, nd), 256, 0, s>>>(src, reinterpret_cast<unsigned char *const *>(table_dev), nbytes, aligned);
    if (cudaGetLastError() != cudaSuccess) return MX_ERR_CUDA;
    return MX_OK;
}
