// Dense-tile SpMV on the tensor cores — the B200 counterpart of the reference's "dense-unfold" kernels
// (src/spmv_kernel/du_tcSpMV_fp64.cu:81-160, src/spmv_kernel/du_tcSpMV_fp16_v2.cu:4-110).
//
// The matrix half handled here is the core-dense block in the reference's fragment format: 8-row panels,
// each a run of 8xK fragments (K = 4 FP64, 8 FP16) stored as a bitmap, a value offset, K gathered-x
// indices and the packed non-zero values.
//
//   * FP64: one mma.sync m8n8k4 f64 per fragment.  Lane l owns bitmap bit l, i.e. A[l/4][l%4].
//   * FP16: one mma.sync m16n8k16 (f16 in, f32 accumulate) per FOUR fragments of the same panel:
//       A rows 0-7  = [frag f | frag f+1] along k,  A rows 8-15 = [frag f+2 | frag f+3],
//       B column 0  = x-segments of f and f+1,      B column 1  = x-segments of f+2 and f+3,
//     so C[r][0] + C[8+r][1] is the panel row's sum over the four fragments (the cross terms land in
//     columns that are never read).  Lane l owns bitmap bits 2l and 2l+1 of every fragment.
//   * A CTA owns a run of consecutive work segments; their bitmaps, value offsets, x indices and packed values are
//     four contiguous ranges, which one thread copies into shared memory with 1-D bulk copies (cp.async.bulk on an
//     mbarrier, bounded wait).  Warps then run their segments out of shared memory: broadcast shared loads for the
//     bitmap and the offset, conflict-free shared loads for the values, and each lane gathers the x value of its own
//     fragment column (4 distinct addresses per instruction) — no shuffles, no dependent global loads but the gathers.
//   * Sums stay in the accumulator registers over the whole fragment run (two independent chains for FP64); one store
//     per row, no atomics on y.  The reference gives every panel one warp; a power-law panel can hold 10^4
//     fragments, so here a panel is cut into segments of at most SEG fragments, one warp each.  Segments of a split
//     panel park their 8 partial sums; the last one to arrive (a counter, no spinning) adds them in segment order.
//   * Measured and dropped: direct global loads with shuffle hand-round (37 warp-instructions per fragment, 193 us on
//     the 100M-nnz block matrix vs 115 us now), gathering x into shared memory behind a CTA-wide barrier (164 us), a
//     persistent 4-stage ring with one producer warp and 4 consumer warps per CTA (275 us: throughput follows the
//     number of resident consumer warps, not the copies in flight).  Stage size sweep 8-64 KB: best at 16 KB x 4 warps.
#include <cstdlib>
#include <type_traits>

#include "device_prims.cuh"
#include "mx_internal.h"

// fragment pairs per unrolled pass of the FP64 loop (A/B on the block matrix, tile half alone: 2: 124.6 us,
// 4: 108.7 us, 8: 114.6 us; explicit operand batches of 8 / 16: 130 / 110 us)
constexpr int TILE_UNROLL = 4;

namespace mx {
namespace {

constexpr int SEG = 64;            // fragments per work segment

__global__ void seg_count_kernel(const int *__restrict__ chunkPtr, int chunkNum, int *__restrict__ segCount,
                                 int *__restrict__ multiCount) {
    int p = blockIdx.x * blockDim.x + threadIdx.x;
    if (p > chunkNum) return;
    int c = 0;
    if (p < chunkNum) {
        int nf = chunkPtr[p + 1] - chunkPtr[p];
        c = nf <= SEG ? 1 : (nf + SEG - 1) / SEG;
    }
    segCount[p] = c;
    multiCount[p] = c > 1 ? c : 0;
}

__global__ void seg_fill_kernel(const int *__restrict__ chunkPtr, int chunkNum, const int *__restrict__ panelFirstSeg,
                                const int *__restrict__ panelFirstSlot, int *__restrict__ segPanel,
                                int *__restrict__ segBegin, int *__restrict__ segEnd, int *__restrict__ segSlot) {
    int p = blockIdx.x * blockDim.x + threadIdx.x;
    if (p >= chunkNum) return;
    int s0 = panelFirstSeg[p], ns = panelFirstSeg[p + 1] - s0;
    int f0 = chunkPtr[p], f1 = chunkPtr[p + 1];
    for (int j = 0; j < ns; ++j) {
        segPanel[s0 + j] = p;
        segBegin[s0 + j] = f0 + j * SEG;
        segEnd[s0 + j] = min(f1, f0 + (j + 1) * SEG);
        segSlot[s0 + j] = ns > 1 ? panelFirstSlot[p] + j : -1;
    }
}

__device__ __forceinline__ void put(double *o, double v) { *o = v; }
__device__ __forceinline__ void put(float *o, float v) { *o = v; }
__device__ __forceinline__ void put(__half *o, float v) { *o = __float2half_rn(v); }
__device__ __forceinline__ double get(const double *o) { return *o; }
__device__ __forceinline__ float get(const float *o) { return *o; }
__device__ __forceinline__ float get(const __half *o) { return __half2float(*o); }

// Hands the 8 row sums of one segment over: directly to `out` when the panel has a single segment, through `partial`
// and an arrival counter otherwise (the last segment of the panel to arrive adds the parked sums in segment order, so
// the result does not depend on arrival order; nobody spins).  rowLane: this lane holds the sum of panel row g.  The
// slot comes with the packed segment descriptor and the output row was looked up before the fragment loop; slots of a
// split panel are consecutive from its first segment.
template <typename A, typename OutT, bool ACCUM>
__device__ __forceinline__ void finish_staged(A sum, bool rowLane, int g, int lane, int p, int s, int slot, int myRow,
                                              int outRow, int dRows, const int *__restrict__ panelFirstSeg,
                                              A *__restrict__ partial, unsigned *__restrict__ panelCount,
                                              OutT *__restrict__ out) {
    if (slot >= 0) {
        if (rowLane) __stcg(partial + (size_t)slot * 8 + g, sum);
        __threadfence();
        __syncwarp();
        const int first = panelFirstSeg[p], nseg = panelFirstSeg[p + 1] - first;
        unsigned old = 0;
        if (lane == 0) old = atomicAdd(panelCount + p, 1u);
        old = __shfl_sync(0xffffffffu, old, 0);
        if (old != (unsigned)(nseg - 1)) return;  // not the last segment of the panel to finish
        __threadfence();
        if (lane == 0) panelCount[p] = 0;  // ready for the next launch
        const int slot0 = slot - (s - first);
        sum = A(0);
        if (rowLane)
            for (int j = 0; j < nseg; ++j) sum += __ldcg(partial + (size_t)(slot0 + j) * 8 + g);
    }
    if (rowLane && myRow < dRows) {
        if (ACCUM) sum += (A)get(out + outRow);
        put(out + outRow, sum);
    }
}

// ------------------------------------------------------------------------------------------------------------------
// TMA staging.  A CTA owns a run of consecutive work segments; because segments are consecutive, the bitmaps,
// value offsets, x indices and packed values they touch are four contiguous ranges.  One elected thread copies the
// four ranges into shared memory with 1-D bulk copies (cp.async.bulk, completion counted on an mbarrier, no
// multicast); every warp then runs its segments out of shared memory, so the fragment loop has no dependent global
// load left except the x gathers.  Several CTAs per SM overlap one CTA's copies with another's arithmetic.
// ------------------------------------------------------------------------------------------------------------------
struct CtaDesc {  // computed at plan time
    int seg0, seg1;  // work segments [seg0, seg1)
    int f0, f1;      // fragments [f0, f1) they cover
    int v0, v1;      // packed values [v0, v1)
    int full;        // 1: every fragment of the run is completely filled (no bitmap decode needed)
    int pad1;
};

constexpr int STAGE_WARPS = 4;   // warps per CTA (8 measured slower)
int g_tile_prefetch = -1;        // L2 prefetch distance in CTAs; default 5 per SM (A/B on the block matrix: tile half
                                 // 113.8 -> 108.7 us; 10 per SM 110.1, 20 per SM 122.8); 0 = off
constexpr int STAGE_BYTES_TARGET = 16 * 1024;  // per CTA; a CTA may exceed it by one segment (sweep: 8-64 KB)

// byte layout of a CTA's shared-memory stage; every range starts 16-byte aligned in global AND shared memory
template <typename B, typename V, int K>
struct StageLayout {
    int fa, va;                  // fragment / value index the copies start at (rounded down to 16 bytes)
    uint32_t nBit, nPtr, nX, nV;  // copy sizes in bytes (multiples of 16)
    uint32_t oBit, oPtr, oX, oV;  // offsets in the stage
    __host__ __device__ StageLayout(int f0, int f1, int v0, int v1) {
        constexpr int FA = 16 / (int)sizeof(B) > 4 ? 16 / (int)sizeof(B) : 4;  // covers bitmaps and the int offsets
        constexpr int VA = 16 / (int)sizeof(V);
        fa = f0 & ~(FA - 1);
        va = v0 & ~(VA - 1);
        auto up16 = [](size_t b) { return (uint32_t)((b + 15) & ~(size_t)15); };
        nBit = up16((size_t)(f1 - fa) * sizeof(B));
        nPtr = up16((size_t)(f1 + 1 - fa) * 4);
        nX = up16((size_t)(f1 - f0) * K * 4);
        nV = up16((size_t)(v1 - va) * sizeof(V));
        oBit = 16;  // the first 16 bytes hold the mbarrier
        oPtr = oBit + nBit;
        oX = oPtr + nPtr;
        oV = oX + nX;
    }
    __host__ __device__ uint32_t total() const { return oV + nV; }
};

// one work segment, run out of a landed stage
template <typename B, typename V, int K, typename OutT, bool ACCUM>
__device__ __forceinline__ void run_segment(const int4 sd, int s, int lane, const B *sBit, const int *sPtr,
                                            const int *sX, const V *sVal, const V *__restrict__ x_d,
                                            const int *__restrict__ panelFirstSeg,
                                            typename std::conditional<sizeof(V) == 8, double, float>::type *partial,
                                            unsigned *panelCount, OutT *out, const int *row_map, int dRows) {
    const int p = sd.x, f0 = sd.y, f1 = sd.z;
    // where the row this lane may store goes: asked for before the fragment loop so that it is there afterwards
    const int myRow = p * 8 + (lane >> 2);
    const int outRow = (row_map && myRow < dRows) ? __ldg(row_map + myRow) : myRow;
    if constexpr (sizeof(V) == 8) {
        const uint32_t below = (1u << lane) - 1u;
        const int kx = lane & 3;
        double c0 = 0.0, c1 = 0.0, e0 = 0.0, e1 = 0.0;  // two independent accumulator chains
        int f = f0;
#pragma unroll(TILE_UNROLL)
        for (; f + 1 < f1; f += 2) {
            const uint32_t bmA = (uint32_t)sBit[f], bmB = (uint32_t)sBit[f + 1];
            const double aA = ((bmA >> lane) & 1u) ? sVal[sPtr[f] + __popc(bmA & below)] : 0.0;
            const double aB = ((bmB >> lane) & 1u) ? sVal[sPtr[f + 1] + __popc(bmB & below)] : 0.0;
            // every lane gathers the x value of its own fragment column: 4 distinct addresses per instruction
            const double bA = __ldg(x_d + sX[(size_t)f * 4 + kx]), bB = __ldg(x_d + sX[(size_t)(f + 1) * 4 + kx]);
            asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0,%1}, {%2}, {%3}, {%0,%1};"
                         : "+d"(c0), "+d"(c1)
                         : "d"(aA), "d"(bA));
            asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0,%1}, {%2}, {%3}, {%0,%1};"
                         : "+d"(e0), "+d"(e1)
                         : "d"(aB), "d"(bB));
        }
        if (f < f1) {
            const uint32_t bmA = (uint32_t)sBit[f];
            const double aA = ((bmA >> lane) & 1u) ? sVal[sPtr[f] + __popc(bmA & below)] : 0.0;
            const double bA = __ldg(x_d + sX[(size_t)f * 4 + kx]);
            asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0,%1}, {%2}, {%3}, {%0,%1};"
                         : "+d"(c0), "+d"(c1)
                         : "d"(aA), "d"(bA));
        }
        // lane 4g holds C[g][0], the sum of panel row g
        finish_staged<double, OutT, ACCUM>(c0 + e0, (lane & 3) == 0, lane >> 2, lane, p, s, sd.w, myRow, outRow, dRows,
                                           panelFirstSeg, (double *)partial, panelCount, out);
    } else {
        const int g = lane >> 2, tq = lane & 3;
        const int lo = 2 * lane;
        const uint64_t below = (1ull << lo) - 1ull;
        float c0 = 0.f, c1 = 0.f, c2 = 0.f, c3 = 0.f;
        for (int f = f0; f < f1; f += 4) {
            unsigned a[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                a[j] = 0u;
                if (f + j < f1) {  // warp-uniform
                    const uint64_t bm = (uint64_t)sBit[f + j];
                    const int off = sPtr[f + j] + __popcll(bm & below);
                    const unsigned bit0 = (unsigned)(bm >> lo) & 1u, bit1 = (unsigned)(bm >> (lo + 1)) & 1u;
                    const unsigned h0 = bit0 ? (unsigned)__half_as_ushort(sVal[off]) : 0u;
                    const unsigned h1 = bit1 ? (unsigned)__half_as_ushort(sVal[off + bit0]) : 0u;
                    a[j] = h0 | (h1 << 16);
                }
            }
            // B column g: g = 0 -> x-segments of fragments f, f+1; g = 1 -> of f+2, f+3; other columns zero
            unsigned b0 = 0u, b1 = 0u;
            if (g < 2) {
                const int fb = f + 2 * g;
                if (fb < f1) {
                    const int2 ix = *reinterpret_cast<const int2 *>(sX + (size_t)fb * 8 + 2 * tq);
                    b0 = (unsigned)__half_as_ushort(__ldg(x_d + ix.x)) |
                         ((unsigned)__half_as_ushort(__ldg(x_d + ix.y)) << 16);
                }
                if (fb + 1 < f1) {
                    const int2 ix = *reinterpret_cast<const int2 *>(sX + (size_t)(fb + 1) * 8 + 2 * tq);
                    b1 = (unsigned)__half_as_ushort(__ldg(x_d + ix.x)) |
                         ((unsigned)__half_as_ushort(__ldg(x_d + ix.y)) << 16);
                }
            }
            // A registers: {rows g, k low} = frag 0, {rows g+8, k low} = frag 2, {rows g, k high} = frag 1,
            // {rows g+8, k high} = frag 3
            asm volatile(
                "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
                "{%0,%1,%2,%3};"
                : "+f"(c0), "+f"(c1), "+f"(c2), "+f"(c3)
                : "r"(a[0]), "r"(a[2]), "r"(a[1]), "r"(a[3]), "r"(b0), "r"(b1));
        }
        // lane 4g: c0 = C[g][0] (fragments f, f+1), c3 = C[g+8][1] (fragments f+2, f+3)
        finish_staged<float, OutT, ACCUM>(c0 + c3, tq == 0, g, lane, p, s, sd.w, myRow, outRow, dRows, panelFirstSeg,
                                          (float *)partial, panelCount, out);
    }
}

// A work segment whose fragments are all completely filled needs neither its bitmaps nor its value offsets: fragment f
// holds the values [v(f0) + (f - f0) * 8K, ...) in bit order, so every lane streams its own values straight from global
// memory (coalesced, 256 / 128 bytes per fragment) and only the K x-indices of a fragment are shared by its 8 rows.
// Per non-zero that is sizeof(value) + 4/8 bytes (FP64: 8.5 B against 12 B as CSR).
__device__ __forceinline__ double ldg_nc_stream(const double *p) {
    double r;
    asm volatile("ld.global.nc.L1::no_allocate.f64 %0, [%1];" : "=d"(r) : "l"(p));
    return r;
}
__device__ __forceinline__ unsigned ldg_nc_stream(const unsigned *p) {
    unsigned r;
    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(r) : "l"(p));
    return r;
}

template <typename B, typename V, int K, typename OutT, bool ACCUM>
__device__ __forceinline__ void run_segment_full(const int4 sd, int s, int lane, int vseg, const V *__restrict__ tcVal,
                                                 const int *__restrict__ AToX, const V *__restrict__ x_d,
                                                 const int *__restrict__ panelFirstSeg,
                                                 typename std::conditional<sizeof(V) == 8, double, float>::type *partial,
                                                 unsigned *panelCount, OutT *out, const int *row_map, int dRows) {
    const int p = sd.x, f0 = sd.y, f1 = sd.z;  // vseg: value offset of fragment f0
    const int myRow = p * 8 + (lane >> 2);
    const int outRow = (row_map && myRow < dRows) ? __ldg(row_map + myRow) : myRow;
    if constexpr (sizeof(V) == 8) {
        const int kx = lane & 3;
        const double *vp = tcVal + vseg + lane;
        const int *xp = AToX + (size_t)f0 * 4 + kx;
        double c0 = 0.0, c1 = 0.0, e0 = 0.0, e1 = 0.0;
        int f = f0;
#pragma unroll 4
        for (; f + 1 < f1; f += 2, vp += 64, xp += 8) {
            const double aA = ldg_nc_stream(vp), aB = ldg_nc_stream(vp + 32);
            const double bA = __ldg(x_d + __ldg(xp)), bB = __ldg(x_d + __ldg(xp + 4));
            asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0,%1}, {%2}, {%3}, {%0,%1};"
                         : "+d"(c0), "+d"(c1)
                         : "d"(aA), "d"(bA));
            asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0,%1}, {%2}, {%3}, {%0,%1};"
                         : "+d"(e0), "+d"(e1)
                         : "d"(aB), "d"(bB));
        }
        if (f < f1) {
            const double aA = ldg_nc_stream(vp);
            const double bA = __ldg(x_d + __ldg(xp));
            asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0,%1}, {%2}, {%3}, {%0,%1};"
                         : "+d"(c0), "+d"(c1)
                         : "d"(aA), "d"(bA));
        }
        finish_staged<double, OutT, ACCUM>(c0 + e0, (lane & 3) == 0, lane >> 2, lane, p, s, sd.w, myRow, outRow, dRows,
                                           panelFirstSeg, (double *)partial, panelCount, out);
    } else {
        // lane l owns bits 2l, 2l+1 of every fragment: one 4-byte load per fragment
        const int g = lane >> 2, tq = lane & 3;
        const unsigned *vp = reinterpret_cast<const unsigned *>(tcVal + vseg) + lane;
        float c0 = 0.f, c1 = 0.f, c2 = 0.f, c3 = 0.f;
        for (int f = f0; f < f1; f += 4, vp += 128) {
            unsigned a[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) a[j] = f + j < f1 ? ldg_nc_stream(vp + 32 * j) : 0u;
            unsigned b0 = 0u, b1 = 0u;
            if (g < 2) {
                const int fb = f + 2 * g;
                if (fb < f1) {
                    const int2 ix = __ldg(reinterpret_cast<const int2 *>(AToX + (size_t)fb * 8 + 2 * tq));
                    b0 = (unsigned)__half_as_ushort(__ldg(x_d + ix.x)) |
                         ((unsigned)__half_as_ushort(__ldg(x_d + ix.y)) << 16);
                }
                if (fb + 1 < f1) {
                    const int2 ix = __ldg(reinterpret_cast<const int2 *>(AToX + (size_t)(fb + 1) * 8 + 2 * tq));
                    b1 = (unsigned)__half_as_ushort(__ldg(x_d + ix.x)) |
                         ((unsigned)__half_as_ushort(__ldg(x_d + ix.y)) << 16);
                }
            }
            asm volatile(
                "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
                "{%0,%1,%2,%3};"
                : "+f"(c0), "+f"(c1), "+f"(c2), "+f"(c3)
                : "r"(a[0]), "r"(a[2]), "r"(a[1]), "r"(a[3]), "r"(b0), "r"(b1));
        }
        finish_staged<float, OutT, ACCUM>(c0 + c3, tq == 0, g, lane, p, s, sd.w, myRow, outRow, dRows, panelFirstSeg,
                                          (float *)partial, panelCount, out);
    }
}

// Every fragment of the matrix completely filled (block-structured matrices): one warp per work segment, no shared
// memory, the value offset of fragment f is f * 8K.
template <typename B, typename V, int K, typename OutT, bool ACCUM>
__global__ void __launch_bounds__(128)
    tile_kernel_full(const V *__restrict__ x_d, const V *__restrict__ tcVal, const int *__restrict__ AToX,
                     const int4 *__restrict__ segDesc, int numSegs, const int *__restrict__ panelFirstSeg,
                     typename std::conditional<sizeof(V) == 8, double, float>::type *__restrict__ partial,
                     unsigned *__restrict__ panelCount, OutT *__restrict__ out, const int *__restrict__ row_map,
                     int dRows) {
    const int s = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (s >= numSegs) return;
    const int4 sd = __ldg(segDesc + s);
    run_segment_full<B, V, K, OutT, ACCUM>(sd, s, lane, sd.y * 8 * K, tcVal, AToX, x_d, panelFirstSeg, partial,
                                           panelCount, out, row_map, dRows);
}

template <typename B, typename V, int K, typename OutT, bool ACCUM, int NWARPS>
__global__ void __launch_bounds__(NWARPS * 32)
    tile_kernel_staged(const V *__restrict__ x_d, const int *__restrict__ fragPtr, const B *__restrict__ fragBit,
                       const V *__restrict__ tcVal, const int *__restrict__ AToX, const CtaDesc *__restrict__ desc,
                       const int4 *__restrict__ segDesc, const int *__restrict__ panelFirstSeg,
                       typename std::conditional<sizeof(V) == 8, double, float>::type *__restrict__ partial,
                       unsigned *__restrict__ panelCount, OutT *__restrict__ out, const int *__restrict__ row_map,
                       int dRows, int *__restrict__ devErr, int prefetchCtas) {
    extern __shared__ __align__(16) unsigned char stage[];
    uint64_t *bar = reinterpret_cast<uint64_t *>(stage);
    const CtaDesc d = desc[blockIdx.x];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const StageLayout<B, V, K> L(d.f0, d.f1, d.v0, d.v1);
    if (threadIdx.x == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(bar)) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        const uint32_t bytes = L.nBit + L.nPtr + L.nX + L.nV;
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                     : "memory");
        if (L.nX) bulk_g2s(stage + L.oX, AToX + (size_t)d.f0 * K, L.nX, bar);  // first: the x gathers wait on it
        if (L.nBit) bulk_g2s(stage + L.oBit, fragBit + L.fa, L.nBit, bar);
        if (L.nPtr) bulk_g2s(stage + L.oPtr, fragPtr + L.fa, L.nPtr, bar);
        if (L.nV) bulk_g2s(stage + L.oV, tcVal + L.va, L.nV, bar);
    }
    if (prefetchCtas > 0 && blockIdx.x + prefetchCtas < gridDim.x) {
        // while this stage is in flight: ask L2 for the stage of the CTA one wave ahead
        const CtaDesc dn = desc[blockIdx.x + prefetchCtas];
        const StageLayout<B, V, K> Ln(dn.f0, dn.f1, dn.v0, dn.v1);
        const char *base[4] = {reinterpret_cast<const char *>(AToX + (size_t)dn.f0 * K),
                               reinterpret_cast<const char *>(fragBit + Ln.fa),
                               reinterpret_cast<const char *>(fragPtr + Ln.fa),
                               reinterpret_cast<const char *>(tcVal + Ln.va)};
        const uint32_t len[4] = {Ln.nX, Ln.nBit, Ln.nPtr, Ln.nV};
#pragma unroll
        for (int r = 0; r < 4; ++r)
            for (uint32_t off = threadIdx.x * 128u; off < len[r]; off += NWARPS * 32 * 128u)
                asm volatile("prefetch.global.L2 [%0];" ::"l"(base[r] + off));
    }
    if (!mbar_wait_bounded(bar)) {  // never expected; leaves a mark instead of spinning for ever
        if (lane == 0 && devErr) atomicOr(devErr, DEVERR_TILE_RANGE);
        return;
    }
    const B *sBit = reinterpret_cast<const B *>(stage + L.oBit) - L.fa;      // index with the global fragment id
    const int *sPtr = reinterpret_cast<const int *>(stage + L.oPtr) - L.fa;  // "
    const V *sVal = reinterpret_cast<const V *>(stage + L.oV) - L.va;        // index with the global value offset
    const int *sX = reinterpret_cast<const int *>(stage + L.oX) - (size_t)d.f0 * K;  // index with fragment id * K + k

    int s = d.seg0 + warp;
    int4 sd = s < d.seg1 ? __ldg(segDesc + s) : make_int4(0, 0, 0, -1);
    while (s < d.seg1) {
        const int sn = s + NWARPS;
        const int4 sdn = sn < d.seg1 ? __ldg(segDesc + sn) : make_int4(0, 0, 0, -1);  // next descriptor, early
        run_segment<B, V, K, OutT, ACCUM>(sd, s, lane, sBit, sPtr, sX, sVal, x_d, panelFirstSeg, partial, panelCount,
                                          out, row_map, dRows);
        s = sn;
        sd = sdn;
    }
}

__global__ void seg_pack_kernel(const int *__restrict__ segPanel, const int *__restrict__ segBegin,
                                const int *__restrict__ segEnd, const int *__restrict__ segSlot, int numSegs,
                                int4 *__restrict__ segDesc) {
    int s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s < numSegs) segDesc[s] = make_int4(segPanel[s], segBegin[s], segEnd[s], segSlot[s]);
}

// bytes a segment brings into shared memory
template <typename B, typename V, int K>
__global__ void seg_cost_kernel(const int *__restrict__ segBegin, const int *__restrict__ segEnd,
                                const int *__restrict__ fragPtr, int numSegs, long long *__restrict__ cost) {
    int s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s > numSegs) return;
    long long c = 0;
    if (s < numSegs) {
        const int f0 = segBegin[s], f1 = segEnd[s];
        c = (long long)(f1 - f0) * (sizeof(B) + 4 + 4 * K) + (long long)(fragPtr[f1] - fragPtr[f0]) * sizeof(V);
    }
    cost[s] = c;
}

// CTA c starts at the first segment whose byte prefix reaches c * STAGE_BYTES
template <typename B, typename V, int K>
__global__ void cta_desc_kernel(const long long *__restrict__ prefix, const int *__restrict__ segBegin,
                                const int *__restrict__ segEnd, const int *__restrict__ fragPtr, int numSegs,
                                int numCtas, int STAGE_BYTES, CtaDesc *__restrict__ desc,
                                unsigned *__restrict__ maxBytes) {
    int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= numCtas) return;
    auto first = [&](int cc) {
        if (cc >= numCtas) return numSegs;
        const long long target = (long long)cc * STAGE_BYTES;
        int lo = 0, hi = numSegs;
        while (lo < hi) {
            int mid = (lo + hi) >> 1;
            if (prefix[mid] < target)
                lo = mid + 1;
            else
                hi = mid;
        }
        return lo;
    };
    CtaDesc d;
    d.seg0 = c == 0 ? 0 : first(c);
    d.seg1 = first(c + 1);
    d.full = d.pad1 = 0;
    if (d.seg1 > d.seg0) {
        d.f0 = segBegin[d.seg0];
        d.f1 = segEnd[d.seg1 - 1];
    } else {
        d.f0 = d.f1 = 0;
    }
    d.v0 = fragPtr[d.f0];
    d.v1 = fragPtr[d.f1];
    d.full = d.f1 > d.f0 && (long long)(d.v1 - d.v0) == (long long)(d.f1 - d.f0) * 8 * K;
    desc[c] = d;
    atomicMax(maxBytes, StageLayout<B, V, K>(d.f0, d.f1, d.v0, d.v1).total());
}

}  // namespace

cudaError_t tile_plan_build(int dtype, TilePlan &P, cudaStream_t s) {
    cudaError_t e;
    if (P.A.chunkNum <= 0) {
        P.numSegs = 0;
        return cudaSuccess;
    }
    int *segCount = nullptr, *multiCount = nullptr, *firstSlot = nullptr;
    size_t np = (size_t)P.A.chunkNum + 1;
    if ((e = cudaMallocAsync(&segCount, np * sizeof(int), s)) != cudaSuccess) return e;
    if ((e = cudaMallocAsync(&multiCount, np * sizeof(int), s)) != cudaSuccess) return e;
    if ((e = cudaMallocAsync(&firstSlot, np * sizeof(int), s)) != cudaSuccess) return e;
    if ((e = cudaMallocAsync(&P.panelFirstSeg, np * sizeof(int), s)) != cudaSuccess) return e;
    seg_count_kernel<<<(int)((np + 255) / 256), 256, 0, s>>>(P.A.chunkPtr, P.A.chunkNum, segCount, multiCount);
    TempBuf tmp;
    if ((e = exclusive_sum(tmp, segCount, P.panelFirstSeg, (int)np, s)) != cudaSuccess) return e;
    if ((e = exclusive_sum(tmp, multiCount, firstSlot, (int)np, s)) != cudaSuccess) return e;
    int totals[2];
    if ((e = cudaMemcpyAsync(&totals[0], P.panelFirstSeg + P.A.chunkNum, sizeof(int), cudaMemcpyDeviceToHost, s)) !=
        cudaSuccess)
        return e;
    if ((e = cudaMemcpyAsync(&totals[1], firstSlot + P.A.chunkNum, sizeof(int), cudaMemcpyDeviceToHost, s)) !=
        cudaSuccess)
        return e;
    if ((e = cudaStreamSynchronize(s)) != cudaSuccess) return e;
    P.numSegs = totals[0];
    P.numMultiSegs = totals[1];
    size_t ns = (size_t)P.numSegs;
    if ((e = cudaMallocAsync(&P.segPanel, ns * sizeof(int), s)) != cudaSuccess) return e;
    if ((e = cudaMallocAsync(&P.segBegin, ns * sizeof(int), s)) != cudaSuccess) return e;
    if ((e = cudaMallocAsync(&P.segEnd, ns * sizeof(int), s)) != cudaSuccess) return e;
    if ((e = cudaMallocAsync(&P.segSlot, ns * sizeof(int), s)) != cudaSuccess) return e;
    if ((e = cudaMallocAsync(&P.partial, (size_t)(P.numMultiSegs > 0 ? P.numMultiSegs : 1) * 8 * acc_bytes(dtype),
                             s)) != cudaSuccess)
        return e;
    if ((e = cudaMallocAsync(&P.panelCount, (size_t)P.A.chunkNum * sizeof(unsigned), s)) != cudaSuccess) return e;
    if ((e = cudaMemsetAsync(P.panelCount, 0, (size_t)P.A.chunkNum * sizeof(unsigned), s)) != cudaSuccess) return e;
    seg_fill_kernel<<<(P.A.chunkNum + 255) / 256, 256, 0, s>>>(P.A.chunkPtr, P.A.chunkNum, P.panelFirstSeg, firstSlot,
                                                             P.segPanel, P.segBegin, P.segEnd, P.segSlot);
    e = cudaGetLastError();
    cudaError_t e2 = cudaStreamSynchronize(s);
    if (segCount) cudaFreeAsync(segCount, s);
    if (multiCount) cudaFreeAsync(multiCount, s);
    if (firstSlot) cudaFreeAsync(firstSlot, s);
    if (e != cudaSuccess) return e;
    if (e2 != cudaSuccess) return e2;
    if ((e = cudaMallocAsync(&P.segDesc, (ns > 0 ? ns : 1) * sizeof(int4), s)) != cudaSuccess) return e;
    seg_pack_kernel<<<(P.numSegs + 255) / 256, 256, 0, s>>>(P.segPanel, P.segBegin, P.segEnd, P.segSlot, P.numSegs,
                                                            (int4 *)P.segDesc);
    // CTA descriptors of the TMA-staged kernel: consecutive segments grouped by the bytes they stage
    long long *cost = nullptr, *prefix = nullptr;
    unsigned *maxBytes = nullptr;
    if ((e = cudaMallocAsync(&cost, (ns + 1) * sizeof(long long), s)) != cudaSuccess) return e;
    if ((e = cudaMallocAsync(&prefix, (ns + 1) * sizeof(long long), s)) != cudaSuccess) return e;
    if ((e = cudaMallocAsync(&maxBytes, sizeof(unsigned), s)) != cudaSuccess) return e;
    if ((e = cudaMemsetAsync(maxBytes, 0, sizeof(unsigned), s)) != cudaSuccess) return e;
    const int cgrid = (P.numSegs + 1 + 255) / 256;
    if (dtype == MX_FP64)
        seg_cost_kernel<uint32_t, double, 4><<<cgrid, 256, 0, s>>>(P.segBegin, P.segEnd, P.A.fragPtr, P.numSegs, cost);
    else
        seg_cost_kernel<uint64_t, __half, 8><<<cgrid, 256, 0, s>>>(P.segBegin, P.segEnd, P.A.fragPtr, P.numSegs, cost);
    if ((e = exclusive_sum(tmp, cost, prefix, P.numSegs + 1, s)) != cudaSuccess) return e;
    long long totalBytes = 0;
    if ((e = cudaMemcpyAsync(&totalBytes, prefix + P.numSegs, sizeof(long long), cudaMemcpyDeviceToHost, s)) !=
        cudaSuccess)
        return e;
    if ((e = cudaStreamSynchronize(s)) != cudaSuccess) return e;
    if (g_tile_prefetch < 0) {
        int dev = 0, sms = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        g_tile_prefetch = 5 * sms;
    }
    // all fragments completely filled <=> the packed values are exactly 8K per fragment
    P.allFull = P.A.totalFrags > 0 && (long long)P.A.nvals == (long long)P.A.totalFrags * 8 * (dtype == MX_FP64 ? 4 : 8) &&
                true;
    P.useFull = P.allFull;
    const int STAGE_BYTES = STAGE_BYTES_TARGET;
    P.numCtas = (int)((totalBytes + STAGE_BYTES - 1) / STAGE_BYTES);
    if (P.numCtas < 1) P.numCtas = 1;
    if ((e = cudaMallocAsync(&P.ctaDesc, (size_t)P.numCtas * sizeof(CtaDesc), s)) != cudaSuccess) return e;
    if (dtype == MX_FP64)
        cta_desc_kernel<uint32_t, double, 4><<<(P.numCtas + 127) / 128, 128, 0, s>>>(
            prefix, P.segBegin, P.segEnd, P.A.fragPtr, P.numSegs, P.numCtas, STAGE_BYTES, (CtaDesc *)P.ctaDesc, maxBytes);
    else
        cta_desc_kernel<uint64_t, __half, 8><<<(P.numCtas + 127) / 128, 128, 0, s>>>(
            prefix, P.segBegin, P.segEnd, P.A.fragPtr, P.numSegs, P.numCtas, STAGE_BYTES, (CtaDesc *)P.ctaDesc, maxBytes);
    unsigned mb = 0;
    if ((e = cudaMemcpyAsync(&mb, maxBytes, sizeof(unsigned), cudaMemcpyDeviceToHost, s)) != cudaSuccess) return e;
    e = cudaStreamSynchronize(s);
    P.stageBytes = (int)mb;
    if (cost) cudaFreeAsync(cost, s);
    if (prefix) cudaFreeAsync(prefix, s);
    if (maxBytes) cudaFreeAsync(maxBytes, s);
    if (e != cudaSuccess) return e;
    return cudaGetLastError();
}

void tile_plan_free(TilePlan &P, cudaStream_t s) {
    if (P.segPanel) cudaFreeAsync(P.segPanel, s);
    if (P.segBegin) cudaFreeAsync(P.segBegin, s);
    if (P.segEnd) cudaFreeAsync(P.segEnd, s);
    if (P.segSlot) cudaFreeAsync(P.segSlot, s);
    if (P.panelFirstSeg) cudaFreeAsync(P.panelFirstSeg, s);
    if (P.partial) cudaFreeAsync(P.partial, s);
    if (P.panelCount) cudaFreeAsync(P.panelCount, s);
    if (P.ctaDesc) cudaFreeAsync(P.ctaDesc, s);
    if (P.segDesc) cudaFreeAsync(P.segDesc, s);
    P.ctaDesc = P.segDesc = nullptr;
    P.numCtas = 0;
    P.segPanel = P.segBegin = P.segEnd = P.segSlot = P.panelFirstSeg = nullptr;
    P.partial = nullptr;
    P.panelCount = nullptr;
    P.numSegs = 0;
}

int tile_launches(const TilePlan &P) { return P.numSegs > 0 ? 1 : 0; }

cudaError_t tile_spmv(int dtype, const TilePlan &P, const void *x_d, void *out, const int *row_map, bool out_is_acc,
                      bool accumulate, int *dev_err, cudaStream_t s) {
    if (P.numSegs <= 0) return cudaSuccess;
    if (P.allFull && P.useFull) {  // nothing to decode anywhere: the streaming kernel
        const dim3 fg((P.numSegs + 3) / 4), fb(128);
#define MX_FULL(BT, VT, KK, OT, AC, AT)                                                                              \
    tile_kernel_full<BT, VT, KK, OT, AC><<<fg, fb, 0, s>>>((const VT *)x_d, (const VT *)P.A.tcVal, P.A.AToX,         \
                                                           (const int4 *)P.segDesc, P.numSegs, P.panelFirstSeg,      \
                                                           (AT *)P.partial, P.panelCount, (OT *)out, row_map,        \
                                                           P.A.dRows)
        if (dtype == MX_FP64) {
            if (accumulate)
                MX_FULL(uint32_t, double, 4, double, true, double);
            else
                MX_FULL(uint32_t, double, 4, double, false, double);
        } else if (out_is_acc) {
            MX_FULL(uint64_t, __half, 8, float, false, float);
        } else if (accumulate) {
            MX_FULL(uint64_t, __half, 8, __half, true, float);
        } else {
            MX_FULL(uint64_t, __half, 8, __half, false, float);
        }
#undef MX_FULL
        return cudaGetLastError();
    }
    if (P.ctaDesc && P.stageBytes > 0 && P.stageBytes <= 200 * 1024) {
        dim3 sg(P.numCtas), sb(STAGE_WARPS * 32);
        const size_t smem = (size_t)P.stageBytes;
#define MX_STAGED(BT, VT, KK, OT, AC, AT)                                                                            \
    do {                                                                                                             \
        auto kern = tile_kernel_staged<BT, VT, KK, OT, AC, STAGE_WARPS>;                                             \
        if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);   \
        kern<<<sg, sb, smem, s>>>((const VT *)x_d, P.A.fragPtr, (const BT *)P.A.fragBit, (const VT *)P.A.tcVal,      \
                                  P.A.AToX, (const CtaDesc *)P.ctaDesc, (const int4 *)P.segDesc,                     \
                                  P.panelFirstSeg, (AT *)P.partial, P.panelCount, (OT *)out, row_map, P.A.dRows,     \
                                  dev_err, g_tile_prefetch);                                                         \
    } while (0)
        if (dtype == MX_FP64) {
            if (accumulate)
                MX_STAGED(uint32_t, double, 4, double, true, double);
            else
                MX_STAGED(uint32_t, double, 4, double, false, double);
        } else if (out_is_acc) {
            MX_STAGED(uint64_t, __half, 8, float, false, float);
        } else if (accumulate) {
            MX_STAGED(uint64_t, __half, 8, __half, true, float);
        } else {
            MX_STAGED(uint64_t, __half, 8, __half, false, float);
        }
#undef MX_STAGED
        return cudaGetLastError();
    }
    return cudaErrorInvalidConfiguration;  // a work segment is at most SEG fragments: its stage always fits
}

}  // namespace mx
