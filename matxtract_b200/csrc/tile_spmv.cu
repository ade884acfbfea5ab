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
//   * Bitmaps, value offsets and x indices of 8 fragments are fetched with one coalesced load each and
//     handed round with warp shuffles; the gathered x values likewise (one gather per lane).
//   * Sums stay in the accumulator registers over the whole fragment run; one store per row, no atomics
//     on y.  The reference gives every panel one warp; a power-law panel can hold 10^4 fragments, so
//     here a panel is cut into segments of at most SEG fragments, one warp each.  Segments of a split
//     panel park their 8 partial sums; the last one to arrive (a counter, no spinning) adds them in
//     segment order, so the result does not depend on arrival order.
#include "device_prims.cuh"
#include "mx_internal.h"

namespace mx {
namespace {

constexpr int SEG = 64;            // fragments per work segment
constexpr int TILE_WARPS = 4;      // warps per CTA

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

// Hands the 8 row sums of one segment over: directly to `out` when the panel has a single segment,
// through `partial` + arrival counter otherwise.  rowLane: this lane holds the sum of panel row g.
template <typename A, typename OutT, bool ACCUM>
__device__ __forceinline__ void finish_segment(A sum, bool rowLane, int g, int lane, int p, int s, int dRows,
                                               const int *__restrict__ segSlot,
                                               const int *__restrict__ panelFirstSeg, A *__restrict__ partial,
                                               unsigned *__restrict__ panelCount, OutT *__restrict__ out,
                                               const int *__restrict__ row_map) {
    const int row = p * 8 + g;
    const int slot = segSlot[s];
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
        const int slot0 = segSlot[first];
        sum = A(0);
        if (rowLane)
            for (int j = 0; j < nseg; ++j) sum += __ldcg(partial + (size_t)(slot0 + j) * 8 + g);
    }
    if (rowLane && row < dRows) {
        const int o = row_map ? row_map[row] : row;
        if (ACCUM) sum += (A)get(out + o);
        put(out + o, sum);
    }
}

template <typename OutT, bool ACCUM>
__global__ void __launch_bounds__(TILE_WARPS * 32)
    tile_kernel_fp64(const double *__restrict__ x_d, const int *__restrict__ fragPtr,
                     const uint32_t *__restrict__ fragBit, const double *__restrict__ tcVal,
                     const int *__restrict__ AToX, const int *__restrict__ segPanel, const int *__restrict__ segBegin,
                     const int *__restrict__ segEnd, const int *__restrict__ segSlot,
                     const int *__restrict__ panelFirstSeg, double *__restrict__ partial,
                     unsigned *__restrict__ panelCount, OutT *__restrict__ out, const int *__restrict__ row_map,
                     int dRows, int numSegs) {
    const int lane = threadIdx.x & 31;
    const int s = blockIdx.x * TILE_WARPS + (threadIdx.x >> 5);
    if (s >= numSegs) return;
    const int p = segPanel[s], f0 = segBegin[s], f1 = segEnd[s];
    const uint32_t below = (1u << lane) - 1u;
    double c0 = 0.0, c1 = 0.0;
    for (int f = f0; f < f1; f += 8) {
        const int nb = min(8, f1 - f);
        const uint32_t bm_l = lane < nb ? __ldg(fragBit + f + lane) : 0u;
        const int ptr_l = lane < nb ? __ldg(fragPtr + f + lane) : 0;
        const int xi = (lane >> 2) < nb ? __ldg(AToX + (size_t)f * 4 + lane) : -1;
        const double xv = xi >= 0 ? __ldg(x_d + xi) : 0.0;
        double a[8], b[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const uint32_t bm = __shfl_sync(0xffffffffu, bm_l, j);
            const int ptr = __shfl_sync(0xffffffffu, ptr_l, j);
            b[j] = __shfl_sync(0xffffffffu, xv, 4 * j + (lane & 3));
            a[j] = ((bm >> lane) & 1u) ? __ldg(tcVal + ptr + __popc(bm & below)) : 0.0;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j)
            asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0,%1}, {%2}, {%3}, {%0,%1};"
                         : "+d"(c0), "+d"(c1)
                         : "d"(a[j]), "d"(b[j]));
    }
    // lane 4g holds C[g][0], the sum of panel row g
    finish_segment<double, OutT, ACCUM>(c0, (lane & 3) == 0, lane >> 2, lane, p, s, dRows, segSlot, panelFirstSeg,
                                        partial, panelCount, out, row_map);
}

template <typename OutT, bool ACCUM>
__global__ void __launch_bounds__(TILE_WARPS * 32)
    tile_kernel_fp16(const __half *__restrict__ x_d, const int *__restrict__ fragPtr,
                     const uint64_t *__restrict__ fragBit, const __half *__restrict__ tcVal,
                     const int *__restrict__ AToX, const int *__restrict__ segPanel, const int *__restrict__ segBegin,
                     const int *__restrict__ segEnd, const int *__restrict__ segSlot,
                     const int *__restrict__ panelFirstSeg, float *__restrict__ partial,
                     unsigned *__restrict__ panelCount, OutT *__restrict__ out, const int *__restrict__ row_map,
                     int dRows, int numSegs) {
    const int lane = threadIdx.x & 31, g = lane >> 2, tq = lane & 3;
    const int s = blockIdx.x * TILE_WARPS + (threadIdx.x >> 5);
    if (s >= numSegs) return;
    const int p = segPanel[s], f0 = segBegin[s], f1 = segEnd[s];
    const int lo = 2 * lane;
    const uint64_t below = (1ull << lo) - 1ull;
    // source lanes of the packed x pairs this lane needs as B (column g of B; only g = 0, 1 are non-zero)
    const int src0 = (g == 0) ? 2 * tq : 2 * (8 + tq);
    const int src1 = src0 + 8;
    float c0 = 0.f, c1 = 0.f, c2 = 0.f, c3 = 0.f;
    for (int f = f0; f < f1; f += 8) {
        const int nb = min(8, f1 - f);
        const uint64_t bm_l = lane < nb ? __ldg(reinterpret_cast<const unsigned long long *>(fragBit) + f + lane) : 0ull;
        const int ptr_l = lane < nb ? __ldg(fragPtr + f + lane) : 0;
        const int xi0 = (lane >> 3) < nb ? __ldg(AToX + (size_t)f * 8 + lane) : -1;
        const int xi1 = 4 + (lane >> 3) < nb ? __ldg(AToX + (size_t)f * 8 + 32 + lane) : -1;
        const unsigned xb0 = xi0 >= 0 ? (unsigned)__half_as_ushort(__ldg(x_d + xi0)) : 0u;
        const unsigned xb1 = xi1 >= 0 ? (unsigned)__half_as_ushort(__ldg(x_d + xi1)) : 0u;
        // even lane 2q now holds x pair q = (column 2q', 2q'+1) of fragment q/4
        const unsigned pair0 = xb0 | (__shfl_down_sync(0xffffffffu, xb0, 1) << 16);
        const unsigned pair1 = xb1 | (__shfl_down_sync(0xffffffffu, xb1, 1) << 16);
#pragma unroll
        for (int m = 0; m < 2; ++m) {
            if (m == 1 && nb <= 4) break;  // warp-uniform
            const unsigned pair = m == 0 ? pair0 : pair1;
            unsigned b0 = __shfl_sync(0xffffffffu, pair, src0);
            unsigned b1 = __shfl_sync(0xffffffffu, pair, src1);
            if (g > 1) {
                b0 = 0u;
                b1 = 0u;
            }
            unsigned a[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint64_t bm = __shfl_sync(0xffffffffu, bm_l, 4 * m + j);
                const int ptr = __shfl_sync(0xffffffffu, ptr_l, 4 * m + j);
                const int off = ptr + __popcll(bm & below);
                const unsigned bit0 = (unsigned)(bm >> lo) & 1u, bit1 = (unsigned)(bm >> (lo + 1)) & 1u;
                const unsigned h0 = bit0 ? (unsigned)__half_as_ushort(__ldg(tcVal + off)) : 0u;
                const unsigned h1 = bit1 ? (unsigned)__half_as_ushort(__ldg(tcVal + off + bit0)) : 0u;
                a[j] = h0 | (h1 << 16);
            }
            // A registers: {rows g, k low} = frag 0, {rows g+8, k low} = frag 2, {rows g, k high} = frag 1,
            // {rows g+8, k high} = frag 3
            asm volatile(
                "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
                "{%0,%1,%2,%3};"
                : "+f"(c0), "+f"(c1), "+f"(c2), "+f"(c3)
                : "r"(a[0]), "r"(a[2]), "r"(a[1]), "r"(a[3]), "r"(b0), "r"(b1));
        }
    }
    // lane 4g: c0 = C[g][0] (fragments f, f+1), c3 = C[g+8][1] (fragments f+2, f+3)
    finish_segment<float, OutT, ACCUM>(c0 + c3, tq == 0, g, lane, p, s, dRows, segSlot, panelFirstSeg, partial,
                                       panelCount, out, row_map);
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
    if ((e = cudaMalloc(&segCount, np * sizeof(int))) != cudaSuccess) return e;
    if ((e = cudaMalloc(&multiCount, np * sizeof(int))) != cudaSuccess) return e;
    if ((e = cudaMalloc(&firstSlot, np * sizeof(int))) != cudaSuccess) return e;
    if ((e = cudaMalloc(&P.panelFirstSeg, np * sizeof(int))) != cudaSuccess) return e;
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
    if ((e = cudaMalloc(&P.segPanel, ns * sizeof(int))) != cudaSuccess) return e;
    if ((e = cudaMalloc(&P.segBegin, ns * sizeof(int))) != cudaSuccess) return e;
    if ((e = cudaMalloc(&P.segEnd, ns * sizeof(int))) != cudaSuccess) return e;
    if ((e = cudaMalloc(&P.segSlot, ns * sizeof(int))) != cudaSuccess) return e;
    if ((e = cudaMalloc(&P.partial, (size_t)(P.numMultiSegs > 0 ? P.numMultiSegs : 1) * 8 * acc_bytes(dtype))) !=
        cudaSuccess)
        return e;
    if ((e = cudaMalloc(&P.panelCount, (size_t)P.A.chunkNum * sizeof(unsigned))) != cudaSuccess) return e;
    if ((e = cudaMemsetAsync(P.panelCount, 0, (size_t)P.A.chunkNum * sizeof(unsigned), s)) != cudaSuccess) return e;
    seg_fill_kernel<<<(P.A.chunkNum + 255) / 256, 256, 0, s>>>(P.A.chunkPtr, P.A.chunkNum, P.panelFirstSeg, firstSlot,
                                                             P.segPanel, P.segBegin, P.segEnd, P.segSlot);
    e = cudaGetLastError();
    cudaError_t e2 = cudaStreamSynchronize(s);
    cudaFree(segCount);
    cudaFree(multiCount);
    cudaFree(firstSlot);
    return e != cudaSuccess ? e : e2;
}

void tile_plan_free(TilePlan &P) {
    cudaFree(P.segPanel);
    cudaFree(P.segBegin);
    cudaFree(P.segEnd);
    cudaFree(P.segSlot);
    cudaFree(P.panelFirstSeg);
    cudaFree(P.partial);
    cudaFree(P.panelCount);
    P.segPanel = P.segBegin = P.segEnd = P.segSlot = P.panelFirstSeg = nullptr;
    P.partial = nullptr;
    P.panelCount = nullptr;
    P.numSegs = 0;
}

int tile_launches(const TilePlan &P) { return P.numSegs > 0 ? 1 : 0; }

cudaError_t tile_spmv(int dtype, const TilePlan &P, const void *x_d, void *out, const int *row_map, bool out_is_acc,
                      bool accumulate, int *, cudaStream_t s) {
    if (P.numSegs <= 0) return cudaSuccess;
    dim3 grid((P.numSegs + TILE_WARPS - 1) / TILE_WARPS), block(TILE_WARPS * 32);
#define MX_TILE_ARGS(BT, VT, AT)                                                                                   \
    (const VT *)x_d, P.A.fragPtr, (const BT *)P.A.fragBit, (const VT *)P.A.tcVal, P.A.AToX, P.segPanel, P.segBegin, P.segEnd, \
        P.segSlot, P.panelFirstSeg, (AT *)P.partial, P.panelCount
    if (dtype == MX_FP64) {
        if (accumulate)
            tile_kernel_fp64<double, true><<<grid, block, 0, s>>>(MX_TILE_ARGS(uint32_t, double, double),
                                                                  (double *)out, row_map, P.A.dRows, P.numSegs);
        else
            tile_kernel_fp64<double, false><<<grid, block, 0, s>>>(MX_TILE_ARGS(uint32_t, double, double),
                                                                   (double *)out, row_map, P.A.dRows, P.numSegs);
    } else {
        if (out_is_acc)
            tile_kernel_fp16<float, false><<<grid, block, 0, s>>>(MX_TILE_ARGS(uint64_t, __half, float),
                                                                  (float *)out, row_map, P.A.dRows, P.numSegs);
        else if (accumulate)
            tile_kernel_fp16<__half, true><<<grid, block, 0, s>>>(MX_TILE_ARGS(uint64_t, __half, float),
                                                                  (__half *)out, row_map, P.A.dRows, P.numSegs);
        else
            tile_kernel_fp16<__half, false><<<grid, block, 0, s>>>(MX_TILE_ARGS(uint64_t, __half, float),
                                                                   (__half *)out, row_map, P.A.dRows, P.numSegs);
    }
#undef MX_TILE_ARGS
    return cudaGetLastError();
}

}  // namespace mx
