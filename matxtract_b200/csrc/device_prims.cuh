// Thin wrappers over CUB's device-wide scan / sort (generic primitives; the domain kernels are hand-written).
#pragma once
#include <cub/cub.cuh>
#include <cuda_runtime.h>
#include <stdint.h>

namespace mx {

// workspace of the CUB calls, from the stream-ordered pool of the stream it is used on
struct TempBuf {
    void *p = nullptr;
    size_t cap = 0;
    cudaStream_t s = nullptr;
    cudaError_t reserve(size_t bytes, cudaStream_t stream) {
        if (bytes <= cap) return cudaSuccess;
        if (p) cudaFreeAsync(p, s);
        p = nullptr;
        cap = 0;
        s = stream;
        cudaError_t e = cudaMallocAsync(&p, bytes, s);
        if (e == cudaSuccess) cap = bytes;
        return e;
    }
    ~TempBuf() {
        if (p) cudaFreeAsync(p, s);
    }
};

template <typename InT, typename OutT>
inline cudaError_t exclusive_sum(TempBuf &tmp, const InT *in, OutT *out, int n, cudaStream_t s) {
    size_t bytes = 0;
    cudaError_t e = cub::DeviceScan::ExclusiveSum(nullptr, bytes, in, out, n, s);
    if (e != cudaSuccess) return e;
    if ((e = tmp.reserve(bytes, s)) != cudaSuccess) return e;
    return cub::DeviceScan::ExclusiveSum(tmp.p, bytes, in, out, n, s);
}

template <typename InT, typename OutT>
inline cudaError_t inclusive_sum(TempBuf &tmp, const InT *in, OutT *out, int n, cudaStream_t s) {
    size_t bytes = 0;
    cudaError_t e = cub::DeviceScan::InclusiveSum(nullptr, bytes, in, out, n, s);
    if (e != cudaSuccess) return e;
    if ((e = tmp.reserve(bytes, s)) != cudaSuccess) return e;
    return cub::DeviceScan::InclusiveSum(tmp.p, bytes, in, out, n, s);
}

// ---- 1-D bulk copies (TMA) into shared memory, completing on an mbarrier; no multicast ----
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void bulk_g2s(void *dst_smem, const void *src_gmem, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst_smem)),
                 "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// waits for phase 0 of the barrier; gives up after a bounded number of polls (returns false)
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t *bar) {
    const uint32_t a = smem_u32(bar);
    for (int it = 0; it < (1 << 22); ++it) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(a), "r"(0u)
            : "memory");
        if (ok) return true;
    }
    return false;
}

}  // namespace mx
