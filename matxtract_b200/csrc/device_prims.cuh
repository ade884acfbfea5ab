// Thin wrappers over CUB's device-wide scan / sort (generic primitives; the domain kernels are hand-written).
#pragma once
#include <cub/cub.cuh>
#include <cuda_runtime.h>

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

}  // namespace mx
