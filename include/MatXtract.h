// Host API of the MatXtract SpMV kernels — source-compatible with the reference's include/MatXtract.h.
// Same names, argument order and conventions: every pointer is a HOST pointer owned by the caller, vectors are passed
// by value, each call is synchronous, allocates and frees its own device memory, times 200 warm-up + 4000 timed
// launches and returns milliseconds per launch through its last argument; a CUDA failure prints a message and exits
// (include/common.h:81-90 of the reference).  Implemented in libMatXtract_fp64.so / libMatXtract_fp16.so on top of the
// C ABI in mx_capi.h.
#pragma once
#include "common.h"

// y += A x on the CUDA cores; Y_val is in/out (reference src/spmv_kernel/cdSpMV.cu:395-491).
void cdspmv(valT *csrVal, indT *csrRowPtr, indT *csrColInd, valT *X_val, valT *Y_val, int rowA, int colA, indT nnzA,
            double *cdTime, double *cdPre);
#ifdef fp64
// Fragment-format SpMV on the tensor cores; Y_val is added to (reference src/spmv_kernel/du_tcSpMV_fp64.cu:258-350).
void du_tcspmv_fp64(indT *chunkPtr, std::vector<int> fragPtr, std::vector<uint32_t> fragBit, std::vector<double> tcVal,
                    indT *sparse_AToX_index, valT *X_val, valT *Y_val, int rowA, int colA, int *row_order,
                    double *tcTime);
// SpMV of the core-dense block given as CSR; Y_val[i] belongs to input row order_rid[i]
// (reference src/spmv_kernel/se_tcSpMV_fp64.cu:496-1496).  NUM, threshold and block_longest tune the reference's
// row-length bucketing and are accepted and ignored here.
void se_tcspmv_fp64(valT *csrValA, indT *csrRowPtrA, int *csrColIdxA, valT *X_val, valT *Y_val, int *order_rid,
                    int rowA, int colA, indT nnzA, int NUM, double threshold, int block_longest, double *tcTime);
#else
// 8x4 fragments with 32-bit bitmaps (the reference's older FP16 kernels, src/spmv_kernel/du_tcSpMV_fp16.cu).
void du_tcspmv_fp16_v0(int *chunkPtr, std::vector<int> fragPtr, std::vector<uint32_t> fragBit, std::vector<half> tcVal,
                       int *sparse_AToX_index, half *X_val, half *Y_val, int rowA, int colA, int *row_order,
                       double *tcTime);
void du_tcspmv_fp16_v1(int *chunkPtr, std::vector<int> fragPtr, std::vector<uint32_t> fragBit, std::vector<half> tcVal,
                       int *sparse_AToX_index, half *X_val, half *Y_val, int rowA, int colA, int *row_order,
                       double *tcTime);
// 8x8 fragments with 64-bit bitmaps; Y_val is overwritten (reference src/spmv_kernel/du_tcSpMV_fp16_v2.cu:112-203).
void du_tcspmv_fp16_v2(indT *chunkPtr, std::vector<int> fragPtr, std::vector<uint64_t> fragBit, std::vector<half> tcVal,
                       indT *sparse_AToX_index, half *X_val, half *Y_val, int rowA, int colA, int *row_order,
                       double *tcTime);
void se_tcspmv_fp16(valT *csrValA, indT *csrRowPtrA, int *csrColIdxA, valT *X_val, valT *Y_val, int *order_rid,
                    int rowA, int colA, indT nnzA, int NUM, double threshold, int block_longest, double *tcTime);
#endif
