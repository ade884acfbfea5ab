// C++ host API (include/MatXtract.h, include/csr2csc.h) over the C ABI.  Behaviour on failure follows the reference's
// CUDA_CHECK_ERROR (include/common.h:81-90): message on stderr, exit(EXIT_FAILURE).
#include <cstring>

#include "MatXtract.h"
#include "csr2csc.h"
#include "mx_capi.h"

namespace {
#ifdef fp64
const int kDtype = MX_FP64;
#else
const int kDtype = MX_FP16;
#endif
const int kWarm = 200, kIters = 4000;  // every reference wrapper: 200 warm-up + 4000 timed launches

void check(int st, const char *what) {
    if (st != MX_OK) {
        fprintf(stderr, "MatXtract Error: %s in %s\n", mx_status_string(st), what);
        exit(EXIT_FAILURE);
    }
}

void transpose_stable(int n_in, int n_out, int nnz, const int *ptr, const int *ind, const valT *val, valT **oval,
                      int **optr, int **oind) {
    int *p = (int *)calloc((size_t)n_out + 1, sizeof(int));
    int *oi = (int *)malloc(sizeof(int) * (size_t)(nnz > 0 ? nnz : 1));
    valT *ov = (valT *)malloc(sizeof(valT) * (size_t)(nnz > 0 ? nnz : 1));
    for (int e = 0; e < nnz; ++e) p[ind[e] + 1]++;
    for (int j = 0; j < n_out; ++j) p[j + 1] += p[j];
    std::vector<int> cur(p, p + n_out);
    for (int i = 0; i < n_in; ++i)
        for (int e = ptr[i]; e < ptr[i + 1]; ++e) {
            int q = cur[ind[e]]++;
            oi[q] = i;
            ov[q] = val[e];
        }
    *oval = ov;
    *optr = p;
    *oind = oi;
}
}  // namespace

void cdspmv(valT *csrVal, indT *csrRowPtr, indT *csrColInd, valT *X_val, valT *Y_val, int rowA, int colA, indT nnzA,
            double *cdTime, double *cdPre) {
    check(mx_cdspmv(kDtype, csrVal, csrRowPtr, csrColInd, X_val, Y_val, rowA, colA, nnzA, kWarm, kIters, cdTime, cdPre),
          "cdspmv");
}

void csr2csc(valT *csrVal, indT *csrRowPtr, indT *csrColInd, int rowA, int colA, indT nnzA, valT **cscVal,
             indT **cscColPtr, indT **cscRowInd) {
    transpose_stable(rowA, colA, nnzA, csrRowPtr, csrColInd, csrVal, cscVal, cscColPtr, cscRowInd);
}
void csc2csr(valT *cscVal, indT *cscColPtr, indT *cscRowInd, int rowA, int colA, indT nnzA, valT **csrVal,
             indT **csrRowPtr, indT **csrColInd) {
    transpose_stable(colA, rowA, nnzA, cscColPtr, cscRowInd, cscVal, csrVal, csrRowPtr, csrColInd);
}

#ifdef fp64
void du_tcspmv_fp64(indT *chunkPtr, std::vector<int> fragPtr, std::vector<uint32_t> fragBit, std::vector<double> tcVal,
                    indT *sparse_AToX_index, valT *X_val, valT *Y_val, int rowA, int colA, int *, double *tcTime) {
    check(mx_du_tcspmv(kDtype, chunkPtr, fragPtr.data(), fragBit.data(), tcVal.data(), (int)tcVal.size(),
                       sparse_AToX_index, X_val, Y_val, rowA, colA, kWarm, kIters, tcTime),
          "du_tcspmv_fp64");
}
void se_tcspmv_fp64(valT *csrValA, indT *csrRowPtrA, int *csrColIdxA, valT *X_val, valT *Y_val, int *order_rid,
                    int rowA, int colA, indT nnzA, int NUM, double threshold, int block_longest, double *tcTime) {
    check(mx_se_tcspmv(kDtype, csrValA, csrRowPtrA, csrColIdxA, X_val, Y_val, order_rid, rowA, colA, nnzA, NUM,
                       threshold, block_longest, kWarm, kIters, tcTime),
          "se_tcspmv_fp64");
}
#else
void du_tcspmv_fp16_v2(indT *chunkPtr, std::vector<int> fragPtr, std::vector<uint64_t> fragBit, std::vector<half> tcVal,
                       indT *sparse_AToX_index, half *X_val, half *Y_val, int rowA, int colA, int *, double *tcTime) {
    check(mx_du_tcspmv(kDtype, chunkPtr, fragPtr.data(), fragBit.data(), tcVal.data(), (int)tcVal.size(),
                       sparse_AToX_index, X_val, Y_val, rowA, colA, kWarm, kIters, tcTime),
          "du_tcspmv_fp16_v2");
}
void se_tcspmv_fp16(valT *csrValA, indT *csrRowPtrA, int *csrColIdxA, valT *X_val, valT *Y_val, int *order_rid,
                    int rowA, int colA, indT nnzA, int NUM, double threshold, int block_longest, double *tcTime) {
    check(mx_se_tcspmv(kDtype, csrValA, csrRowPtrA, csrColIdxA, X_val, Y_val, order_rid, rowA, colA, nnzA, NUM,
                       threshold, block_longest, kWarm, kIters, tcTime),
          "se_tcspmv_fp16");
}
// The 8x4 / 32-bit-bitmap format of the reference's older FP16 kernels: unpacked to CSR on the host and run through the
// same device path as se_tcspmv_fp16 (the format is superseded by v2; the symbols are kept for source compatibility).
static void du_fp16_8x4(int *chunkPtr, const std::vector<int> &fragPtr, const std::vector<uint32_t> &fragBit,
                        const std::vector<half> &tcVal, int *AToX, half *X_val, half *Y_val, int rowA, int colA,
                        double *tcTime) {
    const int K = 4, chunkNum = (rowA + 7) / 8;
    std::vector<std::vector<std::pair<int, half>>> rows(rowA);
    for (int p = 0; p < chunkNum; ++p)
        for (int f = chunkPtr[p]; f < chunkPtr[p + 1]; ++f) {
            int vi = fragPtr[f];
            for (int m = 0; m < 8; ++m)
                for (int k = 0; k < K; ++k)
                    if ((fragBit[f] >> (m * K + k)) & 1u) {
                        int r = p * 8 + m;
                        if (r < rowA) rows[r].push_back({AToX[f * K + k], tcVal[vi]});
                        ++vi;
                    }
        }
    std::vector<int> ptr(rowA + 1, 0), ind;
    std::vector<half> val;
    for (int r = 0; r < rowA; ++r) {
        for (auto &e : rows[r]) {
            ind.push_back(e.first);
            val.push_back(e.second);
        }
        ptr[r + 1] = (int)ind.size();
    }
    std::vector<int> order(rowA);
    std::vector<half> sorted(rowA);
    check(mx_se_tcspmv(MX_FP16, val.data(), ptr.data(), ind.data(), X_val, sorted.data(), order.data(), rowA, colA,
                       (int)ind.size(), 4, 0.75, 256, kWarm, kIters, tcTime),
          "du_tcspmv_fp16_v0/v1");
    for (int i = 0; i < rowA; ++i) Y_val[order[i]] = sorted[i];  // results leave in the layout's row order
}
void du_tcspmv_fp16_v0(int *chunkPtr, std::vector<int> fragPtr, std::vector<uint32_t> fragBit, std::vector<half> tcVal,
                       int *sparse_AToX_index, half *X_val, half *Y_val, int rowA, int colA, int *, double *tcTime) {
    du_fp16_8x4(chunkPtr, fragPtr, fragBit, tcVal, sparse_AToX_index, X_val, Y_val, rowA, colA, tcTime);
}
void du_tcspmv_fp16_v1(int *chunkPtr, std::vector<int> fragPtr, std::vector<uint32_t> fragBit, std::vector<half> tcVal,
                       int *sparse_AToX_index, half *X_val, half *Y_val, int rowA, int colA, int *, double *tcTime) {
    du_fp16_8x4(chunkPtr, fragPtr, fragBit, tcVal, sparse_AToX_index, X_val, Y_val, rowA, colA, tcTime);
}
#endif
