// Glue that lets the test-suite call the REFERENCE's own host pipeline (compiled unmodified from the
// reference sources by oracle/Makefile into oracle/_ref/) without a GPU.
//
// TEST INFRASTRUCTURE ONLY — never linked into the shipped library.
//
// What is the reference's and what is not:
//   * test/test_autotc_spmv.cpp is compiled as-is with -Dmain=matxtract_reference_main.  Its main()
//     (argv parsing, ranking, tau cuts, D/S split, dd/ds split, ecrPreprocess_opt1, chunkPtr/AToX glue,
//     generateFormat_opt[_fp16], merge2CSR_opt, spmv_serial, eQcheck) therefore runs exactly as shipped.
//     utilities/mmio.cpp is compiled as-is too (Matrix Market input).
//   * The five functions main() calls into the GPU side (csr2csc, csc2csr, cdspmv, du_tcspmv_*,
//     se_tcspmv_*; declared in include/MatXtract.h and include/csr2csc.h) are defined HERE as CPU
//     stand-ins that (a) record every array main() passes them — i.e. the complete partition the
//     reference built — and (b) return a serial CPU result so that main()'s own eQcheck still runs.
//     The transposes are stable (ascending minor index); cuSPARSE's order is not pinned by any
//     reference test.
// Build with -Dfp64 for the FP64 variant, without for FP16 (same switch as the reference's CMake).
#include "mmio.h"
#include "csr2csc.h"
#include "MatXtract.h"

#include <map>
#include <string>
#include <vector>

// ---- functions defined in the reference TU (declared here, bodies are the reference's) ----
int matxtract_reference_main(int argc, char **argv);
void spmv_serial(valT *csrVal, indT *csrRowPtr, indT *csrColInd, valT *X_val, valT *Y_val, int rowA, int colA,
                 indT nnzA);
int eQcheck(valT *tmp1, valT *tmp2, int length);
void ecrPreprocess_opt1(int *csrColInd, int *csrRowPtr, int rowA, int colA, int fragSize_h, int fragSize_w,
                        int *blockPartition, int *ecrId, int **use_x_id, int *nec_num);
#ifdef fp64
typedef uint32_t bitT;
void generateFormat_opt(const valT *vals, const int *rowPtr, const int *ecrId, int dRows, int dCols, int *chunkPtr,
                        std::vector<int> &fragPtr, std::vector<uint32_t> &fragBit, std::vector<valT> &tcVal);
void tcspmv_serial(const valT *x_d, valT *y_d, const int *chunkPtr, const std::vector<int> &fragPtr,
                   const std::vector<uint32_t> &fragBit, const std::vector<valT> &tcVal, const int *sparse_AToX_index,
                   int dRows, int dCols, int fragM, int fragK);
#else
typedef uint64_t bitT;
void generateFormat_opt_fp16(const valT *vals, const int *rowPtr, const int *ecrId, int dRows, int dCols,
                             int *chunkPtr, std::vector<int> &fragPtr, std::vector<uint64_t> &fragBit,
                             std::vector<valT> &tcVal);
#endif
void merge2CSR_opt(int rowA, int sCols, int nnzColS, const valT *csrVal_S, const int *csrRowPtr_S,
                   const int *csrColInd_S, int sRows, int dCols, int nnzRowS, const valT *csrVal_D,
                   const int *csrRowPtr_D, const int *csrColInd_D, const int *newArray, const valT *x_d,
                   const valT *x_s, valT *&csrVal_CD, int *&csrRowPtr_CD, int *&csrColInd_CD, valT *&x_CD);

namespace {
std::map<std::string, std::vector<int>> g_ints;
std::map<std::string, std::vector<unsigned char>> g_bytes;

void put_i(const char *k, const int *p, size_t n) { g_ints[k].assign(p, p + n); }
void put_b(const char *k, const void *p, size_t nbytes) {
    g_bytes[k].assign((const unsigned char *)p, (const unsigned char *)p + nbytes);
}

void transpose_stable(int n_in, int n_out, int nnz, const int *ptr, const int *ind, const valT *val, valT **oval,
                      int **optr, int **oind) {
    int *p = (int *)calloc(n_out + 1, sizeof(int));
    int *oi = (int *)malloc(sizeof(int) * (nnz > 0 ? nnz : 1));
    valT *ov = (valT *)malloc(sizeof(valT) * (nnz > 0 ? nnz : 1));
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
int g_csc2csr_calls = 0;
}  // namespace

// ---- CPU stand-ins for the reference's GPU-side API ----
void csr2csc(valT *csrVal, indT *csrRowPtr, indT *csrColInd, int rowA, int colA, indT nnzA, valT **cscVal,
             indT **cscColPtr, indT **cscRowInd) {
    transpose_stable(rowA, colA, nnzA, csrRowPtr, csrColInd, csrVal, cscVal, cscColPtr, cscRowInd);
    g_csc2csr_calls = 0;
}
void csc2csr(valT *cscVal, indT *cscColPtr, indT *cscRowInd, int rowA, int colA, indT nnzA, valT **csrVal,
             indT **csrRowPtr, indT **csrColInd) {
    transpose_stable(colA, rowA, nnzA, cscColPtr, cscRowInd, cscVal, csrVal, csrRowPtr, csrColInd);
    // first call = D part (colA = dCols), second = S part (test_autotc_spmv.cpp:1234-1238)
    const char *tag = g_csc2csr_calls++ == 0 ? "d" : "s";
    put_i((std::string(tag) + "csrRowPtr").c_str(), *csrRowPtr, rowA + 1);
    put_i((std::string(tag) + "csrColInd").c_str(), *csrColInd, nnzA);
    int dims[3] = {rowA, colA, nnzA};
    put_i((std::string(tag) + "csr_dims").c_str(), dims, 3);
}
void cdspmv(valT *csrVal, indT *csrRowPtr, indT *csrColInd, valT *X_val, valT *Y_val, int rowA, int colA, indT nnzA,
            double *cdTime, double *cdPre) {
    put_i("rowPtr_CD", csrRowPtr, rowA + 1);
    put_i("colInd_CD", csrColInd, nnzA);
    put_b("val_CD", csrVal, sizeof(valT) * nnzA);
    put_b("x_CD", X_val, sizeof(valT) * colA);
    put_b("y_before_cd", Y_val, sizeof(valT) * rowA);
    int dims[3] = {rowA, colA, nnzA};
    put_i("cd_dims", dims, 3);
    spmv_serial(csrVal, csrRowPtr, csrColInd, X_val, Y_val, rowA, colA, nnzA);  // Y_val is in/out
    put_b("y_final", Y_val, sizeof(valT) * rowA);
    *cdTime = 1.0;
    *cdPre = 0.0;
}
static void capture_du(indT *chunkPtr, std::vector<int> &fragPtr, std::vector<bitT> &fragBit, std::vector<valT> &tcVal,
                       indT *AToX, valT *X_val, valT *Y_val, int rowA, int colA, int *row_order) {
    int chunkNum = (rowA + fragM - 1) / fragM;
    put_i("chunkPtr", chunkPtr, chunkNum + 1);
    put_i("fragPtr", fragPtr.data(), fragPtr.size());
    put_b("fragBit", fragBit.data(), fragBit.size() * sizeof(bitT));
    put_b("tcVal", tcVal.data(), tcVal.size() * sizeof(valT));
    put_i("AToX", AToX, (size_t)chunkPtr[chunkNum] * fragK);
    put_b("x_d", X_val, sizeof(valT) * colA);
    put_i("rId", row_order, rowA);
    int dims[2] = {rowA, colA};
    put_i("du_dims", dims, 2);
    for (int i = 0; i < rowA; ++i) Y_val[i] = static_cast<valT>(0.0);
    for (int p = 0; p < chunkNum; ++p)
        for (int f = chunkPtr[p]; f < chunkPtr[p + 1]; ++f) {
            int vi = 0;
            for (int m = 0; m < fragM; ++m)
                for (int k = 0; k < fragK; ++k)
                    if ((fragBit[f] >> (m * fragK + k)) & 1) {
                        int row = p * fragM + m;
                        if (row < rowA) Y_val[row] = Y_val[row] + tcVal[fragPtr[f] + vi] * X_val[AToX[f * fragK + k]];
                        vi++;
                    }
        }
}
static void capture_se(valT *csrValA, indT *csrRowPtrA, int *csrColIdxA, valT *X_val, valT *Y_val, int *order_rid,
                       int rowA, int colA, indT nnzA) {
    put_i("rowPtr_dd", csrRowPtrA, rowA + 1);
    put_i("colInd_dd", csrColIdxA, nnzA);
    put_b("val_dd", csrValA, sizeof(valT) * nnzA);
    put_b("x_d", X_val, sizeof(valT) * colA);
    int dims[3] = {rowA, colA, nnzA};
    put_i("se_dims", dims, 3);
    for (int i = 0; i < rowA; ++i) {
        order_rid[i] = i;
        Y_val[i] = static_cast<valT>(0.0);
    }
    spmv_serial(csrValA, csrRowPtrA, csrColIdxA, X_val, Y_val, rowA, colA, nnzA);
}
#ifdef fp64
void du_tcspmv_fp64(indT *chunkPtr, std::vector<int> fragPtr, std::vector<uint32_t> fragBit, std::vector<double> tcVal,
                    indT *sparse_AToX_index, valT *X_val, valT *Y_val, int rowA, int colA, int *row_order,
                    double *tcTime) {
    capture_du(chunkPtr, fragPtr, fragBit, tcVal, sparse_AToX_index, X_val, Y_val, rowA, colA, row_order);
    *tcTime = 1.0;
}
void se_tcspmv_fp64(valT *csrValA, indT *csrRowPtrA, int *csrColIdxA, valT *X_val, valT *Y_val, int *order_rid,
                    int rowA, int colA, indT nnzA, int, double, int, double *tcTime) {
    capture_se(csrValA, csrRowPtrA, csrColIdxA, X_val, Y_val, order_rid, rowA, colA, nnzA);
    *tcTime = 1.0;
}
#else
void du_tcspmv_fp16_v2(indT *chunkPtr, std::vector<int> fragPtr, std::vector<uint64_t> fragBit, std::vector<half> tcVal,
                       indT *sparse_AToX_index, half *X_val, half *Y_val, int rowA, int colA, int *row_order,
                       double *tcTime) {
    capture_du(chunkPtr, fragPtr, fragBit, tcVal, sparse_AToX_index, X_val, Y_val, rowA, colA, row_order);
    *tcTime = 1.0;
}
void se_tcspmv_fp16(valT *csrValA, indT *csrRowPtrA, int *csrColIdxA, valT *X_val, valT *Y_val, int *order_rid,
                    int rowA, int colA, indT nnzA, int, double, int, double *tcTime) {
    capture_se(csrValA, csrRowPtrA, csrColIdxA, X_val, Y_val, order_rid, rowA, colA, nnzA);
    *tcTime = 1.0;
}
#endif

extern "C" {

int ref_value_bytes() { return (int)sizeof(valT); }
int ref_frag_k() { return fragK; }

// Runs the reference's main() as `matxtract_perftest tau_c tau_r file` (or with the file only when
// tau_c is NULL) and leaves the captured arrays for ref_get_*.
int ref_run_main(const char *tau_c, const char *tau_r, const char *mtx) {
    g_ints.clear();
    g_bytes.clear();
    std::vector<std::string> a = {"matxtract_perftest"};
    if (tau_c) {
        a.push_back(tau_c);
        a.push_back(tau_r);
    }
    a.push_back(mtx);
    std::vector<char *> argv;
    for (auto &s : a) argv.push_back(const_cast<char *>(s.c_str()));
    int rc = matxtract_reference_main((int)argv.size(), argv.data());
    fflush(stdout);
    return rc;
}
long ref_get_ints(const char *name, const int **p) {
    auto it = g_ints.find(name);
    if (it == g_ints.end()) return -1;
    *p = it->second.data();
    return (long)it->second.size();
}
long ref_get_bytes(const char *name, const unsigned char **p) {
    auto it = g_bytes.find(name);
    if (it == g_bytes.end()) return -1;
    *p = it->second.data();
    return (long)it->second.size();
}

// Matrix Market -> CSR through the reference's reader.  Arrays are malloc'd by the reader; copy them
// out with ref_get_* ("mm_rowPtr", "mm_colInd", "mm_val").
int ref_read_mtx(const char *path, int *m, int *n, int *nnz) {
    int sym;
    indT *rp, *ci;
    valT *v;
    int rc = mmio_allinone(m, n, nnz, &sym, &rp, &ci, &v, const_cast<char *>(path));
    if (rc != 0) return rc;
    put_i("mm_rowPtr", rp, *m + 1);
    put_i("mm_colInd", ci, *nnz);
    put_b("mm_val", v, sizeof(valT) * *nnz);
    free(rp);
    free(ci);
    free(v);
    return 0;
}

void ref_spmv_serial(void *val, int *ptr, int *ind, void *x, void *y, int rowA, int colA, int nnzA) {
    spmv_serial((valT *)val, ptr, ind, (valT *)x, (valT *)y, rowA, colA, nnzA);
}
int ref_eqcheck(void *a, void *b, int n) {
    int rc = eQcheck((valT *)a, (valT *)b, n);
    fflush(stdout);
    return rc;
}

// The reference's tile-format builders applied to a dd block given as CSR (rows in hot-rank order,
// column ids = density ranks): ecrPreprocess_opt1, then the chunkPtr / sparse_AToX_index glue of
// main() (test_autotc_spmv.cpp:1369-1404, the only lines restated here), then generateFormat_opt[_fp16].
int ref_build_tiles(void *val_dd, int *rowPtr_dd, int *colInd_dd, int dRows, int dCols) {
    int nnzRowD = rowPtr_dd[dRows];
    int chunkNum = (dRows + fragM - 1) / fragM;
    std::vector<int> ecrId(nnzRowD > 0 ? nnzRowD : 1, 0), blockPartition(chunkNum + 1, 0), nec_num(chunkNum + 1, 0);
    std::vector<int *> use_x_id(chunkNum + 1, nullptr);
    ecrPreprocess_opt1(colInd_dd, rowPtr_dd, dRows, dCols, fragM, fragK, blockPartition.data(), ecrId.data(),
                       use_x_id.data(), nec_num.data());
    std::vector<int> chunkPtr(chunkNum + 1, 0);
    for (int i = 1; i <= chunkNum; i++) chunkPtr[i] = chunkPtr[i - 1] + blockPartition[i - 1];
    int totalTcFrags = chunkPtr[chunkNum];
    std::vector<int> AToX((size_t)totalTcFrags * fragK, 0);
    for (int p = 0; p < chunkNum; ++p)
        if (use_x_id[p]) {
            memcpy(AToX.data() + (size_t)chunkPtr[p] * fragK, use_x_id[p], nec_num[p] * sizeof(int));
            free(use_x_id[p]);
        }
    std::vector<int> fragPtr;
    std::vector<bitT> fragBit;
    std::vector<valT> tcVal;
#ifdef fp64
    generateFormat_opt((valT *)val_dd, rowPtr_dd, ecrId.data(), dRows, dCols, chunkPtr.data(), fragPtr, fragBit, tcVal);
#else
    generateFormat_opt_fp16((valT *)val_dd, rowPtr_dd, ecrId.data(), dRows, dCols, chunkPtr.data(), fragPtr, fragBit,
                            tcVal);
#endif
    put_i("chunkPtr", chunkPtr.data(), chunkPtr.size());
    put_i("AToX", AToX.data(), AToX.size());
    put_i("fragPtr", fragPtr.data(), fragPtr.size());
    put_b("fragBit", fragBit.data(), fragBit.size() * sizeof(bitT));
    put_b("tcVal", tcVal.data(), tcVal.size() * sizeof(valT));
    put_i("ecrId", ecrId.data(), nnzRowD);
    return 0;
}

#ifdef fp64
// The reference's serial statement of the fragment format (32-bit bitmaps only).
void ref_tcspmv_serial(double *x_d, double *y_d, int *chunkPtr, int *fragPtr, int nfrag, uint32_t *fragBit,
                       double *tcVal, int nval, int *AToX, int dRows, int dCols) {
    std::vector<int> fp(fragPtr, fragPtr + nfrag + 1);
    std::vector<uint32_t> fb(fragBit, fragBit + nfrag);
    std::vector<double> tv(tcVal, tcVal + nval);
    tcspmv_serial(x_d, y_d, chunkPtr, fp, fb, tv, AToX, dRows, dCols, fragM, fragK);
}
#endif

}  // extern "C"
