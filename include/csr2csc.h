// CSR <-> CSC conversion with the reference's signatures (include/csr2csc.h); the outputs are malloc'd host arrays
// the caller frees.  Entries keep ascending minor index inside each output row/column (stable transpose).
// The extraction in this library (mx_partition) needs no transposes; these exist for callers of the old API.
//
// Contract of both functions (what the reference's callers rely on, utilities/csr2csc.cpp:4-104 and :106-203):
//   * inputs are host arrays with 0-based indices; the pointer array has rowA + 1 (CSR) or colA + 1 (CSC) entries;
//   * the three outputs are allocated here with malloc and handed to the caller, who releases them with free();
//   * values move unchanged (no arithmetic); an empty matrix gives a pointer array of zeros;
//   * the reference runs cusparseCsr2cscEx2 on the device for this; here it is a counting transpose on the host, which
//     fixes the one thing cuSPARSE leaves open - the order of the entries inside an output row or column.
#pragma once
#include "common.h"

void csr2csc(valT *csrVal, indT *csrRowPtr, indT *csrColInd, int rowA, int colA, indT nnzA, valT **cscVal,
             indT **cscColPtr, indT **cscRowInd);
void csc2csr(valT *cscVal, indT *cscColPtr, indT *cscRowInd, int rowA, int colA, indT nnzA, valT **csrVal,
             indT **csrRowPtr, indT **csrColInd);
