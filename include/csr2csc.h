// CSR <-> CSC conversion with the reference's signatures (include/csr2csc.h); the outputs are malloc'd host arrays
// the caller frees.  Entries keep ascending minor index inside each output row/column (stable transpose).
// The extraction in this library (mx_partition) needs no transposes; these exist for callers of the old API.
#pragma once
#include "common.h"

void csr2csc(valT *csrVal, indT *csrRowPtr, indT *csrColInd, int rowA, int colA, indT nnzA, valT **cscVal,
             indT **cscColPtr, indT **cscRowInd);
void csc2csr(valT *cscVal, indT *cscColPtr, indT *cscRowInd, int rowA, int colA, indT nnzA, valT **csrVal,
             indT **csrRowPtr, indT **csrColInd);
