// Matrix Market input with the reference's entry point (include/mmio.h, utilities/mmio.cpp:1547): coordinate files,
// real / integer / pattern, general or symmetric (expanded), rows in file order.  Arrays are malloc'd; the caller frees.
#pragma once
#include "common.h"

int mmio_allinone(int *m, int *n, indT *nnz, int *isSymmetric, indT **csrRowPtr, indT **csrColIdx, valT **csrVal,
                  char *filename);
