// The reference's Matrix Market entry point (utilities/mmio.cpp:1547-1713) on top of the library's parallel reader:
// same arguments, same return codes, arrays owned by the caller (free()).
#include "mmio.h"
#include "mx_capi.h"

int mmio_allinone(int *m, int *n, indT *nnz, int *isSymmetric, indT **csrRowPtr, indT **csrColIdx, valT **csrVal,
                  char *filename) {
#ifdef fp64
    const int dtype = MX_FP64;
#else
    const int dtype = MX_FP16;
#endif
    int sym = 0;
    void *val = nullptr;
    const int st = mx_read_matrix_market(filename, dtype, 0, m, n, nnz, &sym, csrRowPtr, csrColIdx, &val);
    if (st != 0) return st;
    *isSymmetric = sym;
    *csrVal = static_cast<valT *>(val);
    return 0;
}
