// Matrix Market coordinate reader with the reference's entry point (utilities/mmio.cpp:1547-1713): real / integer /
// pattern / complex (real part) values, general, symmetric, skew-symmetric or hermitian storage (mirrored entries are
// added for every off-diagonal entry), 1-based indices, CSR rows filled in file order.
#include <cctype>
#include <cstring>
#include <string>

#include "mmio.h"

int mmio_allinone(int *m, int *n, indT *nnz, int *isSymmetric, indT **csrRowPtr, indT **csrColIdx, valT **csrVal,
                  char *filename) {
    FILE *f = fopen(filename, "r");
    if (!f) return -1;
    char line[1100];
    if (!fgets(line, sizeof line, f)) {
        fclose(f);
        return -2;
    }
    std::string banner(line);
    for (auto &ch : banner) ch = (char)tolower(ch);
    if (banner.rfind("%%matrixmarket", 0) != 0 || banner.find("matrix") == std::string::npos ||
        banner.find("coordinate") == std::string::npos) {
        printf("Could not process Matrix Market banner.\n");
        fclose(f);
        return -2;
    }
    const bool pattern = banner.find("pattern") != std::string::npos;
    const bool complex_ = banner.find("complex") != std::string::npos;
    const bool sym = banner.find("symmetric") != std::string::npos || banner.find("hermitian") != std::string::npos;
    do {
        if (!fgets(line, sizeof line, f)) {
            fclose(f);
            return -4;
        }
    } while (line[0] == '%' || line[0] == '\n');
    int rows = 0, cols = 0;
    long long entries = 0;
    if (sscanf(line, "%d %d %lld", &rows, &cols, &entries) != 3) {
        fclose(f);
        return -4;
    }
    std::vector<int> ri(entries), ci(entries);
    std::vector<double> va(entries);
    std::vector<int> count(rows + 1, 0);
    for (long long e = 0; e < entries; ++e) {
        double re = 1.0, im = 0.0;
        int r, c;
        int got = pattern ? fscanf(f, "%d %d", &r, &c)
                          : (complex_ ? fscanf(f, "%d %d %lg %lg", &r, &c, &re, &im) : fscanf(f, "%d %d %lg", &r, &c, &re));
        if (got < 2) {
            fclose(f);
            return -4;
        }
        ri[e] = r - 1;
        ci[e] = c - 1;
        va[e] = re;
        count[ri[e]]++;
        if (sym && ri[e] != ci[e]) count[ci[e]]++;
    }
    fclose(f);
    long long total = 0;
    std::vector<long long> start(rows + 1, 0);
    for (int r = 0; r < rows; ++r) {
        start[r] = total;
        total += count[r];
    }
    start[rows] = total;
    if (total > 2147483647LL) return -5;
    indT *rp = (indT *)malloc(sizeof(indT) * ((size_t)rows + 1));
    indT *cx = (indT *)malloc(sizeof(indT) * (size_t)(total > 0 ? total : 1));
    valT *vx = (valT *)malloc(sizeof(valT) * (size_t)(total > 0 ? total : 1));
    for (int r = 0; r <= rows; ++r) rp[r] = (indT)start[r];
    std::vector<long long> cur(start.begin(), start.end() - 1);
    for (long long e = 0; e < entries; ++e) {
        long long q = cur[ri[e]]++;
        cx[q] = ci[e];
        vx[q] = static_cast<valT>((float)va[e]);
        if (sym && ri[e] != ci[e]) {
            q = cur[ci[e]]++;
            cx[q] = ri[e];
            vx[q] = static_cast<valT>((float)va[e]);
        }
    }
    *m = rows;
    *n = cols;
    *nnz = (indT)total;
    *isSymmetric = sym ? 1 : 0;
    *csrRowPtr = rp;
    *csrColIdx = cx;
    *csrVal = vx;
    return 0;
}
