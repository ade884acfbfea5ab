// Matrix Market coordinate files -> host CSR, in parallel.
//
// Same result as the reference's reader (utilities/mmio.cpp:1547-1713, mm_read_banner :246-414): real / complex (real
// part) / integer / pattern (value 1) entries, 1-based indices; for `symmetric` and `hermitian` storage every
// off-diagonal entry is also stored transposed (`skew-symmetric` is NOT mirrored, as in the reference, whose test looks
// at the 'S' code only); rows are filled in file order, the mirrored copy of entry i directly after entry i; values go
// double -> valT in one rounding.  The reference parses with one fscanf per entry on one core, which dominates the wall
// time of its driver for real matrices; here the file is mapped, cut at line ends into one piece per thread, each
// piece is parsed with a hand-written number scanner, and the CSR is filled by threads that each own a range of rows
// (every thread walks the entry list in file order and keeps the entries of its rows, so the order inside a row is
// the file order without any sort).
#include <cctype>
#include <cerrno>
#include <charconv>
#include <climits>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <algorithm>
#include <string>
#include <vector>

#include <fcntl.h>
#include <omp.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cuda_fp16.h>

#include "mx_capi.h"

namespace {

struct Mapped {
    const char *p = nullptr;
    size_t n = 0;
    int fd = -1;
    bool is_map = false;
    std::vector<char> buf;
    ~Mapped() {
        if (is_map && p) munmap(const_cast<char *>(p), n);
        if (fd >= 0) close(fd);
    }
    bool open_file(const char *path) {
        fd = ::open(path, O_RDONLY);
        if (fd < 0) return false;
        struct stat st;
        if (fstat(fd, &st) != 0) return false;
        n = (size_t)st.st_size;
        if (n == 0) return true;
        void *m = mmap(nullptr, n, PROT_READ, MAP_PRIVATE, fd, 0);
        if (m != MAP_FAILED) {
            p = (const char *)m;
            is_map = true;
            madvise(m, n, MADV_SEQUENTIAL);
            return true;
        }
        buf.resize(n);  // e.g. a pipe: read it
        size_t got = 0;
        while (got < n) {
            ssize_t r = ::read(fd, buf.data() + got, n - got);
            if (r <= 0) break;
            got += (size_t)r;
        }
        n = got;
        p = buf.data();
        return true;
    }
};

inline bool is_space(char c) { return c == ' ' || c == '\t' || c == '\r' || c == '\n' || c == '\v' || c == '\f'; }

// scanf("%d")-like: optional sign, digits.  Returns the position after the number, or nullptr.
inline const char *scan_int(const char *s, const char *e, long long &out) {
    while (s < e && is_space(*s)) ++s;
    if (s >= e) return nullptr;
    bool neg = false;
    if (*s == '-' || *s == '+') {
        neg = *s == '-';
        ++s;
    }
    if (s >= e || *s < '0' || *s > '9') return nullptr;
    long long v = 0;
    while (s < e && *s >= '0' && *s <= '9') {
        v = v * 10 + (*s - '0');
        ++s;
    }
    out = neg ? -v : v;
    return s;
}

// scanf("%lg")-like
inline const char *scan_double(const char *s, const char *e, double &out) {
    while (s < e && is_space(*s)) ++s;
    if (s >= e) return nullptr;
    if (*s == '+') ++s;
    auto r = std::from_chars(s, e, out);
    if (r.ec == std::errc()) return r.ptr;
    if (r.ec == std::errc::result_out_of_range) {  // as strtod: +-HUGE_VAL or 0
        char tmp[64];
        size_t k = 0;
        while (s + k < e && !is_space(s[k]) && k < sizeof tmp - 1) {
            tmp[k] = s[k];
            ++k;
        }
        tmp[k] = 0;
        char *endp = nullptr;
        out = strtod(tmp, &endp);
        return endp != tmp ? s + (endp - tmp) : nullptr;
    }
    return nullptr;
}

enum Field { F_REAL, F_COMPLEX, F_INTEGER, F_PATTERN };

struct Entry {
    int r, c;
    double v;
};

// one entry starting at s; returns the position after it or nullptr
inline const char *scan_entry(const char *s, const char *e, Field field, Entry &out) {
    long long r, c;
    if (!(s = scan_int(s, e, r))) return nullptr;
    if (!(s = scan_int(s, e, c))) return nullptr;
    out.r = (int)(r - 1);
    out.c = (int)(c - 1);
    out.v = 1.0;
    if (field == F_REAL) {
        if (!(s = scan_double(s, e, out.v))) return nullptr;
    } else if (field == F_COMPLEX) {
        double im;
        if (!(s = scan_double(s, e, out.v))) return nullptr;
        if (!(s = scan_double(s, e, im))) return nullptr;
    } else if (field == F_INTEGER) {
        long long iv;
        if (!(s = scan_int(s, e, iv))) return nullptr;
        out.v = (double)(int)iv;
    }
    return s;
}

inline void lower(std::string &s) {
    for (auto &ch : s) ch = (char)tolower((unsigned char)ch);
}

template <typename V>
inline V to_val(double v);
template <>
inline double to_val<double>(double v) {
    return v;
}
template <>
inline __half to_val<__half>(double v) {
    return __double2half(v);
}

template <typename V>
int build_csr(const std::vector<int> &ri, const std::vector<int> &ci, const std::vector<double> &va, int rows,
              bool mirror, int threads, int **row_ptr, int **col_ind, void **val, int *nnz_out) {
    const long long E = (long long)ri.size();
    std::vector<long long> start((size_t)rows + 1, 0);
    {
        std::vector<int> cnt((size_t)rows, 0);
#pragma omp parallel for num_threads(threads) schedule(static)
        for (long long e = 0; e < E; ++e) {
#pragma omp atomic
            cnt[ri[e]]++;
            if (mirror && ri[e] != ci[e]) {
#pragma omp atomic
                cnt[ci[e]]++;
            }
        }
        long long total = 0;
        for (int r = 0; r < rows; ++r) {
            start[r] = total;
            total += cnt[r];
        }
        start[rows] = total;
    }
    const long long total = start[rows];
    if (total > INT_MAX) return -5;
    int *rp = (int *)malloc(sizeof(int) * ((size_t)rows + 1));
    int *cx = (int *)malloc(sizeof(int) * (size_t)(total > 0 ? total : 1));
    V *vx = (V *)malloc(sizeof(V) * (size_t)(total > 0 ? total : 1));
    if (!rp || !cx || !vx) {
        free(rp);
        free(cx);
        free(vx);
        return -5;
    }
    for (int r = 0; r <= rows; ++r) rp[r] = (int)start[r];
    // thread t owns the rows [lo_t, hi_t) that hold about 1/threads of the stored entries
    std::vector<int> bound((size_t)threads + 1, rows);
    bound[0] = 0;
    for (int t = 1; t < threads; ++t) {
        const long long want = total * t / threads;
        bound[t] = (int)(std::lower_bound(start.begin(), start.end(), want) - start.begin());
        if (bound[t] > rows) bound[t] = rows;
        if (bound[t] < bound[t - 1]) bound[t] = bound[t - 1];
    }
#pragma omp parallel for num_threads(threads) schedule(static, 1)
    for (int t = 0; t < threads; ++t) {  // a loop over the ranges: complete even if the team is smaller than asked
        const int lo = bound[t], hi = bound[t + 1];
        if (lo < hi) {
            std::vector<long long> cur(start.begin() + lo, start.begin() + hi);
            for (long long e = 0; e < E; ++e) {
                const int r = ri[e], c = ci[e];
                if (r >= lo && r < hi) {
                    const long long q = cur[r - lo]++;
                    cx[q] = c;
                    vx[q] = to_val<V>(va[e]);
                }
                if (mirror && r != c && c >= lo && c < hi) {
                    const long long q = cur[c - lo]++;
                    cx[q] = r;
                    vx[q] = to_val<V>(va[e]);
                }
            }
        }
    }
    *row_ptr = rp;
    *col_ind = cx;
    *val = vx;
    *nnz_out = (int)total;
    return 0;
}

}  // namespace

extern "C" void mx_host_free(void *p) { free(p); }

extern "C" int mx_read_matrix_market(const char *path, int dtype, int threads, int *rows_out, int *cols_out,
                                     int *nnz_out, int *is_symmetric, int **row_ptr, int **col_ind, void **val) {
    if (!path || !rows_out || !cols_out || !nnz_out || !row_ptr || !col_ind || !val ||
        (dtype != MX_FP64 && dtype != MX_FP16))
        return -3;
    Mapped F;
    if (!F.open_file(path)) return -1;
    const char *p = F.p, *end = F.p + F.n;
    // ---- banner: "%%MatrixMarket matrix coordinate <field> <symmetry>" ----
    const char *eol = p ? (const char *)memchr(p, '\n', F.n) : nullptr;
    if (!eol) {
        printf("Could not process Matrix Market banner.\n");
        return -2;
    }
    std::string tok[5];
    {
        const char *s = p;
        for (int k = 0; k < 5; ++k) {
            while (s < eol && is_space(*s)) ++s;
            const char *b = s;
            while (s < eol && !is_space(*s)) ++s;
            tok[k].assign(b, s);
        }
    }
    for (int k = 1; k < 5; ++k) lower(tok[k]);
    Field field;
    if (tok[4].empty() || tok[0].rfind("%%MatrixMarket", 0) != 0 || tok[1] != "matrix" || tok[2] != "coordinate") {
        printf("Could not process Matrix Market banner.\n");
        return -2;
    }
    if (tok[3] == "real")
        field = F_REAL;
    else if (tok[3] == "complex")
        field = F_COMPLEX;
    else if (tok[3] == "integer")
        field = F_INTEGER;
    else if (tok[3] == "pattern")
        field = F_PATTERN;
    else {
        printf("Could not process Matrix Market banner.\n");
        return -2;
    }
    if (tok[4] != "general" && tok[4] != "symmetric" && tok[4] != "hermitian" && tok[4] != "skew-symmetric") {
        printf("Could not process Matrix Market banner.\n");
        return -2;
    }
    const bool mirror = tok[4] == "symmetric" || tok[4] == "hermitian";
    // ---- comments, then the size line ----
    const char *s = eol + 1;
    long long rows = 0, cols = 0, entries = 0;
    for (;;) {
        if (s >= end) return -4;
        const char *le = (const char *)memchr(s, '\n', (size_t)(end - s));
        const char *next = le ? le + 1 : end;
        if (*s == '%') {
            s = next;
            continue;
        }
        const char *q = s, *lim = le ? le : end;
        if ((q = scan_int(q, lim, rows)) && (q = scan_int(q, lim, cols)) && (q = scan_int(q, lim, entries))) {
            s = next;
            break;
        }
        s = next;  // blank (or short) line before the sizes: keep looking, as the reference does
    }
    if (rows < 0 || cols < 0 || entries < 0 || rows > INT_MAX || cols > INT_MAX || entries > INT_MAX) return -4;
    if (threads <= 0) threads = omp_get_max_threads();
    threads = std::max(1, std::min(threads, 256));
    // ---- body: one piece per thread, cut at line ends; a piece's entries are its non-blank lines ----
    const char *body = s;
    const size_t blen = (size_t)(end - body);
    const int pieces = (int)std::max<size_t>(1, std::min<size_t>((size_t)threads, blen / (1 << 16) + 1));
    std::vector<const char *> cut((size_t)pieces + 1, end);
    cut[0] = body;
    for (int k = 1; k < pieces; ++k) {
        const char *c = body + blen * (size_t)k / (size_t)pieces;
        if (c < cut[k - 1]) c = cut[k - 1];
        const char *nl = c < end ? (const char *)memchr(c, '\n', (size_t)(end - c)) : nullptr;
        cut[k] = nl ? nl + 1 : end;
    }
    std::vector<long long> first((size_t)pieces + 1, 0);
#pragma omp parallel for num_threads(threads) schedule(static, 1)
    for (int k = 0; k < pieces; ++k) {
        long long lines = 0;
        const char *a = cut[k], *b = cut[k + 1];
        while (a < b) {
            const char *le = (const char *)memchr(a, '\n', (size_t)(b - a));
            const char *lim = le ? le : b;
            const char *q = a;
            while (q < lim && is_space(*q)) ++q;
            if (q < lim) ++lines;
            a = le ? le + 1 : b;
        }
        first[(size_t)k + 1] = lines;
    }
    for (int k = 0; k < pieces; ++k) first[(size_t)k + 1] += first[k];
    if (first[pieces] < entries) return -4;  // fewer entry lines than announced (the reference reads past the end here)
    std::vector<int> ri((size_t)entries), ci((size_t)entries);
    std::vector<double> va((size_t)entries);
    int bad = 0;
#pragma omp parallel for num_threads(threads) schedule(static, 1) reduction(| : bad)
    for (int k = 0; k < pieces; ++k) {
        long long idx = first[k];
        const char *a = cut[k], *b = cut[k + 1];
        while (a < b && idx < entries) {  // lines after the announced count are ignored, like the reference
            const char *le = (const char *)memchr(a, '\n', (size_t)(b - a));
            const char *lim = le ? le : b;
            const char *q = a;
            while (q < lim && is_space(*q)) ++q;
            if (q < lim) {
                Entry en;
                if (!scan_entry(q, lim, field, en) || en.r < 0 || en.r >= rows || en.c < 0 || en.c >= cols ||
                    (mirror && en.c >= rows)) {
                    bad = 1;
                } else {
                    ri[(size_t)idx] = en.r;
                    ci[(size_t)idx] = en.c;
                    va[(size_t)idx] = en.v;
                }
                ++idx;
            }
            a = le ? le + 1 : b;
        }
    }
    if (bad) return -4;  // an entry line that does not parse or lies outside the announced shape
    int st;
    if (dtype == MX_FP64)
        st = build_csr<double>(ri, ci, va, (int)rows, mirror, threads, row_ptr, col_ind, val, nnz_out);
    else
        st = build_csr<__half>(ri, ci, va, (int)rows, mirror, threads, row_ptr, col_ind, val, nnz_out);
    if (st != 0) return st;
    *rows_out = (int)rows;
    *cols_out = (int)cols;
    if (is_symmetric) *is_symmetric = mirror ? 1 : 0;
    return 0;
}
