// Stored partitions: reader and validator (host code).  See partition_file.h.
#include "partition_file.h"

#include <cstdio>
#include <cstring>

#include "mx_capi.h"

namespace mx {
namespace {

struct FileCloser {
    FILE *f;
    ~FileCloser() {
        if (f) fclose(f);
    }
};

std::string at(const char *what, long long i) { return std::string(what) + " at index " + std::to_string(i); }

// p[0] == 0, non-decreasing, p[n] == total
std::string pointer_problem(const char *name, const int32_t *p, long long n, long long total) {
    if (p[0] != 0) return std::string(name) + "[0] != 0";
    long long bad = -1;
#pragma omp parallel for reduction(max : bad) schedule(static)
    for (long long i = 0; i < n; ++i)
        if (p[i + 1] < p[i]) bad = bad > i ? bad : i;
    if (bad >= 0) return at((std::string(name) + " decreases").c_str(), bad);
    if (p[n] != total) return std::string(name) + " does not end at its count";
    return "";
}

// every value in [0, bound)
std::string range_problem(const char *name, const int32_t *v, long long n, long long bound) {
    long long bad = -1;
#pragma omp parallel for reduction(max : bad) schedule(static)
    for (long long i = 0; i < n; ++i)
        if (v[i] < 0 || v[i] >= bound) bad = bad > i ? bad : i;
    if (bad >= 0) return at((std::string(name) + " out of range").c_str(), bad);
    return "";
}

// values in [0, bound) and pairwise distinct
std::string distinct_problem(const char *name, const int32_t *v, long long n, long long bound) {
    std::string r = range_problem(name, v, n, bound);
    if (!r.empty()) return r;
    std::vector<unsigned char> seen((size_t)bound, 0);
    for (long long i = 0; i < n; ++i) {
        if (seen[(size_t)v[i]]) return at((std::string(name) + " repeats a value").c_str(), i);
        seen[(size_t)v[i]] = 1;
    }
    return "";
}

}  // namespace

void part_array_bytes(const PartFileHeader &h, uint64_t out[PA_COUNT]) {
    const uint64_t vb = h.dtype == MX_FP64 ? 8 : 2, bb = h.dtype == MX_FP64 ? 4 : 8, K = (uint64_t)h.fragK;
    out[PA_XPERM] = 4ull * (uint64_t)h.n_cols;
    out[PA_RID] = 4ull * (uint64_t)h.dRows;
    out[PA_ROWPTR_DD] = 4ull * ((uint64_t)h.dRows + 1);
    out[PA_COLIND_DD] = 4ull * (uint64_t)h.nnzRowD;
    out[PA_VAL_DD] = vb * (uint64_t)h.nnzRowD;
    out[PA_CHUNKPTR] = 4ull * ((uint64_t)h.chunkNum + 1);
    out[PA_ATOX] = 4ull * (uint64_t)h.totalFrags * K;
    out[PA_FRAGPTR] = 4ull * ((uint64_t)h.totalFrags + 1);
    out[PA_FRAGBIT] = bb * (uint64_t)h.totalFrags;
    out[PA_TCVAL] = vb * (uint64_t)h.nnzRowD;
    out[PA_ROWPTR_CD] = 4ull * ((uint64_t)h.n_rows + 1);
    out[PA_COLIND_CD] = 4ull * (uint64_t)h.nnzCD;
    out[PA_VAL_CD] = vb * (uint64_t)h.nnzCD;
}

std::string part_header_problem(const PartFileHeader &h, int dtype) {
    if (memcmp(h.magic, kPartMagic, 8) != 0 || h.version != kPartVersion) return "not a stored partition of this version";
    if (h.dtype != MX_FP64 && h.dtype != MX_FP16) return "unknown value type";
    if (h.dtype != dtype) return "stored partition has the other value type";
    if (h.fragK != (h.dtype == MX_FP64 ? 4 : 8)) return "fragment width does not match the value type";
    const int32_t all[] = {h.n_rows, h.n_cols, h.nnz,   h.dCols,    h.nnzColD,    h.sCols, h.nnzColS, h.dRows,
                           h.nnzRowD, h.sRows, h.nnzRowS, h.chunkNum, h.totalFrags, h.nnzCD};
    for (int32_t v : all)
        if (v < 0) return "negative count in the header";
    if (h.dCols < 1 || h.dCols > h.n_cols || h.sCols != h.n_cols - h.dCols) return "column counts are inconsistent";
    if (h.dRows < 1 || h.dRows > h.n_rows || h.sRows != h.n_rows - h.dRows) return "row counts are inconsistent";
    if ((long long)h.nnzColD + h.nnzColS != h.nnz) return "nnzColD + nnzColS != nnz";
    if ((long long)h.nnzRowD + h.nnzRowS != h.nnzColD) return "nnzRowD + nnzRowS != nnzColD";
    if ((long long)h.nnzColS + h.nnzRowS != h.nnzCD) return "nnzCD != nnzColS + nnzRowS";
    if (h.chunkNum != (h.dRows + 7) / 8) return "chunkNum != ceil(dRows / 8)";
    if ((long long)h.totalFrags * h.fragK > 2147483647LL) return "fragment count exceeds int32";
    if ((long long)h.totalFrags * 8 * h.fragK < h.nnzRowD) return "fewer fragment slots than core-dense entries";
    return "";
}

std::string part_file_read(const char *path, int dtype, PartFile &out) {
    FileCloser fc{fopen(path, "rb")};
    if (!fc.f) return std::string("cannot open: ") + path;
    if (fread(&out.hd, sizeof out.hd, 1, fc.f) != 1) return "not a stored partition";
    std::string p = part_header_problem(out.hd, dtype);
    if (!p.empty()) return p;
    uint64_t want[PA_COUNT];
    part_array_bytes(out.hd, want);
    for (int a = 0; a < PA_COUNT; ++a) {
        uint64_t n = 0;
        if (fread(&n, sizeof n, 1, fc.f) != 1 || n != want[a]) return "array size does not match its header";
        out.arr[a].resize(n);
        if (n > 0 && fread(out.arr[a].data(), 1, n, fc.f) != n) return "truncated file";
    }
    return "";
}

std::string part_file_problem(const PartFile &f) {
    const PartFileHeader &h = f.hd;
    auto ints = [&](int a) { return reinterpret_cast<const int32_t *>(f.arr[a].data()); };
    std::string r;
    if (!(r = distinct_problem("xperm", ints(PA_XPERM), h.n_cols, h.n_cols)).empty()) return r;
    if (!(r = distinct_problem("rId", ints(PA_RID), h.dRows, h.n_rows)).empty()) return r;
    if (!(r = pointer_problem("rowPtr_dd", ints(PA_ROWPTR_DD), h.dRows, h.nnzRowD)).empty()) return r;
    if (!(r = range_problem("colInd_dd", ints(PA_COLIND_DD), h.nnzRowD, h.dCols)).empty()) return r;
    if (!(r = pointer_problem("chunkPtr", ints(PA_CHUNKPTR), h.chunkNum, h.totalFrags)).empty()) return r;
    if (!(r = range_problem("sparse_AToX_index", ints(PA_ATOX), (long long)h.totalFrags * h.fragK, h.dCols)).empty())
        return r;
    if (!(r = pointer_problem("fragPtr", ints(PA_FRAGPTR), h.totalFrags, h.nnzRowD)).empty()) return r;
    {
        const int32_t *fp = ints(PA_FRAGPTR);
        long long bad = -1;
        if (h.dtype == MX_FP64) {
            const uint32_t *b = reinterpret_cast<const uint32_t *>(f.arr[PA_FRAGBIT].data());
#pragma omp parallel for reduction(max : bad) schedule(static)
            for (long long i = 0; i < h.totalFrags; ++i)
                if (fp[i + 1] - fp[i] != __builtin_popcount(b[i])) bad = bad > i ? bad : i;
        } else {
            const uint64_t *b = reinterpret_cast<const uint64_t *>(f.arr[PA_FRAGBIT].data());
#pragma omp parallel for reduction(max : bad) schedule(static)
            for (long long i = 0; i < h.totalFrags; ++i)
                if (fp[i + 1] - fp[i] != __builtin_popcountll(b[i])) bad = bad > i ? bad : i;
        }
        if (bad >= 0) return at("fragPtr step differs from the bitmap's population count", bad);
    }
    if (!(r = pointer_problem("rowPtr_CD", ints(PA_ROWPTR_CD), h.n_rows, h.nnzCD)).empty()) return r;
    if (!(r = range_problem("colInd_CD", ints(PA_COLIND_CD), h.nnzCD, h.n_cols)).empty()) return r;
    return "";
}

}  // namespace mx

extern "C" int mx_check_partition_file(const char *path, int dtype, char *msg, int msg_len) {
    if (!path || (dtype != MX_FP64 && dtype != MX_FP16)) return MX_ERR_INVALID;
    mx::PartFile f;
    std::string p = mx::part_file_read(path, dtype, f);
    if (p.empty()) p = mx::part_file_problem(f);
    if (msg && msg_len > 0) {
        strncpy(msg, p.c_str(), (size_t)msg_len - 1);
        msg[msg_len - 1] = 0;
    }
    return p.empty() ? MX_OK : MX_ERR_INVALID;
}
