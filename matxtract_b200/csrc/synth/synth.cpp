// Seeded synthetic CSR generators (host code, no CUDA).
//
// The reference evaluates on SuiteSparse files that are not redistributable here, so the benchmark and
// the tests use matrices generated from shape statistics only.  Every row is generated independently
// from a counter-based stream keyed by (seed, row), so any row range can be regenerated on its own
// (one range per GPU) and the result does not depend on the thread count.  Columns inside a row are
// distinct and ascending.  Indices are int32 like the reference's indT (include/common.h:79).
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>

#include <cuda_fp16.h>

#include "mx_synth.h"

namespace {

struct Rng {
    uint64_t s;
    explicit Rng(uint64_t seed, uint64_t stream) {
        s = seed * 0x9E3779B97F4A7C15ull + stream * 0xD1B54A32D192ED03ull + 0x2545F4914F6CDD1Dull;
        next();
        next();
    }
    uint64_t next() {  // splitmix64
        uint64_t z = (s += 0x9E3779B97F4A7C15ull);
        z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
        z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
        return z ^ (z >> 31);
    }
    double uni() { return (double)(next() >> 11) * (1.0 / 9007199254740992.0); }  // [0,1)
    int64_t below(int64_t n) { return (int64_t)(uni() * (double)n); }
    double normal() {
        double u1 = 1.0 - uni(), u2 = uni();
        return std::sqrt(-2.0 * std::log(u1)) * std::cos(6.283185307179586 * u2);
    }
};

int poisson(Rng &r, double lambda) {  // Knuth; lambda is small (10)
    double L = std::exp(-lambda), p = 1.0;
    int k = 0;
    do {
        k++;
        p *= r.uni();
    } while (p > L);
    return k - 1;
}

// Discrete power law with P(K >= k) = k^-(s-1), scaled by alpha and clipped to [1, maxlen].
int powerlaw_len(Rng &r, double s, double alpha, int maxlen) {
    double u = 1.0 - r.uni();  // (0,1]
    double k = std::floor(std::pow(u, -1.0 / (s - 1.0)));
    double len = std::ceil(alpha * k);
    if (!(len < (double)maxlen)) return maxlen;
    return len < 1.0 ? 1 : (int)len;
}

int64_t gcd64(int64_t a, int64_t b) { return b ? gcd64(b, a % b) : a; }

struct Gen {
    mx_synth_params P;
    int64_t hot_a = 1, hot_b = 0, n_hot = 0;
    explicit Gen(const mx_synth_params &p) : P(p) {
        if (P.kind == MX_SYNTH_HOTCOL) {
            n_hot = std::max<int64_t>(1, (int64_t)std::llround(P.hot_col_frac * (double)P.n));
            hot_a = (int64_t)(0.6180339887 * (double)P.n) | 1;
            while (gcd64(hot_a, P.n) != 1) hot_a += 2;
            hot_b = (int64_t)(P.seed % (uint64_t)P.n);
        }
    }
    // columns of one row into `c` (sorted, distinct)
    void row_cols(int64_t i, Rng &r, std::vector<int> &c) const {
        c.clear();
        const int64_t n = P.n;
        switch (P.kind) {
            case MX_SYNTH_UNIFORM: {
                int len = std::min<int64_t>(poisson(r, P.mean_len), n);
                while ((int)c.size() < len) {  // without replacement: redraw duplicates
                    int v = (int)r.below(n);
                    if (std::find(c.begin(), c.end(), v) == c.end()) c.push_back(v);
                }
                std::sort(c.begin(), c.end());
                return;
            }
            case MX_SYNTH_POWERLAW: {
                int len = powerlaw_len(r, P.zipf_s, P.alpha, (int)std::min<int64_t>(P.max_len, n));
                int64_t lo = std::max<int64_t>(0, i - P.local_halfwidth), hi = std::min<int64_t>(n - 1, i + P.local_halfwidth);
                // draw until the row holds `len` distinct columns; after the first round (the +-halfwidth window
                // may be saturated) the missing ones are drawn uniformly
                for (int round = 0; (int)c.size() < len && round < 64; ++round) {
                    int need = len - (int)c.size();
                    for (int k = 0; k < need; ++k) {
                        if (round == 0 && r.uni() < P.local_frac)
                            c.push_back((int)(lo + r.below(hi - lo + 1)));
                        else
                            c.push_back((int)r.below(n));
                    }
                    std::sort(c.begin(), c.end());
                    c.erase(std::unique(c.begin(), c.end()), c.end());
                }
                return;
            }
            case MX_SYNTH_BLOCK: {
                // all 8 rows of a block row share one stream (keyed by the block row), so blocks are dense 8x8
                const int bs = 8;
                int64_t nb = n / bs, bi = i / bs;
                int64_t lo = std::max<int64_t>(0, bi - P.local_halfwidth), hi = std::min<int64_t>(nb - 1, bi + P.local_halfwidth);
                int want = (int)std::min<int64_t>(P.blocks_per_row, hi - lo + 1);
                std::vector<int64_t> bc;
                while ((int)bc.size() < want) {
                    int64_t v = lo + r.below(hi - lo + 1);
                    if (std::find(bc.begin(), bc.end(), v) == bc.end()) bc.push_back(v);
                }
                std::sort(bc.begin(), bc.end());
                for (int64_t b : bc)
                    for (int k = 0; k < bs; ++k) c.push_back((int)(b * bs + k));
                return;
            }
            case MX_SYNTH_HOTCOL: {
                // 1 + geometric with mean (mean_len - 1)
                double q = 1.0 / P.mean_len;  // P(stop) per trial so that E[len] = mean_len
                int len = 1 + (int)std::floor(std::log(1.0 - r.uni()) / std::log(1.0 - q));
                len = (int)std::min<int64_t>(len, n);
                for (int round = 0; (int)c.size() < len && round < 64; ++round) {
                    int need = len - (int)c.size();
                    for (int k = 0; k < need; ++k) {
                        if (r.uni() < P.hot_nnz_frac) {
                            int64_t h = r.below(n_hot);
                            c.push_back((int)((hot_a * h + hot_b) % n));
                        } else
                            c.push_back((int)r.below(n));
                    }
                    std::sort(c.begin(), c.end());
                    c.erase(std::unique(c.begin(), c.end()), c.end());
                }
                return;
            }
        }
        std::sort(c.begin(), c.end());
        c.erase(std::unique(c.begin(), c.end()), c.end());
    }
    Rng row_rng(int64_t i) const { return Rng(P.seed, P.kind == MX_SYNTH_BLOCK ? (uint64_t)(i / 8) : (uint64_t)i); }
};

void store_val(int dtype, void *val, int64_t p, double v) {
    if (dtype == MX_SYNTH_FP64)
        ((double *)val)[p] = v;
    else
        ((__half *)val)[p] = __float2half((float)v);
}

}  // namespace

extern "C" {

int mx_synth_row_lengths(const mx_synth_params *p, int64_t row_begin, int64_t row_end, int *row_ptr_out) {
    if (!p || !row_ptr_out || row_begin < 0 || row_end > p->n || row_begin > row_end) return 1;  // bad argument
    Gen g(*p);
    int64_t rows = row_end - row_begin;
    std::vector<int> len(rows);
#pragma omp parallel
    {
        std::vector<int> c;
#pragma omp for schedule(dynamic, 4096)
        for (int64_t i = 0; i < rows; ++i) {
            Rng r = g.row_rng(row_begin + i);
            g.row_cols(row_begin + i, r, c);
            len[i] = (int)c.size();
        }
    }
    int64_t acc = 0;
    row_ptr_out[0] = 0;
    for (int64_t i = 0; i < rows; ++i) {
        acc += len[i];
        if (acc > 2147483647LL) return 5;  // more than INT_MAX entries
        row_ptr_out[i + 1] = (int)acc;
    }
    return 0;
}

int mx_synth_fill(const mx_synth_params *p, int dtype, int64_t row_begin, int64_t row_end, const int *row_ptr,
                  int *col_ind, void *val) {
    if (!p || !row_ptr || !col_ind || !val) return 1;  // bad argument
    Gen g(*p);
    int64_t rows = row_end - row_begin;
    int bad = 0;
#pragma omp parallel
    {
        std::vector<int> c;
#pragma omp for schedule(dynamic, 4096)
        for (int64_t i = 0; i < rows; ++i) {
            Rng r = g.row_rng(row_begin + i);
            g.row_cols(row_begin + i, r, c);
            if ((int)c.size() != row_ptr[i + 1] - row_ptr[i]) {
                bad = 1;
                continue;
            }
            // values come from a second stream so that they do not depend on how many draws the columns took
            Rng rv(p->seed ^ 0xA5A5A5A5DEADBEEFull, (uint64_t)(row_begin + i));
            int64_t q = row_ptr[i];
            for (size_t k = 0; k < c.size(); ++k, ++q) {
                col_ind[q] = c[k];
                store_val(dtype, val, q, p->normal_values ? rv.normal() : 2.0 * rv.uni() - 1.0);
            }
        }
    }
    return bad ? 1 : 0;
}

// x ~ U(-1,1), element i from stream (seed, i): independent of the length requested.
int mx_synth_vector(uint64_t seed, int dtype, int64_t begin, int64_t end, void *x) {
    if (!x || begin > end) return 1;  // bad argument
#pragma omp parallel for schedule(static)
    for (int64_t i = begin; i < end; ++i) {
        Rng r(seed ^ 0x5851F42D4C957F2Dull, (uint64_t)i);
        store_val(dtype, x, i - begin, 2.0 * r.uni() - 1.0);
    }
    return 0;
}

}  // extern "C"
