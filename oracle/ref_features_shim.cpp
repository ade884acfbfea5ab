// Test infrastructure: the reference's feature extractor (ML/extract_features.cpp) compiled unmodified from where it
// lies, with its main() renamed, so that its computeDistStats can be called on in-memory count arrays.  Part of
// oracle/_ref/libref_fp64.so; never linked into the shipped library.
#define main reference_features_main
#include "ML/extract_features.cpp"
#undef main

extern "C" void ref_dist_stats(const long long *arr, long long n, double *out) {
    std::vector<long long> v(arr, arr + n);
    const std::vector<double> cover = {0.1, 0.2, 0.3, 0.4, 0.5, 0.6, 0.7, 0.8, 0.9};  // the list of its main()
    DistStats s = computeDistStats(v, cover);
    for (int i = 0; i < 24; ++i) out[i] = 0.0;
    out[0] = s.meanVal;
    out[1] = s.stdVal;
    out[2] = (double)s.minVal;
    out[3] = (double)s.maxVal;
    out[4] = s.pRatio;
    for (size_t i = 0; i < s.topRatios.size() && i < 10; ++i) out[5 + i] = s.topRatios[i];
    for (size_t i = 0; i < s.hotCoverage.size() && i < 9; ++i) out[15 + i] = s.hotCoverage[i];
}
