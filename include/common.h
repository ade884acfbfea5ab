// Types of the MatXtract host API (drop-in for the reference's include/common.h:53-79,237-245).
// Build with -Dfp64 for double values and 8x4 fragments; without it values are half and fragments 8x8.
#pragma once
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include <cuda_fp16.h>

#ifdef fp64
#define valT double
const int fragM = 8;
const int fragK = 4;
#else
#define valT half
const int fragM = 8;
const int fragK = 8;
#endif
#define indT int
const int WARP_SIZE = 32;

// vec[i] = (valT)(float)(i % 15): the values every reference driver multiplies with (include/common.h:237-245)
inline void initVec(valT *vec, int length) {
    for (int i = 0; i < length; ++i) vec[i] = static_cast<valT>(static_cast<float>(i % 15));
}
