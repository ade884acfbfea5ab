// Stored partitions: file layout, reader and validator (host code, no CUDA).
//
// A stored partition is what mx_save_partition writes and mx_load_partition restores: a header with the counts of the
// extraction followed by its thirteen arrays, each preceded by its byte count.  Everything in the file is later used
// as an address on the device (row ids, column ids, value offsets), so the loader validates every array on the host
// BEFORE anything is uploaded: a stale, truncated or bit-flipped file is refused with a message instead of turning
// into an out-of-bounds access on a GPU that other jobs share.
#pragma once
#include <cstdint>
#include <string>
#include <vector>

namespace mx {

constexpr char kPartMagic[8] = {'M', 'X', 'P', 'A', 'R', 'T', '0', '2'};
constexpr int32_t kPartVersion = 2;

struct PartFileHeader {
    char magic[8];
    int32_t version, dtype, n_rows, n_cols, nnz;
    int32_t dCols, nnzColD, sCols, nnzColS, dRows, nnzRowD, sRows, nnzRowS, chunkNum, totalFrags, nnzCD, fragK;
    int32_t reserved;
    double tc_nnz_ratio;
};

// order of the arrays in the file
enum PartArrayId {
    PA_XPERM = 0, PA_RID, PA_ROWPTR_DD, PA_COLIND_DD, PA_VAL_DD, PA_CHUNKPTR, PA_ATOX, PA_FRAGPTR, PA_FRAGBIT, PA_TCVAL,
    PA_ROWPTR_CD, PA_COLIND_CD, PA_VAL_CD, PA_COUNT
};

// byte size every array must have for this header (dtype decides the value and bitmap widths)
void part_array_bytes(const PartFileHeader &h, uint64_t out[PA_COUNT]);

// "" when the header's counts are consistent with each other and with `dtype`, else what is wrong
std::string part_header_problem(const PartFileHeader &h, int dtype);

struct PartFile {
    PartFileHeader hd{};
    std::vector<unsigned char> arr[PA_COUNT];
};

// Reads the whole file into host memory; "" on success, else what is wrong (cannot open, bad magic, sizes that do not
// follow from the header, truncated file).
std::string part_file_read(const char *path, int dtype, PartFile &out);

// "" when every array is safe to use as addresses: pointer arrays start at 0, are monotone and end at their count;
// row ids are distinct and in range; xperm is a permutation of the columns; every column id is in range; every
// fragment's value count equals the population count of its bitmap.
std::string part_file_problem(const PartFile &f);

}  // namespace mx
