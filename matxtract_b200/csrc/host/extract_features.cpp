// extract_features <mtx_root_folder> <output_csv> - the reference's feature extractor (ML/extract_features.cpp:95-217)
// on this library: every <root>/<name>/<name>.mtx is read with the parallel Matrix Market reader, uploaded, and its
// row / column distribution statistics are computed on the device (mx_features).  Same CSV header, same column
// order, same default stream formatting, same closing message, so ML/train_and_save_model.py and
// ML/load_and_predict_test.py read the file unchanged.
#include <filesystem>
#include <fstream>
#include <iostream>
#include <string>

#include "mx_capi.h"

namespace fs = std::filesystem;

static void put(std::ofstream &o, const mx_dist_features &d, bool last) {
    o << d.mean << "," << d.std_dev << "," << d.min << "," << d.max << "," << d.p_ratio << ",";
    for (double t : d.top) o << t << ",";
    for (int i = 0; i < 9; ++i) {
        o << d.hot[i];
        if (i + 1 < 9) o << ",";
    }
    o << (last ? "\n" : ",");
}

int main(int argc, char *argv[]) {
    if (argc < 3) {
        std::cerr << "Usage: " << argv[0] << " <mtx_root_folder> <output_csv>\n";
        return 1;
    }
    std::ofstream ofs(argv[2]);
    if (!ofs.is_open()) {
        std::cerr << "[Error] Cannot open output CSV: " << argv[2] << "\n";
        return 1;
    }
    ofs << "MatrixName,nrows,ncols,nnz,rowMean,rowStd,rowMin,rowMax,rowPRatio,";
    ofs << "rowTop1,rowTop2,rowTop3,rowTop4,rowTop5,rowTop10,rowTop50,rowTop100,rowTop200,rowTop300,";
    ofs << "rowHot10,rowHot20,rowHot30,rowHot40,rowHot50,rowHot60,rowHot70,rowHot80,rowHot90,";
    ofs << "colMean,colStd,colMin,colMax,colPRatio,";
    ofs << "colTop1,colTop2,colTop3,colTop4,colTop5,colTop10,colTop50,colTop100,colTop200,colTop300,";
    ofs << "colHot10,colHot20,colHot30,colHot40,colHot50,colHot60,colHot70,colHot80,colHot90\n";
    mx_handle_t h = nullptr;
    int st = mx_create(&h, 0, MX_FP64);
    if (st != MX_OK) {
        std::cerr << "[Error] " << mx_status_string(st) << "\n";
        return 1;
    }
    for (const auto &entry : fs::directory_iterator(argv[1])) {
        if (!entry.is_directory()) continue;
        const std::string name = entry.path().filename().string();
        const fs::path mtx = entry.path() / (name + ".mtx");
        if (!fs::exists(mtx)) continue;
        int rows = 0, cols = 0, nnz = 0, sym = 0, *rp = nullptr, *ci = nullptr;
        void *val = nullptr;
        if (mx_read_matrix_market(mtx.string().c_str(), MX_FP64, 0, &rows, &cols, &nnz, &sym, &rp, &ci, &val) != 0) {
            std::cerr << "[Warning] cannot read " << mtx.string() << "\n";
            continue;
        }
        mx_matrix_features f;
        st = mx_upload_csr(h, rows, cols, nnz, rp, ci, val);
        if (st == MX_OK) st = mx_features(h, &f);
        mx_host_free(rp);
        mx_host_free(ci);
        mx_host_free(val);
        if (st != MX_OK) {
            std::cerr << "[Warning] " << name << ": " << mx_last_error_string(h) << "\n";
            continue;
        }
        ofs << name << "," << f.rows << "," << f.cols << "," << f.nnz << ",";
        put(ofs, f.row, false);
        put(ofs, f.col, true);
    }
    mx_destroy(h);
    ofs.close();
    std::cout << "Feature extraction done. Results saved to " << argv[2] << std::endl;
    return 0;
}
