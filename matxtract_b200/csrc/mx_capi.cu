// C ABI of libmatxtract_b200.so: handle management, matrix upload, extraction, SpMV, timing loops, and the
// stateless mirrors of the reference's host API (include/MatXtract.h).  See include/mx_capi.h.
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>

#include "mx_internal.h"
#include "partition_file.h"

using namespace mx;

struct mx_handle_s {
    int device = 0, dtype = MX_FP64;
    cudaStream_t stream = nullptr;
    std::string err;
    // input matrix
    bool has_matrix = false;
    int n_rows = 0, n_cols = 0, nnz = 0;
    int *row_ptr = nullptr, *col_ind = nullptr;
    void *val = nullptr;
    // extraction
    bool planned = false;  // some plan (with or without partition) is ready for mx_spmv
    mx_partition_stats stats{};
    PartArrays part;
    ResidPlan resid;
    TilePlan tile;
    ResidPlan ddcsr;         // the core-dense block as CSR, for the low-fill executor
    int dd_mode = MX_DD_AUTO;
    int dd_exec = MX_DD_TILE;  // the executor in use: MX_DD_TILE, MX_DD_CSR or MX_DD_SE
    SePlan se;                 // sparse-encode layout of the core-dense block (built when dd_mode allows that executor)
    int *se_col_perm[2] = {nullptr, nullptr}, *se_col_orig[2] = {nullptr, nullptr};  // slab / tail column ids
    float dd_ms[4] = {0, 0, 0, 0};  // tuned time of the block alone, indexed by executor (0 = not timed)
    float tuning_ms = 0;            // host time the plan-time tuners took in the last mx_partition / mx_load_partition
    // column-slab execution of the plain CSR product (tau = (0,0)) when x is far larger than L2
    int slab_mode = -1;             // -1 = automatic, 0 = off, k >= 2 = k slabs
    long long row_offset = 0;       // global index of the uploaded slab's first row (mx_set_row_offset)
    ColSlabs slabs;
    bool use_slabs = false;
    float slab_ms_plain = 0, slab_ms_slabbed = 0;
    void *peer_table = nullptr;     // 64 bytes: peer row addresses for the slab path's push
    // execution column space: the partition numbers columns by density rank (x must be permuted every product);
    // the same entries with their ORIGINAL column ids read x directly and keep the matrix's own locality
    int colspace_mode = MX_COLSPACE_AUTO;
    bool use_orig_cols = false;
    int *colInd_CD_orig = nullptr, *colInd_dd_orig = nullptr, *AToX_orig = nullptr;
    float tune_ms_perm = 0, tune_ms_orig = 0;
    // hot-column prefix of the permuted x in shared memory (persistent CSR kernel)
    int hot_mode = MX_HOT_AUTO;
    int hot_budget = 0;       // columns that fit (0: not applicable)
    bool use_hot = false;
    float tune_ms_hot = 0, tune_ms_nohot = 0;
    void *ytile = nullptr;   // [n_rows] accumulate-type carrier of the tile half
    void *x_perm = nullptr;  // [n_cols] x in partition order
    // staging for the host-pointer entry point
    void *x_stage = nullptr, *y_stage = nullptr;
    // pipelined host-pointer products (mx_spmv_host_async): a second pair of staging buffers, one stream per copy
    // direction, and per slot the events "x has arrived", "product done", "y has left"
    void *x_stage2 = nullptr, *y_stage2 = nullptr;
    cudaStream_t copy_in = nullptr, copy_out = nullptr;
    cudaEvent_t ev_in[2] = {nullptr, nullptr}, ev_done[2] = {nullptr, nullptr}, ev_out[2] = {nullptr, nullptr};
    unsigned long long async_calls = 0;
    int *dev_err = nullptr;

    int fail(int status, const std::string &msg) {
        err = msg;
        return status;
    }
    int cuda_fail(cudaError_t e, const char *what) {
        err = std::string(what) + ": " + cudaGetErrorString(e);
        return MX_ERR_CUDA;
    }
};

#define HCK(call)                                               \
    do {                                                        \
        cudaError_t e_ = (call);                                \
        if (e_ != cudaSuccess) return h->cuda_fail(e_, #call);  \
    } while (0)

namespace {

// two timing events that are destroyed on every way out of a function
struct EventPair {
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    cudaError_t create() {
        cudaError_t e = cudaEventCreate(&e0);
        return e == cudaSuccess ? cudaEventCreate(&e1) : e;
    }
    ~EventPair() {
        if (e0) cudaEventDestroy(e0);
        if (e1) cudaEventDestroy(e1);
    }
};

void drop_plan(mx_handle_t h) {
    cudaStream_t s = h->stream;  // frees are ordered after whatever the stream still has in flight
    resid_plan_free(h->resid, s);
    resid_plan_free(h->ddcsr, s);
    col_slabs_free(h->slabs, s);
    h->use_slabs = false;
    tile_plan_free(h->tile, s);
    if (h->se_col_perm[0]) {  // the plan owns the permuted column ids, the handle the original-numbered copies
        h->se.slabCol = h->se_col_perm[0];
        h->se.tailCol = h->se_col_perm[1];
    }
    se_plan_free(h->se, s);
    for (int *b : h->se_col_orig)
        if (b) cudaFreeAsync(b, s);
    h->se_col_perm[0] = h->se_col_perm[1] = h->se_col_orig[0] = h->se_col_orig[1] = nullptr;
    part_arrays_free(h->part, s);
    void *bufs[] = {h->ytile, h->x_perm, h->colInd_CD_orig, h->colInd_dd_orig, h->AToX_orig};
    for (void *b : bufs)
        if (b) cudaFreeAsync(b, s);
    h->colInd_CD_orig = h->colInd_dd_orig = h->AToX_orig = nullptr;
    h->use_orig_cols = h->use_hot = false;
    h->hot_budget = 0;
    h->ytile = h->x_perm = nullptr;
    h->planned = false;
    h->stats = mx_partition_stats{};
}

void drop_matrix(mx_handle_t h) {
    drop_plan(h);
    if (h->copy_in) cudaStreamSynchronize(h->copy_in);  // copies of a pipelined product may still use the buffers
    if (h->copy_out) cudaStreamSynchronize(h->copy_out);
    void *bufs[] = {h->row_ptr, h->col_ind, h->val, h->x_stage, h->y_stage, h->x_stage2, h->y_stage2};
    for (void *b : bufs)
        if (b) cudaFreeAsync(b, h->stream);
    h->row_ptr = h->col_ind = nullptr;
    h->val = h->x_stage = h->y_stage = h->x_stage2 = h->y_stage2 = nullptr;
    h->async_calls = 0;
    h->has_matrix = false;
    h->n_rows = h->n_cols = h->nnz = 0;
}

int check_device() {
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n <= 0) {
        cudaGetLastError();
        return MX_ERR_NO_DEVICE;
    }
    return MX_OK;
}

}  // namespace

namespace {
struct DevBufs {  // frees on scope exit
    void *p[16] = {};
    int n = 0;
    template <typename T>
    cudaError_t up(T **d, const void *src, size_t bytes) {
        cudaError_t e = cudaMalloc((void **)d, bytes + 64);  // slack: the tile kernel's bulk copies round up to 16 bytes
        if (e != cudaSuccess) return e;
        p[n++] = *d;
        if (src && bytes > 0) e = cudaMemcpy(*d, src, bytes, cudaMemcpyHostToDevice);
        return e;
    }
    ~DevBufs() {
        for (int i = 0; i < n; ++i) cudaFree(p[i]);
    }
};
}  // namespace

extern "C" {

int mx_version(void) { return 100; }

const char *mx_status_string(int status) {
    switch (status) {
        case MX_OK: return "ok";
        case MX_ERR_INVALID: return "invalid argument";
        case MX_ERR_CUDA: return "CUDA error";
        case MX_ERR_TAU: return "invalid tau (tau_c < tau_r, or a threshold no prefix reaches)";
        case MX_ERR_STATE: return "call out of order";
        case MX_ERR_OVERFLOW: return "count exceeds int32";
        case MX_ERR_TIMEOUT: return "bounded device wait ran out";
        case MX_ERR_NOMEM: return "out of memory";
        case MX_ERR_NO_DEVICE: return "no CUDA device (this library has no CPU fallback)";
        case MX_ERR_TOO_LARGE: return "matrix exceeds the fixed scratch of the allocation-free entry point";
    }
    return "unknown status";
}

int mx_create(mx_handle_t *out, int device, int dtype) {
    if (!out || (dtype != MX_FP64 && dtype != MX_FP16)) return MX_ERR_INVALID;
    *out = nullptr;
    int st = check_device();
    if (st != MX_OK) return st;
    if (cudaSetDevice(device) != cudaSuccess) {
        cudaGetLastError();
        return MX_ERR_INVALID;
    }
    {
        // keep freed buffers in the stream-ordered pool: re-extracting a matrix then costs no driver allocation
        cudaMemPool_t pool;
        if (cudaDeviceGetDefaultMemPool(&pool, device) == cudaSuccess) {
            unsigned long long keep = ~0ull;
            cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep);
        }
        cudaGetLastError();
    }
    mx_handle_t h = new mx_handle_s;
    h->device = device;
    h->dtype = dtype;
    if (cudaStreamCreateWithFlags(&h->stream, cudaStreamNonBlocking) != cudaSuccess ||
        cudaMalloc(&h->dev_err, sizeof(int)) != cudaSuccess || cudaMemset(h->dev_err, 0, sizeof(int)) != cudaSuccess ||
        cudaMalloc(&h->peer_table, 64) != cudaSuccess) {
        delete h;
        return MX_ERR_CUDA;
    }
    *out = h;
    return MX_OK;
}

int mx_destroy(mx_handle_t h) {
    if (!h) return MX_ERR_INVALID;
    cudaSetDevice(h->device);
    cudaStreamSynchronize(h->stream);
    drop_matrix(h);
    cudaStreamSynchronize(h->stream);
    cudaFree(h->dev_err);
    cudaFree(h->peer_table);
    for (int i = 0; i < 2; ++i)
        for (cudaEvent_t e : {h->ev_in[i], h->ev_done[i], h->ev_out[i]})
            if (e) cudaEventDestroy(e);
    if (h->copy_in) cudaStreamDestroy(h->copy_in);
    if (h->copy_out) cudaStreamDestroy(h->copy_out);
    cudaStreamDestroy(h->stream);
    delete h;
    return MX_OK;
}

const char *mx_last_error_string(mx_handle_t h) { return h ? h->err.c_str() : "null handle"; }
void *mx_stream(mx_handle_t h) { return h ? (void *)h->stream : nullptr; }

int mx_sync(mx_handle_t h) {
    if (!h) return MX_ERR_INVALID;
    HCK(cudaSetDevice(h->device));
    HCK(cudaStreamSynchronize(h->stream));
    return MX_OK;
}

int mx_upload_csr(mx_handle_t h, int n_rows, int n_cols, int nnz, const int *row_ptr, const int *col_ind,
                  const void *val) {
    if (!h) return MX_ERR_INVALID;
    if (n_rows < 0 || n_cols < 0 || nnz < 0 || !row_ptr || (nnz > 0 && (!col_ind || !val)))
        return h->fail(MX_ERR_INVALID, "mx_upload_csr: bad sizes or null arrays");
    if (row_ptr[0] != 0 || row_ptr[n_rows] != nnz) return h->fail(MX_ERR_INVALID, "mx_upload_csr: row_ptr ends != nnz");
    HCK(cudaSetDevice(h->device));
    drop_matrix(h);
    const size_t vb = val_bytes(h->dtype);
    HCK(cudaMallocAsync(&h->row_ptr, sizeof(int) * ((size_t)n_rows + 1), h->stream));
    HCK(cudaMallocAsync(&h->col_ind, sizeof(int) * (size_t)(nnz > 0 ? nnz : 1), h->stream));
    HCK(cudaMallocAsync(&h->val, vb * (size_t)(nnz > 0 ? nnz : 1), h->stream));
    HCK(cudaMallocAsync(&h->x_stage, vb * (size_t)(n_cols > 0 ? n_cols : 1), h->stream));
    HCK(cudaMallocAsync(&h->y_stage, vb * (size_t)(n_rows > 0 ? n_rows : 1), h->stream));
    HCK(cudaMemcpyAsync(h->row_ptr, row_ptr, sizeof(int) * ((size_t)n_rows + 1), cudaMemcpyHostToDevice, h->stream));
    if (nnz > 0) {
        HCK(cudaMemcpyAsync(h->col_ind, col_ind, sizeof(int) * (size_t)nnz, cudaMemcpyHostToDevice, h->stream));
        HCK(cudaMemcpyAsync(h->val, val, vb * (size_t)nnz, cudaMemcpyHostToDevice, h->stream));
    }
    // Every index of the matrix becomes an address in the kernels (x gathers, histogram bins, row segments), so one
    // pass on the device checks them before anything dereferences one: row pointers non-decreasing, column ids in
    // [0, n_cols).  A bad matrix is refused here and never reaches a kernel that would use it.
    int bad = 0;
    HCK(cudaMemsetAsync(h->dev_err, 0, sizeof(int), h->stream));
    HCK(validate_csr(n_rows, n_cols, nnz, h->row_ptr, h->col_ind, h->dev_err, h->stream));
    HCK(cudaMemcpyAsync(&bad, h->dev_err, sizeof(int), cudaMemcpyDeviceToHost, h->stream));
    HCK(cudaStreamSynchronize(h->stream));
    if (bad) {
        HCK(cudaMemsetAsync(h->dev_err, 0, sizeof(int), h->stream));
        drop_matrix(h);
        return h->fail(MX_ERR_INVALID, "mx_upload_csr: row_ptr decreases or a column index is outside [0, n_cols)");
    }
    h->n_rows = n_rows;
    h->n_cols = n_cols;
    h->nnz = nnz;
    h->has_matrix = true;
    return MX_OK;
}

// points the execution plans at the column numbering in use; `hot` = serve the hot-column prefix of the permuted x
// from shared memory (only meaningful in the permuted numbering)
static void select_colspace(mx_handle_t h, bool orig, bool hot = false) {
    h->use_orig_cols = orig;
    h->use_hot = !orig && hot && h->hot_budget > 0;
    h->resid.col_ind = orig ? h->colInd_CD_orig : h->part.colInd_CD;
    h->ddcsr.col_ind = orig ? h->colInd_dd_orig : h->part.colInd_dd;
    h->tile.A.AToX = orig ? h->AToX_orig : h->part.tiles.AToX;
    if (h->se_col_perm[0]) {
        h->se.slabCol = orig ? h->se_col_orig[0] : h->se_col_perm[0];
        h->se.tailCol = orig ? h->se_col_orig[1] : h->se_col_perm[1];
    }
    h->resid.hot_cols = h->ddcsr.hot_cols = h->use_hot ? h->hot_budget : 0;
}

// the core-dense block: tensor-core tile kernel, or (low fill) the CSR kernel on the same entries
static cudaError_t dd_enqueue(mx_handle_t h, const void *x) {
    if (h->dd_exec == MX_DD_TILE)
        return tile_spmv(h->dtype, h->tile, x, h->ytile, h->part.rId, true, false, h->dev_err, h->stream);
    if (h->dd_exec == MX_DD_SE) return se_spmv(h->dtype, h->se, x, h->ytile, true, false, h->stream);
    return resid_spmv_to_carrier(h->dtype, h->ddcsr, x, h->ytile, h->part.rId, h->stream);
}

static int spmv_enqueue(mx_handle_t h, const void *x_dev, void *y_dev, bool do_tile, bool do_resid,
                        bool permute = true, void *const *peers = nullptr, int n_peers = 0, long long row_offset = 0,
                        void *mc_y = nullptr) {
    if (peers && h->use_slabs && !h->stats.active) {
        // the far passes' sums go into this GPU's own rows of its own y; the band follows in row ranges whose
        // finished rows a second stream sends to the other GPUs
        int self = -1;
        for (int g = 0; g < n_peers && self < 0; ++g) {
            cudaPointerAttributes at{};
            if (cudaPointerGetAttributes(&at, peers[g]) == cudaSuccess && at.device == h->device &&
                at.type == cudaMemoryTypeDevice)
                self = g;
        }
        cudaGetLastError();
        if (self < 0) return h->fail(MX_ERR_INVALID, "mx_spmv_peers: none of the buffers lives on this handle's GPU");
        const size_t vb = val_bytes(h->dtype);
        void *y_own = static_cast<char *>(peers[self]) + (size_t)row_offset * vb;
        if (h->slabs.has_band) {
            HCK(col_slabs_spmv_peers(h->dtype, h->slabs, x_dev, peers, n_peers, self, row_offset, h->stream));
            return MX_OK;
        }
        // no band (the slab spans all columns' rows): accumulate locally, then push the finished rows
        HCK(col_slabs_spmv(h->dtype, h->slabs, x_dev, y_own, vb * (size_t)h->n_rows, h->stream));
        int pst = mx_peer_push(h->dtype, peers, n_peers, self, row_offset, h->n_rows, h->peer_table, h->stream);
        return pst == MX_OK ? MX_OK : h->fail(pst, "mx_spmv_peers: peer push failed");
    }
    if (peers) {  // final rows go to every GPU's y
        const void *x = x_dev;
        if (h->stats.active) {
            if (!h->use_orig_cols) {
                HCK(gather_vector(h->dtype, x_dev, h->part.xperm, h->x_perm, h->n_cols, h->stream));
                x = h->x_perm;
            }
            HCK(dd_enqueue(h, x));
        }
        HCK(resid_spmv_peers(h->dtype, h->resid, x, peers, n_peers, row_offset, h->stats.active ? h->ytile : nullptr,
                             h->stats.active ? h->part.hotmask : nullptr, h->stream,
                             h->stats.active != 0 && h->dd_exec == MX_DD_CSR, mc_y));
        return MX_OK;
    }
    if (h->stats.active) {
        const void *x = x_dev;
        if (!h->use_orig_cols) {
            if (permute) HCK(gather_vector(h->dtype, x_dev, h->part.xperm, h->x_perm, h->n_cols, h->stream));
            x = h->x_perm;
        }
        if (do_tile) HCK(dd_enqueue(h, x));
        if (do_resid)
            HCK(resid_spmv(h->dtype, h->resid, x, y_dev, h->ytile, h->part.hotmask, false, h->stream,
                           /*chained=*/do_tile && h->dd_exec == MX_DD_CSR));
    } else if (do_resid) {
        if (h->use_slabs)
            HCK(col_slabs_spmv(h->dtype, h->slabs, x_dev, y_dev, val_bytes(h->dtype) * (size_t)h->n_rows, h->stream));
        else
            HCK(resid_spmv(h->dtype, h->resid, x_dev, y_dev, nullptr, nullptr, false, h->stream));
    }
    return MX_OK;
}

// Times the whole product on scratch vectors in the candidate execution set-ups and keeps the fastest: the permuted
// column numbering without and with the hot-column prefix in shared memory, and the original numbering.
static int tune_colspace(mx_handle_t h) {
    h->tune_ms_perm = h->tune_ms_orig = h->tune_ms_hot = h->tune_ms_nohot = 0;
    const bool try_orig = h->colspace_mode != MX_COLSPACE_PERMUTED, try_perm = h->colspace_mode != MX_COLSPACE_ORIGINAL;
    const bool try_hot = try_perm && h->hot_budget > 0 && h->hot_mode != MX_HOT_OFF;
    const bool try_nohot = try_perm && !(try_hot && h->hot_mode == MX_HOT_ON);
    if (!try_perm) {
        select_colspace(h, true);
        return MX_OK;
    }
    if (!try_orig && try_hot != try_nohot) {  // nothing to choose
        select_colspace(h, false, try_hot);
        return MX_OK;
    }
    EventPair ev;
    HCK(ev.create());
    HCK(cudaMemsetAsync(h->x_stage, 0, val_bytes(h->dtype) * (size_t)h->n_cols, h->stream));
    auto measure = [&](bool orig, bool hot, float *ms) -> int {
        select_colspace(h, orig, hot);
        for (int i = 0; i < 3 + 10; ++i) {
            if (i == 3) HCK(cudaEventRecord(ev.e0, h->stream));
            int st = spmv_enqueue(h, h->x_stage, h->y_stage, true, true);
            if (st != MX_OK) return st;
        }
        HCK(cudaEventRecord(ev.e1, h->stream));
        HCK(cudaEventSynchronize(ev.e1));
        HCK(cudaEventElapsedTime(ms, ev.e0, ev.e1));
        *ms /= 10;
        return MX_OK;
    };
    int st;
    if (try_nohot && (st = measure(false, false, &h->tune_ms_nohot)) != MX_OK) return st;
    if (try_hot && (st = measure(false, true, &h->tune_ms_hot)) != MX_OK) return st;
    if (try_orig && (st = measure(true, false, &h->tune_ms_orig)) != MX_OK) return st;
    const bool hot = try_hot && (!try_nohot || h->tune_ms_hot < h->tune_ms_nohot);
    h->tune_ms_perm = hot ? h->tune_ms_hot : h->tune_ms_nohot;
    select_colspace(h, try_orig && h->tune_ms_orig < h->tune_ms_perm, hot);
    return MX_OK;
}

// The CSR kernel's L2 prefetch (ResidPlan::prefetch_tiles) helps or hurts with the matrix: each CSR plan in use whose
// size rule proposes a distance is timed with and without it (its half of the product alone), and the faster stays.
static int tune_prefetch(mx_handle_t h) {
    if (getenv("MX_RESID_PREFETCH")) return MX_OK;  // forced by the environment
    ResidPlan *plans[2] = {&h->resid, (h->stats.active && h->dd_exec == MX_DD_CSR) ? &h->ddcsr : nullptr};
    EventPair ev;
    for (ResidPlan *P : plans) {
        if (!P || P->prefetch_tiles <= 0 || P->num_tiles <= P->prefetch_tiles + 1) continue;
        if (!ev.e0) {
            HCK(ev.create());
            HCK(cudaMemsetAsync(h->x_stage, 0, val_bytes(h->dtype) * (size_t)h->n_cols, h->stream));
        }
        const int cand[2] = {P->prefetch_tiles, 0};
        float ms[2] = {0, 0};
        for (int v = 0; v < 2; ++v) {
            P->prefetch_tiles = cand[v];
            for (int i = 0; i < 2 + 6; ++i) {
                if (i == 2) HCK(cudaEventRecord(ev.e0, h->stream));
                const bool isResid = P == &h->resid;  // the half that owns the plan, alone
                int st = spmv_enqueue(h, h->x_stage, h->y_stage, !isResid, isResid);
                if (st != MX_OK) return st;
            }
            HCK(cudaEventRecord(ev.e1, h->stream));
            HCK(cudaEventSynchronize(ev.e1));
            HCK(cudaEventElapsedTime(&ms[v], ev.e0, ev.e1));
        }
        P->prefetch_tiles = ms[0] <= ms[1] ? cand[0] : 0;
    }
    return MX_OK;
}

// Plain CSR product (tau = (0,0)) of a matrix whose x is far larger than L2: build the column slabs, time the product
// both ways on scratch vectors and keep the faster.  FP64 only (the passes add into y in the value type).
static int tune_col_slabs(mx_handle_t h) {
    h->use_slabs = false;
    h->slab_ms_plain = h->slab_ms_slabbed = 0;
    if (h->dtype != MX_FP64 || h->slab_mode == 0 || h->stats.active || h->nnz <= 0) return MX_OK;
    int l2 = 0;
    cudaDeviceGetAttribute(&l2, cudaDevAttrL2CacheSize, h->device);
    const size_t xbytes = val_bytes(h->dtype) * (size_t)h->n_cols;
    CsrDev A;
    A.n_rows = h->n_rows, A.n_cols = h->n_cols, A.nnz = h->nnz;
    A.row_ptr = h->row_ptr, A.col_ind = h->col_ind, A.val = h->val;
    if (h->slab_mode > 0) {  // forced
        int status = MX_OK;
        HCK(col_slabs_build(h->dtype, A, h->slab_mode, h->row_offset, h->slabs, &status, h->stream));
        h->use_slabs = status == MX_OK;  // rows not sorted by column: the plain kernel stays
        return MX_OK;
    }
    if (l2 <= 0 || xbytes <= (size_t)l2) return MX_OK;  // x fits L2: nothing to gain
    // candidates: x ranges of 64, 44 and 32 MB per pass (fewer passes leave fewer partial sums to combine, narrower
    // ones keep their x range in L2 more safely; 96 MB never won); each is built, timed against the plain kernel on
    // scratch vectors, and the fastest stays
    EventPair ev;
    HCK(ev.create());
    HCK(cudaMemsetAsync(h->x_stage, 0, xbytes, h->stream));
    auto time_product = [&](float *ms) -> int {
        for (int i = 0; i < 2 + 5; ++i) {
            if (i == 2) HCK(cudaEventRecord(ev.e0, h->stream));
            int st = spmv_enqueue(h, h->x_stage, h->y_stage, false, true);
            if (st != MX_OK) return st;
        }
        HCK(cudaEventRecord(ev.e1, h->stream));
        HCK(cudaEventSynchronize(ev.e1));
        HCK(cudaEventElapsedTime(ms, ev.e0, ev.e1));
        *ms /= 5;
        return MX_OK;
    };
    int st = time_product(&h->slab_ms_plain);
    if (st != MX_OK) return st;
    float best = h->slab_ms_plain;
    int best_count = 0, last = 0;
    for (size_t mb : {64, 44, 32}) {
        const int count = (int)std::min<size_t>(64, (xbytes + (mb << 20) - 1) / (mb << 20));
        if (count < 2 || count == last) continue;
        last = count;
        ColSlabs trial;
        int status = MX_OK;
        HCK(col_slabs_build(h->dtype, A, count, h->row_offset, trial, &status, h->stream));
        if (status != MX_OK) return MX_OK;  // rows not sorted by column
        ColSlabs keep = h->slabs;
        h->slabs = trial;
        h->use_slabs = true;
        float ms = 0;
        st = time_product(&ms);
        h->use_slabs = false;
        h->slabs = keep;
        if (st != MX_OK) {
            col_slabs_free(trial, h->stream);
            return st;
        }
        if (h->slab_ms_slabbed == 0 || ms < h->slab_ms_slabbed) h->slab_ms_slabbed = ms;
        if (ms < best) {
            best = ms;
            best_count = count;
            col_slabs_free(h->slabs, h->stream);
            h->slabs = trial;
        } else {
            col_slabs_free(trial, h->stream);
        }
    }
    h->use_slabs = best_count > 0;
    return MX_OK;
}

// sparse-encode layout of the core-dense block, plus its column ids in the original numbering
static int build_se_plan(mx_handle_t h) {
    if (h->se_col_perm[0]) return MX_OK;
    h->se.n_rows = h->stats.dRows;
    h->se.n_cols = h->stats.dCols;
    h->se.nnz = h->stats.nnzRowD;
    HCK(se_plan_build(h->dtype, h->se, h->part.rowPtr_dd, h->part.colInd_dd, h->part.val_dd, h->part.rId, h->stream));
    h->se_col_perm[0] = h->se.slabCol;
    h->se_col_perm[1] = h->se.tailCol;
    const size_t slots = (size_t)h->se.numSlabs * 8 * (h->dtype == MX_FP64 ? 4 : 16);
    HCK(cudaMallocAsync(&h->se_col_orig[0], sizeof(int) * (slots > 0 ? slots : 1), h->stream));
    HCK(cudaMallocAsync(&h->se_col_orig[1], sizeof(int) * (size_t)(h->se.tailNnz > 0 ? h->se.tailNnz : 1), h->stream));
    HCK(map_indices(h->se_col_perm[0], h->part.xperm, h->se_col_orig[0], (long long)slots, h->stream));
    HCK(map_indices(h->se_col_perm[1], h->part.xperm, h->se_col_orig[1], h->se.tailNnz, h->stream));
    return MX_OK;
}

// MX_DD_AUTO: the core-dense block alone is timed through each of its three executors (tensor-core fragments,
// CUDA-core CSR, tensor-core sparse-encode) on the device and the fastest is kept.  The reference decides from two
// fixed thresholds tuned on another GPU (test/test_autotc_spmv.cpp:1507,1518).
static int tune_dd_executor(mx_handle_t h) {
    h->dd_ms[MX_DD_TILE] = h->dd_ms[MX_DD_CSR] = h->dd_ms[MX_DD_SE] = 0;
    if (h->dd_mode != MX_DD_AUTO || !h->stats.active) return MX_OK;
    EventPair ev;
    HCK(ev.create());
    HCK(cudaMemsetAsync(h->x_stage, 0, val_bytes(h->dtype) * (size_t)h->n_cols, h->stream));
    auto time_block = [&](float *ms) -> int {
        for (int i = 0; i < 2 + 6; ++i) {
            if (i == 2) HCK(cudaEventRecord(ev.e0, h->stream));
            int st = spmv_enqueue(h, h->x_stage, h->y_stage, true, false, /*permute=*/i == 0);
            if (st != MX_OK) return st;
        }
        HCK(cudaEventRecord(ev.e1, h->stream));
        HCK(cudaEventSynchronize(ev.e1));
        HCK(cudaEventElapsedTime(ms, ev.e0, ev.e1));
        *ms /= 6;
        return MX_OK;
    };
    int best = MX_DD_CSR;
    for (int ex : {MX_DD_TILE, MX_DD_CSR, MX_DD_SE}) {
        h->dd_exec = ex;
        int st = time_block(&h->dd_ms[ex]);
        if (st != MX_OK) return st;
        if (ex == MX_DD_TILE && h->tile.allFull) {
            // completely filled fragments: the streaming tile kernel was timed; now the staged one, keep the faster
            float staged = 0;
            h->tile.useFull = false;
            if ((st = time_block(&staged)) != MX_OK) return st;
            if (staged < h->dd_ms[ex])
                h->dd_ms[ex] = staged;
            else
                h->tile.useFull = true;
        }
        if (ex == MX_DD_TILE || h->dd_ms[ex] < h->dd_ms[best]) best = ex;
    }
    h->dd_exec = best;
    return MX_OK;
}

// Everything that follows the extraction proper (or the loading of a stored partition): execution plans of the two
// halves, the carrier, the index arrays in original column numbering, and the choice of the execution column space.
static int finish_partition(mx_handle_t h) {
    h->resid.n_rows = h->n_rows;
    h->resid.n_cols = h->n_cols;
    h->resid.nnz = h->stats.nnzCD;
    h->resid.row_ptr = h->part.rowPtr_CD;
    h->resid.col_ind = h->part.colInd_CD;
    h->resid.val = h->part.val_CD;
    HCK(resid_plan_build(h->dtype, h->resid, h->stream));
    h->tile.A = h->part.tiles;
    HCK(tile_plan_build(h->dtype, h->tile, h->stream));
    h->ddcsr.n_rows = h->stats.dRows;
    h->ddcsr.n_cols = h->stats.dCols;
    h->ddcsr.nnz = h->stats.nnzRowD;
    h->ddcsr.row_ptr = h->part.rowPtr_dd;
    h->ddcsr.col_ind = h->part.colInd_dd;
    h->ddcsr.val = h->part.val_dd;
    HCK(resid_plan_build(h->dtype, h->ddcsr, h->stream));
    h->resid.dev_err = h->ddcsr.dev_err = h->dev_err;
    h->hot_budget = resid_hot_cols_budget(h->dtype, h->stats.dCols);
    if (h->dd_mode == MX_DD_AUTO || h->dd_mode == MX_DD_SE) {
        int sst = build_se_plan(h);
        if (sst != MX_OK) return sst;
    }
    h->dd_exec = h->dd_mode == MX_DD_AUTO ? (h->stats.tc_nnz_ratio >= MX_DD_AUTO_FILL ? MX_DD_TILE : MX_DD_CSR)
                                          : h->dd_mode;
    HCK(cudaMallocAsync(&h->ytile, acc_bytes(h->dtype) * (size_t)h->n_rows, h->stream));
    HCK(cudaMemsetAsync(h->ytile, 0, acc_bytes(h->dtype) * (size_t)h->n_rows, h->stream));
    HCK(cudaMallocAsync(&h->x_perm, val_bytes(h->dtype) * (size_t)h->n_cols, h->stream));
    // the same entries numbered by their original columns
    const size_t nAToX = (size_t)h->stats.totalFrags * h->stats.fragK;
    HCK(cudaMallocAsync(&h->colInd_CD_orig, sizeof(int) * (size_t)(h->stats.nnzCD > 0 ? h->stats.nnzCD : 1), h->stream));
    HCK(cudaMallocAsync(&h->colInd_dd_orig, sizeof(int) * (size_t)(h->stats.nnzRowD > 0 ? h->stats.nnzRowD : 1), h->stream));
    HCK(cudaMallocAsync(&h->AToX_orig, sizeof(int) * (nAToX > 0 ? nAToX : 1), h->stream));
    HCK(map_indices(h->part.colInd_CD, h->part.xperm, h->colInd_CD_orig, h->stats.nnzCD, h->stream));
    HCK(map_indices(h->part.colInd_dd, h->part.xperm, h->colInd_dd_orig, h->stats.nnzRowD, h->stream));
    HCK(map_indices(h->part.tiles.AToX, h->part.xperm, h->AToX_orig, (long long)nAToX, h->stream));
    h->planned = true;  // the tuners run real products
    const auto t0 = std::chrono::steady_clock::now();
    select_colspace(h, false);
    int tst = tune_dd_executor(h);
    if (tst == MX_OK) tst = tune_colspace(h);
    if (tst == MX_OK) tst = tune_prefetch(h);
    if (tst != MX_OK) {
        drop_plan(h);
        return tst;
    }
    h->tuning_ms = std::chrono::duration<float, std::milli>(std::chrono::steady_clock::now() - t0).count();
    return MX_OK;
}

static int partition_impl(mx_handle_t h, double tau_c, double tau_r, mx_partition_stats *stats, const GlobalRanking *G);

int mx_partition(mx_handle_t h, double tau_c, double tau_r, mx_partition_stats *stats) {
    return partition_impl(h, tau_c, tau_r, stats, nullptr);
}

int mx_partition_global(mx_handle_t h, double tau_c, double tau_r, const int *global_col_counts_dev,
                        long long global_nnz, int row_cut_count, long long row_cut_index, long long row_offset,
                        mx_partition_stats *stats) {
    if (!h || !global_col_counts_dev || global_nnz < 0 || global_nnz > 2147483647LL || row_offset < 0)
        return MX_ERR_INVALID;
    GlobalRanking G;
    G.col_counts = global_col_counts_dev;
    G.nnz = global_nnz;
    G.has_row_cut = true;
    G.row_cut_count = row_cut_count;
    G.row_cut_index = row_cut_index;
    G.row_offset = row_offset;
    return partition_impl(h, tau_c, tau_r, stats, &G);
}

int mx_col_counts(mx_handle_t h, int *counts_dev) {
    if (!h || !counts_dev) return MX_ERR_INVALID;
    if (!h->has_matrix) return h->fail(MX_ERR_STATE, "mx_col_counts: no matrix uploaded");
    HCK(cudaSetDevice(h->device));
    CsrDev A;
    A.n_rows = h->n_rows, A.n_cols = h->n_cols, A.nnz = h->nnz;
    A.row_ptr = h->row_ptr, A.col_ind = h->col_ind, A.val = h->val;
    HCK(column_counts(A, counts_dev, h->stream));
    HCK(cudaStreamSynchronize(h->stream));
    return MX_OK;
}

int mx_row_counts_in_hot_columns(mx_handle_t h, double tau_c, const int *global_col_counts_dev, long long global_nnz,
                                 int *row_counts_dev) {
    if (!h || !row_counts_dev || global_nnz < 0 || global_nnz > 2147483647LL) return MX_ERR_INVALID;
    if (!h->has_matrix) return h->fail(MX_ERR_STATE, "mx_row_counts_in_hot_columns: no matrix uploaded");
    HCK(cudaSetDevice(h->device));
    CsrDev A;
    A.n_rows = h->n_rows, A.n_cols = h->n_cols, A.nnz = h->nnz;
    A.row_ptr = h->row_ptr, A.col_ind = h->col_ind, A.val = h->val;
    GlobalRanking G;
    G.col_counts = global_col_counts_dev;
    G.nnz = global_nnz;
    int status = MX_OK;
    HCK(partition_row_counts(h->dtype, A, (float)tau_c, global_col_counts_dev ? &G : nullptr, row_counts_dev, &status,
                             h->stream));
    if (status != MX_OK) return h->fail(status, "tau_c threshold never reached by the ranking prefix");
    return MX_OK;
}

int mx_rank_cut(mx_handle_t h, const int *counts_dev, int n, long long threshold, long long out[4]) {
    if (!h || !counts_dev || !out || n < 0 || threshold < 0 || threshold > 2147483647LL) return MX_ERR_INVALID;
    HCK(cudaSetDevice(h->device));
    HCK(rank_cut(counts_dev, n, (int)threshold, out, h->stream));
    return MX_OK;
}

static int partition_impl(mx_handle_t h, double tau_c, double tau_r, mx_partition_stats *stats, const GlobalRanking *G) {
    if (!h) return MX_ERR_INVALID;
    if (!h->has_matrix) return h->fail(MX_ERR_STATE, "mx_partition: no matrix uploaded");
    if (tau_c < tau_r) return h->fail(MX_ERR_TAU, "col_frac must be greater than hot_frac");
    HCK(cudaSetDevice(h->device));
    drop_plan(h);
    h->tuning_ms = 0;
    const float colProp = (float)tau_c, rowProp = (float)tau_r;
    EventPair ev;
    HCK(ev.create());
    const cudaEvent_t e0 = ev.e0, e1 = ev.e1;
    HCK(cudaEventRecord(e0, h->stream));
    h->stats = mx_partition_stats{};
    h->stats.fragK = frag_k(h->dtype);
    if (rowProp == 0.0f && colProp == 0.0f) {
        // tau = (0,0): the reference skips the extraction and runs cdspmv on the input CSR
        h->resid.n_rows = h->n_rows;
        h->resid.n_cols = h->n_cols;
        h->resid.nnz = h->nnz;
        h->resid.row_ptr = h->row_ptr;
        h->resid.col_ind = h->col_ind;
        h->resid.val = h->val;
        HCK(resid_plan_build(h->dtype, h->resid, h->stream));
        h->stats.nnzCD = h->nnz;
        h->stats.sCols = h->n_cols;
        h->stats.sRows = h->n_rows;
        h->stats.nnzColS = h->nnz;
        h->planned = true;  // the tuner runs real products
        const auto t0 = std::chrono::steady_clock::now();
        int tst = tune_prefetch(h);
        if (tst == MX_OK) tst = tune_col_slabs(h);
        if (tst != MX_OK) {
            drop_plan(h);
            return tst;
        }
        h->tuning_ms = std::chrono::duration<float, std::milli>(std::chrono::steady_clock::now() - t0).count();
    } else {
        // The reference assumes a square matrix (its tau_c scan runs i < rowA over the column table,
        // test/test_autotc_spmv.cpp:1133).  A rectangular row slab (one GPU's share of a row-partitioned
        // matrix) is accepted too: the scan then runs over min(rows, cols) ranked columns.
        CsrDev A;
        A.n_rows = h->n_rows;
        A.n_cols = h->n_cols;
        A.nnz = h->nnz;
        A.row_ptr = h->row_ptr;
        A.col_ind = h->col_ind;
        A.val = h->val;
        int status = MX_OK;
        cudaError_t ce = partition_run(h->dtype, A, colProp, rowProp, h->part, h->stats, &status, h->stream, G);
        if (ce != cudaSuccess) {
            drop_plan(h);
            return h->cuda_fail(ce, "partition_run");
        }
        if (status != MX_OK) {
            drop_plan(h);
            return h->fail(status, status == MX_ERR_TAU ? "tau threshold never reached by the ranking prefix"
                                                        : "fragment count exceeds int32");
        }
        int fst = finish_partition(h);
        if (fst != MX_OK) return fst;
    }
    HCK(cudaEventRecord(e1, h->stream));
    HCK(cudaEventSynchronize(e1));
    float ms = 0;
    HCK(cudaEventElapsedTime(&ms, e0, e1));
    // the tuners' timed products are reported on their own, not as extraction time
    h->stats.tuning_ms = h->tuning_ms;
    h->stats.preprocess_ms = ms > h->tuning_ms ? ms - h->tuning_ms : ms;
    h->planned = true;
    if (stats) *stats = h->stats;
    return MX_OK;
}

// ---- stored partitions ---------------------------------------------------------------------------------------
int mx_save_partition(mx_handle_t h, const char *path) {
    if (!h || !path) return MX_ERR_INVALID;
    if (!h->planned || !h->stats.active) return h->fail(MX_ERR_STATE, "mx_save_partition: no active partition");
    HCK(cudaSetDevice(h->device));
    const mx_partition_stats &s = h->stats;
    PartFileHeader hd{};
    memcpy(hd.magic, kPartMagic, 8);
    hd.version = kPartVersion;
    hd.dtype = h->dtype;
    hd.n_rows = h->n_rows;
    hd.n_cols = h->n_cols;
    hd.nnz = h->nnz;
    hd.dCols = s.dCols, hd.nnzColD = s.nnzColD, hd.sCols = s.sCols, hd.nnzColS = s.nnzColS;
    hd.dRows = s.dRows, hd.nnzRowD = s.nnzRowD, hd.sRows = s.sRows, hd.nnzRowS = s.nnzRowS;
    hd.chunkNum = s.chunkNum, hd.totalFrags = s.totalFrags, hd.nnzCD = s.nnzCD, hd.fragK = s.fragK;
    hd.tc_nnz_ratio = s.tc_nnz_ratio;
    struct FileCloser {
        FILE *f;
        ~FileCloser() {
            if (f) fclose(f);
        }
    } fc{fopen(path, "wb")};
    if (!fc.f) return h->fail(MX_ERR_INVALID, std::string("cannot open for writing: ") + path);
    if (fwrite(&hd, sizeof hd, 1, fc.f) != 1) return h->fail(MX_ERR_INVALID, "write failed");
    uint64_t bytes[PA_COUNT];
    part_array_bytes(hd, bytes);
    const void *dev[PA_COUNT] = {h->part.xperm,          h->part.rId,         h->part.rowPtr_dd,     h->part.colInd_dd,
                                 h->part.val_dd,         h->part.tiles.chunkPtr, h->part.tiles.AToX, h->part.tiles.fragPtr,
                                 h->part.tiles.fragBit,  h->part.tiles.tcVal, h->part.rowPtr_CD,     h->part.colInd_CD,
                                 h->part.val_CD};
    std::string buf;
    for (int a = 0; a < PA_COUNT; ++a) {
        const uint64_t n = bytes[a];
        if (fwrite(&n, sizeof n, 1, fc.f) != 1) return h->fail(MX_ERR_INVALID, "write failed");
        if (n == 0) continue;
        buf.resize(n);
        HCK(cudaMemcpyAsync(&buf[0], dev[a], n, cudaMemcpyDeviceToHost, h->stream));
        HCK(cudaStreamSynchronize(h->stream));
        if (fwrite(buf.data(), 1, n, fc.f) != n) return h->fail(MX_ERR_INVALID, "write failed");
    }
    return MX_OK;
}

int mx_load_partition(mx_handle_t h, const char *path, mx_partition_stats *stats) {
    if (!h || !path) return MX_ERR_INVALID;
    // the whole file is read and validated on the host before anything reaches the device: its arrays become
    // addresses in the kernels
    PartFile pf;
    std::string problem = part_file_read(path, h->dtype, pf);
    if (problem.empty()) problem = part_file_problem(pf);
    if (!problem.empty()) return h->fail(MX_ERR_INVALID, "stored partition: " + problem);
    const PartFileHeader &hd = pf.hd;
    HCK(cudaSetDevice(h->device));
    drop_matrix(h);  // a loaded partition replaces the matrix: it holds every entry (no re-extraction from it)
    auto refuse = [&](int status) {  // nothing of a half-loaded partition stays behind
        drop_matrix(h);
        h->n_rows = h->n_cols = h->nnz = 0;
        return status;
    };
    h->n_rows = hd.n_rows;
    h->n_cols = hd.n_cols;
    h->nnz = hd.nnz;
    mx_partition_stats &s = h->stats;
    s = mx_partition_stats{};
    s.dCols = hd.dCols, s.nnzColD = hd.nnzColD, s.sCols = hd.sCols, s.nnzColS = hd.nnzColS;
    s.dRows = hd.dRows, s.nnzRowD = hd.nnzRowD, s.sRows = hd.sRows, s.nnzRowS = hd.nnzRowS;
    s.chunkNum = hd.chunkNum, s.totalFrags = hd.totalFrags, s.nnzCD = hd.nnzCD, s.fragK = hd.fragK;
    s.tc_nnz_ratio = hd.tc_nnz_ratio;
    s.active = 1;
    const size_t vb = val_bytes(h->dtype);
    void **dev[PA_COUNT] = {(void **)&h->part.xperm,          (void **)&h->part.rId,
                            (void **)&h->part.rowPtr_dd,      (void **)&h->part.colInd_dd,
                            (void **)&h->part.val_dd,         (void **)&h->part.tiles.chunkPtr,
                            (void **)&h->part.tiles.AToX,     (void **)&h->part.tiles.fragPtr,
                            (void **)&h->part.tiles.fragBit,  (void **)&h->part.tiles.tcVal,
                            (void **)&h->part.rowPtr_CD,      (void **)&h->part.colInd_CD,
                            (void **)&h->part.val_CD};
    for (int a = 0; a < PA_COUNT; ++a) {
        const size_t n = pf.arr[a].size();
        // slack: the tile kernel's bulk copies round up to 16 bytes
        cudaError_t e = cudaMallocAsync(dev[a], n + 64 + 16, h->stream);
        if (e == cudaSuccess && n > 0)
            e = cudaMemcpyAsync(*dev[a], pf.arr[a].data(), n, cudaMemcpyHostToDevice, h->stream);
        if (e != cudaSuccess) {
            refuse(MX_ERR_CUDA);
            return h->cuda_fail(e, "mx_load_partition: upload");
        }
    }
    cudaError_t e = cudaStreamSynchronize(h->stream);  // the host copies go out of scope with pf
    h->part.tiles.dRows = s.dRows;
    h->part.tiles.dCols = s.dCols;
    h->part.tiles.chunkNum = s.chunkNum;
    h->part.tiles.totalFrags = s.totalFrags;
    h->part.tiles.nvals = s.nnzRowD;
    if (e == cudaSuccess) e = hotmask_from_rid(h->part.rId, s.dRows, h->n_rows, &h->part.hotmask, h->stream);
    if (e == cudaSuccess) e = cudaMallocAsync(&h->x_stage, vb * (size_t)(h->n_cols > 0 ? h->n_cols : 1), h->stream);
    if (e == cudaSuccess) e = cudaMallocAsync(&h->y_stage, vb * (size_t)(h->n_rows > 0 ? h->n_rows : 1), h->stream);
    if (e != cudaSuccess) {
        refuse(MX_ERR_CUDA);
        return h->cuda_fail(e, "mx_load_partition");
    }
    int st = finish_partition(h);
    if (st != MX_OK) return refuse(st);
    HCK(cudaStreamSynchronize(h->stream));
    h->stats.tuning_ms = h->tuning_ms;
    if (stats) *stats = h->stats;
    return MX_OK;
}

// ---- tau search on the device --------------------------------------------------------------------------------
int mx_autotune_tau(mx_handle_t h, int grid, double *tau_c, double *tau_r, float *ms_best, float *ms_plain) {
    if (!h || grid < 1 || grid > 16 || !tau_c || !tau_r) return MX_ERR_INVALID;
    if (!h->has_matrix) return h->fail(MX_ERR_STATE, "mx_autotune_tau: no matrix uploaded");
    HCK(cudaSetDevice(h->device));
    EventPair ev;
    HCK(ev.create());
    const cudaEvent_t e0 = ev.e0, e1 = ev.e1;
    double bc = 0, br = 0;
    float best = -1.f, plain = 0.f;
    for (int i = 0; i <= grid; ++i)  // tau_c = i / grid up to 1 (everything in the core-dense block's columns)
        for (int j = 0; j <= i; ++j) {
            if (i == 0 && j > 0) continue;
            const double tc = (double)i / grid, tr = (double)j / grid;
            int st = mx_partition(h, tc, tr, nullptr);
            if (st == MX_ERR_TAU) continue;  // no prefix of the ranking reaches the threshold: not a candidate
            if (st != MX_OK) return st;
            HCK(cudaMemsetAsync(h->x_stage, 0, val_bytes(h->dtype) * (size_t)h->n_cols, h->stream));
            for (int it = 0; it < 3 + 10; ++it) {
                if (it == 3) HCK(cudaEventRecord(e0, h->stream));
                st = spmv_enqueue(h, h->x_stage, h->y_stage, true, true);
                if (st != MX_OK) return st;
            }
            HCK(cudaEventRecord(e1, h->stream));
            HCK(cudaEventSynchronize(e1));
            float ms = 0;
            HCK(cudaEventElapsedTime(&ms, e0, e1));
            ms /= 10;
            if (i == 0) plain = ms;
            if (best < 0 || ms < best) {
                best = ms;
                bc = tc;
                br = tr;
            }
        }
    int st = mx_partition(h, bc, br, nullptr);
    if (st != MX_OK) return st;
    *tau_c = bc;
    *tau_r = br;
    if (ms_best) *ms_best = best;
    if (ms_plain) *ms_plain = plain;
    return MX_OK;
}

int mx_fragment_count_status(long long total_frags, int dtype) {
    if (dtype != MX_FP64 && dtype != MX_FP16) return MX_ERR_INVALID;
    return fragment_count_status(total_frags, frag_k(dtype));
}

int mx_dims(mx_handle_t h, int *n_rows, int *n_cols, int *nnz) {
    if (!h) return MX_ERR_INVALID;
    if (n_rows) *n_rows = h->n_rows;
    if (n_cols) *n_cols = h->n_cols;
    if (nnz) *nnz = h->nnz;
    return MX_OK;
}

int mx_partition_stats_get(mx_handle_t h, mx_partition_stats *stats) {
    if (!h || !stats) return MX_ERR_INVALID;
    if (!h->planned) return h->fail(MX_ERR_STATE, "no partition");
    *stats = h->stats;
    return MX_OK;
}

int mx_download_partition(mx_handle_t h, const mx_partition_arrays *o) {
    if (!h || !o) return MX_ERR_INVALID;
    if (!h->planned || !h->stats.active) return h->fail(MX_ERR_STATE, "mx_download_partition: no active partition");
    HCK(cudaSetDevice(h->device));
    const mx_partition_stats &s = h->stats;
    const size_t vb = val_bytes(h->dtype), bb = bit_bytes(h->dtype);
    const int K = s.fragK;
#define DL(dst, src, bytes)                                                                              \
    do {                                                                                                 \
        if ((dst) && (bytes) > 0) HCK(cudaMemcpyAsync((dst), (src), (bytes), cudaMemcpyDeviceToHost, h->stream)); \
    } while (0)
    DL(o->xperm, h->part.xperm, sizeof(int) * (size_t)h->n_cols);
    DL(o->rId, h->part.rId, sizeof(int) * (size_t)s.dRows);
    DL(o->rowPtr_dd, h->part.rowPtr_dd, sizeof(int) * ((size_t)s.dRows + 1));
    DL(o->colInd_dd, h->part.colInd_dd, sizeof(int) * (size_t)s.nnzRowD);
    DL(o->val_dd, h->part.val_dd, vb * (size_t)s.nnzRowD);
    DL(o->chunkPtr, h->part.tiles.chunkPtr, sizeof(int) * ((size_t)s.chunkNum + 1));
    DL(o->AToX, h->part.tiles.AToX, sizeof(int) * (size_t)s.totalFrags * K);
    DL(o->fragPtr, h->part.tiles.fragPtr, sizeof(int) * ((size_t)s.totalFrags + 1));
    DL(o->fragBit, h->part.tiles.fragBit, bb * (size_t)s.totalFrags);
    DL(o->tcVal, h->part.tiles.tcVal, vb * (size_t)s.nnzRowD);
    DL(o->rowPtr_CD, h->part.rowPtr_CD, sizeof(int) * ((size_t)h->n_rows + 1));
    DL(o->colInd_CD, h->part.colInd_CD, sizeof(int) * (size_t)s.nnzCD);
    DL(o->val_CD, h->part.val_CD, vb * (size_t)s.nnzCD);
#undef DL
    HCK(cudaStreamSynchronize(h->stream));
    return MX_OK;
}

int mx_spmv(mx_handle_t h, const void *x_dev, void *y_dev) {
    if (!h || !x_dev || !y_dev) return MX_ERR_INVALID;
    if (!h->planned) return h->fail(MX_ERR_STATE, "mx_spmv: call mx_partition first");
    HCK(cudaSetDevice(h->device));
    return spmv_enqueue(h, x_dev, y_dev, true, true);
}

int mx_spmv_peers(mx_handle_t h, const void *x_dev, void *const *y_peers, int n_peers, long long row_offset) {
    if (!h || !x_dev || !y_peers || n_peers < 1 || n_peers > 8 || row_offset < 0) return MX_ERR_INVALID;
    for (int g = 0; g < n_peers; ++g)
        if (!y_peers[g]) return MX_ERR_INVALID;
    if (!h->planned) return h->fail(MX_ERR_STATE, "mx_spmv_peers: call mx_partition first");
    HCK(cudaSetDevice(h->device));
    return spmv_enqueue(h, x_dev, nullptr, true, true, true, y_peers, n_peers, row_offset);
}

int mx_spmv_multicast(mx_handle_t h, const void *x_dev, void *const *y_peers, int n_peers, void *y_multicast,
                      long long row_offset) {
    if (!h || !x_dev || !y_peers || !y_multicast || n_peers < 1 || n_peers > 8 || row_offset < 0) return MX_ERR_INVALID;
    for (int g = 0; g < n_peers; ++g)
        if (!y_peers[g]) return MX_ERR_INVALID;
    if (((uintptr_t)y_multicast & 7u) != 0) return h->fail(MX_ERR_INVALID, "mx_spmv_multicast: address not 8-byte aligned");
    if (!h->planned) return h->fail(MX_ERR_STATE, "mx_spmv_multicast: call mx_partition first");
    HCK(cudaSetDevice(h->device));
    return spmv_enqueue(h, x_dev, nullptr, true, true, true, y_peers, n_peers, row_offset, y_multicast);
}

int mx_spmv_host(mx_handle_t h, const void *x_host, void *y_host) {
    if (!h || !x_host || !y_host) return MX_ERR_INVALID;
    if (!h->planned) return h->fail(MX_ERR_STATE, "mx_spmv_host: call mx_partition first");
    HCK(cudaSetDevice(h->device));
    if (h->copy_in) {  // pipelined products still in flight share the first pair of staging buffers: let them finish
        HCK(cudaStreamSynchronize(h->copy_in));
        HCK(cudaStreamSynchronize(h->stream));
        HCK(cudaStreamSynchronize(h->copy_out));
    }
    const size_t vb = val_bytes(h->dtype);
    HCK(cudaMemcpyAsync(h->x_stage, x_host, vb * (size_t)h->n_cols, cudaMemcpyHostToDevice, h->stream));
    int st = spmv_enqueue(h, h->x_stage, h->y_stage, true, true);
    if (st != MX_OK) return st;
    HCK(cudaMemcpyAsync(y_host, h->y_stage, vb * (size_t)h->n_rows, cudaMemcpyDeviceToHost, h->stream));
    HCK(cudaStreamSynchronize(h->stream));
    return MX_OK;
}

// Products with host buffers, pipelined: the copy of x in, the product and the copy of y out run on three streams
// over two sets of staging buffers, so the transfers of one product overlap the kernels of its neighbours.
int mx_spmv_host_async(mx_handle_t h, const void *x_host, void *y_host) {
    if (!h || !x_host || !y_host) return MX_ERR_INVALID;
    if (!h->planned) return h->fail(MX_ERR_STATE, "mx_spmv_host_async: call mx_partition first");
    HCK(cudaSetDevice(h->device));
    const size_t vb = val_bytes(h->dtype);
    const size_t xb = vb * (size_t)(h->n_cols > 0 ? h->n_cols : 1), yb = vb * (size_t)(h->n_rows > 0 ? h->n_rows : 1);
    if (!h->copy_in) {  // first use: the second buffer pair, the copy streams and the events
        HCK(cudaStreamSynchronize(h->stream));
        HCK(cudaMallocAsync(&h->x_stage2, xb, h->stream));
        HCK(cudaMallocAsync(&h->y_stage2, yb, h->stream));
        HCK(cudaStreamSynchronize(h->stream));
        for (int i = 0; i < 2; ++i) {
            HCK(cudaEventCreateWithFlags(&h->ev_in[i], cudaEventDisableTiming));
            HCK(cudaEventCreateWithFlags(&h->ev_done[i], cudaEventDisableTiming));
            HCK(cudaEventCreateWithFlags(&h->ev_out[i], cudaEventDisableTiming));
        }
        HCK(cudaStreamCreateWithFlags(&h->copy_out, cudaStreamNonBlocking));
        HCK(cudaStreamCreateWithFlags(&h->copy_in, cudaStreamNonBlocking));
    } else if (!h->x_stage2) {  // a new matrix was uploaded since
        HCK(cudaMallocAsync(&h->x_stage2, xb, h->stream));
        HCK(cudaMallocAsync(&h->y_stage2, yb, h->stream));
    }
    const int slot = (int)(h->async_calls & 1ull);
    const bool reuse = h->async_calls >= 2;  // the slot's previous product must have left it
    void *xs = slot ? h->x_stage2 : h->x_stage, *ys = slot ? h->y_stage2 : h->y_stage;
    if (h->async_calls < 2) {  // the buffers were allocated (or last used) on the compute stream
        HCK(cudaEventRecord(h->ev_done[slot], h->stream));
        HCK(cudaStreamWaitEvent(h->copy_in, h->ev_done[slot], 0));
    }
    if (reuse) HCK(cudaStreamWaitEvent(h->copy_in, h->ev_done[slot], 0));  // its product has read x
    HCK(cudaMemcpyAsync(xs, x_host, vb * (size_t)h->n_cols, cudaMemcpyHostToDevice, h->copy_in));
    HCK(cudaEventRecord(h->ev_in[slot], h->copy_in));
    HCK(cudaStreamWaitEvent(h->stream, h->ev_in[slot], 0));
    if (reuse) HCK(cudaStreamWaitEvent(h->stream, h->ev_out[slot], 0));  // its y has left the buffer
    int st = spmv_enqueue(h, xs, ys, true, true);
    if (st != MX_OK) return st;
    HCK(cudaEventRecord(h->ev_done[slot], h->stream));
    HCK(cudaStreamWaitEvent(h->copy_out, h->ev_done[slot], 0));
    HCK(cudaMemcpyAsync(y_host, ys, vb * (size_t)h->n_rows, cudaMemcpyDeviceToHost, h->copy_out));
    HCK(cudaEventRecord(h->ev_out[slot], h->copy_out));
    ++h->async_calls;
    return MX_OK;
}

int mx_host_sync(mx_handle_t h) {
    if (!h) return MX_ERR_INVALID;
    HCK(cudaSetDevice(h->device));
    if (h->copy_in) HCK(cudaStreamSynchronize(h->copy_in));
    HCK(cudaStreamSynchronize(h->stream));
    if (h->copy_out) HCK(cudaStreamSynchronize(h->copy_out));
    return MX_OK;
}

int mx_spmv_launches(mx_handle_t h) {
    if (!h || !h->planned) return 0;
    int n = resid_launches(h->resid);
    if (h->use_slabs) n = col_slabs_launches(h->slabs);
    if (h->stats.active)
        n += (h->use_orig_cols ? 0 : 1) + (h->dd_exec == MX_DD_TILE ? tile_launches(h->tile)
                                         : h->dd_exec == MX_DD_SE ? se_launches(h->se)
                                                                  : resid_launches(h->ddcsr));
    return n;
}

int mx_set_dd_executor(mx_handle_t h, int mode) {
    if (!h || mode < MX_DD_AUTO || mode > MX_DD_SE) return MX_ERR_INVALID;
    h->dd_mode = mode;
    if (h->planned && h->stats.active) {
        HCK(cudaSetDevice(h->device));
        HCK(cudaStreamSynchronize(h->stream));
        if (mode == MX_DD_AUTO || mode == MX_DD_SE) {
            int st = build_se_plan(h);
            if (st != MX_OK) return st;
            select_colspace(h, h->use_orig_cols, h->use_hot);
        }
        if (mode == MX_DD_AUTO) return tune_dd_executor(h);
        h->dd_exec = mode;
    }
    return MX_OK;
}

int mx_dd_executor_times(mx_handle_t h, float *ms_tile, float *ms_csr, float *ms_se) {
    if (!h) return MX_ERR_INVALID;
    if (ms_tile) *ms_tile = h->dd_ms[MX_DD_TILE];
    if (ms_csr) *ms_csr = h->dd_ms[MX_DD_CSR];
    if (ms_se) *ms_se = h->dd_ms[MX_DD_SE];
    return MX_OK;
}

int mx_set_column_space(mx_handle_t h, int mode) {
    if (!h || mode < MX_COLSPACE_AUTO || mode > MX_COLSPACE_ORIGINAL) return MX_ERR_INVALID;
    h->colspace_mode = mode;
    if (h->planned && h->stats.active) {
        HCK(cudaSetDevice(h->device));
        HCK(cudaStreamSynchronize(h->stream));
        return tune_colspace(h);
    }
    return MX_OK;
}

int mx_set_column_slabs(mx_handle_t h, int count) {
    if (!h || count < -1 || count == 1 || count > 64) return MX_ERR_INVALID;
    if (count > 0 && h->dtype != MX_FP64) return h->fail(MX_ERR_INVALID, "column slabs are available for FP64 only");
    h->slab_mode = count;
    if (h->planned && !h->stats.active) {
        HCK(cudaSetDevice(h->device));
        HCK(cudaStreamSynchronize(h->stream));
        col_slabs_free(h->slabs, h->stream);
        return tune_col_slabs(h);
    }
    return MX_OK;
}

int mx_set_row_offset(mx_handle_t h, long long first_global_row) {
    if (!h || first_global_row < 0) return MX_ERR_INVALID;
    h->row_offset = first_global_row;
    return MX_OK;
}

int mx_column_slabs(mx_handle_t h, int *count, float *ms_plain, float *ms_slabbed) {
    if (!h) return MX_ERR_INVALID;
    if (count) *count = h->use_slabs ? h->slabs.count : 0;
    if (ms_plain) *ms_plain = h->slab_ms_plain;
    if (ms_slabbed) *ms_slabbed = h->slab_ms_slabbed;
    return MX_OK;
}

int mx_set_hot_prefix(mx_handle_t h, int mode) {
    if (!h || mode < MX_HOT_AUTO || mode > MX_HOT_ON) return MX_ERR_INVALID;
    h->hot_mode = mode;
    if (h->planned && h->stats.active) {
        HCK(cudaSetDevice(h->device));
        HCK(cudaStreamSynchronize(h->stream));
        return tune_colspace(h);
    }
    return MX_OK;
}

int mx_hot_prefix(mx_handle_t h, int *hot_cols, float *ms_with, float *ms_without) {
    if (!h) return MX_ERR_INVALID;
    const bool on = h->planned && h->stats.active && h->use_hot;
    if (hot_cols) *hot_cols = on ? h->hot_budget : 0;
    if (ms_with) *ms_with = h->tune_ms_hot;
    if (ms_without) *ms_without = h->tune_ms_nohot;
    return MX_OK;
}

int mx_column_space(mx_handle_t h, float *ms_permuted, float *ms_original) {
    if (!h || !h->planned || !h->stats.active) return MX_COLSPACE_AUTO;
    if (ms_permuted) *ms_permuted = h->tune_ms_perm;
    if (ms_original) *ms_original = h->tune_ms_orig;
    return h->use_orig_cols ? MX_COLSPACE_ORIGINAL : MX_COLSPACE_PERMUTED;
}

int mx_dd_executor(mx_handle_t h) {
    if (!h || !h->planned || !h->stats.active) return MX_DD_AUTO;
    return h->dd_exec;
}

int mx_device_error(mx_handle_t h, int *err) {
    if (!h || !err) return MX_ERR_INVALID;
    HCK(cudaSetDevice(h->device));
    HCK(cudaMemcpyAsync(err, h->dev_err, sizeof(int), cudaMemcpyDeviceToHost, h->stream));
    HCK(cudaStreamSynchronize(h->stream));
    return MX_OK;
}

int mx_spmv_timed(mx_handle_t h, const void *x_dev, void *y_dev, int warm, int iters, float *ms_tile, float *ms_resid,
                  float *ms_total) {
    if (!h || !x_dev || !y_dev || warm < 0 || iters <= 0) return MX_ERR_INVALID;
    if (!h->planned) return h->fail(MX_ERR_STATE, "mx_spmv_timed: call mx_partition first");
    HCK(cudaSetDevice(h->device));
    EventPair ev;
    HCK(ev.create());
    const cudaEvent_t e0 = ev.e0, e1 = ev.e1;
    float out[3] = {0, 0, 0};
    for (int phase = 0; phase < 3; ++phase) {
        const bool do_tile = phase != 1, do_resid = phase != 0;
        if (phase == 0 && !h->stats.active) continue;
        for (int i = 0; i < warm + iters; ++i) {
            if (i == warm) HCK(cudaEventRecord(e0, h->stream));
            int st;
            if (phase == 2) {
                st = spmv_enqueue(h, x_dev, y_dev, true, true);
            } else if (h->stats.active) {
                // one half alone, on an x that is already permuted (the reference times its halves the same way)
                st = spmv_enqueue(h, x_dev, y_dev, do_tile, do_resid, /*permute=*/i == 0);
            } else {
                st = spmv_enqueue(h, x_dev, y_dev, false, true);
            }
            if (st != MX_OK) return st;
        }
        HCK(cudaEventRecord(e1, h->stream));
        HCK(cudaEventSynchronize(e1));
        float ms = 0;
        HCK(cudaEventElapsedTime(&ms, e0, e1));
        out[phase] = ms / iters;
    }
    if (ms_tile) *ms_tile = out[0];
    if (ms_resid) *ms_resid = out[1];
    if (ms_total) *ms_total = out[2];
    return MX_OK;
}

int mx_features(mx_handle_t h, mx_matrix_features *out) {
    if (!h || !out) return MX_ERR_INVALID;
    if (!h->has_matrix) return h->fail(MX_ERR_STATE, "mx_features: call mx_upload_csr first");
    HCK(cudaSetDevice(h->device));
    CsrDev A;
    A.n_rows = h->n_rows;
    A.n_cols = h->n_cols;
    A.nnz = h->nnz;
    A.row_ptr = h->row_ptr;
    A.col_ind = h->col_ind;
    A.val = h->val;
    HCK(matrix_features(A, *out, h->stream));
    return MX_OK;
}

int mx_csr_prefetch(mx_handle_t h, int *resid_tiles, int *dd_tiles) {
    if (!h) return MX_ERR_INVALID;
    if (!h->planned) return h->fail(MX_ERR_STATE, "mx_csr_prefetch: call mx_partition first");
    if (resid_tiles) *resid_tiles = h->resid.prefetch_tiles;
    if (dd_tiles) *dd_tiles = h->stats.active ? h->ddcsr.prefetch_tiles : 0;
    return MX_OK;
}

int mx_stream_gather_floor(mx_handle_t h, const void *x_dev, int warm, int iters, float *ms) {
    if (!h || !x_dev || !ms || warm < 0 || iters <= 0) return MX_ERR_INVALID;
    if (!h->has_matrix) return h->fail(MX_ERR_STATE, "mx_stream_gather_floor: call mx_upload_csr first");
    HCK(cudaSetDevice(h->device));
    float *sink = nullptr;
    HCK(cudaMallocAsync((void **)&sink, sizeof(float), h->stream));
    EventPair ev;
    cudaError_t e = ev.create();
    const cudaEvent_t e0 = ev.e0, e1 = ev.e1;
    for (int i = 0; e == cudaSuccess && i < warm + iters; ++i) {
        if (i == warm) e = cudaEventRecord(e0, h->stream);
        if (e == cudaSuccess) e = stream_gather_pass(h->dtype, h->col_ind, h->val, x_dev, sink, h->nnz, h->stream);
    }
    if (e == cudaSuccess) e = cudaEventRecord(e1, h->stream);
    if (e == cudaSuccess) e = cudaEventSynchronize(e1);
    float t = 0;
    if (e == cudaSuccess) e = cudaEventElapsedTime(&t, e0, e1);
    cudaFreeAsync(sink, h->stream);
    if (e != cudaSuccess) return h->cuda_fail(e, "mx_stream_gather_floor");
    *ms = t / iters;
    return MX_OK;
}

// ---------------------------------------------------------------------------------------------------
// Stateless mirrors of include/MatXtract.h.  Errors are reported as a status; the C++ shims turn a
// non-zero status into the reference's behaviour (message + exit).
// ---------------------------------------------------------------------------------------------------
#define SCK(call)                                                                           \
    do {                                                                                    \
        cudaError_t e_ = (call);                                                            \
        if (e_ != cudaSuccess) {                                                            \
            fprintf(stderr, "CUDA Error: %s at %s:%d\n", cudaGetErrorString(e_), __FILE__, __LINE__); \
            return MX_ERR_CUDA;                                                             \
        }                                                                                   \
    } while (0)


int mx_cdspmv(int dtype, const void *csrVal, const int *csrRowPtr, const int *csrColInd, const void *x, void *y,
              int rowA, int colA, int nnzA, int warm, int iters, double *ms_per_spmv, double *pre_ms) {
    if ((dtype != MX_FP64 && dtype != MX_FP16) || !csrRowPtr || !x || !y || rowA < 0 || colA < 0 || nnzA < 0 ||
        (nnzA > 0 && (!csrVal || !csrColInd)))
        return MX_ERR_INVALID;
    int st = check_device();
    if (st != MX_OK) return st;
    const size_t vb = val_bytes(dtype);
    DevBufs B;
    int *d_ptr, *d_ind;
    void *d_val, *d_x, *d_y, *d_scratch;
    SCK(B.up(&d_ptr, csrRowPtr, sizeof(int) * ((size_t)rowA + 1)));
    SCK(B.up(&d_ind, csrColInd, sizeof(int) * (size_t)nnzA));
    SCK(B.up(&d_val, csrVal, vb * (size_t)nnzA));
    SCK(B.up(&d_x, x, vb * (size_t)colA));
    SCK(B.up(&d_y, y, vb * (size_t)rowA));
    SCK(B.up(&d_scratch, nullptr, vb * (size_t)rowA));
    ResidPlan P;
    P.n_rows = rowA;
    P.n_cols = colA;
    P.nnz = nnzA;
    P.row_ptr = d_ptr;
    P.col_ind = d_ind;
    P.val = d_val;
    EventPair ev;
    SCK(ev.create());
    const cudaEvent_t e0 = ev.e0, e1 = ev.e1;
    SCK(cudaEventRecord(e0, 0));
    cudaError_t ce = resid_plan_build(dtype, P, 0);
    SCK(cudaEventRecord(e1, 0));
    SCK(cudaEventSynchronize(e1));
    float ms = 0;
    cudaEventElapsedTime(&ms, e0, e1);
    if (pre_ms) *pre_ms = ms;
    if (ce == cudaSuccess) {
        for (int i = 0; i < warm + iters && ce == cudaSuccess; ++i) {
            if (i == warm) cudaEventRecord(e0, 0);
            ce = resid_spmv(dtype, P, d_x, d_scratch, nullptr, nullptr, false, 0);
        }
        cudaEventRecord(e1, 0);
        cudaEventSynchronize(e1);
        cudaEventElapsedTime(&ms, e0, e1);
        if (ms_per_spmv) *ms_per_spmv = iters > 0 ? ms / iters : 0.0;
        if (ce == cudaSuccess) ce = resid_spmv(dtype, P, d_x, d_y, nullptr, nullptr, true, 0);  // y += A x
        if (ce == cudaSuccess) ce = cudaMemcpy(y, d_y, vb * (size_t)rowA, cudaMemcpyDeviceToHost);
    }
    resid_plan_free(P, 0);
    SCK(ce);
    return MX_OK;
}

static int run_tiles(int dtype, TileArrays &T, const void *d_x, void *d_y, void *d_scratch, int warm, int iters,
                     bool accumulate, double *ms_per_spmv) {
    TilePlan P;
    P.A = T;
    cudaError_t ce = tile_plan_build(dtype, P, 0);
    EventPair ev;
    SCK(ev.create());
    const cudaEvent_t e0 = ev.e0, e1 = ev.e1;
    for (int i = 0; i < warm + iters && ce == cudaSuccess; ++i) {
        if (i == warm) cudaEventRecord(e0, 0);
        ce = tile_spmv(dtype, P, d_x, d_scratch, nullptr, false, false, nullptr, 0);
    }
    if (iters > 0 && ce == cudaSuccess) {
        cudaEventRecord(e1, 0);
        cudaEventSynchronize(e1);
        float ms = 0;
        cudaEventElapsedTime(&ms, e0, e1);
        if (ms_per_spmv) *ms_per_spmv = ms / iters;
    }
    if (ce == cudaSuccess) ce = tile_spmv(dtype, P, d_x, d_y, nullptr, false, accumulate, nullptr, 0);
    if (ce == cudaSuccess) ce = cudaDeviceSynchronize();
    tile_plan_free(P, 0);
    SCK(ce);
    return MX_OK;
}

int mx_du_tcspmv(int dtype, const int *chunkPtr, const int *fragPtr, const void *fragBit, const void *tcVal,
                 int n_vals, const int *AToX, const void *x, void *y, int dRows, int dCols, int warm, int iters,
                 double *ms_per_spmv) {
    if ((dtype != MX_FP64 && dtype != MX_FP16) || !chunkPtr || !fragPtr || !x || !y || dRows < 0 || dCols < 0 ||
        n_vals < 0)
        return MX_ERR_INVALID;
    int st = check_device();
    if (st != MX_OK) return st;
    const size_t vb = val_bytes(dtype);
    const int K = frag_k(dtype);
    const int chunkNum = (dRows + 7) / 8;
    const int totalFrags = chunkPtr[chunkNum];
    if (totalFrags > 0 && (!fragBit || !AToX)) return MX_ERR_INVALID;
    if (n_vals > 0 && !tcVal) return MX_ERR_INVALID;
    DevBufs B;
    TileArrays T;
    T.dRows = dRows;
    T.dCols = dCols;
    T.chunkNum = chunkNum;
    T.totalFrags = totalFrags;
    T.nvals = n_vals;
    void *d_x, *d_y, *d_scratch;
    SCK(B.up(&T.chunkPtr, chunkPtr, sizeof(int) * ((size_t)chunkNum + 1)));
    SCK(B.up(&T.fragPtr, fragPtr, sizeof(int) * ((size_t)totalFrags + 1)));
    SCK(B.up(&T.fragBit, fragBit, bit_bytes(dtype) * (size_t)totalFrags));
    SCK(B.up(&T.tcVal, tcVal, vb * (size_t)n_vals));
    SCK(B.up(&T.AToX, AToX, sizeof(int) * (size_t)totalFrags * K));
    SCK(B.up(&d_x, x, vb * (size_t)dCols));
    SCK(B.up(&d_y, y, vb * (size_t)dRows));
    SCK(B.up(&d_scratch, nullptr, vb * (size_t)dRows));
    // FP64: the reference preloads y and adds to it; FP16: y is zeroed and stored
    st = run_tiles(dtype, T, d_x, d_y, d_scratch, warm, iters, dtype == MX_FP64, ms_per_spmv);
    if (st != MX_OK) return st;
    SCK(cudaMemcpy(y, d_y, vb * (size_t)dRows, cudaMemcpyDeviceToHost));
    return MX_OK;
}

int mx_se_tcspmv(int dtype, const void *csrVal, const int *csrRowPtr, const int *csrColIdx, const void *x, void *y,
                 int *order_rid, int rowA, int colA, int nnzA, int NUM, double threshold, int block_longest, int warm,
                 int iters, double *ms_per_spmv) {
    if ((dtype != MX_FP64 && dtype != MX_FP16) || !csrRowPtr || !x || !y || !order_rid || rowA < 0 || colA < 0 ||
        nnzA < 0 || (nnzA > 0 && (!csrVal || !csrColIdx)))
        return MX_ERR_INVALID;
    int st = check_device();
    if (st != MX_OK) return st;
    const size_t vb = val_bytes(dtype);
    DevBufs B;
    int *d_ptr, *d_ind;
    void *d_val, *d_x, *d_y;
    SCK(B.up(&d_ptr, csrRowPtr, sizeof(int) * ((size_t)rowA + 1)));
    SCK(B.up(&d_ind, csrColIdx, sizeof(int) * (size_t)nnzA));
    SCK(B.up(&d_val, csrVal, vb * (size_t)nnzA));
    SCK(B.up(&d_x, x, vb * (size_t)colA));
    SCK(B.up(&d_y, nullptr, vb * (size_t)rowA));
    SePlan P;
    P.n_rows = rowA;
    P.n_cols = colA;
    P.nnz = nnzA;
    if (NUM > 0) P.warps_per_cta = NUM;
    if (threshold >= 0.0) P.threshold = threshold;
    if (block_longest > 0) P.block_longest = block_longest;
    cudaError_t ce = se_plan_build(dtype, P, d_ptr, d_ind, d_val, nullptr, 0);
    EventPair ev;
    if (ce == cudaSuccess) ce = ev.create();
    for (int i = 0; i < warm + iters && ce == cudaSuccess; ++i) {
        if (i == warm) cudaEventRecord(ev.e0, 0);
        ce = se_spmv(dtype, P, d_x, d_y, false, false, 0);
    }
    if (iters > 0 && ce == cudaSuccess) {
        cudaEventRecord(ev.e1, 0);
        cudaEventSynchronize(ev.e1);
        float ms = 0;
        cudaEventElapsedTime(&ms, ev.e0, ev.e1);
        if (ms_per_spmv) *ms_per_spmv = ms / iters;
    }
    // Y_val[i] is the result of input row order_rid[i]: rows leave in the layout's length-sorted order
    if (ce == cudaSuccess) ce = se_spmv(dtype, P, d_x, d_y, false, false, 0);
    if (ce == cudaSuccess && rowA > 0) ce = cudaMemcpy(y, d_y, vb * (size_t)rowA, cudaMemcpyDeviceToHost);
    if (ce == cudaSuccess && rowA > 0) ce = cudaMemcpy(order_rid, P.order, sizeof(int) * (size_t)rowA, cudaMemcpyDeviceToHost);
    se_plan_free(P, 0);
    cudaDeviceSynchronize();
    SCK(ce);
    return MX_OK;
}

}  // extern "C"
