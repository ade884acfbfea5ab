// Multi-GPU entry of the C ABI: one process drives the GPUs of one box (see include/mx_capi.h, "multi-GPU").
//
// The reference is single-GPU.  Rows are cut into contiguous slabs of equal non-zero count, one per GPU; x is
// replicated; every GPU extracts and multiplies its own slab through an ordinary handle; y is assembled in every
// GPU's full-length buffer either by the kernels themselves (the fused epilogue / push of mx_spmv_peers: peer stores
// over NVLink) followed by an event barrier, or by NCCL broadcasts of the slabs.  Nothing spins: GPUs wait on each
// other's CUDA events in stream order.  NCCL is bound at run time (dlopen) so that a process that already carries an
// NCCL — torch does — keeps using its own copy.
#include <dlfcn.h>
#include <nccl.h>

#include <algorithm>
#include <string>
#include <vector>

#include "mx_internal.h"

namespace {

constexpr int MG_MAX = 8;

struct NcclApi {
    void *lib = nullptr;
    ncclResult_t (*CommInitAll)(ncclComm_t *, int, const int *) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*GroupStart)() = nullptr;
    ncclResult_t (*GroupEnd)() = nullptr;
    ncclResult_t (*Broadcast)(const void *, void *, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    bool load() {
        if (lib) return true;
        lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_LOCAL);
        if (!lib) return false;
        CommInitAll = reinterpret_cast<decltype(CommInitAll)>(dlsym(lib, "ncclCommInitAll"));
        CommDestroy = reinterpret_cast<decltype(CommDestroy)>(dlsym(lib, "ncclCommDestroy"));
        GroupStart = reinterpret_cast<decltype(GroupStart)>(dlsym(lib, "ncclGroupStart"));
        GroupEnd = reinterpret_cast<decltype(GroupEnd)>(dlsym(lib, "ncclGroupEnd"));
        Broadcast = reinterpret_cast<decltype(Broadcast)>(dlsym(lib, "ncclBroadcast"));
        return CommInitAll && CommDestroy && GroupStart && GroupEnd && Broadcast;
    }
};

}  // namespace

struct mx_mg_s {
    int n = 0, dtype = MX_FP64;
    int dev[MG_MAX] = {};
    mx_handle_t h[MG_MAX] = {};
    int n_rows = 0, n_cols = 0;
    long long nnz = 0;
    std::vector<int> bounds;        // [n+1]
    void *x[MG_MAX] = {};           // x replica of every GPU
    void *y[MG_MAX][2] = {};        // full-length y of every GPU, two alternating buffers
    int turn = 0;                   // buffer the next product writes
    cudaEvent_t done[MG_MAX] = {};  // this GPU's part of the current product has been issued and finished
    cudaEvent_t t0[MG_MAX] = {}, t1[MG_MAX] = {};
    int exchange = MX_MG_EXCHANGE_PEER;
    bool peer_ok = true;
    NcclApi nccl;
    ncclComm_t comm[MG_MAX] = {};
    bool has_comm = false;
    bool ready = false;
    int local_ranking = 0;  // 1: every slab ranks its own columns and rows instead of the whole matrix's
    std::string err;
    int fail(int st, const std::string &m) {
        err = m;
        return st;
    }
};

__global__ void k_mg_add(int *__restrict__ a, const int *__restrict__ b, int n) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) a[i] += b[i];
}

#define MGCK(call)                                                                      \
    do {                                                                                \
        cudaError_t e_ = (call);                                                        \
        if (e_ != cudaSuccess) return mg->fail(MX_ERR_CUDA, std::string(#call) + ": " + cudaGetErrorString(e_)); \
    } while (0)

static void mg_release_buffers(mx_mg_t mg) {
    for (int g = 0; g < mg->n; ++g) {
        cudaSetDevice(mg->dev[g]);
        if (mg->h[g]) mx_sync(mg->h[g]);
        for (void *p : {mg->x[g], mg->y[g][0], mg->y[g][1]})
            if (p) cudaFree(p);
        mg->x[g] = mg->y[g][0] = mg->y[g][1] = nullptr;
    }
    mg->ready = false;
}

// every GPU's stream waits until all GPUs have finished their part of the current product
static int mg_barrier(mx_mg_t mg) {
    for (int g = 0; g < mg->n; ++g) {
        MGCK(cudaSetDevice(mg->dev[g]));
        MGCK(cudaEventRecord(mg->done[g], (cudaStream_t)mx_stream(mg->h[g])));
    }
    for (int g = 0; g < mg->n; ++g) {
        MGCK(cudaSetDevice(mg->dev[g]));
        for (int p = 0; p < mg->n; ++p)
            if (p != g) MGCK(cudaStreamWaitEvent((cudaStream_t)mx_stream(mg->h[g]), mg->done[p], 0));
    }
    return MX_OK;
}

// one product on the device-resident x replicas; the result is complete in y[g][turn] of every GPU once every stream
// has passed the barrier that ends the call
static int mg_enqueue(mx_mg_t mg) {
    const int k = mg->turn;
    const size_t vb = mx::val_bytes(mg->dtype);
    void *peers[MG_MAX];
    for (int g = 0; g < mg->n; ++g) peers[g] = mg->y[g][k];
    if (mg->n == 1) {
        int st = mx_spmv(mg->h[0], mg->x[0], mg->y[0][k]);
        if (st != MX_OK) return mg->fail(st, mx_last_error_string(mg->h[0]));
    } else if (mg->exchange == MX_MG_EXCHANGE_PEER) {
        for (int g = 0; g < mg->n; ++g) {  // rows leave the kernels for every GPU's buffer
            int st = mx_spmv_peers(mg->h[g], mg->x[g], peers, mg->n, mg->bounds[g]);
            if (st != MX_OK) return mg->fail(st, mx_last_error_string(mg->h[g]));
        }
        int st = mg_barrier(mg);
        if (st != MX_OK) return st;
    } else {
        for (int g = 0; g < mg->n; ++g) {  // own rows into the own buffer, then NCCL moves the slabs
            int st = mx_spmv(mg->h[g], mg->x[g], static_cast<char *>(mg->y[g][k]) + (size_t)mg->bounds[g] * vb);
            if (st != MX_OK) return mg->fail(st, mx_last_error_string(mg->h[g]));
        }
        const ncclDataType_t dt = mg->dtype == MX_FP64 ? ncclFloat64 : ncclFloat16;
        if (mg->nccl.GroupStart() != ncclSuccess) return mg->fail(MX_ERR_CUDA, "ncclGroupStart failed");
        for (int root = 0; root < mg->n; ++root) {
            const size_t count = (size_t)(mg->bounds[root + 1] - mg->bounds[root]);
            if (count == 0) continue;
            for (int g = 0; g < mg->n; ++g) {
                void *buf = static_cast<char *>(mg->y[g][k]) + (size_t)mg->bounds[root] * vb;
                if (mg->nccl.Broadcast(buf, buf, count, dt, root, mg->comm[g], (cudaStream_t)mx_stream(mg->h[g])) !=
                    ncclSuccess)
                    return mg->fail(MX_ERR_CUDA, "ncclBroadcast failed");
            }
        }
        if (mg->nccl.GroupEnd() != ncclSuccess) return mg->fail(MX_ERR_CUDA, "ncclGroupEnd failed");
        int st = mg_barrier(mg);  // a buffer is not rewritten before every GPU is past this product
        if (st != MX_OK) return st;
    }
    mg->turn ^= 1;
    return MX_OK;
}

extern "C" {

int mx_mg_partition_rows(const int *row_ptr, int n_rows, int n_parts, int *bounds) {
    if (!row_ptr || !bounds || n_rows < 0 || n_parts < 1) return MX_ERR_INVALID;
    const long long nnz = row_ptr[n_rows];
    bounds[0] = 0;
    for (int g = 1; g < n_parts; ++g) {
        const long long target = nnz * g / n_parts;
        const int *p = std::lower_bound(row_ptr, row_ptr + n_rows + 1, target,
                                        [](int v, long long t) { return (long long)v < t; });
        bounds[g] = std::max(bounds[g - 1], (int)std::min<long long>(p - row_ptr, n_rows));
    }
    bounds[n_parts] = n_rows;
    return MX_OK;
}

int mx_mg_create(mx_mg_t *out, int n_devices, const int *devices, int dtype) {
    if (!out || n_devices < 1 || n_devices > MG_MAX || (dtype != MX_FP64 && dtype != MX_FP16)) return MX_ERR_INVALID;
    *out = nullptr;
    int avail = 0;
    if (cudaGetDeviceCount(&avail) != cudaSuccess || avail <= 0) {
        cudaGetLastError();
        return MX_ERR_NO_DEVICE;
    }
    mx_mg_t mg = new mx_mg_s;
    mg->n = n_devices;
    mg->dtype = dtype;
    for (int g = 0; g < n_devices; ++g) {
        mg->dev[g] = devices ? devices[g] : g;
        if (mg->dev[g] < 0 || mg->dev[g] >= avail) {
            delete mg;
            return MX_ERR_INVALID;
        }
        for (int p = 0; p < g; ++p)
            if (mg->dev[p] == mg->dev[g]) {  // kernels of two slabs must never wait on each other on one GPU
                delete mg;
                return MX_ERR_INVALID;
            }
    }
    int st = MX_OK;
    for (int g = 0; g < n_devices && st == MX_OK; ++g) {
        st = mx_create(&mg->h[g], mg->dev[g], dtype);
        if (st != MX_OK) break;
        cudaSetDevice(mg->dev[g]);
        if (cudaEventCreateWithFlags(&mg->done[g], cudaEventDisableTiming) != cudaSuccess ||
            cudaEventCreate(&mg->t0[g]) != cudaSuccess || cudaEventCreate(&mg->t1[g]) != cudaSuccess)
            st = MX_ERR_CUDA;
        for (int p = 0; p < n_devices && st == MX_OK; ++p) {
            if (p == g) continue;
            int can = 0;
            const int pd = devices ? devices[p] : p;
            cudaDeviceCanAccessPeer(&can, mg->dev[g], pd);
            if (!can) {
                mg->peer_ok = false;
                continue;
            }
            cudaError_t e = cudaDeviceEnablePeerAccess(pd, 0);
            if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) mg->peer_ok = false;
            cudaGetLastError();
        }
    }
    if (st != MX_OK) {
        mx_mg_destroy(mg);
        return st;
    }
    if (!mg->peer_ok && n_devices > 1) {
        st = mx_mg_set_exchange(mg, MX_MG_EXCHANGE_NCCL);
        if (st != MX_OK) {
            mx_mg_destroy(mg);
            return st;
        }
    }
    *out = mg;
    return MX_OK;
}

int mx_mg_destroy(mx_mg_t mg) {
    if (!mg) return MX_ERR_INVALID;
    mg_release_buffers(mg);
    if (mg->has_comm)
        for (int g = 0; g < mg->n; ++g)
            if (mg->comm[g]) mg->nccl.CommDestroy(mg->comm[g]);
    for (int g = 0; g < mg->n; ++g) {
        cudaSetDevice(mg->dev[g]);
        for (cudaEvent_t e : {mg->done[g], mg->t0[g], mg->t1[g]})
            if (e) cudaEventDestroy(e);
        if (mg->h[g]) mx_destroy(mg->h[g]);
    }
    delete mg;
    return MX_OK;
}

const char *mx_mg_last_error_string(mx_mg_t mg) { return mg ? mg->err.c_str() : "null handle"; }

int mx_mg_set_exchange(mx_mg_t mg, int mode) {
    if (!mg || (mode != MX_MG_EXCHANGE_PEER && mode != MX_MG_EXCHANGE_NCCL)) return MX_ERR_INVALID;
    if (mode == MX_MG_EXCHANGE_PEER && !mg->peer_ok && mg->n > 1)
        return mg->fail(MX_ERR_STATE, "the GPUs of this handle cannot address each other's memory");
    if (mode == MX_MG_EXCHANGE_NCCL && mg->n > 1 && !mg->has_comm) {
        if (!mg->nccl.load()) return mg->fail(MX_ERR_STATE, "libnccl.so.2 could not be loaded");
        if (mg->nccl.CommInitAll(mg->comm, mg->n, mg->dev) != ncclSuccess)
            return mg->fail(MX_ERR_CUDA, "ncclCommInitAll failed");
        mg->has_comm = true;
    }
    mg->exchange = mode;
    return MX_OK;
}

int mx_mg_upload_csr(mx_mg_t mg, int n_rows, int n_cols, int nnz, const int *row_ptr, const int *col_ind,
                     const void *val) {
    if (!mg) return MX_ERR_INVALID;
    if (n_rows < 0 || n_cols < 0 || nnz < 0 || !row_ptr || (nnz > 0 && (!col_ind || !val)) || row_ptr[0] != 0 ||
        row_ptr[n_rows] != nnz)
        return mg->fail(MX_ERR_INVALID, "mx_mg_upload_csr: bad sizes or null arrays");
    mg_release_buffers(mg);
    mg->bounds.assign((size_t)mg->n + 1, 0);
    mx_mg_partition_rows(row_ptr, n_rows, mg->n, mg->bounds.data());
    mg->n_rows = n_rows;
    mg->n_cols = n_cols;
    mg->nnz = nnz;
    const size_t vb = mx::val_bytes(mg->dtype);
    std::vector<int> rp;
    for (int g = 0; g < mg->n; ++g) {
        const int r0 = mg->bounds[g], r1 = mg->bounds[g + 1], lo = row_ptr[r0], hi = row_ptr[r1];
        rp.resize((size_t)(r1 - r0) + 1);
        for (int r = r0; r <= r1; ++r) rp[(size_t)(r - r0)] = row_ptr[r] - lo;
        int st = mx_upload_csr(mg->h[g], r1 - r0, n_cols, hi - lo, rp.data(), col_ind ? col_ind + lo : nullptr,
                               val ? static_cast<const char *>(val) + (size_t)lo * vb : nullptr);
        if (st != MX_OK) return mg->fail(st, mx_last_error_string(mg->h[g]));
        mx_set_row_offset(mg->h[g], r0);
        MGCK(cudaSetDevice(mg->dev[g]));
        MGCK(cudaMalloc(&mg->x[g], vb * (size_t)std::max(n_cols, 1)));
        for (int k = 0; k < 2; ++k) {
            MGCK(cudaMalloc(&mg->y[g][k], vb * (size_t)std::max(n_rows, 1)));
            MGCK(cudaMemset(mg->y[g][k], 0, vb * (size_t)std::max(n_rows, 1)));
        }
    }
    return MX_OK;
}

// Extraction with the rankings of the whole matrix: column counts summed over the GPUs, per-row counts inside the hot
// columns gathered in row order, one cut for all.
static int mg_partition_global(mx_mg_t mg, double tau_c, double tau_r, mx_partition_stats *per_device) {
    const int n = mg->n;
    const size_t cbytes = sizeof(int) * (size_t)std::max(mg->n_cols, 1), rbytes = sizeof(int) * (size_t)std::max(mg->n_rows, 1);
    int *cnt[MG_MAX] = {}, *rowcnt[MG_MAX] = {}, *tmp0 = nullptr, *rows0 = nullptr;
    struct Cleanup {
        mx_mg_t mg;
        int **a, **b, **c, **d;
        ~Cleanup() {
            for (int g = 0; g < mg->n; ++g) {
                cudaSetDevice(mg->dev[g]);
                if (a[g]) cudaFree(a[g]);
                if (b[g]) cudaFree(b[g]);
            }
            cudaSetDevice(mg->dev[0]);
            if (*c) cudaFree(*c);
            if (*d) cudaFree(*d);
        }
    } cleanup{mg, cnt, rowcnt, &tmp0, &rows0};
    for (int g = 0; g < n; ++g) {  // 1. local column histograms
        MGCK(cudaSetDevice(mg->dev[g]));
        MGCK(cudaMalloc(&cnt[g], cbytes));
        MGCK(cudaMalloc(&rowcnt[g], sizeof(int) * (size_t)std::max(mg->bounds[g + 1] - mg->bounds[g], 1)));
        int st = mx_col_counts(mg->h[g], cnt[g]);
        if (st != MX_OK) return mg->fail(st, mx_last_error_string(mg->h[g]));
    }
    MGCK(cudaSetDevice(mg->dev[0]));  //    summed on GPU 0, the sum copied back to every GPU
    MGCK(cudaMalloc(&tmp0, cbytes));
    MGCK(cudaMalloc(&rows0, rbytes));
    for (int g = 1; g < n; ++g) {
        MGCK(cudaMemcpyPeer(tmp0, mg->dev[0], cnt[g], mg->dev[g], cbytes));
        k_mg_add<<<(mg->n_cols + 255) / 256, 256>>>(cnt[0], tmp0, mg->n_cols);
        MGCK(cudaGetLastError());
    }
    MGCK(cudaDeviceSynchronize());
    for (int g = 1; g < n; ++g) MGCK(cudaMemcpyPeer(cnt[g], mg->dev[g], cnt[0], mg->dev[0], cbytes));
    for (int g = 0; g < n; ++g) {  // the copies have landed before any handle's own stream reads them
        MGCK(cudaSetDevice(mg->dev[g]));
        MGCK(cudaDeviceSynchronize());
    }
    for (int g = 0; g < n; ++g) {  // 2. per-row counts inside the hot columns, gathered in row order on GPU 0
        int st = mx_row_counts_in_hot_columns(mg->h[g], tau_c, cnt[g], mg->nnz, rowcnt[g]);
        if (st != MX_OK) return mg->fail(st, mx_last_error_string(mg->h[g]));
        const size_t rows = (size_t)(mg->bounds[g + 1] - mg->bounds[g]);
        if (rows > 0) MGCK(cudaMemcpyPeer(rows0 + mg->bounds[g], mg->dev[0], rowcnt[g], mg->dev[g], sizeof(int) * rows));
    }
    MGCK(cudaSetDevice(mg->dev[0]));
    MGCK(cudaDeviceSynchronize());
    // 3. the row cut of the whole matrix (threshold computed like the reference: int * float, truncated)
    const int threshold = (int)mg->nnz * (float)tau_r;
    long long cut[4] = {0, 0, 0, 0};
    int st = mx_rank_cut(mg->h[0], rows0, mg->n_rows, threshold, cut);
    if (st != MX_OK) return mg->fail(st, mx_last_error_string(mg->h[0]));
    if (cut[0] == 0) return mg->fail(MX_ERR_TAU, "tau_r threshold never reached by the ranking prefix");
    for (int g = 0; g < n; ++g) {  // 4. every slab extracts with the whole matrix's rankings
        st = mx_partition_global(mg->h[g], tau_c, tau_r, cnt[g], mg->nnz, (int)cut[2], cut[3], mg->bounds[g],
                                 per_device ? per_device + g : nullptr);
        if (st != MX_OK) return mg->fail(st, mx_last_error_string(mg->h[g]));
    }
    return MX_OK;
}

int mx_mg_partition(mx_mg_t mg, double tau_c, double tau_r, mx_partition_stats *per_device) {
    if (!mg) return MX_ERR_INVALID;
    if (mg->bounds.empty()) return mg->fail(MX_ERR_STATE, "mx_mg_partition: no matrix uploaded");
    if (tau_c < tau_r) return mg->fail(MX_ERR_TAU, "col_frac must be greater than hot_frac");
    const bool inactive = (float)tau_c == 0.0f && (float)tau_r == 0.0f;
    if (mg->n > 1 && !inactive && mg->local_ranking == 0) {
        int st = mg_partition_global(mg, tau_c, tau_r, per_device);
        if (st != MX_OK) return st;
    } else {
        for (int g = 0; g < mg->n; ++g) {
            int st = mx_partition(mg->h[g], tau_c, tau_r, per_device ? per_device + g : nullptr);
            if (st != MX_OK) return mg->fail(st, mx_last_error_string(mg->h[g]));
        }
    }
    mg->ready = true;
    return MX_OK;
}

int mx_mg_set_local_ranking(mx_mg_t mg, int on) {
    if (!mg) return MX_ERR_INVALID;
    mg->local_ranking = on ? 1 : 0;
    return MX_OK;
}

int mx_mg_bounds(mx_mg_t mg, int *bounds) {
    if (!mg || !bounds || mg->bounds.empty()) return MX_ERR_INVALID;
    std::copy(mg->bounds.begin(), mg->bounds.end(), bounds);
    return MX_OK;
}

int mx_mg_devices(mx_mg_t mg) { return mg ? mg->n : 0; }
mx_handle_t mx_mg_handle(mx_mg_t mg, int g) { return (mg && g >= 0 && g < mg->n) ? mg->h[g] : nullptr; }

int mx_mg_spmv(mx_mg_t mg, const void *x_host, void *y_host) {
    if (!mg || !x_host || !y_host) return MX_ERR_INVALID;
    if (!mg->ready) return mg->fail(MX_ERR_STATE, "mx_mg_spmv: call mx_mg_upload_csr and mx_mg_partition first");
    const size_t vb = mx::val_bytes(mg->dtype);
    for (int g = 0; g < mg->n; ++g) {
        MGCK(cudaSetDevice(mg->dev[g]));
        MGCK(cudaMemcpyAsync(mg->x[g], x_host, vb * (size_t)mg->n_cols, cudaMemcpyHostToDevice,
                             (cudaStream_t)mx_stream(mg->h[g])));
    }
    const int k = mg->turn;
    int st = mg_enqueue(mg);
    if (st != MX_OK) return st;
    MGCK(cudaSetDevice(mg->dev[0]));
    MGCK(cudaMemcpyAsync(y_host, mg->y[0][k], vb * (size_t)mg->n_rows, cudaMemcpyDeviceToHost,
                         (cudaStream_t)mx_stream(mg->h[0])));
    for (int g = 0; g < mg->n; ++g) {
        st = mx_sync(mg->h[g]);
        if (st != MX_OK) return mg->fail(st, mx_last_error_string(mg->h[g]));
    }
    return MX_OK;
}

int mx_mg_download_y(mx_mg_t mg, int g, void *y_host) {
    if (!mg || !y_host || g < 0 || g >= mg->n) return MX_ERR_INVALID;
    if (!mg->ready) return mg->fail(MX_ERR_STATE, "mx_mg_download_y: nothing computed yet");
    MGCK(cudaSetDevice(mg->dev[g]));
    for (int p = 0; p < mg->n; ++p) mx_sync(mg->h[p]);
    MGCK(cudaMemcpy(y_host, mg->y[g][mg->turn ^ 1], mx::val_bytes(mg->dtype) * (size_t)mg->n_rows,
                    cudaMemcpyDeviceToHost));
    return MX_OK;
}

int mx_mg_spmv_timed(mx_mg_t mg, const void *x_host, int warm, int iters, float *ms_per_spmv) {
    if (!mg || !x_host || warm < 0 || iters <= 0 || !ms_per_spmv) return MX_ERR_INVALID;
    if (!mg->ready) return mg->fail(MX_ERR_STATE, "mx_mg_spmv_timed: call mx_mg_upload_csr and mx_mg_partition first");
    const size_t vb = mx::val_bytes(mg->dtype);
    for (int g = 0; g < mg->n; ++g) {
        MGCK(cudaSetDevice(mg->dev[g]));
        MGCK(cudaMemcpyAsync(mg->x[g], x_host, vb * (size_t)mg->n_cols, cudaMemcpyHostToDevice,
                             (cudaStream_t)mx_stream(mg->h[g])));
    }
    for (int i = 0; i < warm + iters; ++i) {
        if (i == warm) {
            int st = mg_barrier(mg);  // all GPUs start the timed region together
            if (st != MX_OK) return st;
            for (int g = 0; g < mg->n; ++g) {
                MGCK(cudaSetDevice(mg->dev[g]));
                MGCK(cudaEventRecord(mg->t0[g], (cudaStream_t)mx_stream(mg->h[g])));
            }
        }
        int st = mg_enqueue(mg);
        if (st != MX_OK) return st;
    }
    float worst = 0.f;
    for (int g = 0; g < mg->n; ++g) {
        MGCK(cudaSetDevice(mg->dev[g]));
        MGCK(cudaEventRecord(mg->t1[g], (cudaStream_t)mx_stream(mg->h[g])));
    }
    for (int g = 0; g < mg->n; ++g) {
        MGCK(cudaSetDevice(mg->dev[g]));
        MGCK(cudaEventSynchronize(mg->t1[g]));
        float ms = 0.f;
        MGCK(cudaEventElapsedTime(&ms, mg->t0[g], mg->t1[g]));
        worst = std::max(worst, ms);
    }
    *ms_per_spmv = worst / iters;  // device time, the slowest GPU
    return MX_OK;
}

}  // extern "C"
