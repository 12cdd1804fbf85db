// Multi-GPU layer behind the C ABI: one host thread drives several devices of one node.
//
// The reference is single-GPU.  Its products shard without any data-path exchange -- dense
// GEMM by row blocks of A and C with B replicated, batched GEMM by pages, CSR x dense by CSR
// row ranges with B replicated -- so a sharded call is one launch of the single-GPU kernel per
// device, each on that device's own stream, and nothing else.  A collective runs only when the
// caller asks for the result assembled: NCCL over NVLink (grouped broadcasts of the shards for
// "every device gets all rows", grouped send / receive for "the first device gets all rows"),
// and for the one-off replication of B.  NCCL is loaded at run time (dlopen) the first time a
// collective is needed, so the library has no link-time dependency on it and single-GPU users
// never touch it.
//
// Everything is asynchronous on the context's per-device streams; klas_b200_mg_synchronize
// waits for all of them.
#include <dlfcn.h>

#include <algorithm>
#include <mutex>
#include <vector>

#include "klas_internal.h"

// ---- the few NCCL declarations used, so that building needs no NCCL header -------------------
extern "C" {
typedef struct ncclComm *klas_nccl_comm;
typedef int klas_nccl_result;          // ncclSuccess == 0
constexpr int KLAS_NCCL_INT8 = 0;      // ncclInt8 / ncclChar
}

namespace klas {
namespace mg {

struct Nccl {
    void *handle = nullptr;
    klas_nccl_result (*CommInitAll)(klas_nccl_comm *, int, const int *) = nullptr;
    klas_nccl_result (*CommDestroy)(klas_nccl_comm) = nullptr;
    klas_nccl_result (*GroupStart)() = nullptr;
    klas_nccl_result (*GroupEnd)() = nullptr;
    klas_nccl_result (*Broadcast)(const void *, void *, size_t, int, int, klas_nccl_comm, cudaStream_t) = nullptr;
    klas_nccl_result (*Send)(const void *, size_t, int, int, klas_nccl_comm, cudaStream_t) = nullptr;
    klas_nccl_result (*Recv)(void *, size_t, int, int, klas_nccl_comm, cudaStream_t) = nullptr;
    const char *(*GetErrorString)(klas_nccl_result) = nullptr;
    bool ok = false;
};

static std::mutex g_nccl_mutex;
static Nccl g_nccl;

static int load_nccl(Nccl **out) {
    std::lock_guard<std::mutex> lock(g_nccl_mutex);
    if (!g_nccl.ok) {
        for (const char *name : {"libnccl.so.2", "libnccl.so"}) {
            g_nccl.handle = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
            if (g_nccl.handle) break;
        }
        if (!g_nccl.handle) return fail(KLAS_ERR_UNSUPPORTED, "multi-GPU gather needs NCCL: libnccl.so.2 could not be loaded (%s)", dlerror());
#define KLAS_NCCL_SYM(field, name)                                                            \
    g_nccl.field = reinterpret_cast<decltype(g_nccl.field)>(dlsym(g_nccl.handle, name));      \
    if (!g_nccl.field) return fail(KLAS_ERR_UNSUPPORTED, "NCCL library lacks %s", name)
        KLAS_NCCL_SYM(CommInitAll, "ncclCommInitAll");
        KLAS_NCCL_SYM(CommDestroy, "ncclCommDestroy");
        KLAS_NCCL_SYM(GroupStart, "ncclGroupStart");
        KLAS_NCCL_SYM(GroupEnd, "ncclGroupEnd");
        KLAS_NCCL_SYM(Broadcast, "ncclBroadcast");
        KLAS_NCCL_SYM(Send, "ncclSend");
        KLAS_NCCL_SYM(Recv, "ncclRecv");
        KLAS_NCCL_SYM(GetErrorString, "ncclGetErrorString");
#undef KLAS_NCCL_SYM
        g_nccl.ok = true;
    }
    *out = &g_nccl;
    return KLAS_OK;
}

}  // namespace mg
}  // namespace klas

struct klas_mg_context_s {
    std::vector<int> devices;
    std::vector<cudaStream_t> streams;
    std::vector<klas_nccl_comm> comms;   // empty until a collective is needed
    int saved_device = 0;
};

using namespace klas;

namespace {

// Restores the caller's current device when a call returns.
struct DeviceGuard {
    int saved = 0;
    bool have = false;
    DeviceGuard() { have = cudaGetDevice(&saved) == cudaSuccess; }
    ~DeviceGuard() {
        if (have) cudaSetDevice(saved);
    }
};

int nccl_check(mg::Nccl *n, klas_nccl_result rc, const char *what) {
    if (rc == 0) return KLAS_OK;
    return fail(KLAS_ERR_CUDA, "%s: %s", what, n->GetErrorString(rc));
}

int ensure_comms(klas_mg_context *ctx, mg::Nccl **out) {
    mg::Nccl *n = nullptr;
    if (int rc = mg::load_nccl(&n)) return rc;
    if (ctx->comms.empty()) {
        ctx->comms.resize(ctx->devices.size());
        if (int rc = nccl_check(n, n->CommInitAll(ctx->comms.data(), int(ctx->devices.size()), ctx->devices.data()),
                                "ncclCommInitAll")) {
            ctx->comms.clear();
            return rc;
        }
    }
    *out = n;
    return KLAS_OK;
}

// Assembles shards (shard i = `bytes[i]` bytes at `shards[i]` on device i) in shard order:
// gather == KLAS_MG_GATHER_ALL: into full[i] on every device; KLAS_MG_GATHER_FIRST: into full[0] only.
int gather_shards(klas_mg_context *ctx, const void *const *shards, const size_t *bytes, int gather, void *const *full) {
    const int n = int(ctx->devices.size());
    if (gather == KLAS_MG_NO_GATHER) return KLAS_OK;
    if (gather != KLAS_MG_GATHER_ALL && gather != KLAS_MG_GATHER_FIRST) return fail(KLAS_ERR_INVALID, "mg: bad gather mode %d", gather);
    if (!full || !full[0]) return fail(KLAS_ERR_INVALID, "mg: gather asked for but no destination given");
    std::vector<size_t> off(n + 1, 0);
    for (int i = 0; i < n; ++i) off[i + 1] = off[i] + bytes[i];
    if (n == 1) {   // one device: a copy on its stream
        KLAS_TRY_CUDA(cudaSetDevice(ctx->devices[0]));
        if (bytes[0]) KLAS_TRY_CUDA(cudaMemcpyAsync(full[0], shards[0], bytes[0], cudaMemcpyDeviceToDevice, ctx->streams[0]));
        return KLAS_OK;
    }
    mg::Nccl *nc = nullptr;
    if (int rc = ensure_comms(ctx, &nc)) return rc;
    if (gather == KLAS_MG_GATHER_ALL) {
        for (int i = 0; i < n; ++i)
            if (!full[i]) return fail(KLAS_ERR_INVALID, "mg: null gather destination for device %d", i);
        if (int rc = nccl_check(nc, nc->GroupStart(), "ncclGroupStart")) return rc;
        for (int r = 0; r < n; ++r) {
            if (bytes[r] == 0) continue;
            for (int i = 0; i < n; ++i) {
                char *dst = static_cast<char *>(full[i]) + off[r];
                if (int rc = nccl_check(nc, nc->Broadcast(i == r ? shards[r] : dst, dst, bytes[r], KLAS_NCCL_INT8, r,
                                                          ctx->comms[i], ctx->streams[i]), "ncclBroadcast"))
                    return rc;
            }
        }
        return nccl_check(nc, nc->GroupEnd(), "ncclGroupEnd");
    }
    // the first device receives every other device's shard; its own is a local copy
    KLAS_TRY_CUDA(cudaSetDevice(ctx->devices[0]));
    if (bytes[0]) KLAS_TRY_CUDA(cudaMemcpyAsync(full[0], shards[0], bytes[0], cudaMemcpyDeviceToDevice, ctx->streams[0]));
    if (int rc = nccl_check(nc, nc->GroupStart(), "ncclGroupStart")) return rc;
    for (int r = 1; r < n; ++r) {
        if (bytes[r] == 0) continue;
        if (int rc = nccl_check(nc, nc->Send(shards[r], bytes[r], KLAS_NCCL_INT8, 0, ctx->comms[r], ctx->streams[r]), "ncclSend")) return rc;
        if (int rc = nccl_check(nc, nc->Recv(static_cast<char *>(full[0]) + off[r], bytes[r], KLAS_NCCL_INT8, r, ctx->comms[0],
                                             ctx->streams[0]), "ncclRecv"))
            return rc;
    }
    return nccl_check(nc, nc->GroupEnd(), "ncclGroupEnd");
}

int check_ctx(const klas_mg_context *ctx) {
    if (!ctx || ctx->devices.empty()) return fail(KLAS_ERR_INVALID, "mg: null or empty context");
    return KLAS_OK;
}

template <typename Index>
int check_bounds(const Index *bounds, int parts, const char *what) {
    if (!bounds) return fail(KLAS_ERR_INVALID, "mg: null %s bounds", what);
    for (int i = 0; i < parts; ++i)
        if (bounds[i + 1] < bounds[i]) return fail(KLAS_ERR_INVALID, "mg: %s bounds decrease at part %d", what, i);
    return KLAS_OK;
}

}  // namespace

extern "C" {

int klas_b200_mg_create(const int *devices, int count, klas_mg_context **out) {
    clear_error();
    if (!out) return fail(KLAS_ERR_INVALID, "mg_create: null result pointer");
    *out = nullptr;
    if (!devices || count < 1 || count > 64) return fail(KLAS_ERR_INVALID, "mg_create: 1 to 64 devices, got %d", count);
    int visible = 0;
    KLAS_TRY_CUDA(cudaGetDeviceCount(&visible));
    for (int i = 0; i < count; ++i) {
        if (devices[i] < 0 || devices[i] >= visible) return fail(KLAS_ERR_INVALID, "mg_create: device %d is not visible (%d are)", devices[i], visible);
        for (int j = 0; j < i; ++j)
            if (devices[j] == devices[i]) return fail(KLAS_ERR_INVALID, "mg_create: device %d listed twice", devices[i]);
    }
    DeviceGuard guard;
    klas_mg_context *ctx = new klas_mg_context_s;
    ctx->devices.assign(devices, devices + count);
    ctx->streams.assign(count, nullptr);
    for (int i = 0; i < count; ++i) {
        cudaError_t rc = cudaSetDevice(devices[i]);
        if (rc == cudaSuccess) rc = cudaStreamCreateWithFlags(&ctx->streams[i], cudaStreamNonBlocking);
        if (rc != cudaSuccess) {
            for (int j = 0; j < i; ++j) {
                cudaSetDevice(devices[j]);
                cudaStreamDestroy(ctx->streams[j]);
            }
            delete ctx;
            return fail(KLAS_ERR_CUDA, "mg_create: device %d: %s", devices[i], cudaGetErrorString(rc));
        }
    }
    *out = ctx;
    return KLAS_OK;
}

int klas_b200_mg_destroy(klas_mg_context *ctx) {
    clear_error();
    if (!ctx) return KLAS_OK;
    DeviceGuard guard;
    int status = KLAS_OK;
    for (size_t i = 0; i < ctx->devices.size(); ++i) {
        if (cudaSetDevice(ctx->devices[i]) != cudaSuccess) continue;
        if (cudaStreamSynchronize(ctx->streams[i]) != cudaSuccess) status = KLAS_ERR_CUDA;
    }
    if (!ctx->comms.empty() && mg::g_nccl.ok)
        for (klas_nccl_comm c : ctx->comms) mg::g_nccl.CommDestroy(c);
    for (size_t i = 0; i < ctx->devices.size(); ++i) {
        if (cudaSetDevice(ctx->devices[i]) != cudaSuccess) continue;
        cudaStreamDestroy(ctx->streams[i]);
    }
    delete ctx;
    return status == KLAS_OK ? KLAS_OK : fail(KLAS_ERR_CUDA, "mg_destroy: a stream failed to synchronise");
}

int klas_b200_mg_count(const klas_mg_context *ctx) { return ctx ? int(ctx->devices.size()) : 0; }

void *klas_b200_mg_stream(const klas_mg_context *ctx, int index) {
    return ctx && index >= 0 && size_t(index) < ctx->streams.size() ? static_cast<void *>(ctx->streams[index]) : nullptr;
}

int klas_b200_mg_synchronize(klas_mg_context *ctx) {
    clear_error();
    if (int rc = check_ctx(ctx)) return rc;
    DeviceGuard guard;
    for (size_t i = 0; i < ctx->devices.size(); ++i) {
        KLAS_TRY_CUDA(cudaSetDevice(ctx->devices[i]));
        KLAS_TRY_CUDA(cudaStreamSynchronize(ctx->streams[i]));
    }
    // a bounded wait of a tensor-core kernel that gave up shows in the device's status word
    for (size_t i = 0; i < ctx->devices.size(); ++i) {
        KLAS_TRY_CUDA(cudaSetDevice(ctx->devices[i]));
        if (klas_b200_gemm_tc_status_peek() != 0) return klas_b200_gemm_tc_status(nullptr);
    }
    return KLAS_OK;
}

// ---- partitioners (host only) ------------------------------------------------------------------
int klas_b200_mg_row_blocks(uint64_t rows, int parts, uint64_t align, uint64_t *bounds) {
    clear_error();
    if (parts < 1 || align < 1 || !bounds) return fail(KLAS_ERR_INVALID, "mg_row_blocks: bad arguments");
    const uint64_t units = (rows + align - 1) / align;   // tiles, the last one possibly ragged
    uint64_t start = 0;
    for (int r = 0; r < parts; ++r) {
        bounds[r] = start;
        const uint64_t n_units = units / uint64_t(parts) + (uint64_t(r) < units % uint64_t(parts) ? 1 : 0);
        start = std::min(rows, start + n_units * align);
    }
    bounds[parts] = rows;
    return KLAS_OK;
}

int klas_b200_mg_csr_row_ranges(const uint32_t *row_off, uint32_t rows, int parts, int balance_nnz, uint32_t *bounds) {
    clear_error();
    if (parts < 1 || !bounds || (balance_nnz && !row_off)) return fail(KLAS_ERR_INVALID, "mg_csr_row_ranges: bad arguments");
    bounds[0] = 0;
    if (!balance_nnz) {
        for (int r = 1; r < parts; ++r) bounds[r] = uint32_t(uint64_t(rows) * uint64_t(r) / uint64_t(parts));
    } else {
        const uint64_t nnz = row_off[rows];
        for (int r = 1; r < parts; ++r) {
            const uint32_t target = uint32_t(nnz * uint64_t(r) / uint64_t(parts));
            const uint32_t cut = uint32_t(std::lower_bound(row_off, row_off + rows + 1, target) - row_off);
            bounds[r] = std::min(std::max(cut, bounds[r - 1]), rows);
        }
    }
    bounds[parts] = rows;
    return KLAS_OK;
}

// ---- replication -------------------------------------------------------------------------------
int klas_b200_mg_broadcast(klas_mg_context *ctx, void *const *buffers, size_t bytes, int root) {
    clear_error();
    if (int rc = check_ctx(ctx)) return rc;
    const int n = int(ctx->devices.size());
    if (!buffers || root < 0 || root >= n) return fail(KLAS_ERR_INVALID, "mg_broadcast: bad arguments");
    if (bytes == 0 || n == 1) return KLAS_OK;
    for (int i = 0; i < n; ++i)
        if (!buffers[i]) return fail(KLAS_ERR_INVALID, "mg_broadcast: null buffer for device %d", i);
    DeviceGuard guard;
    mg::Nccl *nc = nullptr;
    if (int rc = ensure_comms(ctx, &nc)) return rc;
    if (int rc = nccl_check(nc, nc->GroupStart(), "ncclGroupStart")) return rc;
    for (int i = 0; i < n; ++i)
        if (int rc = nccl_check(nc, nc->Broadcast(buffers[i], buffers[i], bytes, KLAS_NCCL_INT8, root, ctx->comms[i], ctx->streams[i]),
                                "ncclBroadcast"))
            return rc;
    return nccl_check(nc, nc->GroupEnd(), "ncclGroupEnd");
}

// ---- sharded products --------------------------------------------------------------------------
int klas_b200_mg_gemm_tc(klas_mg_context *ctx, int in_dtype, int out_dtype, int b_major, const uint64_t *row_bounds,
                         uint64_t shared, uint64_t cols, const void *const *A_shards, const void *const *B_replicas,
                         void *const *D_shards, int gather, void *const *D_full) {
    clear_error();
    if (int rc = check_ctx(ctx)) return rc;
    const int n = int(ctx->devices.size());
    if (int rc = check_bounds(row_bounds, n, "row")) return rc;
    if (!A_shards || !B_replicas || !D_shards) return fail(KLAS_ERR_INVALID, "mg_gemm_tc: null pointer array");
    const size_t os = dtype_size(out_dtype);
    if (os == 0) return fail(KLAS_ERR_INVALID, "mg_gemm_tc: bad out_dtype");
    DeviceGuard guard;
    std::vector<size_t> bytes(n);
    for (int i = 0; i < n; ++i) {
        const uint64_t m = row_bounds[i + 1] - row_bounds[i];
        bytes[i] = size_t(m) * cols * os;
        if (m == 0) continue;
        KLAS_TRY_CUDA(cudaSetDevice(ctx->devices[i]));
        if (int rc = launch_gemm_umma(in_dtype, out_dtype, b_major, 1, m, shared, cols, A_shards[i], B_replicas[i], nullptr,
                                      D_shards[i], 1.0f, 0.0f, nullptr, ctx->streams[i]))
            return rc;
    }
    return gather_shards(ctx, const_cast<const void *const *>(D_shards), bytes.data(), gather, D_full);
}

int klas_b200_mg_gemm_tc_batched(klas_mg_context *ctx, int in_dtype, int out_dtype, int b_major, const uint64_t *page_bounds,
                                 uint64_t rows, uint64_t shared, uint64_t cols, const void *const *A_pages,
                                 const void *const *B_pages, void *const *D_pages, int gather, void *const *D_full) {
    clear_error();
    if (int rc = check_ctx(ctx)) return rc;
    const int n = int(ctx->devices.size());
    if (int rc = check_bounds(page_bounds, n, "page")) return rc;
    if (!A_pages || !B_pages || !D_pages) return fail(KLAS_ERR_INVALID, "mg_gemm_tc_batched: null pointer array");
    const size_t os = dtype_size(out_dtype);
    if (os == 0) return fail(KLAS_ERR_INVALID, "mg_gemm_tc_batched: bad out_dtype");
    DeviceGuard guard;
    std::vector<size_t> bytes(n);
    for (int i = 0; i < n; ++i) {
        const uint64_t pages = page_bounds[i + 1] - page_bounds[i];
        bytes[i] = size_t(pages) * rows * cols * os;
        if (pages == 0) continue;
        if (pages > 0xffffffffull) return fail(KLAS_ERR_TOO_LARGE, "mg_gemm_tc_batched: too many pages");
        KLAS_TRY_CUDA(cudaSetDevice(ctx->devices[i]));
        if (int rc = launch_gemm_umma(in_dtype, out_dtype, b_major, uint32_t(pages), rows, shared, cols, A_pages[i], B_pages[i],
                                      nullptr, D_pages[i], 1.0f, 0.0f, nullptr, ctx->streams[i]))
            return rc;
    }
    return gather_shards(ctx, const_cast<const void *const *>(D_pages), bytes.data(), gather, D_full);
}

int klas_b200_mg_gemm(klas_mg_context *ctx, int dtype, const uint64_t *row_bounds, uint64_t n_cols, uint64_t k,
                      const void *const *A_shards, const void *const *B_replicas, void *const *C_shards, int gather,
                      void *const *C_full) {
    clear_error();
    if (int rc = check_ctx(ctx)) return rc;
    const int n = int(ctx->devices.size());
    if (int rc = check_bounds(row_bounds, n, "row")) return rc;
    if (!A_shards || !B_replicas || !C_shards) return fail(KLAS_ERR_INVALID, "mg_gemm: null pointer array");
    const size_t es = dtype_size(dtype);
    if (es == 0) return fail(KLAS_ERR_INVALID, "mg_gemm: bad dtype");
    DeviceGuard guard;
    std::vector<size_t> bytes(n);
    for (int i = 0; i < n; ++i) {
        const uint64_t m = row_bounds[i + 1] - row_bounds[i];
        bytes[i] = size_t(m) * n_cols * es;
        if (m == 0) continue;
        KLAS_TRY_CUDA(cudaSetDevice(ctx->devices[i]));
        if (int rc = launch_gemm_simt(dtype, KLAS_RRR, 1, m, n_cols, k, nullptr, nullptr, A_shards[i], B_replicas[i], C_shards[i],
                                      ctx->streams[i]))
            return rc;
    }
    return gather_shards(ctx, const_cast<const void *const *>(C_shards), bytes.data(), gather, C_full);
}

int klas_b200_mg_spmm(klas_mg_context *ctx, int dtype, const uint32_t *row_bounds, uint32_t shared, uint32_t cols,
                      const uint32_t *nnz, const void *const *elems, const uint32_t *const *col_ind,
                      const uint32_t *const *row_off, const void *const *B_replicas, void *const *C_shards, int gather,
                      void *const *C_full) {
    clear_error();
    if (int rc = check_ctx(ctx)) return rc;
    const int n = int(ctx->devices.size());
    if (int rc = check_bounds(row_bounds, n, "CSR row")) return rc;
    if (!nnz || !elems || !col_ind || !row_off || !B_replicas || !C_shards) return fail(KLAS_ERR_INVALID, "mg_spmm: null pointer array");
    DeviceGuard guard;
    std::vector<size_t> bytes(n);
    for (int i = 0; i < n; ++i) {
        const uint32_t m = row_bounds[i + 1] - row_bounds[i];
        bytes[i] = size_t(m) * cols * 4;
        if (m == 0) continue;
        KLAS_TRY_CUDA(cudaSetDevice(ctx->devices[i]));
        if (int rc = launch_spmm(dtype, m, shared, cols, nnz[i], elems[i], col_ind[i], row_off[i], nullptr, B_replicas[i],
                                 C_shards[i], ctx->streams[i]))
            return rc;
    }
    return gather_shards(ctx, const_cast<const void *const *>(C_shards), bytes.data(), gather, C_full);
}

}  // extern "C"
