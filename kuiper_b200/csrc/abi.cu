// extern "C" entry points of libklas_b200.so (declared in include/klas_b200.h),
// plus the small amount of per-thread / per-device state behind them.
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <sched.h>
#include <sys/syscall.h>
#include <unistd.h>

#include <atomic>
#include <climits>
#include <cstring>
#include <mutex>

#include "klas_internal.h"

namespace klas {

static thread_local char tls_error[512] = "";

int fail(int code, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(tls_error, sizeof tls_error, fmt, ap);
    va_end(ap);
    return code;
}

void clear_error() { tls_error[0] = '\0'; }

// tuning knobs (klas_knob): defaults = the library's own choice
static std::atomic<int> g_knobs[KLAS_KNOB_COUNT] = {{0}, {0}, {0}, {0}, {-1}, {-1}, {0}, {0}, {0}};
struct KnobRange { int lo, hi; };
static const KnobRange g_knob_range[KLAS_KNOB_COUNT] = {{0, 5}, {0, 1024}, {0, 2}, {0, 1}, {-1, 2}, {-1, 16}, {0, 128}, {0, 8}, {0, 2}};

int debug_knob(int knob) {
    return knob >= 0 && knob < KLAS_KNOB_COUNT ? g_knobs[knob].load(std::memory_order_relaxed) : INT_MIN;
}

constexpr int MAX_DEVICES = 64;
static std::mutex g_mutex;
static DeviceInfo g_info[MAX_DEVICES];

int device_info(DeviceInfo *out) {
    int dev = 0;
    KLAS_TRY_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= MAX_DEVICES) return fail(KLAS_ERR_INVALID, "device index %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_mutex);
    DeviceInfo &d = g_info[dev];
    if (d.device != dev) {
        KLAS_TRY_CUDA(cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev));
        KLAS_TRY_CUDA(cudaDeviceGetAttribute(&d.l2_bytes, cudaDevAttrL2CacheSize, dev));
        KLAS_TRY_CUDA(cudaDeviceGetAttribute(&d.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
        KLAS_TRY_CUDA(cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, dev));
        KLAS_TRY_CUDA(cudaDeviceGetAttribute(&d.cc_minor, cudaDevAttrComputeCapabilityMinor, dev));
        d.device = dev;
    }
    *out = d;
    return KLAS_OK;
}

// ------------------------------------------------------------------ workspace
constexpr int WS_SLOTS = 8;
struct Workspace {
    void *ptr[WS_SLOTS] = {};
    size_t cap[WS_SLOTS] = {};
};
static Workspace g_ws[MAX_DEVICES];

int workspace_reserve(int slot, size_t bytes, void **ptr) {
    int dev = 0;
    KLAS_TRY_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= MAX_DEVICES || slot < 0 || slot >= WS_SLOTS)
        return fail(KLAS_ERR_INVALID, "workspace: bad device or slot");
    std::lock_guard<std::mutex> lock(g_mutex);
    Workspace &w = g_ws[dev];
    if (bytes == 0) bytes = 16;
    if (w.cap[slot] < bytes) {
        if (w.ptr[slot]) KLAS_TRY_CUDA(cudaFree(w.ptr[slot]));
        w.ptr[slot] = nullptr;
        w.cap[slot] = 0;
        KLAS_TRY_CUDA(cudaMalloc(&w.ptr[slot], bytes));
        w.cap[slot] = bytes;
    }
    *ptr = w.ptr[slot];
    return KLAS_OK;
}

int workspace_release() {
    int dev = 0;
    KLAS_TRY_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= MAX_DEVICES) return fail(KLAS_ERR_INVALID, "workspace: bad device");
    std::lock_guard<std::mutex> lock(g_mutex);
    Workspace &w = g_ws[dev];
    for (int s = 0; s < WS_SLOTS; ++s) {
        if (w.ptr[s]) KLAS_TRY_CUDA(cudaFree(w.ptr[s]));
        w.ptr[s] = nullptr;
        w.cap[s] = 0;
    }
    return KLAS_OK;
}

int umma_read_status(int *value);
int umma_peek_status();
int umma_plan(uint64_t rows, uint64_t shared, uint64_t cols, uint32_t batch, int sm_count, int *kind, int *tile_cols,
              int *k_parts, int *tail_cut);
int umma_release_split_workspace();
int umma_clear_status();
int umma_wait_probe(uint32_t limit_ms, int *gave_up, cudaStream_t stream);

// Streams and events of the chunked host-buffer calls, one set per device, created on first use.
struct HostPipe {
    static constexpr int MAX_CHUNKS = 8;
    static constexpr int GRID_2D = 16;                  // row blocks of A = column blocks of B in the 2-D schedule
    static constexpr int EVENTS = 2 * GRID_2D + 2;      // which loads and computes 2 x GRID_2D pieces
    cudaStream_t in = nullptr, compute = nullptr, out = nullptr;
    cudaEvent_t loaded[EVENTS] = {}, computed[EVENTS] = {};
    bool ready = false;
};
static HostPipe g_pipes[MAX_DEVICES];

// The host-buffer entry points share one workspace and one set of streams and events per device:
// each holds this device's lock from start to finish, so calls from several host threads on one
// device take turns instead of overwriting each other's staging buffers.
static std::mutex g_host_call[MAX_DEVICES];
struct HostCallLock {
    std::unique_lock<std::mutex> lock;
    int rc = KLAS_OK;
    HostCallLock() {
        int dev = 0;
        rc = check_cuda(cudaGetDevice(&dev), "cudaGetDevice");
        if (rc == KLAS_OK && (dev < 0 || dev >= MAX_DEVICES)) rc = fail(KLAS_ERR_INVALID, "device index %d out of range", dev);
        if (rc == KLAS_OK) lock = std::unique_lock<std::mutex>(g_host_call[dev]);
    }
};

static int host_pipe(HostPipe **out) {
    int dev = 0;
    KLAS_TRY_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= MAX_DEVICES) return fail(KLAS_ERR_INVALID, "device index %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_mutex);
    HostPipe &h = g_pipes[dev];
    if (!h.ready) {
        KLAS_TRY_CUDA(cudaStreamCreateWithFlags(&h.in, cudaStreamNonBlocking));
        KLAS_TRY_CUDA(cudaStreamCreateWithFlags(&h.compute, cudaStreamNonBlocking));
        KLAS_TRY_CUDA(cudaStreamCreateWithFlags(&h.out, cudaStreamNonBlocking));
        for (int i = 0; i < HostPipe::EVENTS; ++i) {
            KLAS_TRY_CUDA(cudaEventCreateWithFlags(&h.loaded[i], cudaEventDisableTiming));
            KLAS_TRY_CUDA(cudaEventCreateWithFlags(&h.computed[i], cudaEventDisableTiming));
        }
        h.ready = true;
    }
    *out = &h;
    return KLAS_OK;
}

// Stages `bytes` from host pointer `src` into workspace slot `slot`.
static int stage_in(int slot, const void *src, size_t bytes, cudaStream_t s, void **dptr) {
    if (int rc = workspace_reserve(slot, bytes, dptr)) return rc;
    if (bytes && src) KLAS_TRY_CUDA(cudaMemcpyAsync(*dptr, src, bytes, cudaMemcpyHostToDevice, s));
    return KLAS_OK;
}

}  // namespace klas

using namespace klas;

extern "C" {

const char *klas_b200_last_error(void) { return tls_error; }

int klas_b200_version(void) { return 1000; }

int klas_b200_sm_count(void) {
    DeviceInfo info;
    if (device_info(&info)) return 0;
    return info.sm_count;
}

int klas_b200_gemm(int dtype, int layout, uint32_t batch, uint64_t m, uint64_t n, uint64_t k,
                   const void *alpha, const void *beta, const void *A, const void *B, void *C,
                   void *stream) {
    clear_error();
    return launch_gemm_simt(dtype, layout, batch, m, n, k, alpha, beta, A, B, C,
                            static_cast<cudaStream_t>(stream));
}

int klas_b200_gemm_compensated(int dtype, int layout, uint64_t m, uint64_t n, uint64_t k, const void *A, const void *B,
                               void *C, void *stream) {
    clear_error();
    return launch_gemm_simt_compensated(dtype, layout, m, n, k, A, B, C, static_cast<cudaStream_t>(stream));
}

int klas_b200_gemm_tc(int in_dtype, int out_dtype, int b_major, uint32_t batch, uint64_t rows,
                      uint64_t shared, uint64_t cols, const void *A, const void *B, const void *C,
                      void *D, float alpha, float beta, int *status_word, void *stream) {
    clear_error();
    return launch_gemm_umma(in_dtype, out_dtype, b_major, batch, rows, shared, cols, A, B, C, D,
                            alpha, beta, status_word, static_cast<cudaStream_t>(stream));
}

int klas_b200_gemm_strided(int dtype, uint32_t batch, uint64_t m, uint64_t n, uint64_t k, const void *alpha,
                           const void *beta, const void *A, uint64_t lda, uint64_t stride_a, const void *B,
                           uint64_t ldb, uint64_t stride_b, void *C, uint64_t ldc, uint64_t stride_c, int map_a,
                           int map_b, int comb, void *stream) {
    clear_error();
    return launch_gemm_simt_strided(dtype, batch, m, n, k, alpha, beta, A, lda, stride_a, B, ldb, stride_b, C, ldc,
                                    stride_c, map_a, map_b, comb, static_cast<cudaStream_t>(stream));
}

int klas_b200_gemm_tc_fused(int in_dtype, int out_dtype, int b_major, uint32_t batch, uint64_t rows,
                            uint64_t shared, uint64_t cols, const void *A, const void *B, const void *C,
                            void *D, float alpha, float beta, int map_a, int map_b, int comb,
                            int *status_word, void *stream) {
    clear_error();
    return launch_gemm_umma_fused(in_dtype, out_dtype, b_major, batch, rows, shared, cols, A, B, C, D, alpha, beta,
                                  map_a, map_b, comb, status_word, static_cast<cudaStream_t>(stream));
}

int klas_b200_gemm_tc_strided(int in_dtype, int out_dtype, int b_major, uint32_t batch, uint64_t rows,
                              uint64_t shared, uint64_t cols, const void *A, uint64_t lda, uint64_t stride_a,
                              const void *B, uint64_t ldb, uint64_t stride_b, const void *C, void *D, uint64_t ldd,
                              uint64_t stride_d, float alpha, float beta, int map_a, int map_b, int comb,
                              int *status_word, void *stream) {
    clear_error();
    const TcStrides st{lda, stride_a, ldb, stride_b, ldd, stride_d};
    return launch_gemm_umma_strided(in_dtype, out_dtype, b_major, batch, rows, shared, cols, A, B, C, D, st, alpha, beta,
                                    map_a, map_b, comb, status_word, static_cast<cudaStream_t>(stream));
}

int klas_b200_csr_count(int dtype, uint32_t rows, uint32_t cols, const void *dense, uint32_t *row_off, void *stream) {
    clear_error();
    return launch_csr_count(dtype, rows, cols, dense, row_off, static_cast<cudaStream_t>(stream));
}

int klas_b200_csr_fill(int dtype, uint32_t rows, uint32_t cols, const void *dense, const uint32_t *row_off,
                       void *elems, uint32_t *col_ind, void *stream) {
    clear_error();
    return launch_csr_fill(dtype, rows, cols, dense, row_off, elems, col_ind, static_cast<cudaStream_t>(stream));
}

size_t klas_b200_csr_row_order_scratch_bytes(uint32_t rows) { return csr_row_order_scratch_bytes(rows); }

int klas_b200_csr_row_order(uint32_t rows, const uint32_t *row_off, uint32_t *row_indices, void *scratch,
                            size_t scratch_bytes, void *stream) {
    clear_error();
    return launch_csr_row_order(rows, row_off, row_indices, scratch, scratch_bytes, static_cast<cudaStream_t>(stream));
}

int klas_b200_minplus_u16(uint32_t m, uint32_t n, uint32_t k, const uint16_t *A, const uint16_t *B, uint16_t *C,
                          void *stream) {
    clear_error();
    return launch_minplus_u16(m, n, k, A, B, C, static_cast<cudaStream_t>(stream));
}

int klas_b200_sdpa(int dtype, uint32_t pages, uint64_t l, uint64_t s, uint64_t e, uint64_t ev, const void *Q,
                   const void *K, const void *V, void *bias_scores, int has_bias, void *out, float scale,
                   void *stream) {
    clear_error();
    if (dtype != KLAS_F16 && dtype != KLAS_BF16) return fail(KLAS_ERR_INVALID, "sdpa: dtype must be KLAS_F16 or KLAS_BF16");
    if (pages == 0 || l == 0 || ev == 0) return KLAS_OK;
    if (s == 0) return fail(KLAS_ERR_INVALID, "sdpa: no keys (s == 0): the softmax of an empty row is undefined");
    if (!Q || !K || !V || !bias_scores || !out) return fail(KLAS_ERR_INVALID, "sdpa: null pointer");
    if (e % 8 || s % 8 || ev % 8)
        return fail(KLAS_ERR_UNSUPPORTED, "sdpa: e (%llu), s (%llu) and ev (%llu) must be multiples of 8",
                    (unsigned long long)e, (unsigned long long)s, (unsigned long long)ev);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // S = scale * Q.K^T (+ bias): K's rows are the columns of K^T, i.e. a column-major B operand
    if (int rc = launch_gemm_umma_fused(dtype, dtype, KLAS_B_COL_MAJOR, pages, l, e, s, Q, K, has_bias ? bias_scores : nullptr,
                                        bias_scores, scale, 1.0f, KLAS_MAP_ID, KLAS_MAP_ID,
                                        has_bias ? KLAS_COMB_AXPBY : KLAS_COMB_SCALED, nullptr, st))
        return rc;
    if (int rc = launch_softmax_rows(dtype, 0, uint64_t(pages) * l, s, bias_scores, st)) return rc;
    return launch_gemm_umma(dtype, dtype, KLAS_B_ROW_MAJOR, pages, l, s, ev, bias_scores, V, nullptr, out, 1.0f, 0.0f,
                            nullptr, st);
}

int klas_b200_sdpa_fused(int dtype, uint32_t pages, uint64_t l, uint64_t s, uint64_t e, const void *Q, const void *K,
                         const void *V, void *out, float scale, void *stream) {
    clear_error();
    return launch_sdpa_fused(dtype, pages, l, s, e, Q, K, V, out, scale, static_cast<cudaStream_t>(stream));
}

int klas_b200_gemm_tc_status(int *site) {
    clear_error();
    int v = 0;
    if (int rc = umma_read_status(&v)) return rc;
    if (site) *site = v;
    if (v == 0) return KLAS_OK;
    if (int rc = umma_clear_status()) return rc;
    return fail(KLAS_ERR_TIMEOUT, "gemm_tc: a device-side wait gave up at site 0x%x", v);
}

int klas_b200_gemm_tc_status_peek(void) { return umma_peek_status(); }

int klas_b200_debug_wait_probe(uint32_t limit_ms, int *gave_up, void *stream) {
    clear_error();
    if (limit_ms == 0 || limit_ms > 1000) return fail(KLAS_ERR_INVALID, "wait_probe: limit must be 1..1000 ms");
    return umma_wait_probe(limit_ms, gave_up, static_cast<cudaStream_t>(stream));
}

int klas_b200_spmm(int dtype, uint32_t rows, uint32_t shared, uint32_t cols, uint32_t nnz,
                   const void *elems, const uint32_t *col_ind, const uint32_t *row_off,
                   const uint32_t *row_indices, const void *B, void *C, void *stream) {
    clear_error();
    return launch_spmm(dtype, rows, shared, cols, nnz, elems, col_ind, row_off, row_indices, B, C,
                       static_cast<cudaStream_t>(stream));
}

int klas_b200_spmm_gather_probe(uint32_t shared, uint32_t cols, uint32_t nnz, const uint32_t *col_ind, const void *B,
                                void *stream) {
    clear_error();
    return launch_spmm_gather_probe(shared, cols, nnz, col_ind, static_cast<const float *>(B),
                                    static_cast<cudaStream_t>(stream));
}

int klas_b200_gemm_host(int dtype, int layout, uint32_t batch, uint64_t m, uint64_t n, uint64_t k,
                        const void *alpha, const void *beta, const void *A, const void *B,
                        void *C) {
    clear_error();
    HostCallLock turn;
    if (turn.rc) return turn.rc;
    const size_t es = dtype_size(dtype);
    if (es == 0) return fail(KLAS_ERR_INVALID, "gemm_host: bad dtype");
    const size_t a_bytes = size_t(batch) * m * k * es, b_bytes = size_t(batch) * k * n * es,
                 c_bytes = size_t(batch) * m * n * es;
    if (c_bytes == 0) return KLAS_OK;
    if (!C) return fail(KLAS_ERR_INVALID, "gemm_host: null C");
    cudaStream_t s = nullptr;
    void *dA, *dB, *dC;
    if (int rc = stage_in(0, A, a_bytes, s, &dA)) return rc;
    if (int rc = stage_in(1, B, b_bytes, s, &dB)) return rc;
    if (int rc = stage_in(2, alpha ? C : nullptr, c_bytes, s, &dC)) return rc;
    if (int rc = launch_gemm_simt(dtype, layout, batch, m, n, k, alpha, beta, dA, dB, dC, s)) return rc;
    KLAS_TRY_CUDA(cudaMemcpyAsync(C, dC, c_bytes, cudaMemcpyDeviceToHost, s));
    KLAS_TRY_CUDA(cudaStreamSynchronize(s));
    return KLAS_OK;
}

// One large product D = A.B from host buffers, scheduled so that the device->host copy of D
// overlaps the host->device copies of A and B from early on.  A is cut into G row blocks and B
// into G column blocks; they are sent alternately (A_0, B_0, A_1, B_1, ...) and after every
// arrival the part of D that has just become computable is multiplied and sent back:
//   after A_t:  D[rows of A_t][columns of B_0 .. B_(t-1)]
//   after B_t:  D[rows of A_0 .. A_t][columns of B_t]
// so after 2(t+1) of the 2G input pieces (t+1)^2 of the G^2 output tiles are on their way.
// With one block of rows per chunk instead (the other schedule below), no output can leave
// before all of B has arrived, and a call costs bytes(B) + bytes(D) over the link instead of
// about max(bytes in, bytes out).  (How far that goes is limited by the product itself: after a
// fraction f of the input only f^2 of the output can exist, so the outbound copy starves early.)
static int gemm_tc_host_2d(HostPipe *hp, int in_dtype, int out_dtype, int b_major, uint64_t rows, uint64_t shared,
                           uint64_t cols, const void *A, const void *B, void *D, void *dA, void *dB, void *dD) {
    const size_t is = dtype_size(in_dtype), os = dtype_size(out_dtype);
    uint64_t G = 4;   // measured best at 8192^3 bf16 -> f32: 7.54 ms (4), 7.79 (8), 7.77 (16), 8.36 (2)
    if (const int v = debug_knob(KLAS_KNOB_HOST_GRID); v >= 1 && v <= HostPipe::GRID_2D) G = uint64_t(v);
    const uint64_t rc = ((rows + G - 1) / G + 511) / 512 * 512;   // rows per block of A
    const uint64_t cc = ((cols + G - 1) / G + 255) / 256 * 256;   // columns per block of B
    const bool col_major = b_major == KLAS_B_COL_MAJOR;
    char *out_dev = static_cast<char *>(dD);   // output blocks are laid one after another here
    int n_loaded = 0, n_computed = 0;
    // one product of `m` rows of A from row r0 with `n` columns of B from column c0, then its copy home
    auto product = [&](uint64_t r0, uint64_t m, uint64_t c0, uint64_t n, cudaEvent_t after) -> int {
        if (m == 0 || n == 0) return KLAS_OK;
        KLAS_TRY_CUDA(cudaStreamWaitEvent(hp->compute, after, 0));
        const char *a_dev = static_cast<const char *>(dA) + r0 * shared * is;
        const char *b_dev = static_cast<const char *>(dB) + c0 * shared * is;   // block c0 starts here in both layouts
        if (int rc2 = launch_gemm_umma(in_dtype, out_dtype, b_major, 1, m, shared, n, a_dev, b_dev, nullptr, out_dev, 1.0f,
                                       0.0f, nullptr, hp->compute))
            return rc2;
        cudaEvent_t done = hp->computed[n_computed++ % HostPipe::EVENTS];   // waits are enqueued right after each record, so reuse is safe
        KLAS_TRY_CUDA(cudaEventRecord(done, hp->compute));
        KLAS_TRY_CUDA(cudaStreamWaitEvent(hp->out, done, 0));
        KLAS_TRY_CUDA(cudaMemcpy2DAsync(static_cast<char *>(D) + (r0 * cols + c0) * os, cols * os, out_dev, n * os, n * os, m,
                                        cudaMemcpyDeviceToHost, hp->out));
        out_dev += m * n * os;
        return KLAS_OK;
    };
    for (uint64_t t = 0; t < G; ++t) {
        const uint64_t r0 = t * rc < rows ? t * rc : rows, r1 = r0 + rc < rows ? r0 + rc : rows;
        const uint64_t c0 = t * cc < cols ? t * cc : cols, c1 = c0 + cc < cols ? c0 + cc : cols;
        // A_t
        if (r1 > r0 && shared)
            KLAS_TRY_CUDA(cudaMemcpyAsync(static_cast<char *>(dA) + r0 * shared * is, static_cast<const char *>(A) + r0 * shared * is,
                                          (r1 - r0) * shared * is, cudaMemcpyHostToDevice, hp->in));
        cudaEvent_t a_in = hp->loaded[n_loaded++];
        KLAS_TRY_CUDA(cudaEventRecord(a_in, hp->in));
        if (col_major) {
            // columns [0, c0) of B are one contiguous operand (rows of the stored cols x shared matrix)
            if (int rc2 = product(r0, r1 - r0, 0, c0, a_in)) return rc2;
        } else {
            for (uint64_t j = 0; j < t && j * cc < cols; ++j)   // row-major B: every column block is its own shared x cc operand
                if (int rc2 = product(r0, r1 - r0, j * cc, (j + 1) * cc < cols ? cc : cols - j * cc, a_in)) return rc2;
        }
        // B_t
        if (c1 > c0 && shared) {
            char *b_dst = static_cast<char *>(dB) + c0 * shared * is;
            if (col_major)
                KLAS_TRY_CUDA(cudaMemcpyAsync(b_dst, static_cast<const char *>(B) + c0 * shared * is, (c1 - c0) * shared * is,
                                              cudaMemcpyHostToDevice, hp->in));
            else   // gather the column block into a contiguous shared x (c1 - c0) matrix
                KLAS_TRY_CUDA(cudaMemcpy2DAsync(b_dst, (c1 - c0) * is, static_cast<const char *>(B) + c0 * is, cols * is,
                                                (c1 - c0) * is, shared, cudaMemcpyHostToDevice, hp->in));
        }
        cudaEvent_t b_in = hp->loaded[n_loaded++];
        KLAS_TRY_CUDA(cudaEventRecord(b_in, hp->in));
        if (int rc2 = product(0, r1, c0, c1 - c0, b_in)) return rc2;
    }
    KLAS_TRY_CUDA(cudaStreamSynchronize(hp->out));
    KLAS_TRY_CUDA(cudaStreamSynchronize(hp->in));
    return klas_b200_gemm_tc_status(nullptr);
}

int klas_b200_gemm_tc_host(int in_dtype, int out_dtype, int b_major, uint32_t batch, uint64_t rows,
                           uint64_t shared, uint64_t cols, const void *A, const void *B,
                           const void *C, void *D, float alpha, float beta) {
    clear_error();
    HostCallLock turn;
    if (turn.rc) return turn.rc;
    const size_t is = dtype_size(in_dtype), os = dtype_size(out_dtype);
    if (is == 0 || os == 0) return fail(KLAS_ERR_INVALID, "gemm_tc_host: bad dtype");
    const size_t a_bytes = size_t(batch) * rows * shared * is,
                 b_bytes = size_t(batch) * shared * cols * is,
                 d_bytes = size_t(batch) * rows * cols * os;
    if (d_bytes == 0) return KLAS_OK;
    if (!D) return fail(KLAS_ERR_INVALID, "gemm_tc_host: null D");
    HostPipe *hp = nullptr;
    if (int rc = host_pipe(&hp)) return rc;
    void *dA, *dB, *dC = nullptr, *dD;
    if (int rc = workspace_reserve(0, a_bytes, &dA)) return rc;
    if (int rc = workspace_reserve(1, b_bytes, &dB)) return rc;
    if (C)
        if (int rc = workspace_reserve(2, d_bytes, &dC)) return rc;
    if (int rc = workspace_reserve(3, d_bytes, &dD)) return rc;
    if (batch == 1 && !C && rows >= 4096 && cols >= 4096 && shared % 8 == 0 && cols % 8 == 0 &&
        (b_major == KLAS_B_COL_MAJOR || b_major == KLAS_B_ROW_MAJOR) && A && B &&
        debug_knob(KLAS_KNOB_HOST_GRID) != 0)
        return gemm_tc_host_2d(hp, in_dtype, out_dtype, b_major, rows, shared, cols, A, B, D, dA, dB, dD);

    // The work is cut into chunks -- row blocks of A/C/D for one matrix, groups of pages for a
    // batch -- that flow through three streams: host->device copies, kernels, device->host
    // copies.  The two copy directions overlap each other and the kernels, so a call costs
    // about max(bytes in, bytes out) over PCIe instead of their sum.
    const bool by_rows = batch == 1;
    const uint64_t units = by_rows ? rows : batch;
    uint64_t per_chunk = by_rows ? ((rows + HostPipe::MAX_CHUNKS - 1) / HostPipe::MAX_CHUNKS + 511) / 512 * 512
                                 : (batch + HostPipe::MAX_CHUNKS - 1) / HostPipe::MAX_CHUNKS;
    if (per_chunk == 0) per_chunk = 1;
    const size_t a_unit = (by_rows ? size_t(shared) : size_t(rows) * shared) * is;     // bytes of A per unit
    const size_t d_unit = (by_rows ? size_t(cols) : size_t(rows) * cols) * os;         // bytes of C/D per unit
    const size_t b_unit = by_rows ? 0 : size_t(shared) * cols * is;                    // bytes of B per page
    if (by_rows && b_bytes)
        KLAS_TRY_CUDA(cudaMemcpyAsync(dB, B, b_bytes, cudaMemcpyHostToDevice, hp->in));
    int chunk = 0;
    for (uint64_t u0 = 0; u0 < units; u0 += per_chunk, ++chunk) {
        const uint64_t n = units - u0 < per_chunk ? units - u0 : per_chunk;
        char *a_dev = static_cast<char *>(dA) + u0 * a_unit;
        char *b_dev = static_cast<char *>(dB) + u0 * b_unit;
        char *c_dev = dC ? static_cast<char *>(dC) + u0 * d_unit : nullptr;
        char *d_dev = static_cast<char *>(dD) + u0 * d_unit;
        if (a_unit && shared)
            KLAS_TRY_CUDA(cudaMemcpyAsync(a_dev, static_cast<const char *>(A) + u0 * a_unit, n * a_unit,
                                          cudaMemcpyHostToDevice, hp->in));
        if (!by_rows && b_unit)
            KLAS_TRY_CUDA(cudaMemcpyAsync(b_dev, static_cast<const char *>(B) + u0 * b_unit, n * b_unit,
                                          cudaMemcpyHostToDevice, hp->in));
        if (c_dev)
            KLAS_TRY_CUDA(cudaMemcpyAsync(c_dev, static_cast<const char *>(C) + u0 * d_unit, n * d_unit,
                                          cudaMemcpyHostToDevice, hp->in));
        KLAS_TRY_CUDA(cudaEventRecord(hp->loaded[chunk], hp->in));
        KLAS_TRY_CUDA(cudaStreamWaitEvent(hp->compute, hp->loaded[chunk], 0));
        if (int rc = launch_gemm_umma(in_dtype, out_dtype, b_major, by_rows ? 1u : uint32_t(n),
                                      by_rows ? n : rows, shared, cols, a_dev, by_rows ? dB : b_dev, c_dev,
                                      d_dev, alpha, beta, nullptr, hp->compute))
            return rc;
        KLAS_TRY_CUDA(cudaEventRecord(hp->computed[chunk], hp->compute));
        KLAS_TRY_CUDA(cudaStreamWaitEvent(hp->out, hp->computed[chunk], 0));
        KLAS_TRY_CUDA(cudaMemcpyAsync(static_cast<char *>(D) + u0 * d_unit, d_dev, n * d_unit,
                                      cudaMemcpyDeviceToHost, hp->out));
    }
    KLAS_TRY_CUDA(cudaStreamSynchronize(hp->out));
    KLAS_TRY_CUDA(cudaStreamSynchronize(hp->in));
    return klas_b200_gemm_tc_status(nullptr);
}

int klas_b200_spmm_host(int dtype, uint32_t rows, uint32_t shared, uint32_t cols, uint32_t nnz,
                        const void *elems, const uint32_t *col_ind, const uint32_t *row_off,
                        const uint32_t *row_indices, const void *B, void *C) {
    clear_error();
    HostCallLock turn;
    if (turn.rc) return turn.rc;
    if (dtype != KLAS_F32 && dtype != KLAS_U32) return fail(KLAS_ERR_INVALID, "spmm_host: bad dtype");
    const size_t c_bytes = size_t(rows) * cols * 4;
    if (c_bytes == 0) return KLAS_OK;
    if (!C || !row_off) return fail(KLAS_ERR_INVALID, "spmm_host: null C or row_off");
    cudaStream_t s = nullptr;
    void *dE, *dCi, *dRo, *dRi = nullptr, *dB, *dC;
    if (int rc = stage_in(0, elems, size_t(nnz) * 4, s, &dE)) return rc;
    if (int rc = stage_in(1, col_ind, size_t(nnz) * 4, s, &dCi)) return rc;
    if (int rc = stage_in(2, row_off, (size_t(rows) + 1) * 4, s, &dRo)) return rc;
    if (row_indices)
        if (int rc = stage_in(3, row_indices, size_t(rows) * 4, s, &dRi)) return rc;
    if (int rc = stage_in(4, B, size_t(shared) * cols * 4, s, &dB)) return rc;
    if (int rc = workspace_reserve(5, c_bytes, &dC)) return rc;
    if (int rc = launch_spmm(dtype, rows, shared, cols, nnz, dE, static_cast<uint32_t *>(dCi),
                             static_cast<uint32_t *>(dRo), static_cast<uint32_t *>(dRi), dB, dC, s))
        return rc;
    KLAS_TRY_CUDA(cudaMemcpyAsync(C, dC, c_bytes, cudaMemcpyDeviceToHost, s));
    KLAS_TRY_CUDA(cudaStreamSynchronize(s));
    return KLAS_OK;
}

size_t klas_b200_softmax_scratch_bytes(uint64_t rows, uint64_t cols) { return softmax_scratch_bytes(rows, cols); }

int klas_b200_softmax(int dtype, int log_softmax, uint64_t rows, uint64_t cols, void *a, void *scratch,
                      size_t scratch_bytes, void *stream) {
    clear_error();
    return launch_softmax(dtype, log_softmax, rows, cols, a, scratch, scratch_bytes, static_cast<cudaStream_t>(stream));
}

int klas_b200_softmax_host(int dtype, int log_softmax, uint64_t rows, uint64_t cols, void *a) {
    clear_error();
    HostCallLock turn;
    if (turn.rc) return turn.rc;
    const size_t es = dtype_size(dtype), bytes = size_t(rows) * cols * es;
    if (es == 0) return fail(KLAS_ERR_INVALID, "softmax_host: bad dtype");
    if (bytes == 0) return KLAS_OK;
    if (!a) return fail(KLAS_ERR_INVALID, "softmax_host: null data pointer");
    cudaStream_t s = nullptr;
    void *dA, *dS;
    if (int rc = stage_in(0, a, bytes, s, &dA)) return rc;
    const size_t sb = softmax_scratch_bytes(rows, cols);
    if (int rc = workspace_reserve(1, sb, &dS)) return rc;
    if (int rc = launch_softmax(dtype, log_softmax, rows, cols, dA, dS, sb, s)) return rc;
    KLAS_TRY_CUDA(cudaMemcpyAsync(a, dA, bytes, cudaMemcpyDeviceToHost, s));
    KLAS_TRY_CUDA(cudaStreamSynchronize(s));
    return KLAS_OK;
}

int klas_b200_rowscale(int dtype, int col_major, uint64_t m, uint64_t n, const void *scale, void *b, void *stream) {
    clear_error();
    return launch_rowscale(dtype, col_major, m, n, scale, b, static_cast<cudaStream_t>(stream));
}

size_t klas_b200_reduce_scratch_bytes(uint64_t n) { return reduce_scratch_bytes(n); }

int klas_b200_reduce_sum(int dtype, uint64_t n, const void *a, void *result, void *scratch, size_t scratch_bytes,
                         void *stream) {
    clear_error();
    return launch_reduce_sum(dtype, n, a, result, scratch, scratch_bytes, static_cast<cudaStream_t>(stream));
}

int klas_b200_reduce_sum_host(int dtype, uint64_t n, const void *a, void *result) {
    clear_error();
    HostCallLock turn;
    if (turn.rc) return turn.rc;
    const size_t es = dtype_size(dtype);
    if (es == 0 || dtype == KLAS_BF16) return fail(KLAS_ERR_INVALID, "reduce_host: bad dtype");
    if (!result) return fail(KLAS_ERR_INVALID, "reduce_host: null result pointer");
    cudaStream_t s = nullptr;
    void *dS, *dOut;
    const size_t sb = reduce_scratch_bytes(n);
    if (int rc = workspace_reserve(6, sb, &dS)) return rc;
    if (int rc = workspace_reserve(7, 16, &dOut)) return rc;
    if (int rc = launch_reduce_sum(dtype, n, a, dOut, dS, sb, s)) return rc;
    KLAS_TRY_CUDA(cudaMemcpyAsync(result, dOut, es, cudaMemcpyDeviceToHost, s));
    KLAS_TRY_CUDA(cudaStreamSynchronize(s));
    return KLAS_OK;
}

// NUMA node the current device hangs off (sysfs of its PCI function), -1 when unknown.
static int device_numa_node() {
    int dev = 0;
    char bus[32] = "";
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetPCIBusId(bus, sizeof bus, dev) != cudaSuccess) return -1;
    for (char *c = bus; *c; ++c)
        if (*c >= 'A' && *c <= 'F') *c = char(*c - 'A' + 'a');
    char path[128];
    snprintf(path, sizeof path, "/sys/bus/pci/devices/%s/numa_node", bus);
    FILE *f = fopen(path, "r");
    if (!f) return -1;
    int node = -1;
    if (fscanf(f, "%d", &node) != 1) node = -1;
    fclose(f);
    return node;
}

int klas_b200_host_numa_node(void) {
    clear_error();
    return device_numa_node();
}

int klas_b200_host_bind_near_device(void) {
    clear_error();
    const int node = device_numa_node();
    if (node < 0) return fail(KLAS_ERR_UNSUPPORTED, "host_bind: the device's NUMA node is not known on this system");
    char path[128];
    snprintf(path, sizeof path, "/sys/devices/system/node/node%d/cpulist", node);
    FILE *f = fopen(path, "r");
    if (!f) return fail(KLAS_ERR_UNSUPPORTED, "host_bind: cannot read %s", path);
    cpu_set_t want, allowed, both;
    CPU_ZERO(&want);
    int lo = 0, hi = 0;
    for (;;) {   // "0-15,64-79"
        if (fscanf(f, "%d", &lo) != 1) break;
        hi = lo;
        int ch = fgetc(f);
        if (ch == '-') {
            if (fscanf(f, "%d", &hi) != 1) break;
            ch = fgetc(f);
        }
        for (int c = lo; c <= hi && c < CPU_SETSIZE; ++c) CPU_SET(c, &want);
        if (ch != ',') break;
    }
    fclose(f);
    if (sched_getaffinity(0, sizeof allowed, &allowed) != 0) return fail(KLAS_ERR_UNSUPPORTED, "host_bind: sched_getaffinity failed");
    CPU_AND(&both, &want, &allowed);
    if (CPU_COUNT(&both) == 0) return fail(KLAS_ERR_UNSUPPORTED, "host_bind: none of node %d's CPUs is available to this process", node);
    if (sched_setaffinity(0, sizeof both, &both) != 0) return fail(KLAS_ERR_UNSUPPORTED, "host_bind: sched_setaffinity failed");
    // memory allocated from now on (pinned buffers included) is taken from that node when it has room
    unsigned long mask[16] = {};
    if (node < int(sizeof mask * 8)) {
        mask[node / (8 * sizeof(unsigned long))] |= 1ul << (node % (8 * sizeof(unsigned long)));
        const long MPOL_PREFERRED = 1;
        syscall(SYS_set_mempolicy, MPOL_PREFERRED, mask, sizeof mask * 8);   // best effort: affinity alone already gives local first touch
    }
    return KLAS_OK;
}

int klas_b200_debug_set(int knob, int value) {
    clear_error();
    if (knob < 0 || knob >= KLAS_KNOB_COUNT) return fail(KLAS_ERR_INVALID, "debug_set: unknown knob %d", knob);
    if (value < g_knob_range[knob].lo || value > g_knob_range[knob].hi)
        return fail(KLAS_ERR_INVALID, "debug_set: knob %d takes values %d..%d, got %d", knob, g_knob_range[knob].lo,
                    g_knob_range[knob].hi, value);
    g_knobs[knob].store(value, std::memory_order_relaxed);
    return KLAS_OK;
}

int klas_b200_debug_get(int knob) { return debug_knob(knob); }

int klas_b200_gemm_tc_plan(uint64_t rows, uint64_t shared, uint64_t cols, uint32_t batch, int sm_count, int *kind,
                           int *tile_cols, int *k_parts, int *tail_cut) {
    clear_error();
    return umma_plan(rows, shared, cols, batch, sm_count, kind, tile_cols, k_parts, tail_cut);
}

int klas_b200_release_workspace(void) {
    clear_error();
    if (int rc = umma_release_split_workspace()) return rc;
    return workspace_release();
}

}  // extern "C"
