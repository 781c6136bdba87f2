// extern "C" entry points of liblookupffn.so (declared in include/lookupffn.h): argument checks,
// error strings, the device status word, and the two whole-layer drivers.
#include <atomic>
#include <cstring>
#include <mutex>

#include <nvtx3/nvToolsExt.h>

#include "common.cuh"

namespace lffn {

static thread_local char g_err[512] = "";

void set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

int cuda_fail(cudaError_t e, const char *what) {
    set_error("CUDA error %d (%s) in %s", (int)e, cudaGetErrorString(e), what);
    return LFFN_ERR_CUDA;
}

constexpr int MAX_DEV = 64;

// Per-device caches are atomics: two host threads that meet on the first call both compute the same value and
// either store wins.
int num_sms() {
    static std::atomic<int> cache[MAX_DEV];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEV) return 148;
    int n = cache[dev].load(std::memory_order_acquire);
    if (n == 0) {
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cache[dev].store(n, std::memory_order_release);
    }
    return n;
}

// The status word is a __device__ variable (one per device that loads the library), not an
// allocation: kernels OR flags into it, lffn_device_status reads and clears it.
__device__ uint32_t g_status_word = 0;
// lffn_device_status takes the word with one atomic exchange and parks the value in one of these slots for the
// copy to the host; concurrent readers get different slots.
constexpr int STATUS_SLOTS = 64;
__device__ uint32_t g_status_slots[STATUS_SLOTS];

__global__ void status_take_kernel(uint32_t *slot) { *slot = atomicExch(&g_status_word, 0u); }

uint32_t *status_word() {
    static std::atomic<uint32_t *> cache[MAX_DEV];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEV) return nullptr;
    uint32_t *w = cache[dev].load(std::memory_order_acquire);
    if (w == nullptr) {
        void *p = nullptr;
        if (cudaGetSymbolAddress(&p, g_status_word) != cudaSuccess) return nullptr;
        w = static_cast<uint32_t *>(p);
        cache[dev].store(w, std::memory_order_release);
    }
    return w;
}

static uint32_t *status_slot() {
    static std::atomic<uint32_t *> base[MAX_DEV];
    static std::atomic<unsigned> next{0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEV) return nullptr;
    uint32_t *b = base[dev].load(std::memory_order_acquire);
    if (b == nullptr) {
        void *p = nullptr;
        if (cudaGetSymbolAddress(&p, g_status_slots) != cudaSuccess) return nullptr;
        b = static_cast<uint32_t *>(p);
        base[dev].store(b, std::memory_order_release);
    }
    return b + next.fetch_add(1, std::memory_order_relaxed) % STATUS_SLOTS;
}

// ---- tracing (off unless lffn_trace_configure turns it on) ------------------------------------------------------
static std::atomic<uint32_t> g_trace_flags{0};

// NVTX range for the duration of an entry point's host-side work (launches are asynchronous: the range brackets
// the enqueue, which is what a timeline tool lines up with the kernels it records itself)
struct TraceRange {
    bool on;
    explicit TraceRange(const char *name) : on((g_trace_flags.load(std::memory_order_relaxed) & LFFN_TRACE_NVTX) != 0) {
        if (on) nvtxRangePushA(name);
    }
    ~TraceRange() {
        if (on) nvtxRangePop();
    }
};

// events around the two stages of the last whole-layer call on each device
struct StageEvents {
    cudaEvent_t e[3] = {nullptr, nullptr, nullptr};
    bool recorded = false;
};
static StageEvents g_stage_events[MAX_DEV];
static std::mutex g_stage_mu[MAX_DEV];

static bool stage_times_on() { return (g_trace_flags.load(std::memory_order_relaxed) & LFFN_TRACE_STAGE_TIMES) != 0; }

// records event `which` of the current device on `st`; creates the three events on first use
static int stage_event_record(int which, cudaStream_t st) {
    int dev = 0;
    LFFN_CHECK_CUDA(cudaGetDevice(&dev));
    LFFN_REQUIRE(dev >= 0 && dev < MAX_DEV, LFFN_ERR_UNSUPPORTED, "device ordinal %d", dev);
    std::lock_guard<std::mutex> lock(g_stage_mu[dev]);
    StageEvents &E = g_stage_events[dev];
    for (int i = 0; i < 3; i++)
        if (E.e[i] == nullptr) LFFN_CHECK_CUDA(cudaEventCreate(&E.e[i]));
    LFFN_CHECK_CUDA(cudaEventRecord(E.e[which], st));
    if (which == 2) E.recorded = true;
    return LFFN_OK;
}

static int check_hash_desc(const lffn_hash_desc *h, int t_begin, int t_count) {
    LFFN_REQUIRE(h != nullptr, LFFN_ERR_INVALID_ARG, "hash descriptor is NULL");
    LFFN_REQUIRE(h->proj_w != nullptr, LFFN_ERR_INVALID_ARG, "hash descriptor: proj_w is NULL");
    LFFN_REQUIRE(h->d_in >= 1 && h->D >= h->d_in && (h->D & (h->D - 1)) == 0, LFFN_ERR_INVALID_ARG,
                 "hash descriptor: need 1 <= d_in (%d) <= D (%d), D a power of two", h->d_in, h->D);
    LFFN_REQUIRE(h->D >= 64 && h->D <= 2048, LFFN_ERR_UNSUPPORTED, "hash: D = %d outside [64, 2048]", h->D);
    LFFN_REQUIRE(h->k >= 1 && h->k <= 16, LFFN_ERR_UNSUPPORTED, "hash: code length k = %d outside [1, 16]", h->k);
    LFFN_REQUIRE(h->T >= 1 && h->S >= 1 && h->R >= 1, LFFN_ERR_INVALID_ARG, "hash descriptor: T, S, R must be >= 1");
    LFFN_REQUIRE((long long)h->R * h->D >= (long long)h->T * h->k, LFFN_ERR_INVALID_ARG,
                 "hash descriptor: R*D = %lld < T*k = %lld", (long long)h->R * h->D, (long long)h->T * h->k);
    LFFN_REQUIRE(h->BS >= 1 && h->D % h->BS == 0, LFFN_ERR_INVALID_ARG, "hash descriptor: BS = %d does not divide D",
                 h->BS);
    LFFN_REQUIRE(h->bit_order == LFFN_BIT_MSB_FIRST || h->bit_order == LFFN_BIT_LSB_FIRST, LFFN_ERR_INVALID_ARG,
                 "hash descriptor: bit_order %d", h->bit_order);
    LFFN_REQUIRE(h->weight_mode >= LFFN_WEIGHT_SCORE && h->weight_mode <= LFFN_WEIGHT_SOFT_FLIP, LFFN_ERR_INVALID_ARG,
                 "hash descriptor: weight_mode %d", h->weight_mode);
    LFFN_REQUIRE(h->weight_mode != LFFN_WEIGHT_SOFT_FLIP || h->tau > 0.f, LFFN_ERR_INVALID_ARG,
                 "hash descriptor: tau must be > 0 for soft-flip weights");
    LFFN_REQUIRE(t_begin >= 0 && t_count >= 1 && t_begin + t_count <= h->T, LFFN_ERR_INVALID_ARG,
                 "table range [%d, %d) outside [0, %d)", t_begin, t_begin + t_count, h->T);
    return LFFN_OK;
}

static int check_gather(int64_t N, int I, int64_t S, int d, int table_dtype) {
    LFFN_REQUIRE(N >= 0 && I >= 0 && S >= 1 && d >= 1, LFFN_ERR_INVALID_ARG, "gather: bad sizes N=%lld I=%d S=%lld d=%d",
                 (long long)N, I, (long long)S, d);
    LFFN_REQUIRE(table_dtype == LFFN_F32 || table_dtype == LFFN_BF16, LFFN_ERR_INVALID_ARG, "gather: table dtype %d",
                 table_dtype);
    const int per = table_dtype == LFFN_F32 ? 4 : 8;
    LFFN_REQUIRE(d % per == 0, LFFN_ERR_UNSUPPORTED, "gather: d = %d must be a multiple of %d for this table dtype", d,
                 per);
    LFFN_REQUIRE(S < (1ll << 31), LFFN_ERR_UNSUPPORTED, "gather: S = %lld rows do not fit int32 indices", (long long)S);
    return LFFN_OK;
}

static int aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace lffn

using namespace lffn;

extern "C" {

int lffn_version(void) { return LFFN_VERSION; }

int lffn_trace_configure(uint32_t flags) {
    LFFN_REQUIRE((flags & ~(uint32_t)(LFFN_TRACE_NVTX | LFFN_TRACE_STAGE_TIMES)) == 0, LFFN_ERR_INVALID_ARG,
                 "trace_configure: unknown flag bits in 0x%x", flags);
    g_trace_flags.store(flags, std::memory_order_relaxed);
    return LFFN_OK;
}

int lffn_trace_last_layer_times(float *hash_ms, float *gather_ms) {
    LFFN_REQUIRE(hash_ms != nullptr && gather_ms != nullptr, LFFN_ERR_INVALID_ARG, "trace_last_layer_times: NULL output");
    int dev = 0;
    LFFN_CHECK_CUDA(cudaGetDevice(&dev));
    LFFN_REQUIRE(dev >= 0 && dev < MAX_DEV, LFFN_ERR_UNSUPPORTED, "device ordinal %d", dev);
    std::lock_guard<std::mutex> lock(g_stage_mu[dev]);
    StageEvents &E = g_stage_events[dev];
    LFFN_REQUIRE(E.recorded, LFFN_ERR_INVALID_ARG,
                 "trace_last_layer_times: no whole-layer call was made on this device with LFFN_TRACE_STAGE_TIMES on");
    LFFN_CHECK_CUDA(cudaEventSynchronize(E.e[2]));
    LFFN_CHECK_CUDA(cudaEventElapsedTime(hash_ms, E.e[0], E.e[1]));
    LFFN_CHECK_CUDA(cudaEventElapsedTime(gather_ms, E.e[1], E.e[2]));
    return LFFN_OK;
}

const char *lffn_last_error_string(void) { return g_err; }

int lffn_device_status(uint32_t *status_out, lffn_stream_t stream) {
    LFFN_REQUIRE(status_out != nullptr, LFFN_ERR_INVALID_ARG, "status_out is NULL");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    uint32_t *slot = status_slot();
    LFFN_REQUIRE(slot != nullptr, LFFN_ERR_CUDA, "no CUDA device");
    // read and clear in one atomic exchange: a flag that a kernel on another stream raises meanwhile is either in
    // this value or still in the word for the next reader, never lost
    status_take_kernel<<<1, 1, 0, st>>>(slot);
    LFFN_CHECK_CUDA(cudaGetLastError());
    LFFN_CHECK_CUDA(cudaMemcpyAsync(status_out, slot, sizeof(uint32_t), cudaMemcpyDeviceToHost, st));
    LFFN_CHECK_CUDA(cudaStreamSynchronize(st));
    return LFFN_OK;
}

int lffn_selftest_bounded_wait(int32_t poll_limit, lffn_stream_t stream) {
    LFFN_REQUIRE(poll_limit >= 1 && poll_limit <= (1 << 20), LFFN_ERR_INVALID_ARG,
                 "selftest_bounded_wait: poll_limit %d outside [1, 2^20]", poll_limit);
    return launch_bounded_wait_selftest(poll_limit, static_cast<cudaStream_t>(stream));
}

int lffn_fwht(const void *x, void *out, int64_t N, int32_t D, int32_t dtype, float scale, lffn_stream_t stream) {
    LFFN_REQUIRE(N >= 0, LFFN_ERR_INVALID_ARG, "fwht: N = %lld", (long long)N);
    if (N == 0) return LFFN_OK;  // nothing to do; empty buffers may be NULL
    LFFN_REQUIRE(x != nullptr && out != nullptr, LFFN_ERR_INVALID_ARG, "fwht: NULL buffer");
    return launch_fwht(x, out, N, D, dtype, scale, static_cast<cudaStream_t>(stream));
}

int lffn_hash_fwd_ln(const lffn_hash_desc *desc, const float *ln_gamma, const float *ln_beta, float ln_eps,
                     const void *x, int32_t x_dtype, int64_t N, int32_t t_begin, int32_t t_count, int32_t *idx_out,
                     float *w_out, float *z_out, lffn_stream_t stream) {
    TraceRange range("lffn_hash_fwd");
    int rc = check_hash_desc(desc, t_begin, t_count);
    if (rc != LFFN_OK) return rc;
    LFFN_REQUIRE(N >= 0, LFFN_ERR_INVALID_ARG, "hash_fwd: N = %lld", (long long)N);
    LFFN_REQUIRE(ln_gamma != nullptr || ln_beta == nullptr, LFFN_ERR_INVALID_ARG,
                 "hash_fwd: a LayerNorm bias without a LayerNorm weight");
    LFFN_REQUIRE(ln_gamma == nullptr || ln_eps >= 0.f, LFFN_ERR_INVALID_ARG, "hash_fwd: LayerNorm eps %g < 0", ln_eps);
    if (N == 0) return LFFN_OK;  // nothing to do; empty buffers may be NULL
    LFFN_REQUIRE(x != nullptr, LFFN_ERR_INVALID_ARG, "hash_fwd: x is NULL");
    LFFN_REQUIRE((idx_out != nullptr) == (w_out != nullptr) && (idx_out != nullptr || z_out != nullptr),
                 LFFN_ERR_INVALID_ARG, "hash_fwd: give idx_out and w_out together, or z_out alone");
    return launch_hash_fwd(*desc, x, x_dtype, N, t_begin, t_count, idx_out, w_out, z_out, ln_gamma, ln_beta, ln_eps,
                           static_cast<cudaStream_t>(stream));
}

int lffn_hash_fwd(const lffn_hash_desc *desc, const void *x, int32_t x_dtype, int64_t N, int32_t t_begin,
                  int32_t t_count, int32_t *idx_out, float *w_out, float *z_out, lffn_stream_t stream) {
    return lffn_hash_fwd_ln(desc, nullptr, nullptr, 0.f, x, x_dtype, N, t_begin, t_count, idx_out, w_out, z_out, stream);
}

int lffn_code_weights(const float *z, int64_t N, int32_t T, int32_t k, int32_t bit_order, int32_t weight_mode,
                      float tau, int32_t add_offsets, int32_t *idx_out, float *w_out, lffn_stream_t stream) {
    LFFN_REQUIRE(N >= 0 && T >= 1, LFFN_ERR_INVALID_ARG, "code_weights: bad sizes");
    LFFN_REQUIRE(N == 0 || (z != nullptr && idx_out != nullptr && w_out != nullptr), LFFN_ERR_INVALID_ARG,
                 "code_weights: NULL buffer");
    LFFN_REQUIRE(k >= 1 && k <= 16, LFFN_ERR_UNSUPPORTED, "code_weights: k = %d outside [1, 16]", k);
    LFFN_REQUIRE(bit_order == LFFN_BIT_MSB_FIRST || bit_order == LFFN_BIT_LSB_FIRST, LFFN_ERR_INVALID_ARG,
                 "code_weights: bit_order %d", bit_order);
    LFFN_REQUIRE(weight_mode >= LFFN_WEIGHT_SCORE && weight_mode <= LFFN_WEIGHT_SOFT_FLIP, LFFN_ERR_INVALID_ARG,
                 "code_weights: weight_mode %d", weight_mode);
    LFFN_REQUIRE(weight_mode != LFFN_WEIGHT_SOFT_FLIP || tau > 0.f, LFFN_ERR_INVALID_ARG, "code_weights: tau <= 0");
    if (N == 0) return LFFN_OK;
    return launch_code_weights(z, N, T, k, bit_order, weight_mode, tau, add_offsets, idx_out, w_out,
                               static_cast<cudaStream_t>(stream));
}

int lffn_code_weights_bwd(const float *z, const float *dw, int64_t N, int32_t T, int32_t k, int32_t weight_mode,
                          float tau, float *dz, lffn_stream_t stream) {
    LFFN_REQUIRE(N >= 0 && T >= 1, LFFN_ERR_INVALID_ARG, "code_weights_bwd: bad sizes");
    LFFN_REQUIRE(N == 0 || (z != nullptr && dw != nullptr && dz != nullptr), LFFN_ERR_INVALID_ARG,
                 "code_weights_bwd: NULL buffer");
    LFFN_REQUIRE(k >= 1 && k <= 16, LFFN_ERR_UNSUPPORTED, "code_weights_bwd: k = %d outside [1, 16]", k);
    LFFN_REQUIRE(weight_mode >= LFFN_WEIGHT_SCORE && weight_mode <= LFFN_WEIGHT_SOFT_FLIP, LFFN_ERR_INVALID_ARG,
                 "code_weights_bwd: weight_mode %d", weight_mode);
    LFFN_REQUIRE(weight_mode != LFFN_WEIGHT_SOFT_FLIP || tau > 0.f, LFFN_ERR_INVALID_ARG, "code_weights_bwd: tau <= 0");
    if (N == 0) return LFFN_OK;
    return launch_code_weights_bwd(z, dw, N, T, k, weight_mode, tau, dz, static_cast<cudaStream_t>(stream));
}

int lffn_gather_fwd(const int32_t *idx, const float *w, const void *tables, int32_t table_dtype, void *out,
                    int32_t out_dtype, int64_t N, int32_t I, int64_t S, int32_t d, const float *bias,
                    lffn_stream_t stream) {
    return lffn_gather_fwd_residual(idx, w, tables, table_dtype, out, out_dtype, N, I, S, d, bias, nullptr, stream);
}

int lffn_gather_fwd_residual(const int32_t *idx, const float *w, const void *tables, int32_t table_dtype, void *out,
                             int32_t out_dtype, int64_t N, int32_t I, int64_t S, int32_t d, const float *bias,
                             const void *residual, lffn_stream_t stream) {
    TraceRange range("lffn_gather_fwd");
    int rc = check_gather(N, I, S, d, table_dtype);
    if (rc != LFFN_OK) return rc;
    LFFN_REQUIRE(out_dtype == LFFN_F32 || out_dtype == LFFN_BF16, LFFN_ERR_INVALID_ARG, "gather_fwd: out dtype %d",
                 out_dtype);
    if (N == 0) return LFFN_OK;  // nothing to do; empty buffers may be NULL
    LFFN_REQUIRE(tables != nullptr && out != nullptr && (I == 0 || (idx != nullptr && w != nullptr)),
                 LFFN_ERR_INVALID_ARG, "gather_fwd: NULL buffer");
    LFFN_REQUIRE(aligned16(tables) && aligned16(out), LFFN_ERR_INVALID_ARG,
                 "gather_fwd: tables and out must be 16-byte aligned");
    return launch_gather_fwd(idx, w, tables, table_dtype, out, out_dtype, N, I, S, d, bias, residual,
                             static_cast<cudaStream_t>(stream));
}

int lffn_gather_fwd_scatter(const int32_t *idx, const float *w, const void *tables, int32_t table_dtype,
                            float *const *out_ptrs, int32_t n_owners, int64_t rows_per_owner, int32_t slab,
                            int32_t first_owner, int64_t N, int32_t I, int64_t S, int32_t d, lffn_stream_t stream) {
    int rc = check_gather(N, I, S, d, table_dtype);
    if (rc != LFFN_OK) return rc;
    LFFN_REQUIRE(n_owners >= 1 && rows_per_owner >= 1 && (int64_t)n_owners * rows_per_owner >= N, LFFN_ERR_INVALID_ARG,
                 "gather_fwd_scatter: %d owners x %lld rows do not cover N = %lld tokens", n_owners,
                 (long long)rows_per_owner, (long long)N);
    if (N == 0) return LFFN_OK;
    LFFN_REQUIRE(tables != nullptr && out_ptrs != nullptr && (I == 0 || (idx != nullptr && w != nullptr)),
                 LFFN_ERR_INVALID_ARG, "gather_fwd_scatter: NULL buffer");
    LFFN_REQUIRE(aligned16(tables), LFFN_ERR_INVALID_ARG, "gather_fwd_scatter: tables must be 16-byte aligned");
    LFFN_REQUIRE(slab >= -2 && (slab < 0 || (slab & ~LFFN_SCATTER_SLAB_BULK) < n_owners), LFFN_ERR_INVALID_ARG,
                 "gather_fwd_scatter: slab %d is neither an add mode (-1, -2) nor a slab in [0, %d)", slab, n_owners);
    LFFN_REQUIRE(first_owner >= 0 && first_owner < n_owners, LFFN_ERR_INVALID_ARG,
                 "gather_fwd_scatter: first_owner %d outside [0, %d)", first_owner, n_owners);
    return launch_gather_fwd_scatter(idx, w, tables, table_dtype, out_ptrs, rows_per_owner, slab, first_owner, N, I, S, d,
                                     static_cast<cudaStream_t>(stream));
}

int lffn_gather_bwd_weights(const int32_t *idx, const float *dy, const void *tables, int32_t table_dtype, float *dw,
                            int64_t N, int32_t I, int64_t S, int32_t d, lffn_stream_t stream) {
    TraceRange range("lffn_gather_bwd_weights");
    int rc = check_gather(N, I, S, d, table_dtype);
    if (rc != LFFN_OK) return rc;
    if (N == 0 || I == 0) return LFFN_OK;  // nothing to do; empty buffers may be NULL
    LFFN_REQUIRE(idx != nullptr && dy != nullptr && tables != nullptr && dw != nullptr, LFFN_ERR_INVALID_ARG,
                 "gather_bwd_weights: NULL buffer");
    LFFN_REQUIRE(aligned16(tables) && aligned16(dy), LFFN_ERR_INVALID_ARG,
                 "gather_bwd_weights: tables and dy must be 16-byte aligned");
    return launch_gather_bwd_weights(idx, dy, tables, table_dtype, dw, N, I, S, d, static_cast<cudaStream_t>(stream));
}

int lffn_gather_bwd_tables(const int32_t *idx, const float *w, const float *dy, float *dtables, int64_t N, int32_t I,
                           int64_t S, int32_t d, lffn_stream_t stream) {
    int rc = check_gather(N, I, S, d, LFFN_F32);
    if (rc != LFFN_OK) return rc;
    LFFN_REQUIRE(dtables != nullptr && (N == 0 || I == 0 || (idx != nullptr && w != nullptr && dy != nullptr)),
                 LFFN_ERR_INVALID_ARG, "gather_bwd_tables: NULL buffer");
    LFFN_REQUIRE(aligned16(dtables) && aligned16(dy), LFFN_ERR_INVALID_ARG,
                 "gather_bwd_tables: dtables and dy must be 16-byte aligned");
    return launch_gather_bwd_tables(idx, w, dy, dtables, N, I, S, d, static_cast<cudaStream_t>(stream));
}

size_t lffn_gather_bwd_tables_sorted_scratch_bytes(int64_t N, int32_t T, int32_t m, int32_t rows) {
    if (N < 0 || T < 1 || m < 1 || rows < 1) return 0;
    return sorted_scratch_bytes(N, T, m, rows);
}

int lffn_gather_bwd_tables_sorted(const int32_t *idx, const float *w, const float *dy, float *dtables, int64_t N,
                                  int32_t T, int32_t m, int32_t rows, int32_t d, void *scratch, size_t scratch_bytes,
                                  lffn_stream_t stream) {
    TraceRange range("lffn_gather_bwd_tables_sorted");
    LFFN_REQUIRE(T >= 1 && m >= 1 && rows >= 1, LFFN_ERR_INVALID_ARG, "gather_bwd_tables_sorted: bad T/m/rows");
    int rc = check_gather(N, T * m, (int64_t)T * rows, d, LFFN_F32);
    if (rc != LFFN_OK) return rc;
    LFFN_REQUIRE(dtables != nullptr && (N == 0 || (idx != nullptr && w != nullptr && dy != nullptr)),
                 LFFN_ERR_INVALID_ARG, "gather_bwd_tables_sorted: NULL buffer");
    LFFN_REQUIRE(aligned16(dtables) && aligned16(dy), LFFN_ERR_INVALID_ARG,
                 "gather_bwd_tables_sorted: dtables and dy must be 16-byte aligned");
    return launch_gather_bwd_tables_sorted(idx, w, dy, dtables, N, T, m, rows, d, scratch, scratch_bytes,
                                           static_cast<cudaStream_t>(stream));
}

int lffn_layer_fwd(const lffn_hash_desc *desc, const void *x, int32_t x_dtype, int64_t N, int32_t t_begin,
                   int32_t t_count, const void *tables, int32_t table_dtype, int32_t d_out, const float *bias,
                   void *out, int32_t out_dtype, int32_t *idx_ws, float *w_ws, lffn_stream_t stream) {
    return lffn_layer_fwd_ln_residual(desc, nullptr, nullptr, 0.f, x, x_dtype, N, t_begin, t_count, tables, table_dtype,
                                      d_out, bias, nullptr, out, out_dtype, idx_ws, w_ws, stream);
}

int lffn_layer_fwd_ln_residual(const lffn_hash_desc *desc, const float *ln_gamma, const float *ln_beta, float ln_eps,
                               const void *x, int32_t x_dtype, int64_t N, int32_t t_begin, int32_t t_count,
                               const void *tables, int32_t table_dtype, int32_t d_out, const float *bias,
                               const void *residual, void *out, int32_t out_dtype, int32_t *idx_ws, float *w_ws,
                               lffn_stream_t stream) {
    TraceRange range("lffn_layer_fwd");
    const bool timed = stage_times_on();
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int rc = LFFN_OK;
    if (timed && (rc = stage_event_record(0, st)) != LFFN_OK) return rc;
    rc = lffn_hash_fwd_ln(desc, ln_gamma, ln_beta, ln_eps, x, x_dtype, N, t_begin, t_count, idx_ws, w_ws, nullptr, stream);
    if (rc != LFFN_OK) return rc;
    if (timed && (rc = stage_event_record(1, st)) != LFFN_OK) return rc;
    const int m = desc->weight_mode == LFFN_WEIGHT_SOFT_FLIP ? desc->k + 1 : 1;
    rc = lffn_gather_fwd_residual(idx_ws, w_ws, tables, table_dtype, out, out_dtype, N, t_count * m,
                                  (int64_t)t_count << desc->k, d_out, bias, residual, stream);
    if (rc != LFFN_OK) return rc;
    if (timed) rc = stage_event_record(2, st);
    return rc;
}

#ifndef LFFN_HOST_LANES
#define LFFN_HOST_LANES 3
#endif
#ifndef LFFN_HOST_RAMP
#define LFFN_HOST_RAMP 1
#endif
constexpr int HOST_LANES = LFFN_HOST_LANES;  // streams alternating over token chunks in lffn_layer_fwd_host
static size_t esize(int dtype) { return dtype == LFFN_BF16 ? 2 : 4; }
static size_t up256(size_t v) { return (v + 255) & ~(size_t)255; }

size_t lffn_layer_fwd_host_ws_bytes(const lffn_hash_desc *desc, int32_t x_dtype, int32_t out_dtype, int32_t d_out,
                                    int64_t chunk_tokens) {
    if (desc == nullptr || chunk_tokens < 1) return 0;
    const int m = desc->weight_mode == LFFN_WEIGHT_SOFT_FLIP ? desc->k + 1 : 1;
    const size_t per_lane = up256((size_t)chunk_tokens * desc->d_in * esize(x_dtype)) +
                            up256((size_t)chunk_tokens * d_out * esize(out_dtype)) +
                            2 * up256((size_t)chunk_tokens * desc->T * m * 4);
    return HOST_LANES * per_lane;
}

// HOST_LANES lanes (streams) take the token chunks in turn; within a lane copy-in, the two kernels and
// copy-out are stream-ordered, and the lanes overlap each other's copies with kernels.
int lffn_layer_fwd_host(const lffn_hash_desc *desc, const void *x_host, int32_t x_dtype, int64_t N,
                        const void *tables, int32_t table_dtype, int32_t d_out, const float *bias, void *out_host,
                        int32_t out_dtype, void *ws, size_t ws_bytes, int64_t chunk_tokens, lffn_stream_t stream) {
    int rc = check_hash_desc(desc, 0, desc ? desc->T : 0);
    if (rc != LFFN_OK) return rc;
    LFFN_REQUIRE(x_host != nullptr && out_host != nullptr && tables != nullptr && ws != nullptr, LFFN_ERR_INVALID_ARG,
                 "layer_fwd_host: NULL buffer");
    LFFN_REQUIRE(chunk_tokens >= 1, LFFN_ERR_INVALID_ARG, "layer_fwd_host: chunk_tokens = %lld", (long long)chunk_tokens);
    LFFN_REQUIRE(ws_bytes >= lffn_layer_fwd_host_ws_bytes(desc, x_dtype, out_dtype, d_out, chunk_tokens),
                 LFFN_ERR_SCRATCH, "layer_fwd_host: workspace of %zu bytes needed, %zu given",
                 lffn_layer_fwd_host_ws_bytes(desc, x_dtype, out_dtype, d_out, chunk_tokens), ws_bytes);
    if (N == 0) return LFFN_OK;

    // The lanes of a device are created once and shared by all calls on that device, so one host-buffer call runs
    // at a time per device (calls on different devices do not wait for each other).
    struct Lanes {
        cudaStream_t s[HOST_LANES] = {};
        cudaEvent_t done[HOST_LANES] = {};
        cudaEvent_t start = nullptr;
        bool ready = false;
        void destroy() {
            for (int i = 0; i < HOST_LANES; i++) {
                if (done[i]) cudaEventDestroy(done[i]);
                if (s[i]) cudaStreamDestroy(s[i]);
                done[i] = nullptr;
                s[i] = nullptr;
            }
            if (start) cudaEventDestroy(start);
            start = nullptr;
        }
    };
    static Lanes lanes[MAX_DEV];
    static std::mutex mu[MAX_DEV];
    int dev = 0;
    LFFN_CHECK_CUDA(cudaGetDevice(&dev));
    LFFN_REQUIRE(dev >= 0 && dev < MAX_DEV, LFFN_ERR_UNSUPPORTED, "device ordinal %d", dev);
    std::lock_guard<std::mutex> lock(mu[dev]);
    Lanes &L = lanes[dev];
    if (!L.ready) {  // built in a local and published only when every stream and event exists
        Lanes fresh;
        cudaError_t e = cudaEventCreateWithFlags(&fresh.start, cudaEventDisableTiming);
        for (int i = 0; i < HOST_LANES && e == cudaSuccess; i++) {
            e = cudaStreamCreateWithFlags(&fresh.s[i], cudaStreamNonBlocking);
            if (e == cudaSuccess) e = cudaEventCreateWithFlags(&fresh.done[i], cudaEventDisableTiming);
        }
        if (e != cudaSuccess) {
            fresh.destroy();
            return cuda_fail(e, "creating the streams of lffn_layer_fwd_host");
        }
        L = fresh;
        L.ready = true;
    }
    cudaStream_t user = static_cast<cudaStream_t>(stream);
    LFFN_CHECK_CUDA(cudaEventRecord(L.start, user));
    const int m = desc->weight_mode == LFFN_WEIGHT_SOFT_FLIP ? desc->k + 1 : 1;
    const size_t xb = up256((size_t)chunk_tokens * desc->d_in * esize(x_dtype));
    const size_t ob = up256((size_t)chunk_tokens * d_out * esize(out_dtype));
    const size_t ib = up256((size_t)chunk_tokens * desc->T * m * 4);
    const size_t per_lane = xb + ob + 2 * ib;
    // From the first enqueue on, an error must not return while copies into out_host may still be in flight:
    // every exit below goes through `finish`, which waits for all lanes.
    auto finish = [&](int code) -> int {
        for (int i = 0; i < HOST_LANES; i++) {
            const cudaError_t e = cudaStreamSynchronize(L.s[i]);
            if (e != cudaSuccess && code == LFFN_OK) code = cuda_fail(e, "cudaStreamSynchronize(lane)");
        }
        return code;
    };
#define LFFN_HOST_CUDA(expr)                                          \
    do {                                                              \
        cudaError_t _e = (expr);                                      \
        if (_e != cudaSuccess) return finish(cuda_fail(_e, #expr));   \
    } while (0)
    for (int i = 0; i < HOST_LANES; i++) LFFN_HOST_CUDA(cudaStreamWaitEvent(L.s[i], L.start, 0));
    // Chunks are chunk_tokens long, except at the two ends of the call: the first two and the last two are half as
    // long, so that the first copy-in and the last copy-out, which nothing can overlap, are short while the chunks in
    // between amortise their launches.
    const int64_t half = (chunk_tokens + 1) / 2;
    int64_t c = 0, nt = 0;
    for (int64_t n0 = 0; n0 < N; n0 += nt, c++) {
        const int lane = (int)(c % HOST_LANES);
        const int64_t left = N - n0;
#if LFFN_HOST_RAMP
        nt = (c < 2 || left <= chunk_tokens) ? half : chunk_tokens;
#else
        nt = chunk_tokens;
#endif
        if (nt > left) nt = left;
        char *base = static_cast<char *>(ws) + lane * per_lane;
        void *xd = base;
        void *od = base + xb;
        int32_t *iw = reinterpret_cast<int32_t *>(base + xb + ob);
        float *ww = reinterpret_cast<float *>(base + xb + ob + ib);
        const char *xs = static_cast<const char *>(x_host) + (size_t)n0 * desc->d_in * esize(x_dtype);
        char *os = static_cast<char *>(out_host) + (size_t)n0 * d_out * esize(out_dtype);
        LFFN_HOST_CUDA(cudaMemcpyAsync(xd, xs, (size_t)nt * desc->d_in * esize(x_dtype), cudaMemcpyHostToDevice, L.s[lane]));
        rc = lffn_layer_fwd(desc, xd, x_dtype, nt, 0, desc->T, tables, table_dtype, d_out, bias, od, out_dtype, iw, ww,
                            L.s[lane]);
        if (rc != LFFN_OK) return finish(rc);
        LFFN_HOST_CUDA(cudaMemcpyAsync(os, od, (size_t)nt * d_out * esize(out_dtype), cudaMemcpyDeviceToHost, L.s[lane]));
    }
    for (int i = 0; i < HOST_LANES; i++) {
        LFFN_HOST_CUDA(cudaEventRecord(L.done[i], L.s[i]));
        LFFN_HOST_CUDA(cudaStreamWaitEvent(user, L.done[i], 0));
    }
#undef LFFN_HOST_CUDA
    LFFN_CHECK_CUDA(cudaStreamSynchronize(user));
    return LFFN_OK;
}

}  // extern "C"
