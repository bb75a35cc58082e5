// extern "C" entry points of libnott_b200.so: argument validation, then the
// launchers.  Declarations and the reference interfaces they replace are in
// include/nott_b200.h.
#include <atomic>
#include <stdarg.h>
#include <string.h>
#include "launchers.h"

namespace nb2 {

static thread_local char g_err[512] = "ok";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

int cuda_status(cudaError_t e, const char* what) {
    if (e == cudaSuccess) return 0;
    set_error("%s: %s (%s)", what, cudaGetErrorString(e), cudaGetErrorName(e));
    return (int)e;
}

int sm_count() {
    static thread_local int cached_dev = -1, cached_sms = 0;
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (dev != cached_dev) {
        int sms = 0;
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
        cached_dev = dev;
        cached_sms = sms;
    }
    return cached_sms;
}

// SMs the persistent norm kernels size their grids for: all of them, less the number a caller set
// aside for a kernel of its own that runs beside them (a collective on another stream).  Those
// kernels give every CTA a fixed share of the rows, so a CTA that finds no free SM at launch would
// run after the others and nearly double the kernel's time.
static std::atomic<int> g_reserved_sms{0};
int launch_sms() {
    const int sms = sm_count() - g_reserved_sms.load(std::memory_order_relaxed);
    return sms < 1 ? 1 : sms;
}
int exchange_reserved_sms(int n) { return g_reserved_sms.exchange(n < 0 ? 0 : n, std::memory_order_relaxed); }

int current_device_slot() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0) dev = 0;
    return dev % kMaxDevices;
}

// One status word per device: the ring kernels record here (code << 16 | CTA) when a
// bounded wait gives up.  The symbol's device address is looked up once per device.
__device__ unsigned int g_device_status[4];
unsigned int* device_status_ptr() {
    static thread_local unsigned int* ptrs[kMaxDevices] = {};
    unsigned int*& p = ptrs[current_device_slot()];
    if (p == nullptr) {
        void* addr = nullptr;
        if (cudaGetSymbolAddress(&addr, g_device_status) == cudaSuccess) p = static_cast<unsigned int*>(addr);
    }
    return p;
}

// A side stream and two events per host thread and device, for work that may run beside the
// caller's stream (forked and joined with events, which a stream capture follows as well).
// Never created while the caller's stream is capturing: the caller then gets nullptr and runs
// the work in line.
struct SideStream { cudaStream_t stream; cudaEvent_t fork, join, fork2, join2; };
static SideStream* side_stream(cudaStream_t user) {
    static thread_local SideStream streams[kMaxDevices] = {};
    static thread_local bool ready[kMaxDevices] = {};
    const int slot = current_device_slot();
    if (!ready[slot]) {
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(user, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) return nullptr;
        SideStream s = {};
        if (cudaStreamCreateWithFlags(&s.stream, cudaStreamNonBlocking) != cudaSuccess) return nullptr;
        if (cudaEventCreateWithFlags(&s.fork, cudaEventDisableTiming) != cudaSuccess ||
            cudaEventCreateWithFlags(&s.join, cudaEventDisableTiming) != cudaSuccess ||
            cudaEventCreateWithFlags(&s.fork2, cudaEventDisableTiming) != cudaSuccess ||
            cudaEventCreateWithFlags(&s.join2, cudaEventDisableTiming) != cudaSuccess) {
            (void)cudaGetLastError();
            return nullptr;
        }
        streams[slot] = s;
        ready[slot] = true;
    }
    return &streams[slot];
}

static bool dtype_ok(int d) { return d == NB2_F32 || d == NB2_BF16; }
static bool act_ok(int a) { return a == NB2_ACT_NONE || a == NB2_ACT_GELU || a == NB2_ACT_SILU; }
static bool idx_ok(int i) { return i == NB2_I32 || i == NB2_I64; }

static int require_device() {
    const int sms = sm_count();
    if (sms > 0) return 0;
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) e = cudaErrorNoDevice;
    return cuda_status(e, "no usable CUDA device (this library has no CPU fallback)");
}

static int norm_fwd(bool rms, const void* x, const void* gamma, const void* beta, void* y, float* mean,
                    float* rstd, int64_t rows, int64_t D, double eps, int dtype, int act, void* stream,
                    const void* res = nullptr, void* sum_out = nullptr) {
    NB2_REQUIRE(dtype_ok(dtype), NB2_ERR_DTYPE, "norm fwd: unknown dtype %d", dtype);
    NB2_REQUIRE(act_ok(act), NB2_ERR_DTYPE, "norm fwd: unknown activation %d", act);
    NB2_REQUIRE(rows >= 0 && D > 0, NB2_ERR_SHAPE, "norm fwd: rows=%lld D=%lld (need rows >= 0, D > 0)", (long long)rows, (long long)D);
    NB2_REQUIRE(D < ((int64_t)1 << 31), NB2_ERR_SHAPE, "norm fwd: D=%lld exceeds 2^31-1", (long long)D);
    if (rows == 0) return 0;
    NB2_REQUIRE(x != nullptr && y != nullptr, NB2_ERR_NULL, "norm fwd: x or y is NULL");
    int rc = require_device();
    if (rc != 0) return rc;
    NormArgs a{};
    a.x = x; a.gamma = gamma; a.beta = rms ? nullptr : beta; a.y = y;
    a.mean_out = mean; a.rstd_out = rstd; a.rows = rows; a.D = D; a.eps = (float)eps;
    a.act = act; a.rms = rms; a.stream = (cudaStream_t)stream;
    a.res = res; a.sum_out = sum_out;
    auto run = [&](const NormArgs& n) {
        if (dtype == NB2_F32) return rms ? launch_norm_fwd<float, true>(n) : launch_norm_fwd<float, false>(n);
        return rms ? launch_norm_fwd<__nv_bfloat16, true>(n) : launch_norm_fwd<__nv_bfloat16, false>(n);
    };
    rc = run(a);
    if (rc == kNotFused) {
        // no fused residual kernel for this shape: the sum in one pass, the norm of the sum in another
        rc = launch_add(x, res, sum_out, rows * D, dtype, (cudaStream_t)stream);
        if (rc != 0) return rc;
        a.x = sum_out; a.res = nullptr; a.sum_out = nullptr;
        rc = run(a);
    }
    return rc;
}

static int norm_bwd(bool rms, const void* x, const void* dy, const void* gamma, const void* beta,
                    const float* mean, const float* rstd, void* dx, float* partials, int64_t* n_partials,
                    int64_t rows, int64_t D, int dtype, int act, void* stream, const void* dres = nullptr) {
    NB2_REQUIRE(dtype_ok(dtype), NB2_ERR_DTYPE, "norm bwd: unknown dtype %d", dtype);
    NB2_REQUIRE(act_ok(act), NB2_ERR_DTYPE, "norm bwd: unknown activation %d", act);
    NB2_REQUIRE(rows >= 0 && D > 0, NB2_ERR_SHAPE, "norm bwd: rows=%lld D=%lld (need rows >= 0, D > 0)", (long long)rows, (long long)D);
    NB2_REQUIRE(D < ((int64_t)1 << 31), NB2_ERR_SHAPE, "norm bwd: D=%lld exceeds 2^31-1", (long long)D);
    if (n_partials) *n_partials = 0;
    if (rows == 0) return 0;
    NB2_REQUIRE(x && dy && dx && rstd && (rms || mean), NB2_ERR_NULL, "norm bwd: x, dy, dx, rstd%s must be non-NULL", rms ? "" : ", mean");
    NB2_REQUIRE(partials == nullptr || n_partials != nullptr, NB2_ERR_NULL, "norm bwd: partials given but n_partials_host is NULL");
    int rc = require_device();
    if (rc != 0) return rc;
    NormArgs a{};
    a.x = x; a.dy = dy; a.gamma = gamma; a.beta = rms ? nullptr : beta; a.mean = mean; a.rstd = rstd;
    a.dx = dx; a.partials = partials; a.rows = rows; a.D = D; a.act = act; a.rms = rms;
    a.stream = (cudaStream_t)stream;
    a.dres = dres;
    auto run = [&](const NormArgs& n) {
        if (dtype == NB2_F32) return rms ? launch_norm_bwd<float, true>(n, n_partials) : launch_norm_bwd<float, false>(n, n_partials);
        return rms ? launch_norm_bwd<__nv_bfloat16, true>(n, n_partials) : launch_norm_bwd<__nv_bfloat16, false>(n, n_partials);
    };
    rc = run(a);
    if (rc == kNotFused) {
        a.dres = nullptr;
        rc = run(a);
        if (rc != 0) return rc;
        rc = launch_add(dx, dres, dx, rows * D, dtype, (cudaStream_t)stream);
    }
    return rc;
}

}  // namespace nb2

using namespace nb2;

extern "C" {

int nb2_abi_version(void) { return NB2_ABI_VERSION; }
const char* nb2_last_error_string(void) { return g_err; }
int nb2_reserve_sms(int n) { return exchange_reserved_sms(n); }
int nb2_attention_softmax_order(int order) {
    const int before = set_softmax_order(order);
    NB2_REQUIRE(before >= 0, NB2_ERR_SHAPE, "attention softmax order: %d is not 0, 1 or 2", order);
    return before;
}
int nb2_sm_count(void) { return sm_count(); }

int nb2_device_status(unsigned int* status_host, int clear) {
    NB2_REQUIRE(status_host != nullptr, NB2_ERR_NULL, "device status: NULL output");
    unsigned int* p = device_status_ptr();
    if (p == nullptr) return cuda_status(cudaGetLastError(), "device status word lookup");
    int rc = cuda_status(cudaMemcpy(status_host, p, sizeof(unsigned int), cudaMemcpyDeviceToHost), "device status read");
    if (rc != 0) return rc;
    if (clear && *status_host != 0) rc = cuda_status(cudaMemset(p, 0, sizeof(unsigned int)), "device status clear");
    if (rc != 0) return rc;
    if (*status_host != 0) {
        set_error("a kernel gave up waiting: code %u in CTA %u (1 = a requested row never arrived in shared memory, 3 = the bounded-wait self-test, 4 = a peer rank's gradient slot never arrived)",
                  *status_host >> 16, *status_host & 0xffffu);
        return NB2_ERR_DEVICE;
    }
    return 0;
}

size_t nb2_workspace_bytes(int op, int64_t a, int64_t b, int dtype) {
    switch (op) {
        case NB2_WS_NORM_BWD: {
            // a = rows, b = D.  Upper bound over LayerNorm (2 partial rows) and both paths.
            if (a <= 0 || b <= 0) return 256;
            int sms = sm_count();
            if (sms <= 0) sms = 148;
            const int epv = dtype == NB2_BF16 ? 8 : 4;
            const int vpt = 16 / epv;
            int64_t parts = norm_bwd_generic_parts(a);
            if (b % epv == 0) {
                const int tpr = pick_tpr(b / epv, vpt);
                if (tpr != 0) {
                    const int64_t g = norm_bwd_grid(a, tpr, sms);
                    if (g > parts) parts = g;
                }
            }
            return (size_t)parts * 2 * (size_t)b * sizeof(float) + 256;
        }
        case NB2_WS_EMBEDDING_BWD: return embedding_bwd_workspace(a, b);
        case NB2_WS_BERT_EMBEDDING_BWD: {
            // a = B << 32 | S, b = vocab << 32 | D
            const int64_t B = a >> 32, S = a & 0xffffffffLL, vocab = b >> 32, D = b & 0xffffffffLL;
            if (a < 0 || vocab <= 0 || D <= 0) return 0;
            const int64_t tokens = B * S;
            const size_t norm_ws = (nb2_workspace_bytes(NB2_WS_NORM_BWD, tokens, D, dtype) + 255) & ~(size_t)255;
            const size_t type_ws = ((size_t)(S + 1) * D * sizeof(float) + 255) & ~(size_t)255;
            return norm_ws + type_ws + embedding_bwd_workspace(tokens, vocab) + 512;
        }
        case NB2_WS_LINEAR: return (size_t)1 << 20;
        case NB2_WS_ROPE_TABLE: return a > 0 && b > 1 ? (size_t)a * (size_t)(b / 2) * 2 * sizeof(float) : 0;
        default: return 0;
    }
}

int nb2_layernorm_fwd(const void* x, const void* gamma, const void* beta, void* y, float* mean, float* rstd,
                      int64_t rows, int64_t D, double eps, int dtype, int act, void* stream) {
    return norm_fwd(false, x, gamma, beta, y, mean, rstd, rows, D, eps, dtype, act, stream);
}
int nb2_layernorm_bwd(const void* x, const void* dy, const void* gamma, const void* beta, const float* mean,
                      const float* rstd, void* dx, float* partials, int64_t* n_partials_host,
                      int64_t rows, int64_t D, int dtype, int act, void* stream) {
    return norm_bwd(false, x, dy, gamma, beta, mean, rstd, dx, partials, n_partials_host, rows, D, dtype, act, stream);
}
int nb2_rmsnorm_fwd(const void* x, const void* weight, void* y, float* rstd, int64_t rows, int64_t D,
                    double eps, int dtype, int act, void* stream) {
    return norm_fwd(true, x, weight, nullptr, y, nullptr, rstd, rows, D, eps, dtype, act, stream);
}
int nb2_rmsnorm_bwd(const void* x, const void* dy, const void* weight, const float* rstd, void* dx,
                    float* partials, int64_t* n_partials_host, int64_t rows, int64_t D, int dtype, int act,
                    void* stream) {
    return norm_bwd(true, x, dy, weight, nullptr, nullptr, rstd, dx, partials, n_partials_host, rows, D, dtype, act, stream);
}

int nb2_add_layernorm_fwd(const void* a, const void* b, const void* gamma, const void* beta, void* sum_out, void* y,
                          float* mean, float* rstd, int64_t rows, int64_t D, double eps, int dtype, void* stream) {
    NB2_REQUIRE(rows == 0 || (b != nullptr && sum_out != nullptr), NB2_ERR_NULL, "add+layernorm fwd: b or sum_out is NULL");
    return norm_fwd(false, a, gamma, beta, y, mean, rstd, rows, D, eps, dtype, NB2_ACT_NONE, stream, b, sum_out);
}
int nb2_add_layernorm_bwd(const void* sum, const void* dy, const void* dsum, const void* gamma, const float* mean,
                          const float* rstd, void* dx, float* partials, int64_t* n_partials_host, int64_t rows,
                          int64_t D, int dtype, void* stream) {
    return norm_bwd(false, sum, dy, gamma, nullptr, mean, rstd, dx, partials, n_partials_host, rows, D, dtype,
                    NB2_ACT_NONE, stream, dsum);
}
int nb2_add_rmsnorm_fwd(const void* a, const void* b, const void* weight, void* sum_out, void* y, float* rstd,
                        int64_t rows, int64_t D, double eps, int dtype, void* stream) {
    NB2_REQUIRE(rows == 0 || (b != nullptr && sum_out != nullptr), NB2_ERR_NULL, "add+rmsnorm fwd: b or sum_out is NULL");
    return norm_fwd(true, a, weight, nullptr, y, nullptr, rstd, rows, D, eps, dtype, NB2_ACT_NONE, stream, b, sum_out);
}
int nb2_add_rmsnorm_bwd(const void* sum, const void* dy, const void* dsum, const void* weight, const float* rstd,
                        void* dx, float* partials, int64_t* n_partials_host, int64_t rows, int64_t D, int dtype,
                        void* stream) {
    return norm_bwd(true, sum, dy, weight, nullptr, nullptr, rstd, dx, partials, n_partials_host, rows, D, dtype,
                    NB2_ACT_NONE, stream, dsum);
}

int nb2_colreduce_partials(const float* partials, int64_t n_partials, int64_t ncols, float* out, void* stream) {
    NB2_REQUIRE(n_partials >= 0 && ncols >= 0, NB2_ERR_SHAPE, "colreduce: n_partials=%lld ncols=%lld", (long long)n_partials, (long long)ncols);
    NB2_REQUIRE(n_partials < ((int64_t)1 << 31), NB2_ERR_SHAPE, "colreduce: too many partials");
    if (ncols == 0) return 0;
    NB2_REQUIRE(out != nullptr && (partials != nullptr || n_partials == 0), NB2_ERR_NULL, "colreduce: NULL pointer");
    int rc = require_device();
    if (rc != 0) return rc;
    return launch_colreduce(partials, n_partials, ncols, out, (cudaStream_t)stream);
}

int nb2_act_fwd(const void* x, void* y, int64_t n, int dtype, int act, void* stream) {
    NB2_REQUIRE(dtype_ok(dtype) && act_ok(act), NB2_ERR_DTYPE, "act fwd: dtype=%d act=%d", dtype, act);
    NB2_REQUIRE(n >= 0, NB2_ERR_SHAPE, "act fwd: n=%lld", (long long)n);
    if (n == 0) return 0;
    NB2_REQUIRE(x && y, NB2_ERR_NULL, "act fwd: NULL pointer");
    int rc = require_device();
    if (rc != 0) return rc;
    return launch_act(x, nullptr, y, n, dtype, act, false, (cudaStream_t)stream);
}
int nb2_act_bwd(const void* x, const void* dy, void* dx, int64_t n, int dtype, int act, void* stream) {
    NB2_REQUIRE(dtype_ok(dtype) && act_ok(act), NB2_ERR_DTYPE, "act bwd: dtype=%d act=%d", dtype, act);
    NB2_REQUIRE(n >= 0, NB2_ERR_SHAPE, "act bwd: n=%lld", (long long)n);
    if (n == 0) return 0;
    NB2_REQUIRE(x && dy && dx, NB2_ERR_NULL, "act bwd: NULL pointer");
    int rc = require_device();
    if (rc != 0) return rc;
    return launch_act(x, dy, dx, n, dtype, act, true, (cudaStream_t)stream);
}

int nb2_silu_gate_fwd(const void* a, int64_t lda, const void* b, int64_t ldb, void* out, int64_t ldo,
                      int64_t rows, int64_t H, int dtype, void* stream) {
    NB2_REQUIRE(dtype_ok(dtype), NB2_ERR_DTYPE, "silu gate fwd: dtype=%d", dtype);
    NB2_REQUIRE(rows >= 0 && H >= 0, NB2_ERR_SHAPE, "silu gate fwd: rows=%lld H=%lld", (long long)rows, (long long)H);
    if (rows == 0 || H == 0) return 0;
    NB2_REQUIRE(lda >= H && ldb >= H && ldo >= H, NB2_ERR_SHAPE, "silu gate fwd: a row stride is smaller than H=%lld", (long long)H);
    NB2_REQUIRE(a && b && out, NB2_ERR_NULL, "silu gate fwd: NULL pointer");
    int rc = require_device();
    if (rc != 0) return rc;
    return launch_silu_gate(a, lda, b, ldb, nullptr, 0, out, ldo, nullptr, 0, rows, H, dtype, false, (cudaStream_t)stream);
}
int nb2_silu_gate_bwd(const void* a, int64_t lda, const void* b, int64_t ldb, const void* dy, int64_t lddy,
                      void* da, int64_t ldda, void* db, int64_t lddb, int64_t rows, int64_t H, int dtype,
                      void* stream) {
    NB2_REQUIRE(dtype_ok(dtype), NB2_ERR_DTYPE, "silu gate bwd: dtype=%d", dtype);
    NB2_REQUIRE(rows >= 0 && H >= 0, NB2_ERR_SHAPE, "silu gate bwd: rows=%lld H=%lld", (long long)rows, (long long)H);
    if (rows == 0 || H == 0) return 0;
    NB2_REQUIRE(lda >= H && ldb >= H && lddy >= H && ldda >= H && lddb >= H, NB2_ERR_SHAPE,
                "silu gate bwd: a row stride is smaller than H=%lld", (long long)H);
    NB2_REQUIRE(a && b && dy && da && db, NB2_ERR_NULL, "silu gate bwd: NULL pointer");
    int rc = require_device();
    if (rc != 0) return rc;
    return launch_silu_gate(a, lda, b, ldb, dy, lddy, da, ldda, db, lddb, rows, H, dtype, true, (cudaStream_t)stream);
}

int nb2_embedding_fwd(const void* table, const void* ids, void* out, int64_t tokens, int64_t vocab, int64_t D,
                      int dtype, int index_type, int64_t* status, void* stream) {
    NB2_REQUIRE(dtype_ok(dtype) && idx_ok(index_type), NB2_ERR_DTYPE, "embedding fwd: dtype=%d index_type=%d", dtype, index_type);
    NB2_REQUIRE(tokens >= 0 && vocab > 0 && D > 0, NB2_ERR_SHAPE, "embedding fwd: tokens=%lld vocab=%lld D=%lld", (long long)tokens, (long long)vocab, (long long)D);
    if (tokens == 0) return 0;
    NB2_REQUIRE(table && ids && out, NB2_ERR_NULL, "embedding fwd: NULL pointer");
    int rc = require_device();
    if (rc != 0) return rc;
    return launch_embedding_fwd(table, ids, out, tokens, vocab, D, dtype, index_type, status, (cudaStream_t)stream);
}
int nb2_embedding_bwd(const void* dout, const void* ids, void* dtable, int64_t tokens, int64_t vocab, int64_t D,
                      int dtype, int index_type, void* workspace, size_t workspace_bytes, void* stream) {
    NB2_REQUIRE(dtype_ok(dtype) && idx_ok(index_type), NB2_ERR_DTYPE, "embedding bwd: dtype=%d index_type=%d", dtype, index_type);
    NB2_REQUIRE(tokens >= 0 && vocab > 0 && vocab < ((int64_t)1 << 31) && D > 0, NB2_ERR_SHAPE,
                "embedding bwd: tokens=%lld vocab=%lld D=%lld", (long long)tokens, (long long)vocab, (long long)D);
    NB2_REQUIRE(dtable && (tokens == 0 || (dout && ids)), NB2_ERR_NULL, "embedding bwd: NULL pointer");
    int rc = require_device();
    if (rc != 0) return rc;
    return launch_embedding_bwd(dout, ids, dtable, tokens, vocab, D, dtype, index_type, workspace, workspace_bytes, (cudaStream_t)stream);
}

int nb2_embedding_index(const void* ids, int64_t tokens, int64_t vocab, int index_type, void* workspace,
                        size_t workspace_bytes, void* stream) {
    NB2_REQUIRE(idx_ok(index_type), NB2_ERR_DTYPE, "embedding index: index_type=%d", index_type);
    NB2_REQUIRE(tokens >= 0 && vocab > 0 && vocab < ((int64_t)1 << 31), NB2_ERR_SHAPE, "embedding index: tokens=%lld vocab=%lld",
                (long long)tokens, (long long)vocab);
    if (tokens == 0) return 0;
    NB2_REQUIRE(ids != nullptr, NB2_ERR_NULL, "embedding index: NULL ids");
    int rc = require_device();
    if (rc != 0) return rc;
    return launch_embedding_bwd_index(ids, tokens, vocab, index_type, workspace, workspace_bytes, (cudaStream_t)stream);
}
int nb2_embedding_bwd_indexed(const void* dout, void* dtable, int64_t tokens, int64_t vocab, int64_t D, int dtype,
                              void* workspace, size_t workspace_bytes, void* stream) {
    NB2_REQUIRE(dtype_ok(dtype), NB2_ERR_DTYPE, "embedding bwd: dtype=%d", dtype);
    NB2_REQUIRE(tokens >= 0 && vocab > 0 && vocab < ((int64_t)1 << 31) && D > 0, NB2_ERR_SHAPE,
                "embedding bwd: tokens=%lld vocab=%lld D=%lld", (long long)tokens, (long long)vocab, (long long)D);
    NB2_REQUIRE(dtable && (tokens == 0 || (dout && workspace)), NB2_ERR_NULL, "embedding bwd: NULL pointer");
    NB2_REQUIRE(tokens == 0 || workspace_bytes >= embedding_bwd_workspace(tokens, vocab), NB2_ERR_WORKSPACE,
                "embedding bwd: workspace %zu < required %zu", workspace_bytes, embedding_bwd_workspace(tokens, vocab));
    int rc = require_device();
    if (rc != 0) return rc;
    return launch_embedding_bwd_sum(dout, dtable, tokens, vocab, D, dtype, workspace, (cudaStream_t)stream);
}

int nb2_bert_embedding_ln_fwd(const void* word, const void* pos, const void* type, const void* ids, const void* gamma,
                              const void* beta, void* sum_out, void* y, float* mean, float* rstd, int64_t B, int64_t S,
                              int64_t vocab, int64_t D, double eps, int dtype, int index_type, int64_t* status,
                              void* stream) {
    NB2_REQUIRE(dtype_ok(dtype) && idx_ok(index_type), NB2_ERR_DTYPE, "bert embedding fwd: dtype=%d index_type=%d", dtype, index_type);
    NB2_REQUIRE(B >= 0 && S >= 0 && vocab > 0 && D > 0 && D < ((int64_t)1 << 31), NB2_ERR_SHAPE,
                "bert embedding fwd: B=%lld S=%lld vocab=%lld D=%lld", (long long)B, (long long)S, (long long)vocab, (long long)D);
    if (B == 0 || S == 0) return 0;
    NB2_REQUIRE(word && gamma && beta && y, NB2_ERR_NULL, "bert embedding fwd: word, gamma, beta and y must be non-NULL");
    if (ids == nullptr) vocab = B * S;          // ready-made embeddings: row t of `word` belongs to token t
    int rc = require_device();
    if (rc != 0) return rc;
    // Preferred: the ring kernel of the residual-add norm with a row lookup (word rows by id as x,
    // position rows repeating with S as the residual, the type row as a constant).  It needs a second
    // streamed source, so without position embeddings the type row plays that part (period 1).
    if (pos != nullptr || type != nullptr) {
        NormArgs a{};
        a.x = word; a.gamma = gamma; a.beta = beta; a.y = y; a.sum_out = sum_out;
        a.mean_out = mean; a.rstd_out = rstd; a.rows = B * S; a.D = D; a.eps = (float)eps;
        a.act = NB2_ACT_NONE; a.rms = false; a.stream = (cudaStream_t)stream;
        a.res = pos != nullptr ? pos : type;
        a.gather.ids = ids; a.gather.vocab = vocab; a.gather.ids_are_i32 = index_type == NB2_I32;
        a.gather.res_period = pos != nullptr ? S : 1;
        a.gather.extra = pos != nullptr ? type : nullptr;
        a.gather.status = status;
        rc = dtype == NB2_F32 ? launch_norm_fwd<float, false>(a) : launch_norm_fwd<__nv_bfloat16, false>(a);
        if (rc != kNotFused) return rc;
    }
    return launch_bert_embed_ln_fwd(word, pos, type, ids, gamma, beta, sum_out, y, mean, rstd, B, S, vocab, D, (float)eps,
                                    dtype, index_type, status, (cudaStream_t)stream);
}

int nb2_bert_embedding_ln_bwd(const void* sum, const void* dy, const void* ids, const void* gamma, const float* mean,
                              const float* rstd, void* dsum, void* dword, void* dpos, int64_t pos_rows, void* dtype0,
                              float* dgamma_dbeta, int64_t B, int64_t S, int64_t vocab, int64_t D, int dtype,
                              int index_type, void* workspace, size_t workspace_bytes, void* stream) {
    NB2_REQUIRE(dtype_ok(dtype) && idx_ok(index_type), NB2_ERR_DTYPE, "bert embedding bwd: dtype=%d index_type=%d", dtype, index_type);
    NB2_REQUIRE(B >= 0 && S >= 0 && B < ((int64_t)1 << 31) && S < ((int64_t)1 << 31) && vocab > 0 && D > 0 &&
                    D < ((int64_t)1 << 31) && pos_rows >= (dpos ? S : 0), NB2_ERR_SHAPE,
                "bert embedding bwd: B=%lld S=%lld vocab=%lld D=%lld pos_rows=%lld", (long long)B, (long long)S,
                (long long)vocab, (long long)D, (long long)pos_rows);
    NB2_REQUIRE(sum && dy && gamma && mean && rstd && dsum && (dword || !ids) && dgamma_dbeta && workspace, NB2_ERR_NULL,
                "bert embedding bwd: a required pointer is NULL");
    const int64_t tokens = B * S;
    const size_t need = nb2_workspace_bytes(NB2_WS_BERT_EMBEDDING_BWD, B * ((int64_t)1 << 32) + S, vocab * ((int64_t)1 << 32) + D, dtype);
    NB2_REQUIRE(workspace_bytes >= need, NB2_ERR_WORKSPACE, "bert embedding bwd: workspace %zu < required %zu", workspace_bytes, need);
    int rc = require_device();
    if (rc != 0) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    const size_t elt = dtype == NB2_F32 ? 4 : 2;
    // workspace: [norm partials | (S + 1) * D floats for the token-type sum | embedding sort scratch]
    uint8_t* base = (uint8_t*)(((uintptr_t)workspace + 255) & ~(uintptr_t)255);
    const size_t norm_ws = (nb2_workspace_bytes(NB2_WS_NORM_BWD, tokens, D, dtype) + 255) & ~(size_t)255;
    float* partials = (float*)base;
    float* type_scratch = (float*)(base + norm_ws);
    const size_t type_ws = ((size_t)(S + 1) * D * sizeof(float) + 255) & ~(size_t)255;
    void* sort_ws = base + norm_ws + type_ws;
    const size_t sort_bytes = embedding_bwd_workspace(tokens, vocab);
    if (dpos != nullptr) {
        rc = cuda_status(cudaMemsetAsync(dpos, 0, (size_t)pos_rows * D * elt, st), "bert embedding bwd: clearing the position gradient");
        if (rc != 0) return rc;
    }
    if (tokens == 0) {
        if (ids != nullptr) rc = cuda_status(cudaMemsetAsync(dword, 0, (size_t)vocab * D * elt, st), "bert embedding bwd memset");
        if (rc == 0) rc = cuda_status(cudaMemsetAsync(dgamma_dbeta, 0, (size_t)2 * D * 4, st), "bert embedding bwd memset");
        if (rc == 0 && dtype0) rc = cuda_status(cudaMemsetAsync(dtype0, 0, (size_t)D * elt, st), "bert embedding bwd memset");
        return rc;
    }
    // The sort of the ids does not depend on the gradient: it runs on a side stream while the
    // LayerNorm backward streams the activations, and joins before the row sums need it.
    // ids == NULL: the input was ready-made embeddings, dsum is its gradient and there is no word table
    SideStream* side = ids != nullptr ? side_stream(st) : nullptr;
    if (side != nullptr) {
        rc = cuda_status(cudaEventRecord(side->fork, st), "bert embedding bwd: fork");
        if (rc == 0) rc = cuda_status(cudaStreamWaitEvent(side->stream, side->fork, 0), "bert embedding bwd: fork");
        if (rc == 0) rc = launch_embedding_bwd_index(ids, tokens, vocab, index_type, sort_ws, sort_bytes, side->stream);
        if (rc == 0) rc = cuda_status(cudaEventRecord(side->join, side->stream), "bert embedding bwd: join");
        if (rc != 0) return rc;
    }
    int64_t n = 0;
    rc = nb2_layernorm_bwd(sum, dy, gamma, nullptr, mean, rstd, dsum, partials, &n, tokens, D, dtype, NB2_ACT_NONE, stream);
    if (rc != 0) return rc;
    // The position and type gradients read dsum and nothing else this call produces: on the side stream (behind the
    // sort, long finished) they run beside the partial reduce and the word-table sum instead of after them.
    if (side != nullptr) {
        rc = cuda_status(cudaEventRecord(side->fork2, st), "bert embedding bwd: second fork");
        if (rc == 0) rc = cuda_status(cudaStreamWaitEvent(side->stream, side->fork2, 0), "bert embedding bwd: second fork");
        if (rc == 0) rc = launch_bert_embed_table_grads(dsum, dpos, dtype0, type_scratch, B, S, D, dtype, side->stream);
        if (rc == 0) rc = cuda_status(cudaEventRecord(side->join2, side->stream), "bert embedding bwd: second join");
        if (rc != 0) return rc;
    }
    rc = nb2_colreduce_partials(partials, n, 2 * D, dgamma_dbeta, stream);
    if (rc != 0) return rc;
    if (ids != nullptr) {
        if (side != nullptr) rc = cuda_status(cudaStreamWaitEvent(st, side->join, 0), "bert embedding bwd: join");
        else rc = launch_embedding_bwd_index(ids, tokens, vocab, index_type, sort_ws, sort_bytes, st);
        if (rc != 0) return rc;
        rc = launch_embedding_bwd_sum(dsum, dword, tokens, vocab, D, dtype, sort_ws, st);
        if (rc != 0) return rc;
    }
    if (side != nullptr) return cuda_status(cudaStreamWaitEvent(st, side->join2, 0), "bert embedding bwd: second join");
    return launch_bert_embed_table_grads(dsum, dpos, dtype0, type_scratch, B, S, D, dtype, st);
}

int nb2_attention_softmax_fwd(const void* scores, const uint8_t* key_padding, const void* attn_mask,
                              int64_t mask_batch_stride, int64_t mask_head_stride, void* attn, int64_t B, int64_t H,
                              int64_t T, int64_t S, double scale, int causal, int dtype, void* stream) {
    NB2_REQUIRE(dtype_ok(dtype), NB2_ERR_DTYPE, "attention softmax: dtype=%d", dtype);
    NB2_REQUIRE(B >= 0 && H >= 0 && T >= 0 && S >= 0 && S < ((int64_t)1 << 31) && H < ((int64_t)1 << 30) && T < ((int64_t)1 << 30) &&
                    mask_batch_stride >= 0 && mask_head_stride >= 0,
                NB2_ERR_SHAPE, "attention softmax: B=%lld H=%lld T=%lld S=%lld mask strides %lld, %lld", (long long)B,
                (long long)H, (long long)T, (long long)S, (long long)mask_batch_stride, (long long)mask_head_stride);
    if (B * H * T * S == 0) return 0;
    NB2_REQUIRE(scores != nullptr && attn != nullptr, NB2_ERR_NULL, "attention softmax: NULL scores or output");
    int rc = require_device();
    if (rc != 0) return rc;
    return launch_attention_softmax_fwd(scores, key_padding, attn_mask, mask_batch_stride, mask_head_stride, attn, B, H, T, S,
                                        (float)scale, causal != 0, dtype, (cudaStream_t)stream);
}
int nb2_attention_softmax_bwd(const void* attn, const void* dattn, void* dscores, int64_t rows, int64_t S, double scale,
                              int dtype, void* stream) {
    NB2_REQUIRE(dtype_ok(dtype), NB2_ERR_DTYPE, "attention softmax bwd: dtype=%d", dtype);
    NB2_REQUIRE(rows >= 0 && S >= 0 && S < ((int64_t)1 << 31), NB2_ERR_SHAPE, "attention softmax bwd: rows=%lld S=%lld",
                (long long)rows, (long long)S);
    if (rows * S == 0) return 0;
    NB2_REQUIRE(attn != nullptr && dattn != nullptr && dscores != nullptr, NB2_ERR_NULL, "attention softmax bwd: NULL tensor");
    int rc = require_device();
    if (rc != 0) return rc;
    return launch_attention_softmax_bwd(attn, dattn, dscores, rows, S, (float)scale, dtype, (cudaStream_t)stream);
}

int nb2_attention_softmax_dropout_fwd(const void* scores, const uint8_t* key_padding, const void* attn_mask,
                                      int64_t mask_batch_stride, int64_t mask_head_stride, const void* noise, void* attn_pre,
                                      void* out, int64_t B, int64_t H, int64_t T, int64_t S, double scale, int causal, int dtype,
                                      void* stream) {
    NB2_REQUIRE(dtype_ok(dtype), NB2_ERR_DTYPE, "attention softmax + dropout: dtype=%d", dtype);
    NB2_REQUIRE(B >= 0 && H >= 0 && T >= 0 && S >= 0 && S < ((int64_t)1 << 31) && H < ((int64_t)1 << 30) && T < ((int64_t)1 << 30) &&
                    mask_batch_stride >= 0 && mask_head_stride >= 0,
                NB2_ERR_SHAPE, "attention softmax + dropout: B=%lld H=%lld T=%lld S=%lld mask strides %lld, %lld", (long long)B,
                (long long)H, (long long)T, (long long)S, (long long)mask_batch_stride, (long long)mask_head_stride);
    if (B * H * T * S == 0) return 0;
    NB2_REQUIRE(scores != nullptr && out != nullptr && noise != nullptr, NB2_ERR_NULL, "attention softmax + dropout: NULL scores, noise or output");
    int rc = require_device();
    if (rc != 0) return rc;
    return launch_attention_softmax_fwd(scores, key_padding, attn_mask, mask_batch_stride, mask_head_stride, out, B, H, T, S,
                                        (float)scale, causal != 0, dtype, (cudaStream_t)stream, noise, attn_pre);
}
int nb2_attention_softmax_dropout_bwd(const void* attn_pre, const void* noise, const void* dout, void* dscores, int64_t rows,
                                      int64_t S, double scale, int dtype, void* stream) {
    NB2_REQUIRE(dtype_ok(dtype), NB2_ERR_DTYPE, "attention softmax + dropout bwd: dtype=%d", dtype);
    NB2_REQUIRE(rows >= 0 && S >= 0 && S < ((int64_t)1 << 31), NB2_ERR_SHAPE, "attention softmax + dropout bwd: rows=%lld S=%lld",
                (long long)rows, (long long)S);
    if (rows * S == 0) return 0;
    NB2_REQUIRE(attn_pre != nullptr && noise != nullptr && dout != nullptr && dscores != nullptr, NB2_ERR_NULL,
                "attention softmax + dropout bwd: NULL tensor");
    int rc = require_device();
    if (rc != 0) return rc;
    return launch_attention_softmax_bwd(attn_pre, dout, dscores, rows, S, (float)scale, dtype, (cudaStream_t)stream, noise);
}

int nb2_linear_bias_act_fwd(const void* x, const void* weight, const void* bias, void* z_out, void* y, int64_t M, int64_t N,
                            int64_t K, int dtype, int act, void* workspace, size_t workspace_bytes, void* stream) {
    NB2_REQUIRE(dtype == NB2_BF16, NB2_ERR_DTYPE, "linear: dtype=%d (the tensor-core path takes bf16; fp32 layers stay with the host framework's GEMM)", dtype);
    NB2_REQUIRE(act_ok(act), NB2_ERR_DTYPE, "linear: unknown activation %d", act);
    NB2_REQUIRE(M >= 0 && N > 0 && K > 0 && M < ((int64_t)1 << 31) && N < ((int64_t)1 << 31) && K < ((int64_t)1 << 31), NB2_ERR_SHAPE,
                "linear: M=%lld N=%lld K=%lld", (long long)M, (long long)N, (long long)K);
    NB2_REQUIRE(N % 8 == 0 && K % 8 == 0, NB2_ERR_SHAPE, "linear: N=%lld and K=%lld must be multiples of 8 (16-byte rows for the bulk tensor copies)",
                (long long)N, (long long)K);
    if (M == 0) return 0;
    NB2_REQUIRE(x && weight && y, NB2_ERR_NULL, "linear: x, weight and y must be non-NULL");
    NB2_REQUIRE(aligned16(x) && aligned16(weight) && aligned16(y) && (bias == nullptr || aligned16(bias)) && (z_out == nullptr || aligned16(z_out)),
                NB2_ERR_ALIGN, "linear: pointers must be 16-byte aligned");
    int rc = require_device();
    if (rc != 0) return rc;
    return launch_linear(x, weight, bias, z_out, y, M, N, K, act, workspace, workspace_bytes, (cudaStream_t)stream);
}
int nb2_linear_available(void) { return linear_library_present() ? 1 : 0; }

int nb2_rope_table(float* cos_sin, const int32_t* positions, int64_t S, int64_t hd, double theta, void* stream) {
    NB2_REQUIRE(S >= 0 && hd >= 2 && hd % 2 == 0, NB2_ERR_SHAPE, "rope table: S=%lld head_dim=%lld (need an even head_dim >= 2)", (long long)S, (long long)hd);
    NB2_REQUIRE(theta > 0.0, NB2_ERR_SHAPE, "rope table: theta=%g must be positive", theta);
    if (S == 0) return 0;
    NB2_REQUIRE(cos_sin != nullptr, NB2_ERR_NULL, "rope table: NULL output");
    int rc = require_device();
    if (rc != 0) return rc;
    return launch_rope_table(cos_sin, positions, S, hd, theta, (cudaStream_t)stream);
}
int nb2_rope_apply(const void* x, const float* cos_sin, void* out, int64_t B, int64_t S, int64_t H, int64_t hd,
                   int dtype, int inverse, void* stream) {
    NB2_REQUIRE(dtype_ok(dtype), NB2_ERR_DTYPE, "rope: dtype=%d", dtype);
    NB2_REQUIRE(B >= 0 && S >= 0 && H >= 0 && hd >= 2 && hd % 2 == 0, NB2_ERR_SHAPE,
                "rope: B=%lld S=%lld H=%lld head_dim=%lld", (long long)B, (long long)S, (long long)H, (long long)hd);
    NB2_REQUIRE(S < ((int64_t)1 << 31) && H * hd < ((int64_t)1 << 31), NB2_ERR_SHAPE, "rope: S or H*head_dim exceeds 2^31-1");
    if (B == 0 || S == 0 || H == 0) return 0;
    NB2_REQUIRE(x && cos_sin && out, NB2_ERR_NULL, "rope: NULL pointer");
    int rc = require_device();
    if (rc != 0) return rc;
    return launch_rope_apply(x, cos_sin, out, B, S, H, hd, dtype, inverse != 0, (cudaStream_t)stream);
}

}  // extern "C"
