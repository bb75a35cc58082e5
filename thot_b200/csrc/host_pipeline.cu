// Host-buffer training step for the fused LayerNorm->activation path: rows are
// cut into chunks that flow host -> device -> host through three streams
// (copy-in, compute, copy-out), so PCIe transfers in both directions overlap
// the kernels.  The reference stages batches from pinned host memory the same
// way (src/core.hpp:4197-4227), one whole batch at a time.
#include <new>
#include "launchers.h"

namespace nb2 {
constexpr int HP_SETS = 3;   // chunk buffer sets in flight
}

struct nb2_host_ctx {
    int device = -1;
    int64_t max_rows = 0, D = 0, chunk_rows = 0, max_chunks = 0;
    int dtype = 0;
    size_t elt = 4;
    cudaStream_t s_in = nullptr, s_run = nullptr, s_out = nullptr;
    struct Set {
        void *x = nullptr, *dy = nullptr, *y = nullptr, *dx = nullptr;
        float *mean = nullptr, *rstd = nullptr, *partials = nullptr;
        cudaEvent_t in_done = nullptr, run_done = nullptr, out_done = nullptr;
    } set[nb2::HP_SETS];
    void *gamma = nullptr, *beta = nullptr;
    float *chunk_sums = nullptr, *total = nullptr;
};

using namespace nb2;

static void host_ctx_free(nb2_host_ctx* c) {
    if (c == nullptr) return;
    for (auto& s : c->set) {
        cudaFree(s.x); cudaFree(s.dy); cudaFree(s.y); cudaFree(s.dx);
        cudaFree(s.mean); cudaFree(s.rstd); cudaFree(s.partials);
        if (s.in_done) cudaEventDestroy(s.in_done);
        if (s.run_done) cudaEventDestroy(s.run_done);
        if (s.out_done) cudaEventDestroy(s.out_done);
    }
    cudaFree(c->gamma); cudaFree(c->beta); cudaFree(c->chunk_sums); cudaFree(c->total);
    if (c->s_in) cudaStreamDestroy(c->s_in);
    if (c->s_run) cudaStreamDestroy(c->s_run);
    if (c->s_out) cudaStreamDestroy(c->s_out);
    delete c;
}

#define HP_CUDA(call)                                                 \
    do {                                                              \
        int rc_ = cuda_status((call), #call);                         \
        if (rc_ != 0) { host_ctx_free(c); return rc_; }               \
    } while (0)

extern "C" int nb2_host_ctx_create(nb2_host_ctx** ctx, int64_t max_rows, int64_t D, int dtype, int64_t chunk_rows) {
    NB2_REQUIRE(ctx != nullptr, NB2_ERR_NULL, "host ctx: NULL out pointer");
    *ctx = nullptr;
    NB2_REQUIRE(dtype == NB2_F32 || dtype == NB2_BF16, NB2_ERR_DTYPE, "host ctx: dtype=%d", dtype);
    NB2_REQUIRE(max_rows > 0 && D > 0, NB2_ERR_SHAPE, "host ctx: max_rows=%lld D=%lld", (long long)max_rows, (long long)D);
    if (chunk_rows <= 0) {
        // default: about 16 MiB of activations per tensor per chunk
        const int64_t bytes_row = D * (dtype == NB2_F32 ? 4 : 2);
        chunk_rows = (16ll << 20) / bytes_row;
        if (chunk_rows < 64) chunk_rows = 64;
    }
    if (chunk_rows > max_rows) chunk_rows = max_rows;
    nb2_host_ctx* c = new (std::nothrow) nb2_host_ctx();
    NB2_REQUIRE(c != nullptr, NB2_ERR_NULL, "host ctx: out of host memory");
    HP_CUDA(cudaGetDevice(&c->device));
    c->max_rows = max_rows; c->D = D; c->dtype = dtype; c->chunk_rows = chunk_rows;
    c->elt = dtype == NB2_F32 ? 4 : 2;
    c->max_chunks = (max_rows + chunk_rows - 1) / chunk_rows;
    HP_CUDA(cudaStreamCreateWithFlags(&c->s_in, cudaStreamNonBlocking));
    HP_CUDA(cudaStreamCreateWithFlags(&c->s_run, cudaStreamNonBlocking));
    HP_CUDA(cudaStreamCreateWithFlags(&c->s_out, cudaStreamNonBlocking));
    const size_t act_bytes = (size_t)chunk_rows * D * c->elt;
    const size_t ws = nb2_workspace_bytes(NB2_WS_NORM_BWD, chunk_rows, D, dtype);
    for (auto& s : c->set) {
        HP_CUDA(cudaMalloc(&s.x, act_bytes));
        HP_CUDA(cudaMalloc(&s.dy, act_bytes));
        HP_CUDA(cudaMalloc(&s.y, act_bytes));
        HP_CUDA(cudaMalloc(&s.dx, act_bytes));
        HP_CUDA(cudaMalloc((void**)&s.mean, (size_t)chunk_rows * 4));
        HP_CUDA(cudaMalloc((void**)&s.rstd, (size_t)chunk_rows * 4));
        HP_CUDA(cudaMalloc((void**)&s.partials, ws));
        HP_CUDA(cudaEventCreateWithFlags(&s.in_done, cudaEventDisableTiming));
        HP_CUDA(cudaEventCreateWithFlags(&s.run_done, cudaEventDisableTiming));
        HP_CUDA(cudaEventCreateWithFlags(&s.out_done, cudaEventDisableTiming));
    }
    HP_CUDA(cudaMalloc(&c->gamma, (size_t)D * c->elt));
    HP_CUDA(cudaMalloc(&c->beta, (size_t)D * c->elt));
    HP_CUDA(cudaMalloc((void**)&c->chunk_sums, (size_t)c->max_chunks * 2 * D * 4));
    HP_CUDA(cudaMalloc((void**)&c->total, (size_t)2 * D * 4));
    *ctx = c;
    return 0;
}

extern "C" int nb2_host_ctx_destroy(nb2_host_ctx* ctx) {
    if (ctx != nullptr) {
        cudaSetDevice(ctx->device);
        cudaDeviceSynchronize();
        host_ctx_free(ctx);
    }
    return 0;
}

#define ST_CUDA(call)                                                 \
    do {                                                              \
        int rc_ = cuda_status((call), #call);                         \
        if (rc_ != 0) { cudaDeviceSynchronize(); return rc_; }        \
    } while (0)
#define ST_RC(call)                                                   \
    do {                                                              \
        int rc_ = (call);                                             \
        if (rc_ != 0) { cudaDeviceSynchronize(); return rc_; }        \
    } while (0)

// One host-buffer step for either norm.  LayerNorm: gamma, beta in, [2, D] gradients out; RMSNorm:
// weight in (beta_host unused), [D] gradient out.
static int norm_act_step_host(nb2_host_ctx* c, bool rms, const void* x_host, const void* dy_host,
                              const void* gamma_host, const void* beta_host, void* y_host, void* dx_host,
                              float* grads_host, int64_t rows, int64_t D, double eps, int dtype, int act) {
    NB2_REQUIRE(c != nullptr, NB2_ERR_NULL, "host step: NULL context");
    NB2_REQUIRE(D == c->D && dtype == c->dtype && rows >= 0 && rows <= c->max_rows, NB2_ERR_SHAPE,
                "host step: rows=%lld D=%lld dtype=%d do not fit the context (max_rows=%lld D=%lld dtype=%d)",
                (long long)rows, (long long)D, dtype, (long long)c->max_rows, (long long)c->D, c->dtype);
    NB2_REQUIRE(x_host && dy_host && gamma_host && (rms || beta_host) && y_host && dx_host && grads_host,
                NB2_ERR_NULL, "host step: NULL pointer");
    ST_CUDA(cudaSetDevice(c->device));
    const size_t row_bytes = (size_t)D * c->elt;
    const int64_t ncols = (rms ? 1 : 2) * D;
    ST_CUDA(cudaMemcpyAsync(c->gamma, gamma_host, row_bytes, cudaMemcpyHostToDevice, c->s_in));
    if (!rms) ST_CUDA(cudaMemcpyAsync(c->beta, beta_host, row_bytes, cudaMemcpyHostToDevice, c->s_in));
    const int64_t nchunks = (rows + c->chunk_rows - 1) / c->chunk_rows;
    for (int64_t i = 0; i < nchunks; ++i) {
        auto& s = c->set[i % HP_SETS];
        const int64_t r0 = i * c->chunk_rows;
        const int64_t n = (rows - r0 < c->chunk_rows) ? rows - r0 : c->chunk_rows;
        const size_t off = (size_t)r0 * row_bytes, bytes = (size_t)n * row_bytes;
        // copy-in may reuse this set once its previous results left the device
        if (i >= HP_SETS) ST_CUDA(cudaStreamWaitEvent(c->s_in, s.out_done, 0));
        ST_CUDA(cudaMemcpyAsync(s.x, (const char*)x_host + off, bytes, cudaMemcpyHostToDevice, c->s_in));
        ST_CUDA(cudaMemcpyAsync(s.dy, (const char*)dy_host + off, bytes, cudaMemcpyHostToDevice, c->s_in));
        ST_CUDA(cudaEventRecord(s.in_done, c->s_in));
        ST_CUDA(cudaStreamWaitEvent(c->s_run, s.in_done, 0));
        int64_t parts = 0;
        if (rms) {
            ST_RC(nb2_rmsnorm_fwd(s.x, c->gamma, s.y, s.rstd, n, D, eps, dtype, act, c->s_run));
            ST_RC(nb2_rmsnorm_bwd(s.x, s.dy, c->gamma, s.rstd, s.dx, s.partials, &parts, n, D, dtype, act, c->s_run));
        } else {
            ST_RC(nb2_layernorm_fwd(s.x, c->gamma, c->beta, s.y, s.mean, s.rstd, n, D, eps, dtype, act, c->s_run));
            ST_RC(nb2_layernorm_bwd(s.x, s.dy, c->gamma, c->beta, s.mean, s.rstd, s.dx, s.partials, &parts, n, D, dtype, act, c->s_run));
        }
        ST_RC(nb2_colreduce_partials(s.partials, parts, ncols, c->chunk_sums + (size_t)i * ncols, c->s_run));
        ST_CUDA(cudaEventRecord(s.run_done, c->s_run));
        ST_CUDA(cudaStreamWaitEvent(c->s_out, s.run_done, 0));
        ST_CUDA(cudaMemcpyAsync((char*)y_host + off, s.y, bytes, cudaMemcpyDeviceToHost, c->s_out));
        ST_CUDA(cudaMemcpyAsync((char*)dx_host + off, s.dx, bytes, cudaMemcpyDeviceToHost, c->s_out));
        ST_CUDA(cudaEventRecord(s.out_done, c->s_out));
    }
    if (nchunks > 0) {
        ST_RC(nb2_colreduce_partials(c->chunk_sums, nchunks, ncols, c->total, c->s_run));
    } else {
        ST_CUDA(cudaMemsetAsync(c->total, 0, (size_t)ncols * 4, c->s_run));
    }
    ST_CUDA(cudaMemcpyAsync(grads_host, c->total, (size_t)ncols * 4, cudaMemcpyDeviceToHost, c->s_run));
    ST_CUDA(cudaStreamSynchronize(c->s_in));
    ST_CUDA(cudaStreamSynchronize(c->s_run));
    ST_CUDA(cudaStreamSynchronize(c->s_out));
    return 0;
}

extern "C" int nb2_layernorm_act_step_host(nb2_host_ctx* c, const void* x_host, const void* dy_host,
                                           const void* gamma_host, const void* beta_host, void* y_host,
                                           void* dx_host, float* dgamma_dbeta_host, int64_t rows, int64_t D,
                                           double eps, int dtype, int act) {
    return norm_act_step_host(c, false, x_host, dy_host, gamma_host, beta_host, y_host, dx_host, dgamma_dbeta_host, rows, D,
                              eps, dtype, act);
}

extern "C" int nb2_rmsnorm_act_step_host(nb2_host_ctx* c, const void* x_host, const void* dy_host,
                                         const void* weight_host, void* y_host, void* dx_host, float* dweight_host,
                                         int64_t rows, int64_t D, double eps, int dtype, int act) {
    return norm_act_step_host(c, true, x_host, dy_host, weight_host, nullptr, y_host, dx_host, dweight_host, rows, D, eps,
                              dtype, act);
}
