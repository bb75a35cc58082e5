// LayerNorm(+activation) backward for callers that are not allowed to allocate.
//
// The ordinary backward (nb2_layernorm_bwd + nb2_colreduce_partials) needs a
// caller-provided scratch buffer for the per-CTA dgamma/dbeta partials.  Some
// hosts cannot supply one at the point where they call us: code running inside
// a region where device allocation is forbidden (a CUDA-graph capture, a
// real-time inference loop with a frozen memory plan, a plugin that is handed
// only its input and output buffers by the framework that owns all device
// memory).  For them this file keeps that scratch in a fixed array inside the
// library image.  Nothing here calls cudaMalloc, cudaFree or any allocating
// library routine.
#include <atomic>
#include "launchers.h"

namespace nb2 {

// 296 partials x [2, 2048] fp32 = 4.6 MiB, resident on every GPU that loads the
// library until the process exits.  296 = two persistent CTAs on each of 148 SMs,
// the largest grid any backward kernel here uses, so every shape with D <= 2048
// fits; wider rows fit only when there are few of them.
constexpr size_t kStaticPartialFloats = (size_t)296 * 2 * 2048;
static __device__ __align__(256) float g_static_partials[kStaticPartialFloats];

// In host code `g_static_partials` names a host-side shadow of the symbol, not
// device memory: a kernel handed that name would read the wrong memory.  The
// device address comes from cudaGetSymbolAddress, asked once per device with
// that device current.
static float* static_partials_ptr(int* rc_out) {
    // one slot per device for the whole process (not per host thread): once any thread has made the
    // first call on a device, every later call on it, from any thread, only reads the cached address
    static std::atomic<float*> ptrs[kMaxDevices];
    std::atomic<float*>& slot = ptrs[current_device_slot()];
    *rc_out = 0;
    float* p = slot.load(std::memory_order_acquire);
    if (p == nullptr) {
        void* addr = nullptr;
        *rc_out = cuda_status(cudaGetSymbolAddress(&addr, g_static_partials), "cudaGetSymbolAddress(static partials)");
        if (*rc_out == 0) {
            p = static_cast<float*>(addr);
            slot.store(p, std::memory_order_release);      // two racing first calls store the same address
        }
    }
    return p;
}

}  // namespace nb2

using namespace nb2;

extern "C" int nb2_layernorm_bwd_static(const void* x, const void* dy, const void* gamma, const void* beta,
                                        const float* mean, const float* rstd, void* dx, float* dgamma_dbeta,
                                        int64_t rows, int64_t D, int dtype, int act, void* stream) {
    NB2_REQUIRE(dgamma_dbeta != nullptr, NB2_ERR_NULL, "static backward: dgamma_dbeta output is NULL");
    NB2_REQUIRE(gamma != nullptr, NB2_ERR_NULL, "static backward: gamma is NULL (without affine parameters use nb2_layernorm_bwd with partials = NULL)");
    NB2_REQUIRE(rows >= 0 && D > 0, NB2_ERR_SHAPE, "static backward: rows=%lld D=%lld", (long long)rows, (long long)D);
    if (rows == 0)
        return cuda_status(cudaMemsetAsync(dgamma_dbeta, 0, (size_t)2 * D * sizeof(float), (cudaStream_t)stream),
                           "static backward: clearing the gradients of an empty batch");
    // the same bound the ordinary path asks its caller to allocate
    const size_t need = (nb2_workspace_bytes(NB2_WS_NORM_BWD, rows, D, dtype) - 256) / sizeof(float);
    NB2_REQUIRE(need <= kStaticPartialFloats, NB2_ERR_WORKSPACE,
                "static backward: rows=%lld D=%lld needs %zu floats of scratch, the built-in array holds %zu "
                "(use nb2_layernorm_bwd with your own workspace for this shape)",
                (long long)rows, (long long)D, need, kStaticPartialFloats);
    int rc = 0;
    float* scratch = static_partials_ptr(&rc);
    if (rc != 0) return rc;
    int64_t n_partials = 0;
    // every CTA overwrites its whole [2, D] block, so nothing in the array has to start at zero
    rc = nb2_layernorm_bwd(x, dy, gamma, beta, mean, rstd, dx, scratch, &n_partials, rows, D, dtype, act, stream);
    if (rc != 0) return rc;
    return nb2_colreduce_partials(scratch, n_partials, 2 * D, dgamma_dbeta, stream);
}
