// Host-side selection of a norm kernel configuration.  Included by the four
// norm_*.cu translation units, each of which instantiates one element type and
// one direction so they compile in parallel.
#pragma once
#include "norm_kernels.cuh"

namespace nb2 {

struct NormArgs {
    const void* x; const void* dy; const void* gamma; const void* beta;
    const float* mean; const float* rstd;       // backward inputs
    float* mean_out; float* rstd_out;           // forward outputs
    void* y; void* dx; float* partials;
    int64_t rows; int64_t D; float eps; int act; bool rms;
    cudaStream_t stream;
};

// Threads per row for `nvec` 16-byte vectors at VPT vectors per thread; 0 when
// the row does not fit the register-row configurations.
static inline int pick_tpr(int64_t nvec, int vpt) {
    for (int tpr = 32; tpr <= 512; tpr *= 2)
        if (nvec <= (int64_t)tpr * vpt) return tpr;
    return 0;
}

// vectors per thread: forward keeps 4 for both types; backward keeps 16
// elements per thread (its dgamma/dbeta accumulators live in registers).
template <typename T> constexpr int fwd_vpt() { return 4; }
template <typename T> constexpr int bwd_vpt() { return 16 / VecTraits<T>::EPV; }

static inline int ctas_per_sm(int tpr) { return tpr > 256 ? 1 : 2; }

// Grid of the persistent backward kernel == number of partials it writes.
// Shared with nb2_workspace_bytes so the caller's buffer always fits.
static inline int64_t norm_bwd_grid(int64_t rows, int tpr, int sms) {
    const int threads = tpr > 256 ? tpr : 256;
    const int rpc = threads / tpr;
    int64_t need = (rows + rpc - 1) / rpc;
    int64_t cap = (int64_t)sms * ctas_per_sm(tpr);
    if (need < 1) need = 1;
    return need < cap ? need : cap;
}
// generic path: row blocks of the column-sum kernel
static inline int64_t norm_bwd_generic_parts(int64_t rows) {
    int64_t p = (rows + 255) / 256;
    if (p < 1) p = 1;
    return p > 256 ? 256 : p;
}

template <typename T> int launch_norm_fwd(const NormArgs& a);
template <typename T> int launch_norm_bwd(const NormArgs& a, int64_t* n_partials);

template <typename T>
static inline bool norm_fast_path_ok(const NormArgs& a, int vpt) {
    constexpr int EPV = VecTraits<T>::EPV;
    if (a.D % EPV != 0) return false;
    if (pick_tpr(a.D / EPV, vpt) == 0) return false;
    if (!aligned16(a.x) || (a.y && !aligned16(a.y)) || (a.dy && !aligned16(a.dy)) ||
        (a.dx && !aligned16(a.dx)) || (a.gamma && !aligned16(a.gamma)) ||
        (a.beta && !aligned16(a.beta)) || (a.partials && !aligned16(a.partials)))
        return false;
    return true;
}

}  // namespace nb2
