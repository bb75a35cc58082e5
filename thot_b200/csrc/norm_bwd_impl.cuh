// Backward launcher: dX + per-CTA partials in one persistent kernel; the
// any-D path uses a dX kernel and a column-sum kernel instead.
#pragma once
#include "norm_dispatch.cuh"

namespace nb2 {

template <typename T, int TPR, int ACT, bool RMS>
static int launch_bwd_cfg(const NormArgs& a, int64_t* n_partials) {
    constexpr int VPT = bwd_vpt<T>();
    constexpr int THREADS = TPR > 256 ? TPR : 256;
    constexpr int MINB = TPR > 256 ? 1 : 2;
    const int grid = (int)norm_bwd_grid(a.rows, TPR, sm_count());
    norm_bwd_kernel<T, TPR, VPT, ACT, RMS, MINB><<<grid, THREADS, 0, a.stream>>>(
        (const T*)a.x, (const T*)a.dy, (const T*)a.gamma, (const T*)a.beta, a.mean, a.rstd,
        (T*)a.dx, a.partials, a.rows, (int)a.D);
    if (n_partials) *n_partials = a.partials ? grid : 0;
    return cuda_status(cudaGetLastError(), "norm_bwd_kernel launch");
}

template <typename T, int ACT, bool RMS>
static int launch_bwd_act(const NormArgs& a, int64_t* n_partials) {
    constexpr int EPV = VecTraits<T>::EPV;
    if (norm_fast_path_ok<T>(a, bwd_vpt<T>())) {
        switch (pick_tpr(a.D / EPV, bwd_vpt<T>())) {
            case 32:  return launch_bwd_cfg<T, 32, ACT, RMS>(a, n_partials);
            case 64:  return launch_bwd_cfg<T, 64, ACT, RMS>(a, n_partials);
            case 128: return launch_bwd_cfg<T, 128, ACT, RMS>(a, n_partials);
            case 256: return launch_bwd_cfg<T, 256, ACT, RMS>(a, n_partials);
            case 512: return launch_bwd_cfg<T, 512, ACT, RMS>(a, n_partials);
            default: break;
        }
    }
    int64_t need = (a.rows + 7) / 8;
    int64_t cap = (int64_t)sm_count() * 8;
    const int grid = (int)(need < cap ? need : cap);
    norm_bwd_generic_dx<T, ACT, RMS><<<grid, 256, 0, a.stream>>>(
        (const T*)a.x, (const T*)a.dy, (const T*)a.gamma, (const T*)a.beta, a.mean, a.rstd,
        (T*)a.dx, a.rows, a.D);
    int rc = cuda_status(cudaGetLastError(), "norm_bwd_generic_dx launch");
    if (rc != 0) return rc;
    if (n_partials) *n_partials = 0;
    if (a.partials != nullptr) {
        const int64_t parts = norm_bwd_generic_parts(a.rows);
        const int64_t rows_per = (a.rows + parts - 1) / parts;
        dim3 g((unsigned)((a.D + 255) / 256), (unsigned)parts);
        norm_bwd_generic_cols<T, ACT, RMS><<<g, 256, 0, a.stream>>>(
            (const T*)a.x, (const T*)a.dy, (const T*)a.gamma, (const T*)a.beta, a.mean, a.rstd,
            a.partials, a.rows, a.D, rows_per);
        rc = cuda_status(cudaGetLastError(), "norm_bwd_generic_cols launch");
        if (n_partials) *n_partials = parts;
    }
    return rc;
}

template <typename T, bool RMS>
static int launch_bwd_rms(const NormArgs& a, int64_t* n_partials) {
    switch (a.act) {
        case NB2_ACT_NONE: return launch_bwd_act<T, NB2_ACT_NONE, RMS>(a, n_partials);
        case NB2_ACT_GELU: return launch_bwd_act<T, NB2_ACT_GELU, RMS>(a, n_partials);
        case NB2_ACT_SILU: return launch_bwd_act<T, NB2_ACT_SILU, RMS>(a, n_partials);
        default: set_error("unknown activation %d", a.act); return NB2_ERR_DTYPE;
    }
}

template <typename T>
int launch_norm_bwd(const NormArgs& a, int64_t* n_partials) {
    return a.rms ? launch_bwd_rms<T, true>(a, n_partials) : launch_bwd_rms<T, false>(a, n_partials);
}

}  // namespace nb2
