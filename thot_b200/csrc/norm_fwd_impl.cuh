// Forward launcher: picks (threads per row, activation, norm kind) and launches
// the persistent register-row kernel, or the any-D kernel when the row is
// not 16-byte vectorisable.
#pragma once
#include "norm_dispatch.cuh"

namespace nb2 {

template <typename T, int TPR, int ACT, bool RMS>
static int launch_fwd_cfg(const NormArgs& a) {
    constexpr int VPT = fwd_vpt<T>();
    constexpr int THREADS = TPR > 256 ? TPR : 256;
    constexpr int MINB = TPR > 256 ? 1 : 2;
    constexpr int RPC = THREADS / TPR;
    int64_t need = (a.rows + RPC - 1) / RPC;
    int64_t cap = (int64_t)sm_count() * MINB;
    const int grid = (int)(need < cap ? need : cap);
    norm_fwd_kernel<T, TPR, VPT, ACT, RMS, MINB><<<grid, THREADS, 0, a.stream>>>(
        (const T*)a.x, (const T*)a.gamma, (const T*)a.beta, (T*)a.y, a.mean_out, a.rstd_out,
        a.rows, (int)a.D, a.eps);
    return cuda_status(cudaGetLastError(), "norm_fwd_kernel launch");
}

template <typename T, int ACT, bool RMS>
static int launch_fwd_act(const NormArgs& a) {
    constexpr int EPV = VecTraits<T>::EPV;
    if (norm_fast_path_ok<T>(a, fwd_vpt<T>())) {
        switch (pick_tpr(a.D / EPV, fwd_vpt<T>())) {
            case 32:  return launch_fwd_cfg<T, 32, ACT, RMS>(a);
            case 64:  return launch_fwd_cfg<T, 64, ACT, RMS>(a);
            case 128: return launch_fwd_cfg<T, 128, ACT, RMS>(a);
            case 256: return launch_fwd_cfg<T, 256, ACT, RMS>(a);
            case 512: return launch_fwd_cfg<T, 512, ACT, RMS>(a);
            default: break;
        }
    }
    int64_t need = (a.rows + 7) / 8;
    int64_t cap = (int64_t)sm_count() * 8;
    const int grid = (int)(need < cap ? need : cap);
    norm_fwd_generic<T, ACT, RMS><<<grid, 256, 0, a.stream>>>(
        (const T*)a.x, (const T*)a.gamma, (const T*)a.beta, (T*)a.y, a.mean_out, a.rstd_out,
        a.rows, a.D, a.eps);
    return cuda_status(cudaGetLastError(), "norm_fwd_generic launch");
}

template <typename T, bool RMS>
static int launch_fwd_rms(const NormArgs& a) {
    switch (a.act) {
        case NB2_ACT_NONE: return launch_fwd_act<T, NB2_ACT_NONE, RMS>(a);
        case NB2_ACT_GELU: return launch_fwd_act<T, NB2_ACT_GELU, RMS>(a);
        case NB2_ACT_SILU: return launch_fwd_act<T, NB2_ACT_SILU, RMS>(a);
        default: set_error("unknown activation %d", a.act); return NB2_ERR_DTYPE;
    }
}

template <typename T>
int launch_norm_fwd(const NormArgs& a) {
    return a.rms ? launch_fwd_rms<T, true>(a) : launch_fwd_rms<T, false>(a);
}

}  // namespace nb2
