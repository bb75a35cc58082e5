// Forward launcher: bulk-async ring kernel where the shape fits it exactly,
// else the register-row kernel, else the any-width kernel.
#pragma once
#include "norm_dispatch.cuh"

namespace nb2 {

template <typename T, int TPR, int VPT, int ACT, bool RMS, bool RES, int NT>
static int launch_fwd_tma_nt(const NormArgs& a) {
    auto kern = norm_fwd_tma_kernel<T, TPR, VPT, ACT, RMS, RES, NT>;
    const TmaTiling t = tma_tiling(a.D, (int)sizeof(T), TPR, RES ? 2 : 1, NT);
    NB2_REQUIRE(t.smem <= kTmaMaxSmem, NB2_ERR_SHAPE, "norm ring kernel: %zu bytes of shared memory exceed the SM", t.smem);
    static thread_local size_t configured_all[kMaxDevices] = {};
    size_t& configured = configured_all[current_device_slot()];
    if (t.smem > configured) {
        int rc = cuda_status(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)t.smem),
                             "norm_fwd_tma_kernel shared memory");
        if (rc != 0) return rc;
        configured = t.smem;
    }
    const int grid = (int)tma_grid(a.rows, TPR, launch_sms(), NT);
    const cudaError_t e = launch_pdl(kern, dim3(grid), dim3(NT), t.smem, a.stream, (const T*)a.x, (const T*)a.res,
                                     (const T*)a.gamma, (const T*)a.beta, (T*)a.sum_out, (T*)a.y, a.mean_out, a.rstd_out,
                                     a.rows, (int)a.D, a.eps, t.stages, device_status_ptr(), a.gather);
    if (e != cudaSuccess) return cuda_status(e, "norm_fwd_tma_kernel launch");
    return 0;
}

template <typename T, int TPR, int VPT, int ACT, bool RMS, bool RES>
static int launch_fwd_tma_res(const NormArgs& a) {
    if constexpr (!RES && (TPR == 128 || TPR == 256 ||
                           ((TPR == 32 || TPR == 64) && sizeof(T) == 2 && ACT == NB2_ACT_GELU && !RMS))) {
        if (fwd_threads(TPR, a.D * (int64_t)sizeof(T), (int)sizeof(T), RMS, ACT == NB2_ACT_GELU) == 768) return launch_fwd_tma_nt<T, TPR, VPT, ACT, RMS, RES, 768>(a);
    }
    return launch_fwd_tma_nt<T, TPR, VPT, ACT, RMS, RES, 512>(a);
}

template <typename T, int TPR, int VPT, int ACT, bool RMS>
static int launch_fwd_tma(const NormArgs& a) {
    if (a.res != nullptr) {
        // the residual form is built without a fused activation (the reference norms a residual sum
        // right before attention or the feed forward, never before an activation)
        if constexpr (ACT == NB2_ACT_NONE) return launch_fwd_tma_res<T, TPR, VPT, ACT, RMS, true>(a);
        set_error("residual + norm is not fused with an activation");
        return NB2_ERR_DTYPE;
    }
    return launch_fwd_tma_res<T, TPR, VPT, ACT, RMS, false>(a);
}

// a ring kernel with a given CTA size (the 7 * 2^k shapes: 448 threads)
template <typename T, int TPR, int VPT, int ACT, bool RMS, int NT>
static int launch_fwd_tma_fixed(const NormArgs& a) {
    if (a.res != nullptr) {
        if constexpr (ACT == NB2_ACT_NONE) return launch_fwd_tma_nt<T, TPR, VPT, ACT, RMS, true, NT>(a);
        set_error("residual + norm is not fused with an activation");
        return NB2_ERR_DTYPE;
    }
    return launch_fwd_tma_nt<T, TPR, VPT, ACT, RMS, false, NT>(a);
}

template <typename T, int ACT, bool RMS>
static int launch_fwd_tma_shape(const NormArgs& a, TmaShape s) {
    constexpr int EPV = VecTraits<T>::EPV;
    if (s.tpr == 224) return s.vpt == 4 ? launch_fwd_tma_fixed<T, 224, 4, ACT, RMS, 448>(a) : launch_fwd_tma_fixed<T, 224, 2, ACT, RMS, 448>(a);
    if (s.tpr == 448) return s.vpt == 4 ? launch_fwd_tma_fixed<T, 448, 4, ACT, RMS, 448>(a) : launch_fwd_tma_fixed<T, 448, 2, ACT, RMS, 448>(a);
    if (s.vpt == 3) {
        switch (s.tpr) {
            case 32:  return launch_fwd_tma<T, 32, 3, ACT, RMS>(a);
            case 64:  return launch_fwd_tma<T, 64, 3, ACT, RMS>(a);
            case 128: return launch_fwd_tma<T, 128, 3, ACT, RMS>(a);
            case 256: return launch_fwd_tma<T, 256, 3, ACT, RMS>(a);
            case 512: if constexpr (EPV == 4) return launch_fwd_tma<T, 512, 3, ACT, RMS>(a);
            default: break;
        }
        set_error("norm fwd: no three-vector ring kernel for threads-per-row %d", s.tpr);
        return NB2_ERR_SHAPE;
    }
    if (s.vpt == 5) {
        switch (s.tpr) {
            case 32:  return launch_fwd_tma<T, 32, 5, ACT, RMS>(a);
            case 64:  return launch_fwd_tma<T, 64, 5, ACT, RMS>(a);
            case 128: return launch_fwd_tma<T, 128, 5, ACT, RMS>(a);
            case 256: return launch_fwd_tma<T, 256, 5, ACT, RMS>(a);
            default: break;
        }
        set_error("norm fwd: no five-vector ring kernel for threads-per-row %d", s.tpr);
        return NB2_ERR_SHAPE;
    }
    switch (s.tpr) {
        case 32:  return launch_fwd_tma<T, 32, 4, ACT, RMS>(a);
        case 64:  return launch_fwd_tma<T, 64, 4, ACT, RMS>(a);
        case 128: return launch_fwd_tma<T, 128, 4, ACT, RMS>(a);
        case 256: return launch_fwd_tma<T, 256, 4, ACT, RMS>(a);
        case 512: return launch_fwd_tma<T, 512, 4, ACT, RMS>(a);
        default: break;
    }
    set_error("norm fwd: no ring kernel for threads-per-row %d", s.tpr);
    return NB2_ERR_SHAPE;
}

template <typename T, int TPR, int ACT, bool RMS>
static int launch_fwd_cfg(const NormArgs& a) {
    constexpr int VPT = fwd_vpt<T>();
    constexpr int THREADS = TPR > 256 ? TPR : 256;
    constexpr int MINB = TPR > 256 ? 1 : 2;
    constexpr int RPC = THREADS / TPR;
    int64_t need = (a.rows + RPC - 1) / RPC;
    int64_t cap = (int64_t)launch_sms() * MINB;
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
        const TmaShape s = tma_fwd_shape(a.D, EPV);
        const bool affine = a.gamma != nullptr && (RMS || a.beta != nullptr);
        if (a.res != nullptr) {
            if (s.tpr != 0 && affine && tma_fits(a.D, (int)sizeof(T), s.tpr, 2)) return launch_fwd_tma_shape<T, ACT, RMS>(a, s);
            return kNotFused;
        }
        if (s.tpr != 0 && affine && tma_preferred(RMS, a.D, (int)sizeof(T), false, ACT) && tma_fits(a.D, (int)sizeof(T), s.tpr, 1, fwd_threads(s.tpr, a.D * (int64_t)sizeof(T), (int)sizeof(T), RMS, ACT == NB2_ACT_GELU)))
            return launch_fwd_tma_shape<T, ACT, RMS>(a, s);
        switch (pick_tpr(a.D / EPV, fwd_vpt<T>())) {
            case 32:  return launch_fwd_cfg<T, 32, ACT, RMS>(a);
            case 64:  return launch_fwd_cfg<T, 64, ACT, RMS>(a);
            case 128: return launch_fwd_cfg<T, 128, ACT, RMS>(a);
            case 256: return launch_fwd_cfg<T, 256, ACT, RMS>(a);
            case 512: return launch_fwd_cfg<T, 512, ACT, RMS>(a);
            default: break;
        }
    }
    if (a.res != nullptr) return kNotFused;
    int64_t need = (a.rows + 7) / 8;
    int64_t cap = (int64_t)sm_count() * 8;
    const int grid = (int)(need < cap ? need : cap);
    norm_fwd_generic<T, ACT, RMS><<<grid, 256, 0, a.stream>>>(
        (const T*)a.x, (const T*)a.gamma, (const T*)a.beta, (T*)a.y, a.mean_out, a.rstd_out,
        a.rows, a.D, a.eps);
    return cuda_status(cudaGetLastError(), "norm_fwd_generic launch");
}

template <typename T, bool RMS>
int launch_norm_fwd(const NormArgs& a) {
    switch (a.act) {
        case NB2_ACT_NONE: return launch_fwd_act<T, NB2_ACT_NONE, RMS>(a);
        case NB2_ACT_GELU: return launch_fwd_act<T, NB2_ACT_GELU, RMS>(a);
        case NB2_ACT_SILU: return launch_fwd_act<T, NB2_ACT_SILU, RMS>(a);
        default: set_error("unknown activation %d", a.act); return NB2_ERR_DTYPE;
    }
}

}  // namespace nb2
