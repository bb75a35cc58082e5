// Backward launcher: dX + per-CTA partials in one persistent kernel (bulk-async
// ring where the shape fits it exactly, else register-row); the any-width path
// uses a dX kernel and a column-sum kernel instead.
#pragma once
#include "norm_dispatch.cuh"
#include "norm_bwd_wide.cuh"

namespace nb2 {

template <typename T, int TPR, int VPT, int ACT, bool RMS, bool RES, int NT>
static int launch_bwd_tma_res(const NormArgs& a, int64_t* n_partials) {
    auto kern = norm_bwd_tma_kernel<T, TPR, VPT, ACT, RMS, RES, NT>;
    const TmaTiling t = tma_tiling(a.D, (int)sizeof(T), TPR, RES ? 3 : 2, NT);
    NB2_REQUIRE(t.smem <= kTmaMaxSmem, NB2_ERR_SHAPE, "norm ring kernel: %zu bytes of shared memory exceed the SM", t.smem);
    static thread_local size_t configured_all[kMaxDevices] = {};
    size_t& configured = configured_all[current_device_slot()];
    if (t.smem > configured) {
        int rc = cuda_status(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)t.smem),
                             "norm_bwd_tma_kernel shared memory");
        if (rc != 0) return rc;
        configured = t.smem;
    }
    const int grid = (int)tma_grid(a.rows, TPR, launch_sms(), NT);
    const cudaError_t e = launch_pdl(kern, dim3(grid), dim3(NT), t.smem, a.stream, (const T*)a.x, (const T*)a.dy,
                                     (const T*)a.dres, (const T*)a.gamma, (const T*)a.beta, a.mean, a.rstd, (T*)a.dx,
                                     a.partials, a.rows, (int)a.D, t.stages, device_status_ptr());
    if (e != cudaSuccess) return cuda_status(e, "norm_bwd_tma_kernel launch");
    if (n_partials) *n_partials = a.partials ? grid : 0;
    return 0;
}

// 32 columns per thread (bf16, no residual): see norm_bwd_wide.cuh
template <int TPR, int ACT, bool RMS>
static int launch_bwd_wide_bf16(const NormArgs& a, int64_t* n_partials) {
    using T = __nv_bfloat16;
    auto kern = norm_bwd_wide_bf16_kernel<TPR, ACT, RMS>;
    TmaTiling t = tma_tiling(a.D, (int)sizeof(T), TPR, 2);
    const size_t fixed = t.smem - (size_t)t.stages * (kTmaThreads / TPR) * a.D * sizeof(T) * 2;
    const size_t layer = (size_t)(kTmaThreads / TPR) * a.D * sizeof(T) * 2;
    t.stages = fixed + 3 * layer <= kTmaMaxSmem ? 3 : 2;      // the slot is held for the whole row: take the third slot whenever it fits
    t.smem = fixed + t.stages * layer;
    if (t.smem > kTmaMaxSmem) return kNotFused;
    static thread_local size_t configured_all[kMaxDevices] = {};
    size_t& configured = configured_all[current_device_slot()];
    if (t.smem > configured) {
        int rc = cuda_status(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)t.smem),
                             "norm_bwd_wide_bf16_kernel shared memory");
        if (rc != 0) return rc;
        configured = t.smem;
    }
    const int grid = (int)tma_grid(a.rows, TPR, launch_sms());
    const cudaError_t e = launch_pdl(kern, dim3(grid), dim3(kTmaThreads), t.smem, a.stream, (const T*)a.x, (const T*)a.dy,
                                     (const T*)a.gamma, (const T*)a.beta, a.mean, a.rstd, (T*)a.dx, a.partials, a.rows,
                                     (int)a.D, t.stages, device_status_ptr());
    if (e != cudaSuccess) return cuda_status(e, "norm_bwd_wide_bf16_kernel launch");
    if (n_partials) *n_partials = a.partials ? grid : 0;
    return 0;
}

template <typename T, int TPR, int VPT, int ACT, bool RMS, int NT = kTmaThreads>
static int launch_bwd_tma(const NormArgs& a, int64_t* n_partials) {
    if (a.dres != nullptr) {
        if constexpr (ACT == NB2_ACT_NONE) return launch_bwd_tma_res<T, TPR, VPT, ACT, RMS, true, NT>(a, n_partials);
        set_error("residual + norm is not fused with an activation");
        return NB2_ERR_DTYPE;
    }
    return launch_bwd_tma_res<T, TPR, VPT, ACT, RMS, false, NT>(a, n_partials);
}

template <typename T, int ACT, bool RMS>
static int launch_bwd_tma_shape(const NormArgs& a, TmaShape s, int64_t* n_partials) {
    constexpr int EPV = VecTraits<T>::EPV;
    constexpr int V16 = 16 / EPV;
    if (s.vpt == 3) {
        switch (s.tpr) {
            case 32:  return launch_bwd_tma<T, 32, 3, ACT, RMS>(a, n_partials);
            case 64:  return launch_bwd_tma<T, 64, 3, ACT, RMS>(a, n_partials);
            case 128: return launch_bwd_tma<T, 128, 3, ACT, RMS>(a, n_partials);
            case 256: return launch_bwd_tma<T, 256, 3, ACT, RMS>(a, n_partials);
            case 512: if constexpr (EPV == 4) return launch_bwd_tma<T, 512, 3, ACT, RMS>(a, n_partials);
            default: break;
        }
        set_error("norm bwd: no three-vector ring kernel for threads-per-row %d", s.tpr);
        return NB2_ERR_SHAPE;
    }
    if (s.tpr == 224 || s.tpr == 448) {
        constexpr int V8 = 8 / EPV;
        if (s.tpr == 224) return s.vpt == V16 ? launch_bwd_tma<T, 224, V16, ACT, RMS, 448>(a, n_partials)
                                              : launch_bwd_tma<T, 224, V8, ACT, RMS, 448>(a, n_partials);
        return s.vpt == V16 ? launch_bwd_tma<T, 448, V16, ACT, RMS, 448>(a, n_partials)
                            : launch_bwd_tma<T, 448, V8, ACT, RMS, 448>(a, n_partials);
    }
    if constexpr (EPV == 8) {
        if (s.tpr == 160) return s.vpt == 2 ? launch_bwd_tma<T, 160, 2, ACT, RMS, 480>(a, n_partials)
                                            : launch_bwd_tma<T, 160, 1, ACT, RMS, 480>(a, n_partials);
        if (s.tpr == 320) return launch_bwd_tma<T, 320, 2, ACT, RMS, 320>(a, n_partials);
    }
    if (s.vpt == 5) {
        if constexpr (EPV == 4) {
            switch (s.tpr) {
                case 32:  return launch_bwd_tma<T, 32, 5, ACT, RMS>(a, n_partials);
                case 64:  return launch_bwd_tma<T, 64, 5, ACT, RMS>(a, n_partials);
                case 128: return launch_bwd_tma<T, 128, 5, ACT, RMS>(a, n_partials);
                case 256: return launch_bwd_tma<T, 256, 5, ACT, RMS>(a, n_partials);
                default: break;
            }
        }
        set_error("norm bwd: no five-vector ring kernel for threads-per-row %d", s.tpr);
        return NB2_ERR_SHAPE;
    }
    // RMSNorm bf16 rows of 4 KiB and more: 32 columns per thread (measured on B200 against the 16-column
    // form with SiLU fused: +3% at D = 2048, +8% at 4096, +14% at 8192, -1% at 1024; with GELU +1-5%).
    // Without a fused activation the 16-column form is the faster one up to D = 4096 (246 us against 295
    // at [131072, 2048], 261 against 280 at [65536, 4096]) and the wide one only at 8192 (258 against 283).
    // LayerNorm's second accumulator column set does not fit the registers beside it (160 bytes spilled,
    // 25% slower), so it stays.
    if constexpr (EPV == 8 && RMS) {
        const int64_t wide_from = ACT == NB2_ACT_NONE ? 8192 : 2048;
        if (a.dres == nullptr && a.D >= wide_from && norm_path_override() == 0) {
            int rc = kNotFused;
            switch (s.tpr) {       // s.tpr threads x 16 columns == s.tpr / 2 threads x 32 columns
                case 64:  rc = launch_bwd_wide_bf16<32, ACT, RMS>(a, n_partials); break;
                case 128: rc = launch_bwd_wide_bf16<64, ACT, RMS>(a, n_partials); break;
                case 256: rc = launch_bwd_wide_bf16<128, ACT, RMS>(a, n_partials); break;
                case 512: rc = launch_bwd_wide_bf16<256, ACT, RMS>(a, n_partials); break;
                default: break;
            }
            if (rc != kNotFused) return rc;
        }
    }
    switch (s.tpr) {
        case 32:  return launch_bwd_tma<T, 32, V16, ACT, RMS>(a, n_partials);
        case 64:  return launch_bwd_tma<T, 64, V16, ACT, RMS>(a, n_partials);
        case 128: return launch_bwd_tma<T, 128, V16, ACT, RMS>(a, n_partials);
        case 256: return launch_bwd_tma<T, 256, V16, ACT, RMS>(a, n_partials);
        case 512: return launch_bwd_tma<T, 512, V16, ACT, RMS>(a, n_partials);
        default: break;
    }
    set_error("norm bwd: no ring kernel for threads-per-row %d", s.tpr);
    return NB2_ERR_SHAPE;
}

template <typename T, int TPR, int ACT, bool RMS>
static int launch_bwd_cfg(const NormArgs& a, int64_t* n_partials) {
    constexpr int VPT = bwd_vpt<T>();
    constexpr int THREADS = TPR > 256 ? TPR : 256;
    constexpr int MINB = TPR > 256 ? 1 : 2;
    const int grid = (int)norm_bwd_grid(a.rows, TPR, launch_sms());
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
        const TmaShape s = tma_bwd_shape(a.D, EPV);
        const bool affine = a.gamma != nullptr && (RMS || a.beta != nullptr || ACT == NB2_ACT_NONE);   // beta only enters through act'(z)
        if (a.dres != nullptr) {
            if (s.tpr != 0 && affine && tma_fits(a.D, (int)sizeof(T), s.tpr, 3)) return launch_bwd_tma_shape<T, ACT, RMS>(a, s, n_partials);
            return kNotFused;
        }
        if (s.tpr != 0 && affine && tma_preferred(RMS, a.D, (int)sizeof(T), true, ACT) && tma_fits(a.D, (int)sizeof(T), s.tpr, 2))
            return launch_bwd_tma_shape<T, ACT, RMS>(a, s, n_partials);
        switch (pick_tpr(a.D / EPV, bwd_vpt<T>())) {
            case 32:  return launch_bwd_cfg<T, 32, ACT, RMS>(a, n_partials);
            case 64:  return launch_bwd_cfg<T, 64, ACT, RMS>(a, n_partials);
            case 128: return launch_bwd_cfg<T, 128, ACT, RMS>(a, n_partials);
            case 256: return launch_bwd_cfg<T, 256, ACT, RMS>(a, n_partials);
            case 512: return launch_bwd_cfg<T, 512, ACT, RMS>(a, n_partials);
            default: break;
        }
    }
    if (a.dres != nullptr) return kNotFused;
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
int launch_norm_bwd(const NormArgs& a, int64_t* n_partials) {
    switch (a.act) {
        case NB2_ACT_NONE: return launch_bwd_act<T, NB2_ACT_NONE, RMS>(a, n_partials);
        case NB2_ACT_GELU: return launch_bwd_act<T, NB2_ACT_GELU, RMS>(a, n_partials);
        case NB2_ACT_SILU: return launch_bwd_act<T, NB2_ACT_SILU, RMS>(a, n_partials);
        default: set_error("unknown activation %d", a.act); return NB2_ERR_DTYPE;
    }
}

}  // namespace nb2
