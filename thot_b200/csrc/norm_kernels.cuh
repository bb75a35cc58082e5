// LayerNorm / RMSNorm (+ fused activation) forward and backward, register-row
// variant: a group of TPR threads owns one row, each thread holds VPT 16-byte
// vectors of it in registers, rows cross HBM exactly once per kernel.
//
// Reference semantics: torch::nn::LayerNorm as Nott's blocks call it
// (src/block/details/transformers/classic.hpp:399-404,436,445,520) and
// RMSNormImpl::forward (src/block/details/transformers/mamba.hpp:124-142),
// followed by Activation::Details::apply (src/activation/apply.hpp:24-57).
#pragma once
#include "nb2_common.cuh"

namespace nb2 {

// Partial rows a backward CTA emits: LayerNorm [dgamma, dbeta], RMSNorm [dweight].
template <bool RMS> struct NormPartials { static constexpr int N = RMS ? 1 : 2; };

// Sum `v` over the TPR threads that share a row.  Every thread of the group
// receives the same value, added in the same order.
template <int TPR>
__device__ __forceinline__ float row_sum(float v, float* red /*[WPR] for this slot*/, int slot_barrier) {
    v = warp_sum(v);
    if constexpr (TPR > 32) {
        constexpr int WPR = TPR / 32;
        const int w = (threadIdx.x % TPR) >> 5;
        if ((threadIdx.x & 31) == 0) red[w] = v;
        named_barrier(slot_barrier, TPR);
        float t = 0.f;
#pragma unroll
        for (int i = 0; i < WPR; ++i) t += red[i];
        v = t;
    }
    return v;
}

// ------------------------------------------------------------------ forward
template <typename T, int TPR, int VPT, int ACT, bool RMS, int MINB>
__global__ void __launch_bounds__((TPR > 256 ? TPR : 256), MINB)
norm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ gamma, const T* __restrict__ beta,
                T* __restrict__ y, float* __restrict__ mean_out, float* __restrict__ rstd_out,
                int64_t rows, int D, float eps) {
    constexpr int EPV = VecTraits<T>::EPV;
    constexpr int THREADS = (TPR > 256 ? TPR : 256);
    constexpr int RPC = THREADS / TPR;            // rows in flight per CTA
    constexpr int WPR = (TPR + 31) / 32;
    __shared__ float red_a[RPC][WPR], red_b[RPC][WPR];

    const int nvec = D / EPV;
    const int slot = threadIdx.x / TPR;
    const int tr   = threadIdx.x % TPR;
    const float inv_d = 1.0f / (float)D;

    bool valid[VPT];
#pragma unroll
    for (int j = 0; j < VPT; ++j) valid[j] = (tr + j * TPR) < nvec;

    // affine parameters of this thread's columns, kept packed
    uint4 gpk[VPT], bpk[VPT];
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        if (gamma != nullptr && valid[j]) gpk[j] = ld_param(gamma + (size_t)(tr + j * TPR) * EPV);
        if (!RMS && beta != nullptr && valid[j]) bpk[j] = ld_param(beta + (size_t)(tr + j * TPR) * EPV);
    }
    const bool has_g = gamma != nullptr;
    const bool has_b = !RMS && beta != nullptr;

    const int64_t stride = (int64_t)gridDim.x * RPC;
    int64_t row = (int64_t)blockIdx.x * RPC + slot;

    uint4 cur[VPT];
    if (row < rows) {
        const T* xr = x + row * (int64_t)D;
#pragma unroll
        for (int j = 0; j < VPT; ++j)
            if (valid[j]) cur[j] = ld_stream(xr + (size_t)(tr + j * TPR) * EPV);
    }

    while (row < rows) {
        const int64_t nrow = row + stride;
        uint4 nxt[VPT];
        if (nrow < rows) {                       // next row's loads go out before this row's math
            const T* xr = x + nrow * (int64_t)D;
#pragma unroll
            for (int j = 0; j < VPT; ++j)
                if (valid[j]) nxt[j] = ld_stream(xr + (size_t)(tr + j * TPR) * EPV);
        }

        float v[VPT][EPV];
        float s = 0.f;
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            if (valid[j]) {
                unpack<T>(cur[j], v[j]);
#pragma unroll
                for (int e = 0; e < EPV; ++e) s += RMS ? v[j][e] * v[j][e] : v[j][e];
            }
        }
        float mu = 0.f, rs;
        if constexpr (RMS) {
            const float ms = row_sum<TPR>(s, red_a[slot], slot + 1) * inv_d;
            rs = rsqrtf(ms + eps);
        } else {
            mu = row_sum<TPR>(s, red_a[slot], slot + 1) * inv_d;
            float q = 0.f;
#pragma unroll
            for (int j = 0; j < VPT; ++j) {
                if (valid[j]) {
#pragma unroll
                    for (int e = 0; e < EPV; ++e) { const float d = v[j][e] - mu; q = fmaf(d, d, q); }
                }
            }
            const float var = row_sum<TPR>(q, red_b[slot], slot + 1) * inv_d;
            rs = rsqrtf(var + eps);
        }
        if (tr == 0) {
            if (!RMS && mean_out != nullptr) mean_out[row] = mu;
            if (rstd_out != nullptr) rstd_out[row] = rs;
        }

        T* yr = y + row * (int64_t)D;
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            if (valid[j]) {
                float g[EPV], b[EPV], o[EPV];
                if (has_g) unpack<T>(gpk[j], g);
                if (has_b) unpack<T>(bpk[j], b);
#pragma unroll
                for (int e = 0; e < EPV; ++e) {
                    float z = (v[j][e] - mu) * rs;
                    if (has_g) z *= g[e];
                    if (has_b) z += b[e];
                    o[e] = act_fwd<ACT>(z);
                }
                st_stream(yr + (size_t)(tr + j * TPR) * EPV, pack<T>(o));
            }
        }
        if constexpr (TPR > 32 && RMS) {
            // red_a is rewritten next iteration; LayerNorm's second barrier already orders that.
            named_barrier(slot + 1, TPR);
        }
#pragma unroll
        for (int j = 0; j < VPT; ++j) cur[j] = nxt[j];
        row = nrow;
    }
}

// ----------------------------------------------------------------- backward
// dz = dy * act'(z);  dgamma += dz*xhat;  dbeta += dz;  g = dz*gamma
// LayerNorm: dx = rstd * (g - mean_row(g) - xhat * mean_row(g*xhat))
// RMSNorm  : dx = rstd * (g - xhat * mean_row(g*xhat)),  xhat = x*rstd
// Each thread owns fixed columns, so its dgamma/dbeta accumulators stay in
// registers for the whole kernel; row slots are combined in a fixed order at
// the end and the CTA writes one [NP, D] fp32 partial.
template <typename T, int TPR, int VPT, int ACT, bool RMS, int MINB>
__global__ void __launch_bounds__((TPR > 256 ? TPR : 256), MINB)
norm_bwd_kernel(const T* __restrict__ x, const T* __restrict__ dy,
                const T* __restrict__ gamma, const T* __restrict__ beta,
                const float* __restrict__ mean_in, const float* __restrict__ rstd_in,
                T* __restrict__ dx, float* __restrict__ partials,
                int64_t rows, int D) {
    constexpr int EPV = VecTraits<T>::EPV;
    constexpr int THREADS = (TPR > 256 ? TPR : 256);
    constexpr int RPC = THREADS / TPR;
    constexpr int WPR = (TPR + 31) / 32;
    constexpr int NP = NormPartials<RMS>::N;
    constexpr int COLS = TPR * VPT * EPV;         // columns this config can hold
    __shared__ float red_a[RPC][WPR], red_b[RPC][WPR];
    __shared__ float comb[(RPC > 1) ? NP * COLS : 1];

    const int nvec = D / EPV;
    const int slot = threadIdx.x / TPR;
    const int tr   = threadIdx.x % TPR;
    const float inv_d = 1.0f / (float)D;

    bool valid[VPT];
#pragma unroll
    for (int j = 0; j < VPT; ++j) valid[j] = (tr + j * TPR) < nvec;

    uint4 gpk[VPT], bpk[VPT];
    const bool has_g = gamma != nullptr;
    const bool has_b = !RMS && beta != nullptr;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        if (has_g && valid[j]) gpk[j] = ld_param(gamma + (size_t)(tr + j * TPR) * EPV);
        if (has_b && valid[j]) bpk[j] = ld_param(beta + (size_t)(tr + j * TPR) * EPV);
    }

    float acc_g[VPT][EPV], acc_b[RMS ? 1 : VPT][EPV];
#pragma unroll
    for (int j = 0; j < VPT; ++j)
#pragma unroll
        for (int e = 0; e < EPV; ++e) { acc_g[j][e] = 0.f; if (!RMS) acc_b[j][e] = 0.f; }

    const int64_t stride = (int64_t)gridDim.x * RPC;
    for (int64_t row = (int64_t)blockIdx.x * RPC + slot; row < rows; row += stride) {
        const T* xr = x + row * (int64_t)D;
        const T* dr = dy + row * (int64_t)D;
        uint4 xp[VPT], dp[VPT];
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            if (valid[j]) {
                xp[j] = ld_stream(xr + (size_t)(tr + j * TPR) * EPV);
                dp[j] = ld_stream(dr + (size_t)(tr + j * TPR) * EPV);
            }
        }
        const float mu = RMS ? 0.f : __ldg(mean_in + row);
        const float rs = __ldg(rstd_in + row);

        float xh[VPT][EPV], gg[VPT][EPV];
        float s1 = 0.f, s2 = 0.f;
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            if (valid[j]) {
                float xv[EPV], dv[EPV], g[EPV], b[EPV];
                unpack<T>(xp[j], xv);
                unpack<T>(dp[j], dv);
                if (has_g) unpack<T>(gpk[j], g);
                if (has_b) unpack<T>(bpk[j], b);
#pragma unroll
                for (int e = 0; e < EPV; ++e) {
                    const float h = (xv[e] - mu) * rs;
                    float dz = dv[e];
                    if constexpr (ACT != NB2_ACT_NONE) {
                        float z = h;
                        if (has_g) z *= g[e];
                        if (has_b) z += b[e];
                        dz *= act_grad<ACT>(z);
                    }
                    acc_g[j][e] = fmaf(dz, h, acc_g[j][e]);
                    if constexpr (!RMS) acc_b[j][e] += dz;
                    const float gv = has_g ? __fmul_rn(dz, g[e]) : dz;   // rounded once: g - mean(g) cancels exactly
                    s1 += gv;
                    s2 = fmaf(gv, h, s2);
                    xh[j][e] = h;
                    gg[j][e] = gv;
                }
            }
        }
        float m1 = 0.f;
        if constexpr (!RMS) m1 = row_sum<TPR>(s1, red_a[slot], slot + 1) * inv_d;
        const float m2 = row_sum<TPR>(s2, red_b[slot], slot + 1) * inv_d;

        T* xo = dx + row * (int64_t)D;
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            if (valid[j]) {
                float o[EPV];
#pragma unroll
                for (int e = 0; e < EPV; ++e) o[e] = rs * (gg[j][e] - m1 - xh[j][e] * m2);
                st_stream(xo + (size_t)(tr + j * TPR) * EPV, pack<T>(o));
            }
        }
        if constexpr (TPR > 32 && RMS) named_barrier(slot + 1, TPR);   // red_b reuse
    }

    if (partials == nullptr) return;
    float* out = partials + (size_t)blockIdx.x * NP * D;
    if constexpr (RPC > 1) {
        // combine row slots 0..RPC-1 in order
        for (int sl = 0; sl < RPC; ++sl) {
            if (slot == sl) {
#pragma unroll
                for (int j = 0; j < VPT; ++j) {
                    if (valid[j]) {
                        const int c0 = (tr + j * TPR) * EPV;
#pragma unroll
                        for (int e = 0; e < EPV; ++e) {
                            if (sl == 0) {
                                comb[c0 + e] = acc_g[j][e];
                                if constexpr (!RMS) comb[COLS + c0 + e] = acc_b[j][e];
                            } else {
                                comb[c0 + e] += acc_g[j][e];
                                if constexpr (!RMS) comb[COLS + c0 + e] += acc_b[j][e];
                            }
                        }
                    }
                }
            }
            __syncthreads();
        }
        for (int c = threadIdx.x; c < D; c += THREADS) {
            out[c] = comb[c];
            if constexpr (!RMS) out[D + c] = comb[COLS + c];
        }
    } else {
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            if (valid[j]) {
                const int c0 = (tr + j * TPR) * EPV;
                *reinterpret_cast<float4*>(out + c0) =
                    make_float4(acc_g[j][0], acc_g[j][1], acc_g[j][2], acc_g[j][3]);
                if constexpr (EPV == 8)
                    *reinterpret_cast<float4*>(out + c0 + 4) =
                        make_float4(acc_g[j][4], acc_g[j][5], acc_g[j][6], acc_g[j][7]);
                if constexpr (!RMS) {
                    *reinterpret_cast<float4*>(out + D + c0) =
                        make_float4(acc_b[j][0], acc_b[j][1], acc_b[j][2], acc_b[j][3]);
                    if constexpr (EPV == 8)
                        *reinterpret_cast<float4*>(out + D + c0 + 4) =
                            make_float4(acc_b[j][4], acc_b[j][5], acc_b[j][6], acc_b[j][7]);
                }
            }
        }
    }
}

// ------------------------------------------------- any-D, any-alignment path
// One warp per row, scalar accesses, the row re-read from L1/L2.  Covers widths
// that are not a multiple of the 16-byte vector, unaligned views, and D beyond
// the register-row configurations.  Correctness path, not a fast path.
template <typename T, int ACT, bool RMS>
__global__ void __launch_bounds__(256)
norm_fwd_generic(const T* __restrict__ x, const T* __restrict__ gamma, const T* __restrict__ beta,
                 T* __restrict__ y, float* __restrict__ mean_out, float* __restrict__ rstd_out,
                 int64_t rows, int64_t D, float eps) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int64_t nwarps = (int64_t)gridDim.x * (blockDim.x >> 5);
    const float inv_d = 1.0f / (float)D;
    for (int64_t row = warp; row < rows; row += nwarps) {
        const T* xr = x + row * D;
        float s = 0.f;
        for (int64_t c = lane; c < D; c += 32) { const float v = to_f32(xr[c]); s += RMS ? v * v : v; }
        s = warp_sum(s);
        float mu = 0.f, rs;
        if constexpr (RMS) {
            rs = rsqrtf(s * inv_d + eps);
        } else {
            mu = s * inv_d;
            float q = 0.f;
            for (int64_t c = lane; c < D; c += 32) { const float d = to_f32(xr[c]) - mu; q = fmaf(d, d, q); }
            rs = rsqrtf(warp_sum(q) * inv_d + eps);
        }
        if (lane == 0) {
            if (!RMS && mean_out != nullptr) mean_out[row] = mu;
            if (rstd_out != nullptr) rstd_out[row] = rs;
        }
        T* yr = y + row * D;
        for (int64_t c = lane; c < D; c += 32) {
            float z = (to_f32(xr[c]) - mu) * rs;
            if (gamma != nullptr) z *= to_f32(gamma[c]);
            if (!RMS && beta != nullptr) z += to_f32(beta[c]);
            yr[c] = from_f32<T>(act_fwd<ACT>(z));
        }
    }
}

template <typename T, int ACT, bool RMS>
__global__ void __launch_bounds__(256)
norm_bwd_generic_dx(const T* __restrict__ x, const T* __restrict__ dy,
                    const T* __restrict__ gamma, const T* __restrict__ beta,
                    const float* __restrict__ mean_in, const float* __restrict__ rstd_in,
                    T* __restrict__ dx, int64_t rows, int64_t D) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int64_t nwarps = (int64_t)gridDim.x * (blockDim.x >> 5);
    const float inv_d = 1.0f / (float)D;
    for (int64_t row = warp; row < rows; row += nwarps) {
        const T* xr = x + row * D;
        const T* dr = dy + row * D;
        const float mu = RMS ? 0.f : mean_in[row];
        const float rs = rstd_in[row];
        float s1 = 0.f, s2 = 0.f;
        for (int64_t c = lane; c < D; c += 32) {
            const float h = (to_f32(xr[c]) - mu) * rs;
            const float g = gamma != nullptr ? to_f32(gamma[c]) : 1.f;
            float dz = to_f32(dr[c]);
            if constexpr (ACT != NB2_ACT_NONE) {
                float z = h * g;
                if (!RMS && beta != nullptr) z += to_f32(beta[c]);
                dz *= act_grad<ACT>(z);
            }
            const float gv = __fmul_rn(dz, g);
            s1 += gv;
            s2 = fmaf(gv, h, s2);
        }
        const float m1 = RMS ? 0.f : warp_sum(s1) * inv_d;
        const float m2 = warp_sum(s2) * inv_d;
        T* xo = dx + row * D;
        for (int64_t c = lane; c < D; c += 32) {
            const float h = (to_f32(xr[c]) - mu) * rs;
            const float g = gamma != nullptr ? to_f32(gamma[c]) : 1.f;
            float dz = to_f32(dr[c]);
            if constexpr (ACT != NB2_ACT_NONE) {
                float z = h * g;
                if (!RMS && beta != nullptr) z += to_f32(beta[c]);
                dz *= act_grad<ACT>(z);
            }
            xo[c] = from_f32<T>(rs * (__fmul_rn(dz, g) - m1 - h * m2));
        }
    }
}

// Column sums for the generic path: CTA `b` owns a row block and writes one
// partial; thread per column, coalesced across the CTA.
template <typename T, int ACT, bool RMS>
__global__ void __launch_bounds__(256)
norm_bwd_generic_cols(const T* __restrict__ x, const T* __restrict__ dy,
                      const T* __restrict__ gamma, const T* __restrict__ beta,
                      const float* __restrict__ mean_in, const float* __restrict__ rstd_in,
                      float* __restrict__ partials, int64_t rows, int64_t D, int64_t rows_per_cta) {
    constexpr int NP = NormPartials<RMS>::N;
    const int64_t r0 = (int64_t)blockIdx.y * rows_per_cta;
    const int64_t r1 = (r0 + rows_per_cta < rows) ? r0 + rows_per_cta : rows;
    const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= D) return;
    const float g = gamma != nullptr ? to_f32(gamma[c]) : 1.f;
    const float b = (!RMS && beta != nullptr) ? to_f32(beta[c]) : 0.f;
    float ag = 0.f, ab = 0.f;
    for (int64_t row = r0; row < r1; ++row) {
        const float mu = RMS ? 0.f : mean_in[row];
        const float h = (to_f32(x[row * D + c]) - mu) * rstd_in[row];
        float dz = to_f32(dy[row * D + c]);
        if constexpr (ACT != NB2_ACT_NONE) dz *= act_grad<ACT>(fmaf(h, g, b));
        ag = fmaf(dz, h, ag);
        ab += dz;
    }
    float* out = partials + (size_t)blockIdx.y * NP * D;
    out[c] = ag;
    if constexpr (!RMS) out[D + c] = ab;
}

}  // namespace nb2
