// Backward ring kernel with 32 columns per thread ("wide"): half the threads per row of
// norm_bwd_tma_kernel, so a 1024-column row is one warp (no barrier in its reductions) and the
// per-row fixed work (wait, request, reductions, addresses) is spread over twice the columns.
//
// 32 columns of dgamma/dbeta accumulators already take 64 registers, so the row's g = dz * gamma
// cannot also stay in registers across the reduction.  It is parked in the row's own ring slot
// instead: a bf16 slot holds x and dy, 2 + 2 bytes per column, exactly the 4 bytes of one fp32 g;
// each thread overwrites only the two 16-byte vectors it has itself just read (x's and dy's), so no
// thread waits for another.  xhat is recomputed from the thread's raw x vectors, which stay in
// registers (16 of them).  The slot is therefore busy until the row's dX has been formed and is
// re-requested then; with three slots per group two rows are still in flight behind the current one.
#pragma once
#include "norm_tma_kernels.cuh"

namespace nb2 {

// generic-proxy writes to shared memory must be ordered before the bulk copy (async proxy) that
// overwrites the same bytes
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Instantiated for RMSNorm only (LayerNorm's dbeta columns would push it over the register file).
template <int TPR, int ACT, bool RMS, int NT = kTmaThreads>
__global__ void __launch_bounds__(NT, 1)
norm_bwd_wide_bf16_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy,
                          const __nv_bfloat16* __restrict__ gamma, const __nv_bfloat16* __restrict__ beta,
                          const float* __restrict__ mean_in, const float* __restrict__ rstd_in,
                          __nv_bfloat16* __restrict__ dx, float* __restrict__ partials,
                          int64_t rows, int D, int stages, unsigned int* __restrict__ status) {
    using T = __nv_bfloat16;
    constexpr int EPV = 8, VPT = 4;
    constexpr int RPC = NT / TPR;
    constexpr int WPR = (TPR + 31) / 32;
    constexpr int NP = NormPartials<RMS>::N;
    constexpr int COLS = TPR * VPT * EPV;
    static_assert(NT % TPR == 0 && RPC <= kTmaMaxGroups, "row groups must tile the CTA");
    static_assert(TPR <= 32 || RPC <= 14, "one named barrier per multi-warp row group");

    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t row_bytes = (uint32_t)D * sizeof(T);
    const uint32_t slot_bytes = 2 * row_bytes;
    const TmaSmem sm(smem, tma_param_bytes(D, (int)sizeof(T)));
    pdl_release();
    pdl_wait();
    tma_setup<T>(sm, RPC, stages, (int)row_bytes, gamma, RMS ? nullptr : beta);

    const int grp = threadIdx.x / TPR;
    const int tr = threadIdx.x % TPR;
    const int nvec = D / EPV;
    const float inv_d = 1.0f / (float)D;
    uint64_t* full = sm.full + grp * kTmaMaxStages;
    volatile int* gave_up = sm.abort_flag + grp;
    uint8_t* ring = sm.ring + (size_t)grp * stages * slot_bytes;
    const uint8_t* src0 = reinterpret_cast<const uint8_t*>(x);
    const uint8_t* src1 = reinterpret_cast<const uint8_t*>(dy);
    const int64_t first = (int64_t)blockIdx.x * RPC + grp;
    const int64_t stride = (int64_t)gridDim.x * RPC;
    uint64_t policy = 0;
    if (tr == 0) {
        policy = policy_evict_first();
        for (int s = 0; s < stages; ++s) {
            const int64_t row = first + s * stride;
            if (row < rows) request_row(&full[s], ring + (size_t)s * slot_bytes, src0, src1, nullptr, row, row_bytes, policy);
        }
    }

    float2 acc_g[VPT][EPV / 2], acc_b[RMS ? 1 : VPT][EPV / 2];
#pragma unroll
    for (int j = 0; j < VPT; ++j)
#pragma unroll
        for (int e = 0; e < EPV / 2; ++e) { acc_g[j][e] = make_float2(0.f, 0.f); if (!RMS) acc_b[j][e] = make_float2(0.f, 0.f); }

    float mu_next = 0.f, rs_next = 0.f;
    if (first < rows) { if (!RMS) mu_next = __ldg(mean_in + first); rs_next = __ldg(rstd_in + first); }

    int i = 0, s = 0;
    uint32_t phase = 0;
    for (int64_t row = first; row < rows; row += stride, ++i) {
        const float mu = mu_next, rs = rs_next;
        if (row + stride < rows) { if (!RMS) mu_next = __ldg(mean_in + row + stride); rs_next = __ldg(rstd_in + row + stride); }
        mbar_wait_bounded(&full[s], phase, gave_up, kStatusFullTimeout, status);
        uint4* sx = reinterpret_cast<uint4*>(ring + (size_t)s * slot_bytes);
        uint4* sd = reinterpret_cast<uint4*>(ring + (size_t)s * slot_bytes + row_bytes);
        uint4 xraw[VPT];
        float2 s1 = make_float2(0.f, 0.f), s2 = make_float2(0.f, 0.f);
        const float2 nmu = splat2(-mu), rs2 = splat2(rs);
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            float2 xv[EPV / 2], dv[EPV / 2], g[EPV / 2], b[EPV / 2], gv[EPV / 2];
            xraw[j] = sx[tr + j * TPR];
            unpack2<T>(xraw[j], xv);
            unpack2<T>(sd[tr + j * TPR], dv);
            load_param2<T>(sm.gamma, tr + j * TPR, nvec, g);
            if constexpr (!RMS && ACT != NB2_ACT_NONE) load_param2<T>(sm.beta, tr + j * TPR, nvec, b);
#pragma unroll
            for (int e = 0; e < EPV / 2; ++e) {
                const float2 h = mul2(add2(xv[e], nmu), rs2);
                float2 dz = dv[e];
                if constexpr (ACT != NB2_ACT_NONE) {
                    const float2 z = RMS ? mul2(h, g[e]) : fma2(h, g[e], b[e]);
                    dz = mul2(dz, act_grad2<ACT>(z));
                }
                acc_g[j][e] = fma2(dz, h, acc_g[j][e]);
                if constexpr (!RMS) acc_b[j][e] = add2(acc_b[j][e], dz);
                gv[e] = mul2(dz, g[e]);
                s1 = add2(s1, gv[e]);
                s2 = fma2(gv[e], h, s2);
            }
            // park g over this thread's own x and dy vectors of the slot
            sx[tr + j * TPR] = make_uint4(__float_as_uint(gv[0].x), __float_as_uint(gv[0].y), __float_as_uint(gv[1].x), __float_as_uint(gv[1].y));
            sd[tr + j * TPR] = make_uint4(__float_as_uint(gv[2].x), __float_as_uint(gv[2].y), __float_as_uint(gv[3].x), __float_as_uint(gv[3].y));
        }
        float m1 = 0.f, m2;
        float* red = (i & 1) ? sm.red_b : sm.red_a;
        if constexpr (!RMS) {
            const float2 m = row_sum2<TPR>(make_float2(s1.x + s1.y, s2.x + s2.y), reinterpret_cast<float2*>(red) + grp * WPR, grp + 1);
            m1 = m.x * inv_d;
            m2 = m.y * inv_d;
        } else {
            m2 = row_sum<TPR>(s2.x + s2.y, red + grp * WPR, grp + 1) * inv_d;
        }
        if (group_gave_up<TPR>(gave_up)) break;
        __nv_bfloat16* xo = dx + row * (int64_t)D;
        const float2 nm1 = splat2(-m1), nm2 = splat2(-m2);
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            float2 xv[EPV / 2], gv[EPV / 2], o[EPV / 2];
            unpack2<T>(xraw[j], xv);
            unpack2<float>(sx[tr + j * TPR], gv);
            unpack2<float>(sd[tr + j * TPR], gv + 2);
#pragma unroll
            for (int e = 0; e < EPV / 2; ++e) {
                const float2 h = mul2(add2(xv[e], nmu), rs2);
                o[e] = mul2(rs2, fma2(h, nm2, add2(gv[e], nm1)));
            }
            st_stream(xo + (size_t)(tr + j * TPR) * EPV, pack2<T>(o));
        }
        // every thread's last access to the slot is behind it: order those against the next bulk copy
        fence_proxy_async_smem();
        if constexpr (TPR > 32) named_barrier(grp + 1, TPR); else __syncwarp();
        if (tr == 0) {
            const int64_t ahead = row + (int64_t)stages * stride;
            if (ahead < rows) request_row(&full[s], ring + (size_t)s * slot_bytes, src0, src1, nullptr, ahead, row_bytes, policy);
        }
        if (++s == stages) { s = 0; phase ^= 1u; }
    }
    if (tr == 0 && *gave_up) {
        for (int b = 0; b < stages; ++b) {
            const int ib = i + b;
            if (first + (int64_t)ib * stride < rows) mbar_wait_drain(&full[ib % stages], (uint32_t)((ib / stages) & 1));
        }
    }

    if (partials == nullptr) return;
    float* comb = reinterpret_cast<float*>(sm.ring);
    float* out = partials + (size_t)blockIdx.x * NP * D;
    __syncthreads();
    for (int sl = 0; sl < RPC; ++sl) {
        if (grp == sl) {
#pragma unroll
            for (int j = 0; j < VPT; ++j) {
                const int c0 = (tr + j * TPR) * EPV;
#pragma unroll
                for (int e = 0; e < EPV; ++e) {
                    const float ag = (e & 1) ? acc_g[j][e / 2].y : acc_g[j][e / 2].x;
                    float ab = 0.f;
                    if constexpr (!RMS) ab = (e & 1) ? acc_b[j][e / 2].y : acc_b[j][e / 2].x;
                    if (sl == 0) {
                        comb[c0 + e] = ag;
                        if constexpr (!RMS) comb[COLS + c0 + e] = ab;
                    } else {
                        comb[c0 + e] += ag;
                        if constexpr (!RMS) comb[COLS + c0 + e] += ab;
                    }
                }
            }
        }
        __syncthreads();
    }
    for (int c = threadIdx.x; c < D; c += NT) {
        out[c] = comb[c];
        if constexpr (!RMS) out[D + c] = comb[COLS + c];
    }
}

}  // namespace nb2
