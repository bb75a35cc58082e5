// Shared device/host helpers for the sm_100a row-op kernels.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/nott_b200.h"

namespace nb2 {

// ---------------------------------------------------------------- host side
void set_error(const char* fmt, ...);
int  cuda_status(cudaError_t e, const char* what);
int  sm_count();           // SMs of the current device (cached per device)
int  launch_sms();         // sm_count() less the SMs set aside by nb2_reserve_sms()

#define NB2_REQUIRE(cond, code, ...)            \
    do {                                        \
        if (!(cond)) {                          \
            ::nb2::set_error(__VA_ARGS__);      \
            return (code);                      \
        }                                       \
    } while (0)

// Launch with programmatic stream serialization: the grid may be scheduled while the previous
// kernel in the stream is still draining, and blocks in pdl_wait() until that kernel has
// completed and its writes are visible.  Behind a kernel that never signals (any kernel not
// from this library) this degenerates to the ordinary stream order.
template <typename... KArgs, typename... Args>
static inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                     cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// -------------------------------------------------------------- device side
// A 16-byte vector of activations: 4 fp32 or 8 bf16.
template <typename T> struct VecTraits;
template <> struct VecTraits<float> { static constexpr int EPV = 4; };
template <> struct VecTraits<__nv_bfloat16> { static constexpr int EPV = 8; };

// Programmatic dependent launch, device side.  pdl_wait(): block until the kernel this one was
// serialized behind has completed (a no-op for an ordinary launch); every kernel calls it before
// its first global-memory access.  pdl_release(): let the next kernel of the stream be scheduled
// onto SMs as this grid's CTAs retire.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Streaming (evict-first) 16-byte global load/store: every activation byte on
// this path is touched once per kernel, so it should not displace the affine
// parameters and rope tables that live in L2.
__device__ __forceinline__ uint4 ld_stream(const void* p) {
    return __ldcs(reinterpret_cast<const uint4*>(p));
}
__device__ __forceinline__ void st_stream(void* p, uint4 v) {
    __stcs(reinterpret_cast<uint4*>(p), v);
}
__device__ __forceinline__ uint4 ld_param(const void* p) {
    return __ldg(reinterpret_cast<const uint4*>(p));
}

// unpack one 16-byte vector into EPV floats / pack EPV floats into 16 bytes
template <typename T> __device__ __forceinline__ void unpack(const uint4& v, float* f);
template <> __device__ __forceinline__ void unpack<float>(const uint4& v, float* f) {
    f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y);
    f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
}
template <> __device__ __forceinline__ void unpack<__nv_bfloat16>(const uint4& v, float* f) {
    // bf16 -> fp32 is a 16-bit left shift; element 0 is the low half-word.
    f[0] = __uint_as_float(v.x << 16); f[1] = __uint_as_float(v.x & 0xffff0000u);
    f[2] = __uint_as_float(v.y << 16); f[3] = __uint_as_float(v.y & 0xffff0000u);
    f[4] = __uint_as_float(v.z << 16); f[5] = __uint_as_float(v.z & 0xffff0000u);
    f[6] = __uint_as_float(v.w << 16); f[7] = __uint_as_float(v.w & 0xffff0000u);
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);   // round-to-nearest-even
    return *reinterpret_cast<uint32_t*>(&h);
}
template <typename T> __device__ __forceinline__ uint4 pack(const float* f);
template <> __device__ __forceinline__ uint4 pack<float>(const float* f) {
    return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]),
                      __float_as_uint(f[2]), __float_as_uint(f[3]));
}
template <> __device__ __forceinline__ uint4 pack<__nv_bfloat16>(const float* f) {
    return make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]),
                      pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
}

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// ------------------------------------------------------------- activations
// GELU is the exact-erf form torch::gelu defaults to; SiLU is x*sigmoid(x).
//
// erf is not taken from the CUDA math library: at B200's HBM rate a forward
// element has an issue budget of ~35 instructions (fp32) or ~18 (bf16), and the
// library erff alone costs more than that.  Instead
//     erfc(|z|/sqrt2) = t * P(t) * exp(-z^2/2),   t = 1 / (1 + p |z|)
// with a degree-5 P fitted (weighted minimax over |z| <= 9.5, weight max(1,|z|)/2)
// to 9e-8; evaluated in fp32 with the approximate rcp/ex2 units the error is
// <= 5e-7 on erfc, i.e. <= 1.3e-7 absolute on GELU(z) and <= 2.6e-7 on GELU'(z):
// inside the 1e-6 absolute tolerance with room to spare, in 13 instructions of
// which 2 are MUFU.
constexpr float kInvSqrt2Pi = 0.39894228040143267794f;
constexpr float kErfcP  = 0.3329536741f;
// half of the fitted coefficients: gelu_half_erfc returns 0.5 * erfc(|z|/sqrt2)
constexpr float kErfcA1 = 0.5f * 2.4810082281e-01f;
constexpr float kErfcA2 = 0.5f * 3.9755105569e-01f;
constexpr float kErfcA3 = 0.5f * -1.5376413303e-01f;
constexpr float kErfcA4 = 0.5f * 7.2612069805e-01f;
constexpr float kErfcA5 = 0.5f * -2.1800861308e-01f;

__device__ __forceinline__ float fast_rcp(float x) {
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ float fast_ex2(float x) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
// q = 0.5 * erfc(|z|/sqrt2) = Phi(-|z|);  e = exp(-z^2/2)
__device__ __forceinline__ void gelu_half_erfc(float z, float& q, float& e) {
    const float az = fabsf(z);
    const float t = fast_rcp(fmaf(kErfcP, az, 1.0f));
    e = fast_ex2(z * z * -0.72134752044448170368f);          // -0.5 * log2(e) * z^2
    float p = fmaf(kErfcA5, t, kErfcA4);
    p = fmaf(p, t, kErfcA3);
    p = fmaf(p, t, kErfcA2);
    p = fmaf(p, t, kErfcA1);
    q = p * t * e;
}

template <int ACT> __device__ __forceinline__ float act_fwd(float z) {
    if constexpr (ACT == NB2_ACT_GELU) {
        float q, e;
        gelu_half_erfc(z, q, e);
        return fmaf(-fabsf(z), q, fmaxf(z, 0.0f));            // z >= 0: z - z q ;  z < 0: z q
    } else if constexpr (ACT == NB2_ACT_SILU) {
        return z * fast_rcp(1.0f + fast_ex2(z * -1.44269504088896340736f));
    } else {
        return z;
    }
}
// d act(z) / dz
template <int ACT> __device__ __forceinline__ float act_grad(float z) {
    if constexpr (ACT == NB2_ACT_GELU) {
        float q, e;
        gelu_half_erfc(z, q, e);
        const float cdf = z >= 0.0f ? 1.0f - q : q;
        return fmaf(z * kInvSqrt2Pi, e, cdf);                 // Phi(z) + z phi(z)
    } else if constexpr (ACT == NB2_ACT_SILU) {
        const float s = fast_rcp(1.0f + fast_ex2(z * -1.44269504088896340736f));
        return s * fmaf(z, 1.0f - s, 1.0f);                   // sigma(z) (1 + z (1 - sigma(z)))
    } else {
        return 1.0f;
    }
}

// ------------------------------------------------- packed fp32 pairs (sm_100)
// Blackwell issues one instruction for two fp32 fused multiply-adds on a 64-bit register pair.
// The norm kernels are bound by instruction issue once an activation is fused in (bf16 most of
// all: half the bytes per element, the same arithmetic), so their per-element maths is written
// on float2 pairs.  Each half is rounded exactly as the scalar instruction would round it, so
// act_fwd2 gives the same bits as act_fwd above; act_grad2 forms Phi(z) without a branch and
// differs from act_grad by at most 1.2e-7.
// PK selects the packed instruction; with PK false the same expression runs as two scalar
// instructions (identical results), which is what the fp32 forward kernels use: they are bound
// by memory, not by issue, and measured 5% slower with the packed forms.
template <bool PK = true> __device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
    if constexpr (PK) return __ffma2_rn(a, b, c);
    else return make_float2(fmaf(a.x, b.x, c.x), fmaf(a.y, b.y, c.y));
}
template <bool PK = true> __device__ __forceinline__ float2 mul2(float2 a, float2 b) {
    if constexpr (PK) return __fmul2_rn(a, b);
    else return make_float2(__fmul_rn(a.x, b.x), __fmul_rn(a.y, b.y));
}
template <bool PK = true> __device__ __forceinline__ float2 add2(float2 a, float2 b) {
    if constexpr (PK) return __fadd2_rn(a, b);
    else return make_float2(__fadd_rn(a.x, b.x), __fadd_rn(a.y, b.y));
}
__device__ __forceinline__ float2 splat2(float s) { return make_float2(s, s); }

// 16 bytes -> EPV/2 pairs of adjacent elements, and back
template <typename T> __device__ __forceinline__ void unpack2(const uint4& v, float2* f);
template <> __device__ __forceinline__ void unpack2<float>(const uint4& v, float2* f) {
    f[0] = make_float2(__uint_as_float(v.x), __uint_as_float(v.y));
    f[1] = make_float2(__uint_as_float(v.z), __uint_as_float(v.w));
}
template <> __device__ __forceinline__ void unpack2<__nv_bfloat16>(const uint4& v, float2* f) {
    f[0] = make_float2(__uint_as_float(v.x << 16), __uint_as_float(v.x & 0xffff0000u));
    f[1] = make_float2(__uint_as_float(v.y << 16), __uint_as_float(v.y & 0xffff0000u));
    f[2] = make_float2(__uint_as_float(v.z << 16), __uint_as_float(v.z & 0xffff0000u));
    f[3] = make_float2(__uint_as_float(v.w << 16), __uint_as_float(v.w & 0xffff0000u));
}
template <typename T> __device__ __forceinline__ uint4 pack2(const float2* f);
template <> __device__ __forceinline__ uint4 pack2<float>(const float2* f) {
    return make_uint4(__float_as_uint(f[0].x), __float_as_uint(f[0].y), __float_as_uint(f[1].x), __float_as_uint(f[1].y));
}
template <> __device__ __forceinline__ uint4 pack2<__nv_bfloat16>(const float2* f) {
    return make_uint4(pack_bf16x2(f[0].x, f[0].y), pack_bf16x2(f[1].x, f[1].y),
                      pack_bf16x2(f[2].x, f[2].y), pack_bf16x2(f[3].x, f[3].y));
}

// q = Phi(-|z|), e = exp(-z^2/2), naz = -|z| for both halves
template <bool PK>
__device__ __forceinline__ void gelu_half_erfc2(float2 z, float2& q, float2& e, float2& naz) {
    naz = make_float2(-fabsf(z.x), -fabsf(z.y));
    const float2 d = fma2<PK>(splat2(-kErfcP), naz, splat2(1.0f));       // 1 + p |z|
    const float2 t = make_float2(fast_rcp(d.x), fast_rcp(d.y));
    const float2 w = mul2<PK>(mul2<PK>(z, z), splat2(-0.72134752044448170368f));
    e = make_float2(fast_ex2(w.x), fast_ex2(w.y));
    float2 p = fma2<PK>(splat2(kErfcA5), t, splat2(kErfcA4));
    p = fma2<PK>(p, t, splat2(kErfcA3));
    p = fma2<PK>(p, t, splat2(kErfcA2));
    p = fma2<PK>(p, t, splat2(kErfcA1));
    q = mul2<PK>(mul2<PK>(p, t), e);
}
template <int ACT, bool PK = true> __device__ __forceinline__ float2 act_fwd2(float2 z) {
    if constexpr (ACT == NB2_ACT_GELU) {
        float2 q, e, naz;
        gelu_half_erfc2<PK>(z, q, e, naz);
        return fma2<PK>(naz, q, make_float2(fmaxf(z.x, 0.0f), fmaxf(z.y, 0.0f)));
    } else if constexpr (ACT == NB2_ACT_SILU) {
        const float2 w = mul2<PK>(z, splat2(-1.44269504088896340736f));
        const float2 d = add2<PK>(splat2(1.0f), make_float2(fast_ex2(w.x), fast_ex2(w.y)));
        return mul2<PK>(z, make_float2(fast_rcp(d.x), fast_rcp(d.y)));
    } else {
        return z;
    }
}
template <int ACT, bool PK = true> __device__ __forceinline__ float2 act_grad2(float2 z) {
    if constexpr (ACT == NB2_ACT_GELU) {
        float2 q, e, naz;
        gelu_half_erfc2<PK>(z, q, e, naz);
        // Phi(z) = 1/2 + sign(z) (1/2 - q): two sign copies instead of two compares and two selects
        const float2 hq = fma2<PK>(q, splat2(-1.0f), splat2(0.5f));
        const float2 sg = make_float2(copysignf(1.0f, z.x), copysignf(1.0f, z.y));
        const float2 cdf = fma2<PK>(sg, hq, splat2(0.5f));
        return fma2<PK>(mul2<PK>(z, splat2(kInvSqrt2Pi)), e, cdf);
    } else if constexpr (ACT == NB2_ACT_SILU) {
        const float2 w = mul2<PK>(z, splat2(-1.44269504088896340736f));
        const float2 d = add2<PK>(splat2(1.0f), make_float2(fast_ex2(w.x), fast_ex2(w.y)));
        const float2 s = make_float2(fast_rcp(d.x), fast_rcp(d.y));
        return mul2<PK>(s, fma2<PK>(z, fma2<PK>(s, splat2(-1.0f), splat2(1.0f)), splat2(1.0f)));
    } else {
        return splat2(1.0f);
    }
}

// ---------------------------------------------------------------- reductions
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// named barrier over `nthreads` threads (a multiple of 32), id 1..15
__device__ __forceinline__ void named_barrier(int id, int nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

}  // namespace nb2
