// Rotary embedding, rotate-half pairing, fp32 maths on fp32/bf16 data.
// The reference has no rotary code (docs/sub/block/README.md:132-136 only
// mentions it); the semantics are: angle(s,i) = float(pos[s]) * float(theta^(-2i/hd)),
// out[i] = x[i]cos - x[i+hd/2]sin, out[i+hd/2] = x[i+hd/2]cos + x[i]sin.
#include <math.h>
#include "launchers.h"

namespace nb2 {

constexpr int ROPE_MAX_HALF = 256;   // inverse frequencies that travel as kernel arguments
struct RopeFreq { float inv_freq[ROPE_MAX_HALF]; };

// cos/sin are evaluated in fp64 and rounded once, so the table equals
// (float)cos((double)angle) of a libm host to the last bit in all but
// double-rounding corner cases.
__global__ void __launch_bounds__(256)
rope_table_kernel(float2* __restrict__ cs, const int32_t* __restrict__ positions, int64_t S, int half,
                  const __grid_constant__ RopeFreq f, double theta, int hd, bool freq_in_args) {
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= S * half) return;
    const int64_t s = idx / half;
    const int i = (int)(idx - s * half);
    const float inv = freq_in_args ? f.inv_freq[i] : (float)pow(theta, -2.0 * (double)i / (double)hd);
    const float pos = positions != nullptr ? (float)positions[s] : (float)s;
    const float ang = pos * inv;
    cs[idx] = make_float2((float)cos((double)ang), (float)sin((double)ang));
}

// One CTA per (b, s) token; threads walk the (head, vector-of-first-half) pairs.
template <typename T, bool VEC>
__global__ void __launch_bounds__(256)
rope_apply_kernel(const T* __restrict__ x, const float2* __restrict__ cs, T* __restrict__ out,
                  int64_t tokens, int S, int H, int hd, float sign) {
    constexpr int EPV = VEC ? VecTraits<T>::EPV : 1;
    const int half = hd >> 1;
    const int hv = half / EPV;                   // vectors per half head
    const int per_token = H * hv;
    for (int64_t tok = blockIdx.x; tok < tokens; tok += gridDim.x) {
        const int s = (int)(tok % S);
        const T* xt = x + tok * (int64_t)H * hd;
        T* ot = out + tok * (int64_t)H * hd;
        const float2* ct = cs + (int64_t)s * half;
        for (int p = threadIdx.x; p < per_token; p += blockDim.x) {
            const int h = p / hv, v = p - h * hv;
            const int o1 = h * hd + v * EPV, o2 = o1 + half;
            if constexpr (VEC) {
                const uint4 p1 = ld_stream(xt + o1), p2 = ld_stream(xt + o2);
                float a[EPV], b[EPV], ra[EPV], rb[EPV];
                unpack<T>(p1, a);
                unpack<T>(p2, b);
#pragma unroll
                for (int e = 0; e < EPV; e += 2) {
                    const float4 c2 = __ldg(reinterpret_cast<const float4*>(ct + v * EPV + e));
                    ra[e]     = a[e] * c2.x - sign * b[e] * c2.y;
                    rb[e]     = b[e] * c2.x + sign * a[e] * c2.y;
                    ra[e + 1] = a[e + 1] * c2.z - sign * b[e + 1] * c2.w;
                    rb[e + 1] = b[e + 1] * c2.z + sign * a[e + 1] * c2.w;
                }
                st_stream(ot + o1, pack<T>(ra));
                st_stream(ot + o2, pack<T>(rb));
            } else {
                const float a = to_f32(xt[o1]), b = to_f32(xt[o2]);
                const float2 c = ct[v];
                ot[o1] = from_f32<T>(a * c.x - sign * b * c.y);
                ot[o2] = from_f32<T>(b * c.x + sign * a * c.y);
            }
        }
    }
}

int launch_rope_table(float* cos_sin, const int32_t* positions, int64_t S, int64_t hd, double theta, cudaStream_t st) {
    const int half = (int)(hd / 2);
    if (S == 0 || half == 0) return 0;
    RopeFreq f;
    const bool in_args = half <= ROPE_MAX_HALF;
    for (int i = 0; i < ROPE_MAX_HALF; ++i)
        f.inv_freq[i] = (in_args && i < half) ? (float)pow(theta, -2.0 * (double)i / (double)hd) : 0.f;
    const int64_t n = S * half;
    rope_table_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(
        reinterpret_cast<float2*>(cos_sin), positions, S, half, f, theta, (int)hd, in_args);
    return cuda_status(cudaGetLastError(), "rope table launch");
}

template <typename T>
static int launch_rope_t(const void* x, const float* cs, void* out, int64_t B, int64_t S, int64_t H,
                         int64_t hd, bool inverse, cudaStream_t st) {
    constexpr int EPV = VecTraits<T>::EPV;
    const int64_t tokens = B * S;
    if (tokens == 0 || H == 0 || hd == 0) return 0;
    const int64_t half = hd / 2;
    const bool vec_ok = (half % EPV == 0) && aligned16(x) && aligned16(out) && aligned16(cs);
    int64_t grid = tokens;
    const int64_t cap = (int64_t)sm_count() * 64;
    if (grid > cap) grid = cap;
    const float sign = inverse ? -1.f : 1.f;
    const int64_t per_token = H * (vec_ok ? half / EPV : half);
    int threads = 256;
    while (threads > 32 && threads / 2 >= per_token) threads /= 2;
    if (vec_ok)
        rope_apply_kernel<T, true><<<(unsigned)grid, threads, 0, st>>>(
            (const T*)x, reinterpret_cast<const float2*>(cs), (T*)out, tokens, (int)S, (int)H, (int)hd, sign);
    else
        rope_apply_kernel<T, false><<<(unsigned)grid, threads, 0, st>>>(
            (const T*)x, reinterpret_cast<const float2*>(cs), (T*)out, tokens, (int)S, (int)H, (int)hd, sign);
    return cuda_status(cudaGetLastError(), "rope apply launch");
}

int launch_rope_apply(const void* x, const float* cs, void* out, int64_t B, int64_t S, int64_t H,
                      int64_t hd, int dtype, bool inverse, cudaStream_t st) {
    return dtype == NB2_F32 ? launch_rope_t<float>(x, cs, out, B, S, H, hd, inverse, st)
                            : launch_rope_t<__nv_bfloat16>(x, cs, out, B, S, H, hd, inverse, st);
}

}  // namespace nb2
