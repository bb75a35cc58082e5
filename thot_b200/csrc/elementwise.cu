// Stand-alone activations and the SiLU gate (forward and backward).
//
// Reference semantics: Nott::Activation::Details::GeLU / SiLU / SwiGLU
// (src/activation/details/gelu.hpp:11-15, silu.hpp:12-16, swiglu.hpp:13-25)
// and Mamba's gated feed forward (src/block/details/transformers/mamba.hpp:441-449).
// Pure streaming kernels: every thread keeps UNROLL independent 16-byte loads
// in flight, maths in fp32, one pass over HBM.
#include "launchers.h"

namespace nb2 {

constexpr int EW_THREADS = 256;
constexpr int EW_UNROLL = 4;

template <typename T, int ACT, bool BWD>
__global__ void __launch_bounds__(EW_THREADS)
act_vec_kernel(const T* __restrict__ x, const T* __restrict__ dy, T* __restrict__ out, int64_t nvec) {
    constexpr int EPV = VecTraits<T>::EPV;
    const int64_t base = (int64_t)blockIdx.x * (EW_THREADS * EW_UNROLL) + threadIdx.x;
    uint4 xv[EW_UNROLL], dv[EW_UNROLL];
#pragma unroll
    for (int k = 0; k < EW_UNROLL; ++k) {
        const int64_t i = base + (int64_t)k * EW_THREADS;
        if (i < nvec) {
            xv[k] = ld_stream(x + i * EPV);
            if (BWD) dv[k] = ld_stream(dy + i * EPV);
        }
    }
#pragma unroll
    for (int k = 0; k < EW_UNROLL; ++k) {
        const int64_t i = base + (int64_t)k * EW_THREADS;
        if (i < nvec) {
            float a[EPV], d[EPV], o[EPV];
            unpack<T>(xv[k], a);
            if (BWD) unpack<T>(dv[k], d);
#pragma unroll
            for (int e = 0; e < EPV; ++e) o[e] = BWD ? d[e] * act_grad<ACT>(a[e]) : act_fwd<ACT>(a[e]);
            st_stream(out + i * EPV, pack<T>(o));
        }
    }
}

template <typename T, int ACT, bool BWD>
__global__ void __launch_bounds__(EW_THREADS)
act_scalar_kernel(const T* __restrict__ x, const T* __restrict__ dy, T* __restrict__ out,
                  int64_t begin, int64_t n) {
    for (int64_t i = begin + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (int64_t)gridDim.x * blockDim.x) {
        const float a = to_f32(x[i]);
        out[i] = from_f32<T>(BWD ? to_f32(dy[i]) * act_grad<ACT>(a) : act_fwd<ACT>(a));
    }
}

template <typename T, int ACT, bool BWD>
static int launch_act_t(const void* x, const void* dy, void* out, int64_t n, cudaStream_t st) {
    constexpr int EPV = VecTraits<T>::EPV;
    if (n == 0) return 0;
    const bool vec_ok = aligned16(x) && aligned16(out) && (!BWD || aligned16(dy));
    int64_t done = 0;
    if (vec_ok && n >= EPV) {
        const int64_t nvec = n / EPV;
        const int64_t per_cta = EW_THREADS * EW_UNROLL;
        const int64_t grid = (nvec + per_cta - 1) / per_cta;
        if (grid > 0x7fffffffLL) { set_error("activation: %lld elements exceed the grid range", (long long)n); return NB2_ERR_SHAPE; }
        act_vec_kernel<T, ACT, BWD><<<(unsigned)grid, EW_THREADS, 0, st>>>((const T*)x, (const T*)dy, (T*)out, nvec);
        done = nvec * EPV;
    }
    if (done < n) {
        const int64_t rest = n - done;
        int64_t grid = (rest + EW_THREADS - 1) / EW_THREADS;
        const int64_t cap = (int64_t)sm_count() * 8;
        if (grid > cap) grid = cap;
        act_scalar_kernel<T, ACT, BWD><<<(unsigned)grid, EW_THREADS, 0, st>>>((const T*)x, (const T*)dy, (T*)out, done, n);
    }
    return cuda_status(cudaGetLastError(), "activation launch");
}

template <typename T, bool BWD>
static int launch_act_a(const void* x, const void* dy, void* out, int64_t n, int act, cudaStream_t st) {
    switch (act) {
        case NB2_ACT_NONE: return launch_act_t<T, NB2_ACT_NONE, BWD>(x, dy, out, n, st);
        case NB2_ACT_GELU: return launch_act_t<T, NB2_ACT_GELU, BWD>(x, dy, out, n, st);
        case NB2_ACT_SILU: return launch_act_t<T, NB2_ACT_SILU, BWD>(x, dy, out, n, st);
        default: set_error("unknown activation %d", act); return NB2_ERR_DTYPE;
    }
}

int launch_act(const void* x, const void* dy, void* out, int64_t n, int dtype, int act, bool bwd, cudaStream_t st) {
    if (dtype == NB2_F32)
        return bwd ? launch_act_a<float, true>(x, dy, out, n, act, st) : launch_act_a<float, false>(x, dy, out, n, act, st);
    return bwd ? launch_act_a<__nv_bfloat16, true>(x, dy, out, n, act, st)
               : launch_act_a<__nv_bfloat16, false>(x, dy, out, n, act, st);
}

// ---------------------------------------------------------------- plain add
// out = a + b (fp32 add, rounded to T): the unfused form of the residual in front of a norm,
// used for shapes the fused residual kernels do not cover.  out may alias a or b.
template <typename T>
__global__ void __launch_bounds__(EW_THREADS)
add_kernel(const T* a, const T* b, T* out, int64_t n, bool vec) {
    constexpr int EPV = VecTraits<T>::EPV;
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, nth = (int64_t)gridDim.x * blockDim.x;
    int64_t done = 0;
    if (vec) {
        const int64_t nvec = n / EPV;
        for (int64_t i = tid; i < nvec; i += nth) {
            float fa[EPV], fb[EPV];
            unpack<T>(ld_stream(a + i * EPV), fa);
            unpack<T>(ld_stream(b + i * EPV), fb);
#pragma unroll
            for (int e = 0; e < EPV; ++e) fa[e] += fb[e];
            st_stream(out + i * EPV, pack<T>(fa));
        }
        done = nvec * EPV;
    }
    for (int64_t i = done + tid; i < n; i += nth) out[i] = from_f32<T>(to_f32(a[i]) + to_f32(b[i]));
}

int launch_add(const void* a, const void* b, void* out, int64_t n, int dtype, cudaStream_t st) {
    if (n == 0) return 0;
    const bool vec = aligned16(a) && aligned16(b) && aligned16(out);
    int64_t grid = (n / 4 + EW_THREADS - 1) / EW_THREADS + 1;
    const int64_t cap = (int64_t)sm_count() * 16;
    if (grid > cap) grid = cap;
    if (dtype == NB2_F32) add_kernel<float><<<(unsigned)grid, EW_THREADS, 0, st>>>((const float*)a, (const float*)b, (float*)out, n, vec);
    else add_kernel<__nv_bfloat16><<<(unsigned)grid, EW_THREADS, 0, st>>>((const __nv_bfloat16*)a, (const __nv_bfloat16*)b, (__nv_bfloat16*)out, n, vec);
    return cuda_status(cudaGetLastError(), "add launch");
}

// ------------------------------------------------------------------ SiLU gate
// Rows may be strided (the two halves of a [rows, 2H] SwiGLU input), so the
// kernel walks (row, column-vector): blockIdx.x picks GATE_ROWS consecutive
// rows, blockIdx.y * blockDim picks the column vector.  Each thread has
// GATE_ROWS x (2 or 3) independent 16-byte loads in flight.
constexpr int GATE_ROWS = 4;

template <typename T, bool BWD>
__global__ void __launch_bounds__(EW_THREADS)
silu_gate_vec_kernel(const T* __restrict__ a, int64_t lda, const T* __restrict__ b, int64_t ldb,
                     const T* __restrict__ dy, int64_t lddy,
                     T* __restrict__ o0, int64_t ldo0, T* __restrict__ o1, int64_t ldo1,
                     int64_t rows, int hv) {
    constexpr int EPV = VecTraits<T>::EPV;
    const int cv = blockIdx.y * EW_THREADS + threadIdx.x;
    if (cv >= hv) return;
    const int64_t r0 = (int64_t)blockIdx.x * GATE_ROWS;
    const int64_t c = (int64_t)cv * EPV;
    uint4 av[GATE_ROWS], bv[GATE_ROWS], dv[GATE_ROWS];
#pragma unroll
    for (int k = 0; k < GATE_ROWS; ++k) {
        const int64_t r = r0 + k;
        if (r < rows) {
            av[k] = ld_stream(a + r * lda + c);
            bv[k] = ld_stream(b + r * ldb + c);
            if (BWD) dv[k] = ld_stream(dy + r * lddy + c);
        }
    }
#pragma unroll
    for (int k = 0; k < GATE_ROWS; ++k) {
        const int64_t r = r0 + k;
        if (r < rows) {
            float fa[EPV], fb[EPV], fd[EPV], r0v[EPV], r1v[EPV];
            unpack<T>(av[k], fa);
            unpack<T>(bv[k], fb);
            if (BWD) unpack<T>(dv[k], fd);
#pragma unroll
            for (int e = 0; e < EPV; ++e) {
                const float s = fast_rcp(1.0f + fast_ex2(fa[e] * -1.44269504088896340736f));
                const float silu = fa[e] * s;
                if (BWD) {
                    r0v[e] = fd[e] * fb[e] * (s * fmaf(fa[e], 1.0f - s, 1.0f));   // da
                    r1v[e] = fd[e] * silu;                                         // db
                } else {
                    r0v[e] = silu * fb[e];
                }
            }
            st_stream(o0 + r * ldo0 + c, pack<T>(r0v));
            if (BWD) st_stream(o1 + r * ldo1 + c, pack<T>(r1v));
        }
    }
}

template <typename T, bool BWD>
__global__ void __launch_bounds__(EW_THREADS)
silu_gate_scalar_kernel(const T* __restrict__ a, int64_t lda, const T* __restrict__ b, int64_t ldb,
                        const T* __restrict__ dy, int64_t lddy,
                        T* __restrict__ o0, int64_t ldo0, T* __restrict__ o1, int64_t ldo1,
                        int64_t rows, int64_t H) {
    const int64_t total = rows * H;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / H, c = i - r * H;
        const float fa = to_f32(a[r * lda + c]), fb = to_f32(b[r * ldb + c]);
        const float s = fast_rcp(1.0f + fast_ex2(fa * -1.44269504088896340736f));
        if (BWD) {
            const float d = to_f32(dy[r * lddy + c]);
            o0[r * ldo0 + c] = from_f32<T>(d * fb * (s * fmaf(fa, 1.0f - s, 1.0f)));
            o1[r * ldo1 + c] = from_f32<T>(d * fa * s);
        } else {
            o0[r * ldo0 + c] = from_f32<T>(fa * s * fb);
        }
    }
}

template <typename T, bool BWD>
static int launch_gate_t(const void* a, int64_t lda, const void* b, int64_t ldb,
                         const void* dy, int64_t lddy, void* o0, int64_t ldo0, void* o1, int64_t ldo1,
                         int64_t rows, int64_t H, cudaStream_t st) {
    constexpr int EPV = VecTraits<T>::EPV;
    if (rows == 0 || H == 0) return 0;
    bool vec_ok = (H % EPV == 0) && (lda % EPV == 0) && (ldb % EPV == 0) && (ldo0 % EPV == 0) &&
                  aligned16(a) && aligned16(b) && aligned16(o0);
    if (BWD) vec_ok = vec_ok && (lddy % EPV == 0) && (ldo1 % EPV == 0) && aligned16(dy) && aligned16(o1);
    const int64_t row_blocks = (rows + GATE_ROWS - 1) / GATE_ROWS;
    const int64_t hv = H / EPV;
    const int64_t col_blocks = (hv + EW_THREADS - 1) / EW_THREADS;
    if (vec_ok && row_blocks <= 0x7fffffffLL && col_blocks <= 65535) {
        dim3 grid((unsigned)row_blocks, (unsigned)col_blocks);
        silu_gate_vec_kernel<T, BWD><<<grid, EW_THREADS, 0, st>>>(
            (const T*)a, lda, (const T*)b, ldb, (const T*)dy, lddy, (T*)o0, ldo0, (T*)o1, ldo1, rows, (int)hv);
    } else {
        int64_t grid = (rows * H + EW_THREADS - 1) / EW_THREADS;
        const int64_t cap = (int64_t)sm_count() * 8;
        if (grid > cap) grid = cap;
        silu_gate_scalar_kernel<T, BWD><<<(unsigned)grid, EW_THREADS, 0, st>>>(
            (const T*)a, lda, (const T*)b, ldb, (const T*)dy, lddy, (T*)o0, ldo0, (T*)o1, ldo1, rows, H);
    }
    return cuda_status(cudaGetLastError(), "silu gate launch");
}

int launch_silu_gate(const void* a, int64_t lda, const void* b, int64_t ldb,
                     const void* dy, int64_t lddy, void* o0, int64_t ldo0, void* o1, int64_t ldo1,
                     int64_t rows, int64_t H, int dtype, bool bwd, cudaStream_t st) {
    if (dtype == NB2_F32)
        return bwd ? launch_gate_t<float, true>(a, lda, b, ldb, dy, lddy, o0, ldo0, o1, ldo1, rows, H, st)
                   : launch_gate_t<float, false>(a, lda, b, ldb, dy, lddy, o0, ldo0, o1, ldo1, rows, H, st);
    return bwd ? launch_gate_t<__nv_bfloat16, true>(a, lda, b, ldb, dy, lddy, o0, ldo0, o1, ldo1, rows, H, st)
               : launch_gate_t<__nv_bfloat16, false>(a, lda, b, ldb, dy, lddy, o0, ldo0, o1, ldo1, rows, H, st);
}

}  // namespace nb2
