// Attention probabilities in one pass over the score matrix:
//   attn = softmax(scores * scale [key padding -> -inf] [+ additive mask] [causal -> -inf], last dim)
// which the reference's ScaledDotProductKernelImpl::forward (src/attention/details/kernel.hpp:33-92)
// forms as a division, two masked_fill, an add and a softmax, each a full read and write of
// [B, H, T, S].  Backward: dscores = scale * attn * (dattn - sum_j attn * dattn).
// Optionally the dropout that follows (kernel.hpp:94; the multiplicative-noise form of
// src/layer/details/dropout.hpp:32-51) rides in the same pass: out = attn * noise with a noise
// tensor the caller drew (a Bernoulli mask over 1-p, or N(1, sqrt(p/(1-p)))), so the random stream
// stays libtorch's; the backward takes the same noise.
//
// One row (b, h, t) per group of TPR threads, the whole row in registers (up to 4 x 16 bytes per
// thread), rows of a CTA independent of one another; persistent grid-stride over rows.  Rows whose
// length or alignment does not fit 16-byte vectors take a three-sweep kernel, one CTA per row.
#include <math.h>
#include <string.h>

#include <atomic>
#include <type_traits>

#include "launchers.h"

namespace nb2 {

namespace {

constexpr float kLog2e = 1.44269504088896340736f;

struct SoftmaxMask {
    const uint8_t* key_padding;   // [B, S], non-zero = masked, or NULL
    const void* add_mask;         // additive, element type of the scores, or NULL
    int64_t mask_sb, mask_sh;     // element strides of add_mask over batch and head (0 = broadcast); row stride S
    int causal;                   // column > row index t -> masked
    const void* noise = nullptr;  // [B, H, T, S] multiplicative dropout noise of the scores' type, or NULL
    void* pre_out = nullptr;      // with noise: where the probabilities before the noise go (the backward's input), or NULL
};

template <int TPR, bool MAX>
__device__ __forceinline__ float group_reduce(float v, float* red, int barrier_id) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float w = __shfl_xor_sync(0xffffffffu, v, o);
        v = MAX ? fmaxf(v, w) : v + w;
    }
    if constexpr (TPR > 32) {
        constexpr int WPR = TPR / 32;
        const int w = (threadIdx.x % TPR) >> 5;
        if ((threadIdx.x & 31) == 0) red[w] = v;
        named_barrier(barrier_id, TPR);
        float t = red[0];
#pragma unroll
        for (int i = 1; i < WPR; ++i) t = MAX ? fmaxf(t, red[i]) : t + red[i];
        v = t;
    }
    return v;
}

// Merge of (max, sum-of-exponentials) pairs in log2 units: x = max, y = sum relative to that max.
__device__ __forceinline__ float2 merge_pair(float2 a, float2 b) {
    const float m = fmaxf(a.x, b.x);
    // two empty sides (max -inf, sum 0) must merge to an empty pair, not to 2^(-inf + inf) = NaN
    const float ms = m == -INFINITY ? 0.f : m;
    return make_float2(m, a.y * fast_ex2(a.x - ms) + b.y * fast_ex2(b.x - ms));
}
template <int TPR>
__device__ __forceinline__ float2 merge_max_sum(float2 v, float2* red, int barrier_id) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float2 w;
        w.x = __shfl_xor_sync(0xffffffffu, v.x, o);
        w.y = __shfl_xor_sync(0xffffffffu, v.y, o);
        v = merge_pair(v, w);
    }
    if constexpr (TPR > 32) {
        constexpr int WPR = TPR / 32;
        const int w = (threadIdx.x % TPR) >> 5;
        if ((threadIdx.x & 31) == 0) red[w] = v;
        named_barrier(barrier_id, TPR);
        float2 t = red[0];
#pragma unroll
        for (int i = 1; i < WPR; ++i) t = merge_pair(t, red[i]);
        v = t;
    }
    return v;
}

// (batch, head, target position) of a row index, advanced by a fixed row stride without dividing:
// a 64-bit division per row and thread cost more than the row's arithmetic.
struct RowPos {
    int64_t b; int h, t;
    int64_t sb; int sh, st;       // the stride, decomposed the same way
    int H, Tq;
    __device__ __forceinline__ RowPos(int64_t row, int64_t stride, int64_t H_, int64_t Tq_) : H((int)H_), Tq((int)Tq_) {
        t = (int)(row % Tq_); const int64_t bh = row / Tq_; h = (int)(bh % H_); b = bh / H_;
        st = (int)(stride % Tq_); const int64_t sbh = stride / Tq_; sh = (int)(sbh % H_); sb = sbh / H_;
    }
    __device__ __forceinline__ void advance() {
        t += st; if (t >= Tq) { t -= Tq; ++h; }
        h += sh; if (h >= H) { h -= H; ++b; }
        if (h >= H) { h -= H; ++b; }
        b += sb;
    }
};

// Which row a group works on and which comes next.  RowOrderFlat: rows in memory order, a fixed stride apart.
// RowOrderHeadsInner: a group takes one (batch, target position) pair and walks its H heads before the next pair, so
// that an additive mask shared by the heads is fetched once per pair and kept on chip (read once per head it
// comes from L2 sixteen times at 16 heads, and that traffic, not DRAM, bounded the masked forward).
struct RowOrderFlat {
    int64_t row, rows, stride;
    RowPos pos;
    __device__ __forceinline__ RowOrderFlat(int64_t first, int64_t stride_, int64_t rows_, int64_t H, int64_t Tq)
        : row(first), rows(rows_), stride(stride_), pos(first, stride_, H, Tq) {}
    __device__ __forceinline__ bool valid() const { return row < rows; }
    __device__ __forceinline__ void advance() { row += stride; pos.advance(); }
    __device__ __forceinline__ int64_t b() const { return pos.b; }
    __device__ __forceinline__ int h() const { return pos.h; }
    __device__ __forceinline__ int t() const { return pos.t; }
    __device__ __forceinline__ bool new_mask_row() const { return true; }
};
struct RowOrderHeadsInner {
    int64_t row, pair, pairs, stride, b_;
    int h_, t_, H, Tq;
    __device__ __forceinline__ RowOrderHeadsInner(int64_t first, int64_t stride_, int64_t rows_, int64_t H_, int64_t Tq_)
        : pair(first), pairs(rows_ / H_), stride(stride_), h_(0), H((int)H_), Tq((int)Tq_) { place(); }
    __device__ __forceinline__ void place() { b_ = pair / Tq; t_ = (int)(pair - b_ * Tq); row = b_ * H * (int64_t)Tq + t_; }
    __device__ __forceinline__ bool valid() const { return pair < pairs; }
    __device__ __forceinline__ void advance() {
        if (++h_ == H) { h_ = 0; pair += stride; place(); }       // one 64-bit division per H rows
        else row += Tq;
    }
    __device__ __forceinline__ int64_t b() const { return b_; }
    __device__ __forceinline__ int h() const { return h_; }
    __device__ __forceinline__ int t() const { return t_; }
    __device__ __forceinline__ bool new_mask_row() const { return h_ == 0; }
};

// FLAGS: bit 0 key padding present, bit 1 additive mask present, bit 2 causal.  Compile-time, so
// that a call without masks spends nothing on them: with run-time tests the kernel executed 33
// instructions per score and was bound by issue (ncu: 71% issue slots busy, ALU pipe 60%).
constexpr int kSmPad = 1, kSmMask = 2, kSmCausal = 4, kSmNoise = 8;

// HIN: heads innermost (RowOrderHeadsInner); only with an additive mask whose head stride is 0.
template <typename T, int TPR, int VPT, int FLAGS, bool HIN>
__global__ void __launch_bounds__((TPR > 256 ? TPR : 256), (TPR > 256 ? 1 : 3))
softmax_fwd_kernel(const T* __restrict__ scores, const SoftmaxMask m, T* __restrict__ out,
                   int64_t rows, int64_t H, int64_t Tq, int S, float scale) {
    constexpr int EPV = VecTraits<T>::EPV;
    constexpr bool PAD = (FLAGS & kSmPad) != 0, MASK = (FLAGS & kSmMask) != 0, CAUSAL = (FLAGS & kSmCausal) != 0;
    constexpr bool NOISE = (FLAGS & kSmNoise) != 0;
    constexpr int THREADS = TPR > 256 ? TPR : 256;
    constexpr int RPC = THREADS / TPR;
    constexpr int WPR = (TPR + 31) / 32;
    __shared__ float red[2][RPC][2 * WPR];               // (max, sum) pairs, alternating by row parity
    const int grp = threadIdx.x / TPR, tr = threadIdx.x % TPR;
    const int nvec = S / EPV;
    int parity = 0;
    pdl_wait();
    const int64_t stride = (int64_t)gridDim.x * RPC;
    // The next row's scores are requested before the current row's arithmetic, so two rows per
    // group are in flight whatever the occupancy.  Under a causal mask the vectors that lie wholly
    // beyond the diagonal are not read at all.
    uint4 cur[VPT], nxt[VPT];
    auto load_row = [&](int64_t row, int t, uint4* raw) {
        const T* src = scores + row * (int64_t)S;
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const int c = tr + j * TPR;
            raw[j] = make_uint4(0u, 0u, 0u, 0u);
            if (c < nvec && !(CAUSAL && c * EPV > t)) raw[j] = ld_stream(src + (size_t)c * EPV);
        }
    };
    using Order = typename std::conditional<HIN, RowOrderHeadsInner, RowOrderFlat>::type;
    Order at((int64_t)blockIdx.x * RPC + grp, stride, rows, H, Tq);      // the row being worked on; `ahead` is the one requested
    // the pair's mask row, kept across its heads: every thread parks the vectors it will itself read back (no barrier
    // needed), in shared memory rather than registers so that the row costs no occupancy
    __shared__ uint4 mkeep[(MASK && HIN) ? VPT * THREADS : 1];
    if (at.valid()) load_row(at.row, at.t(), cur);
    while (at.valid()) {
        const int64_t row = at.row;
        const int t = at.t(), h = at.h();
        const int64_t b = at.b();
        const bool fetch_mask = at.new_mask_row();
        Order ahead = at;
        ahead.advance();
        if (ahead.valid()) load_row(ahead.row, ahead.t(), nxt);
        const T* mrow = MASK ? reinterpret_cast<const T*>(m.add_mask) + b * m.mask_sb + (HIN ? 0 : h * m.mask_sh) + t * (int64_t)S : nullptr;
        const uint8_t* prow = PAD ? m.key_padding + b * (int64_t)S : nullptr;
        if constexpr (MASK && HIN) {
            if (fetch_mask) {
#pragma unroll
                for (int j = 0; j < VPT; ++j) {
                    const int c = tr + j * TPR;
                    if (c < nvec && !(CAUSAL && c * EPV > t)) mkeep[j * THREADS + threadIdx.x] = ld_param(mrow + (size_t)c * EPV);
                }
            }
        }
        float v[VPT][EPV];
        float mx = -INFINITY;
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const int c = tr + j * TPR;
            // a vector past the row's end, or wholly beyond the diagonal, is all -inf and costs nothing more
            if (c < nvec && !(CAUSAL && c * EPV > t)) {
                unpack<T>(cur[j], v[j]);
                float mk[EPV];
                if constexpr (MASK && HIN) unpack<T>(mkeep[j * THREADS + threadIdx.x], mk);
                else if constexpr (MASK) unpack<T>(ld_param(mrow + (size_t)c * EPV), mk);
                uint8_t pad[EPV];
                if constexpr (PAD) {
                    if constexpr (EPV == 4) *reinterpret_cast<uint32_t*>(pad) = __ldg(reinterpret_cast<const uint32_t*>(prow + (size_t)c * EPV));
                    else *reinterpret_cast<uint2*>(pad) = __ldg(reinterpret_cast<const uint2*>(prow + (size_t)c * EPV));
                }
#pragma unroll
                for (int e = 0; e < EPV; ++e) {
                    float sc = v[j][e] * scale;
                    if constexpr (PAD) sc = pad[e] ? -INFINITY : sc;
                    if constexpr (MASK) sc += mk[e];
                    v[j][e] = sc;
                }
                if (CAUSAL && c * EPV + EPV - 1 > t) {        // the one vector that straddles the diagonal
#pragma unroll
                    for (int e = 0; e < EPV; ++e)
                        if (c * EPV + e > t) v[j][e] = -INFINITY;
                }
#pragma unroll
                for (int e = 0; e < EPV; ++e) mx = fmaxf(mx, v[j][e]);
            } else {
#pragma unroll
                for (int e = 0; e < EPV; ++e) v[j][e] = -INFINITY;
            }
        }
        // One reduction round: every thread exponentiates against its OWN maximum, and (max, sum)
        // pairs are merged (m = max(ma, mb), s = sa 2^(ma-m) + sb 2^(mb-m), in log2 units); the
        // thread's factor 2^(m_own - m) / s then rescales its exponentials.  A thread whose columns are
        // all masked uses 0 in place of its -inf maximum; a row with every column masked ends with
        // m = -inf and s = 0, the factor is inf and 0 * inf makes the whole row NaN, as in the reference.
        const float m_own = mx == -INFINITY ? 0.f : mx * kLog2e;
        float sum = 0.f;
#pragma unroll
        for (int j = 0; j < VPT; ++j)
#pragma unroll
            for (int e = 0; e < EPV; ++e) {
                const float p = fast_ex2(fmaf(v[j][e], kLog2e, -m_own));     // masked and out-of-range columns: 2^-inf = 0
                v[j][e] = p;
                sum += p;
            }
        float2 ms = make_float2(mx * kLog2e, sum);
        ms = merge_max_sum<TPR>(ms, reinterpret_cast<float2*>(red[parity][grp]), grp + 1);
        const float inv = fast_ex2(m_own - ms.x) / ms.y;
        T* dst = out + row * (int64_t)S;
        // the noise of this row is requested before the reduction's result is needed
        uint4 nz[NOISE ? VPT : 1];
        if constexpr (NOISE) {
#pragma unroll
            for (int j = 0; j < VPT; ++j) {
                const int c = tr + j * TPR;
                if (c < nvec) nz[j] = ld_stream(reinterpret_cast<const T*>(m.noise) + row * (int64_t)S + (size_t)c * EPV);
            }
        }
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const int c = tr + j * TPR;
            if (c < nvec) {
                float o[EPV];
#pragma unroll
                for (int e = 0; e < EPV; ++e) o[e] = v[j][e] * inv;
                if constexpr (NOISE) {
                    // the probabilities are a tensor of type T before the noise multiplies them (kernel.hpp:93-94)
                    const uint4 pre = pack<T>(o);
                    if (m.pre_out != nullptr) st_stream(reinterpret_cast<T*>(m.pre_out) + row * (int64_t)S + (size_t)c * EPV, pre);
                    float nv[EPV];
                    unpack<T>(pre, o);
                    unpack<T>(nz[j], nv);
#pragma unroll
                    for (int e = 0; e < EPV; ++e) o[e] *= nv[e];
                }
                st_stream(dst + (size_t)c * EPV, pack<T>(o));
            }
        }
#pragma unroll
        for (int j = 0; j < VPT; ++j) cur[j] = nxt[j];
        parity ^= 1;
        at = ahead;
    }
}

// NOISE: dattn is the gradient of (attn * noise); the gradient reaching attn is dattn * noise, a tensor of
// type T in the reference's autograd (rounded before the softmax backward uses it).
template <typename T, int TPR, int VPT, bool NOISE>
__global__ void __launch_bounds__((TPR > 256 ? TPR : 256), (TPR > 256 ? 1 : 2))
softmax_bwd_kernel(const T* __restrict__ attn, const T* __restrict__ dattn, const T* __restrict__ noise,
                   T* __restrict__ dscores, int64_t rows, int S, float scale) {
    constexpr int EPV = VecTraits<T>::EPV;
    constexpr int THREADS = TPR > 256 ? TPR : 256;
    constexpr int RPC = THREADS / TPR;
    constexpr int WPR = (TPR + 31) / 32;
    __shared__ float red_a[2][RPC][WPR];
    const int grp = threadIdx.x / TPR, tr = threadIdx.x % TPR;
    const int nvec = S / EPV;
    pdl_wait();
    int parity = 0;
    const int64_t stride = (int64_t)gridDim.x * RPC;
    uint4 cy[VPT], cd[VPT], ny[VPT], nd[VPT];           // this row and the next, requested one row ahead
    uint4 cn[NOISE ? VPT : 1], nn[NOISE ? VPT : 1];
    auto load_row = [&](int64_t row, uint4* ry, uint4* rd, uint4* rn) {
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const int c = tr + j * TPR;
            if (c < nvec) {
                ry[j] = ld_stream(attn + row * (int64_t)S + (size_t)c * EPV);
                rd[j] = ld_stream(dattn + row * (int64_t)S + (size_t)c * EPV);
                if constexpr (NOISE) rn[j] = ld_stream(noise + row * (int64_t)S + (size_t)c * EPV);
            }
        }
    };
    int64_t row = (int64_t)blockIdx.x * RPC + grp;
    if (row < rows) load_row(row, cy, cd, cn);
    for (; row < rows; row += stride, parity ^= 1) {
        if (row + stride < rows) load_row(row + stride, ny, nd, nn);
        // The row stays in its packed form across the reduction and is unpacked again afterwards: for bf16 the
        // fp32 copies of both tensors (64 registers) next to two rows of three packed streams spilled.
        float dot = 0.f;
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const int c = tr + j * TPR;
            if (c < nvec) {
                float y[EPV], d[EPV];
                unpack<T>(cy[j], y);
                unpack<T>(cd[j], d);
                if constexpr (NOISE) {
                    float nv[EPV];
                    unpack<T>(cn[j], nv);
#pragma unroll
                    for (int e = 0; e < EPV; ++e) d[e] = __fmul_rn(d[e], nv[e]);   // rounded as a product: never fused into the subtraction below
                    cd[j] = pack<T>(d);                          // the gradient of attn as a tensor of type T
                    unpack<T>(cd[j], d);
                }
#pragma unroll
                for (int e = 0; e < EPV; ++e) dot = fmaf(y[e], d[e], dot);
            }
        }
        dot = group_reduce<TPR, false>(dot, red_a[parity][grp], grp + 1);
        T* dst = dscores + row * (int64_t)S;
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const int c = tr + j * TPR;
            if (c < nvec) {
                float y[EPV], d[EPV], o[EPV];
                unpack<T>(cy[j], y);
                unpack<T>(cd[j], d);
#pragma unroll
                for (int e = 0; e < EPV; ++e) o[e] = scale * (y[e] * (d[e] - dot));
                st_stream(dst + (size_t)c * EPV, pack<T>(o));
            }
        }
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            cy[j] = ny[j]; cd[j] = nd[j];
            if constexpr (NOISE) cn[j] = nn[j];
        }
    }
}

// ---- any row length and alignment: one CTA per row, three sweeps over the row
__device__ __forceinline__ float cta_reduce(float v, float* red, bool is_max) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float w = __shfl_xor_sync(0xffffffffu, v, o);
        v = is_max ? fmaxf(v, w) : v + w;
    }
    __syncthreads();                               // red may still be read from the previous use
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = red[0];
    for (int i = 1; i < (int)(blockDim.x >> 5); ++i) t = is_max ? fmaxf(t, red[i]) : t + red[i];
    return t;
}

template <typename T>
__device__ __forceinline__ float masked_score(const T* src, const T* mrow, const uint8_t* prow, int causal, int64_t t, int64_t c, float scale) {
    float s = to_f32(src[c]) * scale;
    if (prow != nullptr && prow[c]) s = -INFINITY;
    if (mrow != nullptr) s += to_f32(mrow[c]);
    if (causal && c > t) s = -INFINITY;
    return s;
}

template <typename T>
__global__ void __launch_bounds__(256)
softmax_fwd_generic(const T* __restrict__ scores, const SoftmaxMask m, T* __restrict__ out,
                    int64_t rows, int64_t H, int64_t Tq, int64_t S, float scale) {
    __shared__ float red[8];
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const int64_t t = row % Tq, bh = row / Tq, h = bh % H, b = bh / H;
        const T* src = scores + row * S;
        const T* mrow = m.add_mask ? reinterpret_cast<const T*>(m.add_mask) + b * m.mask_sb + h * m.mask_sh + t * S : nullptr;
        const uint8_t* prow = m.key_padding ? m.key_padding + b * S : nullptr;
        float mx = -INFINITY;
        for (int64_t c = threadIdx.x; c < S; c += blockDim.x) mx = fmaxf(mx, masked_score(src, mrow, prow, m.causal, t, c, scale));
        mx = cta_reduce(mx, red, true);
        const float off = -mx * kLog2e;
        float sum = 0.f;
        for (int64_t c = threadIdx.x; c < S; c += blockDim.x) sum += fast_ex2(fmaf(masked_score(src, mrow, prow, m.causal, t, c, scale), kLog2e, off));
        sum = cta_reduce(sum, red, false);
        const float inv = 1.0f / sum;
        for (int64_t c = threadIdx.x; c < S; c += blockDim.x) {
            T p = from_f32<T>(fast_ex2(fmaf(masked_score(src, mrow, prow, m.causal, t, c, scale), kLog2e, off)) * inv);
            if (m.noise != nullptr) {
                if (m.pre_out != nullptr) reinterpret_cast<T*>(m.pre_out)[row * S + c] = p;
                p = from_f32<T>(to_f32(p) * to_f32(reinterpret_cast<const T*>(m.noise)[row * S + c]));
            }
            out[row * S + c] = p;
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
softmax_bwd_generic(const T* __restrict__ attn, const T* __restrict__ dattn, const T* __restrict__ noise,
                    T* __restrict__ dscores, int64_t rows, int64_t S, float scale) {
    __shared__ float red[8];
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const T* ya = attn + row * S;
        const T* da = dattn + row * S;
        const T* nz = noise ? noise + row * S : nullptr;
        auto grad = [&](int64_t c) { return nz ? to_f32(from_f32<T>(__fmul_rn(to_f32(da[c]), to_f32(nz[c])))) : to_f32(da[c]); };
        float dot = 0.f;
        for (int64_t c = threadIdx.x; c < S; c += blockDim.x) dot = fmaf(to_f32(ya[c]), grad(c), dot);
        dot = cta_reduce(dot, red, false);
        for (int64_t c = threadIdx.x; c < S; c += blockDim.x)
            dscores[row * S + c] = from_f32<T>(scale * (to_f32(ya[c]) * (grad(c) - dot)));
    }
}

// 4 vectors per thread in both directions and types.  Measured for the bf16 forward: 2 vectors per
// thread (no spills at the three-CTA register budget, but half the bytes in flight per thread and
// twice the threads per row) ran at 0.56 of the copy rate against 0.69 with 4.
template <typename T> constexpr int fwd_vpt() { return 4; }
int pick_softmax_tpr(int64_t nvec, int vpt = 4) {
    for (int tpr = 32; tpr <= 512; tpr *= 2)
        if (nvec <= (int64_t)tpr * vpt) return tpr;
    return 0;
}

int64_t row_grid(int64_t rows, int tpr) {
    const int threads = tpr > 256 ? tpr : 256;
    const int rpc = threads / tpr;
    const int64_t need = (rows + rpc - 1) / rpc;
    const int64_t cap = (int64_t)sm_count() * (tpr > 256 ? 1 : 3) * 4;      // a few CTAs per slot: rows are short-lived
    return need < cap ? (need < 1 ? 1 : need) : cap;
}

// Heads innermost pays when the same mask row serves several heads; NB2_SOFTMAX_ORDER=flat switches it off for measurements.
// It needs enough (batch, position) pairs to give every row group of a full grid several of them: with few pairs the
// heads of one pair would run one after the other in a single group while most of the GPU idles.
// Order override: 0 = by size, 1 = always memory order, 2 = heads innermost whenever the mask allows it.
std::atomic<int> g_softmax_order{-1};
int softmax_order() {
    int v = g_softmax_order.load(std::memory_order_relaxed);
    if (v < 0) {
        const char* e = getenv("NB2_SOFTMAX_ORDER");
        v = (e != nullptr && strcmp(e, "flat") == 0) ? 1 : (e != nullptr && strcmp(e, "inner") == 0) ? 2 : 0;
        g_softmax_order.store(v, std::memory_order_relaxed);
    }
    return v;
}
bool heads_inner_wanted(const SoftmaxMask& m, int64_t H, int64_t pairs, int groups_per_cta) {
    const int order = softmax_order();
    if (order == 1 || m.add_mask == nullptr || m.mask_sh != 0 || H < 2) return false;
    return order == 2 || (H >= 4 && pairs >= (int64_t)sm_count() * 3 * groups_per_cta * 2);
}

template <typename T, int TPR, int FLAGS>
int launch_fwd_flags(const void* scores, const SoftmaxMask& m, void* out, int64_t rows, int64_t H, int64_t Tq, int64_t S,
                     float scale, cudaStream_t st) {
    constexpr int THREADS = TPR > 256 ? TPR : 256;
    if constexpr ((FLAGS & kSmMask) != 0 && TPR <= 256) {
        constexpr int RPC = THREADS / TPR;
        const int64_t pairs = rows / H;
        if (heads_inner_wanted(m, H, pairs, RPC)) {
            const int64_t need = (pairs + RPC - 1) / RPC, cap = (int64_t)sm_count() * 3 * 4;
            return cuda_status(launch_pdl(softmax_fwd_kernel<T, TPR, fwd_vpt<T>(), FLAGS, true>, dim3((unsigned)(need < cap ? need : cap)),
                                          dim3(THREADS), 0, st, (const T*)scores, m, (T*)out, rows, H, Tq, (int)S, scale),
                               "softmax_fwd_kernel launch");
        }
    }
    return cuda_status(launch_pdl(softmax_fwd_kernel<T, TPR, fwd_vpt<T>(), FLAGS, false>, dim3((unsigned)row_grid(rows, TPR)), dim3(THREADS), 0, st,
                                  (const T*)scores, m, (T*)out, rows, H, Tq, (int)S, scale),
                       "softmax_fwd_kernel launch");
}
template <typename T, int TPR>
int launch_fwd_tpr(const void* scores, const SoftmaxMask& m, void* out, int64_t rows, int64_t H, int64_t Tq, int64_t S,
                   float scale, cudaStream_t st) {
    const int flags = (m.key_padding ? kSmPad : 0) | (m.add_mask ? kSmMask : 0) | (m.causal ? kSmCausal : 0) | (m.noise ? kSmNoise : 0);
    switch (flags) {
        case 0: return launch_fwd_flags<T, TPR, 0>(scores, m, out, rows, H, Tq, S, scale, st);
        case 1: return launch_fwd_flags<T, TPR, 1>(scores, m, out, rows, H, Tq, S, scale, st);
        case 2: return launch_fwd_flags<T, TPR, 2>(scores, m, out, rows, H, Tq, S, scale, st);
        case 3: return launch_fwd_flags<T, TPR, 3>(scores, m, out, rows, H, Tq, S, scale, st);
        case 4: return launch_fwd_flags<T, TPR, 4>(scores, m, out, rows, H, Tq, S, scale, st);
        case 5: return launch_fwd_flags<T, TPR, 5>(scores, m, out, rows, H, Tq, S, scale, st);
        case 6: return launch_fwd_flags<T, TPR, 6>(scores, m, out, rows, H, Tq, S, scale, st);
        case 7: return launch_fwd_flags<T, TPR, 7>(scores, m, out, rows, H, Tq, S, scale, st);
        case 8: return launch_fwd_flags<T, TPR, 8>(scores, m, out, rows, H, Tq, S, scale, st);
        case 9: return launch_fwd_flags<T, TPR, 9>(scores, m, out, rows, H, Tq, S, scale, st);
        case 10: return launch_fwd_flags<T, TPR, 10>(scores, m, out, rows, H, Tq, S, scale, st);
        case 11: return launch_fwd_flags<T, TPR, 11>(scores, m, out, rows, H, Tq, S, scale, st);
        case 12: return launch_fwd_flags<T, TPR, 12>(scores, m, out, rows, H, Tq, S, scale, st);
        case 13: return launch_fwd_flags<T, TPR, 13>(scores, m, out, rows, H, Tq, S, scale, st);
        case 14: return launch_fwd_flags<T, TPR, 14>(scores, m, out, rows, H, Tq, S, scale, st);
        default: return launch_fwd_flags<T, TPR, 15>(scores, m, out, rows, H, Tq, S, scale, st);
    }
}
template <typename T, int TPR>
int launch_bwd_tpr(const void* attn, const void* dattn, const void* noise, void* dscores, int64_t rows, int64_t S, float scale,
                   cudaStream_t st) {
    constexpr int THREADS = TPR > 256 ? TPR : 256;
    if (noise != nullptr)
        return cuda_status(launch_pdl(softmax_bwd_kernel<T, TPR, 4, true>, dim3((unsigned)row_grid(rows, TPR)), dim3(THREADS), 0, st,
                                      (const T*)attn, (const T*)dattn, (const T*)noise, (T*)dscores, rows, (int)S, scale),
                           "softmax_bwd_kernel launch");
    return cuda_status(launch_pdl(softmax_bwd_kernel<T, TPR, 4, false>, dim3((unsigned)row_grid(rows, TPR)), dim3(THREADS), 0, st,
                                  (const T*)attn, (const T*)dattn, (const T*)nullptr, (T*)dscores, rows, (int)S, scale),
                       "softmax_bwd_kernel launch");
}

template <typename T>
int launch_fwd_t(const void* scores, const SoftmaxMask& m, void* out, int64_t B, int64_t H, int64_t Tq, int64_t S, float scale,
                 cudaStream_t st) {
    constexpr int EPV = VecTraits<T>::EPV;
    const int64_t rows = B * H * Tq;
    const bool mask_ok = m.add_mask == nullptr || (aligned16(m.add_mask) && m.mask_sb % EPV == 0 && m.mask_sh % EPV == 0);
    const bool pad_ok = m.key_padding == nullptr || (reinterpret_cast<uintptr_t>(m.key_padding) % EPV == 0);
    const bool noise_ok = m.noise == nullptr || (aligned16(m.noise) && (m.pre_out == nullptr || aligned16(m.pre_out)));
    const int tpr = (S % EPV == 0 && aligned16(scores) && aligned16(out) && mask_ok && pad_ok && noise_ok) ? pick_softmax_tpr(S / EPV, fwd_vpt<T>()) : 0;
    switch (tpr) {
        case 32:  return launch_fwd_tpr<T, 32>(scores, m, out, rows, H, Tq, S, scale, st);
        case 64:  return launch_fwd_tpr<T, 64>(scores, m, out, rows, H, Tq, S, scale, st);
        case 128: return launch_fwd_tpr<T, 128>(scores, m, out, rows, H, Tq, S, scale, st);
        case 256: return launch_fwd_tpr<T, 256>(scores, m, out, rows, H, Tq, S, scale, st);
        case 512: return launch_fwd_tpr<T, 512>(scores, m, out, rows, H, Tq, S, scale, st);
        default: break;
    }
    const int64_t cap = (int64_t)sm_count() * 8;
    softmax_fwd_generic<T><<<(unsigned)(rows < cap ? rows : cap), 256, 0, st>>>((const T*)scores, m, (T*)out, rows, H, Tq, S, scale);
    return cuda_status(cudaGetLastError(), "softmax_fwd_generic launch");
}

template <typename T>
int launch_bwd_t(const void* attn, const void* dattn, const void* noise, void* dscores, int64_t rows, int64_t S, float scale,
                 cudaStream_t st) {
    constexpr int EPV = VecTraits<T>::EPV;
    const int tpr = (S % EPV == 0 && aligned16(attn) && aligned16(dattn) && aligned16(dscores) && (noise == nullptr || aligned16(noise)))
                        ? pick_softmax_tpr(S / EPV) : 0;
    switch (tpr) {
        case 32:  return launch_bwd_tpr<T, 32>(attn, dattn, noise, dscores, rows, S, scale, st);
        case 64:  return launch_bwd_tpr<T, 64>(attn, dattn, noise, dscores, rows, S, scale, st);
        case 128: return launch_bwd_tpr<T, 128>(attn, dattn, noise, dscores, rows, S, scale, st);
        case 256: return launch_bwd_tpr<T, 256>(attn, dattn, noise, dscores, rows, S, scale, st);
        case 512: return launch_bwd_tpr<T, 512>(attn, dattn, noise, dscores, rows, S, scale, st);
        default: break;
    }
    const int64_t cap = (int64_t)sm_count() * 8;
    softmax_bwd_generic<T><<<(unsigned)(rows < cap ? rows : cap), 256, 0, st>>>((const T*)attn, (const T*)dattn, (const T*)noise, (T*)dscores, rows, S, scale);
    return cuda_status(cudaGetLastError(), "softmax_bwd_generic launch");
}

}  // namespace

int set_softmax_order(int order) {
    if (order < 0 || order > 2) return -1;
    const int before = softmax_order();
    g_softmax_order.store(order, std::memory_order_relaxed);
    return before;
}

int launch_attention_softmax_fwd(const void* scores, const uint8_t* key_padding, const void* add_mask, int64_t mask_sb,
                                 int64_t mask_sh, void* out, int64_t B, int64_t H, int64_t Tq, int64_t S, float scale,
                                 int causal, int dtype, cudaStream_t st, const void* noise, void* pre_out) {
    SoftmaxMask m = {key_padding, add_mask, mask_sb, mask_sh, causal};
    m.noise = noise;
    m.pre_out = pre_out;
    return dtype == NB2_F32 ? launch_fwd_t<float>(scores, m, out, B, H, Tq, S, scale, st)
                            : launch_fwd_t<__nv_bfloat16>(scores, m, out, B, H, Tq, S, scale, st);
}

int launch_attention_softmax_bwd(const void* attn, const void* dattn, void* dscores, int64_t rows, int64_t S, float scale,
                                 int dtype, cudaStream_t st, const void* noise) {
    return dtype == NB2_F32 ? launch_bwd_t<float>(attn, dattn, noise, dscores, rows, S, scale, st)
                            : launch_bwd_t<__nv_bfloat16>(attn, dattn, noise, dscores, rows, S, scale, st);
}

}  // namespace nb2
