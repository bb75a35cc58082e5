// BERT's embedding front end in one pass: word + position + token-type rows summed and
// LayerNorm'ed per token.
//
// Reference: BertEmbeddingImpl::forward (src/block/details/transformers/bert.hpp:155-194):
//   embeddings = word_embeddings(ids)                         (:162-163, ids int64 [B, S])
//   embeddings += position_embeddings(arange(S) per batch)    (:176-181)
//   embeddings += token_type_embeddings(zeros)                (:183-187: always row 0)
//   embeddings  = layer_norm(embeddings)  eps = 1e-12         (:143-146, :189)
// which libtorch runs as three gathers, two adds and a LayerNorm: 6 passes over [B*S, D].
// Here: one gather-read of the word row per token (the position rows are shared by the batch
// and stay in L2, the type row in L1), one write of the output, optionally one of the sum
// (the backward's LayerNorm input).
#include "launchers.h"
#include "norm_kernels.cuh"

namespace nb2 {

// ids == NULL: `word` already holds one row per token (ready-made embeddings, bert.hpp:164-171)
template <typename I> __device__ __forceinline__ int64_t load_token(const void* ids, int64_t t) {
    return ids == nullptr ? t : (int64_t)reinterpret_cast<const I*>(ids)[t];
}

template <typename T, typename I, int TPR, int VPT>
__global__ void __launch_bounds__((TPR > 256 ? TPR : 256), (TPR > 256 ? 1 : 2))
bert_embed_ln_fwd_kernel(const T* __restrict__ word, const T* __restrict__ pos, const T* __restrict__ type,
                         const void* __restrict__ ids, const T* __restrict__ gamma, const T* __restrict__ beta,
                         T* __restrict__ sum_out, T* __restrict__ y, float* __restrict__ mean_out,
                         float* __restrict__ rstd_out, int64_t tokens, int64_t S, int64_t vocab, int D, float eps,
                         int64_t* __restrict__ status) {
    constexpr int EPV = VecTraits<T>::EPV;
    constexpr int THREADS = (TPR > 256 ? TPR : 256);
    constexpr int RPC = THREADS / TPR;
    constexpr int WPR = (TPR + 31) / 32;
    __shared__ float red_a[RPC][WPR], red_b[RPC][WPR];
    const int nvec = D / EPV;
    const int slot = threadIdx.x / TPR, tr = threadIdx.x % TPR;
    const float inv_d = 1.0f / (float)D;
    pdl_release();
    pdl_wait();

    uint4 gpk[VPT], bpk[VPT], tpk[VPT];
    bool valid[VPT];
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        valid[j] = (tr + j * TPR) < nvec;
        if (valid[j]) {
            gpk[j] = ld_param(gamma + (size_t)(tr + j * TPR) * EPV);
            bpk[j] = ld_param(beta + (size_t)(tr + j * TPR) * EPV);
            if (type != nullptr) tpk[j] = ld_param(type + (size_t)(tr + j * TPR) * EPV);     // row 0
        }
    }
    // Software pipeline over this slot's tokens: the id is read two tokens ahead and the word and
    // position rows one token ahead, so neither the id -> row dependency nor the row's HBM latency
    // sits in front of a token's arithmetic.
    const int64_t stride = (int64_t)gridDim.x * RPC;
    int64_t t = (int64_t)blockIdx.x * RPC + slot;
    int64_t id_cur = t < tokens ? load_token<I>(ids, t) : 0;
    int64_t id_nxt = t + stride < tokens ? load_token<I>(ids, t + stride) : 0;
    uint4 wcur[VPT], pcur[VPT];
    auto fetch = [&](int64_t tok, int64_t id, uint4* w, uint4* p) {
        const bool ok = id >= 0 && id < vocab;
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            if (valid[j]) {
                const size_t off = (size_t)(tr + j * TPR) * EPV;
                w[j] = ok ? __ldg(reinterpret_cast<const uint4*>(word + id * (int64_t)D + off)) : make_uint4(0u, 0u, 0u, 0u);
                if (pos != nullptr) p[j] = __ldg(reinterpret_cast<const uint4*>(pos + (tok % S) * (int64_t)D + off));
            }
        }
    };
    if (t < tokens) fetch(t, id_cur, wcur, pcur);
    for (; t < tokens; t += stride) {
        const int64_t id = id_cur;
        const bool ok = id >= 0 && id < vocab;
        if (!ok && tr == 0 && status != nullptr) { status[0] = 1; status[1] = t; }
        uint4 wnxt[VPT], pnxt[VPT];
        const int64_t id_after = t + 2 * stride < tokens ? load_token<I>(ids, t + 2 * stride) : 0;
        if (t + stride < tokens) fetch(t + stride, id_nxt, wnxt, pnxt);
        float v[VPT][EPV];
        float sum = 0.f;
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            if (valid[j]) {
                const size_t off = (size_t)(tr + j * TPR) * EPV;
                unpack<T>(wcur[j], v[j]);                      // zeros for an id outside the table
                float a[EPV];
                if (pos != nullptr) {
                    unpack<T>(pcur[j], a);
#pragma unroll
                    for (int e = 0; e < EPV; ++e) v[j][e] += a[e];
                }
                if (type != nullptr) {
                    unpack<T>(tpk[j], a);
#pragma unroll
                    for (int e = 0; e < EPV; ++e) v[j][e] += a[e];
                }
                const uint4 packed = pack<T>(v[j]);                       // the sum as a tensor of dtype T
                if (sum_out != nullptr) st_stream(sum_out + t * (int64_t)D + off, packed);
                unpack<T>(packed, v[j]);
#pragma unroll
                for (int e = 0; e < EPV; ++e) sum += v[j][e];
            }
        }
#pragma unroll
        for (int j = 0; j < VPT; ++j) { wcur[j] = wnxt[j]; pcur[j] = pnxt[j]; }
        id_cur = id_nxt;
        id_nxt = id_after;
        const float mu = row_sum<TPR>(sum, red_a[slot], slot + 1) * inv_d;
        float q = 0.f;
#pragma unroll
        for (int j = 0; j < VPT; ++j)
            if (valid[j]) {
#pragma unroll
                for (int e = 0; e < EPV; ++e) { v[j][e] -= mu; q = fmaf(v[j][e], v[j][e], q); }
            }
        const float rs = rsqrtf(row_sum<TPR>(q, red_b[slot], slot + 1) * inv_d + eps);
        if (tr == 0) {
            if (mean_out != nullptr) mean_out[t] = mu;
            if (rstd_out != nullptr) rstd_out[t] = rs;
        }
#pragma unroll
        for (int j = 0; j < VPT; ++j)
            if (valid[j]) {
                float g[EPV], b[EPV], o[EPV];
                unpack<T>(gpk[j], g);
                unpack<T>(bpk[j], b);
#pragma unroll
                for (int e = 0; e < EPV; ++e) o[e] = fmaf(v[j][e] * rs, g[e], b[e]);
                st_stream(y + t * (int64_t)D + (size_t)(tr + j * TPR) * EPV, pack<T>(o));
            }
    }
}

// any width / alignment: one warp per token, scalar
template <typename T, typename I>
__global__ void __launch_bounds__(256)
bert_embed_ln_fwd_generic(const T* __restrict__ word, const T* __restrict__ pos, const T* __restrict__ type,
                          const void* __restrict__ ids, const T* __restrict__ gamma, const T* __restrict__ beta,
                          T* __restrict__ sum_out, T* __restrict__ y, float* __restrict__ mean_out,
                          float* __restrict__ rstd_out, int64_t tokens, int64_t S, int64_t vocab, int64_t D, float eps,
                          int64_t* __restrict__ status) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int64_t nwarps = (int64_t)gridDim.x * (blockDim.x >> 5);
    const float inv_d = 1.0f / (float)D;
    for (int64_t t = warp; t < tokens; t += nwarps) {
        const int64_t id = load_token<I>(ids, t);
        const bool ok = id >= 0 && id < vocab;
        if (!ok && lane == 0 && status != nullptr) { status[0] = 1; status[1] = t; }
        auto value = [&](int64_t c) {
            float v = ok ? to_f32(word[id * D + c]) : 0.f;
            if (pos != nullptr) v += to_f32(pos[(t % S) * D + c]);
            if (type != nullptr) v += to_f32(type[c]);
            return to_f32(from_f32<T>(v));
        };
        float s = 0.f;
        for (int64_t c = lane; c < D; c += 32) s += value(c);
        const float mu = warp_sum(s) * inv_d;
        float q = 0.f;
        for (int64_t c = lane; c < D; c += 32) { const float d = value(c) - mu; q = fmaf(d, d, q); }
        const float rs = rsqrtf(warp_sum(q) * inv_d + eps);
        if (lane == 0) {
            if (mean_out != nullptr) mean_out[t] = mu;
            if (rstd_out != nullptr) rstd_out[t] = rs;
        }
        for (int64_t c = lane; c < D; c += 32) {
            const float v = value(c);
            if (sum_out != nullptr) sum_out[t * D + c] = from_f32<T>(v);
            y[t * D + c] = from_f32<T>(fmaf((v - mu) * rs, to_f32(gamma[c]), to_f32(beta[c])));
        }
    }
}

// dpos[s, :] = sum_b dsum[b, s, :]  (fp32 accumulation, rounded once); the unrounded sums also go
// to `acc_out` ([S, D] fp32) when the token-type gradient (their sum over s) is wanted, so dsum is
// read once for both.
template <typename T>
__global__ void __launch_bounds__(256)
batch_sum_kernel(const T* __restrict__ dsum, T* __restrict__ dpos, float* __restrict__ acc_out, int64_t B, int64_t S, int64_t D) {
    const int64_t total = S * D;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        float acc = 0.f;
#pragma unroll 4
        for (int64_t b = 0; b < B; ++b) acc += to_f32(dsum[b * total + i]);
        if (dpos != nullptr) dpos[i] = from_f32<T>(acc);
        if (acc_out != nullptr) acc_out[i] = acc;
    }
}
// the same sum, one 16-byte vector of the [S, D] plane per thread and 16 batch rows in flight
template <typename T>
__global__ void __launch_bounds__(128)
batch_sum_vec_kernel(const T* __restrict__ dsum, T* __restrict__ dpos, float* __restrict__ acc_out, int64_t B, int64_t nvec_plane) {
    constexpr int EPV = VecTraits<T>::EPV;
    constexpr int U = 16;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec_plane; i += (int64_t)gridDim.x * blockDim.x) {
        float acc[EPV];
#pragma unroll
        for (int e = 0; e < EPV; ++e) acc[e] = 0.f;
        const T* src = dsum + i * EPV;
        for (int64_t b0 = 0; b0 < B; b0 += U) {
            uint4 r[U];
#pragma unroll
            for (int u = 0; u < U; ++u)
                if (b0 + u < B) r[u] = ld_stream(src + (b0 + u) * nvec_plane * EPV);
#pragma unroll
            for (int u = 0; u < U; ++u) {
                if (b0 + u < B) {
                    float f[EPV];
                    unpack<T>(r[u], f);
#pragma unroll
                    for (int e = 0; e < EPV; ++e) acc[e] += f[e];
                }
            }
        }
        if (dpos != nullptr) st_stream(dpos + i * EPV, pack<T>(acc));
        if (acc_out != nullptr) {
#pragma unroll
            for (int e = 0; e < EPV; e += 4)
                *reinterpret_cast<float4*>(acc_out + i * EPV + e) = make_float4(acc[e], acc[e + 1], acc[e + 2], acc[e + 3]);
        }
    }
}
__global__ void __launch_bounds__(256)
cast_row_kernel(const float* __restrict__ src, void* __restrict__ dst, int64_t n, int bf16) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    if (bf16) reinterpret_cast<__nv_bfloat16*>(dst)[i] = __float2bfloat16_rn(src[i]);
    else reinterpret_cast<float*>(dst)[i] = src[i];
}

template <typename T, typename I>
static int launch_fwd_ti(const void* word, const void* pos, const void* type, const void* ids, const void* gamma,
                         const void* beta, void* sum_out, void* y, float* mean, float* rstd, int64_t tokens, int64_t S,
                         int64_t vocab, int64_t D, float eps, int64_t* status, cudaStream_t st) {
    constexpr int EPV = VecTraits<T>::EPV;
    const bool aligned = aligned16(word) && aligned16(y) && aligned16(gamma) && aligned16(beta) &&
                         (pos == nullptr || aligned16(pos)) && (type == nullptr || aligned16(type)) &&
                         (sum_out == nullptr || aligned16(sum_out));
    constexpr int VPT = 16 / EPV;                     // 16 elements per thread and token for either type
    const int tpr = (D % EPV == 0 && aligned) ? pick_tpr(D / EPV, VPT) : 0;
    const int sms = sm_count();
#define NB2_BERT_LAUNCH(TPR_)                                                                                     \
    {                                                                                                             \
        constexpr int THREADS = (TPR_ > 256 ? TPR_ : 256);                                                        \
        constexpr int RPC = THREADS / TPR_;                                                                        \
        int64_t need = (tokens + RPC - 1) / RPC, cap = (int64_t)sms * (TPR_ > 256 ? 1 : 2);                       \
        const cudaError_t e = launch_pdl(bert_embed_ln_fwd_kernel<T, I, TPR_, VPT>, dim3((unsigned)(need < cap ? need : cap)), \
                                         dim3(THREADS), 0, st, (const T*)word, (const T*)pos, (const T*)type, ids, \
                                         (const T*)gamma, (const T*)beta, (T*)sum_out, (T*)y, mean, rstd, tokens, S, \
                                         vocab, (int)D, eps, status);                                             \
        return cuda_status(e, "bert embedding + layernorm launch");                                               \
    }
    switch (tpr) {
        case 32: NB2_BERT_LAUNCH(32)
        case 64: NB2_BERT_LAUNCH(64)
        case 128: NB2_BERT_LAUNCH(128)
        case 256: NB2_BERT_LAUNCH(256)
        case 512: NB2_BERT_LAUNCH(512)
        default: break;
    }
#undef NB2_BERT_LAUNCH
    int64_t need = (tokens + 7) / 8, cap = (int64_t)sms * 8;
    bert_embed_ln_fwd_generic<T, I><<<(unsigned)(need < cap ? need : cap), 256, 0, st>>>(
        (const T*)word, (const T*)pos, (const T*)type, ids, (const T*)gamma, (const T*)beta, (T*)sum_out, (T*)y, mean,
        rstd, tokens, S, vocab, D, eps, status);
    return cuda_status(cudaGetLastError(), "bert embedding + layernorm (any width) launch");
}

int launch_bert_embed_ln_fwd(const void* word, const void* pos, const void* type, const void* ids, const void* gamma,
                             const void* beta, void* sum_out, void* y, float* mean, float* rstd, int64_t B, int64_t S,
                             int64_t vocab, int64_t D, float eps, int dtype, int index_type, int64_t* status,
                             cudaStream_t st) {
    const int64_t tokens = B * S;
    if (dtype == NB2_F32)
        return index_type == NB2_I32
                   ? launch_fwd_ti<float, int32_t>(word, pos, type, ids, gamma, beta, sum_out, y, mean, rstd, tokens, S, vocab, D, eps, status, st)
                   : launch_fwd_ti<float, int64_t>(word, pos, type, ids, gamma, beta, sum_out, y, mean, rstd, tokens, S, vocab, D, eps, status, st);
    return index_type == NB2_I32
               ? launch_fwd_ti<__nv_bfloat16, int32_t>(word, pos, type, ids, gamma, beta, sum_out, y, mean, rstd, tokens, S, vocab, D, eps, status, st)
               : launch_fwd_ti<__nv_bfloat16, int64_t>(word, pos, type, ids, gamma, beta, sum_out, y, mean, rstd, tokens, S, vocab, D, eps, status, st);
}

// dpos (first S rows; the caller zeroed the rest) and dtype0 from dsum [B, S, D].
// scratch: (S + 1) * D floats.
int launch_bert_embed_table_grads(const void* dsum, void* dpos, void* dtype0, float* scratch, int64_t B, int64_t S,
                                  int64_t D, int dtype, cudaStream_t st) {
    const int64_t total = S * D;
    if (B * S == 0 || D == 0 || (dpos == nullptr && dtype0 == nullptr)) return 0;
    int64_t grid = (total + 255) / 256;
    const int64_t cap = (int64_t)sm_count() * 16;
    if (grid > cap) grid = cap;
    float* acc = dtype0 != nullptr ? scratch : nullptr;
    const int elt = dtype == NB2_F32 ? 4 : 2;
    const bool vec = (D * elt) % 16 == 0 && aligned16(dsum) && (dpos == nullptr || aligned16(dpos)) && (acc == nullptr || aligned16(acc));
    if (vec) {
        const int64_t nvec_plane = total * elt / 16;
        const unsigned vgrid = (unsigned)((nvec_plane + 127) / 128 < 2 * cap ? (nvec_plane + 127) / 128 : 2 * cap);
        if (dtype == NB2_F32) batch_sum_vec_kernel<float><<<vgrid, 128, 0, st>>>((const float*)dsum, (float*)dpos, acc, B, nvec_plane);
        else batch_sum_vec_kernel<__nv_bfloat16><<<vgrid, 128, 0, st>>>((const __nv_bfloat16*)dsum, (__nv_bfloat16*)dpos, acc, B, nvec_plane);
    } else if (dtype == NB2_F32) batch_sum_kernel<float><<<(unsigned)grid, 256, 0, st>>>((const float*)dsum, (float*)dpos, acc, B, S, D);
    else batch_sum_kernel<__nv_bfloat16><<<(unsigned)grid, 256, 0, st>>>((const __nv_bfloat16*)dsum, (__nv_bfloat16*)dpos, acc, B, S, D);
    int rc = cuda_status(cudaGetLastError(), "bert position gradient launch");
    if (rc != 0 || dtype0 == nullptr) return rc;
    float* total_row = scratch + (size_t)S * D;
    rc = launch_colreduce(scratch, S, D, total_row, st);          // sum over positions, fp64, fixed order
    if (rc != 0) return rc;
    cast_row_kernel<<<(unsigned)((D + 255) / 256), 256, 0, st>>>(total_row, dtype0, D, dtype == NB2_BF16);
    return cuda_status(cudaGetLastError(), "bert token-type gradient launch");
}

}  // namespace nb2
