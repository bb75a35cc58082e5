/*
 * TEST INFRASTRUCTURE, NOT PRODUCT CODE.  Only tests/, __graft_entry__.smoke()
 * and bench.py's CPU-baseline legs may build, load or call this file; the
 * product path (thot_b200/) never does.
 *
 * Plain-C restatement of the row-op path of the Nott (MoonFlowww/Thot) library:
 * what its modules compute, written as scalar loops in double precision on
 * fp32 inputs.  Paths below are inside the MoonFlowww/Thot project.
 *
 * The arithmetic of LayerNorm, GELU, SiLU and the embedding gather lives in
 * libtorch, an un-vendored and un-pinned dependency of the reference
 * (CMakeLists.txt:13-19, find_package(Torch REQUIRED)); this file restates the
 * published definitions of those ops (torch::nn::LayerNorm: biased variance
 * over the last dim, y = (x-mean)/sqrt(var+eps)*gamma+beta; torch::gelu:
 * exact erf form; torch::silu: x*sigmoid(x)) at the reference's call sites.
 * The restatement is pinned against the reference itself: tests/golden/*.npz
 * hold outputs of the reference's own modules run on CPU through
 * oracle/ref_harness.cpp (libtorch 2.11.0), and tests/test_oracle_golden.py
 * checks every function here against them.  Rotary has no reference
 * implementation: orc_rope_* restates the formula of the benchmark
 * configuration and its parity is unpinned.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

enum { ACT_NONE = 0, ACT_GELU = 1, ACT_SILU = 2 };

/* Nott::Activation::Details::GeLU -> torch::gelu, exact erf
 * (src/activation/details/gelu.hpp:11-15); SiLU -> torch::silu
 * (src/activation/details/silu.hpp:12-16). */
static double act_fwd(int act, double z) {
    if (act == ACT_GELU) return 0.5 * z * (1.0 + erf(z * M_SQRT1_2));
    if (act == ACT_SILU) return z / (1.0 + exp(-z));
    return z;
}
/* d act / dz.  The SiLU derivative is the reference's own dSiLU functor,
 * sigmoid * (1 + x * (1 - sigmoid)) (src/activation/details/dsilu.hpp:14-15). */
static double act_grad(int act, double z) {
    if (act == ACT_GELU) {
        const double cdf = 0.5 * (1.0 + erf(z * M_SQRT1_2));
        const double pdf = exp(-0.5 * z * z) / sqrt(2.0 * M_PI);
        return cdf + z * pdf;
    }
    if (act == ACT_SILU) {
        const double s = 1.0 / (1.0 + exp(-z));
        return s * (1.0 + z * (1.0 - s));
    }
    return 1.0;
}

/*
 * torch::nn::LayerNorm over the last dim as the blocks call it
 * (src/block/details/transformers/classic.hpp:399-404 construction, :436,445,520
 * calls; options eps / elementwise_affine :54-57) followed by
 * Activation::Details::apply (src/activation/apply.hpp:24-57).
 * Backward (what autograd produces for loss.backward(), src/core.hpp:3811-3820):
 *   dz = dy * act'(z), dgamma = sum_rows dz*xhat, dbeta = sum_rows dz,
 *   g = dz*gamma, dx = rstd * (g - mean(g) - xhat * mean(g*xhat)).
 * gamma/beta may be NULL (no affine).  dy NULL -> forward only.
 */
void orc_layernorm_act(const float* x, const float* gamma, const float* beta, const float* dy,
                       int64_t rows, int64_t D, double eps, int act,
                       double* y, double* mean_out, double* rstd_out,
                       double* dx, double* dgamma, double* dbeta) {
    if (dgamma) memset(dgamma, 0, sizeof(double) * (size_t)D);
    if (dbeta) memset(dbeta, 0, sizeof(double) * (size_t)D);
    double* gbuf = (double*)malloc(sizeof(double) * (size_t)(D > 0 ? D : 1));
    double* hbuf = (double*)malloc(sizeof(double) * (size_t)(D > 0 ? D : 1));
    for (int64_t r = 0; r < rows; ++r) {
        const float* xr = x + r * D;
        double s = 0.0;
        for (int64_t c = 0; c < D; ++c) s += xr[c];
        const double mu = s / (double)D;
        double q = 0.0;
        for (int64_t c = 0; c < D; ++c) { const double d = xr[c] - mu; q += d * d; }
        const double rs = 1.0 / sqrt(q / (double)D + eps);
        if (mean_out) mean_out[r] = mu;
        if (rstd_out) rstd_out[r] = rs;
        double s1 = 0.0, s2 = 0.0;
        for (int64_t c = 0; c < D; ++c) {
            const double h = (xr[c] - mu) * rs;
            const double g = gamma ? gamma[c] : 1.0;
            const double z = h * g + (beta ? beta[c] : 0.0);
            if (y) y[r * D + c] = act_fwd(act, z);
            if (dy) {
                const double dz = dy[r * D + c] * act_grad(act, z);
                if (dgamma) dgamma[c] += dz * h;
                if (dbeta) dbeta[c] += dz;
                gbuf[c] = dz * g;
                hbuf[c] = h;
                s1 += gbuf[c];
                s2 += gbuf[c] * h;
            }
        }
        if (dy && dx) {
            const double m1 = s1 / (double)D, m2 = s2 / (double)D;
            for (int64_t c = 0; c < D; ++c) dx[r * D + c] = rs * (gbuf[c] - m1 - hbuf[c] * m2);
        }
    }
    free(gbuf);
    free(hbuf);
}

/*
 * RMSNormImpl::forward (src/block/details/transformers/mamba.hpp:124-142):
 *   variance = x.pow(2).mean(-1); normalized = x * rsqrt(variance + eps);
 *   if weight: normalized *= weight        (options eps=1e-6, learnable :25-28)
 * followed by apply(act).  Backward with g = dz*w, xhat = x*rstd:
 *   dx = rstd * (g - xhat * mean(g*xhat)),  dweight = sum_rows dz * xhat.
 */
void orc_rmsnorm_act(const float* x, const float* weight, const float* dy,
                     int64_t rows, int64_t D, double eps, int act,
                     double* y, double* rstd_out, double* dx, double* dweight) {
    if (dweight) memset(dweight, 0, sizeof(double) * (size_t)D);
    double* gbuf = (double*)malloc(sizeof(double) * (size_t)(D > 0 ? D : 1));
    for (int64_t r = 0; r < rows; ++r) {
        const float* xr = x + r * D;
        double q = 0.0;
        for (int64_t c = 0; c < D; ++c) q += (double)xr[c] * (double)xr[c];
        const double rs = 1.0 / sqrt(q / (double)D + eps);
        if (rstd_out) rstd_out[r] = rs;
        double s2 = 0.0;
        for (int64_t c = 0; c < D; ++c) {
            const double h = xr[c] * rs;
            const double w = weight ? weight[c] : 1.0;
            const double z = h * w;
            if (y) y[r * D + c] = act_fwd(act, z);
            if (dy) {
                const double dz = dy[r * D + c] * act_grad(act, z);
                if (dweight) dweight[c] += dz * h;
                gbuf[c] = dz * w;
                s2 += gbuf[c] * h;
            }
        }
        if (dy && dx) {
            const double m2 = s2 / (double)D;
            for (int64_t c = 0; c < D; ++c) dx[r * D + c] = rs * (gbuf[c] - xr[c] * rs * m2);
        }
    }
    free(gbuf);
}

/* apply(GeLU|SiLU) elementwise (src/activation/apply.hpp:36-39). */
void orc_act(const float* x, const float* dy, int64_t n, int act, double* y, double* dx) {
    for (int64_t i = 0; i < n; ++i) {
        if (y) y[i] = act_fwd(act, x[i]);
        if (dy && dx) dx[i] = dy[i] * act_grad(act, x[i]);
    }
}

/*
 * SwiGLU: chunk(2, -1) then silu(first) * second
 * (src/activation/details/swiglu.hpp:18-23); Mamba: up * silu(gate)
 * (src/block/details/transformers/mamba.hpp:443-446).  a = the SiLU operand,
 * b = the multiplier, both with a row stride in elements; outputs contiguous.
 */
void orc_silu_gate(const float* a, int64_t lda, const float* b, int64_t ldb, const float* dy, int64_t lddy,
                   int64_t rows, int64_t H, double* out, double* da, double* db) {
    for (int64_t r = 0; r < rows; ++r) {
        for (int64_t c = 0; c < H; ++c) {
            const double av = a[r * lda + c], bv = b[r * ldb + c];
            const double s = 1.0 / (1.0 + exp(-av));
            if (out) out[r * H + c] = av * s * bv;
            if (dy) {
                const double d = dy[r * lddy + c];
                if (da) da[r * H + c] = d * bv * (s * (1.0 + av * (1.0 - s)));
                if (db) db[r * H + c] = d * av * s;
            }
        }
    }
}

/*
 * torch::nn::Embedding::forward as a gather of whole rows
 * (src/block/details/transformers/bert.hpp:162-163; ebt.hpp:124-126):
 * out[t,:] = table[ids[t],:], copied byte for byte.  Returns the first token
 * position whose id is outside [0, vocab) (that row is zero-filled), or -1.
 */
int64_t orc_embedding(const void* table, const int64_t* ids, int64_t tokens, int64_t vocab,
                      int64_t row_bytes, void* out) {
    int64_t bad = -1;
    for (int64_t t = 0; t < tokens; ++t) {
        char* dst = (char*)out + t * row_bytes;
        if (ids[t] < 0 || ids[t] >= vocab) {
            memset(dst, 0, (size_t)row_bytes);
            if (bad < 0) bad = t;
        } else {
            memcpy(dst, (const char*)table + ids[t] * row_bytes, (size_t)row_bytes);
        }
    }
    return bad;
}

/* Its autograd: dtable[v,:] = sum over tokens with ids[t]==v of dout[t,:]. */
void orc_embedding_bwd(const float* dout, const int64_t* ids, int64_t tokens, int64_t vocab, int64_t D,
                       double* dtable) {
    memset(dtable, 0, sizeof(double) * (size_t)(vocab * D));
    for (int64_t t = 0; t < tokens; ++t) {
        if (ids[t] < 0 || ids[t] >= vocab) continue;
        for (int64_t c = 0; c < D; ++c) dtable[ids[t] * D + c] += dout[t * D + c];
    }
}

/*
 * Rotary embedding, rotate-half pairing (i, i + hd/2).  No reference code
 * exists (docs/sub/block/README.md:132-136 is prose only); this follows the
 * benchmark configuration: angle(s,i) = float(pos[s]) * float(theta^(-2i/hd)),
 * cos/sin in fp32.  cos_sin is [S, hd/2, 2] fp32.
 */
void orc_rope_table(const int32_t* positions, int64_t S, int64_t hd, double theta, float* cos_sin) {
    const int64_t half = hd / 2;
    for (int64_t s = 0; s < S; ++s) {
        const float pos = positions ? (float)positions[s] : (float)s;
        for (int64_t i = 0; i < half; ++i) {
            const float inv = (float)pow(theta, -2.0 * (double)i / (double)hd);
            const float ang = pos * inv;
            cos_sin[(s * half + i) * 2 + 0] = (float)cos((double)ang);
            cos_sin[(s * half + i) * 2 + 1] = (float)sin((double)ang);
        }
    }
}

/* x, out: [B, S, H, hd].  inverse != 0 rotates by -angle (the backward). */
void orc_rope_apply(const float* x, const float* cos_sin, int64_t B, int64_t S, int64_t H, int64_t hd,
                    int inverse, double* out) {
    const int64_t half = hd / 2;
    const double sign = inverse ? -1.0 : 1.0;
    for (int64_t b = 0; b < B; ++b)
        for (int64_t s = 0; s < S; ++s)
            for (int64_t h = 0; h < H; ++h) {
                const int64_t base = ((b * S + s) * H + h) * hd;
                for (int64_t i = 0; i < half; ++i) {
                    const double c = cos_sin[(s * half + i) * 2], sn = sign * cos_sin[(s * half + i) * 2 + 1];
                    const double x1 = x[base + i], x2 = x[base + i + half];
                    out[base + i] = x1 * c - x2 * sn;
                    out[base + i + half] = x2 * c + x1 * sn;
                }
            }
}

/*
 * Attention probabilities: ScaledDotProductKernelImpl::forward between its two matmuls
 * (src/attention/details/kernel.hpp:33-92).  scores / sqrt(head_dim) (:32-34, here scores * scale),
 * key padding -> -inf (:36-39), + additive mask (:41-84), causal columns s > t -> -inf (:86-91),
 * softmax over the last dim (:93).  mask element (b,h,t,s) sits at b*mask_sb + h*mask_sh + t*S + s.
 * A row with every column masked is NaN, as torch::softmax makes it.
 * Backward of softmax and of the scaling: dscores = scale * attn * (dattn - sum_s attn * dattn).
 */
void orc_attention_softmax_noise(const float* scores, const uint8_t* key_padding, const float* mask, int64_t mask_sb,
                                 int64_t mask_sh, const float* dattn, const float* noise, int64_t B, int64_t H, int64_t T,
                                 int64_t S, double scale, int causal, double* attn, double* dropped, double* dscores);

void orc_attention_softmax(const float* scores, const uint8_t* key_padding, const float* mask, int64_t mask_sb,
                           int64_t mask_sh, const float* dattn, int64_t B, int64_t H, int64_t T, int64_t S,
                           double scale, int causal, double* attn, double* dscores) {
    orc_attention_softmax_noise(scores, key_padding, mask, mask_sb, mask_sh, dattn, NULL, B, H, T, S, scale, causal, attn, NULL,
                                dscores);
}

/*
 * The same with the dropout that follows the softmax in the reference (src/attention/details/kernel.hpp:94;
 * multiplicative-noise form of src/layer/details/dropout.hpp:41-43): dropped = attn * noise for a given noise
 * tensor.  dattn is then the gradient of `dropped`: the gradient reaching attn is dattn * noise.
 */
void orc_attention_softmax_noise(const float* scores, const uint8_t* key_padding, const float* mask, int64_t mask_sb,
                                 int64_t mask_sh, const float* dattn, const float* noise, int64_t B, int64_t H, int64_t T,
                                 int64_t S, double scale, int causal, double* attn, double* dropped, double* dscores) {
    double* row = (double*)malloc(sizeof(double) * (size_t)(S > 0 ? S : 1));
    for (int64_t b = 0; b < B; ++b)
        for (int64_t h = 0; h < H; ++h)
            for (int64_t t = 0; t < T; ++t) {
                const int64_t r = (b * H + h) * T + t;
                const float* src = scores + r * S;
                double mx = -INFINITY;
                for (int64_t s = 0; s < S; ++s) {
                    double v = (double)src[s] * scale;
                    if (key_padding && key_padding[b * S + s]) v = -INFINITY;
                    if (mask) v += (double)mask[b * mask_sb + h * mask_sh + t * S + s];
                    if (causal && s > t) v = -INFINITY;
                    row[s] = v;
                    if (v > mx) mx = v;
                }
                double sum = 0.0;
                for (int64_t s = 0; s < S; ++s) { row[s] = exp(row[s] - mx); sum += row[s]; }
                double dot = 0.0;
                for (int64_t s = 0; s < S; ++s) {
                    const double nz = noise ? (double)noise[r * S + s] : 1.0;
                    row[s] /= sum;
                    if (attn) attn[r * S + s] = row[s];
                    if (dropped) dropped[r * S + s] = row[s] * nz;
                    if (dattn) dot += row[s] * (double)dattn[r * S + s] * nz;
                }
                if (dattn && dscores)
                    for (int64_t s = 0; s < S; ++s) {
                        const double nz = noise ? (double)noise[r * S + s] : 1.0;
                        dscores[r * S + s] = scale * row[s] * ((double)dattn[r * S + s] * nz - dot);
                    }
            }
    free(row);
}
