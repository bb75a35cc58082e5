/*
 * nott_b200.h — C ABI of libnott_b200.so: hand-written sm_100a kernels for the
 * memory-bound row-op path of the Nott (MoonFlowww/Thot) C++ library.
 *
 * Conventions
 *   - Every function returns an int status: 0 = ok, < 0 = invalid argument
 *     (NB2_ERR_*), > 0 = the cudaError_t the launch produced.  Nothing throws.
 *     nb2_last_error_string() describes the last non-zero status of the
 *     calling thread.
 *   - All pointers are DEVICE pointers unless the name ends in `_host`.
 *     Outputs are caller-allocated; no function here allocates or frees device
 *     memory, synchronises the device, or touches any stream but `stream`.
 *     `stream` is a cudaStream_t passed as void* so the header needs no CUDA
 *     include.
 *   - Tensors are row-major `[rows, D]` views of Nott's contiguous `(B,S,D)`
 *     tensors (the reference makes them contiguous in normalise_to_sequence,
 *     src/block/details/transformers/classic.hpp:217-273).
 *   - `dtype` selects the element type of activations AND of the affine
 *     parameters (NB2_F32 or NB2_BF16).  Statistics, partial sums and every
 *     intermediate are fp32 (fp64 in the partial reduce).
 *   - There is no CPU fallback: without a CUDA device every compute entry
 *     point returns the CUDA error.
 *
 * Each declaration cites the reference interface it replaces, by the file's
 * path inside the MoonFlowww/Thot project.
 */
#ifndef NOTT_B200_H
#define NOTT_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* every symbol declared here is exported; everything else in the library is hidden */
#if defined(__GNUC__)
#pragma GCC visibility push(default)
#endif

#define NB2_ABI_VERSION 1

/* element types */
enum { NB2_F32 = 0, NB2_BF16 = 1 };

/* activation fused behind a norm, or applied stand-alone.  The numbering is
 * this library's own; the host layer maps Nott::Activation::Type
 * (src/activation/activation.hpp:6-21) onto it. */
enum { NB2_ACT_NONE = 0, NB2_ACT_GELU = 1, NB2_ACT_SILU = 2 };

/* index types for the embedding gather */
enum { NB2_I32 = 0, NB2_I64 = 1 };

/* status codes (< 0) */
enum {
    NB2_OK = 0,
    NB2_ERR_NULL = -1,        /* a required pointer is NULL              */
    NB2_ERR_SHAPE = -2,       /* rows/D/stride out of the supported range */
    NB2_ERR_DTYPE = -3,       /* unknown dtype / act / index type         */
    NB2_ERR_ALIGN = -4,       /* pointer or stride alignment              */
    NB2_ERR_WORKSPACE = -5,   /* workspace too small                      */
    NB2_ERR_DEVICE = -6,      /* device-side status word reported a fault */
    NB2_ERR_COMM = -7,        /* the gradient exchange failed or its communicator was aborted */
    NB2_ERR_COMM_TIMEOUT = -8, /* the gradient exchange did not finish before the deadline */
    NB2_ERR_UNAVAILABLE = -9  /* an optional part of the library is not installed */
};

/* which operation a workspace query is for */
enum {
    NB2_WS_NORM_BWD = 0,      /* per-CTA dgamma/dbeta (or dweight) partials */
    NB2_WS_EMBEDDING_BWD = 1, /* sort keys + radix-sort temporary           */
    NB2_WS_ROPE_TABLE = 2,    /* cos/sin table [S, hd/2, 2] fp32            */
    NB2_WS_BERT_EMBEDDING_BWD = 3, /* norm partials + type-row sums + sort scratch */
    NB2_WS_LINEAR = 4         /* tile-scheduler scratch of the tensor-core linear layer */
};

int nb2_abi_version(void);
const char* nb2_last_error_string(void);

/* Number of SMs the library sized its persistent grids for on the current
 * device (148 on B200); <= 0 when no device is usable. */
int nb2_sm_count(void);
/*
 * Set aside `n` SMs (0 = none, the default) that the persistent norm kernels leave unused; returns
 * the previous value.  Process-wide.  No counterpart in the reference.  For callers that run a
 * kernel of their own beside these (the allreduce of the previous step on another stream): the
 * norm kernels give each CTA a fixed share of the rows, one CTA per SM, and a CTA that finds its
 * SM taken runs after all the others.
 */
int nb2_reserve_sms(int n);

/*
 * Reads (synchronously) the device status word of the current device into
 * *status_host and, if `clear` != 0, resets it.  The bulk-async norm kernels bound
 * every wait; one that gives up records (code << 16 | CTA index) there and the
 * kernel returns early, so a mis-programmed copy shows up as NB2_ERR_DEVICE
 * from this call instead of a hung GPU.  0 = no kernel gave up.  Has no
 * counterpart in the reference (its errors are host-side C++ exceptions only).
 */
int nb2_device_status(unsigned int* status_host, int clear);

/*
 * Self-test of the bounded device-side wait (no counterpart in the reference).  Launches one
 * small kernel that waits on a barrier nothing will ever complete, with the same wait routine
 * the bulk-async kernels use but a limit of `cycle_limit` SM cycles (<= 2e9).  The wait must run
 * out: afterwards nb2_device_status() returns NB2_ERR_DEVICE with code 3, *waited_cycles (device
 * int64, may be NULL) holds how long the kernel waited, and the context stays usable.
 */
int nb2_selftest_bounded_wait(int64_t cycle_limit, int64_t* waited_cycles, void* stream);

/*
 * Row order of nb2_attention_softmax_fwd when one additive mask row serves all heads (head stride 0).  0 (default):
 * chosen by size -- heads innermost, mask row kept on chip across a (batch, position) pair's heads, when there are enough
 * pairs to fill the GPU, memory order otherwise; 1: always memory order; 2: heads innermost whenever the mask allows it.
 * Results do not depend on it (same arithmetic per row); it exists for measurements and tests.  Process-wide; the
 * environment variable NB2_SOFTMAX_ORDER=flat|inner sets the initial value.  Returns the previous setting, or
 * NB2_ERR_SHAPE for a value outside 0..2.  No counterpart in the reference.
 */
int nb2_attention_softmax_order(int order);

/*
 * Workspace sizes, in bytes, for the calls that need scratch memory.
 *   NB2_WS_NORM_BWD      : a = rows, b = D            -> partials buffer
 *   NB2_WS_EMBEDDING_BWD : a = tokens, b = vocab rows -> sort scratch
 *   NB2_WS_ROPE_TABLE    : a = seq_len, b = head_dim  -> cos/sin table
 *   NB2_WS_BERT_EMBEDDING_BWD : a = (B << 32) | S, b = (vocab << 32) | D
 *   NB2_WS_LINEAR        : a, b unused                -> a fixed upper bound
 * Returns 0 for unknown `op`.
 */
size_t nb2_workspace_bytes(int op, int64_t a, int64_t b, int dtype);

/* ------------------------------------------------------------------ *
 * LayerNorm (+ fused GELU / SiLU)
 * Replaces torch::nn::LayerNorm::forward as Nott's blocks call it
 * (src/block/details/transformers/classic.hpp:436,445,520; bert.hpp:189;
 * vision.hpp:193) followed, when `act` != NONE, by
 * Nott::Activation::Details::apply (src/activation/apply.hpp:24-57) with
 * GeLU (details/gelu.hpp:11-15, exact erf) or SiLU (details/silu.hpp:12-16).
 *   y = act( (x - mean) * rstd * gamma + beta ),  rstd = 1/sqrt(var_biased + eps)
 * gamma/beta may be NULL (elementwise_affine=false, classic.hpp:54-57).
 * mean/rstd ([rows] fp32) are written for the backward; either may be NULL
 * for inference.
 * ------------------------------------------------------------------ */
int nb2_layernorm_fwd(const void* x, const void* gamma, const void* beta,
                      void* y, float* mean, float* rstd,
                      int64_t rows, int64_t D, double eps,
                      int dtype, int act, void* stream);

/*
 * Backward of the above (what libtorch autograd runs for
 * native_layer_norm_backward + gelu_backward/silu_backward when Nott calls
 * loss.backward(), src/core.hpp:3811-3820).  Writes dx and one
 * [2, D] fp32 partial (dgamma row, dbeta row) per CTA into `partials`
 * (size nb2_workspace_bytes(NB2_WS_NORM_BWD, rows, D, dtype)); `n_partials`
 * receives how many were written.  Finish with nb2_colreduce_partials.
 * partials may be NULL when gamma is NULL (no affine gradients wanted).
 */
int nb2_layernorm_bwd(const void* x, const void* dy, const void* gamma, const void* beta,
                      const float* mean, const float* rstd,
                      void* dx, float* partials, int64_t* n_partials_host,
                      int64_t rows, int64_t D,
                      int dtype, int act, void* stream);

/*
 * The same backward for callers that cannot allocate device memory (no
 * counterpart in the reference, which always allocates through libtorch).
 * A host that runs under a frozen memory plan, or that is only ever handed its
 * input and output buffers, has nowhere to get the partials workspace from; here
 * that scratch is a fixed 4.6 MiB array inside the library image (present on
 * every GPU that loads the library, for the life of the process).  The call
 * writes dx and the finished [2, D] fp32 gradients (dgamma row, dbeta row) and
 * performs no cudaMalloc/cudaFree or any other allocating call.
 *   - Limit: the shape must satisfy
 *     nb2_workspace_bytes(NB2_WS_NORM_BWD, rows, D, dtype) <= 296 * 2 * 2048 * 4 + 256,
 *     which holds for D <= 2048 at any row count (and for wider rows when there
 *     are few of them); larger shapes return NB2_ERR_WORKSPACE.
 *   - gamma must be non-NULL.
 *   - The first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress); make that first call outside any stream capture.
 *   - All calls share the one array and it keeps the previous call's contents:
 *     two calls that overlap on the GPU (different streams) race on it.
 */
int nb2_layernorm_bwd_static(const void* x, const void* dy, const void* gamma, const void* beta,
                             const float* mean, const float* rstd,
                             void* dx, float* dgamma_dbeta,
                             int64_t rows, int64_t D,
                             int dtype, int act, void* stream);

/* ------------------------------------------------------------------ *
 * RMSNorm (+ fused GELU / SiLU)
 * Replaces Nott's RMSNormImpl::forward
 * (src/block/details/transformers/mamba.hpp:124-142; options eps=1e-6,
 * learnable, :25-28):  y = act( x * rsqrt(mean(x^2) + eps) * weight ).
 * weight may be NULL (learnable=false).  rstd ([rows] fp32) may be NULL.
 * ------------------------------------------------------------------ */
int nb2_rmsnorm_fwd(const void* x, const void* weight,
                    void* y, float* rstd,
                    int64_t rows, int64_t D, double eps,
                    int dtype, int act, void* stream);

/* Backward: dx and per-CTA [1, D] fp32 dweight partials (same workspace
 * query and second pass as LayerNorm, with 1 row per partial). */
int nb2_rmsnorm_bwd(const void* x, const void* dy, const void* weight,
                    const float* rstd,
                    void* dx, float* partials, int64_t* n_partials_host,
                    int64_t rows, int64_t D,
                    int dtype, int act, void* stream);

/* ------------------------------------------------------------------ *
 * Residual add fused with the norm that follows it.
 * Replaces the pair `output = residual + attention; norm2_->forward(output)`
 * (src/block/details/transformers/classic.hpp:442-445; bert.hpp:291-293
 * post-norm `norm1(residual + attn)`; mamba.hpp:409-415 for RMSNorm):
 *   sum_out = a + b   (rounded to the tensor dtype, as the reference's sum tensor is)
 *   y       = norm(sum_out) * gamma (+ beta)
 * Both are written: the sum is the next residual.  One pass (2 reads, 2 writes)
 * instead of an add (2 reads, 1 write) plus a norm (1 read, 1 write).  Shapes the
 * fused kernels do not cover run as add + norm inside the call.
 * Backward: dx = norm_backward(dy) + dsum, where dsum is the gradient that
 * reaches the sum through the residual branch (NULL = none); da = db = dx.
 * `sum` is the forward's sum_out.  Partials / second pass as for nb2_layernorm_bwd.
 * ------------------------------------------------------------------ */
int nb2_add_layernorm_fwd(const void* a, const void* b, const void* gamma, const void* beta,
                          void* sum_out, void* y, float* mean, float* rstd,
                          int64_t rows, int64_t D, double eps, int dtype, void* stream);
int nb2_add_layernorm_bwd(const void* sum, const void* dy, const void* dsum, const void* gamma,
                          const float* mean, const float* rstd,
                          void* dx, float* partials, int64_t* n_partials_host,
                          int64_t rows, int64_t D, int dtype, void* stream);
int nb2_add_rmsnorm_fwd(const void* a, const void* b, const void* weight,
                        void* sum_out, void* y, float* rstd,
                        int64_t rows, int64_t D, double eps, int dtype, void* stream);
int nb2_add_rmsnorm_bwd(const void* sum, const void* dy, const void* dsum, const void* weight,
                        const float* rstd,
                        void* dx, float* partials, int64_t* n_partials_host,
                        int64_t rows, int64_t D, int dtype, void* stream);

/*
 * Second pass: out[c] = sum_p partials[p, c] for c < ncols, summed in fp64 in
 * a fixed order (deterministic), written as fp32.  For LayerNorm ncols = 2*D
 * (out = [dgamma | dbeta]); for RMSNorm ncols = D.
 */
int nb2_colreduce_partials(const float* partials, int64_t n_partials, int64_t ncols,
                           float* out, void* stream);

/* ------------------------------------------------------------------ *
 * Stand-alone activations: Nott::Activation::Details::GeLU / SiLU
 * (src/activation/details/gelu.hpp:11-15, silu.hpp:12-16; Swish,
 * swish.hpp:12-17, is the same function).  n = number of elements.
 * bwd: dx = dy * act'(x)   (SiLU' is the reference's own dSiLU,
 * src/activation/details/dsilu.hpp:14-15).
 * ------------------------------------------------------------------ */
int nb2_act_fwd(const void* x, void* y, int64_t n, int dtype, int act, void* stream);
int nb2_act_bwd(const void* x, const void* dy, void* dx, int64_t n, int dtype, int act, void* stream);

/* ------------------------------------------------------------------ *
 * SiLU gate: out[r, c] = silu(a[r, c]) * b[r, c],  r < rows, c < H.
 * Replaces Nott::Activation::Details::SwiGLU
 * (src/activation/details/swiglu.hpp:13-25: a | b are the two halves of one
 * [rows, 2H] tensor -> lda = ldb = 2H, b = a + H) and Mamba's gated feed
 * forward `up * silu(gate)` (mamba.hpp:441-449: separate contiguous tensors
 * -> lda = ldb = H, a = gate, b = up).  ld* are row strides in ELEMENTS.
 * out is [rows, H] with row stride ldo.
 * bwd: da = dy * b * silu'(a),  db = dy * silu(a); da/db use strides ldda/lddb.
 * ------------------------------------------------------------------ */
int nb2_silu_gate_fwd(const void* a, int64_t lda, const void* b, int64_t ldb,
                      void* out, int64_t ldo,
                      int64_t rows, int64_t H, int dtype, void* stream);
int nb2_silu_gate_bwd(const void* a, int64_t lda, const void* b, int64_t ldb,
                      const void* dy, int64_t lddy,
                      void* da, int64_t ldda, void* db, int64_t lddb,
                      int64_t rows, int64_t H, int dtype, void* stream);

/* ------------------------------------------------------------------ *
 * Token-embedding gather: out[t, :] = table[ids[t], :], a bit copy.
 * Replaces torch::nn::Embedding::forward as called by BertEmbeddingImpl
 * (src/block/details/transformers/bert.hpp:162-163,176-187),
 * TokenEmbeddingImpl (ebt.hpp:124-126) and the learned positional encoding
 * (classic.hpp:366-370).  ids are int32 or int64 (`index_type`).
 * An id outside [0, vocab) never faults: that output row is zero-filled and,
 * if `status` (device int64[2]) is non-NULL, status[0] is set to 1 and
 * status[1] to the offending token position.
 * ------------------------------------------------------------------ */
int nb2_embedding_fwd(const void* table, const void* ids, void* out,
                      int64_t tokens, int64_t vocab, int64_t D,
                      int dtype, int index_type, int64_t* status, void* stream);

/*
 * Backward: dtable[v, :] = sum over {t : ids[t] == v} of dout[t, :], summed in
 * fp32 in ascending t (deterministic), rows without tokens set to zero.
 * Every row of dtable is written.  `workspace` has
 * nb2_workspace_bytes(NB2_WS_EMBEDDING_BWD, tokens, vocab, dtype) bytes.
 */
int nb2_embedding_bwd(const void* dout, const void* ids, void* dtable,
                      int64_t tokens, int64_t vocab, int64_t D,
                      int dtype, int index_type,
                      void* workspace, size_t workspace_bytes, void* stream);
/*
 * The same backward in two calls.  nb2_embedding_index needs only the ids (it sorts them and
 * records each table row's run of tokens in `workspace`, same size as above), so a host can issue
 * it when the ids arrive -- beside the forward gather, on another stream -- and keep the workspace;
 * nb2_embedding_bwd_indexed then forms dtable from dout and that workspace alone.  Called back to
 * back on one stream they are nb2_embedding_bwd.  One index serves any number of backward calls
 * over the same ids, one at a time (the index also holds the call's list of long token runs).
 */
int nb2_embedding_index(const void* ids, int64_t tokens, int64_t vocab, int index_type,
                        void* workspace, size_t workspace_bytes, void* stream);
int nb2_embedding_bwd_indexed(const void* dout, void* dtable, int64_t tokens, int64_t vocab, int64_t D,
                              int dtype, void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------ *
 * BERT's embedding front end in one pass:
 *   y[b,s,:] = LayerNorm( word[ids[b,s],:] + pos[s,:] + type[0,:] ) * gamma + beta
 * Replaces BertEmbeddingImpl::forward
 * (src/block/details/transformers/bert.hpp:155-194: word gather :162-163,
 * position gather of arange(S) :176-181, token-type gather of zeros :183-187,
 * LayerNorm with eps 1e-12 :143-146,189; dropout is left to the caller).
 * pos ([>= S, D]) and type ([>= 1, D]) may be NULL (the reference's
 * use_position_embeddings / use_token_type switches).  sum_out ([B*S, D], the
 * pre-norm sum rounded to the tensor dtype) may be NULL for inference; the
 * backward needs it, with mean and rstd.  Bad ids behave as in
 * nb2_embedding_fwd (zero word row + status word).
 * ids == NULL selects the module's other branch (bert.hpp:164-171: an input that
 * is not a Long tensor is taken as ready-made embeddings): `word` is then the
 * [B*S, D] embeddings themselves, `vocab` is ignored, and in the backward dsum is
 * the gradient of that input (dword is not written and may be NULL).
 * Backward: dsum = LayerNorm backward of dy (written to the caller's
 * [B*S, D] buffer), dword = deterministic scatter-add of dsum by id, dpos[s] =
 * sum over the batch of dsum[:, s] (rows >= S of the pos_rows-row gradient are
 * zeroed), dtype0 = sum of all dsum rows (gradient of type row 0; other rows
 * of that table receive none), dgamma_dbeta [2, D] fp32.  dpos / dtype0 may be
 * NULL.  workspace: nb2_workspace_bytes(NB2_WS_BERT_EMBEDDING_BWD,
 * (B << 32) | S, (vocab << 32) | D, dtype).
 * ------------------------------------------------------------------ */
int nb2_bert_embedding_ln_fwd(const void* word, const void* pos, const void* type, const void* ids,
                              const void* gamma, const void* beta,
                              void* sum_out, void* y, float* mean, float* rstd,
                              int64_t B, int64_t S, int64_t vocab, int64_t D, double eps,
                              int dtype, int index_type, int64_t* status, void* stream);
int nb2_bert_embedding_ln_bwd(const void* sum, const void* dy, const void* ids, const void* gamma,
                              const float* mean, const float* rstd,
                              void* dsum, void* dword, void* dpos, int64_t pos_rows, void* dtype0,
                              float* dgamma_dbeta,
                              int64_t B, int64_t S, int64_t vocab, int64_t D,
                              int dtype, int index_type,
                              void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------ *
 * Fully connected layer with its bias and activation in the GEMM's epilogue:
 *   y[M, N] = act( x[M, K] . weight[N, K]^T + bias[N] )
 * Replaces Nott's FC layer -- torch::nn::Linear bound into a RegisteredLayer with
 * the activation that follows it (src/layer/details/fc.hpp:31-49), run as
 * `layer.forward` then `apply(layer.activation, .)` by the feed-forward loop of the
 * transformer blocks (src/block/details/transformers/classic.hpp:446-452): a GEMM
 * plus a bias pass plus an activation pass over [M, N] in libtorch.
 * bf16 operands and output, fp32 accumulation on the tcgen05 tensor cores
 * (accumulators in TMEM, operands staged by TMA from this GPU's memory only); the
 * bias row and the activation are applied to the fp32 accumulator tile in registers
 * before its single store.  weight is torch::nn::Linear's [out_features,
 * in_features] tensor as it is; bias may be NULL.  z_out (may be NULL) receives the
 * pre-activation x.W^T + bias rounded to bf16 -- what the backward of the
 * activation needs (nb2_act_bwd).  N and K must be multiples of 8.  fp32 layers are
 * not taken (NB2_ERR_DTYPE): TF32 tensor cores do not meet the fp32 tolerance.
 * workspace: nb2_workspace_bytes(NB2_WS_LINEAR, 0, 0, dtype) bytes.
 * The kernels live in a second library, libnott_b200_linear.so, that this one opens
 * from its own folder on the first call; where it is not installed the call
 * returns NB2_ERR_UNAVAILABLE (nb2_linear_available() tells beforehand) and every
 * other entry point is unaffected.
 * ------------------------------------------------------------------ */
int nb2_linear_available(void);
int nb2_linear_bias_act_fwd(const void* x, const void* weight, const void* bias, void* z_out, void* y,
                            int64_t M, int64_t N, int64_t K, int dtype, int act,
                            void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------ *
 * Rotary embedding, rotate-half pairing (i, i + hd/2).  The reference has no
 * implementation (only docs/sub/block/README.md:132-136 mentions it); the
 * place it belongs is between the (B,H,S,hd) view and the attention kernel
 * in MultiHeadAttentionImpl::forward (src/attention/details/head.hpp:70-74).
 *   angle(s, i) = float(pos[s]) * float(theta^(-2i/hd)),   i < hd/2
 *   out[i]        = x[i]*cos - x[i+hd/2]*sin
 *   out[i+hd/2]   = x[i+hd/2]*cos + x[i]*sin
 * Layout: x, out are [B, S, H, hd] contiguous.  positions (int32 [S]) may be
 * NULL for 0..S-1.  The cos/sin table ([S, hd/2] float2, fp32) is built once
 * by nb2_rope_table and reused for q, k and the backward.
 * bwd is the rotation by -angle (`inverse` != 0).
 * ------------------------------------------------------------------ */
int nb2_rope_table(float* cos_sin, const int32_t* positions,
                   int64_t S, int64_t hd, double theta, void* stream);
int nb2_rope_apply(const void* x, const float* cos_sin, void* out,
                   int64_t B, int64_t S, int64_t H, int64_t hd,
                   int dtype, int inverse, void* stream);

/* ------------------------------------------------------------------ *
 * Attention probabilities: the steps between the two matmuls of
 * ScaledDotProductKernelImpl::forward (src/attention/details/kernel.hpp:33-92),
 *   attn = softmax(scores * scale [key padding -> -inf] [+ attn_mask] [causal -> -inf], last dim)
 * in one read of scores and one write of attn, where the reference makes five
 * passes (division, masked_fill, add, masked_fill, softmax).
 *   scores, attn : [B, H, T, S] contiguous, `dtype`; scale = 1/sqrt(head_dim) there.
 *   key_padding  : [B, S] bytes, non-zero = that key is padding (kernel.hpp:36-39), or NULL.
 *   attn_mask    : additive mask of `dtype` (kernel.hpp:41-84), or NULL; element
 *                  (b, h, t, s) is read at b*mask_batch_stride + h*mask_head_stride + t*S + s,
 *                  so [T,S] is strides (0, 0), [B,T,S] is (T*S, 0), [B,H,T,S] and
 *                  [B*H,T,S] are (H*T*S, T*S).
 *   causal != 0  : columns s > t are masked (Variant::Causal, kernel.hpp:86-91).
 * A row with every column masked comes out as NaN, as torch::softmax gives it.
 * bwd: dscores = scale * attn * (dattn - sum_s attn * dattn), rows = B*H*T; masked
 * columns receive 0, as through masked_fill.  Dropout on attn (kernel.hpp:94) is
 * not part of this call.
 * ------------------------------------------------------------------ */
int nb2_attention_softmax_fwd(const void* scores, const uint8_t* key_padding, const void* attn_mask,
                              int64_t mask_batch_stride, int64_t mask_head_stride, void* attn,
                              int64_t B, int64_t H, int64_t T, int64_t S, double scale, int causal,
                              int dtype, void* stream);
int nb2_attention_softmax_bwd(const void* attn, const void* dattn, void* dscores,
                              int64_t rows, int64_t S, double scale, int dtype, void* stream);

/*
 * The same pass with the dropout that follows it (kernel.hpp:94 `attn = dropout_->forward(attn)`;
 * also the multiplicative-noise module of src/layer/details/dropout.hpp:32-51,
 * `input * N(1, sqrt(p/(1-p)))`):   out = attn * noise,
 * where `noise` ([B, H, T, S], `dtype`) is drawn by the caller with libtorch -- a Bernoulli keep
 * mask divided by 1-p for torch::nn::Dropout, empty_like(attn).normal_(1, std) for the noise
 * module -- so the random stream is the host framework's and results are reproducible against
 * the reference given the same tensor.  attn (rounded to `dtype`, as the reference's tensor is) is
 * also written to attn_pre when that is non-NULL: the backward needs it.
 * bwd: dattn = dout * noise (rounded to `dtype`), then the softmax backward above; 3 reads and 1
 * write where the reference's autograd makes 2 passes (4 reads, 2 writes).
 */
int nb2_attention_softmax_dropout_fwd(const void* scores, const uint8_t* key_padding, const void* attn_mask,
                                      int64_t mask_batch_stride, int64_t mask_head_stride,
                                      const void* noise, void* attn_pre, void* out,
                                      int64_t B, int64_t H, int64_t T, int64_t S, double scale, int causal,
                                      int dtype, void* stream);
int nb2_attention_softmax_dropout_bwd(const void* attn_pre, const void* noise, const void* dout, void* dscores,
                                      int64_t rows, int64_t S, double scale, int dtype, void* stream);

/* ------------------------------------------------------------------ *
 * Host-buffer training step of the fused LayerNorm->activation path: the call
 * a host-resident caller makes (the reference stages batches from pinned host
 * memory itself, src/core.hpp:4197-4227).  x_host, dy_host, y_host, dx_host
 * are HOST pointers (pinned for full speed); the call copies row chunks in on
 * one stream, runs fwd + bwd, copies y and dx out on another, and returns
 * after dgamma_dbeta_host ([2, D] fp32) is complete.  `ctx` is created once
 * per (device, max rows per call, D, dtype) and owns the device staging
 * buffers; creating and destroying it are the only calls in this library that
 * allocate device memory.
 * ------------------------------------------------------------------ */
typedef struct nb2_host_ctx nb2_host_ctx;
int nb2_host_ctx_create(nb2_host_ctx** ctx, int64_t max_rows, int64_t D, int dtype, int64_t chunk_rows);
int nb2_host_ctx_destroy(nb2_host_ctx* ctx);
int nb2_layernorm_act_step_host(nb2_host_ctx* ctx,
                                const void* x_host, const void* dy_host,
                                const void* gamma_host, const void* beta_host,
                                void* y_host, void* dx_host, float* dgamma_dbeta_host,
                                int64_t rows, int64_t D, double eps, int dtype, int act);
/* The same step for RMSNorm (src/block/details/transformers/mamba.hpp:124-142) with its
 * activation: weight_host [D] in, dweight_host [D] fp32 out; same context type. */
int nb2_rmsnorm_act_step_host(nb2_host_ctx* ctx,
                              const void* x_host, const void* dy_host, const void* weight_host,
                              void* y_host, void* dx_host, float* dweight_host,
                              int64_t rows, int64_t D, double eps, int dtype, int act);

/* ------------------------------------------------------------------ *
 * Row-sharded step across the GPUs of one box, one process per GPU.
 * The reference runs on one device (src/core.hpp:1706-1708 pins cuda:0); with
 * rows (batch x sequence) split over ranks the forward and dX need no
 * communication and the only exchange is the sum over ranks of the fp32
 * parameter gradients ([2, D] LayerNorm, [D] RMSNorm), which nothing reads
 * before the optimizer step (src/core.hpp:3811-3820).
 *
 * nb2_comm: one communicator per process.  Rank 0 makes an id
 * (nb2_comm_unique_id, NB2_COMM_ID_BYTES bytes) and hands it to the other
 * ranks by any host-side channel; every rank then calls nb2_comm_create with
 * its device current.  `exchange` selects how gradients travel:
 *   NB2_EXCHANGE_NCCL : ncclAllReduce (fp32 sum, in place) on a side stream the
 *                       communicator owns, after the partial reduce.
 *   NB2_EXCHANGE_PEER : the partial-reduce kernel stores the rank's sums
 *                       straight into every peer's receive buffer over NVLink
 *                       (memory mapped with CUDA IPC) and a small second kernel
 *                       adds the ranks' slots in rank order; NCCL is used at
 *                       creation only (to pass the IPC handles around).
 * max_cols bounds the gradient vector length (2 * D for LayerNorm).
 * Creating and destroying a communicator or a step allocate and free device
 * memory and synchronise; nothing else here does.  With world == 1 no NCCL is
 * needed and `id_host` may be NULL.
 * ------------------------------------------------------------------ */
#define NB2_COMM_ID_BYTES 128
enum { NB2_EXCHANGE_NCCL = 0, NB2_EXCHANGE_PEER = 1 };
enum { NB2_NORM_LAYER = 0, NB2_NORM_RMS = 1 };
typedef struct nb2_comm nb2_comm;
int nb2_comm_unique_id(void* id_host);
int nb2_comm_create(nb2_comm** comm, const void* id_host, int rank, int world, int exchange, int64_t max_cols);
int nb2_comm_destroy(nb2_comm* comm);
int nb2_comm_info(const nb2_comm* comm, int* rank, int* world, int* exchange);

/*
 * Partial reduce + exchange as one stream-ordered unit, in two halves so that
 * the exchange can run beside other work of the stream:
 *   begin : sums the per-CTA partials (as nb2_colreduce_partials does: fp64,
 *           fixed order) and starts the sum over ranks.  `grads` ([ncols] fp32)
 *           must not be read or written by the caller until the exchange is
 *           complete.  An exchange that is still outstanding is completed by
 *           this call first (PEER form: by the same kernel launch, so a step
 *           costs one launch), which is why two gradient buffers alternate.
 *   end   : completes the outstanding exchange: afterwards (in stream order)
 *           its `grads` holds the sum over all ranks, bit-identical on every
 *           rank in the PEER form.  A no-op when nothing is outstanding.
 * comm == NULL, or a one-rank NCCL communicator, makes begin the plain partial
 * reduce.
 */
int nb2_grad_exchange_begin(nb2_comm* comm, const float* partials, int64_t n_partials, int64_t ncols,
                            float* grads, void* stream);
int nb2_grad_exchange_end(nb2_comm* comm, void* stream);

/*
 * Host-side watchdog for the exchange started last (a rank that died or never
 * joined leaves the collective waiting).  Polls the
 * exchange's completion and the communicator's asynchronous error state for at
 * most timeout_s seconds.  On an asynchronous error returns NB2_ERR_COMM, on
 * expiry NB2_ERR_COMM_TIMEOUT; in both cases the communicator has been aborted
 * (ncclCommAbort, which makes a collective kernel that is still waiting leave
 * the GPU) and every later call on it returns NB2_ERR_COMM.  nb2_comm_abort does
 * the same on request (a rank that learned of a peer's death on the host).
 */
int nb2_comm_wait(nb2_comm* comm, double timeout_s);
int nb2_comm_abort(nb2_comm* comm);

/*
 * Self-tests without a counterpart in the reference.
 * nb2_selftest_comm_watchdog runs the watchdog's policy against scripted
 * callbacks (needs no GPU and no second rank): completion is reported after
 * `polls_until_done` polls (< 0: never), an asynchronous error `error_code`
 * after `polls_until_error` polls (< 0: never); returns what nb2_comm_wait would
 * and stores the number of aborts in *aborts_host.
 * nb2_selftest_peer_wait launches the PEER form's device-side wait on a flag no
 * rank will publish, with a limit of cycle_limit SM cycles (<= 2e9): the kernel
 * returns by itself and nb2_device_status() then reports code 4.
 */
int nb2_selftest_comm_watchdog(int polls_until_done, int polls_until_error, int error_code, double timeout_s,
                               int* aborts_host);
int nb2_selftest_peer_wait(nb2_comm* comm, int64_t cycle_limit, void* stream);
/*
 * `world` (<= 16) communicators of the PEER form in one process on the current device, linked to one another as the
 * ranks of a box would be (every peer buffer is local memory), written to comms[0..world).  For tests of the
 * exchange with more ranks than GPUs: issue every rank's nb2_grad_exchange_begin for a step before any rank's begin
 * for the next step (then no launch waits for a later one), nb2_grad_exchange_end for every rank at the end, and
 * destroy each with nb2_comm_destroy.  No counterpart in the reference.
 */
int nb2_selftest_comm_group(nb2_comm** comms, int world, int64_t max_cols);

/*
 * One training step of the fused norm->activation path on this rank's row
 * shard: forward, backward (dX + partials), partial reduce and the exchange.
 * This is the loop body `layer.forward(x)` -> `apply(activation)` ->
 * `loss.backward()` of src/core.hpp:1927-1934,3811-3820 for one norm layer.
 *   run    : enqueues forward(k), backward(k) and begin of exchange(k) on
 *            `stream`; exchange k-1 is completed after forward(k), so it had
 *            that whole kernel to finish in.  `grads` of step k is complete
 *            after the next run (or finish) in stream order: pass two buffers
 *            alternately.
 *   finish : ends the outstanding exchange.
 * The step owns mean/rstd/partials scratch for `rows` x `D`.
 */
typedef struct nb2_step nb2_step;
int nb2_step_create(nb2_step** step, nb2_comm* comm, int norm, int64_t rows, int64_t D, int dtype, int act, double eps);
int nb2_step_destroy(nb2_step* step);
int nb2_step_run(nb2_step* step, const void* x, const void* dy, const void* gamma, const void* beta,
                 void* y, void* dx, float* grads, void* stream);
int nb2_step_finish(nb2_step* step, void* stream);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif

#ifdef __cplusplus
}
#endif
#endif /* NOTT_B200_H */
