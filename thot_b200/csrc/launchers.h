// Internal launch functions behind the extern "C" entry points in api.cu.
#pragma once
#include "nb2_common.cuh"
#include "norm_dispatch.cuh"

namespace nb2 {

int launch_act(const void* x, const void* dy, void* out, int64_t n, int dtype, int act, bool bwd, cudaStream_t st);
int launch_add(const void* a, const void* b, void* out, int64_t n, int dtype, cudaStream_t st);
int launch_silu_gate(const void* a, int64_t lda, const void* b, int64_t ldb,
                     const void* dy, int64_t lddy, void* o0, int64_t ldo0, void* o1, int64_t ldo1,
                     int64_t rows, int64_t H, int dtype, bool bwd, cudaStream_t st);
int launch_colreduce(const float* partials, int64_t n_partials, int64_t ncols, float* out, cudaStream_t st);
int launch_embedding_fwd(const void* table, const void* ids, void* out, int64_t tokens, int64_t vocab,
                         int64_t D, int dtype, int index_type, int64_t* status, cudaStream_t st);
size_t embedding_bwd_workspace(int64_t tokens, int64_t vocab);
// the two phases of launch_embedding_bwd: the index needs only the ids, the sums need the index
int launch_embedding_bwd_index(const void* ids, int64_t tokens, int64_t vocab, int index_type, void* ws,
                               size_t ws_bytes, cudaStream_t st);
int launch_embedding_bwd_sum(const void* dout, void* dtable, int64_t tokens, int64_t vocab, int64_t D, int dtype,
                             void* ws, cudaStream_t st);
int launch_embedding_bwd(const void* dout, const void* ids, void* dtable, int64_t tokens, int64_t vocab,
                         int64_t D, int dtype, int index_type, void* ws, size_t ws_bytes, cudaStream_t st);
int launch_bert_embed_ln_fwd(const void* word, const void* pos, const void* type, const void* ids, const void* gamma,
                             const void* beta, void* sum_out, void* y, float* mean, float* rstd, int64_t B, int64_t S,
                             int64_t vocab, int64_t D, float eps, int dtype, int index_type, int64_t* status,
                             cudaStream_t st);
int launch_bert_embed_table_grads(const void* dsum, void* dpos, void* dtype0, float* scratch, int64_t B, int64_t S,
                                  int64_t D, int dtype, cudaStream_t st);
int launch_rope_table(float* cos_sin, const int32_t* positions, int64_t S, int64_t hd, double theta, cudaStream_t st);
int launch_rope_apply(const void* x, const float* cos_sin, void* out, int64_t B, int64_t S, int64_t H,
                      int64_t hd, int dtype, bool inverse, cudaStream_t st);

int launch_attention_softmax_fwd(const void* scores, const uint8_t* key_padding, const void* add_mask, int64_t mask_sb,
                                 int64_t mask_sh, void* out, int64_t B, int64_t H, int64_t Tq, int64_t S, float scale,
                                 int causal, int dtype, cudaStream_t st, const void* noise = nullptr, void* pre_out = nullptr);
int launch_attention_softmax_bwd(const void* attn, const void* dattn, void* dscores, int64_t rows, int64_t S, float scale,
                                 int dtype, cudaStream_t st, const void* noise = nullptr);

int set_softmax_order(int order);      // 0 by size, 1 memory order, 2 heads innermost whenever the mask is shared by the heads

// tensor-core linear layer: lives in libnott_b200_linear.so (thot_b200/csrc_linear), loaded on first use
int launch_linear(const void* x, const void* w, const void* bias, void* z_out, void* y, int64_t M, int64_t N, int64_t K, int act,
                  void* workspace, size_t workspace_bytes, cudaStream_t st);
bool linear_library_present();

}  // namespace nb2
