// TEST INFRASTRUCTURE, NOT PRODUCT CODE.
//
// The reference's own CPU implementation of the row-op path, compiled from the
// reference's headers where they lie (never copied) against the installed
// libtorch, behind a small C interface so Python can drive it with raw buffers.
// Built by oracle/build_ref.py into oracle/_ref/libnott_ref.so.
//
// Reference code exercised here (paths inside the MoonFlowww/Thot project):
//   - Nott::Activation::Details::apply        src/activation/apply.hpp:24-57
//     (GeLU details/gelu.hpp:11-15, SiLU silu.hpp:12-16, SwiGLU swiglu.hpp:13-25)
//   - Mamba RMSNorm module                    src/block/details/transformers/mamba.hpp:110-150
//   - Mamba gated feed forward `up * silu(gate)`  mamba.hpp:443-446 (that one
//     expression, restated: it is private to EncoderLayerImpl)
//   - torch::nn::LayerNorm built the way the blocks build it
//     src/block/details/transformers/classic.hpp:399-404 (options :54-57)
//   - EBT TokenEmbedding (nn::Embedding gather)   src/block/details/transformers/ebt.hpp:81-160
//   - HardDropout: input * N(1, sqrt(p/(1-p)))   src/layer/details/dropout.hpp:23-58
//   - BertEmbedding (word + position + type gathers, LayerNorm eps 1e-12)
//                                                 src/block/details/transformers/bert.hpp:116-204
//
// Buffers are always fp32 (or int64 ids) on the host; `compute` picks the dtype
// the modules run in: 0 = fp32, 1 = fp64 (arbiter for long sums), 2 = native
// bf16 (informational: the reference rounds after every ATen op there).
#include <torch/torch.h>

#include <chrono>
#include <cstdint>
#include <cstring>
#include <string>

#include "src/activation/apply.hpp"
#include "src/block/details/transformers/mamba.hpp"
#include "src/block/details/transformers/ebt.hpp"
#include "src/attention/details/kernel.hpp"
#include "src/layer/details/dropout.hpp"

// bert.hpp pulls in src/layer/details/recurrent.hpp, which calls an overload of
// at::Context::setFloat32Precision that libtorch 2.11 no longer has (four lines that set
// TF32 flags for CUDA RNNs; nothing on this path).  The macro neutralises those calls.
#include <ATen/cuda/CUDAContext.h>
#include <torch/cuda.h>
#define setFloat32Precision(a, b, c) benchmarkCuDNN()
#include "src/block/details/transformers/bert.hpp"
#undef setFloat32Precision

namespace {

thread_local std::string g_error;

torch::ScalarType compute_type(int compute) {
    switch (compute) {
        case 1: return torch::kFloat64;
        case 2: return torch::kBFloat16;
        default: return torch::kFloat32;
    }
}

torch::Tensor wrap(const float* p, std::vector<int64_t> shape, int compute) {
    auto t = torch::from_blob(const_cast<float*>(p), shape, torch::kFloat32);
    return compute == 0 ? t : t.to(compute_type(compute));
}

void store(const torch::Tensor& t, float* out) {
    if (out == nullptr || !t.defined()) return;
    auto f = t.detach().to(torch::kFloat32).contiguous();
    std::memcpy(out, f.data_ptr<float>(), sizeof(float) * static_cast<size_t>(f.numel()));
}
void store_f64(const torch::Tensor& t, double* out) {
    if (out == nullptr || !t.defined()) return;
    auto f = t.detach().to(torch::kFloat64).contiguous();
    std::memcpy(out, f.data_ptr<double>(), sizeof(double) * static_cast<size_t>(f.numel()));
}

Nott::Activation::Type act_type(int act) {
    // 0 none, 1 GeLU, 2 SiLU -- the numbering of the CUDA library's ABI
    switch (act) {
        case 1: return Nott::Activation::Type::GeLU;
        case 2: return Nott::Activation::Type::SiLU;
        default: return Nott::Activation::Type::Identity;
    }
}

template <class F>
int guarded(F&& f) {
    try {
        f();
        return 0;
    } catch (const std::exception& e) {
        g_error = e.what();
        return 1;
    }
}

}  // namespace

extern "C" {

const char* ref_last_error() { return g_error.c_str(); }
int ref_get_num_threads() { return at::get_num_threads(); }
void ref_set_num_threads(int n) { at::set_num_threads(n); }

// LayerNorm -> activation, forward (+ backward when dy != NULL).
// gamma/beta NULL -> elementwise_affine(false).  dgamma64/dbeta64 receive the
// gradients at the module's compute precision widened to double.
int ref_layernorm_act(const float* x, const float* gamma, const float* beta, const float* dy,
                      int64_t rows, int64_t D, double eps, int act, int compute,
                      float* y, float* dx, float* dgamma, float* dbeta,
                      double* dgamma64, double* dbeta64) {
    return guarded([&] {
        const bool affine = gamma != nullptr;
        auto options = torch::nn::LayerNormOptions(std::vector<int64_t>{D}).eps(eps).elementwise_affine(affine);
        torch::nn::LayerNorm norm(options);
        norm->to(compute_type(compute));
        if (affine) {
            torch::NoGradGuard ng;
            norm->weight.copy_(wrap(gamma, {D}, compute));
            norm->bias.copy_(wrap(beta, {D}, compute));
        }
        auto xin = wrap(x, {rows, D}, compute).clone().requires_grad_(dy != nullptr);
        auto out = Nott::Activation::Details::apply(act_type(act), norm->forward(xin));
        store(out, y);
        if (dy != nullptr) {
            out.backward(wrap(dy, {rows, D}, compute));
            store(xin.grad(), dx);
            if (affine) {
                store(norm->weight.grad(), dgamma);
                store(norm->bias.grad(), dbeta);
                store_f64(norm->weight.grad(), dgamma64);
                store_f64(norm->bias.grad(), dbeta64);
            }
        }
    });
}

// Nott's RMSNorm module -> activation.  weight NULL -> learnable=false.
int ref_rmsnorm_act(const float* x, const float* weight, const float* dy,
                    int64_t rows, int64_t D, double eps, int act, int compute,
                    float* y, float* dx, float* dweight, double* dweight64) {
    return guarded([&] {
        namespace M = Nott::Block::Details::Transformer::Mamba;
        M::RMSNormOptions opt{};
        opt.eps = eps;
        opt.learnable = weight != nullptr;
        M::Detail::RMSNorm norm(D, opt);
        norm->to(compute_type(compute));
        if (weight != nullptr) {
            torch::NoGradGuard ng;
            norm->named_parameters()["weight"].copy_(wrap(weight, {D}, compute));
        }
        auto xin = wrap(x, {rows, D}, compute).clone().requires_grad_(dy != nullptr);
        auto out = Nott::Activation::Details::apply(act_type(act), norm->forward(xin));
        store(out, y);
        if (dy != nullptr) {
            out.backward(wrap(dy, {rows, D}, compute));
            store(xin.grad(), dx);
            if (weight != nullptr) {
                store(norm->named_parameters()["weight"].grad(), dweight);
                store_f64(norm->named_parameters()["weight"].grad(), dweight64);
            }
        }
    });
}

// apply(GeLU|SiLU) on a flat tensor.
int ref_act(const float* x, const float* dy, int64_t n, int act, int compute, float* y, float* dx) {
    return guarded([&] {
        auto xin = wrap(x, {n}, compute).clone().requires_grad_(dy != nullptr);
        auto out = Nott::Activation::Details::apply(act_type(act), xin);
        store(out, y);
        if (dy != nullptr) {
            out.backward(wrap(dy, {n}, compute));
            store(xin.grad(), dx);
        }
    });
}

// The fully connected layer as the reference builds and runs it: torch::nn::Linear(in, out).bias(b)
// (src/layer/details/fc.hpp:36-38), then Activation::Details::apply(layer.activation, .)
// (src/block/details/transformers/classic.hpp:446-452).  weight is [N, K], bias [N] or NULL.
int ref_fc_act(const float* x, const float* weight, const float* bias, int64_t M, int64_t N, int64_t K, int act, int compute,
               float* z, float* y) {
    return guarded([&] {
        torch::nn::Linear fc(torch::nn::LinearOptions(K, N).bias(bias != nullptr));
        fc->to(compute_type(compute));
        {
            torch::NoGradGuard ng;
            fc->weight.copy_(wrap(weight, {N, K}, compute));
            if (bias != nullptr) fc->bias.copy_(wrap(bias, {N}, compute));
        }
        auto pre = fc->forward(wrap(x, {M, K}, compute));
        store(pre, z);
        store(Nott::Activation::Details::apply(act_type(act), pre), y);
    });
}

// apply(SwiGLU) on one [rows, 2H] tensor; dinput is [rows, 2H].
int ref_swiglu(const float* input, const float* dy, int64_t rows, int64_t H, int compute,
               float* out, float* dinput) {
    return guarded([&] {
        auto xin = wrap(input, {rows, 2 * H}, compute).clone().requires_grad_(dy != nullptr);
        auto o = Nott::Activation::Details::apply(Nott::Activation::Type::SwiGLU, xin);
        store(o, out);
        if (dy != nullptr) {
            o.backward(wrap(dy, {rows, H}, compute));
            store(xin.grad(), dinput);
        }
    });
}

// Mamba's gated feed forward on separate tensors: up * silu(gate).
int ref_mamba_gate(const float* gate, const float* up, const float* dy, int64_t rows, int64_t H, int compute,
                   float* out, float* dgate, float* dup) {
    return guarded([&] {
        auto g = wrap(gate, {rows, H}, compute).clone().requires_grad_(dy != nullptr);
        auto u = wrap(up, {rows, H}, compute).clone().requires_grad_(dy != nullptr);
        auto o = u * torch::silu(g);
        store(o, out);
        if (dy != nullptr) {
            o.backward(wrap(dy, {rows, H}, compute));
            store(g.grad(), dgate);
            store(u.grad(), dup);
        }
    });
}

// EBT TokenEmbedding (discrete modality) gather; ids int64 as the reference requires.
// dout != NULL also returns the dense table gradient.
int ref_token_embedding(const float* table, const int64_t* ids, const float* dout,
                        int64_t tokens, int64_t vocab, int64_t D, int compute,
                        float* out, float* dtable) {
    return guarded([&] {
        namespace E = Nott::Block::Details::Transformer::EBT;
        E::ModalityOptions opt{};
        opt.type = E::ModalityType::Discrete;
        opt.vocab_size = vocab;
        opt.embed_dim = D;
        E::Detail::TokenEmbedding emb(opt);
        emb->to(compute_type(compute));
        auto weight = emb->named_parameters()["embedding.weight"];
        {
            torch::NoGradGuard ng;
            weight.copy_(wrap(table, {vocab, D}, compute));
        }
        auto idt = torch::from_blob(const_cast<int64_t*>(ids), {tokens}, torch::kInt64);
        auto o = emb->forward(idt);
        store(o, out);
        if (dout != nullptr) {
            o.backward(wrap(dout, {tokens, D}, compute));
            store(weight.grad(), dtable);
        }
    });
}

// The residual add in front of a norm, as the blocks write it:
//   `output = residual + attention; norm2_->forward(output)`  (classic.hpp:442-445, LayerNorm)
//   `output = residual + ...; norm2_->forward(output)`         (mamba.hpp:409-415, Nott's RMSNorm)
// Returns the sum, the normalised sum, and with dy/dsum the gradients of
// sum(y*dy) + sum(s*dsum): da (== db) and the parameter gradients.
int ref_add_norm(int rms, const float* a, const float* b, const float* gamma, const float* beta, const float* dy,
                 const float* dsum, int64_t rows, int64_t D, double eps, int compute,
                 float* sum_out, float* y, float* da, float* dgamma, float* dbeta) {
    return guarded([&] {
        namespace M = Nott::Block::Details::Transformer::Mamba;
        const auto dt = compute_type(compute);
        torch::nn::LayerNorm ln(torch::nn::LayerNormOptions(std::vector<int64_t>{D}).eps(eps));
        M::RMSNormOptions opt{};
        opt.eps = eps;
        M::Detail::RMSNorm rn(D, opt);
        ln->to(dt);
        rn->to(dt);
        {
            torch::NoGradGuard ng;
            if (rms) {
                rn->named_parameters()["weight"].copy_(wrap(gamma, {D}, compute));
            } else {
                ln->weight.copy_(wrap(gamma, {D}, compute));
                ln->bias.copy_(wrap(beta, {D}, compute));
            }
        }
        auto residual = wrap(a, {rows, D}, compute).clone().requires_grad_(dy != nullptr);
        auto attention = wrap(b, {rows, D}, compute).clone().requires_grad_(dy != nullptr);
        auto output = residual + attention;
        auto normed = rms ? rn->forward(output) : ln->forward(output);
        store(output, sum_out);
        store(normed, y);
        if (dy != nullptr) {
            auto loss = (normed * wrap(dy, {rows, D}, compute)).sum();
            if (dsum != nullptr) loss = loss + (output * wrap(dsum, {rows, D}, compute)).sum();
            loss.backward();
            store(residual.grad(), da);
            if (rms) {
                store(rn->named_parameters()["weight"].grad(), dgamma);
            } else {
                store(ln->weight.grad(), dgamma);
                store(ln->bias.grad(), dbeta);
            }
        }
    });
}

// BertEmbeddingImpl::forward (bert.hpp:155-194), dropout 0.  Tables are given in fp32; gradients of
// all three tables and of the LayerNorm parameters come back (type table: [type_vocab, D]).
int ref_bert_embedding(const float* word, const float* pos, const float* type, const float* gamma, const float* beta,
                       const int64_t* ids, const float* dy, int64_t B, int64_t S, int64_t vocab, int64_t max_pos,
                       int64_t type_vocab, int64_t D, int compute,
                       float* y, float* dword, float* dpos, float* dtype, float* dgamma, float* dbeta) {
    return guarded([&] {
        namespace Bt = Nott::Block::Details::Transformer::Bert;
        Bt::EmbeddingOptions opt{};
        opt.vocab_size = vocab;
        opt.type_vocab_size = type_vocab;
        opt.max_position_embeddings = max_pos;
        opt.dropout = 0.0;
        opt.use_token_type = type != nullptr;
        opt.use_position_embeddings = pos != nullptr;
        Bt::Detail::BertEmbedding emb(D, opt);
        emb->to(compute_type(compute));
        auto params = emb->named_parameters();
        {
            torch::NoGradGuard ng;
            params["word_embeddings.weight"].copy_(wrap(word, {vocab, D}, compute));
            if (pos) params["position_embeddings.weight"].copy_(wrap(pos, {max_pos, D}, compute));
            if (type) params["token_type_embeddings.weight"].copy_(wrap(type, {type_vocab, D}, compute));
            params["layer_norm.weight"].copy_(wrap(gamma, {D}, compute));
            params["layer_norm.bias"].copy_(wrap(beta, {D}, compute));
        }
        auto idt = torch::from_blob(const_cast<int64_t*>(ids), {B, S}, torch::kInt64);
        auto out = emb->forward(idt);
        store(out, y);
        if (dy != nullptr) {
            out.backward(wrap(dy, {B, S, D}, compute));
            store(params["word_embeddings.weight"].grad(), dword);
            if (pos) store(params["position_embeddings.weight"].grad(), dpos);
            if (type) store(params["token_type_embeddings.weight"].grad(), dtype);
            store(params["layer_norm.weight"].grad(), dgamma);
            store(params["layer_norm.bias"].grad(), dbeta);
        }
    });
}

// The other branch of BertEmbeddingImpl::forward (bert.hpp:164-171): an input that is not a Long tensor is taken
// as ready-made [B, S, D] embeddings; position and type rows are added and the sum is LayerNorm'ed.  dinput is
// the gradient of that input.
int ref_bert_embedding_from_embeddings(const float* input, const float* pos, const float* type, const float* gamma,
                                       const float* beta, const float* dy, int64_t B, int64_t S, int64_t max_pos,
                                       int64_t type_vocab, int64_t D, int compute,
                                       float* y, float* dinput, float* dpos, float* dtype, float* dgamma, float* dbeta) {
    return guarded([&] {
        namespace Bt = Nott::Block::Details::Transformer::Bert;
        Bt::EmbeddingOptions opt{};
        opt.vocab_size = 4;                               // a word table exists but is not used by this branch
        opt.type_vocab_size = type_vocab;
        opt.max_position_embeddings = max_pos;
        opt.dropout = 0.0;
        opt.use_token_type = type != nullptr;
        opt.use_position_embeddings = pos != nullptr;
        Bt::Detail::BertEmbedding emb(D, opt);
        emb->to(compute_type(compute));
        auto params = emb->named_parameters();
        {
            torch::NoGradGuard ng;
            if (pos) params["position_embeddings.weight"].copy_(wrap(pos, {max_pos, D}, compute));
            if (type) params["token_type_embeddings.weight"].copy_(wrap(type, {type_vocab, D}, compute));
            params["layer_norm.weight"].copy_(wrap(gamma, {D}, compute));
            params["layer_norm.bias"].copy_(wrap(beta, {D}, compute));
        }
        auto in = wrap(input, {B, S, D}, compute).clone().requires_grad_(dy != nullptr);
        auto out = emb->forward(in);
        store(out, y);
        if (dy != nullptr) {
            out.backward(wrap(dy, {B, S, D}, compute));
            store(in.grad(), dinput);
            if (pos) store(params["position_embeddings.weight"].grad(), dpos);
            if (type) store(params["token_type_embeddings.weight"].grad(), dtype);
            store(params["layer_norm.weight"].grad(), dgamma);
            store(params["layer_norm.bias"].grad(), dbeta);
        }
    });
}

// Times forward + autograd backward of LayerNorm->act (rms == 0) or Nott's
// RMSNorm->act (rms != 0) on seeded N(0,1) inputs that are built once; only the
// module calls are inside the clock.  Returns seconds per iteration (mean of
// `iters` after `warmup`), or a negative value on error.
double ref_time_norm_act(int rms, int64_t rows, int64_t D, double eps, int act, int compute,
                         int iters, int warmup) {
    double result = -1.0;
    guarded([&] {
        namespace M = Nott::Block::Details::Transformer::Mamba;
        torch::manual_seed(0);
        const auto dt = compute_type(compute);
        auto x = torch::randn({rows, D}).to(dt).requires_grad_(true);
        auto dy = torch::randn({rows, D}).to(dt);
        torch::nn::LayerNorm ln(torch::nn::LayerNormOptions(std::vector<int64_t>{D}).eps(eps));
        M::RMSNormOptions opt{};
        opt.eps = eps;
        M::Detail::RMSNorm rn(D, opt);
        ln->to(dt);
        rn->to(dt);
        auto once = [&] {
            auto h = rms ? rn->forward(x) : ln->forward(x);
            auto out = Nott::Activation::Details::apply(act_type(act), h);
            out.backward(dy);
            x.mutable_grad().reset();
            for (auto& p : (rms ? rn->parameters() : ln->parameters())) p.mutable_grad().reset();
        };
        for (int i = 0; i < warmup; ++i) once();
        const auto t0 = std::chrono::steady_clock::now();
        for (int i = 0; i < iters; ++i) once();
        const auto t1 = std::chrono::steady_clock::now();
        result = std::chrono::duration<double>(t1 - t0).count() / (iters > 0 ? iters : 1);
    });
    return result;
}

// ScaledDotProductKernelImpl::forward (src/attention/details/kernel.hpp:20-94) run with key = value =
// identity ([S, S], so head_dim == S): then scores == query exactly, and the module's output is its
// attention matrix itself,
//   attn = softmax(query / sqrt(S) [key padding -> -inf] [+ attn_mask] [causal -> -inf], dim -1).
// key_padding: [B, S] bytes (non-zero = padded) or NULL.  attn_mask: additive, mask_dims in {2, 3, 4}
// with shapes [T,S], [B,T,S], [B,H,T,S], or NULL.  With dattn, dquery (the gradient of
// sum(attn * dattn) with respect to query) comes back in dscores.
int ref_attention_softmax(const float* query, const uint8_t* key_padding, const float* attn_mask, int mask_dims,
                          const float* dattn, int64_t B, int64_t H, int64_t T, int64_t S, int causal, int compute,
                          float* attn, float* dscores) {
    return guarded([&] {
        namespace A = Nott::Attention;
        A::Details::ScaledDotProductKernel kernel(0.0, causal ? A::Variant::Causal : A::Variant::Full);
        const auto dt = compute_type(compute);
        auto q = wrap(query, {B, H, T, S}, compute).clone().requires_grad_(dattn != nullptr);
        auto eye = torch::eye(S, torch::TensorOptions().dtype(dt)).expand({B, H, S, S});
        torch::Tensor mask, padding;
        if (attn_mask != nullptr) {
            std::vector<int64_t> shape = mask_dims == 2 ? std::vector<int64_t>{T, S}
                                         : mask_dims == 3 ? std::vector<int64_t>{B, T, S} : std::vector<int64_t>{B, H, T, S};
            mask = wrap(attn_mask, shape, compute);
        }
        if (key_padding != nullptr)
            padding = torch::from_blob(const_cast<uint8_t*>(key_padding), {B, S}, torch::kUInt8).to(torch::kBool);
        auto out = kernel->forward(q, eye, eye, mask, padding);
        store(out, attn);
        if (dattn != nullptr) {
            (out * wrap(dattn, {B, H, T, S}, compute)).sum().backward();
            store(q.grad(), dscores);
        }
    });
}

// Attention probabilities followed by the reference's multiplicative-noise dropout
// (src/layer/details/dropout.hpp:32-51: eps = empty_like(input).normal_(1, sqrt(p/(1-p))), output = input * eps).
// The module draws eps from libtorch's default generator; seeding it with `seed` right before the module runs and
// again before an identical normal_ call here yields the very tensor the module used, which is returned as `noise`
// so that another implementation can be fed the same values.  dout is the gradient of the dropped probabilities.
int ref_attention_softmax_dropout(const float* query, const uint8_t* key_padding, const float* attn_mask, int mask_dims,
                                  const float* dout, int64_t B, int64_t H, int64_t T, int64_t S, int causal, double p,
                                  int64_t seed, int compute, float* attn, float* noise, float* out, float* dscores) {
    return guarded([&] {
        namespace A = Nott::Attention;
        namespace L = Nott::Layer::Details;
        A::Details::ScaledDotProductKernel kernel(0.0, causal ? A::Variant::Causal : A::Variant::Full);
        const auto dt = compute_type(compute);
        auto q = wrap(query, {B, H, T, S}, compute).clone().requires_grad_(dout != nullptr);
        auto eye = torch::eye(S, torch::TensorOptions().dtype(dt)).expand({B, H, S, S});
        torch::Tensor mask, padding;
        if (attn_mask != nullptr) {
            std::vector<int64_t> shape = mask_dims == 2 ? std::vector<int64_t>{T, S}
                                         : mask_dims == 3 ? std::vector<int64_t>{B, T, S} : std::vector<int64_t>{B, H, T, S};
            mask = wrap(attn_mask, shape, compute);
        }
        if (key_padding != nullptr)
            padding = torch::from_blob(const_cast<uint8_t*>(key_padding), {B, S}, torch::kUInt8).to(torch::kBool);
        auto probs = kernel->forward(q, eye, eye, mask, padding);
        store(probs, attn);
        L::HardDropoutOptions options;
        options.probability = p;
        L::HardDropout drop(options);
        drop->train();
        torch::manual_seed(static_cast<uint64_t>(seed));
        auto dropped = drop->forward(probs);
        store(dropped, out);
        torch::manual_seed(static_cast<uint64_t>(seed));
        auto eps = torch::empty_like(probs).normal_(1.0, std::sqrt(p / (1.0 - p)));
        store(eps, noise);
        if (!torch::equal(dropped.detach(), (probs * eps).detach())) throw std::runtime_error("the re-drawn noise is not the module's");
        if (dout != nullptr) {
            (dropped * wrap(dout, {B, H, T, S}, compute)).sum().backward();
            store(q.grad(), dscores);
        }
    });
}

}  // extern "C"
