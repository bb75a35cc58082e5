// nott_b200.hpp — libtorch host layer over libnott_b200.so.
//
// Drop-in counterparts of the pieces of Nott (MoonFlowww/Thot) that sit on the
// memory-bound row-op path, with the same names, constructor arguments,
// parameter names and exception types, so a block that holds the reference
// module can hold this one instead and existing checkpoints keep loading:
//
//   Nott::B200::LayerNorm   <- torch::nn::LayerNorm as the blocks build it
//                              (src/block/details/transformers/classic.hpp:399-404, options :54-57),
//                              optionally fused with the activation that follows it
//   Nott::B200::RMSNorm     <- Mamba::Detail::RMSNorm (src/block/details/transformers/mamba.hpp:110-150)
//   Nott::B200::BertEmbedding <- Bert::Detail::BertEmbedding (bert.hpp:116-204): gathers + LayerNorm in one pass
//   Nott::B200::Embedding   <- torch::nn::Embedding (bert.hpp:126-128, ebt.hpp:94-96)
//   LayerNorm/RMSNorm::forward_residual <- `output = residual + branch; norm(output)` in one pass
//                              (classic.hpp:442-445, bert.hpp:291-293, mamba.hpp:409-415)
//   Nott::B200::apply       <- Nott::Activation::Details::apply (src/activation/apply.hpp:24-57)
//   Nott::B200::silu_gate   <- `up * torch::silu(gate)` (mamba.hpp:443-446)
//   Nott::B200::RotaryTable / rotary  (no reference code; belongs between the head
//                              view and the attention kernel, src/attention/details/head.hpp:70-74)
//
// Every op is a torch::autograd::Function whose forward and backward call the
// extern "C" kernels on the current CUDA stream; outputs come from libtorch's
// caching allocator; nothing synchronises, so the ops can be captured in the
// CUDA graphs Nott records around a training step (src/core.hpp:3856-3879).
// There is no CPU path: a CPU tensor, an unsupported dtype or a missing library
// raises.  Under CUDA autocast the norms run in fp32, like libtorch's.
#pragma once

#include <ATen/autocast_mode.h>
#include <ATen/cuda/CUDAContext.h>
#include <ATen/cuda/CUDAEvent.h>
#include <torch/torch.h>

#include <cmath>
#include <cstdint>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "../../include/nott_b200.h"

namespace Nott::B200 {

// Same enumerators, same order as Nott::Activation::Type (src/activation/activation.hpp:6-21),
// so a value converts with a static_cast in either direction.
enum class ActivationType {
    Identity, ReLU, Sigmoid, Tanh, LeakyReLU, Softmax, SiLU, GeLU, GLU, SwiGLU, dSiLU, PSiLU, Mish, Swish,
};

namespace detail {

inline void check(int status, const char* what) {
    if (status == 0) return;
    const std::string msg = std::string(what) + ": " + nb2_last_error_string();
    if (status < 0) throw std::invalid_argument(msg);
    throw std::runtime_error(msg);
}

inline int dtype_code(const torch::Tensor& t, const char* what) {
    if (t.scalar_type() == torch::kFloat32) return NB2_F32;
    if (t.scalar_type() == torch::kBFloat16) return NB2_BF16;
    throw std::invalid_argument(std::string(what) + " supports float32 and bfloat16 tensors only.");
}

inline void require_cuda(const torch::Tensor& t, const char* what) {
    if (!t.defined()) throw std::invalid_argument(std::string(what) + " requires a defined input tensor.");
    if (!t.is_cuda()) throw std::invalid_argument(std::string(what) + " runs on CUDA tensors only (there is no CPU fallback).");
}

inline void* stream() { return at::cuda::getCurrentCUDAStream().stream(); }

inline const void* ptr_or_null(const torch::Tensor& t) { return t.defined() ? t.data_ptr() : nullptr; }

// which activation the norm kernels can fuse
inline int fused_act_code(ActivationType type) {
    switch (type) {
        case ActivationType::Identity: return NB2_ACT_NONE;
        case ActivationType::GeLU: return NB2_ACT_GELU;
        case ActivationType::SiLU:
        case ActivationType::Swish: return NB2_ACT_SILU;        // swish.hpp:12-17 is x * sigmoid(x)
        default: return -1;
    }
}

inline c10::optional<torch::Tensor> opt(const torch::Tensor& t) {
    return t.defined() ? c10::optional<torch::Tensor>(t) : c10::nullopt;
}

inline torch::Tensor param_like(const torch::Tensor& p, const torch::Tensor& x) {
    if (!p.defined()) return p;
    return p.scalar_type() == x.scalar_type() ? p.contiguous() : p.to(x.scalar_type()).contiguous();
}

}  // namespace detail

// ------------------------------------------------------- residual add + norm, one pass
// `output = residual + attention; norm2_->forward(output)` (classic.hpp:442-445, bert.hpp:291-293,
// mamba.hpp:409-415) as one autograd node with two outputs: the sum (the next residual) and its
// normalisation.  rms == false: LayerNorm (weight, bias); rms == true: RMSNorm (weight).
struct AddNormFunction : public torch::autograd::Function<AddNormFunction> {
    static torch::autograd::tensor_list forward(torch::autograd::AutogradContext* ctx, torch::Tensor a, torch::Tensor b,
                                                torch::Tensor weight, c10::optional<torch::Tensor> bias_opt, double eps,
                                                bool rms) {
        detail::require_cuda(a, "residual add + norm");
        if (!b.defined() || a.sizes() != b.sizes() || a.scalar_type() != b.scalar_type())
            throw std::invalid_argument("residual add + norm expects two tensors of the same shape and dtype.");
        if (!weight.defined()) throw std::invalid_argument("residual add + norm requires the norm's weight.");
        const auto D = a.size(-1);
        auto x = a.contiguous().view({-1, D}), r = b.contiguous().view({-1, D});
        const int code = detail::dtype_code(x, "residual add + norm");
        auto w = detail::param_like(weight, x);
        auto bias = detail::param_like(bias_opt.value_or(torch::Tensor()), x);
        if (!rms && !bias.defined()) throw std::invalid_argument("residual add + LayerNorm requires the bias.");
        const auto rows = x.size(0);
        auto sum = torch::empty_like(x), y = torch::empty_like(x);
        auto stats = torch::empty({2, rows}, x.options().dtype(torch::kFloat32));
        if (rms)
            detail::check(nb2_add_rmsnorm_fwd(x.data_ptr(), r.data_ptr(), w.data_ptr(), sum.data_ptr(), y.data_ptr(),
                                              stats[1].data_ptr<float>(), rows, D, eps, code, detail::stream()),
                          "nb2_add_rmsnorm_fwd");
        else
            detail::check(nb2_add_layernorm_fwd(x.data_ptr(), r.data_ptr(), w.data_ptr(), bias.data_ptr(), sum.data_ptr(),
                                                y.data_ptr(), stats[0].data_ptr<float>(), stats[1].data_ptr<float>(), rows,
                                                D, eps, code, detail::stream()),
                          "nb2_add_layernorm_fwd");
        ctx->save_for_backward({sum, w, stats});
        ctx->saved_data["rms"] = rms;
        ctx->saved_data["has_bias"] = bias.defined();
        ctx->saved_data["weight_dtype"] = (int64_t)weight.scalar_type();
        return {sum.view(a.sizes()), y.view(a.sizes())};
    }

    static torch::autograd::tensor_list backward(torch::autograd::AutogradContext* ctx,
                                                 torch::autograd::tensor_list grads) {
        auto saved = ctx->get_saved_variables();
        auto sum = saved[0], w = saved[1], stats = saved[2];
        const bool rms = ctx->saved_data["rms"].toBool();
        const auto rows = sum.size(0), D = sum.size(1);
        const int code = detail::dtype_code(sum, "residual add + norm backward");
        torch::Tensor dsum, dy;
        if (grads[0].defined()) dsum = grads[0].contiguous().view({rows, D}).to(sum.scalar_type());
        dy = grads[1].defined() ? grads[1].contiguous().view({rows, D}).to(sum.scalar_type()) : torch::zeros_like(sum);
        auto dx = torch::empty_like(sum);
        const auto ws = nb2_workspace_bytes(NB2_WS_NORM_BWD, rows, D, code);
        auto partials = torch::empty({(int64_t)(ws / 4)}, sum.options().dtype(torch::kFloat32));
        const int64_t ncols = rms ? D : 2 * D;
        auto sums = torch::zeros({ncols}, sum.options().dtype(torch::kFloat32));
        int64_t n = 0;
        if (rms)
            detail::check(nb2_add_rmsnorm_bwd(sum.data_ptr(), dy.data_ptr(), detail::ptr_or_null(dsum), w.data_ptr(),
                                              stats[1].data_ptr<float>(), dx.data_ptr(), partials.data_ptr<float>(), &n,
                                              rows, D, code, detail::stream()),
                          "nb2_add_rmsnorm_bwd");
        else
            detail::check(nb2_add_layernorm_bwd(sum.data_ptr(), dy.data_ptr(), detail::ptr_or_null(dsum), w.data_ptr(),
                                                stats[0].data_ptr<float>(), stats[1].data_ptr<float>(), dx.data_ptr(),
                                                partials.data_ptr<float>(), &n, rows, D, code, detail::stream()),
                          "nb2_add_layernorm_bwd");
        if (rows > 0)
            detail::check(nb2_colreduce_partials(partials.data_ptr<float>(), n, ncols, sums.data_ptr<float>(), detail::stream()),
                          "nb2_colreduce_partials");
        const auto wt = (torch::ScalarType)ctx->saved_data["weight_dtype"].toInt();
        auto shaped = dx.view(grads[1].defined() ? grads[1].sizes() : grads[0].sizes());
        torch::Tensor dw = rms ? sums.to(wt) : sums.narrow(0, 0, D).to(wt);
        torch::Tensor db = (!rms && ctx->saved_data["has_bias"].toBool()) ? sums.narrow(0, D, D).to(wt) : torch::Tensor();
        return {shaped, shaped, dw, db, torch::Tensor(), torch::Tensor()};
    }
};

// ------------------------------------------------------------------ LayerNorm (+act)
struct LayerNormActFunction : public torch::autograd::Function<LayerNormActFunction> {
    static torch::Tensor forward(torch::autograd::AutogradContext* ctx, torch::Tensor input,
                                 c10::optional<torch::Tensor> weight_opt, c10::optional<torch::Tensor> bias_opt,
                                 double eps, int64_t act) {
        detail::require_cuda(input, "LayerNorm");
        const torch::Tensor weight = weight_opt.value_or(torch::Tensor()), bias = bias_opt.value_or(torch::Tensor());
        const auto D = input.size(-1);
        auto x = input.contiguous().view({-1, D});
        const int code = detail::dtype_code(x, "LayerNorm");
        auto w = detail::param_like(weight, x), b = detail::param_like(bias, x);
        const auto rows = x.size(0);
        auto y = torch::empty_like(x);
        auto stats = torch::empty({2, rows}, x.options().dtype(torch::kFloat32));
        detail::check(nb2_layernorm_fwd(x.data_ptr(), detail::ptr_or_null(w), detail::ptr_or_null(b), y.data_ptr(),
                                        stats[0].data_ptr<float>(), stats[1].data_ptr<float>(), rows, D, eps, code,
                                        (int)act, detail::stream()),
                      "nb2_layernorm_fwd");
        ctx->save_for_backward({x, w, b, stats});
        ctx->saved_data["act"] = act;
        ctx->saved_data["weight_dtype"] = weight.defined() ? (int64_t)weight.scalar_type() : (int64_t)-1;
        return y.view(input.sizes());
    }

    static torch::autograd::tensor_list backward(torch::autograd::AutogradContext* ctx,
                                                 torch::autograd::tensor_list grads) {
        auto saved = ctx->get_saved_variables();
        auto x = saved[0], w = saved[1], b = saved[2], stats = saved[3];
        const auto act = ctx->saved_data["act"].toInt();
        const auto rows = x.size(0), D = x.size(1);
        const int code = detail::dtype_code(x, "LayerNorm backward");
        auto dy = grads[0].contiguous().view({rows, D});
        if (dy.scalar_type() != x.scalar_type()) dy = dy.to(x.scalar_type());
        auto dx = torch::empty_like(x);
        torch::Tensor dw, db;
        if (w.defined()) {
            const auto ws = nb2_workspace_bytes(NB2_WS_NORM_BWD, rows, D, code);
            auto partials = torch::empty({(int64_t)(ws / 4)}, x.options().dtype(torch::kFloat32));
            int64_t n = 0;
            detail::check(nb2_layernorm_bwd(x.data_ptr(), dy.data_ptr(), w.data_ptr(), detail::ptr_or_null(b),
                                            stats[0].data_ptr<float>(), stats[1].data_ptr<float>(), dx.data_ptr(),
                                            partials.data_ptr<float>(), &n, rows, D, code, (int)act, detail::stream()),
                          "nb2_layernorm_bwd");
            auto sums = torch::zeros({2, D}, x.options().dtype(torch::kFloat32));
            if (rows > 0)
                detail::check(nb2_colreduce_partials(partials.data_ptr<float>(), n, 2 * D, sums.data_ptr<float>(),
                                                     detail::stream()),
                              "nb2_colreduce_partials");
            const auto wt = (torch::ScalarType)ctx->saved_data["weight_dtype"].toInt();
            dw = sums[0].to(wt);
            if (b.defined()) db = sums[1].to(wt);
        } else {
            int64_t n = 0;
            detail::check(nb2_layernorm_bwd(x.data_ptr(), dy.data_ptr(), nullptr, nullptr, stats[0].data_ptr<float>(),
                                            stats[1].data_ptr<float>(), dx.data_ptr(), nullptr, &n, rows, D, code,
                                            (int)act, detail::stream()),
                          "nb2_layernorm_bwd");
        }
        return {dx.view(grads[0].sizes()), dw, db, torch::Tensor(), torch::Tensor()};
    }
};

struct LayerNormOptions {
    double eps{1e-5};                      // classic.hpp:54-57
    bool elementwise_affine{true};
    ActivationType activation{ActivationType::Identity};   // fused behind the norm (the layer.forward + apply seam, core.hpp:1927-1934)
};

class LayerNormImpl : public torch::nn::Module {
public:
    LayerNormImpl(std::int64_t normalized_dim, LayerNormOptions options = {})
        : dim_(normalized_dim), options_(options) {
        if (dim_ <= 0) throw std::invalid_argument("LayerNorm requires a positive normalized dimension.");
        if (detail::fused_act_code(options_.activation) < 0)
            throw std::invalid_argument("LayerNorm can fuse Identity, GeLU, SiLU or Swish only.");
        if (options_.elementwise_affine) {
            weight = register_parameter("weight", torch::ones({dim_}));     // same names as torch::nn::LayerNorm
            bias = register_parameter("bias", torch::zeros({dim_}));
        }
    }

    torch::Tensor forward(torch::Tensor input) {
        if (!input.defined()) throw std::invalid_argument("LayerNorm requires a defined input tensor.");
        if (input.dim() == 0 || input.size(-1) != dim_)
            throw std::invalid_argument("LayerNorm expected last dimension " + std::to_string(dim_) + ".");
        if (at::autocast::is_autocast_enabled(at::kCUDA) && input.scalar_type() != torch::kFloat32)
            input = input.to(torch::kFloat32);                            // libtorch's autocast policy for layer_norm
        return LayerNormActFunction::apply(std::move(input), detail::opt(weight), detail::opt(bias), options_.eps,
                                           (int64_t)detail::fused_act_code(options_.activation));
    }

    // (residual + branch, norm(residual + branch)) in one pass; the module must be affine and unfused
    std::pair<torch::Tensor, torch::Tensor> forward_residual(torch::Tensor residual, torch::Tensor branch) {
        if (!options_.elementwise_affine || options_.activation != ActivationType::Identity)
            throw std::invalid_argument("LayerNorm::forward_residual needs an affine module without a fused activation.");
        auto out = AddNormFunction::apply(std::move(residual), std::move(branch), weight, detail::opt(bias), options_.eps, false);
        return {out[0], out[1]};
    }

    torch::Tensor weight, bias;

private:
    std::int64_t dim_{};
    LayerNormOptions options_{};
};
TORCH_MODULE(LayerNorm);

// -------------------------------------------------------------------- RMSNorm (+act)
struct RMSNormActFunction : public torch::autograd::Function<RMSNormActFunction> {
    static torch::Tensor forward(torch::autograd::AutogradContext* ctx, torch::Tensor input,
                                 c10::optional<torch::Tensor> weight_opt, double eps, int64_t act) {
        detail::require_cuda(input, "RMSNorm");
        const torch::Tensor weight = weight_opt.value_or(torch::Tensor());
        const auto D = input.size(-1);
        auto x = input.contiguous().view({-1, D});
        const int code = detail::dtype_code(x, "RMSNorm");
        auto w = detail::param_like(weight, x);
        const auto rows = x.size(0);
        auto y = torch::empty_like(x);
        auto rstd = torch::empty({rows}, x.options().dtype(torch::kFloat32));
        detail::check(nb2_rmsnorm_fwd(x.data_ptr(), detail::ptr_or_null(w), y.data_ptr(), rstd.data_ptr<float>(), rows,
                                      D, eps, code, (int)act, detail::stream()),
                      "nb2_rmsnorm_fwd");
        ctx->save_for_backward({x, w, rstd});
        ctx->saved_data["act"] = act;
        ctx->saved_data["weight_dtype"] = weight.defined() ? (int64_t)weight.scalar_type() : (int64_t)-1;
        return y.view(input.sizes());
    }

    static torch::autograd::tensor_list backward(torch::autograd::AutogradContext* ctx,
                                                 torch::autograd::tensor_list grads) {
        auto saved = ctx->get_saved_variables();
        auto x = saved[0], w = saved[1], rstd = saved[2];
        const auto act = ctx->saved_data["act"].toInt();
        const auto rows = x.size(0), D = x.size(1);
        const int code = detail::dtype_code(x, "RMSNorm backward");
        auto dy = grads[0].contiguous().view({rows, D});
        if (dy.scalar_type() != x.scalar_type()) dy = dy.to(x.scalar_type());
        auto dx = torch::empty_like(x);
        torch::Tensor dw;
        int64_t n = 0;
        if (w.defined()) {
            const auto ws = nb2_workspace_bytes(NB2_WS_NORM_BWD, rows, D, code);
            auto partials = torch::empty({(int64_t)(ws / 4)}, x.options().dtype(torch::kFloat32));
            detail::check(nb2_rmsnorm_bwd(x.data_ptr(), dy.data_ptr(), w.data_ptr(), rstd.data_ptr<float>(),
                                          dx.data_ptr(), partials.data_ptr<float>(), &n, rows, D, code, (int)act,
                                          detail::stream()),
                          "nb2_rmsnorm_bwd");
            auto sums = torch::zeros({D}, x.options().dtype(torch::kFloat32));
            if (rows > 0)
                detail::check(nb2_colreduce_partials(partials.data_ptr<float>(), n, D, sums.data_ptr<float>(),
                                                     detail::stream()),
                              "nb2_colreduce_partials");
            dw = sums.to((torch::ScalarType)ctx->saved_data["weight_dtype"].toInt());
        } else {
            detail::check(nb2_rmsnorm_bwd(x.data_ptr(), dy.data_ptr(), nullptr, rstd.data_ptr<float>(), dx.data_ptr(),
                                          nullptr, &n, rows, D, code, (int)act, detail::stream()),
                          "nb2_rmsnorm_bwd");
        }
        return {dx.view(grads[0].sizes()), dw, torch::Tensor(), torch::Tensor()};
    }
};

struct RMSNormOptions {
    double eps{1e-6};                      // mamba.hpp:25-28
    bool learnable{true};
    ActivationType activation{ActivationType::Identity};
};

class RMSNormImpl : public torch::nn::Module {
public:
    RMSNormImpl(std::int64_t embed_dim, RMSNormOptions options) : embed_dim_(embed_dim), options_(options) {
        if (embed_dim_ <= 0) throw std::invalid_argument("RMSNorm requires a positive embedding dimension.");
        if (detail::fused_act_code(options_.activation) < 0)
            throw std::invalid_argument("RMSNorm can fuse Identity, GeLU, SiLU or Swish only.");
        if (options_.learnable) weight_ = register_parameter("weight", torch::ones({embed_dim_}));
    }

    torch::Tensor forward(torch::Tensor input) {
        if (!input.defined()) throw std::invalid_argument("RMSNorm requires a defined input tensor.");
        if (input.dim() == 0) throw std::invalid_argument("RMSNorm expects a tensor with at least one dimension.");
        if (input.size(-1) != embed_dim_)
            throw std::invalid_argument("RMSNorm expected last dimension " + std::to_string(embed_dim_) + ".");
        return RMSNormActFunction::apply(std::move(input), detail::opt(weight_), options_.eps,
                                         (int64_t)detail::fused_act_code(options_.activation));
    }

    std::pair<torch::Tensor, torch::Tensor> forward_residual(torch::Tensor residual, torch::Tensor branch) {
        if (!options_.learnable || options_.activation != ActivationType::Identity)
            throw std::invalid_argument("RMSNorm::forward_residual needs a learnable module without a fused activation.");
        auto out = AddNormFunction::apply(std::move(residual), std::move(branch), weight_, c10::nullopt, options_.eps, true);
        return {out[0], out[1]};
    }

private:
    std::int64_t embed_dim_{};
    RMSNormOptions options_{};
    torch::Tensor weight_{};
};
TORCH_MODULE(RMSNorm);

// ------------------------------------------------------------------------ activations
struct ActivationFunction : public torch::autograd::Function<ActivationFunction> {
    static torch::Tensor forward(torch::autograd::AutogradContext* ctx, torch::Tensor input, int64_t act) {
        detail::require_cuda(input, "activation");
        auto x = input.contiguous();
        auto y = torch::empty_like(x);
        detail::check(nb2_act_fwd(x.data_ptr(), y.data_ptr(), x.numel(), detail::dtype_code(x, "activation"), (int)act,
                                  detail::stream()),
                      "nb2_act_fwd");
        ctx->save_for_backward({x});
        ctx->saved_data["act"] = act;
        return y;
    }
    static torch::autograd::tensor_list backward(torch::autograd::AutogradContext* ctx,
                                                 torch::autograd::tensor_list grads) {
        auto x = ctx->get_saved_variables()[0];
        auto dy = grads[0].contiguous();
        auto dx = torch::empty_like(x);
        detail::check(nb2_act_bwd(x.data_ptr(), dy.data_ptr(), dx.data_ptr(), x.numel(),
                                  detail::dtype_code(x, "activation backward"), (int)ctx->saved_data["act"].toInt(),
                                  detail::stream()),
                      "nb2_act_bwd");
        return {dx, torch::Tensor()};
    }
};

// out = silu(a) * b on two [.., H] operands whose rows may be strided (unit column stride)
struct SiluGateFunction : public torch::autograd::Function<SiluGateFunction> {
    static torch::Tensor forward(torch::autograd::AutogradContext* ctx, torch::Tensor a, torch::Tensor b) {
        detail::require_cuda(a, "SiLU gate");
        if (a.dim() != 2 || b.dim() != 2 || a.sizes() != b.sizes() || a.stride(1) != 1 || b.stride(1) != 1)
            throw std::invalid_argument("SiLU gate expects two [rows, H] operands with unit column stride.");
        const auto rows = a.size(0), H = a.size(1);
        auto out = torch::empty({rows, H}, a.options());
        detail::check(nb2_silu_gate_fwd(a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0), out.data_ptr(), H, rows, H,
                                        detail::dtype_code(a, "SiLU gate"), detail::stream()),
                      "nb2_silu_gate_fwd");
        ctx->save_for_backward({a, b});
        return out;
    }
    static torch::autograd::tensor_list backward(torch::autograd::AutogradContext* ctx,
                                                 torch::autograd::tensor_list grads) {
        auto saved = ctx->get_saved_variables();
        auto a = saved[0], b = saved[1];
        const auto rows = a.size(0), H = a.size(1);
        auto dy = grads[0].contiguous();
        auto da = torch::empty({rows, H}, a.options()), db = torch::empty({rows, H}, a.options());
        detail::check(nb2_silu_gate_bwd(a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0), dy.data_ptr(), H,
                                        da.data_ptr(), H, db.data_ptr(), H, rows, H,
                                        detail::dtype_code(a, "SiLU gate backward"), detail::stream()),
                      "nb2_silu_gate_bwd");
        return {da, db};
    }
};

// Mamba's gated feed forward: up * silu(gate) (mamba.hpp:443-446)
inline torch::Tensor silu_gate(const torch::Tensor& gate, const torch::Tensor& up) {
    const auto H = gate.size(-1);
    auto out = SiluGateFunction::apply(gate.contiguous().view({-1, H}), up.contiguous().view({-1, H}));
    return out.view(gate.sizes());
}

// Nott::Activation::Details::apply for the activations on this path.  GeLU, SiLU, Swish and
// SwiGLU run the sm_100a kernels; Identity returns its input; every other type is not part of
// this path and raises (inside Nott, keep dispatching those to the reference's own functors).
inline torch::Tensor apply(ActivationType type, torch::Tensor input) {
    switch (type) {
        case ActivationType::Identity: return input;
        case ActivationType::GeLU: return ActivationFunction::apply(std::move(input), (int64_t)NB2_ACT_GELU);
        case ActivationType::SiLU:
        case ActivationType::Swish: return ActivationFunction::apply(std::move(input), (int64_t)NB2_ACT_SILU);
        case ActivationType::SwiGLU: {
            // swiglu.hpp:18-23: chunk(2, -1), silu(first) * second; scalars and odd widths follow the reference
            if (input.dim() == 0) return input;
            const auto last = input.size(-1);
            if (last < 2) return input;
            if (last % 2 != 0) throw std::invalid_argument("SwiGLU expects an even last dimension on the fused path.");
            auto flat = input.contiguous().view({-1, last});
            const auto H = last / 2;
            auto out = SiluGateFunction::apply(flat.narrow(1, 0, H), flat.narrow(1, H, H));
            auto shape = input.sizes().vec();
            shape.back() = H;
            return out.view(shape);
        }
        default:
            throw std::invalid_argument("Nott::B200::apply covers Identity, GeLU, SiLU, Swish and SwiGLU.");
    }
}

// ------------------------------------------------------------- fully connected (+act)
// torch::nn::Linear followed by the layer's activation (src/layer/details/fc.hpp:31-49 and the feed-forward loop,
// src/block/details/transformers/classic.hpp:446-452) as one autograd node.  bf16 CUDA tensors whose widths are
// multiples of 8 run the tcgen05 GEMM with the bias and the activation in its epilogue; any other dtype or width
// keeps libtorch's GEMM (as in the reference) and only the activation runs here.
struct LinearActFunction : public torch::autograd::Function<LinearActFunction> {
    // `training`: a backward will follow (decided by the caller: grad mode is always off inside a forward), so the
    // pre-activation is kept.
    static torch::Tensor forward(torch::autograd::AutogradContext* ctx, torch::Tensor input, torch::Tensor weight,
                                 c10::optional<torch::Tensor> bias_opt, int64_t act, bool training) {
        detail::require_cuda(input, "Linear");
        const auto K = input.size(-1), N = weight.size(0);
        if (weight.dim() != 2 || weight.size(1) != K) throw std::invalid_argument("Linear: weight must be [out_features, in_features].");
        auto x = input.contiguous().view({-1, K});
        auto w = detail::param_like(weight, x);
        torch::Tensor b = bias_opt.has_value() ? detail::param_like(*bias_opt, x) : torch::Tensor();
        const bool needs_grad = training;
        const bool tensor_core = x.scalar_type() == torch::kBFloat16 && N % 8 == 0 && K % 8 == 0;
        torch::Tensor y, z;
        if (tensor_core) {
            const auto M = x.size(0);
            y = torch::empty({M, N}, x.options());
            if (needs_grad && act != NB2_ACT_NONE) z = torch::empty({M, N}, x.options());
            auto ws = torch::empty({(int64_t)nb2_workspace_bytes(NB2_WS_LINEAR, 0, 0, NB2_BF16)}, x.options().dtype(torch::kUInt8));
            detail::check(nb2_linear_bias_act_fwd(x.data_ptr(), w.data_ptr(), detail::ptr_or_null(b), z.defined() ? z.data_ptr() : nullptr,
                                                  y.data_ptr(), M, N, K, NB2_BF16, (int)act, ws.data_ptr(), (size_t)ws.numel(),
                                                  detail::stream()),
                          "nb2_linear_bias_act_fwd");
        } else {
            z = torch::linear(x, w, b.defined() ? c10::optional<torch::Tensor>(b) : c10::nullopt);
            if (act == NB2_ACT_NONE) {
                y = z;
            } else {
                y = torch::empty_like(z);
                detail::check(nb2_act_fwd(z.data_ptr(), y.data_ptr(), z.numel(), detail::dtype_code(z, "Linear"), (int)act, detail::stream()),
                              "nb2_act_fwd");
            }
        }
        ctx->save_for_backward({x, w, z.defined() ? z : torch::Tensor()});
        ctx->saved_data["act"] = act;
        ctx->saved_data["has_bias"] = b.defined();
        auto shape = input.sizes().vec();
        shape.back() = N;
        return y.view(shape);
    }
    static torch::autograd::tensor_list backward(torch::autograd::AutogradContext* ctx, torch::autograd::tensor_list grads) {
        auto saved = ctx->get_saved_variables();
        auto x = saved[0], w = saved[1], z = saved[2];
        const auto act = ctx->saved_data["act"].toInt();
        const auto N = w.size(0);
        auto dy = grads[0].contiguous().view({-1, N}).to(x.scalar_type());
        torch::Tensor dz = dy;
        if (act != NB2_ACT_NONE) {
            dz = torch::empty_like(dy);
            detail::check(nb2_act_bwd(z.data_ptr(), dy.data_ptr(), dz.data_ptr(), dz.numel(), detail::dtype_code(dz, "Linear backward"),
                                      (int)act, detail::stream()),
                          "nb2_act_bwd");
        }
        auto dx = torch::matmul(dz, w);                         // the two backward GEMMs stay libtorch calls, as in the reference
        auto dw = torch::matmul(dz.t(), x);
        torch::Tensor db;
        if (ctx->saved_data["has_bias"].toBool()) db = dz.sum(0);
        auto shape = grads[0].sizes().vec();
        shape.back() = x.size(1);
        return {dx.view(shape), dw, db, torch::Tensor(), torch::Tensor()};
    }
};

struct LinearOptions {                 // FCOptions (fc.hpp:19-23) plus the activation the layer is registered with
    std::int64_t in_features{};
    std::int64_t out_features{};
    bool bias{true};
    ActivationType activation{ActivationType::Identity};
};

class LinearImpl : public torch::nn::Module {
public:
    explicit LinearImpl(LinearOptions options) : options_(options) {
        if (options_.in_features <= 0 || options_.out_features <= 0)
            throw std::invalid_argument("Fully connected layers require positive in/out features.");       // fc.hpp:33-35
        if (detail::fused_act_code(options_.activation) < 0)
            throw std::invalid_argument("Linear can fuse Identity, GeLU, SiLU or Swish only.");
        // torch::nn::Linear's own parameters, names and initialisation
        torch::nn::Linear init(torch::nn::LinearOptions(options_.in_features, options_.out_features).bias(options_.bias));
        weight = register_parameter("weight", init->weight.detach().clone());
        if (options_.bias) bias = register_parameter("bias", init->bias.detach().clone());
    }
    torch::Tensor forward(torch::Tensor input) {
        if (!input.defined()) throw std::invalid_argument("Linear requires a defined input tensor.");
        const bool training = torch::GradMode::is_enabled() && (input.requires_grad() || weight.requires_grad() || (bias.defined() && bias.requires_grad()));
        return LinearActFunction::apply(std::move(input), weight, detail::opt(bias), (int64_t)detail::fused_act_code(options_.activation), training);
    }
    torch::Tensor weight, bias;

private:
    LinearOptions options_{};
};
TORCH_MODULE(Linear);

// -------------------------------------------------------------------------- embedding
struct EmbeddingFunction : public torch::autograd::Function<EmbeddingFunction> {
    // `training`: a backward will follow (the caller decides: grad mode is always off inside a forward)
    static torch::Tensor forward(torch::autograd::AutogradContext* ctx, torch::Tensor weight, torch::Tensor ids, bool training = false) {
        detail::require_cuda(weight, "Embedding");
        if (ids.scalar_type() != torch::kInt64 && ids.scalar_type() != torch::kInt32)
            throw std::invalid_argument("Embedding expects int32 or int64 token ids.");
        auto w = weight.contiguous();
        auto flat = ids.contiguous().view({-1});
        const auto vocab = w.size(0), D = w.size(1);
        auto out = torch::empty({flat.size(0), D}, w.options());
        const int code = detail::dtype_code(w, "Embedding");
        const int icode = flat.scalar_type() == torch::kInt32 ? NB2_I32 : NB2_I64;
        // The backward's index (token runs per table row) depends on the ids alone: it is built here, on a
        // pool stream beside the gather, and joined before returning, so the backward is one kernel.
        torch::Tensor index;
        if (training && flat.size(0) > 0) {
            const auto ws = nb2_workspace_bytes(NB2_WS_EMBEDDING_BWD, flat.size(0), vocab, code);
            index = torch::empty({(int64_t)ws}, w.options().dtype(torch::kUInt8));
            auto cur = at::cuda::getCurrentCUDAStream();
            auto side = at::cuda::getStreamFromPool(false, cur.device_index());
            at::cuda::CUDAEvent fork, join;
            fork.record(cur);
            fork.block(side);
            detail::check(nb2_embedding_index(flat.data_ptr(), flat.size(0), vocab, icode, index.data_ptr(), ws, side.stream()),
                          "nb2_embedding_index");
            join.record(side);
            detail::check(nb2_embedding_fwd(w.data_ptr(), flat.data_ptr(), out.data_ptr(), flat.size(0), vocab, D, code, icode,
                                            nullptr, cur.stream()),
                          "nb2_embedding_fwd");
            join.block(cur);
        } else {
            detail::check(nb2_embedding_fwd(w.data_ptr(), flat.data_ptr(), out.data_ptr(), flat.size(0), vocab, D, code, icode,
                                            nullptr, detail::stream()),
                          "nb2_embedding_fwd");
        }
        ctx->save_for_backward({flat, index});
        ctx->saved_data["vocab"] = vocab;
        auto shape = ids.sizes().vec();
        shape.push_back(D);
        return out.view(shape);
    }
    static torch::autograd::tensor_list backward(torch::autograd::AutogradContext* ctx,
                                                 torch::autograd::tensor_list grads) {
        auto saved = ctx->get_saved_variables();
        auto flat = saved[0], index = saved[1];
        const auto vocab = ctx->saved_data["vocab"].toInt();
        const auto D = grads[0].size(-1);
        auto dout = grads[0].contiguous().view({-1, D});
        const int code = detail::dtype_code(dout, "Embedding backward");
        auto dtable = torch::empty({vocab, D}, dout.options());
        if (index.defined()) {
            detail::check(nb2_embedding_bwd_indexed(dout.data_ptr(), dtable.data_ptr(), flat.size(0), vocab, D, code, index.data_ptr(),
                                                    (size_t)index.numel(), detail::stream()),
                          "nb2_embedding_bwd_indexed");
        } else {
            const auto ws = nb2_workspace_bytes(NB2_WS_EMBEDDING_BWD, flat.size(0), vocab, code);
            auto scratch = torch::empty({(int64_t)ws}, dout.options().dtype(torch::kUInt8));
            detail::check(nb2_embedding_bwd(dout.data_ptr(), flat.data_ptr(), dtable.data_ptr(), flat.size(0), vocab, D, code,
                                            flat.scalar_type() == torch::kInt32 ? NB2_I32 : NB2_I64, scratch.data_ptr(), ws,
                                            detail::stream()),
                          "nb2_embedding_bwd");
        }
        return {dtable, torch::Tensor(), torch::Tensor()};
    }
};

class EmbeddingImpl : public torch::nn::Module {
public:
    EmbeddingImpl(std::int64_t num_embeddings, std::int64_t embedding_dim) {
        if (num_embeddings <= 0 || embedding_dim <= 0)
            throw std::invalid_argument("Embedding requires positive vocabulary and embedding sizes.");
        weight = register_parameter("weight", torch::randn({num_embeddings, embedding_dim}));   // N(0,1), as torch::nn::Embedding
    }
    torch::Tensor forward(const torch::Tensor& ids) {
        return EmbeddingFunction::apply(weight, ids, torch::GradMode::is_enabled() && weight.requires_grad());
    }
    torch::Tensor weight;
};
TORCH_MODULE(Embedding);

// ------------------------------------------------------------------- BERT embedding
// BertEmbeddingImpl (src/block/details/transformers/bert.hpp:116-204) as one forward kernel and one
// fused backward: word[ids] + position[arange(S)] + token_type[0], LayerNorm(eps 1e-12), dropout.
struct BertEmbeddingFunction : public torch::autograd::Function<BertEmbeddingFunction> {
    // `input` is either [batch, sequence] token ids (int32 or int64; the reference takes int64 only) or, as in
    // the reference's other branch (bert.hpp:164-171), ready-made [batch, sequence, D] embeddings.
    static torch::Tensor forward(torch::autograd::AutogradContext* ctx, torch::Tensor input, torch::Tensor word,
                                 c10::optional<torch::Tensor> pos_opt, c10::optional<torch::Tensor> type_opt,
                                 torch::Tensor gamma, torch::Tensor beta, double eps) {
        detail::require_cuda(gamma, "BERT embeddings");
        const bool from_ids = input.scalar_type() == torch::kInt64 || input.scalar_type() == torch::kInt32;
        if (from_ids && input.dim() != 2) throw std::invalid_argument("BERT embeddings expect [batch, sequence] token ids.");
        if (!from_ids && input.dim() != 3) throw std::invalid_argument("BERT embeddings expect [batch, sequence, embed_dim] embeddings.");
        if (from_ids && !word.defined()) throw std::invalid_argument("BERT embeddings received token ids but have no word table.");
        auto w = from_ids ? word.contiguous() : input.contiguous();
        detail::require_cuda(w, "BERT embeddings");
        const int code = detail::dtype_code(w, "BERT embeddings");
        auto pos = detail::param_like(pos_opt.value_or(torch::Tensor()), w);
        auto type = detail::param_like(type_opt.value_or(torch::Tensor()), w);
        auto g = detail::param_like(gamma, w), b = detail::param_like(beta, w);
        const auto B = input.size(0), S = input.size(1), D = w.size(-1);
        const auto vocab = from_ids ? w.size(0) : B * S;
        if (pos.defined() && pos.size(0) < S) throw std::invalid_argument("BERT embeddings: sequence longer than max_position_embeddings.");
        auto idc = from_ids ? input.contiguous() : torch::Tensor();
        auto y = torch::empty({B, S, D}, w.options());
        auto sum = torch::empty({B * S, D}, w.options());
        auto stats = torch::empty({2, B * S}, w.options().dtype(torch::kFloat32));
        detail::check(nb2_bert_embedding_ln_fwd(w.data_ptr(), detail::ptr_or_null(pos), detail::ptr_or_null(type),
                                                detail::ptr_or_null(idc), g.data_ptr(), b.data_ptr(), sum.data_ptr(), y.data_ptr(),
                                                stats[0].data_ptr<float>(), stats[1].data_ptr<float>(), B, S, vocab, D, eps, code,
                                                from_ids && idc.scalar_type() == torch::kInt32 ? NB2_I32 : NB2_I64, nullptr,
                                                detail::stream()),
                      "nb2_bert_embedding_ln_fwd");
        ctx->save_for_backward({sum, from_ids ? idc : torch::empty({0}, w.options().dtype(torch::kInt64)), g, stats});
        ctx->saved_data["from_ids"] = from_ids;
        ctx->saved_data["B"] = B;
        ctx->saved_data["S"] = S;
        ctx->saved_data["vocab"] = vocab;
        ctx->saved_data["pos_rows"] = pos.defined() ? pos.size(0) : (int64_t)0;
        ctx->saved_data["type_rows"] = type.defined() ? type.size(0) : (int64_t)0;
        return y;
    }
    static torch::autograd::tensor_list backward(torch::autograd::AutogradContext* ctx, torch::autograd::tensor_list grads) {
        auto saved = ctx->get_saved_variables();
        auto sum = saved[0], ids = saved[1], g = saved[2], stats = saved[3];
        const bool from_ids = ctx->saved_data["from_ids"].toBool();
        const auto B = ctx->saved_data["B"].toInt(), S = ctx->saved_data["S"].toInt(), D = sum.size(1);
        const auto vocab = ctx->saved_data["vocab"].toInt(), pos_rows = ctx->saved_data["pos_rows"].toInt(),
                   type_rows = ctx->saved_data["type_rows"].toInt();
        const int code = detail::dtype_code(sum, "BERT embeddings backward");
        auto dy = grads[0].contiguous().to(sum.scalar_type());
        auto dsum = torch::empty_like(sum);
        torch::Tensor dword, dpos, dtype;
        if (from_ids) dword = torch::empty({vocab, D}, sum.options());
        if (pos_rows > 0) dpos = torch::empty({pos_rows, D}, sum.options());
        if (type_rows > 0) dtype = torch::zeros({type_rows, D}, sum.options());       // rows other than 0 get no gradient
        auto sums = torch::empty({2, D}, sum.options().dtype(torch::kFloat32));
        const auto ws = nb2_workspace_bytes(NB2_WS_BERT_EMBEDDING_BWD, (B << 32) | S, (vocab << 32) | D, code);
        auto scratch = torch::empty({(int64_t)ws}, sum.options().dtype(torch::kUInt8));
        detail::check(nb2_bert_embedding_ln_bwd(sum.data_ptr(), dy.data_ptr(), from_ids ? ids.data_ptr() : nullptr, g.data_ptr(),
                                                stats[0].data_ptr<float>(), stats[1].data_ptr<float>(), dsum.data_ptr(),
                                                dword.defined() ? dword.data_ptr() : nullptr,
                                                dpos.defined() ? dpos.data_ptr() : nullptr, pos_rows,
                                                type_rows > 0 ? dtype.data_ptr() : nullptr, sums.data_ptr<float>(), B, S, vocab, D,
                                                code, from_ids && ids.scalar_type() == torch::kInt32 ? NB2_I32 : NB2_I64,
                                                scratch.data_ptr(), ws, detail::stream()),
                      "nb2_bert_embedding_ln_bwd");
        // ids carry no gradient; ready-made embeddings receive dsum
        return {from_ids ? torch::Tensor() : dsum.view({B, S, D}), dword, dpos, dtype, sums[0].to(g.scalar_type()),
                sums[1].to(g.scalar_type()), torch::Tensor()};
    }
};

struct BertEmbeddingOptions {            // bert.hpp:50-57
    std::int64_t vocab_size{30522};
    std::int64_t type_vocab_size{2};
    std::int64_t max_position_embeddings{512};
    double dropout{0.1};
    bool use_token_type{true};
    bool use_position_embeddings{true};
};

class BertEmbeddingImpl : public torch::nn::Module {
public:
    BertEmbeddingImpl(std::int64_t embed_dim, BertEmbeddingOptions options) : embed_dim_(embed_dim), options_(options) {
        if (embed_dim_ <= 0) throw std::invalid_argument("BERT embeddings require a positive embedding dimension.");
        if (options_.vocab_size <= 0) throw std::invalid_argument("BERT embeddings on this path require a vocabulary.");
        // same submodule and parameter names as the reference: word_embeddings.weight, ..., layer_norm.bias
        word_embeddings_ = register_module("word_embeddings", Embedding(options_.vocab_size, embed_dim_));
        if (options_.use_token_type && options_.type_vocab_size > 0)
            token_type_embeddings_ = register_module("token_type_embeddings", Embedding(options_.type_vocab_size, embed_dim_));
        if (options_.use_position_embeddings && options_.max_position_embeddings > 0)
            position_embeddings_ = register_module("position_embeddings", Embedding(options_.max_position_embeddings, embed_dim_));
        LayerNormOptions norm;
        norm.eps = 1e-12;                                                     // hard-coded in the reference (bert.hpp:143-146)
        layer_norm_ = register_module("layer_norm", LayerNorm(embed_dim_, norm));
        if (options_.dropout > 0.0) dropout_ = register_module("dropout", torch::nn::Dropout(torch::nn::DropoutOptions(options_.dropout)));
    }

    torch::Tensor forward(torch::Tensor input) {
        if (!input.defined()) return input;
        const bool ids = input.scalar_type() == torch::kInt64 || input.scalar_type() == torch::kInt32;
        if (!ids && input.size(-1) != embed_dim_)          // the reference's own check and message (bert.hpp:166-170)
            throw std::invalid_argument("BERT embeddings expected last dimension " + std::to_string(embed_dim_) +
                                        " but received " + std::to_string(input.size(-1)) + ".");
        torch::Tensor out = BertEmbeddingFunction::apply(
            std::move(input), word_embeddings_->weight,
            position_embeddings_ ? detail::opt(position_embeddings_->weight) : c10::nullopt,
            token_type_embeddings_ ? detail::opt(token_type_embeddings_->weight) : c10::nullopt, layer_norm_->weight,
            layer_norm_->bias, 1e-12);
        if (dropout_) out = dropout_->forward(out);
        return out;
    }

private:
    std::int64_t embed_dim_{};
    BertEmbeddingOptions options_{};
    Embedding word_embeddings_{nullptr}, token_type_embeddings_{nullptr}, position_embeddings_{nullptr};
    LayerNorm layer_norm_{nullptr};
    torch::nn::Dropout dropout_{nullptr};
};
TORCH_MODULE(BertEmbedding);

// ----------------------------------------------------------------------------- rotary
// cos/sin of angle(s, i) = pos[s] * theta^(-2i/hd), built once and shared by q, k and the backward
class RotaryTable {
public:
    RotaryTable(std::int64_t seq_len, std::int64_t head_dim, double theta, const torch::Device& device,
                const torch::Tensor& positions = {})
        : seq_len_(seq_len), head_dim_(head_dim) {
        if (head_dim <= 0 || head_dim % 2 != 0) throw std::invalid_argument("Rotary embedding requires an even head dimension.");
        table_ = torch::empty({seq_len, head_dim / 2, 2}, torch::TensorOptions().dtype(torch::kFloat32).device(device));
        torch::Tensor pos;
        if (positions.defined()) pos = positions.to(device, torch::kInt32).contiguous();
        detail::check(nb2_rope_table(table_.data_ptr<float>(), pos.defined() ? pos.data_ptr<int32_t>() : nullptr, seq_len,
                                     head_dim, theta, detail::stream()),
                      "nb2_rope_table");
    }
    const torch::Tensor& table() const { return table_; }
    std::int64_t seq_len() const { return seq_len_; }
    std::int64_t head_dim() const { return head_dim_; }

private:
    std::int64_t seq_len_, head_dim_;
    torch::Tensor table_;
};

// ------------------------------------------------------- attention probabilities, one pass
// attn = softmax(scores * scale [key padding -> -inf] [+ mask] [causal -> -inf]) for scores
// [B, H, T, S]: the steps between the two matmuls of ScaledDotProductKernelImpl::forward
// (src/attention/details/kernel.hpp:33-93).  `mask` is additive and already of rank 2, 3 or 4.
struct AttentionSoftmaxFunction : public torch::autograd::Function<AttentionSoftmaxFunction> {
    // `noise`: optional multiplicative dropout noise of the scores' shape (a keep mask over 1-p for
    // torch::nn::Dropout, kernel.hpp:94; N(1, sqrt(p/(1-p))) for the noise module, dropout.hpp:41-43).  With it the
    // result is attn * noise, formed in the same pass.
    static torch::Tensor forward(torch::autograd::AutogradContext* ctx, torch::Tensor scores, c10::optional<torch::Tensor> mask,
                                 c10::optional<torch::Tensor> key_padding, double scale, bool causal,
                                 c10::optional<torch::Tensor> noise_opt = c10::nullopt) {
        detail::require_cuda(scores, "Attention softmax");
        if (scores.dim() != 4) throw std::invalid_argument("Attention softmax expects scores of shape (batch, heads, target, source).");
        auto x = scores.contiguous();
        const auto B = x.size(0), H = x.size(1), T = x.size(2), S = x.size(3);
        torch::Tensor m, kp;
        int64_t sb = 0, sh = 0;
        if (mask.has_value() && mask->defined() && mask->numel() > 0) {
            m = mask->to(x.scalar_type()).contiguous();
            if (m.dim() == 2) {
                if (m.size(0) != T || m.size(1) != S) throw std::invalid_argument("Attention mask dimensions mismatch: a 2D mask must be (target, source).");
            } else if (m.dim() == 3) {
                if (m.size(1) != T || m.size(2) != S || (m.size(0) != B && m.size(0) != B * H))
                    throw std::invalid_argument("Attention mask dimensions mismatch: a 3D mask must be (batch or batch*heads, target, source).");
                if (m.size(0) == B && H != 1) sb = T * S; else { sb = H * T * S; sh = T * S; }
            } else if (m.dim() == 4) {
                if (m.size(0) != B || m.size(1) != H || m.size(2) != T || m.size(3) != S)
                    throw std::invalid_argument("Attention mask dimensions mismatch: a 4D mask must be (batch, heads, target, source).");
                sb = H * T * S; sh = T * S;
            } else {
                throw std::invalid_argument("Unsupported attention mask dimensionality: " + std::to_string(m.dim()));
            }
        }
        if (key_padding.has_value() && key_padding->defined() && key_padding->numel() > 0) {
            kp = key_padding->to(torch::kBool).to(torch::kUInt8).contiguous();
            if (kp.dim() != 2 || kp.size(0) != B || kp.size(1) != S)
                throw std::invalid_argument("Key padding mask must be (batch, source).");
        }
        const int code = detail::dtype_code(x, "Attention softmax");
        auto attn = torch::empty_like(x);
        ctx->saved_data["scale"] = scale;
        if (noise_opt.has_value() && noise_opt->defined()) {
            auto noise = noise_opt->to(x.scalar_type()).contiguous();
            if (noise.sizes() != x.sizes()) throw std::invalid_argument("Attention dropout noise must have the shape of the scores.");
            auto out = torch::empty_like(x);
            detail::check(nb2_attention_softmax_dropout_fwd(x.data_ptr(), kp.defined() ? kp.data_ptr<uint8_t>() : nullptr,
                                                            detail::ptr_or_null(m), sb, sh, noise.data_ptr(), attn.data_ptr(),
                                                            out.data_ptr(), B, H, T, S, scale, causal ? 1 : 0, code, detail::stream()),
                          "nb2_attention_softmax_dropout_fwd");
            ctx->save_for_backward({attn, noise});
            return out;
        }
        detail::check(nb2_attention_softmax_fwd(x.data_ptr(), kp.defined() ? kp.data_ptr<uint8_t>() : nullptr, detail::ptr_or_null(m),
                                                sb, sh, attn.data_ptr(), B, H, T, S, scale, causal ? 1 : 0, code, detail::stream()),
                      "nb2_attention_softmax_fwd");
        ctx->save_for_backward({attn});
        return attn;
    }
    static torch::autograd::tensor_list backward(torch::autograd::AutogradContext* ctx, torch::autograd::tensor_list grads) {
        auto saved = ctx->get_saved_variables();
        auto attn = saved[0];
        auto dattn = grads[0].contiguous();
        auto ds = torch::empty_like(attn);
        const auto S = attn.size(-1);
        const auto rows = S > 0 ? attn.numel() / S : 0;
        const double scale = ctx->saved_data["scale"].toDouble();
        const int code = detail::dtype_code(attn, "Attention softmax backward");
        if (saved.size() > 1)
            detail::check(nb2_attention_softmax_dropout_bwd(attn.data_ptr(), saved[1].data_ptr(), dattn.data_ptr(), ds.data_ptr(), rows, S,
                                                            scale, code, detail::stream()),
                          "nb2_attention_softmax_dropout_bwd");
        else
            detail::check(nb2_attention_softmax_bwd(attn.data_ptr(), dattn.data_ptr(), ds.data_ptr(), rows, S, scale, code, detail::stream()),
                          "nb2_attention_softmax_bwd");
        return {ds, torch::Tensor(), torch::Tensor(), torch::Tensor(), torch::Tensor(), torch::Tensor()};
    }
};

enum class AttentionVariant { Full, Causal };   // ::Nott::Attention::Variant (src/attention/attention.hpp:9-12)

// Drop-in for Nott::Attention::Details::ScaledDotProductKernel (kernel.hpp:13-103): same constructor
// arguments and forward signature; the two matmuls stay libtorch calls, everything between them -- the
// dropout on the probabilities included -- is the single kernel above.  In training with p > 0 the keep mask
// is drawn with libtorch (bernoulli_(1-p) / (1-p): the distribution of torch::nn::Dropout, from libtorch's
// generator, though not the same draws as its fused dropout kernel) and handed to the kernel as noise.
class ScaledDotProductKernelImpl : public torch::nn::Module {
public:
    explicit ScaledDotProductKernelImpl(double dropout = 0.0, AttentionVariant variant = AttentionVariant::Full)
        : variant_(variant), p_(dropout),
          dropout_(register_module("dropout", torch::nn::Dropout(torch::nn::DropoutOptions(dropout)))) {}

    torch::Tensor forward(const torch::Tensor& query, const torch::Tensor& key, const torch::Tensor& value,
                          const torch::Tensor& attn_mask = {}, const torch::Tensor& key_padding_mask = {}) {
        auto scores = torch::matmul(query, key.transpose(-2, -1));
        const auto head_dim = query.size(-1);
        const double scale = head_dim > 0 ? 1.0 / std::sqrt(static_cast<double>(head_dim)) : 1.0;
        c10::optional<torch::Tensor> noise;
        if (is_training() && p_ > 0.0) noise = torch::empty_like(scores).bernoulli_(1.0 - p_).div_(1.0 - p_);
        auto attn = AttentionSoftmaxFunction::apply(scores, detail::opt(attn_mask), detail::opt(key_padding_mask), scale,
                                                    variant_ == AttentionVariant::Causal, noise);
        return torch::matmul(attn, value);
    }

    // the same with the noise supplied by the caller (reproducible dropout; the multiplicative-noise module)
    torch::Tensor forward_with_noise(const torch::Tensor& query, const torch::Tensor& key, const torch::Tensor& value,
                                     const torch::Tensor& noise, const torch::Tensor& attn_mask = {},
                                     const torch::Tensor& key_padding_mask = {}) {
        auto scores = torch::matmul(query, key.transpose(-2, -1));
        const auto head_dim = query.size(-1);
        const double scale = head_dim > 0 ? 1.0 / std::sqrt(static_cast<double>(head_dim)) : 1.0;
        auto attn = AttentionSoftmaxFunction::apply(scores, detail::opt(attn_mask), detail::opt(key_padding_mask), scale,
                                                    variant_ == AttentionVariant::Causal, detail::opt(noise));
        return torch::matmul(attn, value);
    }

private:
    AttentionVariant variant_{AttentionVariant::Full};
    double p_{0.0};
    torch::nn::Dropout dropout_{nullptr};
};
TORCH_MODULE(ScaledDotProductKernel);


// ------------------------------------------------------------- row-sharded training step
// One process per GPU, rows (batch x sequence) split over the ranks: the reference itself runs on one device
// (src/core.hpp:1706-1708) and consumes parameter gradients only in the optimizer step (src/core.hpp:3811-3820).
// Communicator wraps nb2_comm (the sum over ranks of the fp32 parameter gradients: NCCL allreduce on a side stream,
// or peer stores over NVLink fused into the partial reduce); ShardedNormStep wraps nb2_step (forward, backward,
// partial reduce and exchange of one norm layer in one call).  Status codes become exceptions as everywhere here;
// a failed or timed-out exchange is a std::runtime_error.
class Communicator {
public:
    static std::vector<uint8_t> make_id() {                 // rank 0; the other ranks receive it over any host channel
        std::vector<uint8_t> id(NB2_COMM_ID_BYTES);
        detail::check(nb2_comm_unique_id(id.data()), "nb2_comm_unique_id");
        return id;
    }
    Communicator(const std::vector<uint8_t>& id, int rank, int world, int exchange = NB2_EXCHANGE_NCCL, int64_t max_cols = 2 * 8192) {
        if (world > 1 && id.size() != NB2_COMM_ID_BYTES) throw std::invalid_argument("Communicator: the id must have NB2_COMM_ID_BYTES bytes.");
        detail::check(nb2_comm_create(&comm_, world > 1 ? id.data() : nullptr, rank, world, exchange, max_cols), "nb2_comm_create");
    }
    Communicator(const Communicator&) = delete;
    Communicator& operator=(const Communicator&) = delete;
    ~Communicator() { nb2_comm_destroy(comm_); }
    // blocks the host until the exchange started last has finished; throws (after aborting the communicator) on an
    // asynchronous error or when `timeout_s` passes
    void wait(double timeout_s) {
        const int rc = nb2_comm_wait(comm_, timeout_s);
        if (rc != 0) throw std::runtime_error(std::string("gradient exchange: ") + nb2_last_error_string());
    }
    nb2_comm* get() const { return comm_; }

private:
    nb2_comm* comm_{nullptr};
};

class ShardedNormStep {
public:
    // `comm` may be null (single GPU).  rms: RMSNorm (weight only), else LayerNorm (weight, bias).
    ShardedNormStep(std::shared_ptr<Communicator> comm, bool rms, int64_t rows, int64_t D, torch::ScalarType dtype,
                    ActivationType activation, double eps)
        : comm_(std::move(comm)), rms_(rms), rows_(rows), D_(D) {
        const int act = detail::fused_act_code(activation);
        if (act < 0) throw std::invalid_argument("ShardedNormStep can fuse Identity, GeLU, SiLU or Swish only.");
        if (dtype != torch::kFloat32 && dtype != torch::kBFloat16) throw std::invalid_argument("ShardedNormStep supports float32 and bfloat16.");
        detail::check(nb2_step_create(&step_, comm_ ? comm_->get() : nullptr, rms ? NB2_NORM_RMS : NB2_NORM_LAYER, rows, D,
                                      dtype == torch::kFloat32 ? NB2_F32 : NB2_BF16, act, eps),
                      "nb2_step_create");
    }
    ShardedNormStep(const ShardedNormStep&) = delete;
    ShardedNormStep& operator=(const ShardedNormStep&) = delete;
    ~ShardedNormStep() { nb2_step_destroy(step_); }

    // y, dx: this rank's [rows, D] outputs; grads: [2*D] (LayerNorm: dgamma | dbeta) or [D] fp32, complete after the
    // next run() or finish() in stream order: pass two buffers alternately.
    void run(const torch::Tensor& x, const torch::Tensor& dy, const torch::Tensor& weight, const torch::Tensor& bias,
             torch::Tensor& y, torch::Tensor& dx, torch::Tensor& grads) {
        detail::require_cuda(x, "ShardedNormStep");
        if (x.dim() != 2 || x.size(0) != rows_ || x.size(1) != D_ || !x.is_contiguous() || !dy.is_contiguous() || dy.sizes() != x.sizes())
            throw std::invalid_argument("ShardedNormStep expects contiguous [rows, D] activations of the size it was built for.");
        if (grads.scalar_type() != torch::kFloat32 || grads.numel() != (rms_ ? 1 : 2) * D_ || !grads.is_contiguous())
            throw std::invalid_argument("ShardedNormStep expects a contiguous fp32 gradient buffer of (rms ? 1 : 2) * D elements.");
        detail::check(nb2_step_run(step_, x.data_ptr(), dy.data_ptr(), weight.data_ptr(), rms_ ? nullptr : detail::ptr_or_null(bias),
                                   y.data_ptr(), dx.data_ptr(), grads.data_ptr<float>(), detail::stream()),
                      "nb2_step_run");
    }
    void finish() { detail::check(nb2_step_finish(step_, detail::stream()), "nb2_step_finish"); }

private:
    std::shared_ptr<Communicator> comm_;
    nb2_step* step_{nullptr};
    bool rms_;
    int64_t rows_, D_;
};

struct RotaryFunction : public torch::autograd::Function<RotaryFunction> {
    static torch::Tensor forward(torch::autograd::AutogradContext* ctx, torch::Tensor x, torch::Tensor table) {
        detail::require_cuda(x, "rotary");
        if (x.dim() != 4 || x.size(1) != table.size(0) || x.size(3) != 2 * table.size(1))
            throw std::invalid_argument("rotary expects x[B, S, H, hd] and a table built for (S, hd).");
        auto xc = x.contiguous();
        auto out = torch::empty_like(xc);
        detail::check(nb2_rope_apply(xc.data_ptr(), table.data_ptr<float>(), out.data_ptr(), xc.size(0), xc.size(1),
                                     xc.size(2), xc.size(3), detail::dtype_code(xc, "rotary"), 0, detail::stream()),
                      "nb2_rope_apply");
        ctx->save_for_backward({table});
        return out;
    }
    static torch::autograd::tensor_list backward(torch::autograd::AutogradContext* ctx,
                                                 torch::autograd::tensor_list grads) {
        auto table = ctx->get_saved_variables()[0];
        auto dy = grads[0].contiguous();
        auto dx = torch::empty_like(dy);
        detail::check(nb2_rope_apply(dy.data_ptr(), table.data_ptr<float>(), dx.data_ptr(), dy.size(0), dy.size(1),
                                     dy.size(2), dy.size(3), detail::dtype_code(dy, "rotary backward"), 1,
                                     detail::stream()),
                      "nb2_rope_apply");
        return {dx, torch::Tensor()};
    }
};

inline torch::Tensor rotary(const torch::Tensor& x, const RotaryTable& table) {
    return RotaryFunction::apply(x, table.table());
}

}  // namespace Nott::B200
