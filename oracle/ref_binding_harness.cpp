// TEST INFRASTRUCTURE, NOT PRODUCT CODE.
//
// The reference's own layer binding driving this library's drop-in modules.
// Nott::Model keeps every layer as a RegisteredLayer (src/layer/registry.hpp:33-184): a type-erased
// ForwardBinding {invoke, context} plus the activation that follows the layer, and runs
//     auto out = layer.forward(std::move(tensor));
//     tensor   = Activation::Details::apply(layer.activation, std::move(out));
// for each of them (src/core.hpp:1927-1934; the same pair in src/block/details/blocks/sequential.hpp:31-39).
// This harness compiles registry.hpp, activation.hpp, apply.hpp and common/local.hpp where they lie in
// the reference checkout (never copied), next to thot_b200/host/nott_b200.hpp, and runs that pair
//   (a) with a Nott::B200::LayerNorm bound through RegisteredLayer::bind_module_forward, GeLU fused into
//       the module (LayerNormOptions::activation) and layer.activation = Identity, on a CUDA tensor;
//   (b) through a COPY of that RegisteredLayer, and through a layer bound with bind_inline_forward (a
//       trivially copyable functor kept in the layer's inline context, which the copy constructor has
//       to re-point, registry.hpp:157-168), copied and moved;
//   (c) with the unfused reference pair: torch::nn::LayerNorm bound the same way, layer.activation =
//       GeLU applied by the reference's apply(), on CPU, in fp32 and in fp64;
// each followed by backward through autograd from the same upstream gradient.  Outputs go back as raw
// host buffers so a Python test can compare them.  Built by oracle/build_ref.py into
// oracle/_ref/libnott_binding.so (needs the reference checkout; links libnott_b200.so).
#include <torch/torch.h>

#include <cstdint>
#include <cstring>
#include <string>

#include "src/activation/activation.hpp"
#include "src/activation/apply.hpp"
#include "src/common/local.hpp"
#include "src/layer/registry.hpp"

#include "thot_b200/host/nott_b200.hpp"

namespace {

thread_local std::string g_error;

using Nott::Layer::Details::RegisteredLayer;

// the loop body of src/core.hpp:1927-1934 for one layer
torch::Tensor run_layer(const RegisteredLayer& layer, torch::Tensor tensor) {
    auto module_output = layer.forward(std::move(tensor));
    return Nott::Activation::Details::apply(layer.activation, std::move(module_output));
}

// a trivially copyable functor (one pointer) for bind_inline_forward
struct CallB200LayerNorm {
    Nott::B200::LayerNormImpl* module;
    torch::Tensor operator()(torch::Tensor input) const { return module->forward(std::move(input)); }
};

void copy_out(const torch::Tensor& t, float* dst) {
    if (dst == nullptr) return;
    auto c = t.detach().to(torch::kCPU, torch::kFloat32).contiguous();
    std::memcpy(dst, c.data_ptr<float>(), sizeof(float) * (size_t)c.numel());
}

}  // namespace

extern "C" {

const char* refbind_last_error() { return g_error.c_str(); }

// which: 0 = B200 module bound with bind_module_forward, 1 = a copy of that RegisteredLayer,
//        2 = bind_inline_forward, then copied and moved, 3 = reference pair on CPU in fp32,
//        4 = reference pair on CPU in fp64.
// x, dy: [rows, D] fp32 host; gamma, beta: [D].  Outputs (host fp32, any may be NULL): y, dx [rows, D], dgamma, dbeta [D].
int refbind_layernorm_gelu(int which, const float* x, const float* dy, const float* gamma, const float* beta,
                           int64_t batch, int64_t seq, int64_t D, double eps, int bf16,
                           float* y, float* dx, float* dgamma, float* dbeta) {
    try {
        const auto opts = torch::TensorOptions().dtype(torch::kFloat32);
        auto xt = torch::from_blob(const_cast<float*>(x), {batch, seq, D}, opts).clone();
        auto dyt = torch::from_blob(const_cast<float*>(dy), {batch, seq, D}, opts).clone();
        auto gt = torch::from_blob(const_cast<float*>(gamma), {D}, opts).clone();
        auto bt = torch::from_blob(const_cast<float*>(beta), {D}, opts).clone();
        torch::Tensor out, weight, bias;
        if (which <= 2) {
            if (!torch::cuda::is_available()) throw std::runtime_error("the drop-in modules need a CUDA device");
            const auto dt = bf16 ? torch::kBFloat16 : torch::kFloat32;
            Nott::B200::LayerNormOptions options;
            options.eps = eps;
            options.activation = Nott::B200::ActivationType::GeLU;           // fused behind the norm
            Nott::B200::LayerNorm module(D, options);
            module->to(torch::kCUDA, dt);
            {
                torch::NoGradGuard ng;
                module->weight.copy_(gt);
                module->bias.copy_(bt);
            }
            weight = module->weight;
            bias = module->bias;
            xt = xt.to(torch::kCUDA, dt).requires_grad_(true);
            dyt = dyt.to(torch::kCUDA, dt);

            RegisteredLayer layer;
            layer.module = Nott::Layer::Details::to_shared_module_ptr(module);
            layer.activation = Nott::Activation::Type::Identity;              // nothing left for apply() to do
            layer.name = "b200_layernorm_gelu";
            if (which == 2) layer.bind_inline_forward(CallB200LayerNorm{module.get()});
            else layer.bind_module_forward(module.get());
            if (!layer.forward) throw std::logic_error("binding is empty");

            if (which == 0) {
                out = run_layer(layer, xt);
            } else if (which == 1) {
                RegisteredLayer copy(layer);                                   // module binding: the context is the module itself
                out = run_layer(copy, xt);
            } else {
                RegisteredLayer copy(layer);                                   // inline context must now point into `copy`
                if (copy.forward.context == layer.forward.context) throw std::logic_error("copied layer still points at the source's inline context");
                RegisteredLayer moved(std::move(copy));
                if (copy.forward) throw std::logic_error("moved-from layer kept its binding");
                RegisteredLayer assigned;
                assigned = moved;
                out = run_layer(assigned, xt);
            }
            out.backward(dyt);
        } else {
            const auto dt = which == 4 ? torch::kFloat64 : torch::kFloat32;
            // the module the reference's blocks build (src/block/details/transformers/classic.hpp:399-404)
            torch::nn::LayerNorm module(torch::nn::LayerNormOptions({D}).eps(eps).elementwise_affine(true));
            module->to(dt);
            {
                torch::NoGradGuard ng;
                module->weight.copy_(gt);
                module->bias.copy_(bt);
            }
            weight = module->weight;
            bias = module->bias;
            xt = xt.to(dt).requires_grad_(true);
            dyt = dyt.to(dt);
            RegisteredLayer layer;
            layer.module = Nott::Layer::Details::to_shared_module_ptr(module);
            layer.activation = Nott::Activation::Type::GeLU;                  // applied by the reference's apply()
            layer.bind_module_forward(module.get());
            out = run_layer(layer, xt);
            out.backward(dyt);
        }
        copy_out(out, y);
        copy_out(xt.grad(), dx);
        copy_out(weight.grad(), dgamma);
        copy_out(bias.grad(), dbeta);
        return 0;
    } catch (const std::exception& e) {
        g_error = e.what();
        return -1;
    }
}

// An empty binding raises std::logic_error (registry.hpp:44-46); returns 1 when it did.
int refbind_empty_binding_raises() {
    RegisteredLayer layer;
    try {
        layer.forward(torch::zeros({1}));
    } catch (const std::logic_error&) {
        return 1;
    } catch (...) {
        return 0;
    }
    return 0;
}

}  // extern "C"
