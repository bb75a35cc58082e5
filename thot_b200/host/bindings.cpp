// Python bindings of the C++ host layer (nott_b200.hpp) so the parity tests can drive the
// same autograd functions and modules a Nott build would link.  Not a second API: every
// call forwards to Nott::B200.
#include <torch/extension.h>

#include "nott_b200.hpp"

namespace nb = Nott::B200;

PYBIND11_MODULE(_nott_b200_host, m) {
    m.doc() = "libtorch host layer of libnott_b200 (Nott::B200)";
    m.def("layernorm_act", [](torch::Tensor x, c10::optional<torch::Tensor> w, c10::optional<torch::Tensor> b, double eps,
                              int64_t act) {
        return nb::LayerNormActFunction::apply(std::move(x), w, b, eps, act);
    });
    m.def("rmsnorm_act", [](torch::Tensor x, c10::optional<torch::Tensor> w, double eps, int64_t act) {
        return nb::RMSNormActFunction::apply(std::move(x), w, eps, act);
    });
    m.def("add_norm", [](torch::Tensor a, torch::Tensor b, torch::Tensor w, c10::optional<torch::Tensor> bias, double eps, bool rms) {
        return nb::AddNormFunction::apply(std::move(a), std::move(b), std::move(w), bias, eps, rms);
    });
    m.def("apply", [](int64_t type, torch::Tensor x) { return nb::apply(static_cast<nb::ActivationType>(type), std::move(x)); });
    m.def("silu_gate", [](torch::Tensor gate, torch::Tensor up) { return nb::silu_gate(gate, up); });
    m.def("embedding", [](torch::Tensor weight, torch::Tensor ids) {
        const bool training = torch::GradMode::is_enabled() && weight.requires_grad();
        return nb::EmbeddingFunction::apply(std::move(weight), std::move(ids), training);
    });
    m.def("attention_softmax", [](torch::Tensor scores, c10::optional<torch::Tensor> mask, c10::optional<torch::Tensor> padding,
                                  double scale, bool causal) {
        pybind11::gil_scoped_release nogil;
        return nb::AttentionSoftmaxFunction::apply(std::move(scores), std::move(mask), std::move(padding), scale, causal);
    });
    m.def("scaled_dot_product", [](torch::Tensor q, torch::Tensor k, torch::Tensor v, c10::optional<torch::Tensor> mask,
                                   c10::optional<torch::Tensor> padding, bool causal) {
        pybind11::gil_scoped_release nogil;
        nb::ScaledDotProductKernel kernel(0.0, causal ? nb::AttentionVariant::Causal : nb::AttentionVariant::Full);
        return kernel->forward(q, k, v, mask.value_or(torch::Tensor()), padding.value_or(torch::Tensor()));
    });
    // dropout on the probabilities, fused: with `noise` the caller's tensor is used; without it and p > 0 the
    // module draws a keep mask itself (training mode)
    m.def("scaled_dot_product_dropout", [](torch::Tensor q, torch::Tensor k, torch::Tensor v, c10::optional<torch::Tensor> noise,
                                           double p, bool causal) {
        pybind11::gil_scoped_release nogil;
        nb::ScaledDotProductKernel kernel(p, causal ? nb::AttentionVariant::Causal : nb::AttentionVariant::Full);
        kernel->train();
        if (noise.has_value()) return kernel->forward_with_noise(q, k, v, *noise);
        return kernel->forward(q, k, v);
    });
    // FC layer: Linear + fused activation, forward and backward; returns y, dx, dweight, dbias
    m.def("linear_module_step", [](torch::Tensor x, torch::Tensor weight, c10::optional<torch::Tensor> bias, int64_t act_type, torch::Tensor dy) {
        pybind11::gil_scoped_release nogil;
        nb::LinearOptions opt;
        opt.in_features = weight.size(1); opt.out_features = weight.size(0); opt.bias = bias.has_value();
        opt.activation = static_cast<nb::ActivationType>(act_type);
        nb::Linear mod(opt);
        mod->to(x.device(), x.scalar_type());
        {
            torch::NoGradGuard ng;
            mod->weight.copy_(weight);
            if (bias.has_value()) mod->bias.copy_(*bias);
        }
        auto xin = x.clone().requires_grad_(true);
        auto y = mod->forward(xin);
        y.backward(dy);
        std::vector<std::string> names;
        for (auto& kv : mod->named_parameters()) names.push_back(kv.key());
        std::vector<torch::Tensor> out{y.detach(), xin.grad(), mod->weight.grad()};
        if (bias.has_value()) out.push_back(mod->bias.grad());
        return std::make_pair(names, out);
    });
    // the C++ step driver on a one-rank communicator: three steps with alternating gradient buffers
    m.def("sharded_norm_steps", [](bool rms, int64_t exchange, torch::Tensor x, torch::Tensor dy, torch::Tensor weight,
                                   c10::optional<torch::Tensor> bias, int64_t act_type, double eps, int64_t steps) {
        pybind11::gil_scoped_release nogil;
        auto comm = std::make_shared<nb::Communicator>(std::vector<uint8_t>{}, 0, 1, (int)exchange, (rms ? 1 : 2) * x.size(1));
        nb::ShardedNormStep step(comm, rms, x.size(0), x.size(1), x.scalar_type(), static_cast<nb::ActivationType>(act_type), eps);
        auto y = torch::empty_like(x), dx = torch::empty_like(x);
        std::vector<torch::Tensor> grads{torch::zeros({(rms ? 1 : 2) * x.size(1)}, x.options().dtype(torch::kFloat32)),
                                         torch::zeros({(rms ? 1 : 2) * x.size(1)}, x.options().dtype(torch::kFloat32))};
        for (int64_t k = 0; k < steps; ++k) step.run(x, dy, weight, bias.value_or(torch::Tensor()), y, dx, grads[k & 1]);
        step.finish();
        comm->wait(10.0);
        return std::vector<torch::Tensor>{y, dx, grads[0], grads[1]};
    });
    m.def("rotary_table", [](int64_t S, int64_t hd, double theta, torch::Device device) {
        return nb::RotaryTable(S, hd, theta, device).table();
    });
    m.def("rotary", [](torch::Tensor x, torch::Tensor table) { return nb::RotaryFunction::apply(std::move(x), std::move(table)); });

    // module round trip: construct, run, and expose named parameters (checkpoint key names)
    m.def("layernorm_module_step", [](int64_t D, double eps, bool affine, int64_t act_type, torch::Tensor x, torch::Tensor dy) {
        nb::LayerNormOptions opt;
        opt.eps = eps; opt.elementwise_affine = affine; opt.activation = static_cast<nb::ActivationType>(act_type);
        pybind11::gil_scoped_release no_gil;     // backward() runs the autograd engine
        nb::LayerNorm mod(D, opt);
        mod->to(x.device(), x.scalar_type());
        auto xin = x.clone().requires_grad_(true);
        auto y = mod->forward(xin);
        y.backward(dy);
        std::vector<std::string> names;
        std::vector<torch::Tensor> out{y.detach(), xin.grad()};
        for (auto& kv : mod->named_parameters()) { names.push_back(kv.key()); out.push_back(kv.value().grad()); }
        return std::make_pair(names, out);
    });
    m.def("rmsnorm_module_step", [](int64_t D, double eps, bool learnable, int64_t act_type, torch::Tensor x, torch::Tensor dy) {
        nb::RMSNormOptions opt;
        opt.eps = eps; opt.learnable = learnable; opt.activation = static_cast<nb::ActivationType>(act_type);
        pybind11::gil_scoped_release no_gil;
        nb::RMSNorm mod(D, opt);
        mod->to(x.device(), x.scalar_type());
        auto xin = x.clone().requires_grad_(true);
        auto y = mod->forward(xin);
        y.backward(dy);
        std::vector<std::string> names;
        std::vector<torch::Tensor> out{y.detach(), xin.grad()};
        for (auto& kv : mod->named_parameters()) { names.push_back(kv.key()); out.push_back(kv.value().grad()); }
        return std::make_pair(names, out);
    });
    m.def("bert_embedding_module_step", [](int64_t D, int64_t vocab, int64_t type_vocab, int64_t max_pos, torch::Tensor ids,
                                           torch::Tensor dy, std::vector<torch::Tensor> values) {
        pybind11::gil_scoped_release no_gil;
        nb::BertEmbeddingOptions opt;
        opt.vocab_size = vocab; opt.type_vocab_size = type_vocab; opt.max_position_embeddings = max_pos; opt.dropout = 0.0;
        nb::BertEmbedding mod(D, opt);
        mod->to(dy.device(), dy.scalar_type());
        std::vector<std::string> names;
        {
            torch::NoGradGuard ng;
            size_t i = 0;
            for (auto& kv : mod->named_parameters()) { names.push_back(kv.key()); if (i < values.size()) kv.value().copy_(values[i]); ++i; }
        }
        // `ids` may also be ready-made [B, S, D] embeddings (bert.hpp:164-171); their gradient is appended last
        const bool embeddings = ids.is_floating_point();
        if (embeddings) ids = ids.clone().requires_grad_(true);
        auto y = mod->forward(ids);
        y.backward(dy);
        std::vector<torch::Tensor> out{y.detach()};
        for (auto& kv : mod->named_parameters()) out.push_back(kv.value().grad().defined() ? kv.value().grad() : torch::zeros_like(kv.value()));
        if (embeddings) out.push_back(ids.grad());
        return std::make_pair(names, out);
    });
    m.def("module_errors", []() {
        // the exception types the reference throws for the same mistakes (mamba.hpp:116-132)
        std::vector<std::string> seen;
        try { nb::RMSNorm bad(0, nb::RMSNormOptions{}); } catch (const std::invalid_argument& e) { seen.push_back(e.what()); }
        try { nb::RMSNorm ok(8, nb::RMSNormOptions{}); ok->forward(torch::Tensor()); } catch (const std::invalid_argument& e) { seen.push_back(e.what()); }
        try { nb::RMSNorm ok(8, nb::RMSNormOptions{}); ok->forward(torch::zeros({2, 8})); } catch (const std::invalid_argument& e) { seen.push_back(e.what()); }
        return seen;
    });
}
