// CUDA-resident autograd for the host mirror: graph nodes, the engine and the operations that record
// nodes. Every loop over tensor data that the reference runs on the host during a backward pass is a
// libtfb kernel here, so gradients of CUDA tensors never visit the host.
#include <atomic>
#include <cmath>
#include <queue>
#include <random>
#include <unordered_map>
#include <unordered_set>

#include "../../include/tfb.h"
#include "tensorforge_b200.hpp"

namespace tensorforge {

namespace {

void ok(int rc, const char* what) {
    if (rc != TFB_OK) throw std::runtime_error(std::string(what) + ": " + tfb_last_error_string());
}

void* stream_of(const Tensor& t) { return DeviceContext::for_device(t.device().index).current_stream; }

std::atomic<uint64_t> g_sequence{1};

void require_cuda_f32(const Tensor& t, const char* who) {
    if (t.device().type != DeviceType::CUDA) throw std::invalid_argument(std::string(who) + ": CUDA tensors only");
    if (t.dtype() != Dtype::Float32) throw std::invalid_argument(std::string(who) + ": only Float32 supported");
}

// a + b into fresh storage (a gradient tensor may be shared with another holder, so neither is touched).
Tensor add_on_device(const Tensor& a, const Tensor& b) {
    if (!(a.shape() == b.shape())) throw std::runtime_error("InputBuffer: shape mismatch during gradient accumulation");
    require_cuda_f32(a, "InputBuffer");
    require_cuda_f32(b, "InputBuffer");
    DeviceGuard g(a.device().index);
    Tensor r = Tensor::empty(a.shape(), a.dtype(), a.device());
    const size_t bytes = static_cast<size_t>(a.numel()) * sizeof(float);
    ok(tfb_memcpy(r.data(), a.data(), bytes, 3, stream_of(a)), "tfb_memcpy");
    ok(tfb_accumulate(static_cast<float*>(r.data()), static_cast<const float*>(b.data()), a.numel(), stream_of(a)),
       "tfb_accumulate");
    return r;
}

class LinearBackward : public Node {
public:
    LinearBackward(Tensor x, Tensor y, Tensor w, int64_t in_f, int64_t out_f, bool relu, bool bias)
        : x_(std::move(x)), y_(std::move(y)), w_(std::move(w)), in_f_(in_f), out_f_(out_f), relu_(relu), bias_(bias) {}
    std::vector<Tensor> apply(std::vector<Tensor>&& grads) override {
        const Tensor& dy = grads.at(0);
        DeviceGuard g(x_.device().index);
        const int64_t batch = x_.shape()[0];
        Tensor dx = Tensor::empty(Shape{batch, in_f_}, Dtype::Float32, x_.device());
        Tensor dw = Tensor::empty(Shape{out_f_, in_f_}, Dtype::Float32, x_.device());
        Tensor db = bias_ ? Tensor::empty(Shape{out_f_}, Dtype::Float32, x_.device()) : Tensor();
        ok(tfb_linear_backward(x_.data(), w_.data(), y_.data(), dy.data(), dx.data(), dw.data(),
                               bias_ ? static_cast<float*>(db.data()) : nullptr, batch, in_f_, out_f_, relu_ ? 1 : 0,
                               TFB_DTYPE_F32, stream_of(x_)),
           "tfb_linear_backward");
        return {std::move(dx), std::move(dw), std::move(db)};
    }
    void release_saved() override { x_ = Tensor(); y_ = Tensor(); w_ = Tensor(); }

private:
    Tensor x_, y_, w_;
    int64_t in_f_, out_f_;
    bool relu_, bias_;
};

class CrossEntropyBackward : public Node {
public:
    explicit CrossEntropyBackward(Tensor dlogits) : dlogits_(std::move(dlogits)) {}
    std::vector<Tensor> apply(std::vector<Tensor>&& grads) override {
        const Tensor& up = grads.at(0);   // one element, on the device
        DeviceGuard g(dlogits_.device().index);
        Tensor d = Tensor::empty(dlogits_.shape(), Dtype::Float32, dlogits_.device());
        ok(tfb_scale_by_device_scalar(static_cast<const float*>(dlogits_.data()), static_cast<const float*>(up.data()),
                                      static_cast<float*>(d.data()), d.numel(), stream_of(d)),
           "tfb_scale_by_device_scalar");
        return {std::move(d)};
    }
    void release_saved() override { dlogits_ = Tensor(); }

private:
    Tensor dlogits_;
};

class Conv2dBackward : public Node {
public:
    Conv2dBackward(Tensor x, Tensor w, int k, int stride, int padding, int dilation, bool bias)
        : x_(std::move(x)), w_(std::move(w)), k_(k), stride_(stride), padding_(padding), dilation_(dilation), bias_(bias),
          need_dx_(x_.requires_grad()) {}
    std::vector<Tensor> apply(std::vector<Tensor>&& grads) override {
        const Tensor& dy = grads.at(0);
        const Shape& in = x_.shape();
        const int64_t cout = w_.shape()[0];
        DeviceGuard g(x_.device().index);
        // the input gradient of a first layer is nobody's input: skip that product
        Tensor dx = need_dx_ ? Tensor::empty(Shape{in[0], in[1], in[2], in[3]}, Dtype::Float32, x_.device()) : Tensor();
        Tensor dw = Tensor::empty(Shape{cout, in[1], k_, k_}, Dtype::Float32, x_.device());
        Tensor db = bias_ ? Tensor::empty(Shape{cout}, Dtype::Float32, x_.device()) : Tensor();
        ok(tfb_conv2d_backward(x_.data(), w_.data(), dy.data(), need_dx_ ? dx.data() : nullptr, dw.data(),
                               bias_ ? static_cast<float*>(db.data()) : nullptr, in[0], in[1], in[2], in[3], cout, k_, k_,
                               stride_, stride_, padding_, padding_, dilation_, dilation_, TFB_DTYPE_F32, stream_of(x_)),
           "tfb_conv2d_backward");
        return {std::move(dx), std::move(dw), std::move(db)};
    }
    void release_saved() override { x_ = Tensor(); w_ = Tensor(); }

private:
    Tensor x_, w_;
    int k_, stride_, padding_, dilation_;
    bool bias_, need_dx_;
};

}  // namespace

// ---- Node / AccumulateGrad ------------------------------------------------------------------------
Node::Node() : sequence_nr_(g_sequence.fetch_add(1)) {}

AccumulateGrad::AccumulateGrad(std::weak_ptr<AutogradMeta> meta) : meta_(std::move(meta)) { sequence_nr_ = 0; }

std::vector<Tensor> AccumulateGrad::apply(std::vector<Tensor>&& grads) {
    if (grads.empty() || !grads[0].defined()) throw std::runtime_error("AccumulateGrad::apply received no gradients");
    if (auto meta = meta_.lock()) meta->grad_ = grads[0];
    return {grads[0]};
}

// ---- Tensor autograd accessors ----------------------------------------------------------------------
void Tensor::requires_grad(bool req) {
    if (!autograd_meta_) autograd_meta_ = std::make_shared<AutogradMeta>();
    autograd_meta_->requires_grad_ = req;
}
bool Tensor::requires_grad() const noexcept {
    return autograd_meta_ && (autograd_meta_->requires_grad_ || autograd_meta_->grad_fn_ != nullptr);
}
Tensor Tensor::grad() const { return autograd_meta_ ? autograd_meta_->grad_ : Tensor(); }
std::shared_ptr<Node> Tensor::grad_fn() const { return autograd_meta_ ? autograd_meta_->grad_fn_ : nullptr; }
void Tensor::set_grad_fn(std::shared_ptr<Node> fn, uint32_t output_nr) {
    if (!autograd_meta_) autograd_meta_ = std::make_shared<AutogradMeta>();
    autograd_meta_->grad_fn_ = std::move(fn);
    autograd_meta_->output_nr_ = output_nr;
}
Edge Tensor::gradient_edge() const {
    if (!autograd_meta_) return Edge{};
    if (autograd_meta_->grad_fn_) return Edge{autograd_meta_->grad_fn_, autograd_meta_->output_nr_};
    if (!autograd_meta_->requires_grad_) return Edge{};
    if (!autograd_meta_->grad_accumulator_)
        autograd_meta_->grad_accumulator_ = std::make_shared<AccumulateGrad>(std::weak_ptr<AutogradMeta>(autograd_meta_));
    return Edge{autograd_meta_->grad_accumulator_, 0};
}

void Tensor::backward() {
    if (!autograd_meta_ || !autograd_meta_->grad_fn_)
        throw std::runtime_error("backward() called on tensor without grad_fn");
    require_cuda_f32(*this, "Tensor::backward");
    DeviceGuard g(device().index);
    Tensor grad = Tensor::empty(numel() == 0 ? Shape{1} : shape_, Dtype::Float32, device());
    ok(tfb_fill(static_cast<float*>(grad.data()), grad.numel(), 1.0f, stream_of(grad)), "tfb_fill");
    Engine engine;
    engine.execute(autograd_meta_->grad_fn_, grad, false);
}

// ---- Engine -----------------------------------------------------------------------------------------
void Engine::execute(std::shared_ptr<Node> root, const Tensor& initial_grad, bool keep_graph) {
    if (!root) return;
    // how many gradients each node has to wait for
    std::unordered_map<Node*, int> dependencies;
    {
        std::unordered_set<Node*> seen{root.get()};
        std::vector<Node*> stack{root.get()};
        while (!stack.empty()) {
            Node* n = stack.back();
            stack.pop_back();
            for (const Edge& e : n->next_edges_) {
                if (!e.function) continue;
                ++dependencies[e.function.get()];
                if (seen.insert(e.function.get()).second) stack.push_back(e.function.get());
            }
        }
    }
    std::unordered_map<Node*, std::vector<Tensor>> buffers;
    auto later_first = [](const std::shared_ptr<Node>& a, const std::shared_ptr<Node>& b) {
        return a->sequence_nr_ < b->sequence_nr_;
    };
    std::priority_queue<std::shared_ptr<Node>, std::vector<std::shared_ptr<Node>>, decltype(later_first)> ready(later_first);
    buffers[root.get()] = {initial_grad};
    ready.push(root);
    while (!ready.empty()) {
        std::shared_ptr<Node> node = ready.top();
        ready.pop();
        std::vector<Tensor> grads = std::move(buffers[node.get()]);
        buffers.erase(node.get());
        std::vector<Tensor> outs = node->apply(std::move(grads));
        if (!keep_graph) node->release_saved();
        for (size_t i = 0; i < node->next_edges_.size(); ++i) {
            const Edge& e = node->next_edges_[i];
            if (!e.function) continue;
            if (i < outs.size() && outs[i].defined()) {
                std::vector<Tensor>& buf = buffers[e.function.get()];
                if (buf.size() <= e.input_nr) buf.resize(e.input_nr + 1);
                buf[e.input_nr] = buf[e.input_nr].defined() ? add_on_device(buf[e.input_nr], outs[i]) : outs[i];
            }
            if (--dependencies[e.function.get()] == 0) ready.push(e.function);
        }
    }
}

// ---- operations that record nodes ---------------------------------------------------------------------
void record_matmul(Tensor& out, const Tensor& a, const Tensor& b) {
    if (!a.requires_grad() && !b.requires_grad()) return;
    auto node = std::make_shared<MatmulBackward>(a, b);
    node->next_edges_ = {a.gradient_edge(), b.gradient_edge()};
    out.set_grad_fn(std::move(node));
}

Tensor Tensor::relu() const {
    require_cuda_f32(*this, "Tensor::relu");
    DeviceGuard g(device().index);
    Tensor out = Tensor::empty(shape_, Dtype::Float32, device());
    ok(tfb_relu_forward(static_cast<const float*>(data()), static_cast<float*>(out.data()), numel(), stream_of(*this)),
       "tfb_relu_forward");
    if (requires_grad()) {
        auto node = std::make_shared<ReluBackward>(*this);
        node->next_edges_ = {gradient_edge()};
        out.set_grad_fn(std::move(node));
    }
    return out;
}

std::vector<Tensor> ReluBackward::apply(std::vector<Tensor>&& grads) {
    const Tensor& dy = grads.at(0);
    DeviceGuard g(input_.device().index);
    Tensor dx = Tensor::empty(input_.shape(), Dtype::Float32, input_.device());
    ok(tfb_relu_backward(static_cast<const float*>(input_.data()), static_cast<const float*>(dy.data()),
                         static_cast<float*>(dx.data()), dx.numel(), stream_of(dx)),
       "tfb_relu_backward");
    return {std::move(dx)};
}

void record_linear(Tensor& y, const Tensor& x, const Tensor& w, const Tensor& bias, int64_t in_f, int64_t out_f,
                   bool relu, bool bias_enabled) {
    if (!x.requires_grad() && !w.requires_grad() && !(bias_enabled && bias.requires_grad())) return;
    auto node = std::make_shared<LinearBackward>(x, y, w, in_f, out_f, relu, bias_enabled);
    node->next_edges_ = {x.gradient_edge(), w.gradient_edge(), bias_enabled ? bias.gradient_edge() : Edge{}};
    y.set_grad_fn(std::move(node));
}

Tensor cross_entropy(const Tensor& logits, const Tensor& labels) {
    require_cuda_f32(logits, "cross_entropy");
    if (logits.shape().ndim() != 2) throw std::invalid_argument("cross_entropy: logits must be [N, C]");
    if (labels.dtype() != Dtype::Int64 || labels.numel() != logits.shape()[0] || labels.device() != logits.device())
        throw std::invalid_argument("cross_entropy: labels must be Int64 [N] on the logits' device");
    DeviceGuard g(logits.device().index);
    const int64_t rows = logits.shape()[0], cols = logits.shape()[1];
    Tensor loss = Tensor::empty(Shape{1}, Dtype::Float32, logits.device());
    const bool needs_grad = logits.requires_grad();
    Tensor dlogits = needs_grad ? Tensor::empty(logits.shape(), Dtype::Float32, logits.device()) : Tensor();
    ok(tfb_log_softmax_nll(static_cast<const float*>(logits.data()), static_cast<const int64_t*>(labels.data()),
                           needs_grad ? static_cast<float*>(dlogits.data()) : nullptr, static_cast<float*>(loss.data()),
                           rows, cols, rows, stream_of(logits)),
       "tfb_log_softmax_nll");
    if (needs_grad) {
        auto node = std::make_shared<CrossEntropyBackward>(std::move(dlogits));
        node->next_edges_ = {logits.gradient_edge()};
        loss.set_grad_fn(std::move(node));
    }
    return loss;
}

namespace nn {

Conv2dModule::Conv2dModule(int in_channels, int out_channels, int kernel_size, int stride, int padding, int dilation,
                           bool bias, Device device)
    : in_channels_(in_channels), out_channels_(out_channels), kernel_size_(kernel_size), stride_(stride),
      padding_(padding), dilation_(dilation), bias_enabled_(bias) {
    std::vector<float> w(static_cast<size_t>(out_channels) * in_channels * kernel_size * kernel_size);
    const float bound = std::sqrt(1.0f / static_cast<float>(in_channels * kernel_size * kernel_size));
    std::mt19937 rng(0xC0FFEEu);
    std::uniform_real_distribution<float> dist(-bound, bound);
    for (float& v : w) v = dist(rng);
    weight_ = Tensor::from_host(w.data(), Shape{out_channels, in_channels, kernel_size, kernel_size}, Dtype::Float32, device);
    weight_.requires_grad(true);
    if (bias_enabled_) {
        std::vector<float> b(static_cast<size_t>(out_channels), 0.0f);
        bias_ = Tensor::from_host(b.data(), Shape{out_channels}, Dtype::Float32, device);
        bias_.requires_grad(true);
    }
}

Tensor Conv2dModule::forward(Tensor x) {
    const Shape& s = x.shape();
    if (s.ndim() != 4) throw std::invalid_argument("Conv2dModule.forward expects [N, Cin, H, W]");
    if (s[1] != in_channels_) throw std::invalid_argument("Conv2dModule.forward: Cin mismatch");
    require_cuda_f32(x, "Conv2dModule.forward");
    DeviceGuard g(x.device().index);
    const int64_t oh = tfb_conv_out_dim(s[2], kernel_size_, stride_, padding_, dilation_);
    const int64_t ow = tfb_conv_out_dim(s[3], kernel_size_, stride_, padding_, dilation_);
    if (oh <= 0 || ow <= 0) throw std::invalid_argument("Conv2dModule.forward: empty output");
    Tensor out = Tensor::empty(Shape{s[0], out_channels_, oh, ow}, Dtype::Float32, x.device());
    ok(tfb_conv2d_forward(x.data(), weight_.data(), bias_enabled_ ? static_cast<const float*>(bias_.data()) : nullptr,
                          out.data(), s[0], s[1], s[2], s[3], out_channels_, kernel_size_, kernel_size_, stride_, stride_,
                          padding_, padding_, dilation_, dilation_, 0, TFB_DTYPE_F32, stream_of(x)),
       "tfb_conv2d_forward");
    if (x.requires_grad() || weight_.requires_grad() || (bias_enabled_ && bias_.requires_grad())) {
        auto node = std::make_shared<Conv2dBackward>(x, weight_, kernel_size_, stride_, padding_, dilation_, bias_enabled_);
        node->next_edges_ = {x.gradient_edge(), weight_.gradient_edge(), bias_enabled_ ? bias_.gradient_edge() : Edge{}};
        out.set_grad_fn(std::move(node));
    }
    return out;
}

}  // namespace nn
}  // namespace tensorforge
