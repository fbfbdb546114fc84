// TEST INFRASTRUCTURE — not part of the product.
//
// C entry points that drive the UNMODIFIED reference implementation (compiled from the
// reference checkout by oracle/Makefile into oracle/_ref/libtf_ref.so). They exist so that
// (1) the C restatement in oracle/oracle.c can be pinned against the reference itself,
// (2) golden fixtures can be generated, and (3) bench.py's reference arm can time the
// reference's own CPU matmul. Nothing here is linked into libtfb.so.
//
// Every function returns 0 on success and -1 if the reference threw.
#include <cstdint>
#include <cstring>
#include <exception>
#include <string>

#include "nn/Activations.hpp"
#include "nn/Conv2dModule.hpp"
#include "nn/Linear.hpp"
#include "tensor/AutogradWirer.hpp"
#include "tensor/Tensor.hpp"
#include "tensor/factory.hpp"

using tensorforge::Device;
using tensorforge::Dtype;
using tensorforge::Shape;
using tensorforge::Tensor;

namespace {

thread_local std::string g_what;

Tensor from_host(const float* src, Shape shape) {
    Tensor t = Tensor::empty(shape, Dtype::Float32, Device::cpu());
    std::memcpy(t.data(), src, static_cast<size_t>(t.numel()) * sizeof(float));
    return t;
}

void to_host(const Tensor& t, float* dst) {
    std::memcpy(dst, t.data(), static_cast<size_t>(t.numel()) * sizeof(float));
}

Tensor& weight_of(tensorforge::nn::Module& m) {
    for (auto& kv : m.named_parameters()) {
        if (kv.first == "weight") return kv.second->data_;
    }
    throw std::runtime_error("module has no weight parameter");
}

template <class F>
int guarded(F&& f) {
    try {
        tensorforge::init_tensor_autograd();
        f();
        return 0;
    } catch (const std::exception& e) {
        g_what = e.what();
        return -1;
    }
}

// loss = sum(Y ⊙ G): its gradient with respect to Y is G, which seeds an arbitrary upstream
// gradient through the reference's own engine.
Tensor seeded_loss(const Tensor& y, const Tensor& g) {
    Tensor prod = y * g;
    Tensor rows = prod.sum(1);
    return rows.sum(0, true);
}

}  // namespace

extern "C" {

const char* ref_last_error() { return g_what.c_str(); }

// Tensor::matmul on CPU tensors (tensor/Tensor.cpp:334-368).
int ref_matmul(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K) {
    return guarded([&] {
        Tensor a = from_host(A, Shape{M, K});
        Tensor b = from_host(B, Shape{K, N});
        Tensor c = a.matmul(b);
        to_host(c, C);
    });
}

// A matrix kept as a reference Tensor across calls (the reference never frees storage, so the
// handle lives until the process exits). Used to time row panels of one large product without
// re-copying B for every panel.
void* ref_hold_matrix(const float* src, int64_t rows, int64_t cols) {
    try {
        tensorforge::init_tensor_autograd();
        return new Tensor(from_host(src, Shape{rows, cols}));
    } catch (const std::exception& e) {
        g_what = e.what();
        return nullptr;
    }
}

// C[M,N] = A[M,K] · held B[K,N] through Tensor::matmul. Safe to call from several threads at
// once on different A panels: the call only reads B and allocates its own tensors.
int ref_matmul_held(const float* A, void* held_b, float* C, int64_t M) {
    return guarded([&] {
        const Tensor& b = *static_cast<const Tensor*>(held_b);
        Tensor a = from_host(A, Shape{M, b.shape()[0]});
        Tensor c = a.matmul(b);
        to_host(c, C);
    });
}

// C = A·B followed by backward with upstream gradient G (MatmulBackward,
// autograd/ops/MatmulBackward.hpp:26-34).
int ref_matmul_backward(const float* A, const float* B, const float* G, float* dA, float* dB,
                        int64_t M, int64_t N, int64_t K) {
    return guarded([&] {
        Tensor a = from_host(A, Shape{M, K});
        Tensor b = from_host(B, Shape{K, N});
        a.requires_grad(true);
        b.requires_grad(true);
        Tensor c = a.matmul(b);
        Tensor loss = seeded_loss(c, from_host(G, Shape{M, N}));
        loss.backward();
        to_host(a.grad(), dA);
        to_host(b.grad(), dB);
    });
}

// Weights the reference's nn::Linear constructor draws (nn/Linear.cpp:13-29).
int ref_linear_weight(int in_features, int out_features, float* W) {
    return guarded([&] {
        tensorforge::nn::Linear lin(in_features, out_features);
        to_host(weight_of(lin), W);
    });
}

// Y = relu?(Linear(X)), then backward seeded with G: dX and dW as the reference's autograd
// produces them (nn/Linear.cpp:45-64, ReluBackward, MatmulBackward, TransposeBackward).
// W == NULL keeps the constructor's weights.
int ref_linear_fwd_bwd(const float* X, const float* W, const float* G, int64_t batch,
                       int in_features, int out_features, int relu, float* Y, float* dX, float* dW) {
    return guarded([&] {
        tensorforge::nn::Linear lin(in_features, out_features);
        Tensor& w = weight_of(lin);
        if (W != nullptr) std::memcpy(w.data(), W, static_cast<size_t>(w.numel()) * sizeof(float));
        Tensor x = from_host(X, Shape{batch, in_features});
        x.requires_grad(true);
        Tensor y = lin.forward(x);
        if (relu) y = y.relu();
        if (Y != nullptr) to_host(y, Y);
        if (G != nullptr) {
            Tensor loss = seeded_loss(y, from_host(G, Shape{batch, out_features}));
            loss.backward();
            if (dX != nullptr) to_host(x.grad(), dX);
            if (dW != nullptr) to_host(w.grad(), dW);
        }
    });
}

// Weights the reference's Conv2dModule constructor draws (nn/Conv2dModule.cpp:74-97).
int ref_conv_weight(int cin, int cout, int k, float* W) {
    return guarded([&] {
        tensorforge::nn::Conv2dModule conv(cin, cout, k);
        to_host(weight_of(conv), W);
    });
}

// Conv2dModule::forward (direct CPU convolution, nn/Conv2dModule.cpp:26-70,108-154).
// W == NULL keeps the constructor's weights; the module's bias is zero.
int ref_conv2d_forward(const float* X, const float* W, int64_t N, int cin, int64_t H, int64_t Wd,
                       int cout, int k, int stride, int pad, int dil, float* out) {
    return guarded([&] {
        tensorforge::nn::Conv2dModule conv(cin, cout, k, stride, pad, dil);
        Tensor& w = weight_of(conv);
        if (W != nullptr) std::memcpy(w.data(), W, static_cast<size_t>(w.numel()) * sizeof(float));
        Tensor x = from_host(X, Shape{N, cin, H, Wd});
        Tensor y = conv.forward(x);
        to_host(y, out);
    });
}

// Tensor::log_softmax over the last dimension (tensor/Tensor.cpp:411-447).
int ref_log_softmax(const float* X, int64_t rows, int64_t cols, float* out) {
    return guarded([&] {
        Tensor x = from_host(X, Shape{rows, cols});
        to_host(x.log_softmax(-1), out);
    });
}

// One MLP training step's forward and backward with the reference's ops: three Linear
// layers with ReLU between them, mean negative log-likelihood of log_softmax (the loss
// graph of examples/train_mlp.cpp:54-76). Weights are given by the caller. Outputs the
// scalar loss and the three weight gradients.
int ref_mlp_grads(const float* X, const int64_t* labels, int64_t batch, int d0, int d1, int d2,
                  int d3, const float* W1, const float* W2, const float* W3, float* loss_out,
                  float* dW1, float* dW2, float* dW3) {
    return guarded([&] {
        tensorforge::nn::Linear l1(d0, d1), l2(d1, d2), l3(d2, d3);
        std::memcpy(weight_of(l1).data(), W1, sizeof(float) * d0 * d1);
        std::memcpy(weight_of(l2).data(), W2, sizeof(float) * d1 * d2);
        std::memcpy(weight_of(l3).data(), W3, sizeof(float) * d2 * d3);
        Tensor x = from_host(X, Shape{batch, d0});
        Tensor h1 = l1.forward(x).relu();
        Tensor h2 = l2.forward(h1).relu();
        Tensor z = l3.forward(h2);
        Tensor lsm = z.log_softmax(-1);
        Tensor onehot = tensorforge::zeros(Shape{batch, d3}, Dtype::Float32, Device::cpu());
        float* oh = static_cast<float*>(onehot.data());
        for (int64_t i = 0; i < batch; ++i) {
            if (labels[i] >= 0 && labels[i] < d3) oh[i * d3 + labels[i]] = 1.0f;
        }
        Tensor total = (lsm * onehot).sum(1).sum(0, true);
        Tensor scale = tensorforge::full(Shape{1}, -1.0 / static_cast<double>(batch), Dtype::Float32,
                                         Device::cpu());
        Tensor loss = total * scale;
        loss.backward();
        *loss_out = static_cast<const float*>(loss.data())[0];
        to_host(weight_of(l1).grad(), dW1);
        to_host(weight_of(l2).grad(), dW2);
        to_host(weight_of(l3).grad(), dW3);
    });
}

}  // extern "C"
