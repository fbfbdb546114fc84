// Checks of the host mirror that read like the reference's own tests (known answers of
// cuda/kernels/gemm_*_test.cpp, autograd/ops/autograd_all_ops_test.cpp:281-328,
// nn/conv2d_{forward,backward}_test.cpp, nn/linear_test.cpp, tensor/tensor_cuda_dispatch_test.cpp).
//   host_test cpu   argument checks that need no GPU
//   host_test gpu   everything (needs a B200)
#include <cmath>
#include <cstdio>
#include <cstring>
#include <random>
#include <string>
#include <vector>

#include "../../include/tfb.h"
#include "tensorforge_b200.hpp"

using namespace tensorforge;

static int g_failed = 0;
#define CHECK(cond)                                                                 \
    do {                                                                            \
        if (!(cond)) {                                                              \
            std::printf("CHECK failed at %s:%d: %s\n", __FILE__, __LINE__, #cond);  \
            ++g_failed;                                                             \
        }                                                                           \
    } while (0)
template <class F>
static bool throws(F&& f) {
    try { f(); } catch (const std::exception&) { return true; }
    return false;
}
static bool approx(float a, float b, float eps) { return std::fabs(a - b) <= eps * std::fmax(1.0f, std::fabs(b)); }

static Tensor upload(const std::vector<float>& h, Shape s, Device d = Device::cuda(0)) {
    return Tensor::from_host(h.data(), std::move(s), Dtype::Float32, d);
}
static std::vector<float> download(const Tensor& t) {
    std::vector<float> h(static_cast<size_t>(t.numel()));
    t.copy_to_host(h.data());
    return h;
}

// A node that records when it ran and hands nothing on: the engine's ordering can be checked without a GPU.
struct ProbeNode : Node {
    std::vector<int>* order;
    int id;
    ProbeNode(std::vector<int>* o, int i) : order(o), id(i) {}
    std::vector<Tensor> apply(std::vector<Tensor>&&) override {
        order->push_back(id);
        return std::vector<Tensor>(next_edges_.size());
    }
};

static void engine_order_checks() {
    // diamond: root -> {left, right} -> sink, plus root -> sink directly. The sink must run once, last.
    std::vector<int> order;
    auto sink = std::make_shared<ProbeNode>(&order, 3);
    auto left = std::make_shared<ProbeNode>(&order, 1);
    auto right = std::make_shared<ProbeNode>(&order, 2);
    auto root = std::make_shared<ProbeNode>(&order, 0);
    left->next_edges_ = {Edge{sink, 0}};
    right->next_edges_ = {Edge{sink, 0}, Edge{}};   // a null edge (input that needs no gradient) is skipped
    root->next_edges_ = {Edge{left, 0}, Edge{right, 0}, Edge{sink, 1}};
    Engine().execute(root, Tensor(), false);
    CHECK(order.size() == 4 && order.front() == 0 && order.back() == 3);
    // among ready nodes the later-created one runs first
    CHECK(order.size() == 4 && order[1] == 2 && order[2] == 1);
    Engine().execute(nullptr, Tensor(), false);     // nothing to do
}

static void cpu_checks() {
    CHECK(registered_cuda_matmul() != nullptr);   // the static registrar ran
    Tensor a = Tensor::empty(Shape{2, 3}, Dtype::Float32, Device::cpu());
    Tensor b = Tensor::empty(Shape{4, 2}, Dtype::Float32, Device::cpu());
    Tensor v = Tensor::empty(Shape{3}, Dtype::Float32, Device::cpu());
    CHECK(throws([&] { (void)a.matmul(b); }));    // shape mismatch
    CHECK(throws([&] { (void)a.matmul(v); }));    // not 2-D
    Tensor c = Tensor::empty(Shape{3, 2}, Dtype::Float32, Device::cpu());
    CHECK(throws([&] { (void)a.matmul(c); }));    // CPU tensors are not served here
    register_cuda_matmul(nullptr);
    CHECK(registered_cuda_matmul() == nullptr);
    tfb_register_kernels();
    CHECK(registered_cuda_matmul() != nullptr);
    CHECK(dtype_size(Dtype::BFloat16) == 2 && dtype_size(Dtype::Int64) == 8);
    engine_order_checks();
    CHECK(throws([&] { a.backward(); }));         // no grad_fn (autograd/TensorAutograd.cpp:54-56)
    CHECK(!a.requires_grad() && !a.grad().defined());
    a.requires_grad(true);
    CHECK(a.requires_grad() && a.gradient_edge().function != nullptr);
}

// Backward passes over CUDA tensors: every step of the walk runs on the device.
static void autograd_checks() {
    // matmul_grad of autograd/ops/autograd_all_ops_test.cpp:281-328: c = a.matmul(b); c.backward()
    {
        Tensor a = upload({0, 1, 2, 3, 4, 5}, Shape{2, 3}), b = upload({0, 1, 2, 3, 4, 5}, Shape{3, 2});
        a.requires_grad(true);
        b.requires_grad(true);
        Tensor c = a.matmul(b);
        CHECK(c.requires_grad() && c.grad_fn() != nullptr);
        c.backward();
        auto ga = download(a.grad()), gb = download(b.grad());
        const float ea[6] = {1, 5, 9, 1, 5, 9}, eb[6] = {3, 3, 5, 5, 7, 7};
        for (int i = 0; i < 6; ++i) CHECK(approx(ga[i], ea[i], 1e-5f) && approx(gb[i], eb[i], 1e-5f));
        // no grad requested: no node
        Tensor p = upload({1, 2, 3, 4}, Shape{2, 2});
        CHECK(p.matmul(p).grad_fn() == nullptr);
    }
    // The same product in BFloat16: the result and both gradients have the operands' dtype (the
    // reference's rule, tensor/Tensor.cpp:350), so the upstream gradient MatmulBackward receives is
    // read with the dtype it was written in. The values are small integers, exact in BF16.
    {
        auto bf16 = [](const std::vector<float>& h) {
            std::vector<uint16_t> o(h.size());
            for (size_t i = 0; i < h.size(); ++i) {
                uint32_t u;
                std::memcpy(&u, &h[i], 4);
                o[i] = static_cast<uint16_t>(u >> 16);
            }
            return o;
        };
        auto widen = [](const Tensor& t) {
            std::vector<uint16_t> raw(static_cast<size_t>(t.numel()));
            t.copy_to_host(raw.data());
            std::vector<float> o(raw.size());
            for (size_t i = 0; i < raw.size(); ++i) {
                const uint32_t u = static_cast<uint32_t>(raw[i]) << 16;
                std::memcpy(&o[i], &u, 4);
            }
            return o;
        };
        const auto ah = bf16({0, 1, 2, 3, 4, 5}), bh = bf16({0, 1, 2, 3, 4, 5}), gh = bf16({1, 1, 1, 1});
        Tensor a = Tensor::from_host(ah.data(), Shape{2, 3}, Dtype::BFloat16, Device::cuda(0));
        Tensor b = Tensor::from_host(bh.data(), Shape{3, 2}, Dtype::BFloat16, Device::cuda(0));
        Tensor g = Tensor::from_host(gh.data(), Shape{2, 2}, Dtype::BFloat16, Device::cuda(0));
        a.requires_grad(true);
        b.requires_grad(true);
        Tensor c = a.matmul(b);
        CHECK(c.dtype() == Dtype::BFloat16);
        auto ch = widen(c);
        const float ec[4] = {10, 13, 28, 40};
        for (int i = 0; i < 4; ++i) CHECK(ch[i] == ec[i]);
        Engine engine;
        engine.execute(c.grad_fn(), g);
        CHECK(a.grad().dtype() == Dtype::BFloat16 && b.grad().dtype() == Dtype::BFloat16);
        auto ga = widen(a.grad()), gb = widen(b.grad());
        const float ea[6] = {1, 5, 9, 1, 5, 9}, eb[6] = {3, 3, 5, 5, 7, 7};
        for (int i = 0; i < 6; ++i) CHECK(ga[i] == ea[i] && gb[i] == eb[i]);
    }
    // relu: mask is 0 at x == 0 (autograd/ops/ReluBackward.hpp:26-30)
    {
        Tensor x = upload({-1.f, 0.f, 2.f, 3.f, -0.5f}, Shape{1, 5});
        x.requires_grad(true);
        Tensor y = x.relu();
        auto yh = download(y);
        const float ey[5] = {0, 0, 2, 3, 0};
        for (int i = 0; i < 5; ++i) CHECK(yh[i] == ey[i]);
        y.backward();
        auto gx = download(x.grad());
        const float eg[5] = {0, 0, 1, 1, 0};
        for (int i = 0; i < 5; ++i) CHECK(gx[i] == eg[i]);
    }
    // one tensor feeding two products: y = (x W) W, root gradient of ones;
    // dW = x^T (1 W^T) + (x W)^T 1 accumulated on the device
    {
        const std::vector<float> xh = {1, -2, 0.5f, 3, 0.25f, -1}, wh = {0.5f, -1, 2, 1.5f, 0.25f, -0.75f, -2, 1, 0.5f};
        Tensor x = upload(xh, Shape{2, 3}), W = upload(wh, Shape{3, 3});
        W.requires_grad(true);
        Tensor y = x.matmul(W).matmul(W);
        y.backward();
        auto gw = download(W.grad());
        double h[2][3] = {}, want[3][3] = {};
        for (int i = 0; i < 2; ++i)
            for (int j = 0; j < 3; ++j)
                for (int k = 0; k < 3; ++k) h[i][j] += double(xh[i * 3 + k]) * wh[k * 3 + j];
        for (int r = 0; r < 3; ++r)
            for (int c = 0; c < 3; ++c) {
                for (int i = 0; i < 2; ++i) {
                    double g1 = 0;   // (1 W^T)[i][c] = sum_j W[c][j]
                    for (int j = 0; j < 3; ++j) g1 += wh[c * 3 + j];
                    want[r][c] += double(xh[i * 3 + r]) * g1 + h[i][r];
                }
            }
        for (int r = 0; r < 3; ++r)
            for (int c = 0; c < 3; ++c) CHECK(approx(gw[r * 3 + c], float(want[r][c]), 1e-5f));
        CHECK(!x.grad().defined());   // x did not ask for a gradient
    }
    // the training graph of examples/train_mlp.cpp:161-183: Linear -> relu -> Linear -> cross_entropy ->
    // backward, against the same step done by hand with the (oracle-checked) explicit backward calls
    {
        const int64_t N = 7, D = 6, Hd = 5, C = 3;
        std::vector<float> xh(N * D);
        for (int64_t i = 0; i < N * D; ++i) xh[i] = 0.1f * float((i * 7) % 11) - 0.4f;
        std::vector<int64_t> lab = {0, 2, 1, 1, 0, 2, 2};
        Tensor x = upload(xh, Shape{N, D});
        Tensor labels = Tensor::from_host(lab.data(), Shape{N}, Dtype::Int64, Device::cuda(0));
        nn::Linear fc1(D, Hd), fc2(Hd, C);
        fc1.weight().requires_grad(true); fc1.bias().requires_grad(true);
        fc2.weight().requires_grad(true); fc2.bias().requires_grad(true);
        Tensor h = fc1.forward(x).relu();
        Tensor logits = fc2.forward(h);
        Tensor loss = cross_entropy(logits, labels);
        loss.backward();
        // by hand
        Tensor dz = Tensor::empty(Shape{N, C}, Dtype::Float32, Device::cuda(0));
        Tensor loss2 = Tensor::empty(Shape{1}, Dtype::Float32, Device::cuda(0));
        void* st = DeviceContext::current().current_stream;
        CHECK(tfb_log_softmax_nll(static_cast<const float*>(logits.data()), static_cast<const int64_t*>(labels.data()),
                                  static_cast<float*>(dz.data()), static_cast<float*>(loss2.data()), N, C, N, st) == TFB_OK);
        Tensor pre = fc1.forward(x);
        auto g2 = fc2.backward(h, logits, dz);
        Tensor dpre = Tensor::empty(Shape{N, Hd}, Dtype::Float32, Device::cuda(0));
        CHECK(tfb_relu_backward(static_cast<const float*>(pre.data()), static_cast<const float*>(g2.grad_input.data()),
                                static_cast<float*>(dpre.data()), N * Hd, st) == TFB_OK);
        auto g1 = fc1.backward(x, pre, dpre);
        auto same = [&](const Tensor& a, const Tensor& b) {
            auto ah = download(a), bh = download(b);
            CHECK(ah.size() == bh.size());
            for (size_t i = 0; i < ah.size() && i < bh.size(); ++i) CHECK(approx(ah[i], bh[i], 1e-6f));
        };
        same(loss, loss2);
        same(fc2.weight().grad(), g2.grad_weight);
        same(fc2.bias().grad(), g2.grad_bias);
        same(fc1.weight().grad(), g1.grad_weight);
        same(fc1.bias().grad(), g1.grad_bias);
        auto lh = download(loss);
        CHECK(lh[0] > 0.5f && lh[0] < 2.0f);   // about ln(3) for near-uniform predictions
        // a second backward pass replaces the stored gradients (autograd/AccumulateGrad.cpp:20-23)
        Tensor loss3 = cross_entropy(fc2.forward(fc1.forward(x).relu()), labels);
        loss3.backward();
        same(fc2.weight().grad(), g2.grad_weight);
    }
    // Conv2dModule: reference initialisation, and backward through the recorded node against the explicit
    // Conv2d::backward call (which the oracle checks) — y.backward() seeds a gradient of ones
    {
        nn::Conv2dModule conv(3, 8, 3, 1, 1);
        std::vector<float> wexp(8 * 3 * 9);
        {
            const float bound = std::sqrt(1.0f / 27.0f);
            std::mt19937 rng(0xC0FFEEu);
            std::uniform_real_distribution<float> dist(-bound, bound);
            for (float& v : wexp) v = dist(rng);
        }
        auto wh = download(conv.weight());
        for (size_t i = 0; i < wexp.size(); ++i) CHECK(wh[i] == wexp[i]);
        for (float b : download(conv.bias())) CHECK(b == 0.f);
        std::vector<float> xh(2 * 3 * 6 * 5);
        for (size_t i = 0; i < xh.size(); ++i) xh[i] = 0.05f * float((i * 13) % 17) - 0.4f;
        Tensor x = upload(xh, Shape{2, 3, 6, 5});
        x.requires_grad(true);
        Tensor y = conv.forward(x);
        CHECK(y.shape()[1] == 8 && y.shape()[2] == 6 && y.shape()[3] == 5 && y.grad_fn() != nullptr);
        y.backward();
        nn::Conv2d plain(3, 8, 3, 3, 1, 1, 1, 1);
        plain.weight() = conv.weight();
        auto gr = plain.backward(upload(std::vector<float>(2 * 8 * 6 * 5, 1.f), Shape{2, 8, 6, 5}), x);
        auto eq = [&](const Tensor& a, const Tensor& b) {
            auto ah = download(a), bh = download(b);
            CHECK(ah.size() == bh.size());
            for (size_t i = 0; i < ah.size() && i < bh.size(); ++i) CHECK(approx(ah[i], bh[i], 1e-6f));
        };
        eq(x.grad(), gr.grad_input);
        eq(conv.weight().grad(), gr.grad_weight);
        eq(conv.bias().grad(), gr.grad_bias);
        auto gb = download(conv.bias().grad());
        CHECK(approx(gb[0], 60.f, 1e-6f));   // 2 samples x 30 positions of ones
        // an input that asks for no gradient gets none, the parameters still do
        Tensor x2 = upload(xh, Shape{2, 3, 6, 5});
        conv.forward(x2).backward();
        CHECK(!x2.grad().defined());
        eq(conv.weight().grad(), gr.grad_weight);
        CHECK(throws([&] { (void)conv.forward(upload({1, 2, 3, 4}, Shape{1, 1, 2, 2})); }));   // Cin mismatch
    }
}

static void gpu_checks() {
    // 2x2 hand-computed case
    Tensor A = upload({1, 2, 3, 4}, Shape{2, 2}), B = upload({5, 6, 7, 8}, Shape{2, 2});
    auto C = download(A.matmul(B));
    const float expected[4] = {19, 22, 43, 50};
    for (int i = 0; i < 4; ++i) CHECK(approx(C[i], expected[i], 1e-5f));
    // the launcher signature, non-multiple-of-16 bounds (17x19)*(19x23)
    {
        const int64_t M = 17, K = 19, N = 23;
        std::vector<float> a(M * K), b(K * N), want(M * N, 0.f);
        for (int64_t i = 0; i < M * K; ++i) a[i] = 0.01f * float(i + 1);
        for (int64_t i = 0; i < K * N; ++i) b[i] = 0.02f * float((i % 7) + 1);
        for (int64_t m = 0; m < M; ++m)
            for (int64_t n = 0; n < N; ++n) {
                float s = 0.f;
                for (int64_t k = 0; k < K; ++k) s += a[m * K + k] * b[k * N + n];
                want[m * N + n] = s;
            }
        Tensor At = upload(a, Shape{M, K}), Bt = upload(b, Shape{K, N});
        Tensor Ct = Tensor::empty(Shape{M, N}, Dtype::Float32, Device::cuda(0));
        launch_gemm_optimized(At.data(), Bt.data(), Ct.data(), M, N, K, Dtype::Float32, DeviceContext::current().current_stream);
        auto got = download(Ct);
        for (int64_t i = 0; i < M * N; ++i) CHECK(approx(got[i], want[i], 1e-5f));
    }
    // MatmulBackward on the arange case: gA = [1,5,9;1,5,9], gB = [3,3;5,5;7,7]
    {
        Tensor a = upload({0, 1, 2, 3, 4, 5}, Shape{2, 3}), b = upload({0, 1, 2, 3, 4, 5}, Shape{3, 2});
        auto c = download(a.matmul(b));
        CHECK(approx(c[0], 10, 1e-6f) && approx(c[1], 13, 1e-6f) && approx(c[2], 28, 1e-6f) && approx(c[3], 40, 1e-6f));
        MatmulBackward node(a, b);
        auto grads = node.apply({upload({1, 1, 1, 1}, Shape{2, 2})});
        auto ga = download(grads[0]), gb = download(grads[1]);
        const float ea[6] = {1, 5, 9, 1, 5, 9}, eb[6] = {3, 3, 5, 5, 7, 7};
        for (int i = 0; i < 6; ++i) CHECK(approx(ga[i], ea[i], 1e-5f) && approx(gb[i], eb[i], 1e-5f));
    }
    // nn::Linear shape contract (nn/linear_test.cpp:9-33) and gradient sizes
    {
        nn::Linear lin(3, 2);
        Tensor x = upload({1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12}, Shape{4, 3});
        Tensor y = lin.forward(x);
        CHECK(y.shape()[0] == 4 && y.shape()[1] == 2);
        auto g = lin.backward(x, y, upload(std::vector<float>(8, 1.f), Shape{4, 2}));
        CHECK(g.grad_weight.numel() == 6 && g.grad_input.numel() == 12 && g.grad_bias.numel() == 2);
        auto gb = download(g.grad_bias);
        CHECK(approx(gb[0], 4.f, 1e-6f) && approx(gb[1], 4.f, 1e-6f));
        CHECK(throws([&] { (void)lin.forward(upload({1, 2}, Shape{1, 2})); }));   // in_features mismatch
    }
    // Conv2d 1x1, weight 2: out = 2 * in; backward known answers
    {
        nn::Conv2d conv(1, 1, 1, 1, 1, 1, 0, 0, 1, 1, /*bias*/ false);
        conv.weight() = upload({2.0f}, Shape{1, 1, 1, 1});
        Tensor x = upload({1, 2, 3, 4}, Shape{1, 1, 2, 2});
        auto y = download(conv.forward(x));
        for (int i = 0; i < 4; ++i) CHECK(approx(y[i], 2.f * float(i + 1), 1e-5f));
        auto gr = conv.backward(upload({0.1f, 0.2f, 0.3f, 0.4f}, Shape{1, 1, 2, 2}), x);
        auto gi = download(gr.grad_input);
        const float egi[4] = {0.2f, 0.4f, 0.6f, 0.8f};
        for (int i = 0; i < 4; ++i) CHECK(approx(gi[i], egi[i], 1e-4f));
        CHECK(approx(download(gr.grad_weight)[0], 3.0f, 1e-4f));
        CHECK(approx(download(gr.grad_bias)[0], 0.0f, 1e-6f));   // no bias: zero-filled
        // default constructor fill: weights 0.1, bias 0.05
        nn::Conv2d dflt(2, 3, 3, 3, 1, 1, 1, 1);
        CHECK(approx(download(dflt.weight())[7], 0.1f, 1e-7f) && approx(download(dflt.bias())[2], 0.05f, 1e-7f));
    }
    // allocator: a pool per device, memory really comes back
    {
        int ndev = 0;
        tfb_device_count(&ndev);
        uint64_t used0 = 0, used1 = 0, used2 = 0;
        CudaStorageAllocator::instance().stats(0, nullptr, &used0);
        {
            Tensor big = Tensor::empty(Shape{1024, 1024}, Dtype::Float32, Device::cuda(0));
            CudaStorageAllocator::instance().stats(0, nullptr, &used1);
            CHECK(used1 >= used0 + 4u * 1024 * 1024);
        }
        DeviceContext::for_device(0).synchronize();
        CudaStorageAllocator::instance().stats(0, nullptr, &used2);
        CHECK(used2 <= used1 - 4u * 1024 * 1024);
        if (ndev > 1) {
            // tensors on another device: allocated from that device's pool, multiplied there
            Tensor a1 = upload({1, 2, 3, 4}, Shape{2, 2}, Device::cuda(1)), b1 = upload({5, 6, 7, 8}, Shape{2, 2}, Device::cuda(1));
            auto c1 = download(a1.matmul(b1));
            for (int i = 0; i < 4; ++i) CHECK(approx(c1[i], expected[i], 1e-5f));
            CHECK(throws([&] { (void)A.matmul(b1); }));   // operands on different devices
        } else {
            CHECK(throws([&] { (void)Tensor::empty(Shape{2}, Dtype::Float32, Device::cuda(1)); }));   // as tensor_cuda_dispatch_test.cpp:55-58
        }
    }
    autograd_checks();
    int code = -1;
    CHECK(tfb_device_status(&code) == TFB_OK && code == 0);
}

int main(int argc, char** argv) {
    const std::string mode = argc > 1 ? argv[1] : "cpu";
    try {
        cpu_checks();
        if (mode == "gpu") gpu_checks();
    } catch (const std::exception& e) {
        std::printf("unexpected exception: %s\n", e.what());
        return 2;
    }
    std::printf("%s checks: %s\n", mode.c_str(), g_failed == 0 ? "all passed" : "FAILED");
    return g_failed == 0 ? 0 : 1;
}
