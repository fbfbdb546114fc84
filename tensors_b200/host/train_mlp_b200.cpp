// A training loop over the host mirror, in the shape of the reference's MLP example
// (examples/train_mlp.cpp:161-183): Linear -> relu -> Linear -> cross_entropy -> backward -> SGD, every
// tensor on the GPU for the whole run. The data is synthetic (seeded): ten fixed random prototype
// images plus noise, pixel statistics of normalised MNIST digits; the labels are the prototype indices,
// so the loss has something to learn.
//   train_mlp_b200 [steps=60] [batch=256] [hidden=128]
// Prints the loss every ten steps and exits 0 when the final loss is below half of the first one.
#include <cstdio>
#include <cstdlib>
#include <random>
#include <vector>

#include "../../include/tfb.h"
#include "tensorforge_b200.hpp"

using namespace tensorforge;

namespace {

// p <- p - lr * g with zero momentum: the plain update of the reference example's manual step
// (examples/train_mlp.cpp:140-158), as one device kernel per parameter.
void sgd_update(Tensor& param, float lr, std::vector<Tensor>& velocity, size_t slot) {
    Tensor g = param.grad();
    if (!g.defined()) return;
    if (velocity.size() <= slot) velocity.resize(slot + 1);
    if (!velocity[slot].defined()) velocity[slot] = Tensor::empty(param.shape(), Dtype::Float32, param.device());
    void* stream = DeviceContext::for_device(param.device().index).current_stream;
    if (tfb_sgd_momentum(static_cast<float*>(param.data()), static_cast<float*>(velocity[slot].data()),
                         static_cast<const float*>(g.data()), param.numel(), lr, 0.0f, 1.0f, stream) != TFB_OK)
        throw std::runtime_error(tfb_last_error_string());
}

}  // namespace

int main(int argc, char** argv) {
    const int steps = argc > 1 ? std::atoi(argv[1]) : 60;
    const int64_t batch = argc > 2 ? std::atoll(argv[2]) : 256;
    const int hidden = argc > 3 ? std::atoi(argv[3]) : 128;
    const int64_t D = 784, C = 10;
    try {
        std::mt19937 rng(1234u);
        std::normal_distribution<float> noise(0.f, 0.5f);
        std::uniform_real_distribution<float> pixel(0.f, 1.f);
        std::vector<float> proto(static_cast<size_t>(C * D));
        for (float& v : proto) v = (pixel(rng) - 0.1307f) / 0.3081f;
        std::vector<float> xh(static_cast<size_t>(batch * D));
        std::vector<int64_t> yh(static_cast<size_t>(batch));
        for (int64_t i = 0; i < batch; ++i) {
            yh[i] = static_cast<int64_t>(rng() % C);
            for (int64_t j = 0; j < D; ++j) xh[i * D + j] = proto[yh[i] * D + j] + noise(rng);
        }
        Tensor x = Tensor::from_host(xh.data(), Shape{batch, D}, Dtype::Float32, Device::cuda(0));
        Tensor y = Tensor::from_host(yh.data(), Shape{batch}, Dtype::Int64, Device::cuda(0));

        nn::Linear fc1(static_cast<int>(D), hidden), fc2(hidden, static_cast<int>(C));
        Tensor* params[4] = {&fc1.weight(), &fc1.bias(), &fc2.weight(), &fc2.bias()};
        for (Tensor* p : params) p->requires_grad(true);
        std::vector<Tensor> velocity;
        float first = 0.f, last = 0.f;
        for (int step = 0; step < steps; ++step) {
            Tensor h = fc1.forward(x).relu();
            Tensor logits = fc2.forward(h);
            Tensor loss = cross_entropy(logits, y);
            loss.backward();
            for (size_t k = 0; k < 4; ++k) sgd_update(*params[k], 0.05f, velocity, k);
            if (step % 10 == 0 || step == steps - 1) {
                loss.copy_to_host(&last);   // the only host read of the loop
                if (step == 0) first = last;
                std::printf("[train_mlp_b200] step=%d loss=%.6f\n", step, last);
            }
        }
        int code = -1;
        if (tfb_device_status(&code) != TFB_OK || code != 0) {
            std::printf("device error %d\n", code);
            return 3;
        }
        std::printf("[train_mlp_b200] first_loss=%.6f final_loss=%.6f\n", first, last);
        return last < 0.5f * first ? 0 : 1;
    } catch (const std::exception& e) {
        std::printf("exception: %s\n", e.what());
        return 2;
    }
}
