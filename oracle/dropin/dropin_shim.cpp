// TEST INFRASTRUCTURE: a C entry point over the PATCHED reference (see apply_dropin.py) so that a test
// can run the reference's own Tensor::matmul and Tensor::backward on Device::cuda(0) tensors — the
// reference's classes, allocator, autograd engine and call sites, with libtfb underneath.
#include <cstdint>
#include <cstring>
#include <exception>
#include <string>

#include <cuda_runtime.h>

#include "cuda/CudaContext.hpp"
#include "tensor/AutogradWirer.hpp"
#include "tensor/Tensor.hpp"

using namespace tensorforge;

namespace {
thread_local std::string g_error;

Tensor upload(const float* src, int64_t rows, int64_t cols) {
    Tensor host = Tensor::empty(Shape{rows, cols}, Dtype::Float32, Device::cpu());
    std::memcpy(host.data(), src, static_cast<size_t>(rows * cols) * 4);
    return host.to(Device::cuda(0));
}

void download(const Tensor& t, float* dst) {
    Tensor host = t.to(Device::cpu());
    cudaStreamSynchronize(DeviceContext::current().current_stream);
    std::memcpy(dst, host.data(), static_cast<size_t>(host.numel()) * 4);
}
}  // namespace

extern "C" {

const char* dropin_last_error() { return g_error.c_str(); }

// C = A · B through the reference's Tensor::matmul on CUDA tensors.
int dropin_matmul(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K) {
    try {
        init_tensor_autograd();
        Tensor a = upload(A, M, K), b = upload(B, K, N);
        Tensor c = a.matmul(b);
        if (c.device().type != DeviceType::CUDA) throw std::runtime_error("the product did not stay on the device");
        download(c, C);
        return 0;
    } catch (const std::exception& e) {
        g_error = e.what();
        return 1;
    }
}

// c = a.matmul(b); c.backward() with a root gradient of ones: a.grad() and b.grad().
int dropin_matmul_backward(const float* A, const float* B, float* dA, float* dB, int64_t M, int64_t N, int64_t K) {
    try {
        init_tensor_autograd();
        Tensor a = upload(A, M, K), b = upload(B, K, N);
        a.requires_grad(true);
        b.requires_grad(true);
        Tensor c = a.matmul(b);
        c.backward();
        download(a.grad(), dA);
        download(b.grad(), dB);
        return 0;
    } catch (const std::exception& e) {
        g_error = e.what();
        return 1;
    }
}

// The checks of the reference's own Tensor::matmul still apply on the device path: 0 = threw as expected.
int dropin_matmul_shape_mismatch_throws() {
    try {
        const float z[6] = {0, 0, 0, 0, 0, 0};
        Tensor a = upload(z, 2, 3), b = upload(z, 2, 3);
        (void)a.matmul(b);
        return 1;
    } catch (const std::invalid_argument&) {
        return 0;
    } catch (...) {
        return 2;
    }
}

}  // extern "C"
