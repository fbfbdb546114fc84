// Implementation of the host mirror on libtfb's C-ABI (see tensorforge_b200.hpp).
#include "tensorforge_b200.hpp"

#include <cmath>
#include <map>
#include <random>

#include "../../include/tfb.h"

namespace tensorforge {

// autograd_b200.cpp
void record_matmul(Tensor& out, const Tensor& a, const Tensor& b);
void record_linear(Tensor& y, const Tensor& x, const Tensor& w, const Tensor& bias, int64_t in_f, int64_t out_f,
                   bool relu, bool bias_enabled);

namespace {

[[noreturn]] void raise(const char* what) {
    throw std::runtime_error(std::string(what) + ": " + tfb_last_error_string());
}
void ok(int rc, const char* what) {
    if (rc != TFB_OK) raise(what);
}

MatmulFn g_cuda_matmul = nullptr;

void tfb_matmul_trampoline(const void* a, const void* b, void* c, int64_t M, int64_t N, int64_t K, Dtype in, Dtype out,
                           void* stream) {
    ok(tfb_matmul(a, b, c, M, N, K, int(in), int(out), stream), "tfb_matmul");
}

struct RegisterOnLoad {
    RegisterOnLoad() { tfb_register_kernels(); }
};
RegisterOnLoad g_register_on_load;

thread_local std::map<int32_t, DeviceContext> t_contexts;
thread_local int32_t t_current_device = 0;

}  // namespace

size_t dtype_size(Dtype d) {
    switch (d) {
    case Dtype::Float32: case Dtype::Int32: return 4;
    case Dtype::Float16: case Dtype::BFloat16: return 2;
    case Dtype::Int64: return 8;
    case Dtype::Bool: return 1;
    }
    return 0;
}

// ---- DeviceContext ----------------------------------------------------------------------------------
DeviceContext& DeviceContext::for_device(int32_t device_index) {
    auto it = t_contexts.find(device_index);
    if (it == t_contexts.end()) {
        DeviceContext ctx;
        ctx.device_index = device_index;
        ok(tfb_stream_create(device_index, &ctx.current_stream), "tfb_stream_create");
        it = t_contexts.emplace(device_index, ctx).first;
    }
    return it->second;
}
DeviceContext& DeviceContext::current() { return for_device(t_current_device); }
void DeviceContext::synchronize() const { ok(tfb_stream_synchronize(current_stream), "tfb_stream_synchronize"); }

DeviceGuard::DeviceGuard(int32_t device_index) : prev_(t_current_device) {
    ok(tfb_set_device(device_index), "tfb_set_device");
    t_current_device = device_index;
}
DeviceGuard::~DeviceGuard() {
    t_current_device = prev_;
    (void)tfb_set_device(prev_);
}

// ---- storage ----------------------------------------------------------------------------------------
StorageImpl::~StorageImpl() {
    // Freed on the stream that allocated it, not on the destroying thread's stream: work that thread A
    // queued on the buffer is ordered before the release even when thread B drops the last reference.
    if (ptr != nullptr && device.type == DeviceType::CUDA)
        (void)tfb_free(ptr, device.index, stream != nullptr ? stream : DeviceContext::for_device(device.index).current_stream);
    else if (ptr != nullptr)
        ::operator delete(ptr);
}

CudaStorageAllocator& CudaStorageAllocator::instance() {
    static CudaStorageAllocator inst;
    return inst;
}

Storage CudaStorageAllocator::allocate(size_t size_bytes, Device device, Dtype dtype) {
    if (device.type != DeviceType::CUDA)
        throw std::invalid_argument("CudaStorageAllocator can only allocate CUDA storage");
    void* p = nullptr;
    void* stream = DeviceContext::for_device(device.index).current_stream;
    ok(tfb_alloc(device.index, size_bytes, stream, &p), "tfb_alloc");
    auto s = std::make_shared<StorageImpl>();
    s->ptr = p; s->bytes = size_bytes; s->device = device; s->dtype = dtype; s->stream = stream;
    return s;
}
void CudaStorageAllocator::stats(int32_t device_index, uint64_t* reserved, uint64_t* used) const {
    ok(tfb_pool_stats(device_index, reserved, used, nullptr, nullptr), "tfb_pool_stats");
}
void CudaStorageAllocator::trim(int32_t device_index, size_t keep_bytes) const {
    ok(tfb_pool_trim(device_index, keep_bytes), "tfb_pool_trim");
}

// ---- registry ---------------------------------------------------------------------------------------
void register_cuda_matmul(MatmulFn fn) { g_cuda_matmul = fn; }
MatmulFn registered_cuda_matmul() { return g_cuda_matmul; }
void tfb_register_kernels() { register_cuda_matmul(&tfb_matmul_trampoline); }

void launch_gemm_naive(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K, Dtype dtype, void* stream) {
    ok(tfb_gemm(A, B, C, M, N, K, int(dtype), stream), "tfb_gemm");
}
void launch_gemm_tiled_16x16(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K, Dtype dtype, void* stream) {
    ok(tfb_gemm(A, B, C, M, N, K, int(dtype), stream), "tfb_gemm");
}
void launch_gemm_optimized(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K, Dtype dtype, void* stream) {
    ok(tfb_gemm(A, B, C, M, N, K, int(dtype), stream), "tfb_gemm");
}

// ---- Tensor -----------------------------------------------------------------------------------------
Tensor Tensor::empty(Shape shape, Dtype dtype, Device device) {
    Tensor t;
    const size_t bytes = static_cast<size_t>(shape.numel()) * dtype_size(dtype);
    if (device.type == DeviceType::CUDA) {
        t.storage_ = CudaStorageAllocator::instance().allocate(bytes, device, dtype);
    } else {
        auto s = std::make_shared<StorageImpl>();
        s->ptr = ::operator new(bytes > 0 ? bytes : 1);
        s->bytes = bytes; s->device = device; s->dtype = dtype;
        t.storage_ = s;
    }
    t.shape_ = std::move(shape);
    return t;
}

Tensor Tensor::from_host(const void* src, Shape shape, Dtype dtype, Device device) {
    Tensor t = Tensor::empty(std::move(shape), dtype, device);
    const size_t bytes = static_cast<size_t>(t.numel()) * dtype_size(dtype);
    if (device.type == DeviceType::CUDA) {
        DeviceGuard g(device.index);
        auto& ctx = DeviceContext::for_device(device.index);
        ok(tfb_memcpy(t.data(), src, bytes, 1, ctx.current_stream), "tfb_memcpy");
        ctx.synchronize();   // the source may be a temporary
    } else {
        ok(tfb_memcpy(t.data(), src, bytes, 0, nullptr), "tfb_memcpy");
    }
    return t;
}

void Tensor::copy_to_host(void* dst) const {
    const size_t bytes = static_cast<size_t>(numel()) * dtype_size(dtype());
    if (device().type == DeviceType::CUDA) {
        DeviceGuard g(device().index);
        auto& ctx = DeviceContext::for_device(device().index);
        ok(tfb_memcpy(dst, data(), bytes, 2, ctx.current_stream), "tfb_memcpy");
        ctx.synchronize();
    } else {
        ok(tfb_memcpy(dst, data(), bytes, 0, nullptr), "tfb_memcpy");
    }
}

Tensor Tensor::matmul(const Tensor& other) const {
    if (shape_.ndim() != 2 || other.shape_.ndim() != 2)
        throw std::invalid_argument("Tensor::matmul: both operands must be 2D for v1");
    if (shape_[1] != other.shape_[0])
        throw std::invalid_argument("Tensor::matmul: shape mismatch (a.cols != b.rows)");
    if (device().type != DeviceType::CUDA || other.device().type != DeviceType::CUDA)
        throw std::invalid_argument("Tensor::matmul: this library serves CUDA tensors; CPU tensors stay on the reference loop");
    if (device() != other.device()) throw std::invalid_argument("Tensor::matmul: operands live on different devices");
    if (dtype() != other.dtype()) throw std::invalid_argument("Tensor::matmul: dtype mismatch");
    if (dtype() != Dtype::Float32 && dtype() != Dtype::Float16 && dtype() != Dtype::BFloat16)
        throw std::invalid_argument("Tensor::matmul: Float32, Float16 or BFloat16 only");
    if (g_cuda_matmul == nullptr) throw std::runtime_error("CUDA matmul kernel not registered");
    const int64_t M = shape_[0], K = shape_[1], N = other.shape_[1];
    DeviceGuard g(device().index);
    // The result has the operands' dtype, the reference's rule (tensor/Tensor.cpp:350); accumulation is
    // FP32 whatever the storage type. MatmulBackward relies on it: the upstream gradient it receives
    // then has the dtype it passes to tfb_matmul_backward.
    Tensor out = Tensor::empty(Shape{M, N}, dtype(), device());
    g_cuda_matmul(data(), other.data(), out.data(), M, N, K, dtype(), dtype(),
                  DeviceContext::for_device(device().index).current_stream);
    record_matmul(out, *this, other);
    return out;
}

std::vector<Tensor> MatmulBackward::apply(std::vector<Tensor>&& grads) {
    const Tensor& g = grads.at(0);
    const int64_t M = a_.shape()[0], K = a_.shape()[1], N = b_.shape()[1];
    DeviceGuard guard(a_.device().index);
    Tensor ga = Tensor::empty(Shape{M, K}, a_.dtype(), a_.device());
    Tensor gb = Tensor::empty(Shape{K, N}, b_.dtype(), b_.device());
    ok(tfb_matmul_backward(g.data(), a_.data(), b_.data(), ga.data(), gb.data(), M, N, K, int(a_.dtype()),
                           DeviceContext::for_device(a_.device().index).current_stream),
       "tfb_matmul_backward");
    return {std::move(ga), std::move(gb)};
}

namespace nn {

Linear::Linear(int in_features, int out_features, bool bias, Device device)
    : in_features_(in_features), out_features_(out_features), bias_enabled_(bias) {
    std::vector<float> w(static_cast<size_t>(in_features) * out_features);
    const float bound = std::sqrt(1.0f / static_cast<float>(in_features));
    std::mt19937 rng(0xC0FFEEu);
    std::uniform_real_distribution<float> dist(-bound, bound);
    for (float& v : w) v = dist(rng);
    weight_ = Tensor::from_host(w.data(), Shape{out_features, in_features}, Dtype::Float32, device);
    if (bias_enabled_) {
        std::vector<float> b(static_cast<size_t>(out_features), 0.0f);
        bias_ = Tensor::from_host(b.data(), Shape{out_features}, Dtype::Float32, device);
    }
}

Tensor Linear::forward(Tensor x, bool fuse_relu) {
    if (x.dtype() != Dtype::Float32) throw std::invalid_argument("Linear.forward: only Float32 supported");
    if (x.shape().ndim() != 2) throw std::invalid_argument("Linear.forward expects 2D input [N, in_features]");
    if (x.shape()[1] != in_features_) throw std::invalid_argument("Linear.forward: in_features mismatch");
    if (x.device().type != DeviceType::CUDA) throw std::invalid_argument("Linear.forward: CUDA tensors only");
    DeviceGuard g(x.device().index);
    const int64_t batch = x.shape()[0];
    Tensor y = Tensor::empty(Shape{batch, out_features_}, Dtype::Float32, x.device());
    ok(tfb_linear_forward(x.data(), weight_.data(), bias_enabled_ ? static_cast<const float*>(bias_.data()) : nullptr,
                          y.data(), batch, in_features_, out_features_, fuse_relu ? 1 : 0, TFB_DTYPE_F32,
                          DeviceContext::for_device(x.device().index).current_stream),
       "tfb_linear_forward");
    record_linear(y, x, weight_, bias_, in_features_, out_features_, fuse_relu, bias_enabled_);
    return y;
}

Linear::Grads Linear::backward(const Tensor& x, const Tensor& y, const Tensor& dy, bool fuse_relu) {
    DeviceGuard g(x.device().index);
    const int64_t batch = x.shape()[0];
    Grads r;
    r.grad_input = Tensor::empty(Shape{batch, in_features_}, Dtype::Float32, x.device());
    r.grad_weight = Tensor::empty(Shape{out_features_, in_features_}, Dtype::Float32, x.device());
    r.grad_bias = Tensor::empty(Shape{out_features_}, Dtype::Float32, x.device());
    ok(tfb_linear_backward(x.data(), weight_.data(), y.data(), dy.data(), r.grad_input.data(), r.grad_weight.data(),
                           static_cast<float*>(r.grad_bias.data()), batch, in_features_, out_features_,
                           fuse_relu ? 1 : 0, TFB_DTYPE_F32, DeviceContext::for_device(x.device().index).current_stream),
       "tfb_linear_backward");
    return r;
}

Conv2d::Conv2d(int64_t in_channels, int64_t out_channels, int64_t kernel_h, int64_t kernel_w, int64_t stride_h,
               int64_t stride_w, int64_t pad_h, int64_t pad_w, int64_t dilation_h, int64_t dilation_w, bool bias_enabled)
    : in_channels_(in_channels), out_channels_(out_channels), kernel_h_(kernel_h), kernel_w_(kernel_w),
      stride_h_(stride_h), stride_w_(stride_w), pad_h_(pad_h), pad_w_(pad_w), dilation_h_(dilation_h),
      dilation_w_(dilation_w), bias_enabled_(bias_enabled) {
    std::vector<float> w(static_cast<size_t>(out_channels * in_channels * kernel_h * kernel_w), 0.1f);
    weight_ = Tensor::from_host(w.data(), Shape{out_channels, in_channels, kernel_h, kernel_w}, Dtype::Float32, Device::cuda(0));
    if (bias_enabled_) {
        std::vector<float> b(static_cast<size_t>(out_channels), 0.05f);
        bias_ = Tensor::from_host(b.data(), Shape{out_channels}, Dtype::Float32, Device::cuda(0));
    }
}

int64_t Conv2d::out_h(int64_t H) const { return tfb_conv_out_dim(H, kernel_h_, stride_h_, pad_h_, dilation_h_); }
int64_t Conv2d::out_w(int64_t W) const { return tfb_conv_out_dim(W, kernel_w_, stride_w_, pad_w_, dilation_w_); }

Tensor Conv2d::forward(Tensor input) {
    const Shape& s = input.shape();
    if (s.ndim() != 4) throw std::invalid_argument("Conv2d.forward expects [N, Cin, H, W]");
    if (s[1] != in_channels_) throw std::invalid_argument("Conv2d.forward: Cin mismatch");
    DeviceGuard g(input.device().index);
    Tensor out = Tensor::empty(Shape{s[0], out_channels_, out_h(s[2]), out_w(s[3])}, input.dtype(), input.device());
    ok(tfb_conv2d_forward(input.data(), weight_.data(), bias_enabled_ ? static_cast<const float*>(bias_.data()) : nullptr,
                          out.data(), s[0], s[1], s[2], s[3], out_channels_, kernel_h_, kernel_w_, stride_h_, stride_w_,
                          pad_h_, pad_w_, dilation_h_, dilation_w_, 0, int(input.dtype()),
                          DeviceContext::for_device(input.device().index).current_stream),
       "tfb_conv2d_forward");
    return out;
}

Conv2dGrad Conv2d::backward(Tensor grad_output, Tensor input) {
    const Shape& go = grad_output.shape();
    const Shape& in = input.shape();
    if (go.ndim() != 4) throw std::invalid_argument("Conv2d.backward: grad_output must be [N, Cout, outH, outW]");
    if (in.ndim() != 4) throw std::invalid_argument("Conv2d.backward: input must be [N, Cin, H, W]");
    if (go[1] != out_channels_ || in[1] != in_channels_) throw std::invalid_argument("Conv2d.backward: channel mismatch");
    DeviceGuard g(input.device().index);
    void* stream = DeviceContext::for_device(input.device().index).current_stream;
    Conv2dGrad r;
    r.grad_input = Tensor::empty(Shape{in[0], in[1], in[2], in[3]}, input.dtype(), input.device());
    r.grad_weight = Tensor::empty(Shape{out_channels_, in_channels_, kernel_h_, kernel_w_}, input.dtype(), input.device());
    std::vector<float> zeros(static_cast<size_t>(out_channels_), 0.0f);
    r.grad_bias = Tensor::from_host(zeros.data(), Shape{out_channels_}, Dtype::Float32, input.device());
    ok(tfb_conv2d_backward(input.data(), weight_.data(), grad_output.data(), r.grad_input.data(), r.grad_weight.data(),
                           bias_enabled_ ? static_cast<float*>(r.grad_bias.data()) : nullptr, in[0], in[1], in[2], in[3],
                           out_channels_, kernel_h_, kernel_w_, stride_h_, stride_w_, pad_h_, pad_w_, dilation_h_,
                           dilation_w_, int(input.dtype()), stream),
       "tfb_conv2d_backward");
    return r;
}

}  // namespace nn
}  // namespace tensorforge
