// Host-side mirror of the reference's interface for the dense-contraction path, implemented on
// libtfb's C-ABI. Class, function and parameter names follow the reference (namespace tensorforge)
// so that its call sites and tests read the same:
//
//   Dtype / Device / Shape            tensor/Dtype.hpp:9-16, tensor/Device.hpp, tensor/Shape.hpp
//   Tensor::{empty,to,matmul,relu}    tensor/Tensor.hpp:17-128, tensor/Tensor.cpp:334-368
//   register_cuda_matmul, MatmulFn    the slot added beside cuda/CudaKernelRegistry.hpp:15-26
//   launch_gemm_*                     cuda/kernels/gemm.cuh:33-53
//   DeviceContext, DeviceGuard        cuda/CudaContext.hpp:134-140, cuda/CudaContext.cpp:18-60
//   CudaStorageAllocator              cuda/memory/CudaStorageAllocator.hpp
//   MatmulBackward                    autograd/ops/MatmulBackward.hpp:26-34
//   Node, Edge, Engine, AccumulateGrad autograd/Node.hpp:14-45, autograd/Engine.hpp:12-30, autograd/AccumulateGrad.cpp:10-27
//   ReluBackward, Tensor::backward    autograd/ops/ReluBackward.hpp:22-32, autograd/TensorAutograd.cpp:52-73
//   cross_entropy                     the loss graph of examples/train_mlp.cpp:54-76, as one node
//   nn::Linear, nn::Conv2d            nn/Linear.hpp, nn/Conv2d.hpp:32-61
//   nn::Conv2dModule                  nn/Conv2dModule.hpp:16-32, nn/Conv2dModule.cpp:74-106
//
// Only CUDA tensors are served: CPU tensors stay on the reference's own loops, and there is no
// fallback of any kind — a missing registration or a failing library call throws.
// This header needs no CUDA headers (g++ -std=c++20 is enough), like the reference's host code.
#pragma once

#include <cstddef>
#include <cstdint>
#include <initializer_list>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

namespace tensorforge {

enum class Dtype : uint8_t { Float32 = 0, Float16 = 1, BFloat16 = 2, Int32 = 3, Int64 = 4, Bool = 5 };
size_t dtype_size(Dtype d);

enum class DeviceType : uint8_t { CPU = 0, CUDA = 1 };
struct Device {
    DeviceType type = DeviceType::CPU;
    int32_t index = 0;
    static Device cpu() { return Device{DeviceType::CPU, 0}; }
    static Device cuda(int32_t i = 0) { return Device{DeviceType::CUDA, i}; }
    bool operator==(const Device& o) const { return type == o.type && index == o.index; }
    bool operator!=(const Device& o) const { return !(*this == o); }
};

class Shape {
public:
    Shape() = default;
    Shape(std::initializer_list<int64_t> d) : dims_(d) {}
    explicit Shape(std::vector<int64_t> d) : dims_(std::move(d)) {}
    size_t ndim() const { return dims_.size(); }
    int64_t operator[](size_t i) const { return dims_.at(i); }
    int64_t numel() const {
        int64_t n = 1;
        for (int64_t d : dims_) n *= d;
        return n;
    }
    bool operator==(const Shape& o) const { return dims_ == o.dims_; }

private:
    std::vector<int64_t> dims_;
};

// ---- streams and devices ----------------------------------------------------------------------
// One non-blocking stream per (thread, device); current() follows the innermost DeviceGuard.
struct DeviceContext {
    int32_t device_index = 0;
    void* current_stream = nullptr;
    static DeviceContext& current();
    static DeviceContext& for_device(int32_t device_index);
    void synchronize() const;
};

class DeviceGuard {
public:
    explicit DeviceGuard(int32_t device_index);
    ~DeviceGuard();
    DeviceGuard(const DeviceGuard&) = delete;
    DeviceGuard& operator=(const DeviceGuard&) = delete;

private:
    int32_t prev_;
};

// ---- storage ------------------------------------------------------------------------------------
struct StorageImpl {
    void* ptr = nullptr;
    size_t bytes = 0;
    Device device;
    Dtype dtype = Dtype::Float32;
    void* stream = nullptr;   // the stream the memory was allocated on (CUDA storage)
    ~StorageImpl();   // returns device memory to its pool, stream-ordered
};
using Storage = std::shared_ptr<StorageImpl>;

class CudaStorageAllocator {
public:
    static CudaStorageAllocator& instance();
    Storage allocate(size_t size_bytes, Device device, Dtype dtype);
    // Bytes the device's pool currently holds / has handed out.
    void stats(int32_t device_index, uint64_t* reserved, uint64_t* used) const;
    void trim(int32_t device_index, size_t keep_bytes = 0) const;
};

// ---- kernel registry (the added matmul slot) --------------------------------------------------------
using MatmulFn = void (*)(const void* a, const void* b, void* c, int64_t M, int64_t N, int64_t K, Dtype in,
                          Dtype out, void* stream);
void register_cuda_matmul(MatmulFn fn);
MatmulFn registered_cuda_matmul();
// Registers libtfb's kernels. Also runs from a static initialiser of the mirror library; the
// explicit call exists for consumers that link statically (same reason as init_tensor_autograd()).
void tfb_register_kernels();

// ---- launchers with the reference's signatures ------------------------------------------------------
void launch_gemm_naive(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K, Dtype dtype, void* stream);
void launch_gemm_tiled_16x16(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K, Dtype dtype, void* stream);
void launch_gemm_optimized(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K, Dtype dtype, void* stream);

// ---- Tensor ---------------------------------------------------------------------------------------
class Node;
struct AutogradMeta;
struct Edge {
    std::shared_ptr<Node> function;
    uint32_t input_nr = 0;
};

class Tensor {
public:
    Tensor() = default;
    static Tensor empty(Shape shape, Dtype dtype, Device device);
    // Host <-> device helpers the reference spreads over factory.cpp / Tensor::to.
    static Tensor from_host(const void* src, Shape shape, Dtype dtype, Device device);
    void copy_to_host(void* dst) const;   // synchronises the tensor's stream

    void* data() noexcept { return storage_ ? storage_->ptr : nullptr; }
    const void* data() const noexcept { return storage_ ? storage_->ptr : nullptr; }
    int64_t numel() const noexcept { return shape_.numel(); }
    const Shape& shape() const noexcept { return shape_; }
    Dtype dtype() const noexcept { return storage_ ? storage_->dtype : Dtype::Float32; }
    Device device() const noexcept { return storage_ ? storage_->device : Device::cpu(); }

    // C[M,N] = this[M,K] · other[K,N]. CUDA tensors of one device; the result has the operands' dtype
    // (Float32, Float16 or BFloat16; FP32 accumulation), as in the reference. Same argument checks and messages as
    // the reference (tensor/Tensor.cpp:335-346) where they still apply. Records a MatmulBackward
    // node when an operand requires a gradient.
    Tensor matmul(const Tensor& other) const;
    // max(x, 0) on the device; records a ReluBackward node when this tensor requires a gradient.
    Tensor relu() const;

    // Autograd, with the reference's names (tensor/Tensor.hpp:65-68). Everything a backward pass does
    // to tensor data — the ones-fill of the root gradient, masks, accumulation — runs on the device.
    void requires_grad(bool req);
    bool requires_grad() const noexcept;
    Tensor grad() const;            // an empty Tensor (no storage) until a backward pass reached it
    void backward();                // root gradient of ones; throws without a grad_fn
    bool defined() const noexcept { return static_cast<bool>(storage_); }

    // Plumbing for code that records nodes (nn::Linear, cross_entropy).
    std::shared_ptr<Node> grad_fn() const;
    void set_grad_fn(std::shared_ptr<Node> fn, uint32_t output_nr = 0);
    Edge gradient_edge() const;     // where this tensor's gradient flows: its grad_fn, or a leaf's accumulator

private:
    Storage storage_;
    Shape shape_;
    std::shared_ptr<AutogradMeta> autograd_meta_;
};

// ---- autograd graph -------------------------------------------------------------------------------
class Node : public std::enable_shared_from_this<Node> {
public:
    std::vector<Edge> next_edges_;   // towards the nodes that produced this node's inputs
    uint64_t sequence_nr_ = 0;       // creation order; the engine prefers later nodes among ready ones
    Node();
    virtual std::vector<Tensor> apply(std::vector<Tensor>&& grads) = 0;
    virtual void release_saved() {}
    virtual ~Node() = default;
};

struct AutogradMeta {
    bool requires_grad_ = false;
    Tensor grad_;
    std::shared_ptr<Node> grad_fn_;
    uint32_t output_nr_ = 0;
    std::shared_ptr<Node> grad_accumulator_;   // created on first use for leaves
};

// Leaf sink: stores the incoming gradient as the tensor's grad, replacing an earlier one as the
// reference does (autograd/AccumulateGrad.cpp:20-23).
class AccumulateGrad : public Node {
public:
    explicit AccumulateGrad(std::weak_ptr<AutogradMeta> meta);
    std::vector<Tensor> apply(std::vector<Tensor>&& grads) override;

private:
    std::weak_ptr<AutogradMeta> meta_;
};

class Engine {
public:
    // Runs the graph below `root` once: a node runs when every consumer of its output has delivered
    // its gradient; gradients meeting at one input are added on the device.
    void execute(std::shared_ptr<Node> root, const Tensor& initial_grad, bool keep_graph = false);
};

class ReluBackward : public Node {
public:
    explicit ReluBackward(const Tensor& input) : input_(input) {}
    std::vector<Tensor> apply(std::vector<Tensor>&& grads) override;
    void release_saved() override { input_ = Tensor(); }

private:
    Tensor input_;
};

// loss[1] = -(1/N) * sum_i log_softmax(logits)[i, labels[i]] for logits [N, C] (Float32) and labels [N]
// (Int64), both on one CUDA device: the loss of examples/train_mlp.cpp:54-76 computed by one kernel,
// which also leaves d loss / d logits for the backward node.
Tensor cross_entropy(const Tensor& logits, const Tensor& labels);

// ---- autograd node ----------------------------------------------------------------------------------
class MatmulBackward : public Node {
public:
    MatmulBackward(const Tensor& a, const Tensor& b) : a_(a), b_(b) {}
    // {dA, dB} = {grad · Bᵀ, Aᵀ · grad}, no transpose copies.
    std::vector<Tensor> apply(std::vector<Tensor>&& grads) override;
    void release_saved() override { a_ = Tensor(); b_ = Tensor(); }

private:
    Tensor a_, b_;
};

namespace nn {

class Linear {
public:
    // Same initialisation as the reference: weight [out, in] ~ U(±sqrt(1/in)) from mt19937(0xC0FFEE),
    // bias zeros; parameters are created on `device`.
    Linear(int in_features, int out_features, bool bias = true, Device device = Device::cuda(0));
    // y = x · Wᵀ + b. The bias IS applied (it is zero-initialised, so results equal the reference's,
    // which registers the bias and leaves it out). fuse_relu applies ReLU in the same kernel.
    // When x, the weight or the bias requires a gradient, one node computing all three gradients
    // (tfb_linear_backward) is recorded.
    Tensor forward(Tensor x, bool fuse_relu = false);
    struct Grads {
        Tensor grad_input, grad_weight, grad_bias;
    };
    // Backward for upstream gradient dy; y is the forward output (needed when fuse_relu was set).
    Grads backward(const Tensor& x, const Tensor& y, const Tensor& dy, bool fuse_relu = false);
    Tensor& weight() { return weight_; }
    Tensor& bias() { return bias_; }
    int in_features() const noexcept { return in_features_; }
    int out_features() const noexcept { return out_features_; }

private:
    int in_features_, out_features_;
    bool bias_enabled_;
    Tensor weight_, bias_;
};

struct Conv2dGrad {
    Tensor grad_input, grad_weight, grad_bias;
};

class Conv2d {
public:
    // Weights constant 0.1 and bias constant 0.05 on cuda(0), as the reference constructor fills them
    // (nn/Conv2d.cpp:57-66).
    Conv2d(int64_t in_channels, int64_t out_channels, int64_t kernel_h, int64_t kernel_w, int64_t stride_h = 1,
           int64_t stride_w = 1, int64_t pad_h = 0, int64_t pad_w = 0, int64_t dilation_h = 1,
           int64_t dilation_w = 1, bool bias_enabled = true);
    Tensor forward(Tensor input);
    Conv2dGrad backward(Tensor grad_output, Tensor input);
    Tensor& weight() { return weight_; }
    Tensor& bias() { return bias_; }
    int64_t out_h(int64_t H) const;
    int64_t out_w(int64_t W) const;
    bool bias_enabled() const noexcept { return bias_enabled_; }

private:
    int64_t in_channels_, out_channels_, kernel_h_, kernel_w_, stride_h_, stride_w_, pad_h_, pad_w_, dilation_h_,
        dilation_w_;
    bool bias_enabled_;
    Tensor weight_, bias_;
};

// The trainable convolution of the reference (nn/Conv2dModule.hpp:16-32, nn/Conv2dModule.cpp:74-106), on
// the GPU: square kernel / stride / padding / dilation, weight ~ U(±sqrt(1/(Cin·k·k))) from
// mt19937(0xC0FFEE), zero bias, both requiring gradients. forward() records one node that computes the
// input, weight and bias gradients with tfb_conv2d_backward.
class Conv2dModule {
public:
    Conv2dModule(int in_channels, int out_channels, int kernel_size, int stride = 1, int padding = 0,
                 int dilation = 1, bool bias = true, Device device = Device::cuda(0));
    Tensor forward(Tensor x);
    Tensor& weight() { return weight_; }
    Tensor& bias() { return bias_; }

private:
    int in_channels_, out_channels_, kernel_size_, stride_, padding_, dilation_;
    bool bias_enabled_;
    Tensor weight_, bias_;
};

}  // namespace nn
}  // namespace tensorforge
