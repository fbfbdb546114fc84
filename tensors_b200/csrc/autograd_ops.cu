// Device-side pieces of the autograd walk for FP32 tensors: the loops the reference runs on the host
// while it dereferences tensor data (root gradient fill, ReLU and its mask, gradient accumulation),
// as HBM-bound vector kernels so that a backward pass over CUDA tensors never touches the host.
#include "internal.hpp"

namespace tfb {

namespace {

enum VecOp : int { kOpFill = 0, kOpRelu = 1, kOpReluBackward = 2, kOpAccumulate = 3, kOpScaleByScalar = 4 };

// One kernel, five element-wise operations; float4 when every pointer is 16-byte aligned.
//   fill:  dst = value            relu: dst = max(a, 0)          relu backward: dst = a > 0 ? b : 0
//   accumulate: dst += a          scale: dst = a * scalar[0]
template <int OP>
__global__ void vec_kernel(float* __restrict__ dst, const float* __restrict__ a, const float* __restrict__ b,
                           const float* __restrict__ scalar, float value, long long n, int vec) {
    const float s = (OP == kOpScaleByScalar) ? __ldg(scalar) : value;
    auto f = [&](float d, float x, float y) -> float {
        if (OP == kOpFill) return s;
        if (OP == kOpRelu) return x > 0.f ? x : 0.f;
        if (OP == kOpReluBackward) return x > 0.f ? y : 0.f;
        if (OP == kOpAccumulate) return d + x;
        return x * s;
    };
    const long long stride = (long long)gridDim.x * blockDim.x;
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (vec) {
        const long long n4 = n >> 2;
        for (long long j = i; j < n4; j += stride) {
            float4 d = (OP == kOpAccumulate) ? reinterpret_cast<float4*>(dst)[j] : make_float4(0.f, 0.f, 0.f, 0.f);
            const float4 x = (OP != kOpFill) ? reinterpret_cast<const float4*>(a)[j] : d;
            const float4 y = (OP == kOpReluBackward) ? reinterpret_cast<const float4*>(b)[j] : d;
            reinterpret_cast<float4*>(dst)[j] = make_float4(f(d.x, x.x, y.x), f(d.y, x.y, y.y), f(d.z, x.z, y.z), f(d.w, x.w, y.w));
        }
        i += n4 << 2;   // the tail: elements n4*4 .. n-1
        if (i < n) dst[i] = f(OP == kOpAccumulate ? dst[i] : 0.f, OP != kOpFill ? a[i] : 0.f, OP == kOpReluBackward ? b[i] : 0.f);
    } else {
        for (; i < n; i += stride)
            dst[i] = f(OP == kOpAccumulate ? dst[i] : 0.f, OP != kOpFill ? a[i] : 0.f, OP == kOpReluBackward ? b[i] : 0.f);
    }
}

bool aligned16(const void* p) { return p == nullptr || (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <int OP>
int run_vec(float* dst, const float* a, const float* b, const float* scalar, float value, int64_t n, void* stream,
            const char* what) {
    if (n < 0) return fail(TFB_ERR_INVALID_ARG, "%s: negative length", what);
    if (n == 0) return TFB_OK;
    if (dst == nullptr || (OP != kOpFill && a == nullptr) || (OP == kOpReluBackward && b == nullptr) ||
        (OP == kOpScaleByScalar && scalar == nullptr))
        return fail(TFB_ERR_INVALID_ARG, "%s: null pointer", what);
    DeviceState* st = nullptr;
    int rc = device_state(&st);
    if (rc != TFB_OK) return rc;
    const int vec = aligned16(dst) && aligned16(a) && aligned16(b) ? 1 : 0;
    const long long work = vec ? (n + 3) / 4 : n;
    long long blocks = (work + 255) / 256;
    const long long cap = (long long)st->sm_count * 8;
    if (blocks > cap) blocks = cap;
    vec_kernel<OP><<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(dst, a, b, scalar, value, n, vec);
    TFB_CUDA_OK(cudaGetLastError());
    return TFB_OK;
}

}  // namespace
}  // namespace tfb

extern "C" {

int tfb_fill(float* dst, int64_t n, float value, void* stream) {
    return tfb::run_vec<tfb::kOpFill>(dst, nullptr, nullptr, nullptr, value, n, stream, "fill");
}
int tfb_relu_forward(const float* x, float* y, int64_t n, void* stream) {
    return tfb::run_vec<tfb::kOpRelu>(y, x, nullptr, nullptr, 0.f, n, stream, "relu_forward");
}
int tfb_relu_backward(const float* x, const float* dy, float* dx, int64_t n, void* stream) {
    return tfb::run_vec<tfb::kOpReluBackward>(dx, x, dy, nullptr, 0.f, n, stream, "relu_backward");
}
int tfb_accumulate(float* dst, const float* src, int64_t n, void* stream) {
    return tfb::run_vec<tfb::kOpAccumulate>(dst, src, nullptr, nullptr, 0.f, n, stream, "accumulate");
}
int tfb_scale_by_device_scalar(const float* src, const float* scalar, float* dst, int64_t n, void* stream) {
    return tfb::run_vec<tfb::kOpScaleByScalar>(dst, src, nullptr, scalar, 0.f, n, stream, "scale_by_device_scalar");
}

}  // extern "C"
