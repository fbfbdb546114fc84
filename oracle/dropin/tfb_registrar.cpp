// TEST INFRASTRUCTURE (and the file a maintainer of the reference would add): registers libtfb's
// entry points in the reference's kernel registry at load time, in the pattern of the reference's own
// registrar (cuda/kernels/elementwise.cu:306-336). Compiled against the patched copy of the reference
// that apply_dropin.py makes; only the C-ABI of include/tfb.h is used.
#include <stdexcept>

#include "cuda/CudaContext.hpp"
#include "cuda/CudaKernelRegistry.hpp"
#include "tfb.h"

namespace tensorforge {
namespace {

void matmul_trampoline(const void* a, const void* b, void* c, int64_t M, int64_t N, int64_t K, Dtype in, Dtype out,
                       void* stream) {
    if (tfb_matmul(a, b, c, M, N, K, static_cast<int>(in), static_cast<int>(out), stream) != TFB_OK)
        throw std::runtime_error(tfb_last_error_string());
}

void matmul_backward_trampoline(const void* dC, const void* a, const void* b, void* dA, void* dB, int64_t M, int64_t N,
                                int64_t K, Dtype dtype, void* stream) {
    if (tfb_matmul_backward(dC, a, b, dA, dB, M, N, K, static_cast<int>(dtype), stream) != TFB_OK)
        throw std::runtime_error(tfb_last_error_string());
}

void fill_trampoline(void* dst, int64_t n, float value, void* stream) {
    if (tfb_fill(static_cast<float*>(dst), n, value, stream) != TFB_OK) throw std::runtime_error(tfb_last_error_string());
}

__attribute__((constructor)) void register_tfb_kernels() {
    register_cuda_matmul(&matmul_trampoline);
    register_cuda_matmul_backward(&matmul_backward_trampoline);
    register_cuda_fill(&fill_trampoline);
    // the reference keeps one process-wide stream pointer for its CUDA branches (tensor/Tensor.cpp:77)
    register_current_stream(DeviceContext::current().current_stream);
}

}  // namespace
}  // namespace tensorforge
