// The small HBM-bound kernels that keep an MLP training step on the device between its GEMMs:
// log_softmax + mean negative log-likelihood (loss and gradient with respect to the logits) and
// SGD with momentum. Both are one pass over their data; neither is a contraction.
#include "finish.cuh"
#include "internal.hpp"
#include "ptx.cuh"

namespace tfb {

namespace {

// One warp per row. lsm = x - (max + log(sum exp(x - max))) as Tensor::log_softmax computes it;
// the gradient is g - exp(lsm) * sum(g) with g = onehot * (-1 / global_rows), the result of the
// reference's loss graph followed by LogSoftmaxBackward.
__global__ void log_softmax_nll_kernel(const float* __restrict__ logits, const long long* __restrict__ labels,
                                       float* __restrict__ dlogits, float* __restrict__ row_loss,
                                       long long rows, int cols, float n_inv) {
    pdl_wait();
    pdl_launch_dependents();
    const long long row = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (row >= rows) return;
    const float* x = logits + row * cols;
    float m = -INFINITY;
    for (int j = lane; j < cols; j += 32) m = fmaxf(m, x[j]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    float s = 0.f;
    for (int j = lane; j < cols; j += 32) s += expf(x[j] - m);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    const float log_z = logf(s) + m;
    const long long t = labels[row];
    const bool valid = t >= 0 && t < cols;
    const float scale = -1.0f * n_inv;
    const float gsum = valid ? scale : 0.f;
    for (int j = lane; j < cols; j += 32) {
        const float lsm = x[j] - log_z;
        const float g = (valid && j == t) ? scale : 0.f;
        if (dlogits != nullptr) dlogits[row * cols + j] = g - expf(lsm) * gsum;
    }
    if (lane == 0 && row_loss != nullptr) row_loss[row] = valid ? (x[t] - log_z) : 0.f;
}

// loss = (-1 * sum_r row_loss[r]) * n_inv, summed in a fixed order (strided per thread, then a
// shared-memory tree), so the value does not change from run to run.
__global__ void loss_finish_kernel(const float* __restrict__ row_loss, long long rows, float n_inv,
                                   float* __restrict__ loss_out) {
    __shared__ float sm[1024];
    pdl_wait();
    pdl_launch_dependents();
    loss_finish_block(row_loss, rows, n_inv, loss_out, (int)threadIdx.x, sm);   // launched with 1024 threads
}

// v <- mu * v + g; p <- p - lr * v   (separate multiply and add, like the host formula).
__global__ void sgd_momentum_kernel(float* __restrict__ p, float* __restrict__ v, const float* __restrict__ g,
                                    long long n, float lr, float mu, float grad_scale) {
    pdl_wait();
    pdl_launch_dependents();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (long long)gridDim.x * blockDim.x) {
        const float gi = g[i] * grad_scale;
        const float vi = __fadd_rn(__fmul_rn(mu, v[i]), gi);
        v[i] = vi;
        p[i] = __fsub_rn(p[i], __fmul_rn(lr, vi));
    }
}

}  // namespace

int log_softmax_nll_rows(const float* logits, const int64_t* labels, float* dlogits, float* row_loss, int64_t rows,
                         int64_t cols, int64_t global_rows, cudaStream_t stream) {
    if (rows <= 0) return TFB_OK;
    const float n_inv = (float)(1.0 / (double)global_rows);
    const int block = 256;
    const long long grid = (rows * 32 + block - 1) / block;
    return launch_pdl(log_softmax_nll_kernel, dim3((unsigned)grid), dim3(block), 0, stream, logits,
                      reinterpret_cast<const long long*>(labels), dlogits, row_loss, (long long)rows, (int)cols, n_inv);
}

}  // namespace tfb

extern "C" {

int tfb_log_softmax_nll(const float* logits, const int64_t* labels, float* dlogits, float* loss_out,
                        int64_t rows, int64_t cols, int64_t global_rows, void* stream_v) {
    using namespace tfb;
    if (rows < 0 || cols <= 0 || global_rows <= 0) return fail(TFB_ERR_INVALID_ARG, "log_softmax_nll: bad extent");
    if (logits == nullptr || labels == nullptr) return fail(TFB_ERR_INVALID_ARG, "log_softmax_nll: null pointer");
    if (cols > INT32_MAX) return fail(TFB_ERR_TOO_LARGE, "log_softmax_nll: too many classes");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    DeviceState* st = nullptr;
    int rc = device_state(&st);
    if (rc != TFB_OK) return rc;
    if (rows == 0) {
        if (loss_out != nullptr) TFB_CUDA_OK(cudaMemsetAsync(loss_out, 0, sizeof(float), stream));
        return TFB_OK;
    }
    float* row_loss = nullptr;
    if (loss_out != nullptr) {
        void* ws = nullptr;
        rc = workspace_get(stream, (size_t)rows * sizeof(float), &ws);
        if (rc != TFB_OK) return rc;
        row_loss = static_cast<float*>(ws);
    }
    const float n_inv = (float)(1.0 / (double)global_rows);
    const int block = 256;
    const long long grid = (rows * 32 + block - 1) / block;
    rc = launch_pdl(log_softmax_nll_kernel, dim3((unsigned)grid), dim3(block), 0, stream, logits,
                    reinterpret_cast<const long long*>(labels), dlogits, row_loss, (long long)rows, (int)cols, n_inv);
    if (rc != TFB_OK) return rc;
    if (loss_out != nullptr)
        rc = launch_pdl(loss_finish_kernel, dim3(1), dim3(1024), 0, stream, (const float*)row_loss, (long long)rows, n_inv,
                        loss_out);
    return rc;
}

int tfb_sgd_momentum(float* params, float* velocity, const float* grads, int64_t n, float lr,
                     float momentum, float grad_scale, void* stream_v) {
    using namespace tfb;
    if (n < 0) return fail(TFB_ERR_INVALID_ARG, "sgd_momentum: negative length");
    if (n == 0) return TFB_OK;
    if (params == nullptr || velocity == nullptr || grads == nullptr)
        return fail(TFB_ERR_INVALID_ARG, "sgd_momentum: null pointer");
    DeviceState* st = nullptr;
    int rc = device_state(&st);
    if (rc != TFB_OK) return rc;
    long long grid = (n + 255) / 256;
    const long long cap = (long long)st->sm_count * 8;
    if (grid > cap) grid = cap;
    return launch_pdl(sgd_momentum_kernel, dim3((unsigned)grid), dim3(256), 0, static_cast<cudaStream_t>(stream_v), params,
                      velocity, grads, (long long)n, lr, momentum, grad_scale);
}

}  // extern "C"
