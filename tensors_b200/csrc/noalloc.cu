// FP32 matmul for callers that must not allocate device memory.
//
// Some hosts call into this library from places where cudaMalloc is off the table: inside a
// real-time or latency-critical loop that may not take the allocator's locks or its implicit
// device synchronisation, from a runtime whose memory is entirely owned by its own arena (every
// byte accounted for up front), or late at teardown when the context can no longer grow. The
// regular FP32 product needs scratch for the TF32 hi / lo planes of both operands and takes it
// from a stream-ordered pool. This variant keeps that scratch in a fixed array inside the
// library image instead, so the call itself never allocates or frees anything.
//
// The price is a size limit and sharing: every call on a device uses the same array.
#include <mutex>

#include "internal.hpp"

namespace tfb {
namespace {

// 16 MiB per device that loads the library, held until the process exits.
constexpr size_t kStaticScratchBytes = 16u << 20;

static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];
// Error word for kernels launched through this entry point (the regular one is cudaMalloc'ed).
static __device__ int g_static_status;

struct StaticState {
    bool ready = false;
    DeviceState dev;
    void* scratch = nullptr;
};
StaticState g_static[64];
std::mutex g_static_mu;

// In host code `g_static_scratch` is only a handle for the runtime; the address kernels can use
// has to be asked for, once per device, with that device current.
int static_state(StaticState** out) {
    int dev = -1;
    TFB_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(TFB_ERR_UNSUPPORTED, "device index %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_static_mu);
    StaticState& s = g_static[dev];
    if (!s.ready) {
        int major = 0, sms = 0;
        TFB_CUDA_OK(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
        TFB_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        if (major != 10)
            return fail(TFB_ERR_UNSUPPORTED, "device %d is not sm_100; this library only carries sm_100a kernels", dev);
        void* scratch = nullptr;
        void* status = nullptr;
        TFB_CUDA_OK(cudaGetSymbolAddress(&scratch, g_static_scratch));
        TFB_CUDA_OK(cudaGetSymbolAddress(&status, g_static_status));
        s.dev.device = dev;
        s.dev.sm_count = sms;
        s.dev.status = static_cast<int*>(status);
        s.scratch = scratch;
        s.ready = true;
    }
    *out = &s;
    return TFB_OK;
}

}  // namespace

// The error word of the kernels launched through tfb_matmul_f32_static on the current device: read,
// and cleared if set. Nothing to do (code 0) when that entry point was never used on this device.
// Copies through the address cudaGetSymbolAddress gave; allocates nothing.
int static_status_take(int* code) {
    *code = 0;
    int dev = -1;
    TFB_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return TFB_OK;
    int* word = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_static_mu);
        if (!g_static[dev].ready) return TFB_OK;
        word = g_static[dev].dev.status;
    }
    TFB_CUDA_OK(cudaMemcpy(code, word, sizeof(int), cudaMemcpyDeviceToHost));
    if (*code != 0) TFB_CUDA_OK(cudaMemset(word, 0, sizeof(int)));
    return TFB_OK;
}

int static_status_put(int code) {
    int dev = -1;
    TFB_CUDA_OK(cudaGetDevice(&dev));
    int* word = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_static_mu);
        if (dev < 0 || dev >= 64 || !g_static[dev].ready)
            return fail(TFB_ERR_INVALID_ARG, "tfb_matmul_f32_static has not run on device %d yet", dev);
        word = g_static[dev].dev.status;
    }
    TFB_CUDA_OK(cudaMemcpy(word, &code, sizeof(int), cudaMemcpyHostToDevice));
    return TFB_OK;
}

}  // namespace tfb

extern "C" {

size_t tfb_matmul_f32_static_limit(void) { return tfb::kStaticScratchBytes; }

int tfb_matmul_f32_static(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K,
                          void* stream) {
    using namespace tfb;
    if (M < 0 || N < 0 || K < 0) return fail(TFB_ERR_INVALID_ARG, "matmul_f32_static: negative extent");
    if (A == nullptr || B == nullptr || C == nullptr)
        return fail(TFB_ERR_INVALID_ARG, "matmul_f32_static: null operand pointer");
    GemmCall c;
    c.A = A; c.B = B; c.C = C;
    c.M = M; c.N = N; c.K = K;
    c.lda = K; c.ldb = N; c.ldc = N;
    c.a_kmajor = true; c.b_kmajor = false;
    c.in_dtype = TFB_DTYPE_F32; c.out_dtype = TFB_DTYPE_F32;
    StaticState* s = nullptr;
    int rc = static_state(&s);
    if (rc != TFB_OK) return rc;
    const size_t need = gemm_workspace_bytes(c, s->dev.sm_count);
    if (need > kStaticScratchBytes)
        return fail(TFB_ERR_TOO_LARGE,
                    "matmul_f32_static: the split operands need %zu bytes of scratch, the built-in array holds %zu "
                    "(roughly M*K + K*N <= 2 Mi elements); use tfb_matmul for larger products",
                    need, kStaticScratchBytes);
    // Nothing in the array has to start at zero: the split pass rewrites every byte it later reads,
    // padding columns included.
    c.workspace = s->scratch;
    c.workspace_bytes = kStaticScratchBytes;
    return gemm_run_on(c, static_cast<cudaStream_t>(stream), &s->dev);
}

}  // extern "C"
