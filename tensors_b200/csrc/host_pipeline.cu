// Matmul on HOST buffers: the copies to and from the device are part of the call and overlap with
// the product. B is uploaded (and, for FP32, split into TF32 planes) once; A then streams through in
// row panels on a copy stream while the previous panel multiplies on the caller's stream and the
// panel before that drains back to the host on a third stream. With pinned host memory the three
// engines (H2D copy, SMs, D2H copy) run concurrently; with pageable memory the copies serialise but
// the result is the same.
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

#include "internal.hpp"

namespace tfb {
namespace {

struct CopyStreams {
    cudaStream_t h2d = nullptr, d2h = nullptr;
};
CopyStreams g_copy[64];
std::mutex g_copy_mu;

int copy_streams(CopyStreams** out) {
    int dev = -1;
    TFB_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(TFB_ERR_UNSUPPORTED, "device index %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_copy_mu);
    CopyStreams& c = g_copy[dev];
    if (c.h2d == nullptr) {
        TFB_CUDA_OK(cudaStreamCreateWithFlags(&c.h2d, cudaStreamNonBlocking));
        TFB_CUDA_OK(cudaStreamCreateWithFlags(&c.d2h, cudaStreamNonBlocking));
    }
    *out = &c;
    return TFB_OK;
}

// Stream-ordered device buffers of one call: whatever was allocated is released on `stream` when the
// call returns, on the error paths too.
struct BufferBag {
    cudaStream_t stream;
    std::vector<void*> ptrs;
    explicit BufferBag(cudaStream_t s) : stream(s) {}
    int make(void** out, size_t bytes) {
        TFB_CUDA_OK(cudaMallocAsync(out, bytes, stream));
        ptrs.push_back(*out);
        return TFB_OK;
    }
    // Streams other than `stream` that may still touch the buffers (the copy streams): the frees are
    // ordered after everything enqueued on them so far.
    std::vector<cudaStream_t> users;
    ~BufferBag() {
        for (cudaStream_t u : users) {
            cudaEvent_t e = nullptr;
            if (cudaEventCreateWithFlags(&e, cudaEventDisableTiming) != cudaSuccess) continue;
            if (cudaEventRecord(e, u) == cudaSuccess) (void)cudaStreamWaitEvent(stream, e, 0);
            (void)cudaEventDestroy(e);
        }
        for (void* p : ptrs) (void)cudaFreeAsync(p, stream);
        (void)cudaGetLastError();
    }
};

struct EventBag {
    std::vector<cudaEvent_t> events;
    int make(cudaEvent_t* e) {
        TFB_CUDA_OK(cudaEventCreateWithFlags(e, cudaEventDisableTiming));
        events.push_back(*e);
        return TFB_OK;
    }
    ~EventBag() {
        for (cudaEvent_t e : events) (void)cudaEventDestroy(e);   // released once their work has completed
    }
};

}  // namespace
}  // namespace tfb

namespace tfb {
static int matmul_host_impl(const void* A_host, const void* B_host, bool b_on_device, void* C_host, int64_t M,
                            int64_t N, int64_t K, int dtype, void* stream_v);
}

extern "C" int tfb_matmul_host(const void* A_host, const void* B_host, void* C_host, int64_t M, int64_t N,
                               int64_t K, int dtype, void* stream_v) {
    return tfb::matmul_host_impl(A_host, B_host, false, C_host, M, N, K, dtype, stream_v);
}

extern "C" int tfb_matmul_host_b_resident(const void* A_host, const void* B_device, void* C_host, int64_t M,
                                          int64_t N, int64_t K, int dtype, void* stream_v) {
    return tfb::matmul_host_impl(A_host, B_device, true, C_host, M, N, K, dtype, stream_v);
}

static int tfb::matmul_host_impl(const void* A_host, const void* B_host, bool b_on_device, void* C_host, int64_t M,
                                 int64_t N, int64_t K, int dtype, void* stream_v) {
    using namespace tfb;
    if (M < 0 || N < 0 || K < 0) return fail(TFB_ERR_INVALID_ARG, "matmul_host: negative extent");
    const size_t es = dtype_size(dtype);
    if (es == 0) return fail(TFB_ERR_UNSUPPORTED, "matmul_host: unknown dtype %d", dtype);
    if (M == 0 || N == 0) return TFB_OK;
    if (A_host == nullptr || B_host == nullptr || C_host == nullptr)
        return fail(TFB_ERR_INVALID_ARG, "matmul_host: null pointer");
    if (K == 0) {
        memset(C_host, 0, (size_t)(M * N) * 4);
        return TFB_OK;
    }
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    DeviceState* st = nullptr;
    int rc = device_state(&st);
    if (rc != TFB_OK) return rc;
    CopyStreams* cs = nullptr;
    rc = copy_streams(&cs);
    if (rc != TFB_OK) return rc;
    const bool f32 = dtype == TFB_DTYPE_F32;

    // Panel height: two rows of 256-row tiles (64 pair tiles at N = 8192: most of the SM pairs), small
    // enough that the copy engines interleave finely and the last panel's product and download are a short
    // tail (measured at 8192^3: 13.3 ms per call with 512 rows, 15.7 ms with 1024, 21.1 ms with 2048).
    int64_t panel = tuning(TFB_TUNE_HOST_PANEL_ROWS) > 0 ? tuning(TFB_TUNE_HOST_PANEL_ROWS) : 512;
    if (panel > M) panel = M;
    const int64_t panels = (M + panel - 1) / panel;
    const int64_t ldb4 = (N + 3) / 4 * 4;

    // Device buffers, stream-ordered on the caller's stream.
    uint8_t* dB = nullptr;
    float* dBs = nullptr;   // FP32: hi / lo planes of B
    uint8_t* dA[2] = {nullptr, nullptr};
    float* dC[2] = {nullptr, nullptr};
    // Declared before the events: the buffers are released (stream-ordered, after the waits below
    // have been enqueued) when the call returns, whichever way it returns.
    BufferBag buffers(stream);
    buffers.users = {cs->h2d, cs->d2h};
    if (b_on_device) dB = static_cast<uint8_t*>(const_cast<void*>(B_host));   // already where it is needed
    else if ((rc = buffers.make(reinterpret_cast<void**>(&dB), (size_t)(K * N) * es)) != TFB_OK) return rc;
    if (f32 && (rc = buffers.make(reinterpret_cast<void**>(&dBs), (size_t)(2 * K * ldb4) * 4)) != TFB_OK) return rc;
    for (int i = 0; i < 2; ++i) {
        if ((rc = buffers.make(reinterpret_cast<void**>(&dA[i]), (size_t)(panel * K) * es)) != TFB_OK) return rc;
        if ((rc = buffers.make(reinterpret_cast<void**>(&dC[i]), (size_t)(panel * N) * 4)) != TFB_OK) return rc;
    }
    EventBag bag;
    cudaEvent_t ready, b_loaded;
    if ((rc = bag.make(&ready)) != TFB_OK || (rc = bag.make(&b_loaded)) != TFB_OK) return rc;
    // The copy streams may not touch the buffers before the allocations are ordered.
    TFB_CUDA_OK(cudaEventRecord(ready, stream));
    TFB_CUDA_OK(cudaStreamWaitEvent(cs->h2d, ready, 0));
    TFB_CUDA_OK(cudaStreamWaitEvent(cs->d2h, ready, 0));

    if (!b_on_device) {
        TFB_CUDA_OK(cudaMemcpyAsync(dB, B_host, (size_t)(K * N) * es, cudaMemcpyHostToDevice, cs->h2d));
        TFB_CUDA_OK(cudaEventRecord(b_loaded, cs->h2d));
        TFB_CUDA_OK(cudaStreamWaitEvent(stream, b_loaded, 0));
    }
    if (f32) {
        rc = split_operand(reinterpret_cast<const float*>(dB), K, N, N, nullptr, dBs, dBs + K * ldb4, ldb4, stream);
        if (rc != TFB_OK) return rc;
    }

    std::vector<cudaEvent_t> computed((size_t)panels), drained((size_t)panels);
    for (int64_t p = 0; p < panels; ++p) {
        const int slot = (int)(p & 1);
        const int64_t r0 = p * panel, rows = (M - r0 < panel) ? (M - r0) : panel;
        cudaEvent_t a_loaded;
        if ((rc = bag.make(&a_loaded)) != TFB_OK || (rc = bag.make(&computed[(size_t)p])) != TFB_OK ||
            (rc = bag.make(&drained[(size_t)p])) != TFB_OK)
            return rc;
        // The A buffer of this slot is free once the product of panel p-2 is done.
        if (p >= 2) TFB_CUDA_OK(cudaStreamWaitEvent(cs->h2d, computed[(size_t)(p - 2)], 0));
        TFB_CUDA_OK(cudaMemcpyAsync(dA[slot], static_cast<const uint8_t*>(A_host) + (size_t)(r0 * K) * es,
                                    (size_t)(rows * K) * es, cudaMemcpyHostToDevice, cs->h2d));
        TFB_CUDA_OK(cudaEventRecord(a_loaded, cs->h2d));
        TFB_CUDA_OK(cudaStreamWaitEvent(stream, a_loaded, 0));
        // The C buffer of this slot is free once panel p-2 has been copied out.
        if (p >= 2) TFB_CUDA_OK(cudaStreamWaitEvent(stream, drained[(size_t)(p - 2)], 0));
        GemmCall c;
        c.A = dA[slot]; c.C = dC[slot];
        c.M = rows; c.N = N; c.K = K;
        c.lda = K; c.ldc = N;
        c.a_kmajor = true; c.b_kmajor = false;
        c.in_dtype = dtype; c.out_dtype = TFB_DTYPE_F32;
        if (f32) {
            c.B = dBs; c.ldb = ldb4; c.b_presplit = true; c.b_lo_off = K * ldb4;
        } else {
            c.B = dB; c.ldb = N;
        }
        rc = gemm_run_on(c, stream, st);
        if (rc != TFB_OK) return rc;
        TFB_CUDA_OK(cudaEventRecord(computed[(size_t)p], stream));
        TFB_CUDA_OK(cudaStreamWaitEvent(cs->d2h, computed[(size_t)p], 0));
        TFB_CUDA_OK(cudaMemcpyAsync(static_cast<float*>(C_host) + r0 * N, dC[slot], (size_t)(rows * N) * 4,
                                    cudaMemcpyDeviceToHost, cs->d2h));
        TFB_CUDA_OK(cudaEventRecord(drained[(size_t)p], cs->d2h));
    }
    // The caller's stream completes when the last panels have reached the host.
    TFB_CUDA_OK(cudaStreamWaitEvent(stream, drained[(size_t)(panels - 1)], 0));
    if (panels >= 2) TFB_CUDA_OK(cudaStreamWaitEvent(stream, drained[(size_t)(panels - 2)], 0));
    return TFB_OK;   // `buffers` frees after the waits just enqueued on `stream`
}
