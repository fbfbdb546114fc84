// Library state: error strings, per-device status word, stream-ordered scratch buffers.
#include <cstdarg>
#include <cstdio>
#include <map>
#include <mutex>
#include <utility>

#include "internal.hpp"

namespace tfb {

namespace {
thread_local char g_err[512] = {0};
std::mutex g_mu;
DeviceState g_dev[64];
struct Scratch {
    void* ptr = nullptr;
    size_t bytes = 0;
    bool in_graph = false;   // handed to a stream capture: a CUDA graph may hold this address forever
};
std::map<std::pair<int, cudaStream_t>, Scratch> g_scratch;
}  // namespace

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

size_t dtype_size(int dtype) {
    switch (dtype) {
    case TFB_DTYPE_F32: return 4;
    case TFB_DTYPE_F16: return 2;
    case TFB_DTYPE_BF16: return 2;
    default: return 0;
    }
}

int device_state(DeviceState** out) {
    int dev = -1;
    TFB_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(TFB_ERR_UNSUPPORTED, "device index %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_mu);
    DeviceState& st = g_dev[dev];
    if (st.device < 0) {
        cudaDeviceProp prop;
        TFB_CUDA_OK(cudaGetDeviceProperties(&prop, dev));
        if (prop.major != 10)
            return fail(TFB_ERR_UNSUPPORTED,
                        "device %d is sm_%d%d; this library only carries sm_100a kernels", dev,
                        prop.major, prop.minor);
        int* status = nullptr;
        TFB_CUDA_OK(cudaMalloc(&status, sizeof(int)));
        TFB_CUDA_OK(cudaMemset(status, 0, sizeof(int)));
        st.sm_count = prop.multiProcessorCount;
        st.status = status;
        st.device = dev;
    }
    *out = &st;
    return TFB_OK;
}

int workspace_get(cudaStream_t stream, size_t bytes, void** out) {
    int dev = -1;
    TFB_CUDA_OK(cudaGetDevice(&dev));
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    TFB_CUDA_OK(cudaStreamIsCapturing(stream, &cap));
    std::lock_guard<std::mutex> lock(g_mu);
    if (cap != cudaStreamCaptureStatusNone) {
        // Inside a stream capture nothing may be allocated or freed on behalf of later replays. Hand
        // out the largest buffer an ordinary call has already created on this device and keep it
        // alive from now on. (Graph replays and ordinary calls that run at the same time on different
        // streams then share scratch: order them.)
        Scratch* best = nullptr;
        for (auto& kv : g_scratch)
            if (kv.first.first == dev && (best == nullptr || kv.second.bytes > best->bytes)) best = &kv.second;
        if (best == nullptr || best->bytes < bytes)
            return fail(TFB_ERR_UNSUPPORTED,
                        "this call needs %zu bytes of scratch but is being captured into a CUDA graph and only %zu "
                        "exist: run the same call once outside the capture first",
                        bytes, best ? best->bytes : (size_t)0);
        best->in_graph = true;
        *out = best->ptr;
        return TFB_OK;
    }
    Scratch& s = g_scratch[std::make_pair(dev, stream)];
    if (s.bytes < bytes) {
        // Stream-ordered: the old buffer is released after the work already queued on this stream, the
        // new one is usable by work queued after this point. A buffer a graph may reference is kept.
        if (s.ptr != nullptr && !s.in_graph) TFB_CUDA_OK(cudaFreeAsync(s.ptr, stream));
        s.ptr = nullptr;
        s.bytes = 0;
        s.in_graph = false;
        size_t want = bytes + (bytes >> 2);   // head-room so alternating sizes do not thrash
        want = (want + 0xfffff) & ~(size_t)0xfffff;
        void* p = nullptr;
        cudaError_t e = cudaMallocAsync(&p, want, stream);
        if (e != cudaSuccess) {
            (void)cudaGetLastError();
            return fail(TFB_ERR_NO_MEMORY, "scratch allocation of %zu bytes failed: %s", want,
                        cudaGetErrorString(e));
        }
        s.ptr = p;
        s.bytes = want;
    }
    *out = s.ptr;
    return TFB_OK;
}

}  // namespace tfb

extern "C" {

int tfb_init(void) {
    tfb::DeviceState* st = nullptr;
    return tfb::device_state(&st);
}

const char* tfb_last_error_string(void) { return tfb::g_err; }

int tfb_device_status(int* code_out) {
    tfb::DeviceState* st = nullptr;
    int rc = tfb::device_state(&st);
    if (rc != TFB_OK) return rc;
    TFB_CUDA_OK(cudaDeviceSynchronize());
    int code = 0;
    TFB_CUDA_OK(cudaMemcpy(&code, st->status, sizeof(int), cudaMemcpyDeviceToHost));
    if (code != 0) TFB_CUDA_OK(cudaMemset(st->status, 0, sizeof(int)));
    if (code_out != nullptr) *code_out = code;
    if (code != 0) return tfb::fail(TFB_ERR_DEVICE, "a kernel recorded device error %d", code);
    return TFB_OK;
}

}  // extern "C"
