// Library state: error strings, per-device status word, stream-ordered scratch buffers.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
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

namespace {
// Tuning knobs: defaults, overridden once from the environment (TFB_GEMM_BN, ...) the first time any
// knob is read, and afterwards only through tfb_set_tuning. Nothing on a call path reads the environment.
struct Knob {
    const char* env;
    int def;
};
constexpr Knob kKnobs[TFB_TUNE_COUNT] = {
    {"TFB_GEMM_BN", 0}, {"TFB_GEMM_PAIR", -1}, {"TFB_GEMM_SPLITK", 0}, {"TFB_GEMM_CHUNK_KB", 0},
    {"TFB_CONV_TMA", 1}, {"TFB_CONV_DIRECT", 1}, {"TFB_CONV_PAIR", -1}, {"TFB_HOST_PANEL", 512},
    {"TFB_PDL", 1}, {"TFB_FUSE_PLANES", 1}, {"TFB_GEMM_GROUP_M", 0}, {"TFB_SMALL_GEMM", 1},
    {"TFB_RAW_HI", 0}, {"TFB_CLUSTER_K", 1},
};
std::atomic<int> g_knob[TFB_TUNE_COUNT];
std::once_flag g_knob_once;
void knobs_init() {
    std::call_once(g_knob_once, [] {
        for (int i = 0; i < TFB_TUNE_COUNT; ++i) {
            int v = kKnobs[i].def;
            if (const char* e = getenv(kKnobs[i].env)) v = atoi(e);
            g_knob[i].store(v, std::memory_order_relaxed);
        }
    });
}
}  // namespace

int tuning(int knob) {
    knobs_init();
    return g_knob[knob].load(std::memory_order_relaxed);
}

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

void workspace_release(cudaStream_t stream) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess) return;
    std::lock_guard<std::mutex> lock(g_mu);
    auto it = g_scratch.find(std::make_pair(dev, stream));
    if (it == g_scratch.end()) return;
    // A buffer a captured graph may still name is left alone (and stays allocated).
    if (it->second.ptr != nullptr && !it->second.in_graph) (void)cudaFreeAsync(it->second.ptr, stream);
    if (!it->second.in_graph) g_scratch.erase(it);
    (void)cudaGetLastError();
}

}  // namespace tfb

extern "C" {

int tfb_init(void) {
    tfb::DeviceState* st = nullptr;
    return tfb::device_state(&st);
}

const char* tfb_last_error_string(void) { return tfb::g_err; }

int tfb_scratch_stats(int device, uint64_t* buffers_out, uint64_t* bytes_out) {
    uint64_t n = 0, bytes = 0;
    {
        std::lock_guard<std::mutex> lock(tfb::g_mu);
        for (const auto& kv : tfb::g_scratch)
            if (kv.first.first == device && kv.second.ptr != nullptr) {
                ++n;
                bytes += kv.second.bytes;
            }
    }
    if (buffers_out != nullptr) *buffers_out = n;
    if (bytes_out != nullptr) *bytes_out = bytes;
    return TFB_OK;
}

int tfb_set_tuning(int knob, int value) {
    if (knob < 0 || knob >= TFB_TUNE_COUNT) return tfb::fail(TFB_ERR_INVALID_ARG, "set_tuning: unknown knob %d", knob);
    tfb::knobs_init();
    tfb::g_knob[knob].store(value, std::memory_order_relaxed);
    return TFB_OK;
}

int tfb_get_tuning(int knob, int* value_out) {
    if (knob < 0 || knob >= TFB_TUNE_COUNT || value_out == nullptr)
        return tfb::fail(TFB_ERR_INVALID_ARG, "get_tuning: unknown knob %d or null output", knob);
    *value_out = tfb::tuning(knob);
    return TFB_OK;
}

int tfb_inject_device_status(int word, int code) {
    tfb::DeviceState* st = nullptr;
    int rc = tfb::device_state(&st);
    if (rc != TFB_OK) return rc;
    if (word == 0) {
        TFB_CUDA_OK(cudaMemcpy(st->status, &code, sizeof(int), cudaMemcpyHostToDevice));
        return TFB_OK;
    }
    if (word == 1) return tfb::static_status_put(code);
    return tfb::fail(TFB_ERR_INVALID_ARG, "inject_device_status: word %d (0 = regular, 1 = allocation-free entry point)", word);
}

int tfb_device_status(int* code_out) {
    tfb::DeviceState* st = nullptr;
    int rc = tfb::device_state(&st);
    if (rc != TFB_OK) return rc;
    TFB_CUDA_OK(cudaDeviceSynchronize());
    int code = 0;
    TFB_CUDA_OK(cudaMemcpy(&code, st->status, sizeof(int), cudaMemcpyDeviceToHost));
    if (code != 0) TFB_CUDA_OK(cudaMemset(st->status, 0, sizeof(int)));
    // Kernels launched through tfb_matmul_f32_static record into a word of their own; the first
    // non-zero code of the two is reported and both are cleared.
    int static_code = 0;
    rc = tfb::static_status_take(&static_code);
    if (rc != TFB_OK) return rc;
    if (code == 0) code = static_code;
    if (code_out != nullptr) *code_out = code;
    if (code != 0) return tfb::fail(TFB_ERR_DEVICE, "a kernel recorded device error %d", code);
    return TFB_OK;
}

}  // extern "C"
