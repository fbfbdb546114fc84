// Stream-ordered device memory with one explicit pool per device.
//
// The reference allocates from each device's *default* pool on device 0's stream whatever device
// the tensor names, and never frees (cuda/memory/CudaStorageAllocator.cpp:34-57,101-150;
// tensor/Storage.hpp:27). Here every device gets its own cudaMemPool_t, allocations and frees
// run with that device current on a stream of that device, and peers can be granted access to a
// pool so that row-panel GEMMs can stage a replicated operand with plain peer copies.
#include <mutex>

#include "internal.hpp"

namespace tfb {
namespace {

struct Pool {
    cudaMemPool_t pool = nullptr;
    bool ready = false;
};
Pool g_pools[64];
std::mutex g_pool_mu;
constexpr uint64_t kDefaultReleaseThreshold = 64ull << 20;   // the reference's 64 MiB

// Restores the caller's current device on scope exit.
struct DeviceGuard {
    int prev = -1;
    bool switched = false;
    int enter(int device) {
        TFB_CUDA_OK(cudaGetDevice(&prev));
        if (prev != device) {
            TFB_CUDA_OK(cudaSetDevice(device));
            switched = true;
        }
        return TFB_OK;
    }
    ~DeviceGuard() {
        if (switched) (void)cudaSetDevice(prev);
    }
};

int pool_for(int device, cudaMemPool_t* out) {
    int count = 0;
    TFB_CUDA_OK(cudaGetDeviceCount(&count));
    if (device < 0 || device >= count || device >= 64)
        return fail(TFB_ERR_INVALID_ARG, "device %d does not exist (%d visible)", device, count);
    std::lock_guard<std::mutex> lock(g_pool_mu);
    Pool& p = g_pools[device];
    if (!p.ready) {
        cudaMemPoolProps props = {};
        props.allocType = cudaMemAllocationTypePinned;
        props.handleTypes = cudaMemHandleTypeNone;
        props.location.type = cudaMemLocationTypeDevice;
        props.location.id = device;
        TFB_CUDA_OK(cudaMemPoolCreate(&p.pool, &props));
        uint64_t thr = kDefaultReleaseThreshold;
        TFB_CUDA_OK(cudaMemPoolSetAttribute(p.pool, cudaMemPoolAttrReleaseThreshold, &thr));
        p.ready = true;
    }
    *out = p.pool;
    return TFB_OK;
}

}  // namespace
}  // namespace tfb

extern "C" {

using namespace tfb;

int tfb_device_count(int* count_out) {
    if (count_out == nullptr) return fail(TFB_ERR_INVALID_ARG, "device_count: null pointer");
    TFB_CUDA_OK(cudaGetDeviceCount(count_out));
    return TFB_OK;
}

int tfb_alloc(int device, size_t bytes, void* stream, void** ptr_out) {
    if (ptr_out == nullptr) return fail(TFB_ERR_INVALID_ARG, "alloc: null output pointer");
    *ptr_out = nullptr;
    cudaMemPool_t pool = nullptr;
    int rc = pool_for(device, &pool);
    if (rc != TFB_OK) return rc;
    DeviceGuard guard;
    rc = guard.enter(device);
    if (rc != TFB_OK) return rc;
    if (bytes == 0) bytes = 1;   // as the reference: an empty tensor still owns a distinct pointer
    void* p = nullptr;
    cudaError_t e = cudaMallocFromPoolAsync(&p, bytes, pool, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess || p == nullptr) {
        (void)cudaGetLastError();
        return fail(e == cudaErrorMemoryAllocation ? TFB_ERR_NO_MEMORY : TFB_ERR_CUDA,
                    "alloc of %zu bytes on device %d failed: %s", bytes, device, cudaGetErrorString(e));
    }
    *ptr_out = p;
    return TFB_OK;
}

int tfb_free(void* ptr, int device, void* stream) {
    if (ptr == nullptr) return TFB_OK;
    DeviceGuard guard;
    int rc = guard.enter(device);
    if (rc != TFB_OK) return rc;
    TFB_CUDA_OK(cudaFreeAsync(ptr, static_cast<cudaStream_t>(stream)));
    return TFB_OK;
}

int tfb_pool_set_release_threshold(int device, uint64_t bytes) {
    cudaMemPool_t pool = nullptr;
    int rc = pool_for(device, &pool);
    if (rc != TFB_OK) return rc;
    TFB_CUDA_OK(cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &bytes));
    return TFB_OK;
}

int tfb_pool_trim(int device, size_t keep_bytes) {
    cudaMemPool_t pool = nullptr;
    int rc = pool_for(device, &pool);
    if (rc != TFB_OK) return rc;
    TFB_CUDA_OK(cudaMemPoolTrimTo(pool, keep_bytes));
    return TFB_OK;
}

int tfb_pool_stats(int device, uint64_t* reserved, uint64_t* used, uint64_t* reserved_high, uint64_t* used_high) {
    cudaMemPool_t pool = nullptr;
    int rc = pool_for(device, &pool);
    if (rc != TFB_OK) return rc;
    uint64_t v = 0;
    if (reserved) { TFB_CUDA_OK(cudaMemPoolGetAttribute(pool, cudaMemPoolAttrReservedMemCurrent, &v)); *reserved = v; }
    if (used) { TFB_CUDA_OK(cudaMemPoolGetAttribute(pool, cudaMemPoolAttrUsedMemCurrent, &v)); *used = v; }
    if (reserved_high) { TFB_CUDA_OK(cudaMemPoolGetAttribute(pool, cudaMemPoolAttrReservedMemHigh, &v)); *reserved_high = v; }
    if (used_high) { TFB_CUDA_OK(cudaMemPoolGetAttribute(pool, cudaMemPoolAttrUsedMemHigh, &v)); *used_high = v; }
    return TFB_OK;
}

int tfb_pool_enable_peer(int device, int peer) {
    cudaMemPool_t pool = nullptr;
    int rc = pool_for(device, &pool);
    if (rc != TFB_OK) return rc;
    if (peer == device) return TFB_OK;
    int can = 0;
    TFB_CUDA_OK(cudaDeviceCanAccessPeer(&can, peer, device));
    if (!can) return fail(TFB_ERR_UNSUPPORTED, "device %d cannot access memory of device %d", peer, device);
    cudaMemAccessDesc desc = {};
    desc.location.type = cudaMemLocationTypeDevice;
    desc.location.id = peer;
    desc.flags = cudaMemAccessFlagsProtReadWrite;
    TFB_CUDA_OK(cudaMemPoolSetAccess(pool, &desc, 1));
    return TFB_OK;
}

int tfb_set_device(int device) {
    TFB_CUDA_OK(cudaSetDevice(device));
    return TFB_OK;
}

int tfb_get_device(int* device_out) {
    if (device_out == nullptr) return fail(TFB_ERR_INVALID_ARG, "get_device: null pointer");
    TFB_CUDA_OK(cudaGetDevice(device_out));
    return TFB_OK;
}

int tfb_stream_create(int device, void** stream_out) {
    if (stream_out == nullptr) return fail(TFB_ERR_INVALID_ARG, "stream_create: null pointer");
    DeviceGuard guard;
    int rc = guard.enter(device);
    if (rc != TFB_OK) return rc;
    cudaStream_t s = nullptr;
    TFB_CUDA_OK(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
    *stream_out = s;
    return TFB_OK;
}

int tfb_stream_destroy(void* stream) {
    if (stream == nullptr) return TFB_OK;
    // The library's scratch buffer of this stream goes with it (a later stream may get the same handle
    // value and must not inherit a stale entry). The stream belongs to the device that is current.
    workspace_release(static_cast<cudaStream_t>(stream));
    TFB_CUDA_OK(cudaStreamDestroy(static_cast<cudaStream_t>(stream)));
    return TFB_OK;
}

int tfb_stream_synchronize(void* stream) {
    TFB_CUDA_OK(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
    return TFB_OK;
}

int tfb_memcpy(void* dst, const void* src, size_t bytes, int kind, void* stream) {
    if (bytes == 0) return TFB_OK;
    if (dst == nullptr || src == nullptr) return fail(TFB_ERR_INVALID_ARG, "memcpy: null pointer");
    cudaMemcpyKind k;
    switch (kind) {
    case 0: k = cudaMemcpyHostToHost; break;
    case 1: k = cudaMemcpyHostToDevice; break;
    case 2: k = cudaMemcpyDeviceToHost; break;
    case 3: k = cudaMemcpyDeviceToDevice; break;
    default: return fail(TFB_ERR_INVALID_ARG, "memcpy: unknown kind %d", kind);
    }
    TFB_CUDA_OK(cudaMemcpyAsync(dst, src, bytes, k, static_cast<cudaStream_t>(stream)));
    return TFB_OK;
}

}  // extern "C"
