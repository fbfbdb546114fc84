// A group of GPUs that sum small FP32 buffers through peer memory (tfb_peer_group): the exchange step
// of batch-sharded layers whose gradient is small — a convolution's weight and bias gradient — where a
// library collective is pure latency.
//
// Each rank owns one cudaMalloc'ed region [ in : capacity floats ][ out : capacity floats ][ flags ].
// A rank writes its contribution into `in`; tfb_peer_allreduce_sum then runs one kernel per rank:
//   flag barrier (every rank's contribution is complete)
//   rank r adds slice r of all ranks' `in` buffers in rank order (ordinary peer loads; a fixed order,
//     so every run and every rank gives the same bits) and stores the sums into slice r of every
//     rank's `out` buffer (ordinary peer stores)
//   flag barrier (all slices have landed in my `out`; all peers have finished reading my `in`)
// The flag protocol, its bounded waits and its device-resident step counter are those of the MLP
// exchange (peer_sync.cuh). No cluster-multicast or multimem access is used.
#include <cstring>
#include <new>

#include "internal.hpp"
#include "peer_sync.cuh"

namespace tfb {
namespace {

constexpr int kReduceThreads = 256;

struct ReduceRank {
    uint8_t* region[kMaxWorld];
    int* status;
    int rank;
};
struct ReduceParams {
    ReduceRank ranks[kMaxWorld];   // one entry per rank this launch runs (blockIdx.y selects it)
    int world;
    long long n_vec;               // float4 vectors to sum
    long long out_off, flags_off;  // byte offsets inside a region (`in` is at offset 0)
    unsigned long long wait_ns;
};

__global__ void __launch_bounds__(kReduceThreads) peer_allreduce_kernel(const __grid_constant__ ReduceParams p) {
    pdl_wait();
    pdl_launch_dependents();
    const ReduceRank& me = p.ranks[blockIdx.y];
    const int world = p.world, rank = me.rank, cta = blockIdx.x, t = threadIdx.x;
    uint8_t* mine = me.region[rank];
    uint32_t* epoch_word = reinterpret_cast<uint32_t*>(mine + p.flags_off) + cta;
    const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(epoch_word) + 1u;
    int ok = 1;
    if (world > 1 && t < world) {
        st_relaxed_sys(flag_word(me.region[t], p.flags_off, 0, cta, rank), epoch);   // publishes nothing of this kernel
        if (!wait_flag(flag_word(mine, p.flags_off, 0, cta, t), epoch, p.wait_ns)) {
            ok = 0;
            if (me.status != nullptr) atomicCAS(me.status, 0, kDevTimeoutExchange);
        }
    }
    ok = __syncthreads_and(ok);
    if (ok) {
        const long long v0 = p.n_vec * rank / world, v1 = p.n_vec * (rank + 1) / world;
        for (long long i = v0 + (long long)cta * blockDim.x + t; i < v1; i += (long long)gridDim.x * blockDim.x) {
            float4 s = ld_peer(reinterpret_cast<const float4*>(me.region[0]) + i);
            for (int r = 1; r < world; ++r) {
                const float4 g = ld_peer(reinterpret_cast<const float4*>(me.region[r]) + i);
                s.x = __fadd_rn(s.x, g.x); s.y = __fadd_rn(s.y, g.y);
                s.z = __fadd_rn(s.z, g.z); s.w = __fadd_rn(s.w, g.w);
            }
            for (int r = 0; r < world; ++r) st_peer(reinterpret_cast<float4*>(me.region[r] + p.out_off) + i, s);
        }
    }
    if (world == 1) return;
    __syncthreads();
    if (t < world) {
        __threadfence_system();   // cumulative over the CTA's stores through the barrier above
        st_relaxed_sys(flag_word(me.region[t], p.flags_off, 1, cta, rank), epoch);
        if (ok && !wait_flag(flag_word(mine, p.flags_off, 1, cta, t), epoch, p.wait_ns)) {
            if (me.status != nullptr) atomicCAS(me.status, 0, kDevTimeoutExchange);
        }
    }
    __syncthreads();
    if (t == 0) *reinterpret_cast<volatile uint32_t*>(epoch_word) = epoch;
}

inline size_t align256(size_t x) { return (x + 255) & ~(size_t)255; }

}  // namespace
}  // namespace tfb

struct tfb_peer_group {
    int device = -1;
    int64_t capacity = 0;   // floats, a multiple of 4
    uint8_t* region = nullptr;
    size_t region_bytes = 0, out_off = 0, flags_off = 0;
    int rank = 0, world = 1;
    uint8_t* peer_region[tfb::kMaxWorld] = {nullptr};
    bool ipc_mapped[tfb::kMaxWorld] = {false};
    unsigned long long wait_ns = 2000000000ull;
};

namespace tfb {
namespace {

int check_group(const tfb_peer_group* g, const char* who) {
    if (g == nullptr) return fail(TFB_ERR_INVALID_ARG, "%s: null group", who);
    int dev = -1;
    TFB_CUDA_OK(cudaGetDevice(&dev));
    if (dev != g->device)
        return fail(TFB_ERR_INVALID_ARG, "%s: the group member belongs to device %d but device %d is current", who,
                    g->device, dev);
    return TFB_OK;
}

void reset_peers(tfb_peer_group* g, int rank, int world) {
    for (int r = 0; r < kMaxWorld; ++r) {
        if (g->ipc_mapped[r] && g->peer_region[r] != nullptr) (void)cudaIpcCloseMemHandle(g->peer_region[r]);
        g->ipc_mapped[r] = false;
        g->peer_region[r] = nullptr;
    }
    (void)cudaGetLastError();
    g->rank = rank;
    g->world = world;
}

void fill(const tfb_peer_group* g, ReduceParams& p, int world, int64_t n) {
    memset(&p, 0, sizeof(p));
    p.world = world;
    p.n_vec = (n + 3) / 4;
    p.out_off = (long long)g->out_off;
    p.flags_off = (long long)g->flags_off;
    p.wait_ns = g->wait_ns;
}

void fill_rank(const tfb_peer_group* g, ReduceRank& r, int* status) {
    for (int i = 0; i < kMaxWorld; ++i) r.region[i] = g->peer_region[i];
    r.region[g->rank] = g->region;
    r.status = status;
    r.rank = g->rank;
}

int reduce_grid(int64_t n, int world, int ctas_available) {
    const long long per_rank = ((n + 3) / 4) / world + 1;
    long long g = (per_rank + kReduceThreads - 1) / kReduceThreads;
    if (g > ctas_available) g = ctas_available;
    if (g > kMaxExchangeCtas) g = kMaxExchangeCtas;
    return (int)(g < 1 ? 1 : g);
}

}  // namespace
}  // namespace tfb

extern "C" {

using namespace tfb;

int tfb_peer_group_create(int64_t capacity_floats, tfb_peer_group** out) {
    if (out == nullptr) return fail(TFB_ERR_INVALID_ARG, "peer_group_create: null output pointer");
    *out = nullptr;
    if (capacity_floats < 1) return fail(TFB_ERR_INVALID_ARG, "peer_group_create: capacity must be positive");
    DeviceState* st = nullptr;
    int rc = device_state(&st);
    if (rc != TFB_OK) return rc;
    tfb_peer_group* g = new (std::nothrow) tfb_peer_group();
    if (g == nullptr) return fail(TFB_ERR_NO_MEMORY, "peer_group_create: out of host memory");
    g->device = st->device;
    g->capacity = (capacity_floats + 3) / 4 * 4;
    g->out_off = align256((size_t)g->capacity * 4);
    g->flags_off = 2 * g->out_off;
    g->region_bytes = g->flags_off + align256(kFlagBytes);
    cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&g->region), g->region_bytes);
    if (e == cudaSuccess) e = cudaMemset(g->region, 0, g->region_bytes);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        if (g->region != nullptr) (void)cudaFree(g->region);
        const size_t wanted = g->region_bytes;
        delete g;
        return fail(TFB_ERR_NO_MEMORY, "peer_group_create: %zu bytes: %s", wanted, cudaGetErrorString(e));
    }
    *out = g;
    return TFB_OK;
}

int tfb_peer_group_destroy(tfb_peer_group* g) {
    if (g == nullptr) return TFB_OK;
    int prev = -1;
    TFB_CUDA_OK(cudaGetDevice(&prev));
    if (prev != g->device) TFB_CUDA_OK(cudaSetDevice(g->device));
    (void)cudaDeviceSynchronize();
    reset_peers(g, 0, 1);
    (void)cudaFree(g->region);
    (void)cudaGetLastError();
    if (prev != g->device) (void)cudaSetDevice(prev);
    delete g;
    return TFB_OK;
}

int tfb_peer_group_buffers(tfb_peer_group* g, float** in_out, float** out_out, void** region_out) {
    if (g == nullptr) return fail(TFB_ERR_INVALID_ARG, "peer_group_buffers: null group");
    if (in_out != nullptr) *in_out = reinterpret_cast<float*>(g->region);
    if (out_out != nullptr) *out_out = reinterpret_cast<float*>(g->region + g->out_off);
    if (region_out != nullptr) *region_out = g->region;
    return TFB_OK;
}

int tfb_peer_group_set_wait_limit(tfb_peer_group* g, int64_t nanoseconds) {
    if (g == nullptr || nanoseconds < 1000) return fail(TFB_ERR_INVALID_ARG, "peer_group_set_wait_limit: bad argument");
    g->wait_ns = (unsigned long long)nanoseconds;
    return TFB_OK;
}

int tfb_peer_group_ipc_handle(tfb_peer_group* g, void* handle_out) {
    int rc = check_group(g, "peer_group_ipc_handle");
    if (rc != TFB_OK) return rc;
    if (handle_out == nullptr) return fail(TFB_ERR_INVALID_ARG, "peer_group_ipc_handle: null output");
    cudaIpcMemHandle_t h;
    TFB_CUDA_OK(cudaIpcGetMemHandle(&h, g->region));
    memcpy(handle_out, &h, sizeof(h));
    return TFB_OK;
}

int tfb_peer_group_connect_ipc(tfb_peer_group* g, int rank, int world, const void* handles) {
    int rc = check_group(g, "peer_group_connect_ipc");
    if (rc != TFB_OK) return rc;
    if (world < 1 || world > kMaxWorld || rank < 0 || rank >= world || handles == nullptr)
        return fail(TFB_ERR_INVALID_ARG, "peer_group_connect_ipc: rank %d of %d (at most %d), or null handles", rank, world,
                    kMaxWorld);
    reset_peers(g, rank, world);
    for (int r = 0; r < world; ++r) {
        if (r == rank) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, static_cast<const uint8_t*>(handles) + (size_t)r * sizeof(h), sizeof(h));
        void* p = nullptr;
        cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) {
            (void)cudaGetLastError();
            reset_peers(g, 0, 1);
            return fail(TFB_ERR_CUDA, "peer_group_connect_ipc: opening rank %d's region failed: %s", r, cudaGetErrorString(e));
        }
        g->peer_region[r] = static_cast<uint8_t*>(p);
        g->ipc_mapped[r] = true;
    }
    return TFB_OK;
}

int tfb_peer_group_connect_ptrs(tfb_peer_group* g, int rank, int world, void* const* regions) {
    int rc = check_group(g, "peer_group_connect_ptrs");
    if (rc != TFB_OK) return rc;
    if (world < 1 || world > kMaxWorld || rank < 0 || rank >= world || (regions == nullptr && world > 1))
        return fail(TFB_ERR_INVALID_ARG, "peer_group_connect_ptrs: rank %d of %d (at most %d), or null regions", rank, world,
                    kMaxWorld);
    reset_peers(g, rank, world);
    for (int r = 0; r < world; ++r) {
        if (r == rank) continue;
        if (regions[r] == nullptr) {
            reset_peers(g, 0, 1);
            return fail(TFB_ERR_INVALID_ARG, "peer_group_connect_ptrs: region of rank %d is null", r);
        }
        g->peer_region[r] = static_cast<uint8_t*>(regions[r]);
    }
    return TFB_OK;
}

int tfb_peer_allreduce_sum(tfb_peer_group* g, int64_t n, void* stream) {
    int rc = check_group(g, "peer_allreduce_sum");
    if (rc != TFB_OK) return rc;
    if (n < 0 || n > g->capacity) return fail(TFB_ERR_TOO_LARGE, "peer_allreduce_sum: %lld floats, capacity %lld", (long long)n,
                                              (long long)g->capacity);
    if (n == 0) return TFB_OK;
    for (int r = 0; r < g->world; ++r)
        if (r != g->rank && g->peer_region[r] == nullptr)
            return fail(TFB_ERR_INVALID_ARG, "peer_allreduce_sum: rank %d of %d is not connected", r, g->world);
    DeviceState* st = nullptr;
    rc = device_state(&st);
    if (rc != TFB_OK) return rc;
    ReduceParams p;
    fill(g, p, g->world, n);
    fill_rank(g, p.ranks[0], st->status);
    return launch_pdl(peer_allreduce_kernel, dim3((unsigned)reduce_grid(n, g->world, st->sm_count), 1), dim3(kReduceThreads), 0,
                      static_cast<cudaStream_t>(stream), p);
}

int tfb_peer_allreduce_sum_one_device(tfb_peer_group* const* gs, int world, int64_t n, void* stream) {
    if (gs == nullptr || world < 1 || world > kMaxWorld)
        return fail(TFB_ERR_INVALID_ARG, "peer_allreduce_sum_one_device: 1..%d members", kMaxWorld);
    int rc = check_group(gs[0], "peer_allreduce_sum_one_device");
    if (rc != TFB_OK) return rc;
    for (int r = 0; r < world; ++r)
        if (gs[r] == nullptr || gs[r]->device != gs[0]->device || gs[r]->capacity != gs[0]->capacity || gs[r]->world != world ||
            gs[r]->rank != r)
            return fail(TFB_ERR_INVALID_ARG, "peer_allreduce_sum_one_device: member %d is not rank %d of %d on this device", r, r,
                        world);
    if (n < 0 || n > gs[0]->capacity) return fail(TFB_ERR_TOO_LARGE, "peer_allreduce_sum_one_device: %lld floats", (long long)n);
    if (n == 0) return TFB_OK;
    DeviceState* st = nullptr;
    rc = device_state(&st);
    if (rc != TFB_OK) return rc;
    ReduceParams p;
    fill(gs[0], p, world, n);
    for (int r = 0; r < world; ++r) fill_rank(gs[r], p.ranks[r], st->status);
    // One cooperative grid (blockIdx.y = rank): the CTAs that wait for each other are resident together.
    int per_sm = 0;
    TFB_CUDA_OK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, peer_allreduce_kernel, kReduceThreads, 0));
    const int grid = reduce_grid(n, world, st->sm_count * (per_sm > 0 ? per_sm : 1) / world);
    void* args[1] = {&p};
    TFB_CUDA_OK(cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(peer_allreduce_kernel),
                                            dim3((unsigned)grid, (unsigned)world), dim3(kReduceThreads), args, 0,
                                            static_cast<cudaStream_t>(stream)));
    return TFB_OK;
}

int tfb_conv2d_backward_sharded(tfb_peer_group* g, const void* x, const void* w, const void* grad_out, void* grad_input,
                                int64_t N_local, int64_t Cin, int64_t H, int64_t W, int64_t Cout, int64_t kH, int64_t kW,
                                int64_t stride_h, int64_t stride_w, int64_t pad_h, int64_t pad_w, int64_t dil_h,
                                int64_t dil_w, int allreduce, void* stream) {
    int rc = check_group(g, "conv2d_backward_sharded");
    if (rc != TFB_OK) return rc;
    const int64_t nw = Cout * Cin * kH * kW, nw4 = (nw + 3) / 4 * 4;
    if (nw4 + Cout > g->capacity)
        return fail(TFB_ERR_TOO_LARGE, "conv2d_backward_sharded: %lld gradient floats, the group holds %lld",
                    (long long)(nw4 + Cout), (long long)g->capacity);
    float* in = reinterpret_cast<float*>(g->region);
    // this rank's share of the weight and bias gradient goes straight into its contribution buffer
    rc = tfb_conv2d_backward(x, w, grad_out, grad_input, in, in + nw4, N_local, Cin, H, W, Cout, kH, kW, stride_h, stride_w,
                             pad_h, pad_w, dil_h, dil_w, TFB_DTYPE_F32, stream);
    if (rc != TFB_OK || allreduce == 0) return rc;
    return tfb_peer_allreduce_sum(g, nw4 + Cout, stream);
}

}  // extern "C"
