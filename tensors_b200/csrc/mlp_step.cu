// The data-parallel MLP training step as one C-ABI object (tfb_mlp): Linear -> ReLU -> ... -> Linear ->
// log_softmax + mean NLL -> backward -> gradient exchange -> SGD with momentum, every buffer owned
// here, no host read anywhere in the step (the dataflow of examples/train_mlp.cpp:161-183 with the
// update documented in nn/optim/SGD.hpp:3-6).
//
// Memory. Parameters, gradients and the loss contribution live in one "exchange region" per rank:
//     [ params : numel floats ][ grads : numel floats, then the loss slot ][ flags ]
// allocated with cudaMalloc so that other ranks can map it (same-process peers directly, other
// processes through a CUDA IPC handle). Every weight and bias starts on a 16-byte boundary of the
// flat buffers, so each is a legal TMA operand in place and one launch splits all weights into their
// TF32 hi / lo planes. Activations, their planes and the input gradients are carved from one arena
// sized for `max_rows` rows at creation; a step allocates nothing.
//
// Exchange (dp_exchange_kernel): reduce-scatter -> SGD -> all-gather fused into one kernel over
// NVLink peer memory. Rank r owns slice r of the flat buffers. After a flag barrier (every rank's
// gradients are complete) it loads slice r of every rank's gradient buffer — its own from HBM, the
// others with ordinary peer loads — adds them in rank order (a fixed order, so every run gives the
// same bits), applies the momentum update to its slice of the velocity and the parameters and
// stores the new parameter slice into every rank's parameter buffer with ordinary peer stores. A
// second flag barrier keeps any rank from starting its next step before all slices have landed in
// its parameters and all peers have finished reading its gradients. No load or store in the kernel
// uses cluster multicast or multimem; every wait is bounded by a wall-clock limit, after which the
// kernel records kDevTimeoutExchange in the device status word and returns.
//
// Flags are monotonic step counters (never reset), one word per (CTA, source rank) and barrier, and
// the step counter itself lives in device memory, so the kernel can be replayed from a CUDA graph.
// CTA b of a rank only ever waits for CTA b of the other ranks; all CTAs of the (at most one per
// SM) grid are resident at once, so no CTA waits for one that cannot be scheduled.
#include <cstring>
#include <new>
#include <vector>

#include "internal.hpp"
#include "peer_sync.cuh"
#include "ptx.cuh"

namespace tfb {

constexpr int kExchangeThreads = 512;

namespace {

struct DpRank {
    uint8_t* region[kMaxWorld];   // exchange regions of all ranks as this rank addresses them (own included)
    float* velocity;              // this rank's velocity (full length; only its slice is used when world > 1)
    float* reduced;               // optional: the summed gradient of this rank's slice is also stored here
    float* loss_out;              // sum of all ranks' loss contributions
    int* status;                  // device status word of this rank's device
    unsigned long long* trace;    // optional: CTA 0 stamps %globaltimer at the five phase boundaries
    int rank;
};

struct DpParams {
    DpRank ranks[kMaxWorld];      // one entry per rank this launch runs (blockIdx.y selects it)
    int world;
    long long n_vec;              // float4 vectors in the flat parameter / gradient buffers
    long long vec_lo, vec_hi;     // the part of them this launch exchanges (a "bucket"); rank r owns slice r of it
    int cta_base;                 // first flag row of this launch (concurrent launches use disjoint rows)
    int with_loss;                // this launch also sums the ranks' loss contributions
    long long params_off, grads_off, flags_off;   // byte offsets inside a region
    float lr, mu;
    unsigned long long wait_ns;
};

// WORLD > 0: compile-time group size (all loads of one vector are issued before the first add);
// U vectors per thread and iteration keep U * WORLD 16-byte loads in flight per thread.
template <int WORLD, int U>
__device__ __forceinline__ void exchange_slice_unrolled(const DpParams& p, const DpRank& me) {
    const int rank = me.rank;
    const long long span = p.vec_hi - p.vec_lo;
    const long long v0 = p.vec_lo + span * rank / WORLD, v1 = p.vec_lo + span * (rank + 1) / WORLD;
    const float lr = p.lr, mu = p.mu;
    float4* my_params = reinterpret_cast<float4*>(me.region[rank] + p.params_off);
    float4* vel = reinterpret_cast<float4*>(me.velocity);
    const long long threads = (long long)gridDim.x * blockDim.x;
    for (long long base = v0 + (long long)blockIdx.x * blockDim.x + threadIdx.x; base < v1; base += threads * U) {
        float4 g[U][WORLD], v[U], w[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const long long i = base + u * threads;
            if (i < v1) {
#pragma unroll
                for (int r = 0; r < WORLD; ++r)
                    g[u][r] = ld_peer(reinterpret_cast<const float4*>(me.region[r] + p.grads_off) + i);
                v[u] = vel[i];
                w[u] = my_params[i];
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const long long i = base + u * threads;
            if (i < v1) {
                float4 s = g[u][0];
#pragma unroll
                for (int r = 1; r < WORLD; ++r) {
                    s.x = __fadd_rn(s.x, g[u][r].x); s.y = __fadd_rn(s.y, g[u][r].y);
                    s.z = __fadd_rn(s.z, g[u][r].z); s.w = __fadd_rn(s.w, g[u][r].w);
                }
                if (me.reduced != nullptr) reinterpret_cast<float4*>(me.reduced)[i] = s;
                float4 vv = v[u], ww = w[u];
                // v <- mu * v + g ; p <- p - lr * v, separate multiply and add like the host formula.
                vv.x = __fadd_rn(__fmul_rn(mu, vv.x), s.x); vv.y = __fadd_rn(__fmul_rn(mu, vv.y), s.y);
                vv.z = __fadd_rn(__fmul_rn(mu, vv.z), s.z); vv.w = __fadd_rn(__fmul_rn(mu, vv.w), s.w);
                ww.x = __fsub_rn(ww.x, __fmul_rn(lr, vv.x)); ww.y = __fsub_rn(ww.y, __fmul_rn(lr, vv.y));
                ww.z = __fsub_rn(ww.z, __fmul_rn(lr, vv.z)); ww.w = __fsub_rn(ww.w, __fmul_rn(lr, vv.w));
                vel[i] = vv;
#pragma unroll
                for (int r = 0; r < WORLD; ++r) st_peer(reinterpret_cast<float4*>(me.region[r] + p.params_off) + i, ww);
            }
        }
    }
}

template <int WORLD>
__device__ __forceinline__ void exchange_slice(const DpParams& p, const DpRank& me, int world) {
    const int rank = me.rank;
    const long long span = p.vec_hi - p.vec_lo;
    const long long v0 = p.vec_lo + span * rank / world, v1 = p.vec_lo + span * (rank + 1) / world;
    const float lr = p.lr, mu = p.mu;
    float4* my_params = reinterpret_cast<float4*>(me.region[rank] + p.params_off);
    float4* vel = reinterpret_cast<float4*>(me.velocity);
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = v0 + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < v1; i += stride) {
        float4 g[WORLD > 0 ? WORLD : kMaxWorld];
        const int n = WORLD > 0 ? WORLD : world;
#pragma unroll
        for (int r = 0; r < (WORLD > 0 ? WORLD : kMaxWorld); ++r)
            if (r < n) g[r] = ld_peer(reinterpret_cast<const float4*>(me.region[r] + p.grads_off) + i);
        float4 s = g[0];
#pragma unroll
        for (int r = 1; r < (WORLD > 0 ? WORLD : kMaxWorld); ++r)
            if (r < n) {
                s.x = __fadd_rn(s.x, g[r].x); s.y = __fadd_rn(s.y, g[r].y);
                s.z = __fadd_rn(s.z, g[r].z); s.w = __fadd_rn(s.w, g[r].w);
            }
        if (me.reduced != nullptr) reinterpret_cast<float4*>(me.reduced)[i] = s;
        float4 v = vel[i];
        float4 w = my_params[i];
        // v <- mu * v + g ; p <- p - lr * v, separate multiply and add like the host formula.
        v.x = __fadd_rn(__fmul_rn(mu, v.x), s.x); v.y = __fadd_rn(__fmul_rn(mu, v.y), s.y);
        v.z = __fadd_rn(__fmul_rn(mu, v.z), s.z); v.w = __fadd_rn(__fmul_rn(mu, v.w), s.w);
        w.x = __fsub_rn(w.x, __fmul_rn(lr, v.x)); w.y = __fsub_rn(w.y, __fmul_rn(lr, v.y));
        w.z = __fsub_rn(w.z, __fmul_rn(lr, v.z)); w.w = __fsub_rn(w.w, __fmul_rn(lr, v.w));
        vel[i] = v;
#pragma unroll
        for (int r = 0; r < (WORLD > 0 ? WORLD : kMaxWorld); ++r)
            if (r < n) st_peer(reinterpret_cast<float4*>(me.region[r] + p.params_off) + i, w);
    }
}

__global__ void __launch_bounds__(kExchangeThreads)
dp_exchange_kernel(const __grid_constant__ DpParams p) {
    pdl_wait();
    pdl_launch_dependents();
    const DpRank& me = p.ranks[blockIdx.y];
    const int world = p.world, rank = me.rank, cta = p.cta_base + (int)blockIdx.x;   // flag row
    uint8_t* mine = me.region[rank];
    uint32_t* epoch_word = reinterpret_cast<uint32_t*>(mine + p.flags_off) + cta;
    const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(epoch_word) + 1u;
    const int t = threadIdx.x;
    const bool tracing = me.trace != nullptr && cta == 0 && t == 0 && p.with_loss != 0;
    if (tracing) me.trace[0] = global_timer_ns();

    // Barrier 0: every rank's gradients (written by the kernels before this one on its stream) are complete.
    // A group of one has nobody to wait for and leaves the flags and the step counter alone.
    int ok = 1;
    if (world > 1 && t < world) {
        // nothing this kernel wrote is published here (the gradients were completed by the kernels before
        // it on the stream), so the arrival is a relaxed store
        st_relaxed_sys(flag_word(me.region[t], p.flags_off, 0, cta, rank), epoch);
        if (!wait_flag(flag_word(mine, p.flags_off, 0, cta, t), epoch, p.wait_ns)) {
            ok = 0;
            if (me.status != nullptr) atomicCAS(me.status, 0, kDevTimeoutExchange);
        }
    }
    ok = __syncthreads_and(ok);
    if (tracing) me.trace[1] = global_timer_ns();
    if (ok) {
        if (p.with_loss != 0 && blockIdx.x == 0 && t == 0) {
            // Loss: the ranks' contributions in rank order (the slot after the gradients).
            float l = 0.f;
            for (int r = 0; r < world; ++r) {
                const float4 v = ld_peer(reinterpret_cast<const float4*>(me.region[r] + p.grads_off) + p.n_vec);
                l = r == 0 ? v.x : __fadd_rn(l, v.x);
            }
            *me.loss_out = l;
        }
        switch (world) {
        case 1: exchange_slice_unrolled<1, 4>(p, me); break;
        case 2: exchange_slice_unrolled<2, 4>(p, me); break;
        case 4: exchange_slice_unrolled<4, 2>(p, me); break;
        case 8: exchange_slice_unrolled<8, 1>(p, me); break;
        default: exchange_slice<0>(p, me, world); break;
        }
    }
    // Barrier 1: my slice has landed everywhere and I have finished reading the peers' gradients. It is
    // signalled even after a failed first barrier so that the other ranks are not kept waiting for long.
    if (world == 1) return;
    __syncthreads();
    if (tracing) me.trace[2] = global_timer_ns();
    if (t < world) {
        // one fence at system scope (cumulative over the CTA's stores through the barrier above: all slices
        // this CTA stored have landed), then relaxed arrivals
        __threadfence_system();
        if (tracing) me.trace[3] = global_timer_ns();
        st_relaxed_sys(flag_word(me.region[t], p.flags_off, 1, cta, rank), epoch);
        if (ok && !wait_flag(flag_word(mine, p.flags_off, 1, cta, t), epoch, p.wait_ns)) {
            if (me.status != nullptr) atomicCAS(me.status, 0, kDevTimeoutExchange);
        }
    }
    __syncthreads();
    if (tracing) me.trace[4] = global_timer_ns();
    if (t == 0) *reinterpret_cast<volatile uint32_t*>(epoch_word) = epoch;
}

inline int64_t round_up(int64_t x, int64_t m) { return (x + m - 1) / m * m; }
inline size_t align256(size_t x) { return (x + 255) & ~(size_t)255; }

}  // namespace
}  // namespace tfb

// The opaque handle of include/tfb.h.
struct tfb_mlp {
    int device = -1;
    int L = 0;
    std::vector<int64_t> dims, w_off, b_off;
    int64_t numel = 0;       // floats in the flat buffers (every segment padded to a multiple of 4)
    int64_t max_rows = 0;
    // exchange region
    uint8_t* region = nullptr;
    size_t region_bytes = 0, grads_off = 0, flags_off = 0;
    float* params = nullptr;
    float* grads = nullptr;  // numel floats + the loss slot (4 floats, the first is used)
    // everything else: one arena
    uint8_t* arena = nullptr;
    float* velocity = nullptr;
    float* reduced = nullptr;
    float* loss = nullptr;
    unsigned long long* trace = nullptr;  // 8 words behind the loss
    bool trace_on = false;
    float* pplanes = nullptr;             // hi / lo planes of the flat parameter buffer (2 x numel)
    std::vector<float*> wplanes;          // per layer, only where in_features is not a multiple of 4
    std::vector<float*> act;              // act[i + 1] = output of layer i
    std::vector<float*> xplanes;          // hi / lo planes of the input of layer i
    std::vector<float*> dx;               // gradient with respect to the input of layer i (i > 0)
    float* dz = nullptr;                  // gradient with respect to the logits
    float* row_loss = nullptr;            // per-row losses of the last step (max_rows floats)
    std::vector<float*> colsum;           // per layer: partial column sums of its bias gradient
    std::vector<size_t> colsum_floats;
    // data-parallel group
    int rank = 0, world = 1;
    uint8_t* peer_region[tfb::kMaxWorld] = {nullptr};
    bool ipc_mapped[tfb::kMaxWorld] = {false};
    unsigned long long wait_ns = 2000000000ull;
    int exchange_ctas = 0;                // 0 = choose
    bool keep_reduced = false;
    // Two-bucket step: the gradients of every layer but the first are exchanged on a side stream while the
    // first layer's weight gradient is still being computed.
    int buckets = 1;
    cudaStream_t side = nullptr;
    cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
    // captured step
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t graph_exec = nullptr;
};

namespace tfb {
namespace {

struct DeviceScope {
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
    ~DeviceScope() {
        if (switched) (void)cudaSetDevice(prev);
    }
};

int check_handle(const tfb_mlp* m, const char* who) {
    if (m == nullptr) return fail(TFB_ERR_INVALID_ARG, "%s: null handle", who);
    int dev = -1;
    TFB_CUDA_OK(cudaGetDevice(&dev));
    if (dev != m->device)
        return fail(TFB_ERR_INVALID_ARG, "%s: the handle belongs to device %d but device %d is current", who, m->device,
                    dev);
    return TFB_OK;
}

void fill_rank(const tfb_mlp* m, DpRank& r, int* status) {
    for (int i = 0; i < kMaxWorld; ++i) r.region[i] = m->peer_region[i];
    r.region[m->rank] = m->region;
    r.velocity = m->velocity;
    r.reduced = m->keep_reduced ? m->reduced : nullptr;
    r.loss_out = m->loss;
    r.status = status;
    r.trace = m->trace_on ? m->trace : nullptr;
    r.rank = m->rank;
}

void fill_params(const tfb_mlp* m, DpParams& p, int world, float lr, float mu) {
    memset(&p, 0, sizeof(p));
    p.world = world;
    p.n_vec = m->numel / 4;
    p.vec_lo = 0;
    p.vec_hi = p.n_vec;
    p.cta_base = 0;
    p.with_loss = 1;
    p.params_off = 0;
    p.grads_off = (long long)m->grads_off;
    p.flags_off = (long long)m->flags_off;
    p.lr = lr;
    p.mu = mu;
    p.wait_ns = m->wait_ns;
}

int exchange_grid(const tfb_mlp* m, int sm_count, int ranks_in_launch, int world, long long vecs = -1, int cap = 0) {
    // At most one CTA per SM (all CTAs must be resident while they wait for their peers), and enough
    // of them to keep a few MB of peer loads in flight.
    if (vecs < 0) vecs = m->numel / 4;
    int g = m->exchange_ctas > 0 ? m->exchange_ctas : 128;
    if (cap > 0 && g > cap) g = cap;
    // A group of one waits for nobody, so its CTAs need not all be resident: fill the GPU.
    if (world == 1 && m->exchange_ctas == 0) g = 4 * sm_count;
    else if (g > sm_count / ranks_in_launch) g = sm_count / ranks_in_launch;
    if (g > kMaxExchangeCtas) g = kMaxExchangeCtas;
    const long long vec_per_rank = vecs / (world > 0 ? world : 1) + 1;
    const long long want = (vec_per_rank + kExchangeThreads - 1) / kExchangeThreads;
    if (g > want) g = (int)want;
    if (g < 1) g = 1;
    return g;
}

// Local update of one rank from its own gradient buffer (world = 1 inside the kernel): the plain SGD
// step of a single rank, and the update after an external all-reduce has summed the buffers.
int launch_update(tfb_mlp* m, int world_in_kernel, float lr, float mu, cudaStream_t stream) {
    DeviceState* st = nullptr;
    int rc = device_state(&st);
    if (rc != TFB_OK) return rc;
    DpParams p;
    fill_params(m, p, world_in_kernel, lr, mu);
    fill_rank(m, p.ranks[0], st->status);
    if (world_in_kernel == 1) {
        // the kernel indexes region[rank]; as a group of one this rank is rank 0
        p.ranks[0].rank = 0;
        p.ranks[0].region[0] = m->region;
    }
    const int grid = exchange_grid(m, st->sm_count, 1, world_in_kernel);
    return launch_pdl(dp_exchange_kernel, dim3((unsigned)grid, 1), dim3(kExchangeThreads), 0, stream, p);
}

// The flag rows of the early bucket of a two-bucket step, and its CTA limit: few enough to run on the SMs
// the last weight-gradient product of a shard leaves free.
constexpr int kEarlyBucketFlagRow = 128;
constexpr int kEarlyBucketCtas = 32;

// Exchange + update of the float4 range [lo, hi) of the flat buffers over the whole group.
int launch_bucket(tfb_mlp* m, float lr, float mu, long long lo, long long hi, bool early, cudaStream_t stream) {
    DeviceState* st = nullptr;
    int rc = device_state(&st);
    if (rc != TFB_OK) return rc;
    DpParams p;
    fill_params(m, p, m->world, lr, mu);
    fill_rank(m, p.ranks[0], st->status);
    p.vec_lo = lo;
    p.vec_hi = hi;
    p.cta_base = early ? kEarlyBucketFlagRow : 0;
    p.with_loss = early ? 0 : 1;
    int grid = exchange_grid(m, st->sm_count, 1, m->world, hi - lo, early ? kEarlyBucketCtas : 0);
    if (grid > kEarlyBucketFlagRow) grid = kEarlyBucketFlagRow;   // rows [0, 128) and [128, 256) stay disjoint
    return launch_pdl(dp_exchange_kernel, dim3((unsigned)grid, 1), dim3(kExchangeThreads), 0, stream, p);
}

// True when a whole step of this handle runs as two buckets (tfb_mlp_step, and a captured whole step).
bool two_buckets(const tfb_mlp* m) {
    if (m->buckets != 2 || m->world < 2 || m->L < 2) return false;
    for (int r = 0; r < m->world; ++r)
        if (r != m->rank && m->peer_region[r] == nullptr) return false;
    return true;
}

// The side stream and the two events of the two-bucket step, created on first use.
int bucket_streams(tfb_mlp* m) {
    if (m->side != nullptr) return TFB_OK;
    TFB_CUDA_OK(cudaStreamCreateWithFlags(&m->side, cudaStreamNonBlocking));
    TFB_CUDA_OK(cudaEventCreateWithFlags(&m->ev_fork, cudaEventDisableTiming));
    TFB_CUDA_OK(cudaEventCreateWithFlags(&m->ev_join, cudaEventDisableTiming));
    return TFB_OK;
}

// Forward, loss and backward of one batch. With `exchange` the group's exchange + update is part of the call
// (lr, mu are then used): as one launch behind the backward pass, or — two_buckets(m) — with the gradients
// of layers 1.. exchanged on the side stream as soon as layer 1's backward is enqueued, concurrently with
// layer 0's weight gradient, and layer 0's (with the loss) behind it on `stream`, which then waits for the
// side stream.
int forward_backward(tfb_mlp* m, const float* X, const int64_t* labels, int64_t rows, int64_t global_rows,
                     cudaStream_t stream, bool exchange = false, float lr = 0.f, float mu = 0.f) {
    const int L = m->L;
    const bool bucketed = exchange && two_buckets(m);
    if (bucketed) {
        const int rcs = bucket_streams(m);
        if (rcs != TFB_OK) return rcs;
    }
    // Where an operand can be its own hi plane (aligned, width a multiple of 4) only its lo plane is written:
    // the parameters as one flat vector, the batch, and each hidden activation.
    const bool raw_params = raw_hi_operand(m->params, m->numel, nullptr);
    // ... in one launch with the batch, whose planes the first product needs
    const int64_t in0 = m->dims[0], ld0 = round_up(in0, 4);
    const bool raw_x = raw_hi_operand(X, in0, nullptr);
    int rc = split_operands2(m->params, 1, m->numel, m->numel, raw_params ? nullptr : m->pplanes, m->pplanes + m->numel,
                             m->numel, X, rows, in0, in0, raw_x ? nullptr : m->xplanes[0], m->xplanes[0] + rows * ld0, ld0,
                             stream);
    if (rc != TFB_OK) return rc;
    std::vector<SavedPlanes> xs((size_t)L), ws((size_t)L);
    DeviceState* st = nullptr;
    rc = device_state(&st);
    if (rc != TFB_OK) return rc;
    const int fuse = tuning(TFB_TUNE_FUSE_PLANES);
    bool planes_ready = true;    // are this layer's input planes written already (layer 0: above; else by the product below)?
    bool ready_raw = raw_x;      // ... in the raw-hi form (lo plane only)?
    for (int i = 0; i < L; ++i) {
        const int64_t in_f = m->dims[(size_t)i], out_f = m->dims[(size_t)i + 1];
        const float* in = i == 0 ? X : m->act[(size_t)i];
        const int64_t ldx = round_up(in_f, 4);
        float* xh = m->xplanes[(size_t)i];
        float* xl = xh + rows * ldx;
        // The planes of a hidden layer's input were written by the product that made it (its epilogue);
        // only the batch itself, and inputs whose width is not a multiple of 4, are split here.
        bool raw_in = planes_ready ? ready_raw : raw_hi_operand(in, in_f, nullptr);
        if (!planes_ready) {
            rc = split_operand(in, rows, in_f, in_f, nullptr, raw_in ? nullptr : xh, xl, ldx, stream);
            if (rc != TFB_OK) return rc;
        }
        xs[(size_t)i].hi = raw_in ? in : xh; xs[(size_t)i].lo = xl; xs[(size_t)i].ld = ldx;   // raw: in_f == ldx
        xs[(size_t)i].raw_hi = raw_in;
        if (m->wplanes[(size_t)i] == nullptr) {
            ws[(size_t)i].hi = (raw_params ? m->params : m->pplanes) + m->w_off[(size_t)i];
            ws[(size_t)i].lo = m->pplanes + m->numel + m->w_off[(size_t)i];
            ws[(size_t)i].ld = in_f;
            ws[(size_t)i].raw_hi = raw_params;
        } else {
            float* wh = m->wplanes[(size_t)i];
            float* wl = wh + out_f * ldx;
            rc = split_operand(m->params + m->w_off[(size_t)i], out_f, in_f, in_f, nullptr, wh, wl, ldx, stream);
            if (rc != TFB_OK) return rc;
            ws[(size_t)i].hi = wh; ws[(size_t)i].lo = wl; ws[(size_t)i].ld = ldx;
        }
        GemmCall c;
        c.A = xs[(size_t)i].hi; c.a_presplit = true; c.a_lo_off = xs[(size_t)i].lo - xs[(size_t)i].hi;
        c.a_raw_hi = xs[(size_t)i].raw_hi;
        c.B = ws[(size_t)i].hi; c.b_presplit = true; c.b_lo_off = ws[(size_t)i].lo - ws[(size_t)i].hi;
        c.b_raw_hi = ws[(size_t)i].raw_hi;
        c.C = m->act[(size_t)i + 1];
        c.M = rows; c.N = out_f; c.K = in_f;
        c.lda = ldx; c.ldb = ws[(size_t)i].ld; c.ldc = out_f;
        c.a_kmajor = true; c.b_kmajor = true;
        c.in_dtype = TFB_DTYPE_F32; c.out_dtype = TFB_DTYPE_F32;
        c.bias = m->params + m->b_off[(size_t)i]; c.bias_mode = 1;
        c.relu = i < L - 1;
        // Where it costs nothing the product also writes the planes the next layer multiplies: always in
        // the reduction kernel of a split-K product; in the GEMM epilogue only on request (measured: the
        // longer epilogue costs the large-batch products more than the separate pass it saves).
        planes_ready = false;
        if (i + 1 < L && (out_f & 3) == 0 &&
            (fuse == 2 || (fuse == 1 && (gemm_uses_split_k(c, st->sm_count) || gemm_uses_cluster_k(c, st->sm_count) ||
                                         small_gemm_eligible(c))))) {
            // raw-hi form where the output itself can be the next product's hi plane
            ready_raw = raw_hi_operand(c.C, out_f, nullptr);
            c.planes_hi = ready_raw ? nullptr : m->xplanes[(size_t)i + 1];
            c.planes_lo = m->xplanes[(size_t)i + 1] + rows * out_f;
            planes_ready = true;
        }
        rc = gemm_run(c, stream);
        if (rc != TFB_OK) return rc;
    }
    // The final additions of the loss and of every layer's bias gradient are short single-block-column
    // reductions that nothing in the backward pass waits for: they run as ONE launch at the end instead of one
    // launch each between the products. The loss goes to the slot behind the gradients, so that the exchange
    // sums it too.
    rc = log_softmax_nll_rows(m->act[(size_t)L], labels, m->dz, m->row_loss, rows, m->dims[(size_t)L], global_rows,
                              stream);
    if (rc != TFB_OK) return rc;
    std::vector<DeferredColsum> finish((size_t)L);
    const float* upstream = m->dz;
    for (int i = L - 1; i >= 0; --i) {
        float* dX = i > 0 ? m->dx[(size_t)i] : nullptr;
        SavedPlanes wsv = dX != nullptr ? ws[(size_t)i] : SavedPlanes();
        DeferredColsum& d = finish[(size_t)(L - 1 - i)];
        d.partial = m->colsum[(size_t)i];
        d.capacity_floats = m->colsum_floats[(size_t)i];
        rc = linear_backward_impl(nullptr, nullptr, m->act[(size_t)i + 1], upstream, dX, m->grads + m->w_off[(size_t)i],
                                  m->grads + m->b_off[(size_t)i], rows, m->dims[(size_t)i], m->dims[(size_t)i + 1],
                                  i < L - 1, TFB_DTYPE_F32, stream, xs[(size_t)i], wsv, &d);
        if (rc != TFB_OK) return rc;
        upstream = dX;
        if (bucketed && i == 1) {
            // everything layers 1.. contribute is enqueued: finish their bias gradients and exchange them on
            // the side stream (jobs 0 .. L-2 of `finish` are layers L-1 .. 1)
            TFB_CUDA_OK(cudaEventRecord(m->ev_fork, stream));
            TFB_CUDA_OK(cudaStreamWaitEvent(m->side, m->ev_fork, 0));
            rc = colsum_finish_many(finish.data(), L - 1, nullptr, 0, global_rows, nullptr, m->side);
            if (rc != TFB_OK) return rc;
            rc = launch_bucket(m, lr, mu, m->w_off[1] / 4, m->numel / 4, true, m->side);
            if (rc != TFB_OK) return rc;
            TFB_CUDA_OK(cudaEventRecord(m->ev_join, m->side));
        }
    }
    if (bucketed) {
        rc = colsum_finish_many(&finish[(size_t)L - 1], 1, m->row_loss, rows, global_rows, m->grads + m->numel, stream);
        if (rc != TFB_OK) return rc;
        rc = launch_bucket(m, lr, mu, 0, m->w_off[1] / 4, false, stream);
        if (rc != TFB_OK) return rc;
        TFB_CUDA_OK(cudaStreamWaitEvent(stream, m->ev_join, 0));
        return TFB_OK;
    }
    rc = colsum_finish_many(finish.data(), L, m->row_loss, rows, global_rows, m->grads + m->numel, stream);
    if (rc != TFB_OK || !exchange) return rc;
    if (m->world == 1) return launch_update(m, 1, lr, mu, stream);
    return launch_update(m, m->world, lr, mu, stream);
}

int check_batch(const tfb_mlp* m, const float* X, const int64_t* labels, int64_t rows, int64_t global_rows,
                const char* who) {
    if (X == nullptr || labels == nullptr) return fail(TFB_ERR_INVALID_ARG, "%s: null batch pointer", who);
    if (rows <= 0 || rows > m->max_rows)
        return fail(TFB_ERR_INVALID_ARG, "%s: %lld rows, the handle was created for 1..%lld", who, (long long)rows,
                    (long long)m->max_rows);
    if (global_rows < rows) return fail(TFB_ERR_INVALID_ARG, "%s: global batch smaller than this rank's share", who);
    return TFB_OK;
}

}  // namespace
}  // namespace tfb

extern "C" {

using namespace tfb;

int tfb_mlp_create(int n_layers, const int64_t* dims, int64_t max_rows, tfb_mlp** out) {
    if (out == nullptr) return fail(TFB_ERR_INVALID_ARG, "mlp_create: null output pointer");
    *out = nullptr;
    if (n_layers < 1 || n_layers > 64 || dims == nullptr || max_rows < 1)
        return fail(TFB_ERR_INVALID_ARG, "mlp_create: bad layer count, dims or row limit");
    for (int i = 0; i <= n_layers; ++i)
        if (dims[i] < 1) return fail(TFB_ERR_INVALID_ARG, "mlp_create: dims[%d] = %lld", i, (long long)dims[i]);
    DeviceState* st = nullptr;
    int rc = device_state(&st);
    if (rc != TFB_OK) return rc;
    tfb_mlp* m = new (std::nothrow) tfb_mlp();
    if (m == nullptr) return fail(TFB_ERR_NO_MEMORY, "mlp_create: out of host memory");
    m->device = st->device;
    m->L = n_layers;
    m->dims.assign(dims, dims + n_layers + 1);
    m->max_rows = max_rows;
    int64_t off = 0;
    for (int i = 0; i < n_layers; ++i) {
        m->w_off.push_back(off);
        off += round_up(dims[i + 1] * dims[i], 4);
        m->b_off.push_back(off);
        off += round_up(dims[i + 1], 4);
    }
    m->numel = off;
    m->grads_off = align256((size_t)off * 4);
    m->flags_off = m->grads_off + align256((size_t)(off + 4) * 4);
    m->region_bytes = m->flags_off + align256(kFlagBytes);
    cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&m->region), m->region_bytes);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        const size_t wanted = m->region_bytes;
        delete m;
        return fail(TFB_ERR_NO_MEMORY, "mlp_create: %zu bytes for the exchange region: %s", wanted,
                    cudaGetErrorString(e));
    }
    m->params = reinterpret_cast<float*>(m->region);
    m->grads = reinterpret_cast<float*>(m->region + m->grads_off);
    // arena layout
    size_t need = 0;
    auto reserve = [&](size_t bytes) {
        const size_t at = need;
        need += align256(bytes);
        return at;
    };
    const size_t o_vel = reserve((size_t)off * 4), o_red = reserve((size_t)off * 4), o_loss = reserve(256);
    const size_t o_pp = reserve((size_t)off * 8);
    std::vector<size_t> o_wp((size_t)n_layers, (size_t)-1), o_act((size_t)n_layers + 1, 0), o_xp((size_t)n_layers, 0),
        o_dx((size_t)n_layers, 0);
    for (int i = 0; i < n_layers; ++i) {
        const int64_t ld = round_up(dims[i], 4);
        if (dims[i] % 4 != 0) o_wp[(size_t)i] = reserve((size_t)(2 * dims[i + 1] * ld) * 4);
        o_act[(size_t)i + 1] = reserve((size_t)(max_rows * dims[i + 1]) * 4);
        o_xp[(size_t)i] = reserve((size_t)(2 * max_rows * ld) * 4);
        if (i > 0) o_dx[(size_t)i] = reserve((size_t)(max_rows * dims[i]) * 4);
    }
    const size_t o_dz = reserve((size_t)(max_rows * dims[n_layers]) * 4);
    const size_t o_rl = reserve((size_t)max_rows * 4);
    std::vector<size_t> o_cs((size_t)n_layers, 0);
    m->colsum_floats.assign((size_t)n_layers, 0);
    for (int i = 0; i < n_layers; ++i) {
        m->colsum_floats[(size_t)i] = deferred_colsum_floats(max_rows, dims[i + 1]);
        o_cs[(size_t)i] = reserve(m->colsum_floats[(size_t)i] * 4);
    }
    e = cudaMalloc(reinterpret_cast<void**>(&m->arena), need);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        (void)cudaFree(m->region);
        delete m;
        return fail(TFB_ERR_NO_MEMORY, "mlp_create: %zu bytes for activations and planes: %s", need,
                    cudaGetErrorString(e));
    }
    m->velocity = reinterpret_cast<float*>(m->arena + o_vel);
    m->reduced = reinterpret_cast<float*>(m->arena + o_red);
    m->loss = reinterpret_cast<float*>(m->arena + o_loss);
    m->trace = reinterpret_cast<unsigned long long*>(m->arena + o_loss + 64);
    m->pplanes = reinterpret_cast<float*>(m->arena + o_pp);
    m->wplanes.assign((size_t)n_layers, nullptr);
    m->act.assign((size_t)n_layers + 1, nullptr);
    m->xplanes.assign((size_t)n_layers, nullptr);
    m->dx.assign((size_t)n_layers, nullptr);
    for (int i = 0; i < n_layers; ++i) {
        if (o_wp[(size_t)i] != (size_t)-1) m->wplanes[(size_t)i] = reinterpret_cast<float*>(m->arena + o_wp[(size_t)i]);
        m->act[(size_t)i + 1] = reinterpret_cast<float*>(m->arena + o_act[(size_t)i + 1]);
        m->xplanes[(size_t)i] = reinterpret_cast<float*>(m->arena + o_xp[(size_t)i]);
        if (i > 0) m->dx[(size_t)i] = reinterpret_cast<float*>(m->arena + o_dx[(size_t)i]);
    }
    m->dz = reinterpret_cast<float*>(m->arena + o_dz);
    m->row_loss = reinterpret_cast<float*>(m->arena + o_rl);
    m->colsum.assign((size_t)n_layers, nullptr);
    for (int i = 0; i < n_layers; ++i) m->colsum[(size_t)i] = reinterpret_cast<float*>(m->arena + o_cs[(size_t)i]);
    // parameters, gradients, flags, velocity and loss start at zero
    if (cudaMemset(m->region, 0, m->region_bytes) != cudaSuccess ||
        cudaMemset(m->arena, 0, o_pp) != cudaSuccess) {
        (void)cudaGetLastError();
        (void)cudaFree(m->arena);
        (void)cudaFree(m->region);
        delete m;
        return fail(TFB_ERR_CUDA, "mlp_create: clearing the buffers failed");
    }
    *out = m;
    return TFB_OK;
}

int tfb_mlp_destroy(tfb_mlp* m) {
    if (m == nullptr) return TFB_OK;
    DeviceScope scope;
    int rc = scope.enter(m->device);
    if (rc != TFB_OK) return rc;
    (void)cudaDeviceSynchronize();
    if (m->graph_exec != nullptr) (void)cudaGraphExecDestroy(m->graph_exec);
    if (m->graph != nullptr) (void)cudaGraphDestroy(m->graph);
    if (m->ev_fork != nullptr) (void)cudaEventDestroy(m->ev_fork);
    if (m->ev_join != nullptr) (void)cudaEventDestroy(m->ev_join);
    if (m->side != nullptr) (void)cudaStreamDestroy(m->side);
    for (int r = 0; r < kMaxWorld; ++r)
        if (m->ipc_mapped[r] && m->peer_region[r] != nullptr) (void)cudaIpcCloseMemHandle(m->peer_region[r]);
    (void)cudaFree(m->arena);
    (void)cudaFree(m->region);
    (void)cudaGetLastError();
    delete m;
    return TFB_OK;
}

int64_t tfb_mlp_numel(const tfb_mlp* m) { return m != nullptr ? m->numel : 0; }

int tfb_mlp_segment(const tfb_mlp* m, int layer, int64_t* weight_offset, int64_t* bias_offset) {
    if (m == nullptr || layer < 0 || layer >= m->L) return fail(TFB_ERR_INVALID_ARG, "mlp_segment: bad handle or layer");
    if (weight_offset != nullptr) *weight_offset = m->w_off[(size_t)layer];
    if (bias_offset != nullptr) *bias_offset = m->b_off[(size_t)layer];
    return TFB_OK;
}

int tfb_mlp_buffer(tfb_mlp* m, int which, int layer, void** ptr_out) {
    if (m == nullptr || ptr_out == nullptr) return fail(TFB_ERR_INVALID_ARG, "mlp_buffer: null argument");
    *ptr_out = nullptr;
    switch (which) {
    case TFB_MLP_PARAMS: *ptr_out = m->params; break;
    case TFB_MLP_GRADS: *ptr_out = m->grads; break;
    case TFB_MLP_VELOCITY: *ptr_out = m->velocity; break;
    case TFB_MLP_LOSS: *ptr_out = m->loss; break;
    case TFB_MLP_REDUCED_GRADS: *ptr_out = m->reduced; break;
    case TFB_MLP_ACTIVATION:
        if (layer < 0 || layer >= m->L) return fail(TFB_ERR_INVALID_ARG, "mlp_buffer: layer %d", layer);
        *ptr_out = m->act[(size_t)layer + 1];
        break;
    case TFB_MLP_REGION: *ptr_out = m->region; break;
    case TFB_MLP_EXCHANGE_TRACE: *ptr_out = m->trace; break;
    case TFB_MLP_INPUT_GRAD:
        if (layer < 1 || layer >= m->L) return fail(TFB_ERR_INVALID_ARG, "mlp_buffer: layer %d has no input gradient", layer);
        *ptr_out = m->dx[(size_t)layer];
        break;
    default: return fail(TFB_ERR_INVALID_ARG, "mlp_buffer: unknown buffer %d", which);
    }
    return TFB_OK;
}

int tfb_mlp_forward_backward(tfb_mlp* m, const float* X, const int64_t* labels, int64_t rows, int64_t global_rows,
                             void* stream) {
    int rc = check_handle(m, "mlp_forward_backward");
    if (rc != TFB_OK) return rc;
    if (global_rows <= 0) global_rows = rows;
    rc = check_batch(m, X, labels, rows, global_rows, "mlp_forward_backward");
    if (rc != TFB_OK) return rc;
    return forward_backward(m, X, labels, rows, global_rows, static_cast<cudaStream_t>(stream));
}

int tfb_mlp_update(tfb_mlp* m, float lr, float momentum, void* stream) {
    int rc = check_handle(m, "mlp_update");
    if (rc != TFB_OK) return rc;
    return launch_update(m, 1, lr, momentum, static_cast<cudaStream_t>(stream));
}

int tfb_mlp_exchange_update(tfb_mlp* m, float lr, float momentum, void* stream) {
    int rc = check_handle(m, "mlp_exchange_update");
    if (rc != TFB_OK) return rc;
    if (m->world == 1) return launch_update(m, 1, lr, momentum, static_cast<cudaStream_t>(stream));
    for (int r = 0; r < m->world; ++r)
        if (r != m->rank && m->peer_region[r] == nullptr)
            return fail(TFB_ERR_INVALID_ARG, "mlp_exchange_update: rank %d of %d is not connected", r, m->world);
    return launch_update(m, m->world, lr, momentum, static_cast<cudaStream_t>(stream));
}

static int check_connected(const tfb_mlp* m, const char* who) {
    for (int r = 0; r < m->world; ++r)
        if (r != m->rank && m->peer_region[r] == nullptr)
            return fail(TFB_ERR_INVALID_ARG, "%s: rank %d of %d is not connected", who, r, m->world);
    return TFB_OK;
}

int tfb_mlp_step(tfb_mlp* m, const float* X, const int64_t* labels, int64_t rows, int64_t global_rows, float lr,
                 float momentum, void* stream) {
    int rc = check_handle(m, "mlp_step");
    if (rc != TFB_OK) return rc;
    if (global_rows <= 0) global_rows = rows;
    rc = check_batch(m, X, labels, rows, global_rows, "mlp_step");
    if (rc != TFB_OK) return rc;
    rc = check_connected(m, "mlp_step");
    if (rc != TFB_OK) return rc;
    return forward_backward(m, X, labels, rows, global_rows, static_cast<cudaStream_t>(stream), true, lr, momentum);
}

int tfb_mlp_capture_step(tfb_mlp* m, const float* X, const int64_t* labels, int64_t rows, int64_t global_rows,
                         float lr, float momentum, int what, void* stream_v) {
    int rc = check_handle(m, "mlp_capture_step");
    if (rc != TFB_OK) return rc;
    if (global_rows <= 0) global_rows = rows;
    if (what != TFB_MLP_CAPTURE_UPDATE) {
        rc = check_batch(m, X, labels, rows, global_rows, "mlp_capture_step");
        if (rc != TFB_OK) return rc;
    }
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    if (stream == nullptr || stream == cudaStreamLegacy)
        return fail(TFB_ERR_INVALID_ARG, "mlp_capture_step: the legacy default stream cannot be captured");
    if (m->graph_exec != nullptr) { (void)cudaGraphExecDestroy(m->graph_exec); m->graph_exec = nullptr; }
    if (m->graph != nullptr) { (void)cudaGraphDestroy(m->graph); m->graph = nullptr; }
    if (what == TFB_MLP_CAPTURE_STEP) {
        rc = check_connected(m, "mlp_capture_step");
        if (rc != TFB_OK) return rc;
        if (two_buckets(m)) {
            rc = bucket_streams(m);   // created before the capture begins
            if (rc != TFB_OK) return rc;
        }
    }
    TFB_CUDA_OK(cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal));
    rc = TFB_OK;
    if (what == TFB_MLP_CAPTURE_STEP) rc = forward_backward(m, X, labels, rows, global_rows, stream, true, lr, momentum);
    if (what == TFB_MLP_CAPTURE_FORWARD_BACKWARD) rc = forward_backward(m, X, labels, rows, global_rows, stream);
    if (rc == TFB_OK && what == TFB_MLP_CAPTURE_UPDATE) rc = launch_update(m, 1, lr, momentum, stream);
    cudaGraph_t g = nullptr;
    cudaError_t e = cudaStreamEndCapture(stream, &g);
    if (rc != TFB_OK) {
        if (g != nullptr) (void)cudaGraphDestroy(g);
        (void)cudaGetLastError();
        return rc;
    }
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        return fail(TFB_ERR_CUDA, "mlp_capture_step: ending the capture failed: %s", cudaGetErrorString(e));
    }
    m->graph = g;
    TFB_CUDA_OK(cudaGraphInstantiate(&m->graph_exec, g, 0));
    return TFB_OK;
}

int tfb_mlp_replay(tfb_mlp* m, void* stream) {
    int rc = check_handle(m, "mlp_replay");
    if (rc != TFB_OK) return rc;
    if (m->graph_exec == nullptr) return fail(TFB_ERR_INVALID_ARG, "mlp_replay: nothing has been captured");
    TFB_CUDA_OK(cudaGraphLaunch(m->graph_exec, static_cast<cudaStream_t>(stream)));
    return TFB_OK;
}

int tfb_mlp_set_option(tfb_mlp* m, int option, int64_t value) {
    if (m == nullptr) return fail(TFB_ERR_INVALID_ARG, "mlp_set_option: null handle");
    switch (option) {
    case TFB_MLP_OPT_WAIT_LIMIT_NS:
        if (value < 1000) return fail(TFB_ERR_INVALID_ARG, "mlp_set_option: wait limit below one microsecond");
        m->wait_ns = (unsigned long long)value;
        return TFB_OK;
    case TFB_MLP_OPT_EXCHANGE_CTAS:
        if (value < 0 || value > kMaxExchangeCtas)
            return fail(TFB_ERR_INVALID_ARG, "mlp_set_option: 0..%d exchange CTAs", kMaxExchangeCtas);
        m->exchange_ctas = (int)value;
        return TFB_OK;
    case TFB_MLP_OPT_KEEP_REDUCED_GRADS:
        m->keep_reduced = value != 0;
        return TFB_OK;
    case TFB_MLP_OPT_TRACE_EXCHANGE:
        m->trace_on = value != 0;
        return TFB_OK;
    case TFB_MLP_OPT_EXCHANGE_BUCKETS:
        if (value != 1 && value != 2) return fail(TFB_ERR_INVALID_ARG, "mlp_set_option: 1 or 2 exchange buckets");
        m->buckets = (int)value;
        return TFB_OK;
    default:
        return fail(TFB_ERR_INVALID_ARG, "mlp_set_option: unknown option %d", option);
    }
}

size_t tfb_mlp_ipc_handle_bytes(void) { return sizeof(cudaIpcMemHandle_t); }

int tfb_mlp_ipc_handle(tfb_mlp* m, void* handle_out) {
    int rc = check_handle(m, "mlp_ipc_handle");
    if (rc != TFB_OK) return rc;
    if (handle_out == nullptr) return fail(TFB_ERR_INVALID_ARG, "mlp_ipc_handle: null output");
    cudaIpcMemHandle_t h;
    TFB_CUDA_OK(cudaIpcGetMemHandle(&h, m->region));
    memcpy(handle_out, &h, sizeof(h));
    return TFB_OK;
}

static int set_group(tfb_mlp* m, int rank, int world, const char* who) {
    if (world < 1 || world > kMaxWorld || rank < 0 || rank >= world)
        return fail(TFB_ERR_INVALID_ARG, "%s: rank %d of %d (at most %d ranks)", who, rank, world, kMaxWorld);
    for (int r = 0; r < kMaxWorld; ++r) {
        if (m->ipc_mapped[r] && m->peer_region[r] != nullptr) (void)cudaIpcCloseMemHandle(m->peer_region[r]);
        m->ipc_mapped[r] = false;
        m->peer_region[r] = nullptr;
    }
    m->rank = rank;
    m->world = world;
    return TFB_OK;
}

int tfb_mlp_connect_ipc(tfb_mlp* m, int rank, int world, const void* handles) {
    int rc = check_handle(m, "mlp_connect_ipc");
    if (rc != TFB_OK) return rc;
    if (handles == nullptr) return fail(TFB_ERR_INVALID_ARG, "mlp_connect_ipc: null handle array");
    rc = set_group(m, rank, world, "mlp_connect_ipc");
    if (rc != TFB_OK) return rc;
    for (int r = 0; r < world; ++r) {
        if (r == rank) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, static_cast<const uint8_t*>(handles) + (size_t)r * sizeof(h), sizeof(h));
        void* p = nullptr;
        cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) {
            (void)cudaGetLastError();
            (void)set_group(m, 0, 1, "mlp_connect_ipc");
            return fail(TFB_ERR_CUDA, "mlp_connect_ipc: opening rank %d's region failed: %s", r, cudaGetErrorString(e));
        }
        m->peer_region[r] = static_cast<uint8_t*>(p);
        m->ipc_mapped[r] = true;
    }
    return TFB_OK;
}

int tfb_mlp_connect_ptrs(tfb_mlp* m, int rank, int world, void* const* regions) {
    int rc = check_handle(m, "mlp_connect_ptrs");
    if (rc != TFB_OK) return rc;
    if (regions == nullptr && world > 1) return fail(TFB_ERR_INVALID_ARG, "mlp_connect_ptrs: null region array");
    rc = set_group(m, rank, world, "mlp_connect_ptrs");
    if (rc != TFB_OK) return rc;
    for (int r = 0; r < world; ++r) {
        if (r == rank) continue;
        if (regions[r] == nullptr) {
            (void)set_group(m, 0, 1, "mlp_connect_ptrs");
            return fail(TFB_ERR_INVALID_ARG, "mlp_connect_ptrs: region of rank %d is null", r);
        }
        m->peer_region[r] = static_cast<uint8_t*>(regions[r]);
    }
    return TFB_OK;
}

int tfb_mlp_connect_local(tfb_mlp* const* ms, int world) {
    if (ms == nullptr || world < 1 || world > kMaxWorld)
        return fail(TFB_ERR_INVALID_ARG, "mlp_connect_local: 1..%d handles", kMaxWorld);
    for (int r = 0; r < world; ++r) {
        if (ms[r] == nullptr) return fail(TFB_ERR_INVALID_ARG, "mlp_connect_local: handle %d is null", r);
        if (ms[r]->numel != ms[0]->numel) return fail(TFB_ERR_INVALID_ARG, "mlp_connect_local: different layer sizes");
    }
    for (int r = 0; r < world; ++r) {
        DeviceScope scope;
        int rc = scope.enter(ms[r]->device);
        if (rc != TFB_OK) return rc;
        rc = set_group(ms[r], r, world, "mlp_connect_local");
        if (rc != TFB_OK) return rc;
        for (int q = 0; q < world; ++q) {
            if (q == r) continue;
            if (ms[q]->device != ms[r]->device) {
                int can = 0;
                TFB_CUDA_OK(cudaDeviceCanAccessPeer(&can, ms[r]->device, ms[q]->device));
                if (!can)
                    return fail(TFB_ERR_UNSUPPORTED, "mlp_connect_local: device %d cannot access device %d", ms[r]->device,
                                ms[q]->device);
                cudaError_t e = cudaDeviceEnablePeerAccess(ms[q]->device, 0);
                if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) {
                    (void)cudaGetLastError();
                    return fail(TFB_ERR_CUDA, "mlp_connect_local: enabling peer access %d -> %d: %s", ms[r]->device,
                                ms[q]->device, cudaGetErrorString(e));
                }
                (void)cudaGetLastError();
            }
            ms[r]->peer_region[q] = ms[q]->region;
        }
    }
    return TFB_OK;
}

int tfb_mlp_exchange_update_one_device(tfb_mlp* const* ms, int world, float lr, float momentum, void* stream_v) {
    if (ms == nullptr || world < 1 || world > kMaxWorld)
        return fail(TFB_ERR_INVALID_ARG, "mlp_exchange_update_one_device: 1..%d handles", kMaxWorld);
    int rc = check_handle(ms[0], "mlp_exchange_update_one_device");
    if (rc != TFB_OK) return rc;
    for (int r = 0; r < world; ++r) {
        if (ms[r] == nullptr || ms[r]->device != ms[0]->device || ms[r]->numel != ms[0]->numel ||
            ms[r]->world != world || ms[r]->rank != r)
            return fail(TFB_ERR_INVALID_ARG,
                        "mlp_exchange_update_one_device: handle %d is not rank %d of a %d-rank group on this device", r, r,
                        world);
    }
    DeviceState* st = nullptr;
    rc = device_state(&st);
    if (rc != TFB_OK) return rc;
    DpParams p;
    fill_params(ms[0], p, world, lr, momentum);
    for (int r = 0; r < world; ++r) fill_rank(ms[r], p.ranks[r], st->status);
    // All ranks run as one cooperative grid (blockIdx.y = rank) so that the CTAs that wait for each
    // other are resident together; separate launches on one GPU would have no such guarantee.
    int per_sm = 0;
    TFB_CUDA_OK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, dp_exchange_kernel, kExchangeThreads, 0));
    int grid = exchange_grid(ms[0], st->sm_count * (per_sm > 0 ? per_sm : 1), world, world);
    void* args[1] = {&p};
    TFB_CUDA_OK(cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(dp_exchange_kernel),
                                            dim3((unsigned)grid, (unsigned)world), dim3(kExchangeThreads), args, 0,
                                            static_cast<cudaStream_t>(stream_v)));
    return TFB_OK;
}

}  // extern "C"
