// Declarations shared by the translation units of libtfb.so (not part of the C-ABI).
#pragma once

#include <cstddef>
#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>

#include "../../include/tfb.h"

namespace tfb {

// Records a message retrievable through tfb_last_error_string() and returns `code`.
int fail(int code, const char* fmt, ...);

#define TFB_CUDA_OK(expr)                                                                  \
    do {                                                                                   \
        cudaError_t e_ = (expr);                                                           \
        if (e_ != cudaSuccess) {                                                           \
            (void)cudaGetLastError(); /* reported here: a later call must not see it again */ \
            return ::tfb::fail(TFB_ERR_CUDA, "%s failed: %s (%s:%d)", #expr,               \
                               cudaGetErrorString(e_), __FILE__, __LINE__);                \
        }                                                                                  \
    } while (0)

// Per-device state created on first use with that device current.
struct DeviceState {
    int device = -1;
    int sm_count = 0;
    int* status = nullptr;   // device word: first error code a kernel recorded, 0 = none
};
int device_state(DeviceState** out);   // for the current device
// noalloc.cu keeps a second status word (a __device__ variable, so that its entry point never
// allocates); tfb_device_status consults both.
int static_status_take(int* code);
// Writes that word (host-side injection for tests of the reporting channel); fails if the
// allocation-free entry point has not been used on the current device yet.
int static_status_put(int code);

// Current value of a TFB_TUNE_* knob.
int tuning(int knob);

// Stream-ordered scratch owned by the library, one grow-only buffer per (device, stream).
int workspace_get(cudaStream_t stream, size_t bytes, void** out);
// Drops the buffer of (current device, stream), stream-ordered; called before the stream is destroyed.
void workspace_release(cudaStream_t stream);

// Launches `kernel` with the programmatic-serialization attribute (unless the PDL knob is off): the
// kernel may begin while its predecessor on the stream is still finishing, which hides launch latency
// and the kernel's own prologue in chains of short kernels. Every kernel launched through this MUST
// execute pdl_wait() (ptx.cuh) in every thread before its first access to global memory.
template <typename... KArgs, typename... Args>
int launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = tuning(TFB_TUNE_PDL) != 0 ? 1 : 0;
    TFB_CUDA_OK(cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...));
    return TFB_OK;
}

// Element size of a TFB_DTYPE_* code, 0 if unknown.
size_t dtype_size(int dtype);

// ---------------------------------------------------------------------------
// GEMM (gemm.cu)
// ---------------------------------------------------------------------------
struct GemmCall {
    const void* A = nullptr;   // op(A) is M x K
    const void* B = nullptr;   // op(B) is K x N
    void* C = nullptr;         // M x N row-major
    int64_t M = 0, N = 0, K = 0;
    int64_t lda = 0, ldb = 0, ldc = 0;   // elements
    // a_kmajor: A stored [M,K] row-major (contraction contiguous); else stored [K,M].
    // b_kmajor: B stored [N,K] row-major (contraction contiguous); else stored [K,N].
    bool a_kmajor = true, b_kmajor = false;
    int in_dtype = TFB_DTYPE_F32;
    int out_dtype = TFB_DTYPE_F32;
    const float* bias = nullptr;
    int bias_mode = 0;         // 0 none, 1 per output column, 2 per output row
    bool relu = false;
    // FP32 only: multiply A elementwise by (a_mask > 0) while splitting it (same shape and
    // leading dimension as A). Used to fold the ReLU backward mask into the operand.
    const float* a_mask = nullptr;
    // FP32 only: operands already split by gemm_split_operand (hi at ptr, lo at ptr + lo_off).
    bool a_presplit = false, b_presplit = false;
    int64_t a_lo_off = 0, b_lo_off = 0;   // elements
    // With *_presplit: the hi plane is the operand itself (the tensor core drops its low 13 mantissa bits)
    // and the lo plane is the residual against that truncation, as split_operand writes it for hi == nullptr.
    bool a_raw_hi = false, b_raw_hi = false;
    // FP32 output only, N a multiple of 4: also write the TF32 hi / lo planes of the result (after bias
    // and ReLU) with leading dimension N, for a product that consumes this output next. planes_lo alone:
    // that product reads C itself as its hi plane (raw-hi form, above) and only the residual is written.
    float* planes_hi = nullptr;
    float* planes_lo = nullptr;
    int force_bn = 0;          // 0 = choose; else 64 / 128 / 256
    int chunk_kb = 0;          // FP32: K blocks (of 32) per TMEM accumulation chunk; 0 = default
    void* workspace = nullptr; // optional caller scratch; nullptr = library-owned
    size_t workspace_bytes = 0;
};
int gemm_run(const GemmCall& call, cudaStream_t stream);
// small_gemm.cu: the CUDA-core kernel for FP32 products of at most a few tens of MFLOP (one launch, exact FP32).
bool small_gemm_eligible(const GemmCall& call);
int small_gemm_run(const GemmCall& call, cudaStream_t stream);
// True when gemm_run would split this call's contraction between CTAs (its epilogue then runs in the
// reduction kernel).
bool gemm_uses_split_k(const GemmCall& call, int sm_count);
// True when gemm_run would run this call with each tile's contraction shared by a cluster of two CTAs
// (one tile per cluster, so its epilogue is short and off the critical path of any other tile).
bool gemm_uses_cluster_k(const GemmCall& call, int sm_count);
// True when an FP32 operand at `ptr` with leading dimension `ld` (and no element mask) can be its own hi
// plane: 16-byte aligned, ld a multiple of 4, and the RAW_HI knob on.
bool raw_hi_operand(const void* ptr, int64_t ld, const void* mask);
// Same, with the device facts (SM count, status word) supplied by the caller instead of the
// lazily created per-device state.
int gemm_run_on(const GemmCall& call, cudaStream_t stream, const DeviceState* st);
// Scratch bytes gemm_run needs for this call on a device with sm_count SMs: split / re-packed
// operands plus split-K partial sums (0 for aligned 16-bit inputs with enough output tiles).
size_t gemm_workspace_bytes(const GemmCall& call, int sm_count);

// 2-D tensor map over a row-major matrix (`inner` contiguous elements per row, `outer` rows,
// rows row_stride_bytes apart) with a box of box_inner x box_outer elements and the 128-byte
// swizzle; atom32 selects the variant with 32-byte atoms that MN-major FP32 operands need.
int make_map(CUtensorMap* map, int dtype, const void* base, uint64_t inner, uint64_t outer,
             uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer, bool atom32 = false);

// FP32 tensor map of rank 2..5: dims[0] is the contiguous dimension, strides_bytes[i] is the stride of
// dims[i + 1] (multiples of 16), box the tile; 128-byte swizzle (with 32-byte atoms if atom32).
// elem_strides (optional): traversal stride per dimension — a box of extent b then delivers every
// stride-th element, ceil(b / stride) of them.
int make_map_nd(CUtensorMap* map, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                const uint32_t* box, bool atom32, const uint32_t* elem_strides = nullptr);

// Splits a row-major FP32 matrix (rows x cols, leading dimension ld) into TF32 hi / lo
// planes with leading dimension ld_out (multiple of 4, padding zero-filled).
// Two matrices in one launch (no masks).
int split_operands2(const float* src0, int64_t rows0, int64_t cols0, int64_t ld0, float* hi0, float* lo0, int64_t ld_out0,
                    const float* src1, int64_t rows1, int64_t cols1, int64_t ld1, float* hi1, float* lo1, int64_t ld_out1,
                    cudaStream_t stream);
int split_operand(const float* src, int64_t rows, int64_t cols, int64_t ld, const float* mask,
                  float* hi, float* lo, int64_t ld_out, cudaStream_t stream);

// ---------------------------------------------------------------------------
// nn::Linear (linear.cu)
// ---------------------------------------------------------------------------
int linear_forward(const void* X, const void* W, const float* bias, void* Y, int64_t batch, int64_t in_f,
                   int64_t out_f, bool relu, int dtype, cudaStream_t stream);
int linear_backward(const void* X, const void* W, const void* Y, const void* dY, void* dX, void* dW,
                    float* db, int64_t batch, int64_t in_f, int64_t out_f, bool relu, int dtype,
                    cudaStream_t stream);
// Planes of an FP32 operand that the caller split beforehand (null hi = not supplied).
struct SavedPlanes {
    const float* hi = nullptr;
    const float* lo = nullptr;
    int64_t ld = 0;
    bool raw_hi = false;   // hi is the operand itself, lo its residual against truncation (GemmCall::a_raw_hi)
};
// linear_backward with X and / or W optionally given as saved hi / lo planes (FP32 only; X and W are
// ignored for the operands whose planes are supplied).
// A bias gradient whose final addition the caller batches with others: linear_backward_impl writes the
// per-row-block partial column sums into `partial` (the caller's buffer, `capacity_floats` long; it must stay
// untouched until the finish) and fills in the rest; colsum_finish_many adds them in the usual fixed order.
struct DeferredColsum {
    float* partial = nullptr;
    size_t capacity_floats = 0;
    long long blocks = 0, cols = 0, ld = 0;
    float* out = nullptr;
};
constexpr int kMaxFinishJobs = 8;   // per launch; longer lists take several launches
// Floats of partial sums a deferred bias gradient of `batch` x `out_f` needs.
size_t deferred_colsum_floats(int64_t batch, int64_t out_f);
// One launch (per kMaxFinishJobs jobs) that finishes the bias gradients and, if row_loss != nullptr, the loss
// = -(1 / global_rows) * sum of row_loss[0, rows) — the same bits as the separate finish kernels give.
int colsum_finish_many(const DeferredColsum* jobs, int n, const float* row_loss, int64_t rows, int64_t global_rows,
                       float* loss_out, cudaStream_t stream);
int linear_backward_impl(const void* X, const void* W, const void* Y, const void* dY, void* dX, void* dW,
                         float* db, int64_t batch, int64_t in_f, int64_t out_f, bool relu, int dtype,
                         cudaStream_t stream, SavedPlanes xs, SavedPlanes wsaved, DeferredColsum* defer = nullptr);
// log_softmax + NLL with the per-row losses left in row_loss (rows floats) for a later finish.
int log_softmax_nll_rows(const float* logits, const int64_t* labels, float* dlogits, float* row_loss, int64_t rows,
                         int64_t cols, int64_t global_rows, cudaStream_t stream);

// ---------------------------------------------------------------------------
// nn::Conv2d (conv.cu: gather kernel, entry points; conv_tma.cu: TMA-fed path on the GEMM kernel)
// ---------------------------------------------------------------------------
struct ConvShape {
    int64_t N, Cin, H, W, Cout, kH, kW, sh, sw, ph, pw, dh, dw, outH, outW;
};
// True when a product of this convolution should run on the TMA-fed path: extents within tensor-map
// limits, enough channels in the contraction (forward and weight gradient: Cin; input gradient: Cout) to
// fill the 32-channel K blocks, and a stride the feed can express — any stride whose tile stays within a
// 256-element box for the forward product and the weight gradient (the tensor map traverses the source
// with the convolution's stride), stride 1 for the input gradient (`input_gradient`; its gather form reads
// rows (y + pad - ki * dilation) / stride, which is not a box).
bool conv_tma_eligible(const ConvShape& s, int64_t contraction_channels, bool input_gradient = false);
// True when the debugging override asks for the TMA-fed path wherever it is possible.
bool conv_tma_forced();
int conv_tma_forward(const float* x, const float* w, const float* bias, float* out, const ConvShape& s, bool relu,
                     cudaStream_t stream);
// dX, dW, db may each be null.
int conv_tma_backward(const float* x, const float* w, const float* dY, float* dX, float* dW, float* db,
                      const ConvShape& s, cudaStream_t stream);

// out[c] = sum over rows of partial[row * ld + c], c < cols, in an order fixed by (rows, cols) alone: two
// launches; `stage` is scratch of column_sums_stage_bytes(cols) bytes.
size_t column_sums_stage_bytes(int64_t cols);
int column_sums(const float* partial, int64_t rows, int64_t cols, int64_t ld, float* stage, float* out,
                cudaStream_t stream);

// conv_direct.cu: CUDA-core kernels for short contractions (any stride). Forward: Cin*kH*kW <= 128;
// input gradient: Cin <= 4; weight and bias gradient: Cin*kH*kW < 32.
bool conv_direct_forward_eligible(const ConvShape& s);
bool conv_direct_dgrad_eligible(const ConvShape& s);
int conv_direct_forward(const float* x, const float* w, const float* bias, float* out, const ConvShape& s, bool relu,
                        cudaStream_t stream);
int conv_direct_dgrad(const float* dY, const float* w, float* dX, const ConvShape& s, cudaStream_t stream);
// Weight and bias gradient (either may be null) for Cin*kH*kW + 1 <= 32.
bool conv_direct_wgrad_eligible(const ConvShape& s);
int conv_direct_wgrad(const float* x, const float* dY, float* dW, float* db, const ConvShape& s, cudaStream_t stream);

}  // namespace tfb
