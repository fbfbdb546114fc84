// nn::Linear forward and backward on the tcgen05 GEMM.
//
// forward : Y = relu?(X · Wᵀ + b)            one GEMM, bias and ReLU in its epilogue
// backward: dZ = dY ⊙ (Y > 0)                 folded into the operand-split pass of dZ,
//           db = column sums of dZ            which also emits the partial column sums
//           dX = dZ · W                       W consumed as an MN-major operand
//           dW = dZᵀ · X                      dZ and X consumed as MN-major operands
// No transpose copy is made anywhere: the split planes of dZ feed both backward GEMMs.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "finish.cuh"
#include "internal.hpp"
#include "ptx.cuh"

namespace tfb {

namespace {

// Rows one block of the mask / split pass walks (and sums for the bias gradient): 16 for large batches,
// fewer for small ones so that the grid still fills the GPU. A function of the shape alone, so the
// summation order of the bias gradient is fixed for a given problem.
constexpr int kColsumMaxRowsPerBlock = 16;
inline int colsum_rows_per_block(int64_t rows, int64_t ld_out) {
    // Fewer rows per block while the grid is short of ~64 K threads, but never more than 512 row blocks:
    // the finish kernel adds the blocks' partial sums sequentially (8 at a time).
    const int64_t vecs = rows * (ld_out / 4);
    int r = kColsumMaxRowsPerBlock;
    while (r > 1 && vecs / r < 65536 && rows / (r / 2) <= 512) r >>= 1;
    return r;
}

__device__ __forceinline__ float tf32_rna(float x) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return __uint_as_float(r);
}

// One block covers rows_per_block rows x (4 * blockDim.x) columns. Each thread owns four
// adjacent columns, walks the block's rows in ascending order, writes the masked value's hi / lo
// planes and keeps the running column sums, which land in partial[blockIdx.y][col].
__global__ void split_mask_colsum_kernel(const float* __restrict__ dY, const float* __restrict__ Y,
                                         long long rows, long long cols, long long ld,
                                         float* __restrict__ hi, float* __restrict__ lo, long long ld_out,
                                         float* __restrict__ partial, int rows_per_block) {
    pdl_wait();
    pdl_launch_dependents();
    const long long c = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (c >= ld_out) return;
    const long long r0 = (long long)blockIdx.y * rows_per_block;
    const long long r1 = min(r0 + (long long)rows_per_block, rows);
    const bool vec = ((ld & 3) == 0) && (c + 4 <= cols) && ((reinterpret_cast<uintptr_t>(dY) & 15u) == 0) &&
                     (Y == nullptr || (reinterpret_cast<uintptr_t>(Y) & 15u) == 0);
    float s[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
    for (long long r = r0; r < r1; ++r) {
        float x[4] = {0.f, 0.f, 0.f, 0.f};
        if (vec) {
            const float4 g = *reinterpret_cast<const float4*>(dY + r * ld + c);
            x[0] = g.x; x[1] = g.y; x[2] = g.z; x[3] = g.w;
            if (Y != nullptr) {
                const float4 y = *reinterpret_cast<const float4*>(Y + r * ld + c);
                x[0] = y.x > 0.f ? x[0] : 0.f;
                x[1] = y.y > 0.f ? x[1] : 0.f;
                x[2] = y.z > 0.f ? x[2] : 0.f;
                x[3] = y.w > 0.f ? x[3] : 0.f;
            }
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (c + j < cols) {
                    float v = dY[r * ld + c + j];
                    if (Y != nullptr) v = Y[r * ld + c + j] > 0.f ? v : 0.f;
                    x[j] = v;
                }
            }
        }
        float h[4], l[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            h[j] = tf32_rna(x[j]);
            l[j] = x[j] - h[j];
            s[j] += x[j];
        }
        *reinterpret_cast<float4*>(hi + r * ld_out + c) = make_float4(h[0], h[1], h[2], h[3]);
        *reinterpret_cast<float4*>(lo + r * ld_out + c) = make_float4(l[0], l[1], l[2], l[3]);
    }
    if (partial != nullptr)
        *reinterpret_cast<float4*>(partial + (long long)blockIdx.y * ld_out + c) = make_float4(s[0], s[1], s[2], s[3]);
}

// 16-bit variant: writes the masked gradient in the input type and the partial column sums.
template <typename T>
__global__ void mask_colsum16_kernel(const T* __restrict__ dY, const T* __restrict__ Y, long long rows,
                                     long long cols, long long ld, T* __restrict__ dZ, long long ld_out,
                                     float* __restrict__ partial, int rows_per_block) {
    pdl_wait();
    pdl_launch_dependents();
    const long long c = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= ld_out) return;
    const long long r0 = (long long)blockIdx.y * rows_per_block;
    const long long r1 = min(r0 + (long long)rows_per_block, rows);
    float s = 0.f;
    for (long long r = r0; r < r1; ++r) {
        float v = 0.f;
        if (c < cols) {
            v = static_cast<float>(dY[r * ld + c]);
            if (Y != nullptr) v = static_cast<float>(Y[r * ld + c]) > 0.f ? v : 0.f;
        }
        dZ[r * ld_out + c] = static_cast<T>(v);
        s += v;
    }
    if (partial != nullptr) partial[(long long)blockIdx.y * ld_out + c] = s;
}

// db[c] = sum over row blocks of partial[b][c], in the fixed order of colsum_finish_block.
__global__ void colsum_finish_kernel(const float* __restrict__ partial, long long blocks, long long cols,
                                     long long ld, float* __restrict__ out) {
    __shared__ float sm[kFinishGroups][33];
    pdl_wait();
    pdl_launch_dependents();
    colsum_finish_block(partial, blocks, cols, ld, out, blockIdx.x, sm);
}

// Several such reductions, and optionally a loss, in one launch: blockIdx.y selects the job (the loss is
// the job after the last bias gradient), blockIdx.x the column block.
struct FinishJobs {
    DeferredColsum job[kMaxFinishJobs];
    int n;
    const float* row_loss;   // null: no loss job
    long long rows;
    float n_inv;
    float* loss_out;
};
__global__ void finish_many_kernel(const FinishJobs J) {
    __shared__ float sm[kFinishGroups][33];
    pdl_wait();
    pdl_launch_dependents();
    const int j = (int)blockIdx.y;
    if (j < J.n) {
        const DeferredColsum& d = J.job[j];
        if ((long long)blockIdx.x * 32 >= d.cols) return;
        colsum_finish_block(d.partial, d.blocks, d.cols, d.ld, d.out, blockIdx.x, sm);
    } else if (blockIdx.x == 0) {
        loss_finish_block(J.row_loss, J.rows, J.n_inv, J.loss_out, (int)(threadIdx.y * 32 + threadIdx.x), &sm[0][0]);
    }
}

inline int64_t round_up(int64_t x, int64_t m) { return (x + m - 1) / m * m; }
inline size_t align256(size_t x) { return (x + 255) & ~(size_t)255; }

}  // namespace

int linear_forward(const void* X, const void* W, const float* bias, void* Y, int64_t batch, int64_t in_f,
                   int64_t out_f, bool relu, int dtype, cudaStream_t stream) {
    GemmCall c;
    c.A = X; c.B = W; c.C = Y;
    c.M = batch; c.N = out_f; c.K = in_f;
    c.lda = in_f; c.ldb = in_f; c.ldc = out_f;
    c.a_kmajor = true; c.b_kmajor = true;
    c.in_dtype = dtype; c.out_dtype = dtype;
    c.bias = bias; c.bias_mode = bias != nullptr ? 1 : 0;
    c.relu = relu;
    return gemm_run(c, stream);
}

size_t deferred_colsum_floats(int64_t batch, int64_t out_f) {
    if (batch <= 0 || out_f <= 0) return 0;
    const int64_t ldz = round_up(out_f, 4);
    // colsum_rows_per_block shrinks the row blocks only while there are at most 512 of them (513 with a
    // ragged last one); otherwise there is one per kColsumMaxRowsPerBlock rows. Any batch up to `batch` fits.
    const int64_t full = (batch + kColsumMaxRowsPerBlock - 1) / kColsumMaxRowsPerBlock;
    const int64_t most = full > 513 ? full : 513;
    return (size_t)(most * ldz);
}

int colsum_finish_many(const DeferredColsum* jobs, int n, const float* row_loss, int64_t rows, int64_t global_rows,
                       float* loss_out, cudaStream_t stream) {
    for (int first = 0; first < n || (first == 0 && row_loss != nullptr); first += kMaxFinishJobs) {
        FinishJobs J = {};
        J.n = n - first < kMaxFinishJobs ? n - first : kMaxFinishJobs;
        long long col_blocks = 1;
        for (int i = 0; i < J.n; ++i) {
            J.job[i] = jobs[first + i];
            const long long cb = (J.job[i].cols + 31) / 32;
            if (cb > col_blocks) col_blocks = cb;
        }
        const bool with_loss = first == 0 && row_loss != nullptr;
        if (with_loss) {
            J.row_loss = row_loss;
            J.rows = rows;
            J.n_inv = (float)(1.0 / (double)global_rows);
            J.loss_out = loss_out;
        }
        const int rc = launch_pdl(finish_many_kernel, dim3((unsigned)col_blocks, (unsigned)(J.n + (with_loss ? 1 : 0))),
                                  dim3(32, kFinishGroups), 0, stream, J);
        if (rc != TFB_OK) return rc;
    }
    return TFB_OK;
}

int linear_backward_impl(const void* X, const void* W, const void* Y, const void* dY, void* dX, void* dW,
                                float* db, int64_t batch, int64_t in_f, int64_t out_f, bool relu, int dtype,
                                cudaStream_t stream, SavedPlanes xs, SavedPlanes wsaved, DeferredColsum* defer) {
    DeviceState* st = nullptr;
    int rc = device_state(&st);
    if (rc != TFB_OK) return rc;
    if (batch <= 0 || in_f <= 0 || out_f <= 0) return TFB_OK;
    const bool f32 = dtype == TFB_DTYPE_F32;
    const int64_t ldz = round_up(out_f, f32 ? 4 : 8);
    const int rpb = colsum_rows_per_block(batch, ldz);
    const int64_t row_blocks = (batch + rpb - 1) / rpb;

    // The two products, described first so that their scratch needs are known.
    GemmCall gx, gw;
    gx.M = batch; gx.N = in_f; gx.K = out_f;        // dX = dZ[batch,out] · W[out,in]
    gx.B = W; gx.ldb = in_f; gx.b_kmajor = false;
    gx.C = dX; gx.ldc = in_f;
    gx.a_kmajor = true; gx.lda = ldz;
    gw.M = out_f; gw.N = in_f; gw.K = batch;        // dW = dZᵀ · X, both stored with the contraction outermost
    gw.B = X; gw.ldb = in_f; gw.b_kmajor = false;
    gw.C = dW; gw.ldc = in_f;
    gw.a_kmajor = false; gw.lda = ldz;
    gx.in_dtype = gw.in_dtype = dtype;
    gx.out_dtype = gw.out_dtype = dtype;
    gx.a_presplit = gw.a_presplit = f32;
    gx.a_lo_off = gw.a_lo_off = batch * ldz;
    // Placeholders so that the scratch computation sees aligned A operands.
    gx.A = gw.A = reinterpret_cast<const void*>(static_cast<uintptr_t>(256));
    if (wsaved.hi != nullptr) {
        gx.B = wsaved.hi; gx.ldb = wsaved.ld; gx.b_presplit = true; gx.b_lo_off = wsaved.lo - wsaved.hi;
        gx.b_raw_hi = wsaved.raw_hi;
    }
    if (xs.hi != nullptr) {
        gw.B = xs.hi; gw.ldb = xs.ld; gw.b_presplit = true; gw.b_lo_off = xs.lo - xs.hi;
        gw.b_raw_hi = xs.raw_hi;
    }

    const size_t dz_bytes = align256((size_t)(batch * ldz) * (f32 ? 8 : 2));
    const bool deferred = defer != nullptr && db != nullptr;
    if (deferred && (defer->partial == nullptr || defer->capacity_floats < (size_t)(row_blocks * ldz)))
        return fail(TFB_ERR_INVALID_ARG, "linear_backward: deferred bias-gradient buffer too small");
    const size_t partial_bytes = db != nullptr && !deferred ? align256((size_t)(row_blocks * ldz) * 4) : 0;
    const size_t gx_bytes = dX != nullptr ? gemm_workspace_bytes(gx, st->sm_count) : 0;
    const size_t gw_bytes = dW != nullptr ? gemm_workspace_bytes(gw, st->sm_count) : 0;
    const size_t gemm_bytes = align256(gx_bytes > gw_bytes ? gx_bytes : gw_bytes);
    void* ws_v = nullptr;
    rc = workspace_get(stream, dz_bytes + partial_bytes + gemm_bytes + 256, &ws_v);
    if (rc != TFB_OK) return rc;
    uint8_t* ws = static_cast<uint8_t*>(ws_v);
    void* dz = ws;
    float* partial = db == nullptr ? nullptr : (deferred ? defer->partial : reinterpret_cast<float*>(ws + dz_bytes));
    void* gemm_ws = ws + dz_bytes + partial_bytes;

    const void* mask = relu ? Y : nullptr;
    if (relu && Y == nullptr) return fail(TFB_ERR_INVALID_ARG, "linear_backward: ReLU needs the forward output");
    if (f32) {
        float* hi = static_cast<float*>(dz);
        float* lo = hi + batch * ldz;
        dim3 block(128), grid((unsigned)((ldz / 4 + 127) / 128), (unsigned)row_blocks);
        rc = launch_pdl(split_mask_colsum_kernel, grid, block, 0, stream, static_cast<const float*>(dY),
                        static_cast<const float*>(mask), (long long)batch, (long long)out_f, (long long)out_f, hi, lo,
                        (long long)ldz, partial, rpb);
        if (rc != TFB_OK) return rc;
    } else {
        dim3 block(128), grid((unsigned)((ldz + 127) / 128), (unsigned)row_blocks);
        if (dtype == TFB_DTYPE_BF16)
            rc = launch_pdl(mask_colsum16_kernel<__nv_bfloat16>, grid, block, 0, stream,
                            static_cast<const __nv_bfloat16*>(dY), static_cast<const __nv_bfloat16*>(mask), (long long)batch,
                            (long long)out_f, (long long)out_f, static_cast<__nv_bfloat16*>(dz), (long long)ldz, partial,
                            rpb);
        else
            rc = launch_pdl(mask_colsum16_kernel<__half>, grid, block, 0, stream, static_cast<const __half*>(dY),
                            static_cast<const __half*>(mask), (long long)batch, (long long)out_f, (long long)out_f,
                            static_cast<__half*>(dz), (long long)ldz, partial, rpb);
        if (rc != TFB_OK) return rc;
    }
    if (deferred) {
        // the caller adds the partial sums later, batched with others (colsum_finish_many)
        defer->blocks = row_blocks; defer->cols = out_f; defer->ld = ldz; defer->out = db;
    } else if (db != nullptr) {
        rc = launch_pdl(colsum_finish_kernel, dim3((unsigned)((out_f + 31) / 32)), dim3(32, kFinishGroups), 0, stream,
                        (const float*)partial, (long long)row_blocks, (long long)out_f, (long long)ldz, db);
        if (rc != TFB_OK) return rc;
    }
    gx.A = gw.A = dz;
    gx.workspace = gw.workspace = gemm_ws;
    gx.workspace_bytes = gw.workspace_bytes = gemm_bytes;
    if (dX != nullptr) {
        rc = gemm_run(gx, stream);
        if (rc != TFB_OK) return rc;
    }
    if (dW != nullptr) {
        rc = gemm_run(gw, stream);
        if (rc != TFB_OK) return rc;
    }
    return TFB_OK;
}

int linear_backward(const void* X, const void* W, const void* Y, const void* dY, void* dX, void* dW,
                    float* db, int64_t batch, int64_t in_f, int64_t out_f, bool relu, int dtype,
                    cudaStream_t stream) {
    return linear_backward_impl(X, W, Y, dY, dX, dW, db, batch, in_f, out_f, relu, dtype, stream, SavedPlanes(),
                                SavedPlanes(), nullptr);
}

}  // namespace tfb

extern "C" {

int tfb_linear_forward(const void* X, const void* W, const float* bias, void* Y, int64_t batch,
                       int64_t in_features, int64_t out_features, int relu, int dtype, void* stream) {
    using namespace tfb;
    if (batch < 0 || in_features < 0 || out_features < 0)
        return fail(TFB_ERR_INVALID_ARG, "linear_forward: negative extent");
    if (dtype_size(dtype) == 0) return fail(TFB_ERR_UNSUPPORTED, "linear_forward: unknown dtype %d", dtype);
    if (X == nullptr || W == nullptr || Y == nullptr) return fail(TFB_ERR_INVALID_ARG, "linear_forward: null pointer");
    return linear_forward(X, W, bias, Y, batch, in_features, out_features, relu != 0, dtype,
                          static_cast<cudaStream_t>(stream));
}

int tfb_linear_backward(const void* X, const void* W, const void* Y, const void* dY, void* dX, void* dW,
                        float* dbias, int64_t batch, int64_t in_features, int64_t out_features, int relu,
                        int dtype, void* stream) {
    using namespace tfb;
    if (batch < 0 || in_features < 0 || out_features < 0)
        return fail(TFB_ERR_INVALID_ARG, "linear_backward: negative extent");
    if (dtype_size(dtype) == 0) return fail(TFB_ERR_UNSUPPORTED, "linear_backward: unknown dtype %d", dtype);
    if (dY == nullptr) return fail(TFB_ERR_INVALID_ARG, "linear_backward: null upstream gradient");
    if (dX != nullptr && W == nullptr) return fail(TFB_ERR_INVALID_ARG, "linear_backward: dX needs W");
    if (dW != nullptr && X == nullptr) return fail(TFB_ERR_INVALID_ARG, "linear_backward: dW needs X");
    return linear_backward(X, W, Y, dY, dX, dW, dbias, batch, in_features, out_features, relu != 0, dtype,
                           static_cast<cudaStream_t>(stream));
}

int tfb_linear_backward_presplit(const float* X_hi, const float* X_lo, int64_t ldx, const float* W_hi,
                                 const float* W_lo, int64_t ldw, const float* Y, const float* dY, float* dX,
                                 float* dW, float* dbias, int64_t batch, int64_t in_features,
                                 int64_t out_features, int relu, void* stream) {
    using namespace tfb;
    if (batch < 0 || in_features < 0 || out_features < 0)
        return fail(TFB_ERR_INVALID_ARG, "linear_backward_presplit: negative extent");
    if (dY == nullptr) return fail(TFB_ERR_INVALID_ARG, "linear_backward_presplit: null upstream gradient");
    if (dX != nullptr && (W_hi == nullptr || W_lo == nullptr))
        return fail(TFB_ERR_INVALID_ARG, "linear_backward_presplit: dX needs the planes of W");
    if (dW != nullptr && (X_hi == nullptr || X_lo == nullptr))
        return fail(TFB_ERR_INVALID_ARG, "linear_backward_presplit: dW needs the planes of X");
    SavedPlanes xs, wsaved;
    if (dW != nullptr) { xs.hi = X_hi; xs.lo = X_lo; xs.ld = ldx; }
    if (dX != nullptr) { wsaved.hi = W_hi; wsaved.lo = W_lo; wsaved.ld = ldw; }
    for (const SavedPlanes& pl : {xs, wsaved}) {
        if (pl.hi == nullptr) continue;
        if ((pl.ld & 3) || pl.ld < in_features)
            return fail(TFB_ERR_UNSUPPORTED,
                        "linear_backward_presplit: plane leading dimensions must be multiples of 4 and >= in_features");
        if ((reinterpret_cast<uintptr_t>(pl.hi) | reinterpret_cast<uintptr_t>(pl.lo)) & 15u)
            return fail(TFB_ERR_UNSUPPORTED, "linear_backward_presplit: planes must be 16-byte aligned");
    }
    return linear_backward_impl(nullptr, nullptr, Y, dY, dX, dW, dbias, batch, in_features, out_features,
                                relu != 0, TFB_DTYPE_F32, static_cast<cudaStream_t>(stream), xs, wsaved);
}

}  // extern "C"
