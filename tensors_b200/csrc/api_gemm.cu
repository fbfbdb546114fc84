// extern "C" entry points of the GEMM family.
#include <initializer_list>

#include "internal.hpp"

using namespace tfb;

namespace {
bool known_dtype(int d) { return d == TFB_DTYPE_F32 || d == TFB_DTYPE_F16 || d == TFB_DTYPE_BF16; }
}  // namespace

extern "C" {

int tfb_gemm_ex(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K, int64_t lda,
                int64_t ldb, int64_t ldc, int trans_a, int trans_b, int in_dtype, int out_dtype,
                const float* bias, int epilogue_flags, void* stream) {
    if (M < 0 || N < 0 || K < 0) return fail(TFB_ERR_INVALID_ARG, "gemm_ex: negative extent");
    if (!known_dtype(in_dtype) || !known_dtype(out_dtype))
        return fail(TFB_ERR_UNSUPPORTED, "gemm_ex: unknown dtype (in %d, out %d)", in_dtype, out_dtype);
    if ((epilogue_flags & TFB_EPI_BIAS_COL) && (epilogue_flags & TFB_EPI_BIAS_ROW))
        return fail(TFB_ERR_INVALID_ARG, "gemm_ex: both bias modes requested");
    GemmCall c;
    c.A = A; c.B = B; c.C = C;
    c.M = M; c.N = N; c.K = K;
    c.lda = lda; c.ldb = ldb; c.ldc = ldc;
    c.a_kmajor = (trans_a == 0);
    c.b_kmajor = (trans_b != 0);
    c.in_dtype = in_dtype; c.out_dtype = out_dtype;
    c.bias = bias;
    c.bias_mode = (epilogue_flags & TFB_EPI_BIAS_COL) ? 1 : ((epilogue_flags & TFB_EPI_BIAS_ROW) ? 2 : 0);
    c.relu = (epilogue_flags & TFB_EPI_RELU) != 0;
    return gemm_run(c, static_cast<cudaStream_t>(stream));
}

int tfb_matmul(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K, int in_dtype,
               int out_dtype, void* stream) {
    return tfb_gemm_ex(A, B, C, M, N, K, K, N, N, 0, 0, in_dtype, out_dtype, nullptr, TFB_EPI_NONE, stream);
}

int tfb_matmul_batched(const void* A, const void* B, void* C, int64_t batch, int64_t M, int64_t N, int64_t K,
                       int64_t stride_a, int64_t stride_b, int64_t stride_c, int in_dtype, int out_dtype, void* stream) {
    if (batch < 0 || M < 0 || N < 0 || K < 0 || stride_a < 0 || stride_b < 0 || stride_c < 0)
        return fail(TFB_ERR_INVALID_ARG, "matmul_batched: negative extent or stride");
    if (!known_dtype(in_dtype) || !known_dtype(out_dtype))
        return fail(TFB_ERR_UNSUPPORTED, "matmul_batched: unknown dtype (in %d, out %d)", in_dtype, out_dtype);
    if (batch == 0 || M == 0 || N == 0) return TFB_OK;
    if (A == nullptr || B == nullptr || C == nullptr) return fail(TFB_ERR_INVALID_ARG, "matmul_batched: null pointer");
    if (batch > 1 && stride_c < M * N) return fail(TFB_ERR_INVALID_ARG, "matmul_batched: output matrices overlap");
    const size_t ei = dtype_size(in_dtype), eo = dtype_size(out_dtype);
    // A shared right-hand side under densely stacked left-hand sides is one tall product.
    if (stride_b == 0 && stride_a == M * K && stride_c == M * N)
        return tfb_matmul(A, B, C, batch * M, N, K, in_dtype, out_dtype, stream);
    for (int64_t b = 0; b < batch; ++b) {
        int rc = tfb_matmul(static_cast<const uint8_t*>(A) + (size_t)(b * stride_a) * ei,
                            static_cast<const uint8_t*>(B) + (size_t)(b * stride_b) * ei,
                            static_cast<uint8_t*>(C) + (size_t)(b * stride_c) * eo, M, N, K, in_dtype, out_dtype, stream);
        if (rc != TFB_OK) return rc;
    }
    return TFB_OK;
}

int tfb_gemm(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K, int dtype,
             void* stream) {
    // Mirrors the reference launchers: nothing happens for empty problems or unknown dtypes.
    if (M <= 0 || N <= 0 || K <= 0 || !known_dtype(dtype)) return TFB_OK;
    return tfb_matmul(A, B, C, M, N, K, dtype, dtype, stream);
}

int tfb_matmul_row_panels(int n_devices, const int* devices, const void* const* A_panels,
                          const void* const* B_replicas, void* const* C_panels, const int64_t* panel_rows,
                          int64_t N, int64_t K, int in_dtype, int out_dtype, void* const* streams) {
    if (n_devices < 0 || N < 0 || K < 0) return fail(TFB_ERR_INVALID_ARG, "matmul_row_panels: negative extent");
    if (n_devices == 0) return TFB_OK;
    if (devices == nullptr || A_panels == nullptr || B_replicas == nullptr || C_panels == nullptr ||
        panel_rows == nullptr)
        return fail(TFB_ERR_INVALID_ARG, "matmul_row_panels: null argument array");
    int visible = 0;
    TFB_CUDA_OK(cudaGetDeviceCount(&visible));
    for (int g = 0; g < n_devices; ++g) {
        if (devices[g] < 0 || devices[g] >= visible)
            return fail(TFB_ERR_INVALID_ARG, "matmul_row_panels: device %d is not one of the %d visible", devices[g],
                        visible);
        if (panel_rows[g] < 0) return fail(TFB_ERR_INVALID_ARG, "matmul_row_panels: negative panel height");
    }
    int before = 0;
    TFB_CUDA_OK(cudaGetDevice(&before));
    int rc = TFB_OK;
    // One enqueue per device, none of them waited for: the panels run concurrently.
    for (int g = 0; g < n_devices && rc == TFB_OK; ++g) {
        if (panel_rows[g] == 0) continue;
        cudaError_t e = cudaSetDevice(devices[g]);
        if (e != cudaSuccess) {
            rc = fail(TFB_ERR_CUDA, "matmul_row_panels: cudaSetDevice(%d): %s", devices[g], cudaGetErrorString(e));
            break;
        }
        rc = tfb_matmul(A_panels[g], B_replicas[g], C_panels[g], panel_rows[g], N, K, in_dtype, out_dtype,
                        streams != nullptr ? streams[g] : nullptr);
    }
    (void)cudaSetDevice(before);
    return rc;
}

int tfb_split_tf32(const float* src, int64_t rows, int64_t cols, int64_t ld, float* hi, float* lo,
                   int64_t ld_out, void* stream) {
    if (rows < 0 || cols < 0) return fail(TFB_ERR_INVALID_ARG, "split_tf32: negative extent");
    if (src == nullptr || hi == nullptr || lo == nullptr)
        return fail(TFB_ERR_INVALID_ARG, "split_tf32: null pointer");
    if (ld < cols || ld_out < cols || (ld_out & 3))
        return fail(TFB_ERR_INVALID_ARG, "split_tf32: ld_out must be a multiple of 4 and >= cols");
    if ((reinterpret_cast<uintptr_t>(hi) & 15u) || (reinterpret_cast<uintptr_t>(lo) & 15u))
        return fail(TFB_ERR_UNSUPPORTED, "split_tf32: output planes must be 16-byte aligned");
    return split_operand(src, rows, cols, ld, nullptr, hi, lo, ld_out, static_cast<cudaStream_t>(stream));
}

int tfb_gemm_presplit(const float* A_hi, const float* A_lo, const float* B_hi, const float* B_lo,
                      float* C, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb,
                      int64_t ldc, int trans_a, int trans_b, const float* bias, int epilogue_flags,
                      void* stream) {
    if (M < 0 || N < 0 || K < 0) return fail(TFB_ERR_INVALID_ARG, "gemm_presplit: negative extent");
    if (A_hi == nullptr || A_lo == nullptr || B_hi == nullptr || B_lo == nullptr)
        return fail(TFB_ERR_INVALID_ARG, "gemm_presplit: null operand plane");
    if ((lda & 3) || (ldb & 3))
        return fail(TFB_ERR_UNSUPPORTED, "gemm_presplit: leading dimensions must be multiples of 4");
    for (const float* p : {A_hi, A_lo, B_hi, B_lo})
        if (reinterpret_cast<uintptr_t>(p) & 15u)
            return fail(TFB_ERR_UNSUPPORTED, "gemm_presplit: planes must be 16-byte aligned");
    if ((epilogue_flags & TFB_EPI_BIAS_COL) && (epilogue_flags & TFB_EPI_BIAS_ROW))
        return fail(TFB_ERR_INVALID_ARG, "gemm_presplit: both bias modes requested");
    GemmCall c;
    c.A = A_hi; c.B = B_hi; c.C = C;
    c.M = M; c.N = N; c.K = K;
    c.lda = lda; c.ldb = ldb; c.ldc = ldc;
    c.a_kmajor = (trans_a == 0);
    c.b_kmajor = (trans_b != 0);
    c.in_dtype = TFB_DTYPE_F32; c.out_dtype = TFB_DTYPE_F32;
    c.a_presplit = true; c.b_presplit = true;
    c.a_lo_off = A_lo - A_hi; c.b_lo_off = B_lo - B_hi;
    c.bias = bias;
    c.bias_mode = (epilogue_flags & TFB_EPI_BIAS_COL) ? 1 : ((epilogue_flags & TFB_EPI_BIAS_ROW) ? 2 : 0);
    c.relu = (epilogue_flags & TFB_EPI_RELU) != 0;
    return gemm_run(c, static_cast<cudaStream_t>(stream));
}

int tfb_matmul_backward(const void* dC, const void* A, const void* B, void* dA, void* dB, int64_t M,
                        int64_t N, int64_t K, int dtype, void* stream) {
    if (M < 0 || N < 0 || K < 0) return fail(TFB_ERR_INVALID_ARG, "matmul_backward: negative extent");
    if (!known_dtype(dtype)) return fail(TFB_ERR_UNSUPPORTED, "matmul_backward: unknown dtype %d", dtype);
    if (dC == nullptr) return fail(TFB_ERR_INVALID_ARG, "matmul_backward: null upstream gradient");
    int rc = TFB_OK;
    if (dA != nullptr) {
        // dA[M,K] = dC[M,N] · Bᵀ : B is stored [K,N] = ["n"=K rows, contraction N contiguous].
        if (B == nullptr) return fail(TFB_ERR_INVALID_ARG, "matmul_backward: dA needs B");
        rc = tfb_gemm_ex(dC, B, dA, M, K, N, N, N, K, 0, 1, dtype, dtype, nullptr, TFB_EPI_NONE, stream);
        if (rc != TFB_OK) return rc;
    }
    if (dB != nullptr) {
        // dB[K,N] = Aᵀ · dC : A is stored [M,K] = [contraction M rows, "m"=K contiguous].
        if (A == nullptr) return fail(TFB_ERR_INVALID_ARG, "matmul_backward: dB needs A");
        rc = tfb_gemm_ex(A, dC, dB, K, N, M, K, N, N, 1, 0, dtype, dtype, nullptr, TFB_EPI_NONE, stream);
    }
    return rc;
}

}  // extern "C"
