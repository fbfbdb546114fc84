/* TEST INFRASTRUCTURE — not part of the product, never on the product path.
 *
 * Plain-C restatement of the reference's CPU algorithms for the dense-contraction path.
 * Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline leg may load this file's
 * library (oracle/liboracle.so); libtfb.so neither links nor calls it.
 *
 * Parity pinned: tests/test_oracle_pins.py checks every function below against the
 * reference's own known-answer vectors and against outputs of the unmodified reference
 * (oracle/_ref/libtf_ref.so, and the fixtures under tests/golden/ generated from it).
 * Exceptions, stated where they occur: the bias gradient of Linear, the SGD update and the
 * bias gradient of Conv2d have no usable reference implementation ("parity unpinned").
 *
 * All arithmetic is FP32 with separate multiply and add in the reference's summation order
 * (build with -ffp-contract=off). Citations are file:line in the reference project.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <pthread.h>
#include <unistd.h>

/* ------------------------------------------------------------------------------------ */
/* Row-parallel helper (pthreads). Work is split into contiguous index ranges; every output
 * element is still produced by one thread in the reference's summation order, so results
 * do not depend on the thread count.                                                     */
typedef void (*orc_range_fn)(int64_t begin, int64_t end, void* ctx);
static int g_threads = 0;
void orc_set_threads(int n) { g_threads = n; }
int orc_get_threads(void) {
    if (g_threads > 0) return g_threads;
    long n = sysconf(_SC_NPROCESSORS_ONLN);
    return n > 0 ? (int)n : 1;
}
typedef struct { orc_range_fn fn; void* ctx; int64_t begin, end; } orc_job;
static void* orc_job_main(void* p) {
    orc_job* j = (orc_job*)p;
    j->fn(j->begin, j->end, j->ctx);
    return NULL;
}
static void orc_parallel_for(int64_t n, orc_range_fn fn, void* ctx) {
    int t = orc_get_threads();
    if (t > n) t = (int)(n > 0 ? n : 1);
    if (t <= 1) { fn(0, n, ctx); return; }
    pthread_t* th = (pthread_t*)malloc(sizeof(pthread_t) * (size_t)t);
    orc_job* jobs = (orc_job*)malloc(sizeof(orc_job) * (size_t)t);
    for (int i = 0; i < t; ++i) {
        jobs[i].fn = fn; jobs[i].ctx = ctx;
        jobs[i].begin = n * i / t; jobs[i].end = n * (i + 1) / t;
        if (pthread_create(&th[i], NULL, orc_job_main, &jobs[i]) != 0) {
            jobs[i].fn(jobs[i].begin, jobs[i].end, ctx);
            th[i] = 0;
        }
    }
    for (int i = 0; i < t; ++i) if (th[i]) pthread_join(th[i], NULL);
    free(th); free(jobs);
}

/* ------------------------------------------------------------------------------------ */
/* Tensor::matmul — tensor/Tensor.cpp:354-362: i, j, then k ascending into one FP32
 * accumulator; B walked with stride N.                                                  */
void orc_matmul_f32(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K) {
    for (int64_t i = 0; i < M; ++i) {
        for (int64_t j = 0; j < N; ++j) {
            float acc = 0.0f;
            for (int64_t k = 0; k < K; ++k) acc += A[i * K + k] * B[k * N + j];
            C[i * N + j] = acc;
        }
    }
}

/* Same per-element summation order, rows distributed over threads. B is transposed once
 * so that the inner loop is contiguous; the products and their order are unchanged.      */
typedef struct { const float *A, *Bt; float* C; int64_t N, K; } mm_ctx;
static void mm_rows(int64_t i0, int64_t i1, void* p) {
    mm_ctx* c = (mm_ctx*)p;
    for (int64_t i = i0; i < i1; ++i)
        for (int64_t j = 0; j < c->N; ++j) {
            float acc = 0.0f;
            const float* a = c->A + i * c->K;
            const float* b = c->Bt + j * c->K;
            for (int64_t k = 0; k < c->K; ++k) acc += a[k] * b[k];
            c->C[i * c->N + j] = acc;
        }
}
void orc_matmul_f32_mt(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K) {
    float* Bt = (float*)malloc((size_t)(N * K > 0 ? N * K : 1) * sizeof(float));
    for (int64_t k = 0; k < K; ++k)
        for (int64_t j = 0; j < N; ++j) Bt[j * K + k] = B[k * N + j];
    mm_ctx c = {A, Bt, C, N, K};
    orc_parallel_for(M, mm_rows, &c);
    free(Bt);
}

/* Selected rows of the product only (for sizes where the full loop takes hours):
 * out[r, :] = A[rows[r], :] · B.                                                         */
typedef struct { const float *A, *B; float* out; double* out64; const int64_t* sel; int64_t nsel, M, N, K; } sel_ctx;
static void sel_rows(int64_t r0, int64_t r1, void* p) {
    sel_ctx* c = (sel_ctx*)p;
    for (int64_t r = r0; r < r1; ++r) {
        const float* a = c->A + c->sel[r] * c->K;
        for (int64_t j = 0; j < c->N; ++j) {
            float acc = 0.0f;
            for (int64_t k = 0; k < c->K; ++k) acc += a[k] * c->B[k * c->N + j];
            c->out[r * c->N + j] = acc;
        }
    }
}
void orc_matmul_f32_rows(const float* A, const float* B, float* out, const int64_t* rows,
                         int64_t nrows, int64_t N, int64_t K) {
    sel_ctx c = {A, B, out, NULL, rows, nrows, 0, N, K};
    orc_parallel_for(nrows, sel_rows, &c);
}

/* Selected columns: out[:, c] = A · B[:, cols[c]], stored [M, ncols].                     */
static void sel_cols(int64_t i0, int64_t i1, void* p) {
    sel_ctx* c = (sel_ctx*)p;
    for (int64_t i = i0; i < i1; ++i)
        for (int64_t s = 0; s < c->nsel; ++s) {
            float acc = 0.0f;
            for (int64_t k = 0; k < c->K; ++k) acc += c->A[i * c->K + k] * c->B[k * c->N + c->sel[s]];
            c->out[i * c->nsel + s] = acc;
        }
}
void orc_matmul_f32_cols(const float* A, const float* B, float* out, const int64_t* cols,
                         int64_t ncols, int64_t M, int64_t N, int64_t K) {
    sel_ctx c = {A, B, out, NULL, cols, ncols, M, N, K};
    orc_parallel_for(M, sel_cols, &c);
}

/* FP64 product of the same inputs, used to attribute error budgets.                      */
static void f64_rows(int64_t i0, int64_t i1, void* p) {
    sel_ctx* c = (sel_ctx*)p;
    for (int64_t i = i0; i < i1; ++i)
        for (int64_t j = 0; j < c->N; ++j) {
            double acc = 0.0;
            for (int64_t k = 0; k < c->K; ++k) acc += (double)c->A[i * c->K + k] * (double)c->B[k * c->N + j];
            c->out64[i * c->N + j] = acc;
        }
}
void orc_matmul_f64(const float* A, const float* B, double* C, int64_t M, int64_t N, int64_t K) {
    sel_ctx c = {A, B, NULL, C, NULL, 0, M, N, K};
    orc_parallel_for(M, f64_rows, &c);
}

/* Tensor::transpose for the 2-D case — tensor/Tensor.cpp:579-619 (a full copy).           */
void orc_transpose_2d(const float* in, float* out, int64_t rows, int64_t cols) {
    for (int64_t r = 0; r < rows; ++r)
        for (int64_t c = 0; c < cols; ++c) out[c * rows + r] = in[r * cols + c];
}

/* Round-to-nearest-even FP32 -> BF16 -> FP32, the host-side rounding the BF16 configs use. */
float orc_round_bf16(float x) {
    uint32_t u;
    memcpy(&u, &x, 4);
    if ((u & 0x7f800000u) == 0x7f800000u) return x;
    u += 0x7fffu + ((u >> 16) & 1u);
    u &= 0xffff0000u;
    memcpy(&x, &u, 4);
    return x;
}
void orc_round_bf16_array(const float* in, float* out, int64_t n) {
    for (int64_t i = 0; i < n; ++i) out[i] = orc_round_bf16(in[i]);
}

/* ------------------------------------------------------------------------------------ */
/* Tensor::relu — tensor/Tensor.cpp:227-249; ReluBackward — autograd/ops/ReluBackward.hpp:22-32
 * (mask is 1 only where the forward input was > 0).                                      */
void orc_relu(const float* x, float* y, int64_t n) {
    for (int64_t i = 0; i < n; ++i) y[i] = x[i] > 0.0f ? x[i] : 0.0f;
}
void orc_relu_backward(const float* x, const float* gy, float* gx, int64_t n) {
    for (int64_t i = 0; i < n; ++i) gx[i] = gy[i] * (x[i] > 0.0f ? 1.0f : 0.0f);
}

/* nn::Linear::forward — nn/Linear.cpp:45-64: Wt = transpose(W) then x.matmul(Wt). The
 * reference registers a bias but never adds it; with a non-NULL bias this follows the
 * documented y = x·Wᵀ + b (nn/Linear.hpp:3), added after the accumulation like
 * Tensor::operator+ would. relu != 0 applies Tensor::relu to the result.                  */
void orc_linear_forward(const float* X, const float* W, const float* bias, float* Y, int64_t batch,
                        int64_t in_f, int64_t out_f, int relu) {
    float* Wt = (float*)malloc((size_t)(in_f * out_f) * sizeof(float));
    orc_transpose_2d(W, Wt, out_f, in_f);
    orc_matmul_f32_mt(X, Wt, Y, batch, out_f, in_f);
    free(Wt);
    for (int64_t i = 0; i < batch; ++i)
        for (int64_t j = 0; j < out_f; ++j) {
            float v = Y[i * out_f + j];
            if (bias) v = v + bias[j];
            if (relu) v = v > 0.0f ? v : 0.0f;
            Y[i * out_f + j] = v;
        }
}

/* Backward of y = relu?(x·Wᵀ + b) for upstream gradient dY, in the order the reference's
 * autograd executes it: ReluBackward (mask from the forward output, which is > 0 exactly
 * where the pre-activation was), MatmulBackward — autograd/ops/MatmulBackward.hpp:26-34 —
 * with b = Wt, then TransposeBackward — autograd/ops/TransposeBackward.hpp:26-28.
 *   dX  = dZ · (Wt)ᵀ           [batch, in]
 *   dWt = Xᵀ · dZ, dW = dWtᵀ   [out, in]
 *   db  = column sums of dZ, batch ascending — no reference implementation: parity unpinned.
 * Any output pointer may be NULL.                                                         */
void orc_linear_backward(const float* X, const float* W, const float* Y, const float* dY, float* dX,
                         float* dW, float* db, int64_t batch, int64_t in_f, int64_t out_f, int relu) {
    float* dZ = (float*)malloc((size_t)(batch * out_f) * sizeof(float));
    if (relu) orc_relu_backward(Y, dY, dZ, batch * out_f);
    else memcpy(dZ, dY, (size_t)(batch * out_f) * sizeof(float));
    if (dX) {
        /* (Wt)ᵀ is W itself as a [out, in] matrix. */
        orc_matmul_f32_mt(dZ, W, dX, batch, in_f, out_f);
    }
    if (dW) {
        float* Xt = (float*)malloc((size_t)(batch * in_f) * sizeof(float));
        float* dWt = (float*)malloc((size_t)(in_f * out_f) * sizeof(float));
        orc_transpose_2d(X, Xt, batch, in_f);
        orc_matmul_f32_mt(Xt, dZ, dWt, in_f, out_f, batch);
        orc_transpose_2d(dWt, dW, in_f, out_f);
        free(Xt);
        free(dWt);
    }
    if (db) {
        for (int64_t j = 0; j < out_f; ++j) {
            float s = 0.0f;
            for (int64_t i = 0; i < batch; ++i) s += dZ[i * out_f + j];
            db[j] = s;
        }
    }
    free(dZ);
}

/* ------------------------------------------------------------------------------------ */
/* im2col index map — cuda/kernels/im2col.cu:67-98. For flat column-matrix index
 * idx in [0, N*C*kH*kW*outH*outW) returns the flat NCHW input offset it reads, or -1 when
 * it falls in the padding.                                                               */
int64_t orc_conv_out_dim(int64_t in, int64_t k, int64_t stride, int64_t pad, int64_t dil) {
    return (in + 2 * pad - dil * (k - 1) - 1) / stride + 1; /* im2col.cu:109-110 */
}

int64_t orc_im2col_index(int64_t idx, int64_t C, int64_t H, int64_t W, int64_t kH, int64_t kW,
                         int64_t sh, int64_t sw, int64_t ph, int64_t pw, int64_t dh, int64_t dw,
                         int64_t outH, int64_t outW) {
    const int64_t total_per_n = C * kH * kW * outH * outW;
    const int64_t n = idx / total_per_n;
    const int64_t rem = idx - n * total_per_n;
    const int64_t spatial = outH * outW;
    const int64_t row = rem / spatial;
    const int64_t out_idx = rem - row * spatial;
    const int64_t c = row / (kH * kW);
    const int64_t rk = row - c * (kH * kW);
    const int64_t ki = rk / kW;
    const int64_t kj = rk - ki * kW;
    const int64_t oh = out_idx / outW;
    const int64_t ow = out_idx - oh * outW;
    const int64_t ih = oh * sh + ki * dh - ph;
    const int64_t iw = ow * sw + kj * dw - pw;
    if (ih >= 0 && ih < H && iw >= 0 && iw < W) return ((n * C + c) * H + ih) * W + iw;
    return -1;
}

typedef struct {
    const float* in; float* col; int64_t* idx_out; int64_t first;
    int64_t C, H, W, kH, kW, sh, sw, ph, pw, dh, dw, outH, outW;
} i2c_ctx;
static void i2c_idx(int64_t i0, int64_t i1, void* p) {
    i2c_ctx* c = (i2c_ctx*)p;
    for (int64_t i = i0; i < i1; ++i)
        c->idx_out[i] = orc_im2col_index(c->first + i, c->C, c->H, c->W, c->kH, c->kW, c->sh, c->sw,
                                         c->ph, c->pw, c->dh, c->dw, c->outH, c->outW);
}
void orc_im2col_index_range(int64_t first, int64_t count, int64_t* out, int64_t C, int64_t H,
                            int64_t W, int64_t kH, int64_t kW, int64_t sh, int64_t sw, int64_t ph,
                            int64_t pw, int64_t dh, int64_t dw, int64_t outH, int64_t outW) {
    i2c_ctx c = {NULL, NULL, out, first, C, H, W, kH, kW, sh, sw, ph, pw, dh, dw, outH, outW};
    orc_parallel_for(count, i2c_idx, &c);
}

/* launch_im2col — cuda/kernels/im2col.cu:58-99: col[idx] = in[index(idx)] or 0.            */
static void i2c_fill(int64_t i0, int64_t i1, void* p) {
    i2c_ctx* c = (i2c_ctx*)p;
    for (int64_t i = i0; i < i1; ++i) {
        const int64_t off = orc_im2col_index(i, c->C, c->H, c->W, c->kH, c->kW, c->sh, c->sw, c->ph,
                                             c->pw, c->dh, c->dw, c->outH, c->outW);
        c->col[i] = off >= 0 ? c->in[off] : 0.0f;
    }
}
void orc_im2col_f32(const float* in, float* col, int64_t N, int64_t C, int64_t H, int64_t W,
                    int64_t kH, int64_t kW, int64_t sh, int64_t sw, int64_t ph, int64_t pw,
                    int64_t dh, int64_t dw) {
    const int64_t outH = orc_conv_out_dim(H, kH, sh, ph, dh), outW = orc_conv_out_dim(W, kW, sw, pw, dw);
    i2c_ctx c = {in, col, NULL, 0, C, H, W, kH, kW, sh, sw, ph, pw, dh, dw, outH, outW};
    orc_parallel_for(N * C * kH * kW * outH * outW, i2c_fill, &c);
}

/* Direct convolution — nn/Conv2dModule.cpp:26-70 (cpu_conv2d): accumulation order
 * ci, kh, kw into one FP32 accumulator, bias added last.                                  */
typedef struct {
    const float *in, *weight, *bias; float* out;
    int64_t N, Cin, H, W, Cout, kH, kW, sh, sw, ph, pw, dh, dw, outH, outW;
} conv_ctx;
static void conv_planes(int64_t q0, int64_t q1, void* p) {
    conv_ctx* c = (conv_ctx*)p;
    for (int64_t q = q0; q < q1; ++q) {
        const int64_t n = q / c->Cout, co = q - n * c->Cout;
        for (int64_t oh = 0; oh < c->outH; ++oh)
            for (int64_t ow = 0; ow < c->outW; ++ow) {
                float acc = 0.0f;
                for (int64_t ci = 0; ci < c->Cin; ++ci)
                    for (int64_t kh = 0; kh < c->kH; ++kh)
                        for (int64_t kw = 0; kw < c->kW; ++kw) {
                            const int64_t ih = oh * c->sh - c->ph + kh * c->dh;
                            const int64_t iw = ow * c->sw - c->pw + kw * c->dw;
                            if (ih < 0 || ih >= c->H || iw < 0 || iw >= c->W) continue;
                            acc += c->in[((n * c->Cin + ci) * c->H + ih) * c->W + iw] *
                                   c->weight[((co * c->Cin + ci) * c->kH + kh) * c->kW + kw];
                        }
                if (c->bias) acc += c->bias[co];
                c->out[((n * c->Cout + co) * c->outH + oh) * c->outW + ow] = acc;
            }
    }
}
void orc_conv2d_forward(const float* in, const float* weight, const float* bias, float* out,
                        int64_t N, int64_t Cin, int64_t H, int64_t W, int64_t Cout, int64_t kH,
                        int64_t kW, int64_t sh, int64_t sw, int64_t ph, int64_t pw, int64_t dh,
                        int64_t dw) {
    const int64_t outH = orc_conv_out_dim(H, kH, sh, ph, dh), outW = orc_conv_out_dim(W, kW, sw, pw, dw);
    conv_ctx c = {in, weight, bias, out, N, Cin, H, W, Cout, kH, kW, sh, sw, ph, pw, dh, dw, outH, outW};
    orc_parallel_for(N * Cout, conv_planes, &c);
}

/* nn::Conv2d::forward — nn/Conv2d.cpp:77-138: im2col, one W2d[Cout,K]·col[n][K,P] product per
 * sample (k ascending over c, ki, kj), then launch_bias_add (cuda/kernels/bias_add.cu:49-58).
 * Same values as orc_conv2d_forward except that padding taps contribute explicit +0 terms.  */
void orc_conv2d_forward_im2col(const float* in, const float* weight, const float* bias, float* out,
                               int64_t N, int64_t Cin, int64_t H, int64_t W, int64_t Cout, int64_t kH,
                               int64_t kW, int64_t sh, int64_t sw, int64_t ph, int64_t pw, int64_t dh,
                               int64_t dw) {
    const int64_t outH = orc_conv_out_dim(H, kH, sh, ph, dh), outW = orc_conv_out_dim(W, kW, sw, pw, dw);
    const int64_t K = Cin * kH * kW, P = outH * outW;
    float* col = (float*)malloc((size_t)(N * K * P) * sizeof(float));
    orc_im2col_f32(in, col, N, Cin, H, W, kH, kW, sh, sw, ph, pw, dh, dw);
    for (int64_t n = 0; n < N; ++n) orc_matmul_f32_mt(weight, col + n * K * P, out + n * Cout * P, Cout, P, K);
    if (bias)
        for (int64_t i = 0; i < N * Cout * P; ++i) out[i] = out[i] + bias[(i / P) % Cout];
    free(col);
}

/* nn::Conv2d::backward — nn/Conv2d.cpp:140-260, with the host reference of
 * nn/conv2d_backward_test.cpp:50-106 for the summation it specifies:
 *   grad_input : col_grad[n] = Wᵀ[K,Cout] · dY[n][Cout,P] (co ascending), then col2im
 *                scatter-add (cuda/kernels/col2im.cu:50-80). The reference adds with
 *                atomics in no fixed order; here the column-matrix index ascends.
 *   grad_weight: per sample dY[n][Cout,P] · col[n]ᵀ[P,K] (p ascending), the per-sample
 *                results added on the host in sample order (Conv2d.cpp:215-243).
 *   grad_bias  : sum over n, h, w in that order. The reference's reduce kernel is wrong
 *                for H·W > 256 (cuda/kernels/reduce_sum_axis.cu:84,95-97): parity unpinned.
 * Any output pointer may be NULL.                                                         */
void orc_conv2d_backward(const float* in, const float* weight, const float* dY, float* grad_input,
                         float* grad_weight, float* grad_bias, int64_t N, int64_t Cin, int64_t H,
                         int64_t W, int64_t Cout, int64_t kH, int64_t kW, int64_t sh, int64_t sw,
                         int64_t ph, int64_t pw, int64_t dh, int64_t dw) {
    const int64_t outH = orc_conv_out_dim(H, kH, sh, ph, dh), outW = orc_conv_out_dim(W, kW, sw, pw, dw);
    const int64_t K = Cin * kH * kW, P = outH * outW;
    if (grad_input) {
        float* Wt = (float*)malloc((size_t)(K * Cout) * sizeof(float));
        float* cg = (float*)malloc((size_t)(K * P) * sizeof(float));
        orc_transpose_2d(weight, Wt, Cout, K);
        memset(grad_input, 0, (size_t)(N * Cin * H * W) * sizeof(float));
        for (int64_t n = 0; n < N; ++n) {
            orc_matmul_f32_mt(Wt, dY + n * Cout * P, cg, K, P, Cout);
            for (int64_t t = 0; t < K * P; ++t) {
                const int64_t off = orc_im2col_index(n * K * P + t, Cin, H, W, kH, kW, sh, sw, ph, pw,
                                                     dh, dw, outH, outW);
                if (off >= 0) grad_input[off] += cg[t];
            }
        }
        free(Wt);
        free(cg);
    }
    if (grad_weight) {
        float* col = (float*)malloc((size_t)(K * P) * sizeof(float));
        float* colT = (float*)malloc((size_t)(K * P) * sizeof(float));
        float* acc = (float*)malloc((size_t)(Cout * K) * sizeof(float));
        memset(grad_weight, 0, (size_t)(Cout * K) * sizeof(float));
        for (int64_t n = 0; n < N; ++n) {
            orc_im2col_f32(in + n * Cin * H * W, col, 1, Cin, H, W, kH, kW, sh, sw, ph, pw, dh, dw);
            orc_transpose_2d(col, colT, K, P);
            orc_matmul_f32_mt(dY + n * Cout * P, colT, acc, Cout, K, P);
            for (int64_t i = 0; i < Cout * K; ++i) grad_weight[i] += acc[i];
        }
        free(col);
        free(colT);
        free(acc);
    }
    if (grad_bias) {
        for (int64_t c = 0; c < Cout; ++c) {
            float s = 0.0f;
            for (int64_t n = 0; n < N; ++n)
                for (int64_t p = 0; p < P; ++p) s += dY[(n * Cout + c) * P + p];
            grad_bias[c] = s;
        }
    }
}

/* ------------------------------------------------------------------------------------ */
/* Tensor::log_softmax — tensor/Tensor.cpp:411-447 (row max, exp-sum, log, subtract).       */
void orc_log_softmax(const float* x, float* y, int64_t rows, int64_t cols) {
    for (int64_t r = 0; r < rows; ++r) {
        const float* row = x + r * cols;
        float maxv = row[0];
        for (int64_t j = 1; j < cols; ++j)
            if (row[j] > maxv) maxv = row[j];
        float sum_exp = 0.0f;
        for (int64_t j = 0; j < cols; ++j) sum_exp += expf(row[j] - maxv);
        const float log_z = logf(sum_exp) + maxv;
        for (int64_t j = 0; j < cols; ++j) y[r * cols + j] = row[j] - log_z;
    }
}

/* Mean negative log-likelihood of the training example — examples/train_mlp.cpp:54-76:
 * picked = lsm ⊙ onehot, row sums, sum over rows (ascending), times -1, times 1/N.
 * Returns the loss; if dz != NULL also writes the gradient with respect to the logits as
 * LogSoftmaxBackward (autograd/ops/LogSoftmaxBackward.hpp:26-58) produces it from the
 * upstream g = onehot · (-1 · 1/N):  dz = g − exp(lsm) · rowsum(g).                        */
float orc_nll_mean(const float* logits, const int64_t* labels, float* dz, int64_t rows, int64_t cols,
                   int64_t global_rows) {
    float* lsm = (float*)malloc((size_t)(rows * cols) * sizeof(float));
    orc_log_softmax(logits, lsm, rows, cols);
    const float n_inv = (float)(1.0 / (double)global_rows);
    float total = 0.0f;
    for (int64_t r = 0; r < rows; ++r) {
        float rs = 0.0f;
        for (int64_t j = 0; j < cols; ++j) rs += lsm[r * cols + j] * (labels[r] == j ? 1.0f : 0.0f);
        total += rs;
    }
    const float loss = (-1.0f * total) * n_inv;
    if (dz) {
        const float scale = -1.0f * n_inv;
        for (int64_t r = 0; r < rows; ++r) {
            float s = 0.0f;
            for (int64_t j = 0; j < cols; ++j) s += (labels[r] == j ? 1.0f : 0.0f) * scale;
            for (int64_t j = 0; j < cols; ++j) {
                const float g = (labels[r] == j ? 1.0f : 0.0f) * scale;
                dz[r * cols + j] = g - expf(lsm[r * cols + j]) * s;
            }
        }
    }
    free(lsm);
    return loss;
}

/* SGD with momentum as documented — nn/optim/SGD.hpp:3-6: v <- mu·v + g; p <- p − lr·v.
 * The shipped SGD::step throws for any parameter with more than one element and no
 * reference test covers it: parity unpinned.                                              */
void orc_sgd_momentum(float* p, float* v, const float* g, int64_t n, float lr, float mu) {
    for (int64_t i = 0; i < n; ++i) {
        v[i] = mu * v[i] + g[i];
        p[i] = p[i] - lr * v[i];
    }
}

/* Forward and backward of the three-layer MLP step (784→…→10 in the named configuration):
 * Linear, ReLU, Linear, ReLU, Linear, log_softmax + mean NLL over `global_rows` samples.
 * Biases are added when non-NULL. Gradients of all weights (and biases when dB* non-NULL)
 * are written; the first layer's input gradient is not needed and not computed.           */
float orc_mlp_grads(const float* X, const int64_t* labels, int64_t batch, int64_t global_rows,
                    int64_t d0, int64_t d1, int64_t d2, int64_t d3, const float* W1, const float* b1,
                    const float* W2, const float* b2, const float* W3, const float* b3, float* dW1,
                    float* db1, float* dW2, float* db2, float* dW3, float* db3) {
    float* h1 = (float*)malloc((size_t)(batch * d1) * sizeof(float));
    float* h2 = (float*)malloc((size_t)(batch * d2) * sizeof(float));
    float* z = (float*)malloc((size_t)(batch * d3) * sizeof(float));
    float* dz = (float*)malloc((size_t)(batch * d3) * sizeof(float));
    float* dh2 = (float*)malloc((size_t)(batch * d2) * sizeof(float));
    float* dh1 = (float*)malloc((size_t)(batch * d1) * sizeof(float));
    orc_linear_forward(X, W1, b1, h1, batch, d0, d1, 1);
    orc_linear_forward(h1, W2, b2, h2, batch, d1, d2, 1);
    orc_linear_forward(h2, W3, b3, z, batch, d2, d3, 0);
    const float loss = orc_nll_mean(z, labels, dz, batch, d3, global_rows);
    orc_linear_backward(h2, W3, z, dz, dh2, dW3, db3, batch, d2, d3, 0);
    orc_linear_backward(h1, W2, h2, dh2, dh1, dW2, db2, batch, d1, d2, 1);
    orc_linear_backward(X, W1, h1, dh1, NULL, dW1, db1, batch, d0, d1, 1);
    free(h1); free(h2); free(z); free(dz); free(dh2); free(dh1);
    return loss;
}
