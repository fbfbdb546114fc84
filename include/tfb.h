/* libtfb — C-ABI of the B200-native dense-contraction path for tensorforge.
 *
 * Everything a host runtime needs to route Tensor::matmul, nn::Linear, nn::Conv2d and
 * MatmulBackward through hand-written sm_100a kernels. Plain pointers and sizes only;
 * device pointers refer to the CUDA device that is current on the calling thread.
 * `stream` is a cudaStream_t passed as void* (NULL = legacy default stream), as in the
 * reference launchers, so callers compiled without CUDA headers can use this file.
 *
 * All functions return 0 on success or a negative TFB_ERR_* code; they never throw and
 * never fall back to a CPU or library implementation. Work is enqueued on `stream` and
 * is asynchronous with respect to the host unless stated otherwise.
 *
 * Citations "ref:" name the file:line of the reference interface each entry point
 * replaces (paths relative to the reference project root).
 */
#ifndef TFB_H_
#define TFB_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Same numbering as the reference's `enum class Dtype` (ref: tensor/Dtype.hpp:9-16). */
#define TFB_DTYPE_F32 0
#define TFB_DTYPE_F16 1
#define TFB_DTYPE_BF16 2

#define TFB_OK 0
#define TFB_ERR_INVALID_ARG (-1)   /* null pointer, negative size, bad flag */
#define TFB_ERR_UNSUPPORTED (-2)   /* dtype / layout / alignment the kernels do not take */
#define TFB_ERR_CUDA (-3)          /* a CUDA runtime or driver call failed */
#define TFB_ERR_DEVICE (-4)        /* a kernel recorded an error (see tfb_device_status) */
#define TFB_ERR_NO_MEMORY (-5)
#define TFB_ERR_TOO_LARGE (-6)     /* exceeds a stated fixed limit */

/* Epilogue flags for tfb_gemm_ex. */
#define TFB_EPI_NONE 0
#define TFB_EPI_BIAS_COL 1   /* C[m,n] += bias[n]  (Linear) */
#define TFB_EPI_BIAS_ROW 2   /* C[m,n] += bias[m]  (Conv2d output channel) */
#define TFB_EPI_RELU 4       /* C = max(C, 0) after the bias */

/* ---- library -------------------------------------------------------------------- */

/* Idempotent set-up for the current device (resolves the driver's tensor-map encoder,
 * allocates the device status word, raises the kernels' shared-memory limit). Called
 * implicitly by every other entry point. ref: the static registrars of
 * cuda/kernels/elementwise.cu:306-336 plus the explicit init_tensor_autograd() pattern
 * of tensor/AutogradWirer.hpp:72-76. */
int tfb_init(void);

/* Message of the last failure on the calling thread ("" if none). */
const char* tfb_last_error_string(void);

/* Tuning knobs. Each starts at its default, or at the value of the environment variable of the same
 * purpose (TFB_GEMM_BN, TFB_GEMM_PAIR, TFB_GEMM_SPLITK, TFB_GEMM_CHUNK_KB, TFB_CONV_TMA,
 * TFB_CONV_DIRECT, TFB_CONV_PAIR, TFB_HOST_PANEL) read ONCE when the first knob is consulted; no call
 * path reads the environment. They exist for tests (every kernel must see every shape) and for
 * measurements; results do not depend on them beyond FP32 summation order.
 *   GEMM_TILE_N     0 = choose, else 64 / 128 / 256 columns per single-CTA tile
 *   GEMM_PAIR       -1 = choose, 0 = never pair CTAs, 1 = always
 *   GEMM_SPLIT_K    0 = choose, else the number of K splits
 *   GEMM_CHUNK_KB   0 = default (8), else K blocks per TMEM accumulation chunk of the FP32 path
 *   CONV_TMA        0 = never use the TMA-fed convolution path, 1 = choose, 2 = wherever possible
 *   CONV_DIRECT     0 = never use the CUDA-core kernels for short contractions, 1 = choose
 *   CONV_PAIR       -1 = choose, 0 / 1 = CTA pairs off / on in the TMA-fed convolution path
 *   HOST_PANEL_ROWS rows of A per panel in tfb_matmul_host (default 512)
 *   PDL             1 (default) = kernels are launched so that each may start its prologue while the one
 *                   before it on the stream is finishing (programmatic dependent launch); 0 = plain
 *                   stream order (environment: TFB_PDL)
 *   GEMM_GROUP_M    0 = default, else the number of M tiles per rasterisation group of the GEMM kernel (tiles
 *                   of one group are visited M-fastest, so a wave of CTAs shares that many A panels)
 *   SMALL_GEMM      1 (default) = FP32 products with at most 128 rows (or, run transposed, at most 128 columns),
 *                   at most 16384 outputs and a contraction of 512..2048 run on the one-launch CUDA-core
 *                   kernel (exact FP32 FMAs, K split over a thread-block cluster), 0 = everything on the
 *                   tensor-core path
 *   RAW_HI          1 = a 16-byte aligned FP32 operand whose leading dimension is a multiple of 4 is read by
 *                   the tensor core as its own hi plane (kind::tf32 drops the low 13 mantissa bits) and
 *                   the split pass writes only the lo plane = the residual against that truncation, which
 *                   halves the scratch and a third of the split traffic; 0 (default) = always write
 *                   round-to-nearest hi and lo planes. Off by default because it was measured slower
 *                   where it should matter most: an 8192-cubed product at the power cap runs at ~5 % lower
 *                   clocks when the operand paths carry the 13 mantissa bits that rounded planes hold as
 *                   zeros (216 against 223-230 TFLOP/s on one GPU, alternating runs)
 *   CLUSTER_K       1 (default) = an FP32 product that would run as two K splits of 128 x 128 tiles with at
 *                   most one tile per SM pair runs each tile on a cluster of two CTAs, which add their
 *                   halves through distributed shared memory (no partial sums in scratch, no reduction
 *                   kernel; same bits as the two-kernel form); 0 = partial sums + reduction kernel
 *   FUSE_PLANES     which products of the MLP step also write the TF32 hi / lo planes of their result for
 *                   the next layer instead of leaving that to a separate pass: 0 = none, 1 (default) =
 *                   the split-K products (their reduction kernel writes the planes), 2 = all of them
 *                   (the GEMM epilogue writes the planes too) (environment: TFB_FUSE_PLANES)
 * ref: no counterpart (the reference has one kernel per operation). */
#define TFB_TUNE_GEMM_TILE_N 0
#define TFB_TUNE_GEMM_PAIR 1
#define TFB_TUNE_GEMM_SPLIT_K 2
#define TFB_TUNE_GEMM_CHUNK_KB 3
#define TFB_TUNE_CONV_TMA 4
#define TFB_TUNE_CONV_DIRECT 5
#define TFB_TUNE_CONV_PAIR 6
#define TFB_TUNE_HOST_PANEL_ROWS 7
#define TFB_TUNE_PDL 8
#define TFB_TUNE_FUSE_PLANES 9
#define TFB_TUNE_GEMM_GROUP_M 10
#define TFB_TUNE_SMALL_GEMM 11
#define TFB_TUNE_RAW_HI 12
#define TFB_TUNE_CLUSTER_K 13
#define TFB_TUNE_COUNT 14
int tfb_set_tuning(int knob, int value);
int tfb_get_tuning(int knob, int* value_out);

/* Synchronises the current device and reports the first error code a kernel recorded
 * (0 = none; 101..107 = a bounded wait inside a kernel ran out), then clears it. The
 * reference never checks launches (ref: cuda/kernels/gemm.cu:82-87 has no
 * cudaGetLastError); this is the replacement's fail-soft channel. */
int tfb_device_status(int* code_out);
/* Host-side fault injection for tests of a host's error handling: writes `code` into a status word as
 * a kernel that gave up would have (word 0: the regular one; word 1: the one of tfb_matmul_f32_static,
 * which must have run on this device before). No kernel is made to fail. ref: no counterpart. */
int tfb_inject_device_status(int word, int code);

/* ---- GEMM ------------------------------------------------------------------------ */

/* C[M,N] = A[M,K] · B[K,N], all row-major and dense, C of the same dtype as A and B,
 * FP32 accumulation. FP32 inputs run as an error-compensated 3xTF32 product. Like the
 * reference launchers it is a silent no-op for M, N or K <= 0 and for unknown dtypes.
 * ref: launch_gemm_naive / launch_gemm_tiled_16x16 / launch_gemm_optimized,
 * cuda/kernels/gemm.cuh:33-53, cuda/kernels/gemm.cu:275-357. */
int tfb_gemm(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K, int dtype,
             void* stream);

/* The CUDA branch of Tensor::matmul: same contraction, separate input and output dtypes
 * (F32 -> F32; F16/BF16 -> F32 or the input dtype). Unlike tfb_gemm it reports bad
 * arguments. ref: Tensor::matmul, tensor/Tensor.cpp:334-368; the registry slot it fills
 * sits beside register_cuda_add in cuda/CudaKernelRegistry.hpp:15-26. The slot's function type carries
 * TWO dtypes (in, out) where the reference's launchers carry one: Tensor::matmul passes its own dtype
 * for both (the reference's rule), a caller that wants 16-bit operands with an FP32 result passes F32 as
 * the second. */
int tfb_matmul(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K,
               int in_dtype, int out_dtype, void* stream);

/* Batched product over the leading dimensions of N-D operands: C[b] = A[b] · B[b] for b < batch, every
 * matrix row-major and dense; stride_* are the distances in elements between consecutive matrices
 * (0 = the same matrix for every b). A shared B under densely stacked A and C (stride_b == 0,
 * stride_a == M·K, stride_c == M·N) runs as ONE product of batch·M rows; every other case enqueues one
 * product per matrix on `stream`. ref: no counterpart — Tensor::matmul refuses anything but two 2-D
 * operands (tensor/Tensor.cpp:335-338); this is the N-D extension of the same contraction. */
int tfb_matmul_batched(const void* A, const void* B, void* C, int64_t batch, int64_t M, int64_t N, int64_t K,
                       int64_t stride_a, int64_t stride_b, int64_t stride_c, int in_dtype, int out_dtype,
                       void* stream);

/* Diagnostics: while `device_stamps` (7 uint64 in device memory) is set, CTA 0 of every GEMM launch of the
 * library records nanosecond timestamps at its phase boundaries into it — entry, prologue done, first
 * operand stage landed, last MMA committed, accumulator seen by the epilogue, epilogue drained, exit —
 * so that the fixed latency of small products can be read off directly. NULL turns it off (the default).
 * ref: no counterpart. */
int tfb_gemm_trace(void* device_stamps);
/* Host function (no device needed): which plan tfb_gemm_ex would choose for an M x N x K product of `dtype`
 * operands (both operands aligned, neither pre-split) on a device with `sm_count` SMs, under the current tuning
 * knobs. plan_out receives 5 ints: tile columns (64 / 128 / 256), CTA pairs (0 / 1), K splits (1 = none),
 * cluster split-K (0 / 1), CUDA-core small-product kernel (0 / 1; the other four are then 0). For tests that pin
 * the dispatch and for hosts that want to know what a shape will cost. ref: no counterpart. */
int tfb_gemm_describe_plan(int64_t M, int64_t N, int64_t K, int dtype, int sm_count, int* plan_out);

/* General form. op(A) is M x K, op(B) is K x N:
 *   trans_a = 0: A stored [M,K] row-major (lda >= K); 1: A stored [K,M] row-major (lda >= M)
 *   trans_b = 0: B stored [K,N] row-major (ldb >= N); 1: B stored [N,K] row-major (ldb >= K)
 * C is [M,N] row-major (ldc >= N). `bias` is FP32 and is read only when an
 * TFB_EPI_BIAS_* flag is set. Transposed operands are consumed in place through the
 * matching shared-memory descriptor; no transpose copy is made.
 * ref: replaces launch_transpose_2d + launch_gemm_* pairs (cuda/kernels/transpose.cu:29-37,
 * nn/Conv2d.cpp:182-198) and launch_bias_add (cuda/kernels/bias_add.cu:49-58). */
int tfb_gemm_ex(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K,
                int64_t lda, int64_t ldb, int64_t ldc, int trans_a, int trans_b, int in_dtype,
                int out_dtype, const float* bias, int epilogue_flags, void* stream);

/* FP32 operands can be split once and reused by several products (a weight matrix feeds the
 * forward product and the input-gradient product of the same step).
 * tfb_split_tf32: hi = src rounded to TF32, lo = src - hi, both written row-major with leading
 * dimension ld_out (a multiple of 4, >= cols; padding columns are zero-filled). `src` is
 * rows x cols with leading dimension ld.
 * tfb_gemm_presplit: tfb_gemm_ex for FP32 operands given as such hi / lo planes (leading
 * dimensions multiples of 4, 16-byte aligned bases); C is FP32. Products with few output tiles and a long
 * contraction run split along K and then take library-owned scratch for the partial sums; inside a stream
 * capture that scratch must already exist (run the same call once outside the capture first).
 * ref: no counterpart; the reference has no tensor-core path (cuda/kernels/gemm.cu:60-254). */
int tfb_split_tf32(const float* src, int64_t rows, int64_t cols, int64_t ld, float* hi, float* lo,
                   int64_t ld_out, void* stream);
int tfb_gemm_presplit(const float* A_hi, const float* A_lo, const float* B_hi, const float* B_lo,
                      float* C, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb,
                      int64_t ldc, int trans_a, int trans_b, const float* bias, int epilogue_flags,
                      void* stream);

/* C = A · B with all three matrices in HOST memory (row-major, dense; C is FP32): the call uploads B,
 * streams A through in row panels and downloads C panel by panel, overlapping host-to-device copies,
 * the products and device-to-host copies on three streams. Completion is ordered on `stream`
 * (synchronise it before reading C). Use pinned host memory for the copies to overlap; pageable
 * memory works but serialises them. Device buffers come from the stream-ordered pool and are
 * released by the call. ref: the CPU-tensor use of Tensor::matmul (tensor/Tensor.cpp:334-368) plus
 * the Tensor::to(Device) round trip a CUDA caller would add (tensor/Tensor.hpp:78-84). */
int tfb_matmul_host(const void* A_host, const void* B_host, void* C_host, int64_t M, int64_t N, int64_t K,
                    int dtype, void* stream);
/* The same with B already in DEVICE memory (ordered before the call on `stream`): several GPUs that
 * share one B each upload a slice of it, exchange the slices over NVLink (an all-gather) and then
 * stream their own rows of A, so that B crosses the host link once instead of once per GPU. */
int tfb_matmul_host_b_resident(const void* A_host, const void* B_device, void* C_host, int64_t M, int64_t N,
                               int64_t K, int dtype, void* stream);

/* One large product sharded over the GPUs of this process by row panels: device devices[g] computes
 * C_panels[g][panel_rows[g], N] = A_panels[g][panel_rows[g], K] · B_replicas[g][K, N] on streams[g]
 * (streams == NULL, or a NULL entry: that device's default stream). Every pointer of entry g is
 * memory of device devices[g]; B is replicated, nothing crosses between GPUs and there is no
 * collective. The call enqueues on every device and returns; synchronise each stream before reading
 * its panel. The calling thread's current device is restored. A device may appear more than once
 * (with different streams). ref: no counterpart — the reference runs on device 0 only
 * (cuda/CudaContext.cpp:57-60; cuda/memory/CudaStorageAllocator.cpp:111-115). */
int tfb_matmul_row_panels(int n_devices, const int* devices, const void* const* A_panels,
                          const void* const* B_replicas, void* const* C_panels, const int64_t* panel_rows,
                          int64_t N, int64_t K, int in_dtype, int out_dtype, void* const* streams);

/* FP32 C[M,N] = A[M,K] · B[K,N] (row-major, dense) that never allocates: for hosts that may not
 * call cudaMalloc where they call us — inside a latency-critical loop that cannot take the
 * allocator's locks or its device-wide synchronisation, under a runtime that owns all device
 * memory through its own arena, or during teardown. The scratch for the TF32 hi / lo operand
 * planes is a fixed 16 MiB array inside the library (tfb_matmul_f32_static_limit() bytes; every
 * GPU that loads the library holds it until the process exits), so products whose split operands
 * do not fit — about M·K + K·N > 2 Mi elements — are rejected with TFB_ERR_TOO_LARGE.
 * The first call on each device looks up the array's device address; make that call before any
 * stream capture. All calls on a device share the array: calls that may overlap on the GPU
 * (different streams) race on it, calls on one stream are safe. Same results as tfb_matmul.
 * This entry point has no counterpart in the reference. */
size_t tfb_matmul_f32_static_limit(void);
int tfb_matmul_f32_static(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K,
                          void* stream);

/* dA[M,K] = dC[M,N] · Bᵀ and dB[K,N] = Aᵀ · dC for C = A · B (row-major, dense). Either
 * output pointer may be NULL to skip it. ref: MatmulBackward::apply,
 * autograd/ops/MatmulBackward.hpp:26-34. */
int tfb_matmul_backward(const void* dC, const void* A, const void* B, void* dA, void* dB,
                        int64_t M, int64_t N, int64_t K, int dtype, void* stream);

/* ---- nn::Linear ------------------------------------------------------------------ */

/* Y[batch,out] = X[batch,in] · Wᵀ (+ bias[out]) (then ReLU if relu != 0); W is [out,in] as the
 * reference stores it. One GEMM with the bias and the activation in its epilogue; bias may be
 * NULL (the reference registers a bias but never adds it). Y has the dtype of X and W; bias is
 * FP32. ref: nn::Linear::forward, nn/Linear.cpp:45-64; Tensor::relu, tensor/Tensor.cpp:227-249;
 * CUDA ReluOp, cuda/kernels/elementwise.cu:112-114. */
int tfb_linear_forward(const void* X, const void* W, const float* bias, void* Y, int64_t batch,
                       int64_t in_features, int64_t out_features, int relu, int dtype, void* stream);

/* Backward of the above for the upstream gradient dY[batch,out]:
 *   dZ = relu ? dY ⊙ (Y > 0) : dY      (Y = the forward output; may be NULL when relu == 0)
 *   dX[batch,in] = dZ · W,  dW[out,in] = dZᵀ · X,  dbias[out] = column sums of dZ (FP32).
 * Any of dX, dW, dbias may be NULL. No transposed copy of W, X or dZ is made.
 * ref: ReluBackward, autograd/ops/ReluBackward.hpp:22-32; MatmulBackward,
 * autograd/ops/MatmulBackward.hpp:26-34; TransposeBackward, autograd/ops/TransposeBackward.hpp:26-28. */
int tfb_linear_backward(const void* X, const void* W, const void* Y, const void* dY, void* dX, void* dW,
                        float* dbias, int64_t batch, int64_t in_features, int64_t out_features, int relu,
                        int dtype, void* stream);

/* tfb_linear_backward for FP32 with X and W given as the hi / lo planes tfb_split_tf32 wrote
 * (leading dimensions ldx, ldw: multiples of 4, >= in_features; 16-byte aligned bases). A training
 * step that keeps the planes it made for the forward product (tfb_gemm_presplit with trans_b = 1 and
 * TFB_EPI_BIAS_COL | TFB_EPI_RELU is the forward of such a layer) does not split X and W again. The
 * X planes are read only when dW != NULL, the W planes only when dX != NULL. Results are bit-identical
 * to tfb_linear_backward on the unsplit operands. ref: the tensors MatmulBackward saves,
 * autograd/ops/MatmulBackward.hpp:21-24 — here saved in the form the tensor core consumes. */
int tfb_linear_backward_presplit(const float* X_hi, const float* X_lo, int64_t ldx, const float* W_hi,
                                 const float* W_lo, int64_t ldw, const float* Y, const float* dY, float* dX,
                                 float* dW, float* dbias, int64_t batch, int64_t in_features,
                                 int64_t out_features, int relu, void* stream);

/* ---- nn::Conv2d (implicit GEMM; the im2col / col2im matrices are never materialised) ---- */

/* Output extent of a convolution axis: (in + 2·pad − dilation·(k−1) − 1) / stride + 1.
 * Host function. ref: cuda/kernels/im2col.cu:109-110, nn/Conv2d.cpp:69-75. */
int64_t tfb_conv_out_dim(int64_t in, int64_t k, int64_t stride, int64_t pad, int64_t dilation);

/* out[N,Cout,outH,outW] = conv2d(x[N,Cin,H,W], w[Cout,Cin,kH,kW]) (+ bias[Cout]) (then ReLU if
 * relu != 0), NCHW. dtype is the type of x, w and out (FP32, FP16 or BF16, the reference launchers'
 * dtype surface: cuda/kernels/im2col.cu:124-157); bias is FP32; accumulation is FP32 and 16-bit
 * results are rounded once (16-bit tensors are widened and run through the FP32 kernels). The producers of the GEMM kernel evaluate the im2col index map on the
 * fly; the bias is added in the epilogue. ref: nn::Conv2d::forward, nn/Conv2d.cpp:77-138
 * (launch_im2col cuda/kernels/im2col.cu:58-99 + per-sample launch_gemm_tiled_16x16 +
 * launch_bias_add cuda/kernels/bias_add.cu:49-58). */
int tfb_conv2d_forward(const void* x, const void* w, const float* bias, void* out, int64_t N, int64_t Cin,
                       int64_t H, int64_t W, int64_t Cout, int64_t kH, int64_t kW, int64_t stride_h,
                       int64_t stride_w, int64_t pad_h, int64_t pad_w, int64_t dil_h, int64_t dil_w, int relu,
                       int dtype, void* stream);

/* grad_input[N,Cin,H,W], grad_weight[Cout,Cin,kH,kW] and grad_bias[Cout] for the upstream gradient
 * grad_out[N,Cout,outH,outW]; any output may be NULL. dtype as in tfb_conv2d_forward (grad_bias is
 * always FP32). grad_input is computed in gather form (no
 * atomics, fixed summation order); grad_weight is a split-K product over (sample, position) with a
 * second-stage reduction in fixed order, and the bias gradient comes out of the same product.
 * Uses library-owned scratch memory. ref: nn::Conv2d::backward, nn/Conv2d.cpp:140-260
 * (launch_col2im cuda/kernels/col2im.cu:50-80, launch_transpose_2d,
 * launch_reduce_sum_axis_nchw cuda/kernels/reduce_sum_axis.cu:54-87). */
int tfb_conv2d_backward(const void* x, const void* w, const void* grad_out, void* grad_input, void* grad_weight,
                        float* grad_bias, int64_t N, int64_t Cin, int64_t H, int64_t W, int64_t Cout, int64_t kH,
                        int64_t kW, int64_t stride_h, int64_t stride_w, int64_t pad_h, int64_t pad_w,
                        int64_t dil_h, int64_t dil_w, int dtype, void* stream);

/* Writes the im2col index map the forward kernel uses, for samples [n_first, n_first + n_count):
 * out[((n - n_first)·K + t)·P + p] = flat NCHW offset of the input element that column-matrix
 * entry (n, t, p) reads, or -1 where it falls in the padding (K = Cin·kH·kW, P = outH·outW).
 * `out` is a device buffer of n_count·K·P int64. For verification against
 * ref: cuda/kernels/im2col.cu:67-98. */
int tfb_im2col_index_map(int64_t* out, int64_t n_first, int64_t n_count, int64_t Cin, int64_t H, int64_t W,
                         int64_t kH, int64_t kW, int64_t stride_h, int64_t stride_w, int64_t pad_h, int64_t pad_w,
                         int64_t dil_h, int64_t dil_w, void* stream);

/* ---- MLP training step neighbours ------------------------------------------------- */

/* Mean negative log-likelihood of log_softmax(logits) and its gradient:
 *   loss = -(1/global_rows) · Σ_r log_softmax(logits)[r, labels[r]]      (this call's rows only)
 *   dlogits = (softmax(logits) - onehot(labels)) / global_rows
 * global_rows is the batch size of the whole data-parallel step, so per-rank gradients add up to
 * the full-batch gradient. loss_out (one device float) and dlogits may be NULL. FP32, labels int64.
 * ref: Tensor::log_softmax, tensor/Tensor.cpp:411-447; LogSoftmaxBackward,
 * autograd/ops/LogSoftmaxBackward.hpp:26-58; the loss graph of examples/train_mlp.cpp:54-76. */
int tfb_log_softmax_nll(const float* logits, const int64_t* labels, float* dlogits, float* loss_out,
                        int64_t rows, int64_t cols, int64_t global_rows, void* stream);

/* v <- momentum·v + grad_scale·g ;  p <- p - lr·v, elementwise over n FP32 values.
 * ref: the update documented in nn/optim/SGD.hpp:3-6 (the shipped SGD::step throws for
 * parameters with more than one element, nn/optim/SGD.cpp:38-57). */
int tfb_sgd_momentum(float* params, float* velocity, const float* grads, int64_t n, float lr,
                     float momentum, float grad_scale, void* stream);

/* ---- the data-parallel MLP training step as one object ---------------------------------- */

/* Linear -> ReLU -> ... -> Linear -> log_softmax + mean NLL -> backward -> gradient exchange -> SGD with
 * momentum, with every buffer (flat parameters / gradients / velocity, activations, TF32 planes) owned
 * by the handle and nothing allocated or read back by a step. dims[0..n_layers] are the layer widths
 * (ReLU after every layer but the last); a step takes at most max_rows rows. The handle belongs to the
 * device that is current at creation; that device must be current for every call on it. Weights are
 * [out,in] row-major as the reference stores them and start at zero: fill them through
 * tfb_mlp_buffer(TFB_MLP_PARAMS) + tfb_mlp_segment + tfb_memcpy.
 * ref: the training loop of examples/train_mlp.cpp:161-183 (model :33-52, loss graph :54-76, manual
 * update :140-159) with the momentum update documented in nn/optim/SGD.hpp:3-6. */
typedef struct tfb_mlp tfb_mlp;
int tfb_mlp_create(int n_layers, const int64_t* dims, int64_t max_rows, tfb_mlp** out);
int tfb_mlp_destroy(tfb_mlp* m);
/* Floats in the flat parameter / gradient / velocity buffers (each weight and bias padded to a multiple
 * of 4 floats so that it starts on a 16-byte boundary), and where layer `layer` sits in them. */
int64_t tfb_mlp_numel(const tfb_mlp* m);
int tfb_mlp_segment(const tfb_mlp* m, int layer, int64_t* weight_offset, int64_t* bias_offset);
/* Device pointers of the handle's buffers. PARAMS, VELOCITY, REDUCED_GRADS: numel floats. GRADS:
 * numel floats followed by this rank's loss contribution (so one collective over numel + 4 floats sums
 * both). LOSS: one float, the loss of the last step summed over all ranks. ACTIVATION: the output of
 * layer `layer` of the last forward pass, [rows, dims[layer + 1]]. REGION: the exchange region (what
 * other ranks map). `layer` is ignored for the others. */
#define TFB_MLP_PARAMS 0
#define TFB_MLP_GRADS 1
#define TFB_MLP_VELOCITY 2
#define TFB_MLP_LOSS 3
#define TFB_MLP_REDUCED_GRADS 4
#define TFB_MLP_ACTIVATION 5
#define TFB_MLP_REGION 6
#define TFB_MLP_INPUT_GRAD 7   /* gradient with respect to the input of layer `layer` >= 1, [rows, dims[layer]] */
#define TFB_MLP_EXCHANGE_TRACE 8   /* five uint64 %globaltimer stamps of the last exchange (see TRACE_EXCHANGE) */
int tfb_mlp_buffer(tfb_mlp* m, int which, int layer, void** ptr_out);

/* This rank's share of the full-batch gradient for its `rows` rows of a global batch of global_rows
 * rows (<= 0: rows), into GRADS, and its loss contribution. ref: forward + Tensor::backward of
 * examples/train_mlp.cpp:167-175. */
int tfb_mlp_forward_backward(tfb_mlp* m, const float* X, const int64_t* labels, int64_t rows, int64_t global_rows,
                             void* stream);
/* v <- momentum*v + g ; p <- p - lr*v over the whole flat buffers from this rank's own GRADS, and LOSS <-
 * the loss slot: the update of a single rank, or of every rank after an all-reduce the caller ran over
 * GRADS (numel + 4 floats, e.g. one ncclAllReduce). ref: nn/optim/SGD.hpp:3-6. */
int tfb_mlp_update(tfb_mlp* m, float lr, float momentum, void* stream);
/* The same update fused with the gradient exchange, one kernel over NVLink peer memory: each rank adds
 * its slice of all ranks' GRADS in rank order, updates that slice of the velocity and the parameters and
 * stores the new parameters into every rank's PARAMS; LOSS <- the sum of the ranks' loss slots. Every
 * rank of the group must call it once per step, on a stream that follows its forward_backward; the
 * kernel waits (bounded, TFB_MLP_OPT_WAIT_LIMIT_NS) for the peers and records device error 107 if one
 * does not arrive. VELOCITY is then only maintained for this rank's slice, so do not alternate between
 * this call and tfb_mlp_update on one handle. With a group of one it is tfb_mlp_update.
 * ref: no counterpart (the reference is single-device, cuda/CudaContext.cpp:57-60). */
int tfb_mlp_exchange_update(tfb_mlp* m, float lr, float momentum, void* stream);
/* tfb_mlp_forward_backward followed by tfb_mlp_exchange_update. */
int tfb_mlp_step(tfb_mlp* m, const float* X, const int64_t* labels, int64_t rows, int64_t global_rows, float lr,
                 float momentum, void* stream);
/* Records a step into a CUDA graph held by the handle (replacing an earlier one) and replays it:
 * what = STEP (forward_backward + exchange_update), FORWARD_BACKWARD, or UPDATE (tfb_mlp_update, for
 * callers that run their own all-reduce between two graphs). X and labels are captured by address:
 * refill them in place. Run the same call eagerly once before capturing (the library's scratch buffer
 * must exist), and capture on a stream other than the legacy default stream. */
#define TFB_MLP_CAPTURE_STEP 0
#define TFB_MLP_CAPTURE_FORWARD_BACKWARD 1
#define TFB_MLP_CAPTURE_UPDATE 2
int tfb_mlp_capture_step(tfb_mlp* m, const float* X, const int64_t* labels, int64_t rows, int64_t global_rows,
                         float lr, float momentum, int what, void* stream);
int tfb_mlp_replay(tfb_mlp* m, void* stream);
/* WAIT_LIMIT_NS: how long the exchange kernel waits for a peer (default 2 s). EXCHANGE_CTAS: its grid
 * (0 = choose; every rank of a group must use the same value). KEEP_REDUCED_GRADS: non-zero makes the
 * exchange also store the summed gradient of this rank's slice into REDUCED_GRADS. TRACE_EXCHANGE: non-zero
 * makes CTA 0 of the exchange kernel record nanosecond timestamps at its phase boundaries (start, after the
 * first flag barrier, after the slice has been summed / updated / stored, after the system-scope fence,
 * after the second barrier) into EXCHANGE_TRACE. EXCHANGE_BUCKETS: 1 = one exchange launch behind the backward
 * pass; 2 = a whole step (tfb_mlp_step, or a captured TFB_MLP_CAPTURE_STEP) exchanges the gradients of every
 * layer but the first on a side stream of the handle as soon as they are complete — concurrently with the
 * first layer's weight gradient, on at most 32 SMs — and the first layer's behind it; same sums in the same
 * order, so the same bits (every rank of a group must use the same value). */
#define TFB_MLP_OPT_WAIT_LIMIT_NS 0
#define TFB_MLP_OPT_EXCHANGE_CTAS 1
#define TFB_MLP_OPT_KEEP_REDUCED_GRADS 2
#define TFB_MLP_OPT_TRACE_EXCHANGE 3
#define TFB_MLP_OPT_EXCHANGE_BUCKETS 4
int tfb_mlp_set_option(tfb_mlp* m, int option, int64_t value);

/* Forming a group of `world` <= 8 ranks (one handle per rank, same dims). The library does not own a
 * rendezvous: the host moves the handles or pointers between ranks by whatever means it has.
 * One process per GPU: every rank writes tfb_mlp_ipc_handle_bytes() bytes with tfb_mlp_ipc_handle,
 * the host gathers them in rank order, and every rank calls tfb_mlp_connect_ipc with the gathered array.
 * Peer regions mapped some other way (a symmetric-memory allocator, a driver-level mapping):
 * tfb_mlp_connect_ptrs with the regions as this rank addresses them (entry `rank` is ignored).
 * One process, several devices: tfb_mlp_connect_local over all handles (enables peer access).
 * ref: no counterpart; the reference has no multi-device support (cuda/CudaContext.cpp:57-60). */
size_t tfb_mlp_ipc_handle_bytes(void);
int tfb_mlp_ipc_handle(tfb_mlp* m, void* handle_out);
int tfb_mlp_connect_ipc(tfb_mlp* m, int rank, int world, const void* handles);
int tfb_mlp_connect_ptrs(tfb_mlp* m, int rank, int world, void* const* regions);
int tfb_mlp_connect_local(tfb_mlp* const* ms, int world);
/* The exchange of a whole group whose handles all live on the current device (ranks emulated on one
 * GPU), as ONE cooperative launch in which every rank's CTAs are resident together — separate launches
 * that wait for each other on one GPU have no such guarantee. Handle r must be rank r of `world`. */
int tfb_mlp_exchange_update_one_device(tfb_mlp* const* ms, int world, float lr, float momentum, void* stream);

/* ---- summing small FP32 buffers across GPUs through peer memory ------------------------------- */

/* A member of a group of up to 8 ranks that add FP32 buffers of at most capacity_floats elements: one
 * kernel per rank over NVLink peer memory (flag barrier, rank r adds slice r of all contributions in
 * rank order — a fixed order — and stores it to every rank, flag barrier). Made for the gradient
 * exchange of batch-sharded layers whose gradient is small, where a library collective is pure latency.
 * The member belongs to the device current at creation. Each rank writes its contribution into the
 * `in` buffer and reads the sum from the `out` buffer (tfb_peer_group_buffers). Connecting the ranks
 * works as for tfb_mlp: IPC handles (one process per GPU) or already mapped regions. Waits are bounded
 * (default 2 s; device error 107 when a peer does not arrive).
 * ref: no counterpart (the reference is single-device, cuda/CudaContext.cpp:57-60). */
typedef struct tfb_peer_group tfb_peer_group;
int tfb_peer_group_create(int64_t capacity_floats, tfb_peer_group** out);
int tfb_peer_group_destroy(tfb_peer_group* g);
int tfb_peer_group_buffers(tfb_peer_group* g, float** in_out, float** out_out, void** region_out);
int tfb_peer_group_set_wait_limit(tfb_peer_group* g, int64_t nanoseconds);
int tfb_peer_group_ipc_handle(tfb_peer_group* g, void* handle_out);   /* tfb_mlp_ipc_handle_bytes() bytes */
int tfb_peer_group_connect_ipc(tfb_peer_group* g, int rank, int world, const void* handles);
int tfb_peer_group_connect_ptrs(tfb_peer_group* g, int rank, int world, void* const* regions);
/* out[0..n) on every rank = sum over ranks of in[0..n). Every rank calls it once per exchange. */
int tfb_peer_allreduce_sum(tfb_peer_group* g, int64_t n, void* stream);
/* The same for a group whose members all live on the current device (ranks emulated on one GPU), as
 * one cooperative launch; member r must be rank r of `world`. */
int tfb_peer_allreduce_sum_one_device(tfb_peer_group* const* gs, int world, int64_t n, void* stream);

/* Backward of a convolution whose BATCH is sharded over the ranks of a group (FP32): grad_input for
 * this rank's N_local samples, and this rank's share of grad_weight and grad_bias written into the
 * group's `in` buffer — grad_weight at offset 0, grad_bias at offset round_up(Cout·Cin·kH·kW, 4) —
 * followed (allreduce != 0) by tfb_peer_allreduce_sum, after which `out` holds the full-batch weight
 * and bias gradients on every rank in the same layout. The forward pass of a batch shard is
 * tfb_conv2d_forward on the local samples; it needs no exchange.
 * ref: nn::Conv2d::backward, nn/Conv2d.cpp:140-260 (its per-sample accumulation of grad_weight,
 * :215-243, is the sum this exchange completes across ranks). */
int tfb_conv2d_backward_sharded(tfb_peer_group* g, const void* x, const void* w, const void* grad_out, void* grad_input,
                                int64_t N_local, int64_t Cin, int64_t H, int64_t W, int64_t Cout, int64_t kH, int64_t kW,
                                int64_t stride_h, int64_t stride_w, int64_t pad_h, int64_t pad_w, int64_t dil_h,
                                int64_t dil_w, int allreduce, void* stream);

/* ---- device-side pieces of the autograd walk (FP32, n elements, any alignment) ---------- */

/* dst[i] = value. The ones-fill of the root gradient that Tensor::backward does in a host loop.
 * ref: autograd/TensorAutograd.cpp:57-70. */
int tfb_fill(float* dst, int64_t n, float value, void* stream);
/* y = max(x, 0). ref: Tensor::relu, tensor/Tensor.cpp:227-249; ReluOp, cuda/kernels/elementwise.cu:112-114. */
int tfb_relu_forward(const float* x, float* y, int64_t n, void* stream);
/* dx = x > 0 ? dy : 0 (zero at x == 0), x the ReLU's input — or its output, which has the same sign.
 * ref: ReluBackward, autograd/ops/ReluBackward.hpp:22-32 (host loop building a mask, then a product). */
int tfb_relu_backward(const float* x, const float* dy, float* dx, int64_t n, void* stream);
/* dst += src: gradient accumulation where a tensor feeds several consumers.
 * ref: InputBuffer::add, autograd/InputBuffer.cpp:11-26, 32-41 (host loop). */
int tfb_accumulate(float* dst, const float* src, int64_t n, void* stream);
/* dst = src · scalar[0] with the scalar in device memory (a loss node scaling its saved gradient by
 * the upstream one-element gradient without reading it on the host).
 * ref: the scalar products closing the loss graph, examples/train_mlp.cpp:68-75. */
int tfb_scale_by_device_scalar(const float* src, const float* scalar, float* dst, int64_t n, void* stream);

/* ---- device memory: one explicit stream-ordered pool per device ------------------------ */

/* ref for the whole group: CudaStorageAllocator, cuda/memory/CudaStorageAllocator.cpp:34-57
 * (pool set-up, 64 MiB release threshold), :101-125 (allocate), :127-143 (free), :64-86 (copy
 * callback). Differences by design: a pool per device instead of each device's default pool;
 * the call runs with `device` current (the reference always issues on device 0's stream); a
 * working free, so a Storage deleter can exist (tensor/Storage.hpp:27 has none). */
int tfb_device_count(int* count_out);
/* bytes == 0 allocates one byte, like the reference. `stream` must be a stream of `device`. */
int tfb_alloc(int device, size_t bytes, void* stream, void** ptr_out);
int tfb_free(void* ptr, int device, void* stream);
int tfb_pool_set_release_threshold(int device, uint64_t bytes);
int tfb_pool_trim(int device, size_t keep_bytes);
int tfb_pool_stats(int device, uint64_t* reserved, uint64_t* used, uint64_t* reserved_high,
                   uint64_t* used_high);
/* Lets `peer` read and write memory allocated from `device`'s pool (plain peer loads / copies). */
int tfb_pool_enable_peer(int device, int peer);
/* The scratch the library itself holds on `device` (TF32 planes, split-K partials; one grow-only
 * stream-ordered buffer per stream that has needed one): how many buffers and their total size.
 * ref: no counterpart. */
int tfb_scratch_stats(int device, uint64_t* buffers_out, uint64_t* bytes_out);
/* Device and stream plumbing for hosts compiled without CUDA headers: a non-blocking stream per
 * (thread, device) replaces the reference's single stream of device 0.
 * ref: DeviceContext / CudaStream, cuda/CudaContext.cpp:18-60, cuda/CudaContext.hpp:134-140. */
int tfb_set_device(int device);
int tfb_get_device(int* device_out);
int tfb_stream_create(int device, void** stream_out);
int tfb_stream_destroy(void* stream);
int tfb_stream_synchronize(void* stream);
/* kind: 0 host-to-host, 1 host-to-device, 2 device-to-host, 3 device-to-device (the numbering of
 * allocator_dispatch::CudaCopyKind). Asynchronous on `stream`. */
int tfb_memcpy(void* dst, const void* src, size_t bytes, int kind, void* stream);

#ifdef __cplusplus
}
#endif

#endif /* TFB_H_ */
