// FP32 products with few output rows and a long contraction (the forward product of a 64-row Linear layer,
// the weight gradient of an MLP's 10-class head): one CUDA-core kernel, plain FP32 FMAs in ascending K
// order, no operand split and no second kernel. The tensor-core path pads such a product to 128-row tiles
// and spends ~20 us on it in three launches (split, GEMM, split-K reduction), almost all of it latency;
// this kernel is one launch of ~10 us and, being exact FP32 arithmetic, sits closer to the reference's
// sequential sum than the 3xTF32 product does. Measured per call under CUDA-graph replay (this kernel /
// tensor-core path): 64 x 256 x 784 9.5 / 19.3 us, 10 x 1024 x 1024 10.1 / 19.8 us; products with more
// rows, a short contraction (1024 x 1024 x 10: 15.8 / 6.9 us) or a very long one stay on the tensor cores.
//
// A block of 256 threads computes a 16 x 16 tile of the output, one element per thread, over ITS slice of
// the contraction: up to eight blocks — a thread-block cluster along K — share one tile, so a product with
// K = 784 or 1024 is one round trip to memory deep instead of eight, and the cluster's rank-0 block adds the
// eight partial sums through distributed shared memory in rank order (a fixed order: deterministic) before
// the epilogue. Both operand tiles are staged in shared memory with K contiguous ([16][128 + 4] floats each),
// whatever their layout in global memory, so the inner loop is two 16-byte shared-memory reads per four
// FMAs; the read of the A row is a broadcast within a half-warp. Operands given as TF32 hi / lo planes are
// added back together on the way in (hi + lo is exactly the original value).
#include <utility>

#include "internal.hpp"
#include "ptx.cuh"

namespace tfb {
namespace {

constexpr int kTile = 16, kChunk = 128, kLds = kChunk + 4, kMaxSplit = 8;
// The window in which this kernel is used (from the measurements above).
// (Beyond K ~ 2048 each block walks several 128-element chunks one after the other and the tensor cores
// win again: the 10 x 1024 x 8192 weight gradient of the head at batch 8192 took ~90 us here against 25 us.)
constexpr int64_t kMaxRows = 128, kMaxOutputs = 16384, kMinK = 512, kMaxK = 2048;

struct SmallArgs {
    const float* A;       // op(A)[m][k] at A[m * sa_m + k * sa_k]
    const float* A_lo;    // optional second plane (null: A holds the values themselves)
    const float* B;       // op(B)[k][n] at B[k * sb_k + n * sb_n]
    const float* B_lo;
    float* C;
    int M, N, K;
    int k_per_split;      // K elements per block of the cluster (a multiple of 4)
    long long sa_m, sa_k, sb_k, sb_n;
    long long sc_m, sc_n;  // C[m][n] at C[m * sc_m + n * sc_n]: (ldc, 1), or (1, ldc) when the product runs transposed
    long long sp_m, sp_n;  // the same for the result planes
    const float* bias;
    int bias_mode, relu;
    float* planes_hi;     // optional TF32 planes of the result, leading dimension N
    float* planes_lo;
};

__device__ __forceinline__ float tf32_rn(float x) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return __uint_as_float(r);
}

__device__ __forceinline__ float ld_shared_cluster_f32(uint32_t addr) {
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
    return v;
}

// grid = (N tiles, M tiles, K splits); cluster = (1, 1, K splits)
template <bool A_KFAST, bool B_KFAST>
__global__ void __launch_bounds__(256) small_gemm_kernel(const SmallArgs a) {
    __shared__ __align__(16) float As[kTile][kLds];   // [m][k]
    __shared__ __align__(16) float Bt[kTile][kLds];   // [n][k]
    __shared__ float red[256];
    pdl_wait();
    pdl_launch_dependents();
    const int t = threadIdx.x, tx = t & 15, ty = t >> 4;
    const int m0 = blockIdx.y * kTile, n0 = blockIdx.x * kTile;
    const int splits = gridDim.z, split = blockIdx.z;
    const int k_begin = split * a.k_per_split, k_end = min(a.K, k_begin + a.k_per_split);
    float acc = 0.f;
    for (int k0 = k_begin; k0 < k_end; k0 += kChunk) {
        const int klen = min(kChunk, k_end - k0);
        // 16 x 128 elements per operand, eight per thread, consecutive threads along the contiguous index
#pragma unroll
        for (int h = 0; h < 8; ++h) {
            const int i = t + 256 * h;
            {
                const int m = A_KFAST ? i >> 7 : i & 15, k = A_KFAST ? i & 127 : i >> 4;
                float v = 0.f;
                if (m0 + m < a.M && k < klen) {
                    const long long off = (long long)(m0 + m) * a.sa_m + (long long)(k0 + k) * a.sa_k;
                    v = a.A[off];
                    if (a.A_lo != nullptr) v += a.A_lo[off];
                }
                As[m][k] = v;
            }
            {
                const int n = B_KFAST ? i >> 7 : i & 15, k = B_KFAST ? i & 127 : i >> 4;
                float v = 0.f;
                if (n0 + n < a.N && k < klen) {
                    const long long off = (long long)(k0 + k) * a.sb_k + (long long)(n0 + n) * a.sb_n;
                    v = a.B[off];
                    if (a.B_lo != nullptr) v += a.B_lo[off];
                }
                Bt[n][k] = v;
            }
        }
        __syncthreads();
        const int k4 = (klen + 3) & ~3;   // the tiles are zero beyond klen
        for (int kk = 0; kk < k4; kk += 4) {
            const float4 x = *reinterpret_cast<const float4*>(&As[ty][kk]);
            const float4 y = *reinterpret_cast<const float4*>(&Bt[tx][kk]);
            acc = fmaf(x.x, y.x, acc);
            acc = fmaf(x.y, y.y, acc);
            acc = fmaf(x.z, y.z, acc);
            acc = fmaf(x.w, y.w, acc);
        }
        __syncthreads();
    }
    if (splits > 1) {
        // every block publishes its partial sums; rank 0 adds them in rank order
        red[t] = acc;
        cluster_arrive();
        cluster_wait();
        if (split == 0) {
            const uint32_t mine = smem_u32(&red[t]);
            for (int r = 1; r < splits; ++r) acc += ld_shared_cluster_f32(mapa_shared(mine, (uint32_t)r));
        }
        // nobody leaves while rank 0 may still be reading its shared memory
        cluster_arrive();
        cluster_wait();
        if (split != 0) return;
    }
    const int m = m0 + ty, n = n0 + tx;
    if (m >= a.M || n >= a.N) return;
    if (a.bias_mode == 1) acc += __ldg(a.bias + n);
    if (a.bias_mode == 2) acc += __ldg(a.bias + m);
    if (a.relu) acc = acc > 0.f ? acc : 0.f;
    a.C[(long long)m * a.sc_m + (long long)n * a.sc_n] = acc;
    const long long po = (long long)m * a.sp_m + (long long)n * a.sp_n;
    if (a.planes_hi != nullptr) {
        const float hi = tf32_rn(acc);
        a.planes_hi[po] = hi;
        a.planes_lo[po] = acc - hi;
    } else if (a.planes_lo != nullptr) {   // the consumer reads C itself as the hi plane
        a.planes_lo[po] = tf32_rn(acc - __uint_as_float(__float_as_uint(acc) & 0xFFFFE000u));
    }
}

template <bool A_KFAST, bool B_KFAST>
int launch_small(const SmallArgs& a, dim3 grid, cudaStream_t stream) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(256);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = grid.z;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = tuning(TFB_TUNE_PDL) != 0 ? 2 : 1;
    TFB_CUDA_OK(cudaLaunchKernelEx(&cfg, small_gemm_kernel<A_KFAST, B_KFAST>, a));
    return TFB_OK;
}

}  // namespace

// Few rows, or — the same product read as C^T = B^T A^T — few columns (the 10-class head of an MLP).
bool small_gemm_eligible(const GemmCall& c) {
    return tuning(TFB_TUNE_SMALL_GEMM) != 0 && c.in_dtype == TFB_DTYPE_F32 && c.out_dtype == TFB_DTYPE_F32 &&
           c.a_mask == nullptr && c.force_bn == 0 && (c.M <= kMaxRows || c.N <= kMaxRows) && c.M * c.N <= kMaxOutputs &&
           c.K >= kMinK && c.K <= kMaxK;
}

int small_gemm_run(const GemmCall& c, cudaStream_t stream) {
    SmallArgs a;
    a.A = static_cast<const float*>(c.A);
    a.A_lo = c.a_presplit && !c.a_raw_hi ? a.A + c.a_lo_off : nullptr;   // a raw hi plane is the value itself
    a.B = static_cast<const float*>(c.B);
    a.B_lo = c.b_presplit && !c.b_raw_hi ? a.B + c.b_lo_off : nullptr;
    a.C = static_cast<float*>(c.C);
    a.M = (int)c.M; a.N = (int)c.N; a.K = (int)c.K;
    // a_kmajor: A stored [M][K] (K contiguous); else stored [K][M]
    a.sa_m = c.a_kmajor ? c.lda : 1;
    a.sa_k = c.a_kmajor ? 1 : c.lda;
    // b_kmajor: B stored [N][K] (K contiguous); else stored [K][N]
    a.sb_k = c.b_kmajor ? 1 : c.ldb;
    a.sb_n = c.b_kmajor ? c.ldb : 1;
    a.sc_m = c.ldc; a.sc_n = 1;
    a.sp_m = c.N; a.sp_n = 1;
    a.bias = c.bias; a.bias_mode = c.bias_mode; a.relu = c.relu ? 1 : 0;
    a.planes_hi = c.planes_hi; a.planes_lo = c.planes_lo;
    bool a_kfast = c.a_kmajor, b_kfast = c.b_kmajor;
    if (c.M > kMaxRows) {
        // Many rows, few columns: run C^T = B^T A^T, i.e. swap the operands' roles and store transposed.
        std::swap(a.A, a.B);
        std::swap(a.A_lo, a.B_lo);
        const long long am = a.sa_m, ak = a.sa_k;
        a.sa_m = a.sb_n; a.sa_k = a.sb_k;
        a.sb_n = am; a.sb_k = ak;
        std::swap(a.M, a.N);
        std::swap(a.sc_m, a.sc_n);
        std::swap(a.sp_m, a.sp_n);
        if (a.bias_mode != 0) a.bias_mode = 3 - a.bias_mode;   // per column <-> per row
        std::swap(a_kfast, b_kfast);
    }
    if (a.planes_hi != nullptr && a.planes_lo == nullptr)
        return fail(TFB_ERR_INVALID_ARG, "gemm: a hi result plane without its lo plane");
    // one block of the cluster per 128 elements of K, at most eight (the portable cluster size)
    int splits = (int)((c.K + kChunk - 1) / kChunk);
    if (splits > kMaxSplit) splits = kMaxSplit;
    a.k_per_split = (int)(((c.K + splits - 1) / splits + 3) / 4 * 4);
    splits = (int)((c.K + a.k_per_split - 1) / a.k_per_split);
    const dim3 grid((unsigned)((a.N + kTile - 1) / kTile), (unsigned)((a.M + kTile - 1) / kTile), (unsigned)splits);
    if (a_kfast && b_kfast) return launch_small<true, true>(a, grid, stream);
    if (a_kfast && !b_kfast) return launch_small<true, false>(a, grid, stream);
    if (!a_kfast && b_kfast) return launch_small<false, true>(a, grid, stream);
    return launch_small<false, false>(a, grid, stream);
}

}  // namespace tfb
