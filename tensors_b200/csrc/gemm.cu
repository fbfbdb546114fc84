// Host side of the tcgen05 GEMM: tensor-map construction, operand preparation
// (TF32 hi/lo split, re-packing of unaligned 16-bit operands), tile-shape choice, launch.
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "gemm_kernel.cuh"
#include "internal.hpp"

namespace tfb {

// ---------------------------------------------------------------------------
// Tensor maps
// ---------------------------------------------------------------------------
namespace {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn g_encode = nullptr;
std::once_flag g_encode_once;

int resolve_encoder() {
    std::call_once(g_encode_once, [] {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
        if (e == cudaSuccess && q == cudaDriverEntryPointSuccess)
            g_encode = reinterpret_cast<EncodeTiledFn>(fn);
        else
            (void)cudaGetLastError();
    });
    if (g_encode == nullptr)
        return fail(TFB_ERR_CUDA, "the driver does not export cuTensorMapEncodeTiled");
    return TFB_OK;
}

// `atom32` selects the 128-byte swizzle with 32-byte atoms that MN-major 32-bit operands need.
// 2-D map over a row-major matrix: `inner` contiguous elements per row, `outer` rows,
// rows `row_stride_bytes` apart; box of box_inner x box_outer elements, 128-byte swizzle,
// out-of-range elements read as zero.
}  // namespace

int make_map(CUtensorMap* map, int dtype, const void* base, uint64_t inner, uint64_t outer,
             uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer, bool atom32) {
    int rc0 = resolve_encoder();
    if (rc0 != TFB_OK) return rc0;
    CUtensorMapDataType dt = dtype == TFB_DTYPE_F32   ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                             : dtype == TFB_DTYPE_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                      : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    cuuint64_t gdim[2] = {inner, outer};
    cuuint64_t gstride[1] = {row_stride_bytes};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = g_encode(map, dt, 2, const_cast<void*>(base), gdim, gstride, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE,
                          atom32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(TFB_ERR_CUDA,
                    "cuTensorMapEncodeTiled failed with %d (inner %llu outer %llu stride %llu box %ux%u)",
                    (int)r, (unsigned long long)inner, (unsigned long long)outer,
                    (unsigned long long)row_stride_bytes, box_inner, box_outer);
    return TFB_OK;
}

int make_map_nd(CUtensorMap* map, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                const uint32_t* box, bool atom32, const uint32_t* elem_strides) {
    int rc0 = resolve_encoder();
    if (rc0 != TFB_OK) return rc0;
    if (rank < 2 || rank > 5) return fail(TFB_ERR_INVALID_ARG, "tensor map rank %d", rank);
    cuuint64_t gdim[5];
    cuuint64_t gstride[4];
    cuuint32_t bx[5], estr[5];
    for (int i = 0; i < rank; ++i) {
        gdim[i] = dims[i];
        bx[i] = box[i];
        estr[i] = elem_strides != nullptr ? elem_strides[i] : 1;
        if (i > 0) gstride[i - 1] = strides_bytes[i - 1];
    }
    CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, (cuuint32_t)rank, const_cast<void*>(base), gdim,
                          gstride, bx, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          atom32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(TFB_ERR_CUDA, "cuTensorMapEncodeTiled (rank %d) failed with %d (dims %llu %llu %llu, box %u %u %u)",
                    rank, (int)r, (unsigned long long)dims[0], (unsigned long long)dims[1],
                    (unsigned long long)(rank > 2 ? dims[2] : 0), box[0], box[1], rank > 2 ? box[2] : 0u);
    return TFB_OK;
}

namespace {

// ---------------------------------------------------------------------------
// Operand preparation kernels (HBM-bound, one pass)
// ---------------------------------------------------------------------------
__device__ __forceinline__ float tf32_round(float x) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return __uint_as_float(r);
}
// What the tensor core makes of a raw FP32 operand under kind::tf32: the low 13 mantissa bits dropped.
__device__ __forceinline__ float tf32_trunc(float x) { return __uint_as_float(__float_as_uint(x) & 0xFFFFE000u); }

// hi = x rounded to TF32 (10-bit mantissa), lo = x - hi (exact in FP32).
// One thread per group of 4 output columns; ld_out is a multiple of 4 so the stores are
// 16-byte vectors. Columns in [cols, ld_out) are written as zeros.
// With hi == nullptr only a lo plane is written, for a product that reads the operand itself as its hi
// plane: lo = x - trunc(x), rounded to TF32 (the tensor core would otherwise truncate it too).
struct SplitJob {
    const float* src;
    long long rows, cols, ld;
    const float* mask;
    float* hi;
    float* lo;
    long long ld_out;
};

// The work of blocks [0, nblocks) on one matrix; `block` is this block's index among them.
__device__ __forceinline__ void split_tf32_body(const SplitJob& job, long long block, long long nblocks) {
    const float* __restrict__ src = job.src;
    const float* __restrict__ mask = job.mask;
    float* __restrict__ hi = job.hi;
    float* __restrict__ lo = job.lo;
    const long long rows = job.rows, cols = job.cols, ld = job.ld, ld_out = job.ld_out;
    const long long groups = ld_out >> 2;
    const long long total = rows * groups;
    const bool vec_in = ((ld & 3) == 0) && ((reinterpret_cast<uintptr_t>(src) & 15u) == 0) &&
                        (mask == nullptr || (reinterpret_cast<uintptr_t>(mask) & 15u) == 0);
    for (long long i = block * blockDim.x + threadIdx.x; i < total; i += nblocks * blockDim.x) {
        const long long r = i / groups;
        const long long c = (i - r * groups) << 2;
        float x[4] = {0.f, 0.f, 0.f, 0.f};
        const float* p = src + r * ld + c;
        if (vec_in && c + 4 <= cols) {
            const float4 v = *reinterpret_cast<const float4*>(p);
            x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w;
            if (mask != nullptr) {
                const float4 m = *reinterpret_cast<const float4*>(mask + r * ld + c);
                x[0] = m.x > 0.f ? x[0] : 0.f;
                x[1] = m.y > 0.f ? x[1] : 0.f;
                x[2] = m.z > 0.f ? x[2] : 0.f;
                x[3] = m.w > 0.f ? x[3] : 0.f;
            }
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (c + j < cols) {
                    float v = p[j];
                    if (mask != nullptr) v = mask[r * ld + c + j] > 0.f ? v : 0.f;
                    x[j] = v;
                }
            }
        }
        float h[4], l[4];
        if (hi != nullptr) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                h[j] = tf32_round(x[j]);
                l[j] = x[j] - h[j];
            }
            *reinterpret_cast<float4*>(hi + r * ld_out + c) = make_float4(h[0], h[1], h[2], h[3]);
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) l[j] = tf32_round(x[j] - tf32_trunc(x[j]));
        }
        *reinterpret_cast<float4*>(lo + r * ld_out + c) = make_float4(l[0], l[1], l[2], l[3]);
    }
}

__global__ void split_tf32_kernel(const float* __restrict__ src, long long rows, long long cols,
                                  long long ld, const float* __restrict__ mask,
                                  float* __restrict__ hi, float* __restrict__ lo, long long ld_out) {
    pdl_wait();
    pdl_launch_dependents();
    const SplitJob job{src, rows, cols, ld, mask, hi, lo, ld_out};
    split_tf32_body(job, blockIdx.x, gridDim.x);
}

// Both operands of a product in one launch: blocks [0, blocks_a) split A, the rest split B.
__global__ void split_tf32_pair_kernel(const SplitJob a, const SplitJob b, int blocks_a) {
    pdl_wait();
    pdl_launch_dependents();
    if ((int)blockIdx.x < blocks_a) split_tf32_body(a, blockIdx.x, blocks_a);
    else split_tf32_body(b, (long long)blockIdx.x - blocks_a, (long long)gridDim.x - blocks_a);
}

// Copies a 16-bit matrix into a buffer whose leading dimension is a multiple of 8.
__global__ void pack16_kernel(const uint16_t* __restrict__ src, long long rows, long long cols,
                              long long ld, uint16_t* __restrict__ dst, long long ld_out) {
    pdl_wait();
    pdl_launch_dependents();
    const long long total = rows * ld_out;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / ld_out;
        const long long c = i - r * ld_out;
        dst[i] = c < cols ? src[r * ld + c] : (uint16_t)0;
    }
}

// C = epilogue(0) for a contraction of length zero.
__global__ void empty_k_kernel(const GemmArgs a) {
    pdl_wait();
    pdl_launch_dependents();
    const long long total = (long long)a.M * a.N;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / a.N, c = i - r * a.N;
        float v = 0.f;
        if (a.bias_mode == kBiasPerCol) v = a.bias[c];
        if (a.bias_mode == kBiasPerRow) v = a.bias[r];
        if (a.relu) v = v > 0.f ? v : 0.f;
        if (a.out_type == kOutF32) static_cast<float*>(a.C)[r * a.ldc + c] = v;
        else if (a.out_type == kOutBF16)
            static_cast<__nv_bfloat16*>(a.C)[r * a.ldc + c] = __float2bfloat16_rn(v);
        else static_cast<__half*>(a.C)[r * a.ldc + c] = __float2half_rn(v);
    }
}

// C = epilogue(sum over splits, in split order, of the partial products).
__global__ void splitk_reduce_kernel(const float* __restrict__ partial, int splits, long long M, long long N,
                                     long long ld, long long split_stride, void* __restrict__ C, long long ldc,
                                     int out_type, const float* __restrict__ bias, int bias_mode, int relu,
                                     float* __restrict__ planes_hi, float* __restrict__ planes_lo) {
    pdl_wait();
    pdl_launch_dependents();
    const long long total = M * N;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / N, c = i - r * N;
        float v = 0.f;
        for (int s = 0; s < splits; ++s) v += partial[s * split_stride + r * ld + c];
        if (bias_mode == kBiasPerCol) v += bias[c];
        if (bias_mode == kBiasPerRow) v += bias[r];
        if (relu) v = v > 0.f ? v : 0.f;
        if (out_type == kOutF32) static_cast<float*>(C)[r * ldc + c] = v;
        else if (out_type == kOutBF16) static_cast<__nv_bfloat16*>(C)[r * ldc + c] = __float2bfloat16_rn(v);
        else static_cast<__half*>(C)[r * ldc + c] = __float2half_rn(v);
        if (planes_hi != nullptr) {   // leading dimension N
            const float h = tf32_round(v);
            planes_hi[i] = h;
            planes_lo[i] = v - h;
        } else if (planes_lo != nullptr) {   // the consumer reads C itself as the hi plane
            planes_lo[i] = tf32_round(v - tf32_trunc(v));
        }
    }
}

int grid_for(long long work_items, int block, int sm_count) {
    long long g = (work_items + block - 1) / block;
    const long long cap = (long long)sm_count * 16;
    if (g > cap) g = cap;
    if (g < 1) g = 1;
    return (int)g;
}

// ---------------------------------------------------------------------------
// Launch
// ---------------------------------------------------------------------------
// `workers`: CTAs of the persistent grid, or clusters of two when PAIR (one 256-row tile per pair) or KCL
// (one tile per cluster, its contraction shared by the two CTAs).
template <int KIND, int BN, int STAGES, bool A_MN, bool B_MN, bool PAIR, bool KCL = false>
int launch_variant(const CUtensorMap maps[5], const GemmArgs& args, int workers, cudaStream_t stream) {
    using S = GemmSmem<KIND, BN, STAGES, PAIR>;
    static_assert(S::TOTAL <= 232448, "stage ring + staging exceed the 227 KB shared-memory limit");
    auto kern = gemm_tcgen05_kernel<KIND, BN, STAGES, A_MN, B_MN, PAIR, kConvNone, KCL>;
    // Once per (kernel variant, device); several host threads may get here at the same time.
    static std::atomic<bool> attr_set[64];
    int dev = 0;
    TFB_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(TFB_ERR_UNSUPPORTED, "device index %d out of range", dev);
    if (!attr_set[dev].load(std::memory_order_acquire)) {
        TFB_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL));
        attr_set[dev].store(true, std::memory_order_release);
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)((PAIR || KCL) ? 2 * workers : workers));
    cfg.blockDim = dim3((unsigned)gemm_threads(KIND));
    cfg.dynamicSmemBytes = S::TOTAL;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (PAIR || KCL) ? 2 : 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    // The kernel's prologue (barriers, tensor memory, descriptor prefetch) may overlap the tail of the
    // kernel before it; its pdl_wait() precedes every access to global memory.
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = tuning(TFB_TUNE_PDL) != 0 ? 2 : 1;
    TFB_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, maps[0], maps[1], maps[2], maps[3], maps[4], args));
    return TFB_OK;
}

template <int KIND, int BN, int STAGES, bool PAIR, bool KCL = false>
int launch_layout(bool a_mn, bool b_mn, const CUtensorMap maps[5], const GemmArgs& args, int workers,
                  cudaStream_t stream) {
    if (!a_mn && !b_mn) return launch_variant<KIND, BN, STAGES, false, false, PAIR, KCL>(maps, args, workers, stream);
    if (!a_mn && b_mn) return launch_variant<KIND, BN, STAGES, false, true, PAIR, KCL>(maps, args, workers, stream);
    if (a_mn && !b_mn) return launch_variant<KIND, BN, STAGES, true, false, PAIR, KCL>(maps, args, workers, stream);
    return launch_variant<KIND, BN, STAGES, true, true, PAIR, KCL>(maps, args, workers, stream);
}

int choose_bn(int64_t M, int64_t N, int sm_count) {
    const int cands[3] = {256, 128, 64};
    long long best_cost = -1;
    int best = 256;
    const long long tiles_m = (M + kBlockM - 1) / kBlockM;
    for (int bn : cands) {
        const long long tiles = tiles_m * ((N + bn - 1) / bn);
        const long long waves = (tiles + sm_count - 1) / sm_count;
        // Clocks per 32-byte K step: tensor pipe (BN/2) or shared-memory reads ((128+BN)/4).
        const long long step = bn / 2 > (128 + bn) / 4 ? bn / 2 : (128 + bn) / 4;
        const long long cost = waves * step;
        if (best_cost < 0 || cost < best_cost) {
            best_cost = cost;
            best = bn;
        }
    }
    return best;
}

inline int64_t round_up(int64_t x, int64_t m) { return (x + m - 1) / m * m; }

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

int split_operand_on(int sm_count, const float* src, int64_t rows, int64_t cols, int64_t ld, const float* mask,
                     float* hi, float* lo, int64_t ld_out, cudaStream_t stream) {
    if (rows <= 0 || cols <= 0) return TFB_OK;
    const long long items = rows * (ld_out >> 2);
    return launch_pdl(split_tf32_kernel, dim3((unsigned)grid_for(items, 256, sm_count)), dim3(256), 0, stream, src,
                      (long long)rows, (long long)cols, (long long)ld, mask, hi, lo, (long long)ld_out);
}

int split_operand(const float* src, int64_t rows, int64_t cols, int64_t ld, const float* mask,
                  float* hi, float* lo, int64_t ld_out, cudaStream_t stream) {
    DeviceState* st = nullptr;
    int rc = device_state(&st);
    if (rc != TFB_OK) return rc;
    return split_operand_on(st->sm_count, src, rows, cols, ld, mask, hi, lo, ld_out, stream);
}

int split_operands2(const float* src0, int64_t rows0, int64_t cols0, int64_t ld0, float* hi0, float* lo0, int64_t ld_out0,
                    const float* src1, int64_t rows1, int64_t cols1, int64_t ld1, float* hi1, float* lo1, int64_t ld_out1,
                    cudaStream_t stream) {
    DeviceState* st = nullptr;
    int rc = device_state(&st);
    if (rc != TFB_OK) return rc;
    if (rows0 <= 0 || cols0 <= 0) return split_operand_on(st->sm_count, src1, rows1, cols1, ld1, nullptr, hi1, lo1, ld_out1, stream);
    if (rows1 <= 0 || cols1 <= 0) return split_operand_on(st->sm_count, src0, rows0, cols0, ld0, nullptr, hi0, lo0, ld_out0, stream);
    const SplitJob a{src0, rows0, cols0, ld0, nullptr, hi0, lo0, ld_out0}, b{src1, rows1, cols1, ld1, nullptr, hi1, lo1, ld_out1};
    // blocks shared out in proportion to the two sizes
    const int ga = grid_for(rows0 * (ld_out0 >> 2), 256, st->sm_count), gb = grid_for(rows1 * (ld_out1 >> 2), 256, st->sm_count);
    return launch_pdl(split_tf32_pair_kernel, dim3((unsigned)(ga + gb)), dim3(256), 0, stream, a, b, ga);
}

// Diagnostics: device buffer that CTA 0 of every GEMM launch stamps its phase times into (null = off).
std::atomic<unsigned long long*> g_gemm_trace{nullptr};

// Tile shape, CTA pairing and split-K of one call.
struct GemmPlan {
    int bn = 256;
    bool pair = false;
    int split_k = 1;
    int kb_per_split = 0;
    int k_blocks = 0;
    int64_t rows_per_split = 0;   // rows of one split's partial output (whole tiles)
    int64_t ld_partial = 0;       // its leading dimension (multiple of 4)
    size_t partial_bytes = 0;
    // The two halves of every tile's contraction run in the two CTAs of a cluster and are added on chip
    // (KCL kernels): no partial sums in scratch, no reduction kernel.
    bool cluster_k = false;
};

GemmPlan gemm_plan(const GemmCall& c, int sm_count) {
    GemmPlan p;
    // Tuning overrides (tfb_set_tuning): 0 / -1 / 0 leave the choice to the rules below.
    const int env_bn = tuning(TFB_TUNE_GEMM_TILE_N), env_pair = tuning(TFB_TUNE_GEMM_PAIR),
              env_split = tuning(TFB_TUNE_GEMM_SPLIT_K);
    const int es = c.in_dtype == TFB_DTYPE_F32 ? 4 : 2;
    p.k_blocks = (int)((c.K + 128 / es - 1) / (128 / es));
    // CTA pairs pay off once there are enough 256 x 256 tiles to occupy about half of the SM pairs
    // (measured: faster from 2048^3 up, slower at 1024^3).
    const long long pair_tiles = ((c.M + 255) / 256) * ((c.N + 255) / 256);
    p.pair = c.K > 0 && !c.force_bn && !env_bn &&
             (env_pair >= 0 ? env_pair != 0 : pair_tiles >= (sm_count / 4));
    p.bn = p.pair ? 256 : (c.force_bn ? c.force_bn : (env_bn ? env_bn : choose_bn(c.M, c.N, sm_count)));
    p.kb_per_split = p.k_blocks;
    if (!p.pair && c.K > 0) {
        // Few output tiles but a long contraction (weight gradients: M, N ~ 1k, K = batch; every product of
        // a small-batch shard): share each tile's K range between several CTAs; partial sums go to scratch
        // and are added in fixed order.
        struct Split {
            bool ok = false;
            int kb_per_split = 0, split_k = 1;
            int64_t rows_per_split = 0;
        };
        auto split_plan = [&](long long workers, long long tiles, int tile_rows) {
            Split r;
            long long sp = env_split > 0 ? env_split : workers / tiles;
            if (sp > p.k_blocks / 8) sp = p.k_blocks / 8;
            if (sp > 32) sp = 32;
            if (sp < 2 || !(env_split > 0 || tiles * 2 <= workers)) return r;
            r.kb_per_split = (int)((p.k_blocks + sp - 1) / sp);
            r.split_k = (p.k_blocks + r.kb_per_split - 1) / r.kb_per_split;
            r.rows_per_split = (c.M + tile_rows - 1) / tile_rows * tile_rows;
            r.ok = true;
            return r;
        };
        auto apply = [&](const Split& r, bool pair, int bn) {
            p.pair = pair;
            p.bn = bn;
            p.kb_per_split = r.kb_per_split;
            p.split_k = r.split_k;
            p.rows_per_split = r.rows_per_split;
            p.ld_partial = (c.N + 3) / 4 * 4;
            p.partial_bytes = (size_t)p.split_k * p.rows_per_split * p.ld_partial * 4 + 256;
        };
        // Estimated time of a split plan in SM clocks: the MMA time of one unit's K range per wave, plus
        // writing and re-reading `split_k` partial copies of the output at ~18 bytes per clock and SM (5 TB/s).
        // (Measured on a 1024-row MLP shard: single-CTA 128-wide tiles with 2 splits beat CTA pairs with 4
        // by 13 % although the pair feeds the tensor pipe better, because half as many partials move; for
        // the K = 8192 weight gradients the pair wins.)
        auto cost = [&](const Split& r, long long tiles, long long workers, int clk_per_kb) {
            const long long waves = (tiles * r.split_k + workers - 1) / workers;
            const double mma = (double)waves * r.kb_per_split * clk_per_kb;
            const double partials = (double)r.split_k * c.M * c.N * 8.0 / (18.0 * sm_count);
            return mma + partials;
        };
        const bool f32 = c.in_dtype == TFB_DTYPE_F32;
        const bool pair0 = p.pair;
        const int bn0 = p.bn;   // the plan without a split, to fall back to
        const bool pair_ok = !c.force_bn && !env_bn && env_pair != 0 && c.M >= 256 && c.N >= 256;
        int bn1 = p.bn;
        if (!c.force_bn && !env_bn && c.N >= 128) bn1 = c.N >= 256 ? 256 : 128;   // wide tiles feed the MMA better
        const long long tiles1 = ((c.M + kBlockM - 1) / kBlockM) * ((c.N + bn1 - 1) / bn1);
        const Split sp_pair = pair_ok ? split_plan(sm_count / 2, pair_tiles, 2 * kBlockM) : Split();
        const Split sp_one = split_plan(sm_count, tiles1, kBlockM);
        // third candidate: single-CTA tiles of 128 columns, twice as many tiles and half as many splits
        const long long tiles128 = ((c.M + kBlockM - 1) / kBlockM) * ((c.N + 127) / 128);
        const Split sp_128 = (pair_ok && env_pair < 0) ? split_plan(sm_count, tiles128, kBlockM) : Split();
        // two splits of 128 x 128 FP32 tiles with a tile per SM pair at most add their halves on chip (below):
        // no partial traffic, no second launch; every other split pays for the reduction launch (~8000 clocks)
        const bool kcl_128 = f32 && sp_128.ok && sp_128.split_k == 2 && tiles128 * 2 <= sm_count &&
                             tuning(TFB_TUNE_CLUSTER_K) != 0;
        const double cost_128 = !sp_128.ok ? 0.0
                                : kcl_128  ? ((double)sp_128.kb_per_split * 1000.0 + 5000.0) / 0.9   // measured: a tie at K = 4096
                                           : cost(sp_128, tiles128, sm_count, f32 ? 1000 : 340) + 8000.0;
        if (sp_pair.ok && sp_128.ok && cost_128 < cost(sp_pair, pair_tiles, sm_count / 2, f32 ? 1536 : 512) + 8000.0) {
            apply(sp_128, false, 128);
        } else if (sp_pair.ok) {
            // CTA pairs keep the tensor pipe fuller than single CTAs (deeper ring per MMA), so prefer them
            // whenever whole 256 x 256 tiles exist.
            apply(sp_pair, true, 256);
        } else if (sp_one.ok) {
            apply(sp_one, false, bn1);
        }
        // Two splits of FP32 128 x 128 tiles, at most one tile per SM pair: the halves meet on chip.
        const long long tiles_now = ((c.M + kBlockM - 1) / kBlockM) * ((c.N + p.bn - 1) / p.bn);
        if (f32 && !p.pair && p.bn == 128 && p.split_k == 2 && tiles_now * 2 <= sm_count &&
            tuning(TFB_TUNE_CLUSTER_K) != 0) {
            p.cluster_k = true;
            p.partial_bytes = 0;
        }
        // A split that goes through scratch also pays for a second launch (~8000 clocks with its gap): keep
        // the unsplit plan where that is cheaper (measured: a 1024-cubed BF16 product takes 7.5 us unsplit,
        // 12.9 us as two splits + reduction; with a 4096-long contraction on 512 x 512 outputs the split wins
        // 10.9 to 18.9 us).
        if (p.split_k > 1 && !p.cluster_k && env_split <= 0) {
            auto clk_kb = [&](int bn, bool pair) {
                if (f32) return pair ? 1536 : (bn == 256 ? 1800 : (bn == 128 ? 1000 : 700));
                // 16-bit tiles of one CTA are bound by the latency of a K block, not by the tensor pipe
                // (measured: ~500 clocks per K block for 64- and 128-column tiles)
                return pair ? 512 : (bn == 256 ? 600 : 500);
            };
            Split cur;
            cur.split_k = p.split_k;
            cur.kb_per_split = p.kb_per_split;
            const long long workers_now = p.pair ? sm_count / 2 : sm_count;
            const long long tiles_cur = p.pair ? pair_tiles : tiles_now;
            const double split_cost = cost(cur, tiles_cur, workers_now, clk_kb(p.bn, p.pair)) + 8000.0;
            const long long tiles0 = ((c.M + kBlockM - 1) / kBlockM) * ((c.N + bn0 - 1) / bn0);
            const double plain_cost = (double)((tiles0 + sm_count - 1) / sm_count) * p.k_blocks * clk_kb(bn0, false);
            if (plain_cost <= split_cost) {
                p.pair = pair0;
                p.bn = bn0;
                p.split_k = 1;
                p.kb_per_split = p.k_blocks;
                p.rows_per_split = 0;
                p.ld_partial = 0;
                p.partial_bytes = 0;
            }
        }
    }
    return p;
}

bool gemm_uses_cluster_k(const GemmCall& c, int sm_count) {
    return !small_gemm_eligible(c) && gemm_plan(c, sm_count).cluster_k;
}

bool raw_hi_operand(const void* ptr, int64_t ld, const void* mask) {
    return tuning(TFB_TUNE_RAW_HI) != 0 && mask == nullptr && aligned16(ptr) && (ld & 3) == 0;
}

bool gemm_uses_split_k(const GemmCall& c, int sm_count) {
    if (small_gemm_eligible(c)) return false;
    const GemmPlan p = gemm_plan(c, sm_count);
    return p.split_k > 1 && !p.cluster_k;
}

size_t gemm_workspace_bytes(const GemmCall& c, int sm_count) {
    if (small_gemm_eligible(c)) return 0;   // the CUDA-core kernel needs no scratch
    size_t bytes = 0;
    const int64_t a_rows = c.a_kmajor ? c.M : c.K, a_cols = c.a_kmajor ? c.K : c.M;
    const int64_t b_rows = c.b_kmajor ? c.N : c.K, b_cols = c.b_kmajor ? c.K : c.N;
    if (c.in_dtype == TFB_DTYPE_F32) {
        // two planes per operand, or the lo plane alone where the operand itself can serve as the hi plane
        if (!c.a_presplit)
            bytes += (size_t)((raw_hi_operand(c.A, c.lda, c.a_mask) ? 1 : 2) * a_rows * round_up(a_cols, 4) * 4 + 256);
        if (!c.b_presplit)
            bytes += (size_t)((raw_hi_operand(c.B, c.ldb, nullptr) ? 1 : 2) * b_rows * round_up(b_cols, 4) * 4 + 256);
    } else {
        if (!aligned16(c.A) || (c.lda & 7)) bytes += (size_t)(a_rows * round_up(a_cols, 8) * 2 + 256);
        if (!aligned16(c.B) || (c.ldb & 7)) bytes += (size_t)(b_rows * round_up(b_cols, 8) * 2 + 256);
    }
    bytes += gemm_plan(c, sm_count).partial_bytes;
    return bytes;
}

int gemm_run(const GemmCall& c, cudaStream_t stream) {
    if (c.M <= 0 || c.N <= 0) return TFB_OK;
    DeviceState* st = nullptr;
    int rc = device_state(&st);
    if (rc != TFB_OK) return rc;
    return gemm_run_on(c, stream, st);
}

int gemm_run_on(const GemmCall& c, cudaStream_t stream, const DeviceState* st) {
    if (c.M <= 0 || c.N <= 0) return TFB_OK;
    if (c.A == nullptr || c.B == nullptr || c.C == nullptr)
        return fail(TFB_ERR_INVALID_ARG, "gemm: null operand pointer");
    if (c.in_dtype != TFB_DTYPE_F32 && c.in_dtype != TFB_DTYPE_F16 && c.in_dtype != TFB_DTYPE_BF16)
        return fail(TFB_ERR_UNSUPPORTED, "gemm: unsupported input dtype %d", c.in_dtype);
    if (c.out_dtype != TFB_DTYPE_F32 && c.out_dtype != c.in_dtype)
        return fail(TFB_ERR_UNSUPPORTED, "gemm: output dtype %d must be F32 or the input dtype", c.out_dtype);
    if (c.M > INT32_MAX || c.N > INT32_MAX || c.K > INT32_MAX)
        return fail(TFB_ERR_TOO_LARGE, "gemm: extents above 2^31-1 are not supported");
    const int64_t a_rows = c.a_kmajor ? c.M : c.K, a_cols = c.a_kmajor ? c.K : c.M;
    const int64_t b_rows = c.b_kmajor ? c.N : c.K, b_cols = c.b_kmajor ? c.K : c.N;
    if (c.lda < a_cols || c.ldb < b_cols || c.ldc < c.N)
        return fail(TFB_ERR_INVALID_ARG, "gemm: leading dimension smaller than the row length");
    if (c.bias_mode != 0 && c.bias == nullptr)
        return fail(TFB_ERR_INVALID_ARG, "gemm: bias epilogue requested without a bias pointer");

    if (small_gemm_eligible(c)) return small_gemm_run(c, stream);

    int rc = resolve_encoder();
    if (rc != TFB_OK) return rc;

    const bool f32 = c.in_dtype == TFB_DTYPE_F32;
    const int es = f32 ? 4 : 2;

    // ---- operand preparation into scratch -------------------------------------
    const void* a_ptr[2] = {c.A, nullptr};
    const void* b_ptr[2] = {c.B, nullptr};
    int64_t lda[2] = {c.lda, c.lda}, ldb[2] = {c.ldb, c.ldb};   // per plane
    const size_t need = gemm_workspace_bytes(c, st->sm_count);
    uint8_t* ws = nullptr;
    if (need > 0) {
        if (c.workspace != nullptr) {
            if (c.workspace_bytes < need)
                return fail(TFB_ERR_INVALID_ARG, "gemm: caller scratch of %zu bytes is smaller than the %zu needed",
                            c.workspace_bytes, need);
            ws = static_cast<uint8_t*>(c.workspace);
        } else {
            void* p = nullptr;
            rc = workspace_get(stream, need, &p);
            if (rc != TFB_OK) return rc;
            ws = static_cast<uint8_t*>(p);
        }
    }
    auto carve = [&](size_t bytes) {
        uint8_t* p = ws;
        ws += (bytes + 255) & ~(size_t)255;
        return p;
    };
    if (c.K > 0) {
        if (f32) {
            SplitJob jobs[2];
            int njobs = 0;
            if (c.a_presplit) {
                a_ptr[1] = static_cast<const float*>(c.A) + c.a_lo_off;
            } else {
                const int64_t ldp = round_up(a_cols, 4);
                if (raw_hi_operand(c.A, c.lda, c.a_mask)) {
                    float* lo = reinterpret_cast<float*>(carve((size_t)(a_rows * ldp * 4)));
                    jobs[njobs++] = SplitJob{static_cast<const float*>(c.A), a_rows, a_cols, c.lda, nullptr, nullptr, lo, ldp};
                    a_ptr[1] = lo; lda[1] = ldp;
                } else {
                    float* hi = reinterpret_cast<float*>(carve((size_t)(2 * a_rows * ldp * 4)));
                    float* lo = hi + a_rows * ldp;
                    jobs[njobs++] = SplitJob{static_cast<const float*>(c.A), a_rows, a_cols, c.lda, c.a_mask, hi, lo, ldp};
                    a_ptr[0] = hi; a_ptr[1] = lo; lda[0] = lda[1] = ldp;
                }
            }
            if (c.b_presplit) {
                b_ptr[1] = static_cast<const float*>(c.B) + c.b_lo_off;
            } else {
                const int64_t ldp = round_up(b_cols, 4);
                if (raw_hi_operand(c.B, c.ldb, nullptr)) {
                    float* lo = reinterpret_cast<float*>(carve((size_t)(b_rows * ldp * 4)));
                    jobs[njobs++] = SplitJob{static_cast<const float*>(c.B), b_rows, b_cols, c.ldb, nullptr, nullptr, lo, ldp};
                    b_ptr[1] = lo; ldb[1] = ldp;
                } else {
                    float* hi = reinterpret_cast<float*>(carve((size_t)(2 * b_rows * ldp * 4)));
                    float* lo = hi + b_rows * ldp;
                    jobs[njobs++] = SplitJob{static_cast<const float*>(c.B), b_rows, b_cols, c.ldb, nullptr, hi, lo, ldp};
                    b_ptr[0] = hi; b_ptr[1] = lo; ldb[0] = ldb[1] = ldp;
                }
            }
            if (njobs == 1) {
                rc = split_operand_on(st->sm_count, jobs[0].src, jobs[0].rows, jobs[0].cols, jobs[0].ld, jobs[0].mask,
                                      jobs[0].hi, jobs[0].lo, jobs[0].ld_out, stream);
                if (rc != TFB_OK) return rc;
            } else if (njobs == 2) {
                // one launch for both operands, blocks shared out in proportion to their sizes
                const long long ia = jobs[0].rows * (jobs[0].ld_out >> 2), ib = jobs[1].rows * (jobs[1].ld_out >> 2);
                const int ga = grid_for(ia, 256, st->sm_count), gb = grid_for(ib, 256, st->sm_count);
                rc = launch_pdl(split_tf32_pair_kernel, dim3((unsigned)(ga + gb)), dim3(256), 0, stream, jobs[0], jobs[1], ga);
                if (rc != TFB_OK) return rc;
            }
        } else {
            if (c.a_mask != nullptr)
                return fail(TFB_ERR_UNSUPPORTED, "gemm: operand mask is only available for F32 inputs");
            if (!aligned16(c.A) || (c.lda & 7)) {
                const int64_t ldp = round_up(a_cols, 8);
                uint16_t* d = reinterpret_cast<uint16_t*>(carve((size_t)(a_rows * ldp * 2)));
                rc = launch_pdl(pack16_kernel, dim3((unsigned)grid_for(a_rows * ldp, 256, st->sm_count)), dim3(256), 0, stream,
                                static_cast<const uint16_t*>(c.A), (long long)a_rows, (long long)a_cols, (long long)c.lda, d,
                                (long long)ldp);
                if (rc != TFB_OK) return rc;
                a_ptr[0] = d; lda[0] = ldp;
            }
            if (!aligned16(c.B) || (c.ldb & 7)) {
                const int64_t ldp = round_up(b_cols, 8);
                uint16_t* d = reinterpret_cast<uint16_t*>(carve((size_t)(b_rows * ldp * 2)));
                rc = launch_pdl(pack16_kernel, dim3((unsigned)grid_for(b_rows * ldp, 256, st->sm_count)), dim3(256), 0, stream,
                                static_cast<const uint16_t*>(c.B), (long long)b_rows, (long long)b_cols, (long long)c.ldb, d,
                                (long long)ldp);
                if (rc != TFB_OK) return rc;
                b_ptr[0] = d; ldb[0] = ldp;
            }
        }
    }

    // ---- tile shape and tensor maps ---------------------------------------------
    const int env_chunk = tuning(TFB_TUNE_GEMM_CHUNK_KB);
    const GemmPlan plan = gemm_plan(c, st->sm_count);
    const bool use_pair = plan.pair;
    const int bn = plan.bn;
    if (bn != 64 && bn != 128 && bn != 256) return fail(TFB_ERR_INVALID_ARG, "gemm: tile N %d", bn);
    const int bk = 128 / es;
    const int t_mn = 128 / es;

    GemmArgs args;
    memset(&args, 0, sizeof(args));
    args.M = (int)c.M; args.N = (int)c.N; args.K = (int)c.K;
    args.tiles_m = use_pair ? (int)((c.M + 2 * kBlockM - 1) / (2 * kBlockM)) : (int)((c.M + kBlockM - 1) / kBlockM);
    args.tiles_n = (int)((c.N + bn - 1) / bn);
    args.num_tiles = args.tiles_m * args.tiles_n;
    args.k_blocks = (int)((c.K + bk - 1) / bk);
    args.group_m = 16;
    // FP32: close the TMEM accumulator every 256 K elements (see gemm_kernel.cuh).
    args.split_k = plan.split_k;
    args.kb_per_split = plan.kb_per_split;
    args.chunk_kb = f32 ? (c.chunk_kb > 0 ? c.chunk_kb : (env_chunk > 0 ? env_chunk : 8)) : plan.kb_per_split;
    if (args.chunk_kb < 1) args.chunk_kb = 1;
    args.C = c.C; args.ldc = c.ldc;
    args.out_type = c.out_dtype == TFB_DTYPE_F32 ? kOutF32 : (c.out_dtype == TFB_DTYPE_F16 ? kOutF16 : kOutBF16);
    args.bias = c.bias; args.bias_mode = c.bias_mode; args.relu = c.relu ? 1 : 0;
    args.is_bf16 = c.in_dtype == TFB_DTYPE_BF16 ? 1 : 0;
    args.status = st->status;
    args.trace = g_gemm_trace.load(std::memory_order_relaxed);
    if (c.planes_hi != nullptr || c.planes_lo != nullptr) {
        // planes_hi may be null: the consumer then reads C itself as the hi plane and only lo is written
        if (!f32 || c.out_dtype != TFB_DTYPE_F32 || (c.N & 3) || c.planes_lo == nullptr ||
            !aligned16(c.planes_hi) || !aligned16(c.planes_lo) || c.K <= 0)
            return fail(TFB_ERR_UNSUPPORTED, "gemm: result planes need FP32 in and out, N a multiple of 4 and aligned planes");
        args.planes_hi = c.planes_hi;
        args.planes_lo = c.planes_lo;
        args.ld_planes = c.N;
    }

    if (c.K <= 0) {
        // Empty contraction: the product is zero and only the epilogue remains.
        const long long total = (long long)c.M * c.N;
        return launch_pdl(empty_k_kernel, dim3((unsigned)grid_for(total, 256, st->sm_count)), dim3(256), 0, stream, args);
    }

    CUtensorMap maps[5];
    memset(maps, 0, sizeof(maps));
    const int nplanes = f32 ? 2 : 1;
    for (int p = 0; p < nplanes; ++p) {
        if (c.a_kmajor)
            rc = make_map(&maps[p], c.in_dtype, a_ptr[p], (uint64_t)c.K, (uint64_t)c.M, (uint64_t)lda[p] * es, bk, kBlockM);
        else
            rc = make_map(&maps[p], c.in_dtype, a_ptr[p], (uint64_t)c.M, (uint64_t)c.K, (uint64_t)lda[p] * es, t_mn, bk, f32);
        if (rc != TFB_OK) return rc;
        if (c.b_kmajor)
            rc = make_map(&maps[2 + p], c.in_dtype, b_ptr[p], (uint64_t)c.K, (uint64_t)c.N, (uint64_t)ldb[p] * es, bk,
                          use_pair ? bn / 2 : bn);
        else
            rc = make_map(&maps[2 + p], c.in_dtype, b_ptr[p], (uint64_t)c.N, (uint64_t)c.K, (uint64_t)ldb[p] * es, t_mn, bk, f32);
        if (rc != TFB_OK) return rc;
    }
    if (!f32) { maps[1] = maps[0]; maps[3] = maps[2]; }
    // FP32 output with 16-byte aligned rows leaves through TMA stores of 32 x 32 blocks.
    float* partial = nullptr;
    if (plan.split_k > 1 && !plan.cluster_k) {
        // Units write raw FP32 partial sums; the epilogue proper runs in the reduction kernel.
        partial = reinterpret_cast<float*>(carve(plan.partial_bytes));
        args.C = partial;
        args.ldc = plan.ld_partial;
        args.split_stride = plan.rows_per_split * plan.ld_partial;
        args.out_type = kOutF32;
        args.bias = nullptr; args.bias_mode = 0; args.relu = 0;
        args.planes_hi = nullptr; args.planes_lo = nullptr;   // the reduction kernel writes them
        args.c_tma = 1;
        rc = make_map(&maps[4], TFB_DTYPE_F32, partial, (uint64_t)c.N, (uint64_t)(plan.split_k * plan.rows_per_split),
                      (uint64_t)plan.ld_partial * 4, 32, 32);
        if (rc != TFB_OK) return rc;
    } else {
        args.split_stride = 0;
        args.c_tma = (c.out_dtype == TFB_DTYPE_F32 && aligned16(c.C) && (c.ldc & 3) == 0) ? 1 : 0;
        if (args.planes_lo != nullptr && !args.c_tma)
            return fail(TFB_ERR_UNSUPPORTED, "gemm: result planes need a 16-byte aligned output with ldc a multiple of 4");
        if (args.c_tma) {
            rc = make_map(&maps[4], TFB_DTYPE_F32, c.C, (uint64_t)c.N, (uint64_t)c.M, (uint64_t)c.ldc * 4, 32, 32);
            if (rc != TFB_OK) return rc;
        } else {
            maps[4] = maps[0];
        }
    }

    const long long units = (long long)args.num_tiles * args.split_k;
    const int grid = units < st->sm_count ? (int)units : st->sm_count;
    const bool a_mn = !c.a_kmajor, b_mn = !c.b_kmajor;
    if (use_pair) {
        args.group_m = 8;   // 8 pair tiles = 2048 rows, the same raster width as the single-CTA kernel
        if (tuning(TFB_TUNE_GEMM_GROUP_M) > 0) args.group_m = tuning(TFB_TUNE_GEMM_GROUP_M);
        const int max_pairs = st->sm_count / 2;
        const int pairs = units < max_pairs ? (int)units : max_pairs;
        if (f32) rc = launch_layout<kKindTF32x3, 256, 3, true>(a_mn, b_mn, maps, args, pairs, stream);
        else rc = launch_layout<kKind16, 256, 6, true>(a_mn, b_mn, maps, args, pairs, stream);
    } else if (plan.cluster_k) {
        args.cluster_k = 1;
        rc = launch_layout<kKindTF32x3, 128, 3, false, true>(a_mn, b_mn, maps, args, args.num_tiles, stream);
    } else if (f32) {
        if (bn == 256) rc = launch_layout<kKindTF32x3, 256, 2, false>(a_mn, b_mn, maps, args, grid, stream);
        else if (bn == 128) rc = launch_layout<kKindTF32x3, 128, 3, false>(a_mn, b_mn, maps, args, grid, stream);
        else rc = launch_layout<kKindTF32x3, 64, 4, false>(a_mn, b_mn, maps, args, grid, stream);
    } else {
        if (bn == 256) rc = launch_layout<kKind16, 256, 4, false>(a_mn, b_mn, maps, args, grid, stream);
        else if (bn == 128) rc = launch_layout<kKind16, 128, 6, false>(a_mn, b_mn, maps, args, grid, stream);
        else rc = launch_layout<kKind16, 64, 8, false>(a_mn, b_mn, maps, args, grid, stream);
    }
    if (rc != TFB_OK || plan.split_k == 1 || plan.cluster_k) return rc;
    const long long total = (long long)c.M * c.N;
    return launch_pdl(splitk_reduce_kernel, dim3((unsigned)grid_for(total, 256, st->sm_count)), dim3(256), 0, stream,
                      (const float*)partial, plan.split_k, (long long)c.M, (long long)c.N, (long long)plan.ld_partial,
                      (long long)(plan.rows_per_split * plan.ld_partial), c.C, (long long)c.ldc,
                      (int)(c.out_dtype == TFB_DTYPE_F32 ? kOutF32 : (c.out_dtype == TFB_DTYPE_F16 ? kOutF16 : kOutBF16)),
                      c.bias, c.bias_mode, c.relu ? 1 : 0, c.planes_hi, c.planes_lo);
}

}  // namespace tfb

extern "C" int tfb_gemm_describe_plan(int64_t M, int64_t N, int64_t K, int dtype, int sm_count, int* plan_out) {
    using namespace tfb;
    if (plan_out == nullptr || M <= 0 || N <= 0 || K < 0 || sm_count < 2)
        return fail(TFB_ERR_INVALID_ARG, "gemm_describe_plan: bad extent, SM count or output pointer");
    if (dtype != TFB_DTYPE_F32 && dtype != TFB_DTYPE_F16 && dtype != TFB_DTYPE_BF16)
        return fail(TFB_ERR_UNSUPPORTED, "gemm_describe_plan: unsupported dtype %d", dtype);
    GemmCall c;
    c.M = M; c.N = N; c.K = K;
    c.lda = K; c.ldb = N; c.ldc = N;
    c.in_dtype = dtype; c.out_dtype = TFB_DTYPE_F32;
    if (small_gemm_eligible(c)) {
        plan_out[0] = plan_out[1] = plan_out[2] = plan_out[3] = 0;
        plan_out[4] = 1;
        return TFB_OK;
    }
    const GemmPlan p = gemm_plan(c, sm_count);
    plan_out[0] = p.bn;
    plan_out[1] = p.pair ? 1 : 0;
    plan_out[2] = p.split_k;
    plan_out[3] = p.cluster_k ? 1 : 0;
    plan_out[4] = 0;
    return TFB_OK;
}

extern "C" int tfb_gemm_trace(void* device_stamps) {
    tfb::g_gemm_trace.store(static_cast<unsigned long long*>(device_stamps), std::memory_order_relaxed);
    return TFB_OK;
}
