// Persistent, warp-specialised tcgen05 GEMM for sm_100a.
//
//   D[M,N] (+bias, ReLU) = A · B      with FP32 accumulation in tensor memory.
//
// Roles inside one CTA (192 threads; 320 on the FP32 path):
//   warp 0      TMA producer: fills a ring of shared-memory stages with 128-byte-swizzled
//               operand tiles and signals `full[s]` by transaction bytes.
//   warp 1      MMA issuer: one lane issues tcgen05.mma per 32-byte K step, releases a
//               stage with tcgen05.commit -> `empty[s]`, and hands a finished accumulator
//               to the epilogue with tcgen05.commit -> `tmem_full[b]`.  Also owns the
//               TMEM allocation.
//   warps 2+    epilogue: tcgen05.ld the accumulator (each warp its own 32 TMEM lanes),
//               apply bias / ReLU, convert and store, then release the accumulator with
//               `tmem_empty[b]`.  Two accumulators let the epilogue of tile i overlap the
//               main loop of tile i+1.  FP32 output leaves through a swizzled staging
//               buffer and a TMA store per 32x32 block (whole 128-byte lines, clipped at
//               the matrix edge by the tensor map); other cases store from registers.
//
// Operand layouts.  "K-major": the contraction index is contiguous in memory (A[M,K]
// row-major, B given as [N,K] row-major).  "MN-major": the M (resp. N) index is
// contiguous (A given as [K,M] row-major, B as [K,N] row-major).  Both are fed to the
// tensor core straight from the TMA tiles through the matching shared-memory
// descriptor, so transposed products need no transpose copy.
//
// kKindTF32x3: every FP32 operand arrives pre-split as hi + lo (hi = x rounded to TF32,
// lo = x - hi).  Each K step issues lo·hi, hi·lo and hi·hi into the same FP32
// accumulator, which restores FP32-level accuracy from TF32 tensor-core products.
// The tensor core adds into its accumulator with truncation, an error that grows linearly
// with the number of accumulating instructions; the FP32 path therefore closes the TMEM
// accumulator every `chunk_kb` K blocks and the (eight) epilogue warps sum those chunk
// results in registers with round-to-nearest adds, which keeps the result within FP32
// rounding noise of a sequential FP32 dot product for any K.
//
// PAIR = true: two CTAs of a cluster — a CTA pair on two SMs — compute one 256 x BN tile
// with tcgen05.mma.cta_group::2.  Each CTA stages its own 128 rows of A and only HALF of
// the B tile (BN/2 rows); the tensor cores of both SMs read both halves, and each CTA's
// TMEM receives the accumulator of its own 128 rows.  Per FLOP this halves the B bytes
// that travel L2 -> shared memory.  Rank 0 of the pair is the leader; only its MMA lane
// issues.
//   full[s]       lives in the leader, which announces the bytes of both CTAs (one
//                 arrive.expect_tx); both CTAs' TMA loads signal the leader's barrier.
//                 (A per-stage remote arrive with cluster-scope release from the peer's
//                 producer halved BF16 throughput and was dropped.)
//   empty[s]      one copy per CTA; the leader's commit arrives on both copies.
//   tmem_full[b]  one copy per CTA; the leader's commit arrives on both.
//   tmem_empty[b] lives in the leader; the epilogue threads of both CTAs arrive remotely.
// Cluster barriers bracket the kernel so that no CTA touches its peer's barriers before
// they are initialised or leaves while its peer may still read its shared memory.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "ptx.cuh"

namespace tfb {

// kKind16: f16 or bf16 operands (which one is a run-time flag); kKindTF32x3: split FP32.
enum GemmKind : int { kKind16 = 0, kKindTF32x3 = 2 };
enum OutType : int { kOutF32 = 0, kOutF16 = 1, kOutBF16 = 2 };
enum BiasMode : int { kBiasNone = 0, kBiasPerCol = 1, kBiasPerRow = 2 };

// Convolution feeds of the same kernel (CONV template parameter). Both tensors of a convolution are
// read as NHWC hi / lo planes through 4-D tensor maps (channel, x, y, sample), so a box of positions
// shifted by a filter tap is one TMA load and the padding halo is the load's out-of-range zero fill.
//   kConvSpatial (forward, input gradient; stride 1): rows = a th x tw rectangle of output positions
//     of one sample, columns = output channels, K blocks = (tap, 32 input channels). A from the
//     activation planes, B from weights laid out [column][tap][channel]; the result is stored NCHW.
//   kConvWgrad (weight gradient; stride 1): rows = output channels, columns = (tap, input channel),
//     K blocks = 32 positions (kblk_h x kblk_w) of one sample; both operands MN-major boxes.
enum ConvFeed : int { kConvNone = 0, kConvSpatial = 1, kConvWgrad = 2 };
struct ConvGeom {
    int tw_log2, th;                  // spatial tile: th rows of 2^tw_log2 positions (128 per CTA)
    int tiles_x, tiles_y;             // scheduled tiles per sample along x and y
    int out_h, out_w;                 // extent of the position grid (= of the stored tensor)
    int cblks;                        // 32-channel blocks per tap
    int kw, taps;                     // filter width, number of taps (tap = ki * kw + kj)
    int ay0, ay_step, ax0, ax_step;   // source row = position row * sy + ay0 + ki * ay_step (x alike)
    int sx, sy;                       // convolution stride (the source maps traverse with the same stride)
    int kblk_w_log2, kblk_h;          // kConvWgrad: K block = kblk_h rows of 2^kblk_w_log2 positions
    int kblk_x, kblk_y;               // K blocks per sample along x and y
    int n_samples;
};

struct GemmArgs {
    int M, N, K;
    int tiles_m, tiles_n, num_tiles, k_blocks;
    int chunk_kb;         // K blocks accumulated in TMEM before the epilogue drains them
    int cluster_k;        // KCL kernels: 1 (documentation of the mode; the kernel variant decides)
    int split_k;          // work units per output tile; unit u = split * num_tiles + tile
    int kb_per_split;     // K blocks per unit (the last split may hold fewer)
    long long split_stride;   // elements between the partial outputs of consecutive splits
    int group_m;          // M-tiles per rasterisation group (L2 reuse of B tiles)
    void* C;
    long long ldc;        // elements
    int out_type;         // OutType
    const float* bias;
    int bias_mode;        // BiasMode
    int relu;
    int is_bf16;          // kKind16 only: 1 = bf16 operands, 0 = f16
    int c_tma;            // 1: FP32 output goes through the TMA-store path (tmC is valid)
    int* status;          // device error word (0 = ok)
    // Optional second output of the FP32 path: the TF32 hi / lo planes of the final values (after bias and
    // ReLU), row-major with leading dimension ld_planes, for a consumer that multiplies them next.
    float* planes_hi;
    float* planes_lo;
    long long ld_planes;
    // Optional diagnostics: CTA 0 records %globaltimer at its phase boundaries (tfb_gemm_trace):
    // [0] entry, [1] prologue done (barriers, tensor memory, cluster sync, dependency wait), [2] first
    // operand stage landed, [3] last MMA of the CTA's last unit committed, [4] its accumulator seen by the
    // epilogue, [5] epilogue stores issued and drained, [6] exit.
    unsigned long long* trace;
    ConvGeom cv;          // only read when CONV != kConvNone
};

constexpr int kBlockM = 128;
// Two control warps (TMA, MMA) plus four epilogue warps, eight on the FP32 path.
__host__ __device__ constexpr int gemm_threads(int kind) { return kind == kKindTF32x3 ? 320 : 192; }
__host__ __device__ constexpr int gemm_epi_warps(int kind) { return kind == kKindTF32x3 ? 8 : 4; }

template <int KIND, int BN, int STAGES, bool PAIR>
struct GemmSmem {
    static constexpr int ES = (KIND == kKindTF32x3) ? 4 : 2;   // operand element bytes
    static constexpr int NSPLIT = (KIND == kKindTF32x3) ? 2 : 1;
    static constexpr int BK = 128 / ES;                         // K elements per stage
    static constexpr int BN_CTA = PAIR ? BN / 2 : BN;           // B rows staged by one CTA
    static constexpr int A_TILE = kBlockM * 128;                // bytes
    static constexpr int B_TILE = BN_CTA * 128;
    static constexpr int STAGE_BYTES = NSPLIT * (A_TILE + B_TILE);
    // Epilogue staging: 32 rows x 128 B per buffer; two buffers per warp with four epilogue
    // warps, one with eight, 32 KB either way.
    static constexpr int STAGING_BUFS = (KIND == kKindTF32x3) ? 1 : 2;
    static constexpr int STAGING_BYTES = gemm_epi_warps(KIND) * STAGING_BUFS * 4096;
    static constexpr int BAR_BYTES = 256;
    static constexpr int TOTAL = 1024 + STAGES * STAGE_BYTES + STAGING_BYTES + BAR_BYTES;
};

// Bias and ReLU on 32 consecutive output columns of one row.
__device__ __forceinline__ void epilogue_apply32(float (&v)[32], const GemmArgs& args, int col0, float row_bias) {
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] += row_bias;
    if (args.bias_mode == kBiasPerCol) {
#pragma unroll
        for (int i = 0; i < 32; ++i)
            if (col0 + i < args.N) v[i] += __ldg(args.bias + col0 + i);
    }
    if (args.relu) {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = v[i] > 0.f ? v[i] : 0.f;
    }
}

// Conversion and store of 32 consecutive output columns of one row straight from registers.
__device__ __forceinline__ void epilogue_store32(const float (&v)[32], const GemmArgs& args, int row, int col0) {
    const bool full = (col0 + 32 <= args.N);
    if (args.out_type == kOutF32) {
        float* dst = static_cast<float*>(args.C) + (long long)row * args.ldc + col0;
        if (full && ((reinterpret_cast<uintptr_t>(dst) & 15u) == 0)) {
#pragma unroll
            for (int i = 0; i < 8; ++i)
                reinterpret_cast<float4*>(dst)[i] =
                    make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
        } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
                if (col0 + i < args.N) dst[i] = v[i];
        }
    } else {
        uint16_t h[32];
        if (args.out_type == kOutBF16) {
#pragma unroll
            for (int i = 0; i < 32; ++i) h[i] = __bfloat16_as_ushort(__float2bfloat16_rn(v[i]));
        } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) h[i] = __half_as_ushort(__float2half_rn(v[i]));
        }
        uint16_t* dst = static_cast<uint16_t*>(args.C) + (long long)row * args.ldc + col0;
        if (full && ((reinterpret_cast<uintptr_t>(dst) & 15u) == 0)) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                uint4 pk;
                pk.x = h[8 * i] | ((uint32_t)h[8 * i + 1] << 16);
                pk.y = h[8 * i + 2] | ((uint32_t)h[8 * i + 3] << 16);
                pk.z = h[8 * i + 4] | ((uint32_t)h[8 * i + 5] << 16);
                pk.w = h[8 * i + 6] | ((uint32_t)h[8 * i + 7] << 16);
                reinterpret_cast<uint4*>(dst)[i] = pk;
            }
        } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
                if (col0 + i < args.N) dst[i] = h[i];
        }
    }
}

// One warp's 32 rows x 32 FP32 columns through shared memory: lane r writes its row into a
// 128-byte-swizzled 4 KB buffer (16-byte chunk j of row r at chunk j ^ (r & 7): conflict-free),
// then one lane hands the block to the TMA store engine. Rows and columns beyond the matrix are
// clipped by the tensor map. Lane 0 owns the bulk groups, so it also does the waiting.
template <int NBUF>
__device__ __forceinline__ void epilogue_store32_tma(const float (&v)[32], const CUtensorMap* tmC, uint8_t* staging,
                                                     int& buf_idx, int lane, int row0, int col0) {
    uint8_t* buf = staging + buf_idx * 4096;
    // The buffer about to be overwritten must have been read by its previous store.
    if (lane == 0) tma_store_wait_read<NBUF - 1>();
    __syncwarp();
#pragma unroll
    for (int j = 0; j < 8; ++j)
        *reinterpret_cast<float4*>(buf + lane * 128 + ((j ^ (lane & 7)) << 4)) =
            make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
        tma_store_2d(tmC, smem_u32(buf), col0, row0);
        tma_store_commit();
    }
    buf_idx = (buf_idx + 1 == NBUF) ? 0 : buf_idx + 1;
}

__device__ __forceinline__ float tf32_hi(float x) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return __uint_as_float(r);
}
// what kind::tf32 makes of a raw FP32 operand: the low 13 mantissa bits dropped
__device__ __forceinline__ float tf32_cut(float x) { return __uint_as_float(__float_as_uint(x) & 0xFFFFE000u); }

// One warp's 32 rows x 32 columns (lane = row, v = its 32 values) to a row-major FP32 matrix with whole
// 128-byte lines per store instruction: the block is transposed through the warp's swizzled staging
// buffer (16-byte chunk j of row r at chunk j ^ (r & 7): conflict-free both ways), then lane
// (r & 3, chunk) stores 16 bytes of row 4k + (lane >> 3). PLANE selects what is stored: 1 = the value
// rounded to TF32 (hi), 2 = the value minus that (lo), 3 = the value minus its truncation to TF32, rounded
// (the lo plane that goes with the value itself as hi) — computed on the way into the buffer, so no
// second register array is needed. `m_rows` / `n_cols` clip at the matrix edge (n_cols is a multiple
// of 4). The caller makes sure nothing else is still reading the buffer.
template <int PLANE>
__device__ __forceinline__ void store32x32_via_staging(const float (&v)[32], uint8_t* buf, int lane, float* dst,
                                                        long long ld, int row0, int col0, int m_rows, int n_cols) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        float4 x = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
        if (PLANE == 3) {
            x = make_float4(tf32_hi(x.x - tf32_cut(x.x)), tf32_hi(x.y - tf32_cut(x.y)), tf32_hi(x.z - tf32_cut(x.z)),
                            tf32_hi(x.w - tf32_cut(x.w)));
        } else {
            const float4 h = make_float4(tf32_hi(x.x), tf32_hi(x.y), tf32_hi(x.z), tf32_hi(x.w));
            if (PLANE == 1) x = h;
            else x = make_float4(x.x - h.x, x.y - h.y, x.z - h.z, x.w - h.w);
        }
        *reinterpret_cast<float4*>(buf + lane * 128 + ((j ^ (lane & 7)) << 4)) = x;
    }
    __syncwarp();
    const int chunk = lane & 7;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const int r = 4 * k + (lane >> 3);
        const float4 x = *reinterpret_cast<const float4*>(buf + r * 128 + ((chunk ^ (r & 7)) << 4));
        if (row0 + r < m_rows && col0 + 4 * chunk < n_cols)
            *reinterpret_cast<float4*>(dst + (long long)(row0 + r) * ld + col0 + 4 * chunk) = x;
    }
    __syncwarp();
}

// The TF32 hi / lo planes of a 32 x 32 block of final values: hi = v rounded to TF32, lo = v - hi.
__device__ __forceinline__ void epilogue_store_planes32(const float (&v)[32], const GemmArgs& args, uint8_t* staging,
                                                         int lane, int row0, int col0) {
    // the warp's previous TMA store may still be reading the staging buffer
    if (lane == 0) tma_store_wait_read<0>();
    __syncwarp();
    if (args.planes_hi != nullptr) {
        store32x32_via_staging<1>(v, staging, lane, args.planes_hi, args.ld_planes, row0, col0, args.M, args.N);
        store32x32_via_staging<2>(v, staging, lane, args.planes_lo, args.ld_planes, row0, col0, args.M, args.N);
    } else {
        store32x32_via_staging<3>(v, staging, lane, args.planes_lo, args.ld_planes, row0, col0, args.M, args.N);
    }
}

__device__ __forceinline__ void tile_coords(int t, const GemmArgs& a, int& tm, int& tn) {
    const int group_sz = a.group_m * a.tiles_n;
    const int g = t / group_sz;
    const int first_m = g * a.group_m;
    const int gm = min(a.tiles_m - first_m, a.group_m);
    const int r = t - g * group_sz;
    tm = first_m + r % gm;
    tn = r / gm;
}

// Work unit -> (tile, K-block range). With split_k == 1 a unit is a whole tile.
__device__ __forceinline__ void unit_decode(int u, const GemmArgs& a, int& tile, int& split, int& kb0, int& kb1) {
    split = u / a.num_tiles;
    tile = u - split * a.num_tiles;
    kb0 = split * a.kb_per_split;
    kb1 = min(kb0 + a.kb_per_split, a.k_blocks);
}

// One commit whose arrival is delivered to the barrier at the same shared-memory offset in every
// CTA of `cta_mask` (both CTAs of a pair). A commit is not a copy: no data moves.
__device__ __forceinline__ void umma_commit_pair_both(uint32_t bar, uint16_t cta_mask) {
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
        ::"r"(bar), "h"(cta_mask) : "memory");
}

// KCL ("K split over a cluster"): the two CTAs of a cluster each accumulate half of ONE output tile's
// contraction (split_k = 2, at most one tile per cluster: no tile loop) and then exchange halves of their
// partial tiles through distributed shared memory: CTA k finishes columns [k * BN / 2, (k + 1) * BN / 2) —
// the epilogue warps that hold the other half send it into the peer's epilogue staging buffers (idle until
// the stores begin), the warps that hold its own half add what the peer sent (a sum of two terms: the same
// bits as the split-K reduction kernel's) and run the epilogue. No partial sums in global memory, no
// second kernel, and both CTAs store. FP32 path, single-CTA MMAs.
template <int KIND, int BN, int STAGES, bool A_MN, bool B_MN, bool PAIR, int CONV = kConvNone, bool KCL = false>
__global__ void __launch_bounds__(gemm_threads(KIND), 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmA2,
                    const __grid_constant__ CUtensorMap tmB, const __grid_constant__ CUtensorMap tmB2,
                    const __grid_constant__ CUtensorMap tmC, const GemmArgs args) {
    using S = GemmSmem<KIND, BN, STAGES, PAIR>;
    constexpr int ES = S::ES;
    constexpr int BK = S::BK;
    constexpr int BN_CTA = S::BN_CTA;
    constexpr int CG = PAIR ? 2 : 1;
    constexpr int TILE_M = PAIR ? 2 * kBlockM : kBlockM;   // rows of one scheduled tile
    constexpr bool TF32 = (KIND == kKindTF32x3);
    constexpr int UMMA_K = 32 / ES;          // K elements per tcgen05.mma
    constexpr int KSTEPS = BK / UMMA_K;      // 4
    constexpr int T_MN = 128 / ES;           // M/N elements per 128-byte swizzle row
    constexpr uint32_t TMEM_COLS = (2 * BN <= 32) ? 32 : (2 * BN <= 64) ? 64 : (2 * BN <= 128) ? 128
                                   : (2 * BN <= 256) ? 256 : 512;
    static_assert(BN % 32 == 0 && BN >= 32 && BN <= 256, "BN must be a multiple of 32 up to 256");
    static_assert(!A_MN || (kBlockM % T_MN == 0), "tile M must hold whole swizzle rows");
    static_assert(!B_MN || (BN_CTA % T_MN == 0), "tile N must hold whole swizzle rows");
    constexpr int EPI_WARPS = gemm_epi_warps(KIND);
    constexpr int COLS = BN / (EPI_WARPS / 4);   // accumulator columns handled per epilogue thread
    static_assert(COLS % 32 == 0, "each epilogue thread handles whole 32-column groups");
    static_assert(CONV == kConvNone || TF32, "the convolution feeds exist for FP32 operands only");
    static_assert(CONV != kConvSpatial || (!A_MN && !B_MN), "spatial feed: both operands K-major");
    static_assert(CONV != kConvWgrad || (A_MN && B_MN), "weight-gradient feed: both operands MN-major");
    static_assert(!KCL || (TF32 && !PAIR && CONV == kConvNone), "cluster split-K: FP32 path, single-CTA MMAs");
    static_assert(!KCL || (EPI_WARPS == 8 && COLS * 32 * 4 == 2 * S::STAGING_BUFS * 4096),
                  "cluster split-K: a warp's 32 x COLS partial block must fill two staging buffers");

    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

    uint8_t* staging_all = smem_gen + STAGES * S::STAGE_BYTES;
    const uint32_t bars = smem_base + STAGES * S::STAGE_BYTES + S::STAGING_BYTES;
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
    auto tfull_bar = [&](int b) { return bars + 8u * (2 * STAGES + b); };
    auto tempty_bar = [&](int b) { return bars + 8u * (2 * STAGES + 2 + b); };
    uint8_t* after_bars = smem_gen + STAGES * S::STAGE_BYTES + S::STAGING_BYTES + 8 * (2 * STAGES + 4);
    volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(after_bars);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(after_bars + 4);
    // KCL: the peer's half of my columns has landed in my staging buffers
    const uint32_t xdata_bar = bars + 8u * (2 * STAGES + 4) + 8u;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const bool tracing = args.trace != nullptr && blockIdx.x == 0;
    if (tracing && threadIdx.x == 0) args.trace[0] = global_timer_ns();
    const uint32_t rank = PAIR ? cluster_ctarank() : 0u;   // 0 = leader of the pair
    const uint32_t krank = KCL ? cluster_ctarank() : 0u;   // which half of the contraction (KCL)
    const int worker = (PAIR || KCL) ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
    const int num_workers = (PAIR || KCL) ? (int)(gridDim.x >> 1) : (int)gridDim.x;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(tfull_bar(b), 1);
            mbar_init(tempty_bar(b), CG * 32 * EPI_WARPS);
        }
        if constexpr (KCL) mbar_init(xdata_bar, 32 * EPI_WARPS / 2);
        *abort_flag = 0;
        fence_mbar_init();
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmB);
        if constexpr (TF32) {
            tma_prefetch_desc(&tmA2);
            tma_prefetch_desc(&tmB2);
        }
        if (args.c_tma) tma_prefetch_desc(&tmC);
    }
    if (warp == 1) {
        tmem_alloc<CG>(smem_u32(const_cast<uint32_t*>(tmem_holder)), TMEM_COLS);
        tmem_relinquish<CG>();
    }
    tc_fence_before_sync();
    __syncthreads();
    if constexpr (PAIR) {
        cluster_arrive();
        cluster_wait();
    }
    // KCL: the peer's barrier must be initialised before anything arrives on it, which happens only in the
    // epilogue. Arrive now (release) and wait there — nobody stalls here for the cluster to assemble.
    if constexpr (KCL) cluster_arrive();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_holder;
    // Everything above touched only shared and tensor memory; operands and outputs of the kernels
    // before this one are first accessed below.
    pdl_wait();
    pdl_launch_dependents();
    if (tracing && threadIdx.x == 0) args.trace[1] = global_timer_ns();

    const int num_units = args.num_tiles * args.split_k;
    [[maybe_unused]] bool kcl_waited = false;   // has this thread waited for the prologue's cluster barrier yet?
    // KCL: this CTA's one unit is (tile = cluster index, split = rank in the cluster); no further units.
    const int unit_first = KCL ? (int)krank * args.num_tiles + worker : worker;
    const int unit_step = KCL ? num_units : num_workers;

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int u = unit_first; u < num_units && ok; u += unit_step) {
                int t, split, ub0, ub1, tm, tn;
                unit_decode(u, args, t, split, ub0, ub1);
                tile_coords(t, args, tm, tn);
                const int m0 = tm * TILE_M + (int)rank * kBlockM, n0 = tn * BN + (int)rank * BN_CTA;
                // Convolution feeds: where this tile sits in the position grid / the column boxes.
                const ConvGeom& cv = args.cv;
                [[maybe_unused]] int cs_n = 0, cs_x0 = 0, cs_y0 = 0;                  // kConvSpatial
                [[maybe_unused]] int cw_c[BN_CTA / 32], cw_dx[BN_CTA / 32], cw_dy[BN_CTA / 32], cw_ok[BN_CTA / 32];   // kConvWgrad
                if constexpr (CONV == kConvSpatial) {
                    const int tx = tm % cv.tiles_x, r = tm / cv.tiles_x;
                    const int ty = r % cv.tiles_y;
                    cs_n = r / cv.tiles_y;
                    cs_x0 = tx << cv.tw_log2;
                    cs_y0 = (ty * CG + (int)rank) * cv.th;
                }
                if constexpr (CONV == kConvWgrad) {
#pragma unroll
                    for (int i = 0; i < BN_CTA / 32; ++i) {
                        const int jb = (n0 >> 5) + i;
                        const int tap = jb / cv.cblks, ki = tap / cv.kw;
                        cw_c[i] = (jb - tap * cv.cblks) * 32;
                        cw_dy[i] = cv.ay0 + ki * cv.ay_step;
                        cw_dx[i] = cv.ax0 + (tap - ki * cv.kw) * cv.ax_step;
                        cw_ok[i] = tap < cv.taps;
                    }
                }
                for (int kb = ub0; kb < ub1; ++kb) {
                    ok = mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, args.status, kDevTimeoutEmpty);
                    if (!ok) break;
                    const uint32_t st = smem_base + s * S::STAGE_BYTES;
                    const uint32_t a_hi = st;
                    const uint32_t a_lo = st + S::A_TILE;
                    const uint32_t b_hi = st + S::NSPLIT * S::A_TILE;
                    const uint32_t b_lo = b_hi + S::B_TILE;
                    // Pair: the leader announces the bytes of both CTAs and every load signals the
                    // leader's barrier; the peer only issues its loads.
                    const uint32_t fb = PAIR ? mapa_shared(full_bar(s), 0) : full_bar(s);
                    if (rank == 0) mbar_arrive_expect_tx(full_bar(s), CG * S::STAGE_BYTES);
                    const int k0 = kb * BK;
                    auto load = [&](uint32_t dst, const CUtensorMap* map, int x, int y) {
                        if constexpr (PAIR) tma_load_2d_pair(dst, map, x, y, fb);
                        else tma_load_2d(dst, map, x, y, fb);
                    };
                    if constexpr (CONV == kConvSpatial) {
                        const int tap = kb / cv.cblks, c0 = (kb - tap * cv.cblks) * 32;
                        const int ki = tap / cv.kw, kj = tap - ki * cv.kw;
                        const int sy = cs_y0 * cv.sy + cv.ay0 + ki * cv.ay_step;
                        const int sx = cs_x0 * cv.sx + cv.ax0 + kj * cv.ax_step;
                        tma_load_4d<PAIR>(a_hi, &tmA, c0, sx, sy, cs_n, fb);
                        tma_load_4d<PAIR>(a_lo, &tmA2, c0, sx, sy, cs_n, fb);
                        tma_load_3d<PAIR>(b_hi, &tmB, c0, tap, n0, fb);
                        tma_load_3d<PAIR>(b_lo, &tmB2, c0, tap, n0, fb);
                    } else if constexpr (CONV == kConvWgrad) {
                        const int per = cv.kblk_x * cv.kblk_y;
                        const int n = kb / per, r = kb - n * per;
                        const int by = r / cv.kblk_x, bx = r - by * cv.kblk_x;
                        const int px = bx << cv.kblk_w_log2, py = by * cv.kblk_h;
                        const int qx = px * cv.sx, qy = py * cv.sy;   // the same block in the strided source
#pragma unroll
                        for (int i = 0; i < kBlockM / T_MN; ++i) {
                            tma_load_4d<PAIR>(a_hi + i * (BK * 128), &tmA, m0 + i * T_MN, px, py, n, fb);
                            tma_load_4d<PAIR>(a_lo + i * (BK * 128), &tmA2, m0 + i * T_MN, px, py, n, fb);
                        }
#pragma unroll
                        for (int i = 0; i < BN_CTA / T_MN; ++i) {
                            // column boxes past the last tap read a sample index beyond the tensor: zeros
                            const int nn = cw_ok[i] ? n : cv.n_samples;
                            tma_load_4d<PAIR>(b_hi + i * (BK * 128), &tmB, cw_c[i], qx + cw_dx[i], qy + cw_dy[i], nn, fb);
                            tma_load_4d<PAIR>(b_lo + i * (BK * 128), &tmB2, cw_c[i], qx + cw_dx[i], qy + cw_dy[i], nn, fb);
                        }
                    } else {
                    if constexpr (!A_MN) {
                        load(a_hi, &tmA, k0, m0);
                        if constexpr (TF32) load(a_lo, &tmA2, k0, m0);
                    } else {
#pragma unroll
                        for (int i = 0; i < kBlockM / T_MN; ++i) {
                            load(a_hi + i * (BK * 128), &tmA, m0 + i * T_MN, k0);
                            if constexpr (TF32) load(a_lo + i * (BK * 128), &tmA2, m0 + i * T_MN, k0);
                        }
                    }
                    if constexpr (!B_MN) {
                        load(b_hi, &tmB, k0, n0);
                        if constexpr (TF32) load(b_lo, &tmB2, k0, n0);
                    } else {
#pragma unroll
                        for (int i = 0; i < BN_CTA / T_MN; ++i) {
                            load(b_hi + i * (BK * 128), &tmB, n0 + i * T_MN, k0);
                            if constexpr (TF32) load(b_lo + i * (BK * 128), &tmB2, n0 + i * T_MN, k0);
                        }
                    }
                    }
                    if (++s == STAGES) { s = 0; ph ^= 1u; }
                }
            }
            // Drain: every load this thread issued has landed once the stage it targeted
            // was consumed; on the normal path the final __syncthreads implies that. On an
            // aborted run wait (bounded) for the stages still in flight.
            if (rank == 0 && (!ok || *abort_flag != 0)) {
                for (int i = 0; i < STAGES; ++i) {
                    const uint64_t t0 = global_timer_ns();
                    while (!mbar_try_wait(full_bar(i), 0) && !mbar_try_wait(full_bar(i), 1)) {
                        if (global_timer_ns() - t0 > 100000000ull) {
                            if (args.status != nullptr) atomicCAS(args.status, 0, kDevTimeoutDrain);
                            break;
                        }
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer --------------------------------
        if (lane == 0 && rank == 0) {
            const uint32_t idesc = make_idesc(TF32 ? 2u : (args.is_bf16 ? 1u : 0u),
                                              A_MN ? 1u : 0u, B_MN ? 1u : 0u, TILE_M, BN);
            // K-major: 128-byte swizzle, 8-row groups 1024 B apart, K step = +32 B inside the row.
            // MN-major, 16-bit: 128-byte swizzle; the 128-byte columns of a tile are one TMA box
            //   (BK*128 B) apart (leading offset), 8-row K groups 1024 B apart.
            // MN-major, 32-bit: the tensor core only takes the 128-byte swizzle with 32-byte
            //   atoms, whose K groups are 4 rows (512 B).
            // In both MN-major cases one K step is UMMA_K rows of 128 B.
            constexpr uint32_t MN_SWZ = TF32 ? 1u : 2u;
            constexpr uint32_t MN_SBO = TF32 ? 512u : 1024u;
            constexpr uint32_t A_LBO = A_MN ? (uint32_t)(BK * 128) : 16u;
            constexpr uint32_t B_LBO = B_MN ? (uint32_t)(BK * 128) : 16u;
            constexpr uint32_t A_SBO = A_MN ? MN_SBO : 1024u;
            constexpr uint32_t B_SBO = B_MN ? MN_SBO : 1024u;
            constexpr uint32_t A_SWZ = A_MN ? MN_SWZ : 2u;
            constexpr uint32_t B_SWZ = B_MN ? MN_SWZ : 2u;
            constexpr uint32_t A_KSTEP = A_MN ? (uint32_t)(UMMA_K * 128) : 32u;
            constexpr uint32_t B_KSTEP = B_MN ? (uint32_t)(UMMA_K * 128) : 32u;
            auto commit = [&](uint32_t bar) {
                if constexpr (PAIR) umma_commit_pair_both(bar, (uint16_t)3);
                else umma_commit<1>(bar);
            };
            int s = 0;
            uint32_t ph = 0;
            uint32_t cit = 0;   // accumulator hand-offs so far (chunks, over all tiles)
            bool ok = true;
            for (int u = unit_first; u < num_units && ok; u += unit_step) {
                int t, split, ub0, ub1;
                unit_decode(u, args, t, split, ub0, ub1);
                for (int kb0 = ub0; kb0 < ub1 && ok; kb0 += args.chunk_kb, ++cit) {
                    const uint32_t buf = cit & 1u;
                    const uint32_t use = cit >> 1;
                    ok = mbar_wait(tempty_bar(buf), (use & 1u) ^ 1u, abort_flag, args.status,
                                   kDevTimeoutTmemEmpty);
                    if (!ok) break;
                    tc_fence_after_sync();
                    const uint32_t d_tmem = tmem_base + buf * (uint32_t)BN;
                    const int kb1 = min(kb0 + args.chunk_kb, ub1);
                    for (int kb = kb0; kb < kb1; ++kb) {
                        ok = mbar_wait(full_bar(s), ph, abort_flag, args.status, kDevTimeoutFull);
                        if (!ok) break;
                        tc_fence_after_sync();
                        if (tracing && u == unit_first && kb == ub0) args.trace[2] = global_timer_ns();
                        const uint32_t st = smem_base + s * S::STAGE_BYTES;
                        const uint32_t a_hi = st;
                        const uint32_t a_lo = st + S::A_TILE;
                        const uint32_t b_hi = st + S::NSPLIT * S::A_TILE;
                        const uint32_t b_lo = b_hi + S::B_TILE;
#pragma unroll
                        for (int j = 0; j < KSTEPS; ++j) {
                            const uint32_t acc = (kb > kb0 || j > 0) ? 1u : 0u;
                            const uint64_t da = make_smem_desc(a_hi + j * A_KSTEP, A_LBO, A_SBO, A_SWZ);
                            const uint64_t db = make_smem_desc(b_hi + j * B_KSTEP, B_LBO, B_SBO, B_SWZ);
                            if constexpr (TF32) {
                                const uint64_t dal = make_smem_desc(a_lo + j * A_KSTEP, A_LBO, A_SBO, A_SWZ);
                                const uint64_t dbl = make_smem_desc(b_lo + j * B_KSTEP, B_LBO, B_SBO, B_SWZ);
                                umma_ss<CG, true>(d_tmem, dal, db, idesc, acc);
                                umma_ss<CG, true>(d_tmem, da, dbl, idesc, 1u);
                                umma_ss<CG, true>(d_tmem, da, db, idesc, 1u);
                            } else {
                                umma_ss<CG, false>(d_tmem, da, db, idesc, acc);
                            }
                        }
                        commit(empty_bar(s));
                        if (++s == STAGES) { s = 0; ph ^= 1u; }
                    }
                    if (!ok) break;
                    commit(tfull_bar(buf));
                    if (tracing) args.trace[3] = global_timer_ns();
                }
            }
        }
    } else {
        // ------------------------------ epilogue ----------------------------------
        const int ew = warp - 2;
        const int q = warp & 3;            // TMEM lanes [32q, 32q+32) are the ones this warp may read
        const int cbase = (ew >> 2) * COLS; // first accumulator column of this warp
        uint8_t* staging = staging_all + ew * S::STAGING_BUFS * 4096;
        int stage_buf = 0;
        const bool c_tma = args.c_tma != 0;
        auto release = [&](uint32_t buf) {
            tc_fence_before_sync();
            if constexpr (PAIR) mbar_arrive_cluster(mapa_shared(tempty_bar(buf), 0));
            else mbar_arrive(tempty_bar(buf));
        };
        uint32_t cit = 0;
        bool ok = true;
        for (int u = unit_first; u < num_units && ok; u += unit_step) {
            int t, split, ub0, ub1, tm, tn;
            unit_decode(u, args, t, split, ub0, ub1);
            tile_coords(t, args, tm, tn);
            // Split-K partial outputs are stacked: split s writes rows [s * rows_per_split, ...) of the
            // partial matrix (rows_per_split = split_stride / ldc covers whole tiles, so edge tiles of
            // one split never reach into the next).
            const int row_shift = (int)(args.split_stride / args.ldc) * split;
            const int m0 = tm * TILE_M + (int)rank * kBlockM, n0 = tn * BN + cbase;
            const int row0 = m0 + q * 32 + row_shift;
            const int row = row0 + lane;
            const bool row_ok = (row - row_shift) < args.M;
            float row_bias = 0.f;
            if (args.bias_mode == kBiasPerRow && row_ok) row_bias = __ldg(args.bias + row - row_shift);
            const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)cbase;

            if constexpr (TF32) {
                float acc[COLS];
#pragma unroll
                for (int i = 0; i < COLS; ++i) acc[i] = 0.f;
                for (int kb0 = ub0; kb0 < ub1; kb0 += args.chunk_kb, ++cit) {
                    const uint32_t buf = cit & 1u;
                    const uint32_t use = cit >> 1;
                    ok = mbar_wait(tfull_bar(buf), use & 1u, abort_flag, args.status, kDevTimeoutTmemFull);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    tc_fence_after_sync();
                    if (tracing && ew == 0 && lane == 0) args.trace[4] = global_timer_ns();
#pragma unroll
                    for (int c = 0; c < COLS / 32; ++c) {
                        if (n0 + c * 32 < args.N) {
                            uint32_t r[32];
                            tmem_ld_32x32(lane_addr + buf * (uint32_t)BN + (uint32_t)(c * 32), r);
                            tmem_ld_wait();
#pragma unroll
                            for (int i = 0; i < 32; ++i) acc[c * 32 + i] += __uint_as_float(r[i]);
                        }
                    }
                    release(buf);
                }
                if (!ok) break;
                if constexpr (KCL) {
                    // Warp ew holds column half ew >> 2 of this CTA's partial tile; half k is finished by CTA k.
                    // The same warp index sends in one CTA and receives in the other. A receiving warp's 8 KB
                    // arrive in its own staging buffer (float4 slots 0..7 of each lane) and in that of the
                    // sending warp beside it (slots 8..15), lane-interleaved: conflict-free both ways, and no
                    // other warp's stores can touch them.
                    constexpr int HALF = COLS / 8;   // float4 slots per staging buffer
                    const uint32_t own_off = (uint32_t)(STAGES * S::STAGE_BYTES + ew * 4096 + lane * 16);
                    const uint32_t side_off = (uint32_t)(STAGES * S::STAGE_BYTES + (ew ^ 4) * 4096 + lane * 16);
                    cluster_wait();   // long since complete: the peer arrived in its prologue
                    kcl_waited = true;
                    if ((uint32_t)(ew >> 2) == krank) {
                        ok = mbar_wait(xdata_bar, 0, abort_flag, args.status, kDevTimeoutPeer);
                        ok = __all_sync(0xffffffffu, ok);
                        if (!ok) break;
                        fence_acq_rel_cluster();
#pragma unroll
                        for (int i = 0; i < 2 * HALF; ++i) {
                            const float4 p = *reinterpret_cast<const float4*>(
                                smem_gen + (i < HALF ? own_off + i * 512 : side_off + (i - HALF) * 512));
                            acc[4 * i] += p.x; acc[4 * i + 1] += p.y; acc[4 * i + 2] += p.z; acc[4 * i + 3] += p.w;
                        }
                        __syncwarp();   // the staging buffer is about to be reused for the stores
                    } else {
                        const uint32_t peer = mapa_shared(smem_base, krank ^ 1u);
#pragma unroll
                        for (int i = 0; i < 2 * HALF; ++i)
                            st_shared_cluster_v4(peer + (i < HALF ? own_off + i * 512 : side_off + (i - HALF) * 512),
                                                 acc[4 * i], acc[4 * i + 1], acc[4 * i + 2], acc[4 * i + 3]);
                        fence_acq_rel_cluster();
                        mbar_arrive_cluster(mapa_shared(xdata_bar, krank ^ 1u));
                        break;   // the peer finishes these columns
                    }
                }
                if constexpr (CONV == kConvSpatial) {
                    // Row r of the CTA's 128 is position (y0 + r / tw, x0 + r % tw) of sample n; column j
                    // goes to dst[n][j][y][x] (NCHW): lanes are consecutive x, so each store
                    // instruction writes whole lines.
                    const ConvGeom& cv = args.cv;
                    const int tx = tm % cv.tiles_x, rr = tm / cv.tiles_x;
                    const int ty = rr % cv.tiles_y, n = rr / cv.tiles_y;
                    const int r = q * 32 + lane;
                    const int oy = (ty * CG + (int)rank) * cv.th + (r >> cv.tw_log2);
                    const int ox = (tx << cv.tw_log2) + (r & ((1 << cv.tw_log2) - 1));
                    const bool valid = oy < cv.out_h && ox < cv.out_w;
                    const long long plane = (long long)cv.out_h * cv.out_w;
                    float* dst = static_cast<float*>(args.C) + (long long)n * args.N * plane +
                                 (long long)oy * cv.out_w + ox;
#pragma unroll
                    for (int c = 0; c < COLS / 32; ++c) {
                        const int col0 = n0 + c * 32;
                        if (col0 < args.N) {
                            float v[32];
#pragma unroll
                            for (int i = 0; i < 32; ++i) v[i] = acc[c * 32 + i];
                            epilogue_apply32(v, args, col0, 0.f);
                            if (valid) {
#pragma unroll
                                for (int i = 0; i < 32; ++i)
                                    if (col0 + i < args.N) dst[(long long)(col0 + i) * plane] = v[i];
                            }
                        }
                    }
                } else {
#pragma unroll
                    for (int c = 0; c < COLS / 32; ++c) {
                        const int col0 = n0 + c * 32;
                        if (col0 < args.N && (c_tma ? (row0 - row_shift) < args.M : row_ok)) {
                            float v[32];
#pragma unroll
                            for (int i = 0; i < 32; ++i) v[i] = acc[c * 32 + i];
                            epilogue_apply32(v, args, col0, row_bias);
                            // planes first (plain stores, the staging buffer is free again at once), then the
                            // asynchronous TMA store of the values themselves
                            if (args.planes_lo != nullptr) epilogue_store_planes32(v, args, staging, lane, row0, col0);
                            if (c_tma) epilogue_store32_tma<S::STAGING_BUFS>(v, &tmC, staging, stage_buf, lane, row0, col0);
                            else epilogue_store32(v, args, row, col0);
                        }
                    }
                }
            } else {
                const uint32_t buf = cit & 1u;
                const uint32_t use = cit >> 1;
                ++cit;
                ok = mbar_wait(tfull_bar(buf), use & 1u, abort_flag, args.status, kDevTimeoutTmemFull);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after_sync();
#pragma unroll 1
                for (int c = 0; c < COLS / 32; ++c) {
                    const int col0 = n0 + c * 32;
                    if (col0 >= args.N) break;
                    uint32_t r[32];
                    tmem_ld_32x32(lane_addr + buf * (uint32_t)BN + (uint32_t)(c * 32), r);
                    tmem_ld_wait();
                    if (!(c_tma ? (row0 - row_shift) < args.M : row_ok)) continue;   // warp-uniform on the TMA path
                    float v[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
                    epilogue_apply32(v, args, col0, row_bias);
                    if (c_tma) epilogue_store32_tma<S::STAGING_BUFS>(v, &tmC, staging, stage_buf, lane, row0, col0);
                    else epilogue_store32(v, args, row, col0);
                }
                release(buf);
            }
        }
        // The staging buffers must outlive the TMA engine's reads, and the stores must be complete
        // before the grid is.
        if (c_tma && lane == 0) tma_store_wait_all<0>();
        if (tracing && ew == 0 && lane == 0) args.trace[5] = global_timer_ns();
    }

    // KCL: every thread pairs its prologue arrive with one wait. No second cluster barrier: each CTA has
    // received everything the peer will ever write into it before it gets here.
    if constexpr (KCL) {
        __syncwarp();
        if (!kcl_waited) cluster_wait();
    }
    tc_fence_before_sync();
    __syncthreads();
    if constexpr (PAIR) {
        cluster_arrive();
        cluster_wait();
    }
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc<CG>(tmem_base, TMEM_COLS);
    }
    if (tracing && threadIdx.x == 0) args.trace[6] = global_timer_ns();
}

}  // namespace tfb
