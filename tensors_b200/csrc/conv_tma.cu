// Convolutions on the TMA-fed tcgen05 GEMM kernel.
//
// A pre-pass rewrites the activation tensor (NCHW) as NHWC TF32 hi / lo planes. In that layout the
// slice of the im2col matrix that one K block needs — 32 channels of one filter tap for a rectangle
// of output positions — is a single 4-D box of the tensor, shifted by the tap's offset, and the
// padding halo is the box's out-of-range part, which the TMA unit fills with zeros. So the im2col
// index map costs no instructions and the main loop is the plain GEMM pipeline. A convolution stride is the
// tensor map's traversal stride (the box then spans stride x as many source positions and delivers every
// stride-th one), so it costs nothing either; the input gradient is stride-1 only (its gather form divides
// by the stride).
//
//   forward          rows = positions, columns = Cout, K = (tap, Cin)       A: x planes   B: W[co][tap][ci]
//   input gradient   rows = positions, columns = Cin,  K = (tap, Cout)      A: dY planes  B: W[ci][tap][co]
//                    gather form: source row = y + pad - ki * dilation
//   weight gradient  rows = Cout, columns = (tap, Cin), K = positions of all samples, split between CTAs
//                    A: dY planes (MN-major boxes)  B: x planes shifted by the tap (MN-major boxes)
//   bias gradient    column sums taken by the dY pre-pass
//
// Outputs are written NCHW (forward, input gradient) by the kernel's epilogue.
#include <atomic>
#include <cstdlib>
#include <cstring>

#include "gemm_kernel.cuh"
#include "internal.hpp"

namespace tfb {

namespace {

inline int64_t round_up(int64_t x, int64_t m) { return (x + m - 1) / m * m; }
inline size_t align256(size_t x) { return (x + 255) & ~(size_t)255; }

__device__ __forceinline__ float tf32_rna_c(float x) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return __uint_as_float(r);
}

// src[n][c][p] (NCHW, p = y * W + x) -> hi / lo[n][p][cp] (NHWC, channels padded with zeros to cp).
// One block transposes a 32-channel x 128-position tile through shared memory: reads are contiguous in p
// (16 bytes per lane where the rows allow it, four of them in flight per thread — the pass is bound by bytes
// in flight, not by DRAM), writes contiguous in c. If colsum != nullptr, colsum[(n * pblocks + pb) * cp + c]
// receives, for each of the tile's four 32-position blocks pb, the sum of its positions in ascending order
// (the bias-gradient partial sums).
constexpr int kSplitTileP = 128;
__global__ void nhwc_split_kernel(const float* __restrict__ src, int C, int P, int cp, float* __restrict__ hi,
                                  float* __restrict__ lo, float* __restrict__ colsum, int pblocks) {
    __shared__ float tile[32][kSplitTileP + 1];
    pdl_wait();
    pdl_launch_dependents();
    const int n = blockIdx.z, c0 = blockIdx.y * 32, p0 = blockIdx.x * kSplitTileP;
    const int tx = threadIdx.x, ty = threadIdx.y;
    const float* s = src + (long long)n * C * P;
    const bool vec = (P & 3) == 0 && (reinterpret_cast<uintptr_t>(src) & 15u) == 0;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int cl = ty + 8 * k, c = c0 + cl, p = p0 + 4 * tx;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (c < C) {
            const float* row = s + (long long)c * P;
            if (vec && p + 3 < P) {
                v = *reinterpret_cast<const float4*>(row + p);
            } else {
                if (p < P) v.x = row[p];
                if (p + 1 < P) v.y = row[p + 1];
                if (p + 2 < P) v.z = row[p + 2];
                if (p + 3 < P) v.w = row[p + 3];
            }
        }
        tile[cl][4 * tx] = v.x; tile[cl][4 * tx + 1] = v.y; tile[cl][4 * tx + 2] = v.z; tile[cl][4 * tx + 3] = v.w;
    }
    __syncthreads();
    const int c = c0 + tx;
    if (c < cp) {
#pragma unroll 4
        for (int k = 0; k < kSplitTileP / 8; ++k) {
            const int pl = ty + 8 * k, p = p0 + pl;
            if (p < P) {
                const float v = tile[tx][pl];
                const float h = tf32_rna_c(v);
                const long long o = ((long long)n * P + p) * cp + c;
                hi[o] = h;
                lo[o] = v - h;
            }
        }
        if (colsum != nullptr && ty < kSplitTileP / 32) {
            const int pb = blockIdx.x * (kSplitTileP / 32) + ty;
            if (pb < pblocks) {
                float t = 0.f;
#pragma unroll
                for (int pl = 0; pl < 32; ++pl) t += tile[tx][ty * 32 + pl];
                colsum[((long long)n * pblocks + pb) * cp + c] = t;
            }
        }
    }
}

// Filter planes for the spatial feed: out[j][tap][c] (c padded to cp) with
//   forward (by_cin == 0): j = output channel, c = input channel
//   gradient (by_cin == 1): j = input channel,  c = output channel
// both reading W[co][ci][tap].
__global__ void filter_planes_kernel(const float* __restrict__ W, int Cout, int Cin, int khw, int cp, int by_cin,
                                     float* __restrict__ hi, float* __restrict__ lo) {
    pdl_wait();
    pdl_launch_dependents();
    const int J = by_cin ? Cin : Cout, Cc = by_cin ? Cout : Cin;
    const long long total = (long long)J * khw * cp;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int c = (int)(i % cp);
        const long long r = i / cp;
        const int tap = (int)(r % khw), j = (int)(r / khw);
        float v = 0.f;
        if (c < Cc) {
            const int co = by_cin ? c : j, ci = by_cin ? j : c;
            v = W[((long long)co * Cin + ci) * khw + tap];
        }
        const float h = tf32_rna_c(v);
        hi[i] = h;
        lo[i] = v - h;
    }
}

// dW[co][ci][tap] = sum over splits (ascending) of partial[s][co][tap * cp32 + ci].
__global__ void wgrad_planes_reduce_kernel(const float* __restrict__ partial, int splits, long long split_stride,
                                           long long ld, int Cout, int Cin, int khw, int cp32,
                                           float* __restrict__ dW) {
    pdl_wait();
    pdl_launch_dependents();
    const long long total = (long long)Cout * Cin * khw;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int tap = (int)(i % khw);
        const long long r = i / khw;
        const int ci = (int)(r % Cin), co = (int)(r / Cin);
        const float* p = partial + (long long)co * ld + (long long)tap * cp32 + ci;
        float s = 0.f;
        for (int k = 0; k < splits; ++k) s += p[(long long)k * split_stride];
        dW[i] = s;
    }
}

// out[blockIdx.y][c] = sum of partial[b][c] over the block's rows b in [y * rows_per_block, ...): a block
// covers 32 columns; its eight row groups each keep four independent running sums (rows g, g + 32, ...;
// g + 8, ...; g + 16, ...; g + 24, ...), combined in a fixed order, then the eight group sums are added in
// ascending order. Run it once over many row blocks and once more over their results.
__global__ void colsum_kernel(const float* __restrict__ partial, long long rows, int cols, long long ld,
                              long long rows_per_block, float* __restrict__ out, int out_ld) {
    __shared__ float sm[8][33];
    pdl_wait();
    pdl_launch_dependents();
    const int c = blockIdx.x * 32 + threadIdx.x;
    const long long r0 = (long long)blockIdx.y * rows_per_block;
    const long long r1 = r0 + rows_per_block < rows ? r0 + rows_per_block : rows;
    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
    if (c < cols) {
        for (long long b = r0 + threadIdx.y; b < r1; b += 32) {
            a0 += partial[b * ld + c];
            if (b + 8 < r1) a1 += partial[(b + 8) * ld + c];
            if (b + 16 < r1) a2 += partial[(b + 16) * ld + c];
            if (b + 24 < r1) a3 += partial[(b + 24) * ld + c];
        }
    }
    sm[threadIdx.y][threadIdx.x] = (a0 + a1) + (a2 + a3);
    __syncthreads();
    if (threadIdx.y == 0 && c < cols) {
        float t = 0.f;
#pragma unroll
        for (int g = 0; g < 8; ++g) t += sm[g][threadIdx.x];
        out[(long long)blockIdx.y * out_ld + c] = t;
    }
}

template <int BN, int STAGES, bool PAIR, int CONV>
int launch_feed(const CUtensorMap maps[5], const GemmArgs& args, int workers, cudaStream_t stream) {
    using S = GemmSmem<kKindTF32x3, BN, STAGES, PAIR>;
    static_assert(S::TOTAL <= 232448, "stage ring + staging exceed the 227 KB shared-memory limit");
    constexpr bool MN = (CONV == kConvWgrad);
    auto kern = gemm_tcgen05_kernel<kKindTF32x3, BN, STAGES, MN, MN, PAIR, CONV>;
    // once per (kernel variant, device); several host threads may get here at the same time
    static std::atomic<bool> attr_set[64];
    int dev = 0;
    TFB_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(TFB_ERR_UNSUPPORTED, "device index %d out of range", dev);
    if (!attr_set[dev].load(std::memory_order_acquire)) {
        TFB_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL));
        attr_set[dev].store(true, std::memory_order_release);
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(PAIR ? 2 * workers : workers));
    cfg.blockDim = dim3((unsigned)gemm_threads(kKindTF32x3));
    cfg.dynamicSmemBytes = S::TOTAL;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = PAIR ? 2 : 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    // every kernel of a convolution call waits in-kernel for the one before it (pdl_wait), so prologues
    // and launch latencies overlap the predecessor's tail
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = tuning(TFB_TUNE_PDL) != 0 ? 2 : 1;
    TFB_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, maps[0], maps[1], maps[2], maps[3], maps[4], args));
    return TFB_OK;
}

unsigned grid_1d(long long total) {
    const long long blocks = (total + 255) / 256;
    return (unsigned)(blocks < 1184 ? (blocks < 1 ? 1 : blocks) : 1184);
}

int pow2_ceil_log2(int64_t v) {
    int l = 0;
    while ((1ll << l) < v) ++l;
    return l;
}

int to_nhwc_planes(const float* src, int64_t N, int64_t C, int64_t P, int64_t cp, float* hi, float* lo,
                   float* colsum, cudaStream_t stream) {
    dim3 grid((unsigned)((P + kSplitTileP - 1) / kSplitTileP), (unsigned)((cp + 31) / 32), (unsigned)N), block(32, 8);
    return launch_pdl(nhwc_split_kernel, grid, block, 0, stream, src, (int)C, (int)P, (int)cp, hi, lo, colsum,
                      (int)((P + 31) / 32));
}

// 4-D maps (channel, x, y, sample) over NHWC hi / lo planes with a box of 32 channels x bw x bh positions,
// taken every sw-th / sh-th position of the tensor.
int plane_maps(CUtensorMap out[2], const float* hi, const float* lo, int64_t cp, int64_t W, int64_t H, int64_t N,
               uint32_t bw, uint32_t bh, bool atom32, uint32_t sw = 1, uint32_t sh = 1) {
    const uint64_t dims[4] = {(uint64_t)cp, (uint64_t)W, (uint64_t)H, (uint64_t)N};
    const uint64_t strides[3] = {(uint64_t)cp * 4, (uint64_t)(W * cp) * 4, (uint64_t)(H * W * cp) * 4};
    const uint32_t box[4] = {32, (bw - 1) * sw + 1, (bh - 1) * sh + 1, 1};
    const uint32_t estr[4] = {1, sw, sh, 1};
    int rc = make_map_nd(&out[0], hi, 4, dims, strides, box, atom32, estr);
    if (rc != TFB_OK) return rc;
    return make_map_nd(&out[1], lo, 4, dims, strides, box, atom32, estr);
}

struct SpatialCall {
    const float* src_hi; const float* src_lo;   // NHWC planes of the tensor the taps are gathered from
    int64_t src_c, src_cp, src_H, src_W;        // its channels (contraction), padded channels, extent
    const float* f_hi; const float* f_lo;       // filter planes [J][taps][src_cp]
    int64_t J;                                  // output channels of this product
    int64_t out_H, out_W;                       // position grid = extent of the stored tensor
    int ay0, ay_step, ax0, ax_step;
    int sy = 1, sx = 1;                         // position -> source stride (forward: the convolution's)
    float* dst; const float* bias; bool relu;
};

int run_spatial(const SpatialCall& c, const ConvShape& s, const DeviceState* st, cudaStream_t stream) {
    const int64_t khw = s.kH * s.kW;
    const int cblks = (int)((c.src_c + 31) / 32);
    const int env_pair = tuning(TFB_TUNE_CONV_PAIR);
    const int tw_log2 = pow2_ceil_log2(c.out_W < 128 ? c.out_W : 128);
    const int tw = 1 << tw_log2, th = 128 / tw;
    const int64_t tiles_x = (c.out_W + tw - 1) / tw;
    const int64_t single_tiles = s.N * tiles_x * ((c.out_H + th - 1) / th);
    const bool pair = c.J > 64 && (env_pair >= 0 ? env_pair != 0 : single_tiles >= st->sm_count);
    const int cg = pair ? 2 : 1;
    const int bn = c.J <= 64 ? 64 : 128;
    const int64_t tiles_y = (c.out_H + cg * th - 1) / (cg * th);
    if (s.N * tiles_x * tiles_y * cg * kBlockM >= (1ll << 31))
        return fail(TFB_ERR_TOO_LARGE, "conv2d: more output tiles than the 32-bit tile index holds");

    GemmArgs a;
    memset(&a, 0, sizeof(a));
    a.tiles_m = (int)(s.N * tiles_x * tiles_y);
    a.tiles_n = (int)((c.J + bn - 1) / bn);
    a.num_tiles = a.tiles_m * a.tiles_n;
    a.M = a.tiles_m * cg * kBlockM; a.N = (int)c.J; a.K = (int)(khw * cblks * 32);
    a.k_blocks = (int)(khw * cblks);
    a.chunk_kb = 8; a.split_k = 1; a.kb_per_split = a.k_blocks; a.split_stride = 0;
    a.group_m = 16;
    a.C = c.dst; a.ldc = 0; a.out_type = kOutF32;
    a.bias = c.bias; a.bias_mode = c.bias != nullptr ? kBiasPerCol : kBiasNone; a.relu = c.relu ? 1 : 0;
    a.c_tma = 0; a.status = st->status;
    a.cv.tw_log2 = tw_log2; a.cv.th = th;
    a.cv.tiles_x = (int)tiles_x; a.cv.tiles_y = (int)tiles_y;
    a.cv.out_h = (int)c.out_H; a.cv.out_w = (int)c.out_W;
    a.cv.cblks = cblks; a.cv.kw = (int)s.kW; a.cv.taps = (int)khw;
    a.cv.ay0 = c.ay0; a.cv.ay_step = c.ay_step; a.cv.ax0 = c.ax0; a.cv.ax_step = c.ax_step;
    a.cv.sx = c.sx; a.cv.sy = c.sy;
    a.cv.n_samples = (int)s.N;

    CUtensorMap maps[5];
    memset(maps, 0, sizeof(maps));
    int rc = plane_maps(&maps[0], c.src_hi, c.src_lo, c.src_cp, c.src_W, c.src_H, s.N, (uint32_t)tw, (uint32_t)th, false,
                        (uint32_t)c.sx, (uint32_t)c.sy);
    if (rc != TFB_OK) return rc;
    const uint64_t fdims[3] = {(uint64_t)c.src_cp, (uint64_t)khw, (uint64_t)c.J};
    const uint64_t fstr[2] = {(uint64_t)c.src_cp * 4, (uint64_t)(khw * c.src_cp) * 4};
    const uint32_t fbox[3] = {32, 1, (uint32_t)(pair ? bn / 2 : bn)};
    rc = make_map_nd(&maps[2], c.f_hi, 3, fdims, fstr, fbox, false);
    if (rc != TFB_OK) return rc;
    rc = make_map_nd(&maps[3], c.f_lo, 3, fdims, fstr, fbox, false);
    if (rc != TFB_OK) return rc;
    maps[4] = maps[0];   // no TMA store on this path

    if (pair) {
        const int max_pairs = st->sm_count / 2;
        const int pairs = a.num_tiles < max_pairs ? a.num_tiles : max_pairs;
        return launch_feed<128, 4, true, kConvSpatial>(maps, a, pairs, stream);
    }
    const int grid = a.num_tiles < st->sm_count ? a.num_tiles : st->sm_count;
    if (bn == 64) return launch_feed<64, 4, false, kConvSpatial>(maps, a, grid, stream);
    return launch_feed<128, 3, false, kConvSpatial>(maps, a, grid, stream);
}

}  // namespace

constexpr int kColsumStageBlocks = 32;   // row blocks of the first reduction stage

size_t column_sums_stage_bytes(int64_t cols) { return (size_t)(kColsumStageBlocks * ((cols + 3) / 4 * 4)) * 4; }

int column_sums(const float* partial, int64_t rows, int64_t cols, int64_t ld, float* stage, float* out,
                cudaStream_t stream) {
    if (cols <= 0) return TFB_OK;
    const int64_t stage_ld = (cols + 3) / 4 * 4;
    const long long per_block = (rows + kColsumStageBlocks - 1) / kColsumStageBlocks;
    const unsigned col_blocks = (unsigned)((cols + 31) / 32);
    int rc = launch_pdl(colsum_kernel, dim3(col_blocks, kColsumStageBlocks), dim3(32, 8), 0, stream, partial,
                        (long long)rows, (int)cols, (long long)ld, (long long)(per_block > 0 ? per_block : 1), stage,
                        (int)stage_ld);
    if (rc != TFB_OK) return rc;
    return launch_pdl(colsum_kernel, dim3(col_blocks, 1), dim3(32, 8), 0, stream, (const float*)stage,
                      (long long)kColsumStageBlocks, (int)cols, (long long)stage_ld, (long long)kColsumStageBlocks, out, 0);
}

bool conv_tma_forced() {
    return tuning(TFB_TUNE_CONV_TMA) == 2;
}

bool conv_tma_eligible(const ConvShape& s, int64_t contraction_channels, bool input_gradient) {
    const int mode = tuning(TFB_TUNE_CONV_TMA);   // 0 never, 1 by the rules below, 2 whenever possible
    if (mode == 0) return false;
    // A K block holds 32 channels of one tap: with few channels most of it is zero fill and the
    // gather kernel, which packs taps densely, is faster.
    if (mode == 1 && contraction_channels < 16) return false;
    // A box of positions must be a box of the source traversed with the stride: at most 256 source
    // elements per box dimension (tiles are at most 128 positions wide and high); tensor-map extents
    // and 32-bit tile arithmetic bound the rest.
    if (input_gradient) {
        if (s.sh != 1 || s.sw != 1) return false;
    } else {
        const int64_t tw = 1ll << pow2_ceil_log2(s.outW < 128 ? s.outW : 128), th = 128 / tw;
        if (s.sw > 8 || s.sh > 8 || (tw - 1) * s.sw + 1 > 256 || (th - 1) * s.sh + 1 > 256) return false;
    }
    return s.N >= 1 && s.N < 65536 && s.H < (1 << 15) && s.W < (1 << 15) &&
           s.Cin < (1 << 15) && s.Cout < (1 << 15) && s.kH * s.kW * ((s.Cin + 31) / 32) < (1 << 20) &&
           s.kH * s.kW * ((s.Cout + 31) / 32) < (1 << 20);
}

int conv_tma_forward(const float* x, const float* w, const float* bias, float* out, const ConvShape& s, bool relu,
                     cudaStream_t stream) {
    DeviceState* st = nullptr;
    int rc = device_state(&st);
    if (rc != TFB_OK) return rc;
    const int64_t khw = s.kH * s.kW, P = s.H * s.W, cp = round_up(s.Cin, 4);
    const size_t x_bytes = align256((size_t)(2 * s.N * P * cp) * 4);
    const size_t f_bytes = align256((size_t)(2 * s.Cout * khw * cp) * 4);
    void* ws_v = nullptr;
    rc = workspace_get(stream, x_bytes + f_bytes, &ws_v);
    if (rc != TFB_OK) return rc;
    float* x_hi = static_cast<float*>(ws_v);
    float* x_lo = x_hi + s.N * P * cp;
    float* f_hi = reinterpret_cast<float*>(static_cast<uint8_t*>(ws_v) + x_bytes);
    float* f_lo = f_hi + s.Cout * khw * cp;
    rc = to_nhwc_planes(x, s.N, s.Cin, P, cp, x_hi, x_lo, nullptr, stream);
    if (rc != TFB_OK) return rc;
    const long long ftotal = (long long)s.Cout * khw * cp;
    rc = launch_pdl(filter_planes_kernel, dim3(grid_1d(ftotal)), dim3(256), 0, stream, w, (int)s.Cout, (int)s.Cin, (int)khw,
                    (int)cp, 0, f_hi, f_lo);
    if (rc != TFB_OK) return rc;
    SpatialCall c;
    c.src_hi = x_hi; c.src_lo = x_lo; c.src_c = s.Cin; c.src_cp = cp; c.src_H = s.H; c.src_W = s.W;
    c.f_hi = f_hi; c.f_lo = f_lo; c.J = s.Cout; c.out_H = s.outH; c.out_W = s.outW;
    c.ay0 = (int)-s.ph; c.ay_step = (int)s.dh; c.ax0 = (int)-s.pw; c.ax_step = (int)s.dw;
    c.sy = (int)s.sh; c.sx = (int)s.sw;
    c.dst = out; c.bias = bias; c.relu = relu;
    return run_spatial(c, s, st, stream);
}

int conv_tma_backward(const float* x, const float* w, const float* dY, float* dX, float* dW, float* db,
                      const ConvShape& s, cudaStream_t stream) {
    DeviceState* st = nullptr;
    int rc = device_state(&st);
    if (rc != TFB_OK) return rc;
    const int64_t khw = s.kH * s.kW, P = s.H * s.W, Po = s.outH * s.outW;
    const int64_t cp = round_up(s.Cin, 4), cop = round_up(s.Cout, 4);
    const int64_t pblocks = (Po + 31) / 32;
    const bool want_dx = dX != nullptr, want_dw = dW != nullptr, want_db = db != nullptr;

    // weight-gradient tiling
    const int cblks = (int)((s.Cin + 31) / 32), cp32 = cblks * 32;
    const int64_t ncols = khw * cp32, ld_part = ncols;
    const int bn_w = 128;
    const int kw_log2 = pow2_ceil_log2(s.outW < 32 ? s.outW : 32);
    const int kbw = 1 << kw_log2, kbh = 32 / kbw;
    const int64_t kblk_x = (s.outW + kbw - 1) / kbw, kblk_y = (s.outH + kbh - 1) / kbh;
    const int64_t k_blocks = s.N * kblk_x * kblk_y;
    const int64_t w_tiles_m = (s.Cout + kBlockM - 1) / kBlockM, w_tiles_n = (ncols + bn_w - 1) / bn_w;
    int64_t splits = st->sm_count / (w_tiles_m * w_tiles_n);
    if (splits > k_blocks / 8) splits = k_blocks / 8;
    if (splits > 64) splits = 64;
    if (splits < 1) splits = 1;
    const int64_t kb_per = (k_blocks + splits - 1) / splits;
    splits = (k_blocks + kb_per - 1) / kb_per;
    const int64_t rows_per_split = w_tiles_m * kBlockM;

    size_t off = 0;
    auto take = [&](size_t bytes) { size_t o = off; off += align256(bytes); return o; };
    const size_t o_dy = take((size_t)(2 * s.N * Po * cop) * 4);
    const size_t o_bsum = want_db ? take((size_t)(s.N * pblocks * cop) * 4) : 0;
    const size_t o_bstage = want_db ? take(column_sums_stage_bytes(s.Cout)) : 0;
    const size_t o_fd = want_dx ? take((size_t)(2 * s.Cin * khw * cop) * 4) : 0;
    const size_t o_x = want_dw ? take((size_t)(2 * s.N * P * cp) * 4) : 0;
    const size_t o_part = want_dw ? take((size_t)(splits * rows_per_split * ld_part) * 4) : 0;
    void* ws_v = nullptr;
    rc = workspace_get(stream, off + 256, &ws_v);
    if (rc != TFB_OK) return rc;
    uint8_t* ws = static_cast<uint8_t*>(ws_v);

    float* dy_hi = reinterpret_cast<float*>(ws + o_dy);
    float* dy_lo = dy_hi + s.N * Po * cop;
    float* bsum = want_db ? reinterpret_cast<float*>(ws + o_bsum) : nullptr;
    rc = to_nhwc_planes(dY, s.N, s.Cout, Po, cop, dy_hi, dy_lo, bsum, stream);
    if (rc != TFB_OK) return rc;
    if (want_db) {
        rc = column_sums(bsum, s.N * pblocks, s.Cout, cop, reinterpret_cast<float*>(ws + o_bstage), db, stream);
        if (rc != TFB_OK) return rc;
    }
    if (want_dx) {
        float* f_hi = reinterpret_cast<float*>(ws + o_fd);
        float* f_lo = f_hi + s.Cin * khw * cop;
        const long long ftotal = (long long)s.Cin * khw * cop;
        rc = launch_pdl(filter_planes_kernel, dim3(grid_1d(ftotal)), dim3(256), 0, stream, w, (int)s.Cout, (int)s.Cin,
                        (int)khw, (int)cop, 1, f_hi, f_lo);
        if (rc != TFB_OK) return rc;
        SpatialCall c;
        c.src_hi = dy_hi; c.src_lo = dy_lo; c.src_c = s.Cout; c.src_cp = cop; c.src_H = s.outH; c.src_W = s.outW;
        c.f_hi = f_hi; c.f_lo = f_lo; c.J = s.Cin; c.out_H = s.H; c.out_W = s.W;
        c.ay0 = (int)s.ph; c.ay_step = (int)-s.dh; c.ax0 = (int)s.pw; c.ax_step = (int)-s.dw;
        c.dst = dX; c.bias = nullptr; c.relu = false;
        rc = run_spatial(c, s, st, stream);
        if (rc != TFB_OK) return rc;
    }
    if (want_dw) {
        float* x_hi = reinterpret_cast<float*>(ws + o_x);
        float* x_lo = x_hi + s.N * P * cp;
        rc = to_nhwc_planes(x, s.N, s.Cin, P, cp, x_hi, x_lo, nullptr, stream);
        if (rc != TFB_OK) return rc;
        float* partial = reinterpret_cast<float*>(ws + o_part);

        GemmArgs a;
        memset(&a, 0, sizeof(a));
        a.M = (int)s.Cout; a.N = (int)ncols; a.K = (int)(k_blocks * 32);
        a.tiles_m = (int)w_tiles_m; a.tiles_n = (int)w_tiles_n; a.num_tiles = a.tiles_m * a.tiles_n;
        a.k_blocks = (int)k_blocks; a.chunk_kb = 8;
        a.split_k = (int)splits; a.kb_per_split = (int)kb_per;
        a.split_stride = rows_per_split * ld_part;
        a.group_m = 16;
        a.C = partial; a.ldc = ld_part; a.out_type = kOutF32;
        a.bias = nullptr; a.bias_mode = kBiasNone; a.relu = 0; a.c_tma = 1; a.status = st->status;
        a.cv.cblks = cblks; a.cv.kw = (int)s.kW; a.cv.taps = (int)khw;
        a.cv.ay0 = (int)-s.ph; a.cv.ay_step = (int)s.dh; a.cv.ax0 = (int)-s.pw; a.cv.ax_step = (int)s.dw;
        a.cv.sx = (int)s.sw; a.cv.sy = (int)s.sh;
        a.cv.kblk_w_log2 = kw_log2; a.cv.kblk_h = kbh; a.cv.kblk_x = (int)kblk_x; a.cv.kblk_y = (int)kblk_y;
        a.cv.n_samples = (int)s.N;

        CUtensorMap maps[5];
        memset(maps, 0, sizeof(maps));
        rc = plane_maps(&maps[0], dy_hi, dy_lo, cop, s.outW, s.outH, s.N, (uint32_t)kbw, (uint32_t)kbh, true);
        if (rc != TFB_OK) return rc;
        rc = plane_maps(&maps[2], x_hi, x_lo, cp, s.W, s.H, s.N, (uint32_t)kbw, (uint32_t)kbh, true, (uint32_t)s.sw,
                        (uint32_t)s.sh);
        if (rc != TFB_OK) return rc;
        rc = make_map(&maps[4], TFB_DTYPE_F32, partial, (uint64_t)ncols, (uint64_t)(splits * rows_per_split),
                      (uint64_t)ld_part * 4, 32, 32);
        if (rc != TFB_OK) return rc;
        const long long units = (long long)a.num_tiles * a.split_k;
        const int grid = units < st->sm_count ? (int)units : st->sm_count;
        rc = launch_feed<128, 3, false, kConvWgrad>(maps, a, grid, stream);
        if (rc != TFB_OK) return rc;
        const long long total = (long long)s.Cout * s.Cin * khw;
        rc = launch_pdl(wgrad_planes_reduce_kernel, dim3(grid_1d(total)), dim3(256), 0, stream, (const float*)partial,
                        (int)splits, (long long)(rows_per_split * ld_part), (long long)ld_part, (int)s.Cout, (int)s.Cin,
                        (int)khw, (int)cp32, dW);
        if (rc != TFB_OK) return rc;
    }
    return TFB_OK;
}

}  // namespace tfb
