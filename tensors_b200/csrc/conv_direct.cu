// Direct (CUDA-core) convolution kernels for the shapes whose contraction is too short to feed a tensor
// core: a first layer with 3 input channels has 27 products per output and 13 FLOP per byte, so it is
// bound by HBM traffic and latency, not by arithmetic. One thread owns one position and a strip of
// channels, keeps the partial sums in registers, reads the activations straight from the NCHW tensor
// (lanes = consecutive positions: coalesced) and the filter from shared memory (all lanes read the same
// address: a broadcast). Plain FP32 FMAs in the reference's accumulation order (channel, then filter
// row, then filter column); any stride, padding and dilation.
#include <atomic>
#include <cstdlib>

#include "internal.hpp"

namespace tfb {

namespace {

constexpr int kDirectThreads = 128;
constexpr int kDirectCout = 32;      // output channels per thread in the forward kernel
constexpr int kDirectMaxTaps = 128;  // Cin * kH * kW the forward kernel accepts
constexpr int kDirectCin = 4;        // input channels per thread in the input-gradient kernel
static_assert(kDirectCin == 4, "the input-gradient kernel keeps exactly two accumulator pairs");

struct DirectArgs {
    int N, Cin, H, W, Cout, kH, kW, sh, sw, ph, pw, dh, dw, outH, outW;
};

// out[n][co][p] = bias[co] + sum_k x[n][c][iy][ix] * w[co][k], k = (c, ki, kj) ascending.
// grid = (position blocks, Cout / kDirectCout, N).
__global__ void __launch_bounds__(kDirectThreads)
conv_direct_forward_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ bias,
                           float* __restrict__ out, const DirectArgs a, int relu) {
    __shared__ __align__(16) float w_s[kDirectMaxTaps][kDirectCout];
    const int taps = a.Cin * a.kH * a.kW;
    const int co0 = blockIdx.y * kDirectCout;
    // consecutive threads read consecutive filter elements (the strip's rows are contiguous in w)
    for (int i = threadIdx.x; i < taps * kDirectCout; i += kDirectThreads) {
        const int j = i / taps, k = i - j * taps;
        w_s[k][j] = (co0 + j < a.Cout) ? w[(long long)co0 * taps + i] : 0.f;
    }
    __syncthreads();
    const int P = a.outH * a.outW;
    const int p = blockIdx.x * kDirectThreads + threadIdx.x;
    if (p >= P) return;
    const int n = blockIdx.z;
    const int oy = p / a.outW, ox = p - oy * a.outW;
    const int iy0 = oy * a.sh - a.ph, ix0 = ox * a.sw - a.pw;
    // Accumulators in pairs: sm_100 issues two FP32 FMAs per instruction on packed operands.
    float2 acc2[kDirectCout / 2];
#pragma unroll
    for (int j = 0; j < kDirectCout / 2; ++j) acc2[j] = make_float2(0.f, 0.f);
    const float* xs = x + (long long)n * a.Cin * a.H * a.W;
    int k = 0;
    for (int c = 0; c < a.Cin; ++c) {
        const float* xc = xs + (long long)c * a.H * a.W;
        for (int ki = 0; ki < a.kH; ++ki) {
            const int iy = iy0 + ki * a.dh;
            const bool row_ok = iy >= 0 && iy < a.H;
            for (int kj = 0; kj < a.kW; ++kj, ++k) {
                const int ix = ix0 + kj * a.dw;
                const float v = (row_ok && ix >= 0 && ix < a.W) ? __ldg(xc + (long long)iy * a.W + ix) : 0.f;
                const float2 vv = make_float2(v, v);
                const float4* wr = reinterpret_cast<const float4*>(w_s[k]);
#pragma unroll
                for (int j = 0; j < kDirectCout / 4; ++j) {
                    const float4 ww = wr[j];
                    acc2[2 * j] = __ffma2_rn(vv, make_float2(ww.x, ww.y), acc2[2 * j]);
                    acc2[2 * j + 1] = __ffma2_rn(vv, make_float2(ww.z, ww.w), acc2[2 * j + 1]);
                }
            }
        }
    }
    float* o = out + ((long long)n * a.Cout + co0) * P + p;
#pragma unroll
    for (int j = 0; j < kDirectCout; ++j) {
        if (co0 + j < a.Cout) {
            float r = ((j & 1) ? acc2[j >> 1].y : acc2[j >> 1].x) + (bias != nullptr ? __ldg(bias + co0 + j) : 0.f);
            if (relu) r = r > 0.f ? r : 0.f;
            o[(long long)j * P] = r;
        }
    }
}

// The same sums for stride 1, dilation 1 and a filter shape known at compile time, with every loop unrolled
// and no index arithmetic in it: a block of four warps computes an 8-row x 32-column tile of output
// positions of one sample for ALL output channels. The input patch the tile reads ((8 + KH - 1) x
// (32 + KW - 1) x CIN values, zero outside the image, so the padding needs no test) and the whole filter sit
// in shared memory; a thread owns two vertically adjacent positions (their input rows overlap, so the
// KH + 1 rows it reads serve both) and a strip of 32 channels at a time: per filter tap 8 broadcast
// 16-byte reads of the filter row feed 32 two-wide FMAs. Same accumulation order as the kernel above.
constexpr int kTileRows = 8, kTileCols = 32, kTiledThreads = 128;

template <int CIN, int KH, int KW>
__global__ void __launch_bounds__(kTiledThreads)
conv_direct_forward_tiled_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ bias,
                                 float* __restrict__ out, const DirectArgs a, int relu, int cout_pad) {
    constexpr int TAPS = CIN * KH * KW, PH = kTileRows + KH - 1, PW = kTileCols + KW - 1;
    extern __shared__ __align__(16) float tiled_s[];
    float* w_s = tiled_s;                          // [TAPS][cout_pad]
    float* patch = tiled_s + TAPS * cout_pad;      // [CIN][PH][PW]
    const int n = blockIdx.z, oy0 = blockIdx.y * kTileRows, ox0 = blockIdx.x * kTileCols;
    for (int i = threadIdx.x; i < TAPS * cout_pad; i += kTiledThreads) {
        const int k = i / cout_pad, co = i - k * cout_pad;
        w_s[i] = co < a.Cout ? __ldg(w + (long long)co * TAPS + k) : 0.f;
    }
    const float* xs = x + (long long)n * CIN * a.H * a.W;
    for (int i = threadIdx.x; i < CIN * PH * PW; i += kTiledThreads) {
        const int c = i / (PH * PW), r = (i - c * PH * PW) / PW, q = i - c * PH * PW - r * PW;
        const int iy = oy0 - a.ph + r, ix = ox0 - a.pw + q;
        patch[i] = (iy >= 0 && iy < a.H && ix >= 0 && ix < a.W) ? __ldg(xs + ((long long)c * a.H + iy) * a.W + ix) : 0.f;
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, ry = 2 * (threadIdx.x >> 5);
    const int oy = oy0 + ry, ox = ox0 + lane;
    const long long P = (long long)a.outH * a.outW;
    for (int strip = 0; strip < cout_pad; strip += 32) {
        float2 acc0[16], acc1[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) acc0[j] = acc1[j] = make_float2(0.f, 0.f);
#pragma unroll
        for (int c = 0; c < CIN; ++c) {
            float v[KH + 1][KW];
#pragma unroll
            for (int r = 0; r < KH + 1; ++r)
#pragma unroll
                for (int q = 0; q < KW; ++q) v[r][q] = patch[(c * PH + ry + r) * PW + lane + q];
#pragma unroll
            for (int ki = 0; ki < KH; ++ki)
#pragma unroll
                for (int kj = 0; kj < KW; ++kj) {
                    const float4* wr = reinterpret_cast<const float4*>(w_s + ((c * KH + ki) * KW + kj) * cout_pad + strip);
                    const float2 p0 = make_float2(v[ki][kj], v[ki][kj]), p1 = make_float2(v[ki + 1][kj], v[ki + 1][kj]);
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const float4 ww = wr[j];
                        acc0[2 * j] = __ffma2_rn(p0, make_float2(ww.x, ww.y), acc0[2 * j]);
                        acc0[2 * j + 1] = __ffma2_rn(p0, make_float2(ww.z, ww.w), acc0[2 * j + 1]);
                        acc1[2 * j] = __ffma2_rn(p1, make_float2(ww.x, ww.y), acc1[2 * j]);
                        acc1[2 * j + 1] = __ffma2_rn(p1, make_float2(ww.z, ww.w), acc1[2 * j + 1]);
                    }
                }
        }
        if (ox < a.outW) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                const int co = strip + j;
                if (co < a.Cout) {
                    const float b = bias != nullptr ? __ldg(bias + co) : 0.f;
                    float r0 = ((j & 1) ? acc0[j >> 1].y : acc0[j >> 1].x) + b;
                    float r1 = ((j & 1) ? acc1[j >> 1].y : acc1[j >> 1].x) + b;
                    if (relu) {
                        r0 = r0 > 0.f ? r0 : 0.f;
                        r1 = r1 > 0.f ? r1 : 0.f;
                    }
                    float* o = out + ((long long)n * a.Cout + co) * P + (long long)oy * a.outW + ox;
                    if (oy < a.outH) o[0] = r0;
                    if (oy + 1 < a.outH) o[a.outW] = r1;
                }
            }
        }
    }
}

// dX[n][c][y][x] = sum over (ki, kj, co) of dY[n][co][oy][ox] * w[co][c][ki][kj] with
// oy = (y + ph - ki * dh) / sh where that division is exact and in range (x alike) — the gather form
// of the transposed convolution: no atomics, a fixed order. One thread owns one input position and up
// to kDirectCin input channels; grid = (position blocks, ceil(Cin / kDirectCin), N).
// Shared memory: the filter slice w_s[co * khw + tap][c], (Cout * khw * kDirectCin) floats.
__global__ void __launch_bounds__(kDirectThreads)
conv_direct_dgrad_kernel(const float* __restrict__ dY, const float* __restrict__ w, float* __restrict__ dX,
                         const DirectArgs a) {
    extern __shared__ __align__(16) float wd_s[];
    const int khw = a.kH * a.kW;
    const int c0 = blockIdx.y * kDirectCin;
    for (int i = threadIdx.x; i < a.Cout * khw * kDirectCin; i += kDirectThreads) {
        const int c = i % kDirectCin, r = i / kDirectCin;   // r = co * khw + tap
        const int co = r / khw, tap = r - co * khw;
        wd_s[i] = (c0 + c < a.Cin) ? __ldg(w + ((long long)co * a.Cin + c0 + c) * khw + tap) : 0.f;
    }
    __syncthreads();
    const int P = a.H * a.W, Po = a.outH * a.outW;
    const int p = blockIdx.x * kDirectThreads + threadIdx.x;
    if (p >= P) return;
    const int n = blockIdx.z;
    const int y = p / a.W, xx = p - y * a.W;
    float2 a01 = make_float2(0.f, 0.f), a23 = make_float2(0.f, 0.f);
    const float* g = dY + (long long)n * a.Cout * Po;
    for (int ki = 0; ki < a.kH; ++ki) {
        const int ny = y + a.ph - ki * a.dh;
        if (ny < 0 || ny % a.sh != 0) continue;
        const int oy = ny / a.sh;
        if (oy >= a.outH) continue;
        for (int kj = 0; kj < a.kW; ++kj) {
            const int nx = xx + a.pw - kj * a.dw;
            if (nx < 0 || nx % a.sw != 0) continue;
            const int ox = nx / a.sw;
            if (ox >= a.outW) continue;
            const float* gp = g + (long long)oy * a.outW + ox;
            const float4* wr = reinterpret_cast<const float4*>(wd_s) + (ki * a.kW + kj);
#pragma unroll 4
            for (int co = 0; co < a.Cout; ++co) {
                const float v = __ldg(gp + (long long)co * Po);
                const float4 ww = wr[co * khw];
                a01 = __ffma2_rn(make_float2(v, v), make_float2(ww.x, ww.y), a01);
                a23 = __ffma2_rn(make_float2(v, v), make_float2(ww.z, ww.w), a23);
            }
        }
    }
    const float acc[kDirectCin] = {a01.x, a01.y, a23.x, a23.y};
#pragma unroll
    for (int c = 0; c < kDirectCin; ++c)
        if (c0 + c < a.Cin) dX[((long long)n * a.Cin + c0 + c) * P + p] = acc[c];
}

// Weight and bias gradient for short filters (Cin * kH * kW + 1 <= 32):
//   dW[co][k] = sum over samples and positions of dY[n][co][p] * x[n][c][iy][ix],  db[co] = sum of dY[n][co][p].
// A block takes one sample and `chunks` runs of 128 output positions: it stages the dY tile
// (64 channels x 128 positions) and the gathered activation patch (one row per filter tap, plus a row of
// ones whose product is the bias gradient) in shared memory and multiplies them there; thread
// (channel, tap group) keeps 8 sums in registers, walking the positions in ascending order. Each block
// writes its 64 x 32 partial result; column_sums adds the blocks in a fixed order.
constexpr int kWgPositions = 128, kWgCout = 64, kWgTaps = 32, kWgLd = kWgPositions + 4, kWgThreads = 256;
constexpr size_t kWgSmem = (size_t)(kWgCout + kWgTaps) * kWgLd * sizeof(float);

__global__ void __launch_bounds__(kWgThreads)
conv_direct_wgrad_kernel(const float* __restrict__ x, const float* __restrict__ dY, float* __restrict__ partial,
                         const DirectArgs a, int chunks, int chunk_groups, int cout_pad) {
    extern __shared__ __align__(16) float wg_s[];
    float (*dy_s)[kWgLd] = reinterpret_cast<float (*)[kWgLd]>(wg_s);
    float (*xc_s)[kWgLd] = reinterpret_cast<float (*)[kWgLd]>(wg_s + kWgCout * kWgLd);
    const int taps = a.Cin * a.kH * a.kW, khw = a.kH * a.kW;
    const int Po = a.outH * a.outW;
    const int n = blockIdx.z, co0 = blockIdx.y * kWgCout;
    // thread (channel co_i, kq) owns taps k = 4 * j + kq, j < 8: the four kq of a channel read four
    // different shared-memory rows whose bank offsets differ, so the reads do not conflict
    const int co_i = threadIdx.x >> 2, kq = threadIdx.x & 3;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    const float* xs = x + (long long)n * a.Cin * a.H * a.W;
    const float* gs = dY + ((long long)n * a.Cout + co0) * Po;
    for (int ch = 0; ch < chunks; ++ch) {
        const int p0 = (blockIdx.x * chunks + ch) * kWgPositions;
        if (p0 >= Po) break;
        for (int i = threadIdx.x; i < kWgCout * kWgPositions; i += kWgThreads) {
            const int co = i / kWgPositions, p = i - co * kWgPositions;
            dy_s[co][p] = (co0 + co < a.Cout && p0 + p < Po) ? __ldg(gs + (long long)co * Po + p0 + p) : 0.f;
        }
        for (int i = threadIdx.x; i < kWgTaps * kWgPositions; i += kWgThreads) {
            const int k = i / kWgPositions, p = i - k * kWgPositions;
            float v = 0.f;
            if (p0 + p < Po) {
                if (k < taps) {
                    const int c = k / khw, r = k - c * khw, ki = r / a.kW, kj = r - ki * a.kW;
                    const int oy = (p0 + p) / a.outW, ox = (p0 + p) - oy * a.outW;
                    const int iy = oy * a.sh - a.ph + ki * a.dh, ix = ox * a.sw - a.pw + kj * a.dw;
                    if (iy >= 0 && iy < a.H && ix >= 0 && ix < a.W) v = __ldg(xs + ((long long)c * a.H + iy) * a.W + ix);
                } else if (k == taps) {
                    v = 1.f;
                }
            }
            xc_s[k][p] = v;
        }
        __syncthreads();
#pragma unroll 2
        for (int p = 0; p < kWgPositions; p += 4) {
            const float4 g = *reinterpret_cast<const float4*>(&dy_s[co_i][p]);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float4 b = *reinterpret_cast<const float4*>(&xc_s[4 * j + kq][p]);
                acc[j] = fmaf(g.x, b.x, acc[j]);
                acc[j] = fmaf(g.y, b.y, acc[j]);
                acc[j] = fmaf(g.z, b.z, acc[j]);
                acc[j] = fmaf(g.w, b.w, acc[j]);
            }
        }
        __syncthreads();
    }
    float* out = partial + (((long long)n * chunk_groups + blockIdx.x) * cout_pad + co0 + co_i) * kWgTaps + kq;
#pragma unroll
    for (int j = 0; j < 8; ++j) out[4 * j] = acc[j];
}

// dW[co][k] = sums[co * 32 + k] for k < taps; db[co] = sums[co * 32 + taps].
__global__ void wgrad_direct_finish_kernel(const float* __restrict__ sums, int Cout, int taps, float* __restrict__ dW,
                                           float* __restrict__ db) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= Cout * kWgTaps) return;
    const int co = i / kWgTaps, k = i - co * kWgTaps;
    if (k < taps) {
        if (dW != nullptr) dW[(long long)co * taps + k] = sums[i];
    } else if (k == taps && db != nullptr) {
        db[co] = sums[i];
    }
}

DirectArgs direct_args(const ConvShape& s) {
    return DirectArgs{(int)s.N, (int)s.Cin, (int)s.H, (int)s.W, (int)s.Cout, (int)s.kH, (int)s.kW, (int)s.sh,
                      (int)s.sw, (int)s.ph, (int)s.pw, (int)s.dh, (int)s.dw, (int)s.outH, (int)s.outW};
}

template <int CIN, int KH, int KW>
int launch_forward_tiled(const float* x, const float* w, const float* bias, float* out, const ConvShape& s, bool relu,
                         cudaStream_t stream) {
    const int cout_pad = (int)((s.Cout + 31) / 32 * 32);
    const size_t smem = (size_t)(CIN * KH * KW * cout_pad + CIN * (kTileRows + KH - 1) * (kTileCols + KW - 1)) * sizeof(float);
    dim3 grid((unsigned)((s.outW + kTileCols - 1) / kTileCols), (unsigned)((s.outH + kTileRows - 1) / kTileRows), (unsigned)s.N);
    conv_direct_forward_tiled_kernel<CIN, KH, KW><<<grid, kTiledThreads, smem, stream>>>(x, w, bias, out, direct_args(s),
                                                                                         relu ? 1 : 0, cout_pad);
    TFB_CUDA_OK(cudaGetLastError());
    return TFB_OK;
}

bool direct_enabled() {
    return tuning(TFB_TUNE_CONV_DIRECT) != 0;
}

constexpr size_t kDgradSmemLimit = 200 * 1024;

}  // namespace

bool conv_direct_forward_eligible(const ConvShape& s) {
    return direct_enabled() && s.Cin * s.kH * s.kW <= kDirectMaxTaps && s.N < 65536 &&
           (s.Cout + kDirectCout - 1) / kDirectCout < 65536 && s.outH * s.outW < (1ll << 31) - kDirectThreads;
}

bool conv_direct_dgrad_eligible(const ConvShape& s) {
    return direct_enabled() && s.Cin <= kDirectCin && s.N < 65536 &&
           (size_t)(s.Cout * s.kH * s.kW * kDirectCin) * 4 <= kDgradSmemLimit && s.H * s.W < (1ll << 31) - kDirectThreads;
}

int conv_direct_forward(const float* x, const float* w, const float* bias, float* out, const ConvShape& s, bool relu,
                        cudaStream_t stream) {
    // stride 1, no dilation, a filter shape with an unrolled instance, the filter within 40 KB of shared memory
    if (s.sh == 1 && s.sw == 1 && s.dh == 1 && s.dw == 1 && s.kH == 3 && s.kW == 3 && s.Cout <= 256 &&
        (s.outH + kTileRows - 1) / kTileRows < 65536) {
        if (s.Cin == 3) return launch_forward_tiled<3, 3, 3>(x, w, bias, out, s, relu, stream);
        if (s.Cin == 1) return launch_forward_tiled<1, 3, 3>(x, w, bias, out, s, relu, stream);
        if (s.Cin == 4) return launch_forward_tiled<4, 3, 3>(x, w, bias, out, s, relu, stream);
    }
    const long long P = s.outH * s.outW;
    dim3 grid((unsigned)((P + kDirectThreads - 1) / kDirectThreads), (unsigned)((s.Cout + kDirectCout - 1) / kDirectCout),
              (unsigned)s.N);
    conv_direct_forward_kernel<<<grid, kDirectThreads, 0, stream>>>(x, w, bias, out, direct_args(s), relu ? 1 : 0);
    TFB_CUDA_OK(cudaGetLastError());
    return TFB_OK;
}

int conv_direct_dgrad(const float* dY, const float* w, float* dX, const ConvShape& s, cudaStream_t stream) {
    const long long P = s.H * s.W;
    const size_t smem = (size_t)(s.Cout * s.kH * s.kW * kDirectCin) * 4;
    static std::atomic<size_t> attr_set[64];   // per device; several host threads may get here at once
    int dev = 0;
    TFB_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(TFB_ERR_UNSUPPORTED, "device index %d out of range", dev);
    if (smem > 48 * 1024 && attr_set[dev].load(std::memory_order_acquire) < smem) {
        TFB_CUDA_OK(cudaFuncSetAttribute(conv_direct_dgrad_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)kDgradSmemLimit));
        attr_set[dev].store(kDgradSmemLimit, std::memory_order_release);
    }
    dim3 grid((unsigned)((P + kDirectThreads - 1) / kDirectThreads), (unsigned)((s.Cin + kDirectCin - 1) / kDirectCin),
              (unsigned)s.N);
    conv_direct_dgrad_kernel<<<grid, kDirectThreads, smem, stream>>>(dY, w, dX, direct_args(s));
    TFB_CUDA_OK(cudaGetLastError());
    return TFB_OK;
}

}  // namespace tfb

namespace tfb {

bool conv_direct_wgrad_eligible(const ConvShape& s) {
    return direct_enabled() && s.Cin * s.kH * s.kW + 1 <= kWgTaps && s.N < 65536 &&
           (s.Cout + kWgCout - 1) / kWgCout < 65536 && s.outH * s.outW < (1ll << 30);
}

int conv_direct_wgrad(const float* x, const float* dY, float* dW, float* db, const ConvShape& s, cudaStream_t stream) {
    DeviceState* st = nullptr;
    int rc = device_state(&st);
    if (rc != TFB_OK) return rc;
    const int64_t Po = s.outH * s.outW;
    const int64_t pos_chunks = (Po + kWgPositions - 1) / kWgPositions;
    const int64_t co_tiles = (s.Cout + kWgCout - 1) / kWgCout, cout_pad = co_tiles * kWgCout;
    // enough blocks to fill the GPU a few times over, few enough partial results to add up quickly
    int64_t chunks = 1;
    while (chunks < pos_chunks && s.N * co_tiles * ((pos_chunks + chunks - 1) / chunks) > 8ll * st->sm_count) chunks *= 2;
    const int64_t chunk_groups = (pos_chunks + chunks - 1) / chunks;
    const int64_t rows = s.N * chunk_groups, cols = cout_pad * kWgTaps;
    const size_t part_bytes = ((size_t)(rows * cols) * 4 + 255) & ~(size_t)255;
    const size_t sums_bytes = ((size_t)cols * 4 + 255) & ~(size_t)255;
    void* ws_v = nullptr;
    rc = workspace_get(stream, part_bytes + sums_bytes + column_sums_stage_bytes(cols) + 256, &ws_v);
    if (rc != TFB_OK) return rc;
    float* partial = static_cast<float*>(ws_v);
    float* sums = reinterpret_cast<float*>(static_cast<uint8_t*>(ws_v) + part_bytes);
    float* stage = reinterpret_cast<float*>(static_cast<uint8_t*>(ws_v) + part_bytes + sums_bytes);
    static std::atomic<bool> attr_set[64];
    int dev = 0;
    TFB_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(TFB_ERR_UNSUPPORTED, "device index %d out of range", dev);
    if (!attr_set[dev].load(std::memory_order_acquire)) {
        TFB_CUDA_OK(cudaFuncSetAttribute(conv_direct_wgrad_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kWgSmem));
        attr_set[dev].store(true, std::memory_order_release);
    }
    dim3 grid((unsigned)chunk_groups, (unsigned)co_tiles, (unsigned)s.N);
    conv_direct_wgrad_kernel<<<grid, kWgThreads, kWgSmem, stream>>>(x, dY, partial, direct_args(s), (int)chunks,
                                                                    (int)chunk_groups, (int)cout_pad);
    TFB_CUDA_OK(cudaGetLastError());
    rc = column_sums(partial, rows, cols, cols, stage, sums, stream);
    if (rc != TFB_OK) return rc;
    const int total = (int)(s.Cout * kWgTaps);
    wgrad_direct_finish_kernel<<<(total + 255) / 256, 256, 0, stream>>>(sums, (int)s.Cout, (int)(s.Cin * s.kH * s.kW), dW, db);
    TFB_CUDA_OK(cudaGetLastError());
    return TFB_OK;
}

}  // namespace tfb
