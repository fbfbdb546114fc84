// Host side of the implicit-GEMM convolution: tap tables, operand preparation, tiling, launches,
// and the extern "C" entry points of nn::Conv2d forward / backward.
#include <atomic>
#include <cstring>

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <vector>

#include "conv_kernel.cuh"
#include "internal.hpp"

namespace tfb {

namespace {

inline int64_t round_up(int64_t x, int64_t m) { return (x + m - 1) / m * m; }
inline size_t align256(size_t x) { return (x + 255) & ~(size_t)255; }

__device__ __forceinline__ float tf32_rna_h(float x) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return __uint_as_float(r);
}

// dgrad weights: Wd[c][(co*kH + ki)*kW + kj] = W[co][c][ki][kj], written as TF32 hi / lo planes
// with leading dimension ld (padding zero-filled).
__global__ void dgrad_weight_kernel(const float* __restrict__ W, float* __restrict__ hi, float* __restrict__ lo,
                                    int Cout, int Cin, int khw, int ld) {
    const int total = Cin * ld;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        const int c = i / ld, t = i - c * ld;
        float v = 0.f;
        if (t < Cout * khw) {
            const int co = t / khw, r = t - co * khw;
            v = W[((long long)co * Cin + c) * khw + r];
        }
        const float h = tf32_rna_h(v);
        hi[i] = h;
        lo[i] = v - h;
    }
}

// dW[co][t] = Σ_s partial[s][co][t] for t < taps; db[co] = Σ_s partial[s][co][taps], in a fixed order.
__global__ void wgrad_reduce_kernel(const float* __restrict__ partial, int splits, int Cout, int taps,
                                    int taps_total, float* __restrict__ dW, float* __restrict__ db) {
    const int total = Cout * taps_total;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        const int co = i / taps_total, t = i - co * taps_total;
        // eight independent running sums (splits k, k + 8, ... each) keep eight loads in flight; they
        // are combined in a fixed order, so the result does not depend on the launch
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int k = 0; k < splits; k += 8) {
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if (k + j < splits) acc[j] += partial[(long long)(k + j) * total + i];
        }
        const float s = ((acc[0] + acc[1]) + (acc[2] + acc[3])) + ((acc[4] + acc[5]) + (acc[6] + acc[7]));
        if (t < taps) {
            if (dW != nullptr) dW[(long long)co * taps + t] = s;
        } else if (t == taps && db != nullptr) {
            db[co] = s;
        }
    }
}

// Writes, for every column-matrix element (n, t, p) of samples [n0, n0 + count), the flat NCHW
// input offset the forward producers read for it, or -1 for padding — evaluated with the same
// tap table and offset function as the convolution kernel.
__global__ void index_map_kernel(long long* __restrict__ out, const TapInfo* __restrict__ table,
                                 const ConvArgs args, int n0, int count, int taps, long long sample_elems) {
    const long long per_n = (long long)taps * args.pos_count;
    const long long total = per_n * count;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const long long n = i / per_n;
        const long long rem = i - n * per_n;
        const int t = (int)(rem / args.pos_count);
        const int p = (int)(rem - (long long)t * args.pos_count);
        const int oy = p / args.pos_W, ox = p - oy * args.pos_W;
        const int y0 = oy * args.mul_h, x0 = ox * args.mul_w;
        int off;
        if (args.kH <= 32 && args.kW <= 32) {   // what the forward producers evaluate
            const uint32_t ymask = conv_axis_mask(y0, args.ay0, args.ay_step, args.kH, args.src_H);
            const uint32_t xmask = conv_axis_mask(x0, args.ax0, args.ax_step, args.kW, args.src_W);
            if (args.kH * args.kW <= 30) {
                const uint32_t vmask = conv_combined_mask(ymask, xmask, args.kH, args.kW, true);
                const bool valid = ((vmask >> ((uint32_t)table[t].kidx >> 16)) & 1u) != 0;
                off = valid ? y0 * args.src_W + x0 + table[t].delta : -1;
            } else {
                off = conv_src_offset_fast(table[t], y0 * args.src_W + x0, ymask, xmask);
            }
        } else {
            off = conv_src_offset<kConvFprop>(table[t], y0, x0, args);
        }
        out[i] = off >= 0 ? (n0 + n) * sample_elems + off : -1;
    }
}

template <int MODE, int BN, int STAGES>
int launch_conv(const CUtensorMap maps[2], const ConvArgs& args, int grid, size_t table_bytes, cudaStream_t stream) {
    using S = ConvSmem<BN, STAGES>;
    auto kern = conv_igemm_kernel<MODE, BN, STAGES>;
    const size_t smem = (size_t)S::fixed() + table_bytes;
    // largest size set so far per (kernel variant, device); several host threads may get here at once
    static std::atomic<size_t> attr_set[64];
    int dev = 0;
    TFB_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(TFB_ERR_UNSUPPORTED, "device index %d out of range", dev);
    if (attr_set[dev].load(std::memory_order_acquire) < smem) {
        TFB_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr_set[dev].store(smem, std::memory_order_release);
    }
    kern<<<grid, kConvThreads, smem, stream>>>(maps[0], maps[1], args);
    TFB_CUDA_OK(cudaGetLastError());
    return TFB_OK;
}

constexpr size_t kMaxSmem = 232448;

template <int MODE>
int dispatch_conv(int bn, const CUtensorMap maps[2], const ConvArgs& args, int grid, cudaStream_t stream) {
    const size_t table_bytes = (size_t)args.taps_table * sizeof(TapInfo);
    if (bn == 64) {
        if (ConvSmem<64, 4>::fixed() + table_bytes <= kMaxSmem)
            return launch_conv<MODE, 64, 4>(maps, args, grid, table_bytes, stream);
        if (ConvSmem<64, 2>::fixed() + table_bytes <= kMaxSmem)
            return launch_conv<MODE, 64, 2>(maps, args, grid, table_bytes, stream);
    } else {
        if (ConvSmem<128, 3>::fixed() + table_bytes <= kMaxSmem)
            return launch_conv<MODE, 128, 3>(maps, args, grid, table_bytes, stream);
        if (ConvSmem<128, 2>::fixed() + table_bytes <= kMaxSmem)
            return launch_conv<MODE, 128, 2>(maps, args, grid, table_bytes, stream);
    }
    return fail(TFB_ERR_TOO_LARGE, "conv2d: %d filter taps exceed the shared-memory tap table", args.taps);
}

int check_shape(const ConvShape& s) {
    if (s.N < 0 || s.Cin <= 0 || s.H <= 0 || s.W <= 0 || s.Cout <= 0 || s.kH <= 0 || s.kW <= 0 || s.sh <= 0 ||
        s.sw <= 0 || s.ph < 0 || s.pw < 0 || s.dh <= 0 || s.dw <= 0)
        return fail(TFB_ERR_INVALID_ARG, "conv2d: non-positive extent, stride or dilation");
    if (s.outH <= 0 || s.outW <= 0) return fail(TFB_ERR_INVALID_ARG, "conv2d: empty output");
    if (s.Cin * s.H * s.W >= (1ll << 31) || s.Cout * s.outH * s.outW >= (1ll << 31) ||
        s.Cin * s.kH * s.kW >= (1 << 20) || s.Cout * s.kH * s.kW >= (1 << 20) || s.N >= (1 << 24))
        return fail(TFB_ERR_TOO_LARGE, "conv2d: a sample or the filter exceeds the 32-bit index range");
    return TFB_OK;
}

// Tap table for gathers from a tensor with `planes` channels of plane_elems elements each:
// forward form (ay = ki*d - pad) or gradient form (ay = pad - ki*d). Built on the device so that a
// convolution call enqueues no host-to-device copy.
struct TapParams {
    int planes, plane_elems, src_W, kH, kW, ph, pw, dh, dw, gradient_form, ones_tap, table_len;
};

__global__ void build_taps_kernel(TapInfo* __restrict__ table, const TapParams p) {
    const int khw = p.kH * p.kW;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < p.table_len; i += gridDim.x * blockDim.x) {
        TapInfo ti;
        ti.delta = 0;
        ti.kidx = 31 << 16;
        if (i < p.planes * khw) {
            const int ch = i / khw, r = i - ch * khw, ki = r / p.kW, kj = r - ki * p.kW;
            ti.plane_off = ch * p.plane_elems;
            ti.ay = (short)(p.gradient_form ? p.ph - ki * p.dh : ki * p.dh - p.ph);
            ti.ax = (short)(p.gradient_form ? p.pw - kj * p.dw : kj * p.dw - p.pw);
            ti.delta = ti.plane_off + (int)ti.ay * p.src_W + (int)ti.ax;
            ti.kidx = ki | (kj << 8) | ((khw <= 30 ? ki * p.kW + kj : 31) << 16);
        } else {
            ti.plane_off = (p.ones_tap && i == p.planes * khw) ? -2 : -1;
            if (ti.plane_off == -2) ti.kidx = 30 << 16;
            ti.ay = ti.ax = 0;
        }
        table[i] = ti;
    }
}

int build_taps(TapInfo* table_d, int64_t planes, int64_t plane_elems, int64_t src_W, const ConvShape& s,
               bool gradient_form, bool ones_tap, int64_t table_len, cudaStream_t stream) {
    TapParams p{(int)planes, (int)plane_elems, (int)src_W, (int)s.kH, (int)s.kW, (int)s.ph, (int)s.pw,
                (int)s.dh, (int)s.dw, gradient_form ? 1 : 0, ones_tap ? 1 : 0, (int)table_len};
    build_taps_kernel<<<(unsigned)((table_len + 255) / 256), 256, 0, stream>>>(table_d, p);
    TFB_CUDA_OK(cudaGetLastError());
    return TFB_OK;
}

void fill_forward_geometry(ConvArgs& a, const ConvShape& s, const float* x) {
    a.src = x;
    a.src_sample = s.Cin * s.H * s.W;
    a.src_H = (int)s.H; a.src_W = (int)s.W;
    a.div_h = a.div_w = 1;
    a.kH = (int)s.kH; a.kW = (int)s.kW;
    a.ay0 = (int)-s.ph; a.ay_step = (int)s.dh;
    a.ax0 = (int)-s.pw; a.ax_step = (int)s.dw;
    a.mul_h = (int)s.sh; a.mul_w = (int)s.sw;
    a.pos_W = (int)s.outW;
    a.pos_count = (int)(s.outH * s.outW);
    a.n_samples = (int)s.N;
}

}  // namespace

int conv2d_forward(const float* x, const float* w, const float* bias, float* out, const ConvShape& s, bool relu,
                   cudaStream_t stream) {
    int rc = check_shape(s);
    if (rc != TFB_OK) return rc;
    if (s.N == 0) return TFB_OK;
    if (conv_tma_eligible(s, s.Cin)) return conv_tma_forward(x, w, bias, out, s, relu, stream);
    if (conv_direct_forward_eligible(s)) return conv_direct_forward(x, w, bias, out, s, relu, stream);
    DeviceState* st = nullptr;
    rc = device_state(&st);
    if (rc != TFB_OK) return rc;
    const int64_t taps = s.Cin * s.kH * s.kW, ldw = round_up(taps, 4);
    const int64_t table_len = round_up(taps, 128);
    const size_t w_bytes = align256((size_t)(2 * s.Cout * ldw) * 4);
    const size_t table_bytes = align256((size_t)table_len * sizeof(TapInfo));
    void* ws_v = nullptr;
    rc = workspace_get(stream, w_bytes + table_bytes, &ws_v);
    if (rc != TFB_OK) return rc;
    uint8_t* ws = static_cast<uint8_t*>(ws_v);
    float* w_hi = reinterpret_cast<float*>(ws);
    float* w_lo = w_hi + s.Cout * ldw;
    TapInfo* table_d = reinterpret_cast<TapInfo*>(ws + w_bytes);
    rc = build_taps(table_d, s.Cin, s.H * s.W, s.W, s, false, false, table_len, stream);
    if (rc != TFB_OK) return rc;
    rc = split_operand(w, s.Cout, taps, taps, nullptr, w_hi, w_lo, ldw, stream);
    if (rc != TFB_OK) return rc;

    const int bn = s.Cout <= 64 ? 64 : 128;
    ConvArgs a;
    memset(&a, 0, sizeof(a));
    fill_forward_geometry(a, s, x);
    a.taps = (int)taps; a.taps_table = (int)table_len; a.tap_table = table_d;
    a.dst = out; a.J = (int)s.Cout; a.rows_ext = a.pos_count;
    a.bias = bias; a.relu = relu ? 1 : 0;
    a.row_tiles = (a.pos_count + 127) / 128;
    a.col_tiles = (int)((s.Cout + bn - 1) / bn);
    a.num_tiles = (int)(s.N * a.row_tiles * a.col_tiles);
    a.k_blocks = (int)((taps + 31) / 32);
    a.pos_blocks = 0; a.splits = 1; a.chunk_kb = 8; a.b_rows_per_sample = 0;
    a.status = st->status;
    CUtensorMap maps[2];
    rc = make_map(&maps[0], TFB_DTYPE_F32, w_hi, (uint64_t)ldw, (uint64_t)s.Cout, (uint64_t)ldw * 4, 32, bn);
    if (rc != TFB_OK) return rc;
    rc = make_map(&maps[1], TFB_DTYPE_F32, w_lo, (uint64_t)ldw, (uint64_t)s.Cout, (uint64_t)ldw * 4, 32, bn);
    if (rc != TFB_OK) return rc;
    const int grid = a.num_tiles < st->sm_count ? a.num_tiles : st->sm_count;
    return dispatch_conv<kConvFprop>(bn, maps, a, grid, stream);
}

int conv2d_backward(const float* x, const float* w, const float* dY, float* dX, float* dW, float* db,
                    const ConvShape& s, cudaStream_t stream) {
    int rc = check_shape(s);
    if (rc != TFB_OK) return rc;
    DeviceState* st = nullptr;
    rc = device_state(&st);
    if (rc != TFB_OK) return rc;
    const int64_t khw = s.kH * s.kW, P = s.outH * s.outW;
    if (s.N == 0) {
        if (dW != nullptr) TFB_CUDA_OK(cudaMemsetAsync(dW, 0, (size_t)(s.Cout * s.Cin * khw) * 4, stream));
        if (db != nullptr) TFB_CUDA_OK(cudaMemsetAsync(db, 0, (size_t)s.Cout * 4, stream));
        return TFB_OK;
    }
    {
        // Each product goes its own way: an input gradient with at most 4 channels to the CUDA-core
        // kernel, products with enough contraction channels and stride 1 to the TMA-fed path, the rest
        // to the gather kernel.
        if (dX != nullptr && !conv_tma_forced() && conv_direct_dgrad_eligible(s)) {
            rc = conv_direct_dgrad(dY, w, dX, s, stream);
            if (rc != TFB_OK) return rc;
            dX = nullptr;
            if (dW == nullptr && db == nullptr) return TFB_OK;
        }
        if ((dW != nullptr || db != nullptr) && !conv_tma_forced() && conv_direct_wgrad_eligible(s)) {
            rc = conv_direct_wgrad(x, dY, dW, db, s, stream);
            if (rc != TFB_OK) return rc;
            dW = nullptr, db = nullptr;
            if (dX == nullptr) return TFB_OK;
        }
        const bool t_dx = dX != nullptr && conv_tma_eligible(s, s.Cout, true);
        const bool t_w = (dW != nullptr || db != nullptr) && conv_tma_eligible(s, s.Cin);
        if (t_dx || t_w) {
            rc = conv_tma_backward(x, w, dY, t_dx ? dX : nullptr, t_w ? dW : nullptr, t_w ? db : nullptr, s, stream);
            if (rc != TFB_OK) return rc;
            if (t_dx) dX = nullptr;
            if (t_w) dW = nullptr, db = nullptr;
            if (dX == nullptr && dW == nullptr && db == nullptr) return TFB_OK;
        }
    }
    // ---- scratch layout -------------------------------------------------------------------
    const int64_t d_taps = s.Cout * khw, d_ld = round_up(d_taps, 4), d_table = round_up(d_taps, 128);
    const int64_t w_taps = s.Cin * khw, w_total = w_taps + 1, w_table = round_up(w_total, 128);
    const int64_t ldp = round_up(P, 4);
    const int bn_w = s.Cout <= 64 ? 64 : 128;
    const int w_row_tiles = (int)(w_table / 128), w_col_tiles = (int)((s.Cout + bn_w - 1) / bn_w);
    const int pos_blocks = (int)((P + 31) / 32);
    const int64_t k_blocks = s.N * pos_blocks;
    int64_t splits = st->sm_count / (w_row_tiles * w_col_tiles);
    if (splits < 1) splits = 1;
    if (splits > k_blocks) splits = k_blocks;
    const int64_t per = (k_blocks + splits - 1) / splits;
    splits = (k_blocks + per - 1) / per;   // every split owns at least one K block

    const bool want_dx = dX != nullptr, want_w = dW != nullptr || db != nullptr;
    size_t off = 0;
    auto take = [&](size_t bytes) { size_t o = off; off += align256(bytes); return o; };
    const size_t o_dtab = want_dx ? take((size_t)d_table * sizeof(TapInfo)) : 0;
    const size_t o_wd = want_dx ? take((size_t)(2 * s.Cin * d_ld) * 4) : 0;
    const size_t o_wtab = want_w ? take((size_t)w_table * sizeof(TapInfo)) : 0;
    const size_t o_dy = want_w ? take((size_t)(2 * s.N * s.Cout * ldp) * 4) : 0;
    const size_t o_part = want_w ? take((size_t)(splits * s.Cout * w_total) * 4) : 0;
    void* ws_v = nullptr;
    rc = workspace_get(stream, off + 256, &ws_v);
    if (rc != TFB_OK) return rc;
    uint8_t* ws = static_cast<uint8_t*>(ws_v);

    if (want_dx) {
        TapInfo* table_d = reinterpret_cast<TapInfo*>(ws + o_dtab);
        rc = build_taps(table_d, s.Cout, P, s.outW, s, true, false, d_table, stream);
        if (rc != TFB_OK) return rc;
        float* wd_hi = reinterpret_cast<float*>(ws + o_wd);
        float* wd_lo = wd_hi + s.Cin * d_ld;
        const int total = (int)(s.Cin * d_ld);
        dgrad_weight_kernel<<<(total + 255) / 256, 256, 0, stream>>>(w, wd_hi, wd_lo, (int)s.Cout, (int)s.Cin, (int)khw, (int)d_ld);
        TFB_CUDA_OK(cudaGetLastError());
        const int bn = s.Cin <= 64 ? 64 : 128;
        ConvArgs a;
        memset(&a, 0, sizeof(a));
        a.src = dY;
        a.src_sample = s.Cout * P;
        a.src_H = (int)s.outH; a.src_W = (int)s.outW;
        a.div_h = (int)s.sh; a.div_w = (int)s.sw;
        a.kH = (int)s.kH; a.kW = (int)s.kW;
        a.ay0 = (int)s.ph; a.ay_step = (int)-s.dh;
        a.ax0 = (int)s.pw; a.ax_step = (int)-s.dw;
        a.mul_h = a.mul_w = 1;
        a.pos_W = (int)s.W; a.pos_count = (int)(s.H * s.W);
        a.n_samples = (int)s.N;
        a.taps = (int)d_taps; a.taps_table = (int)d_table; a.tap_table = table_d;
        a.dst = dX; a.J = (int)s.Cin; a.rows_ext = a.pos_count;
        a.bias = nullptr; a.relu = 0;
        a.row_tiles = (a.pos_count + 127) / 128;
        a.col_tiles = (int)((s.Cin + bn - 1) / bn);
        a.num_tiles = (int)(s.N * a.row_tiles * a.col_tiles);
        a.k_blocks = (int)((d_taps + 31) / 32);
        a.splits = 1; a.chunk_kb = 8;
        a.status = st->status;
        CUtensorMap maps[2];
        rc = make_map(&maps[0], TFB_DTYPE_F32, wd_hi, (uint64_t)d_ld, (uint64_t)s.Cin, (uint64_t)d_ld * 4, 32, bn);
        if (rc != TFB_OK) return rc;
        rc = make_map(&maps[1], TFB_DTYPE_F32, wd_lo, (uint64_t)d_ld, (uint64_t)s.Cin, (uint64_t)d_ld * 4, 32, bn);
        if (rc != TFB_OK) return rc;
        const int grid = a.num_tiles < st->sm_count ? a.num_tiles : st->sm_count;
        rc = dispatch_conv<kConvDgrad>(bn, maps, a, grid, stream);
        if (rc != TFB_OK) return rc;
    }
    if (want_w) {
        TapInfo* table_d = reinterpret_cast<TapInfo*>(ws + o_wtab);
        rc = build_taps(table_d, s.Cin, s.H * s.W, s.W, s, false, true, w_table, stream);
        if (rc != TFB_OK) return rc;
        float* dy_hi = reinterpret_cast<float*>(ws + o_dy);
        float* dy_lo = dy_hi + s.N * s.Cout * ldp;
        rc = split_operand(dY, s.N * s.Cout, P, P, nullptr, dy_hi, dy_lo, ldp, stream);
        if (rc != TFB_OK) return rc;
        float* partial = reinterpret_cast<float*>(ws + o_part);
        ConvArgs a;
        memset(&a, 0, sizeof(a));
        fill_forward_geometry(a, s, x);
        a.taps = (int)w_total; a.taps_table = (int)w_table; a.tap_table = table_d;
        a.dst = partial; a.J = (int)s.Cout; a.rows_ext = (int)w_total;
        a.bias = nullptr; a.relu = 0;
        a.row_tiles = w_row_tiles; a.col_tiles = w_col_tiles;
        a.num_tiles = (int)(splits * w_row_tiles * w_col_tiles);
        a.k_blocks = (int)k_blocks; a.pos_blocks = pos_blocks; a.splits = (int)splits; a.chunk_kb = 8;
        a.b_rows_per_sample = (int)s.Cout;
        a.status = st->status;
        CUtensorMap maps[2];
        rc = make_map(&maps[0], TFB_DTYPE_F32, dy_hi, (uint64_t)ldp, (uint64_t)(s.N * s.Cout), (uint64_t)ldp * 4, 32, bn_w);
        if (rc != TFB_OK) return rc;
        rc = make_map(&maps[1], TFB_DTYPE_F32, dy_lo, (uint64_t)ldp, (uint64_t)(s.N * s.Cout), (uint64_t)ldp * 4, 32, bn_w);
        if (rc != TFB_OK) return rc;
        const int grid = a.num_tiles < st->sm_count ? a.num_tiles : st->sm_count;
        rc = dispatch_conv<kConvWgrad>(bn_w, maps, a, grid, stream);
        if (rc != TFB_OK) return rc;
        const int total = (int)(s.Cout * w_total);
        wgrad_reduce_kernel<<<(total + 255) / 256, 256, 0, stream>>>(partial, (int)splits, (int)s.Cout, (int)w_taps,
                                                                     (int)w_total, dW, db);
        TFB_CUDA_OK(cudaGetLastError());
    }
    return TFB_OK;
}

}  // namespace tfb

namespace {

// Float16 / BFloat16 tensors. The reference's launchers take all three dtypes for every convolution
// kernel with FP32 accumulation and a result of the input type (cuda/kernels/im2col.cu:124-157,
// cuda/kernels/gemm.cu:280-299). Here 16-bit tensors are widened to FP32 (exact), run through the
// same FP32 kernels (FP32 accumulation; no 16-bit rounding between the im2col and GEMM stages because
// those stages do not exist) and the results are rounded to the tensor type once.
template <typename T>
__global__ void widen16_kernel(const T* __restrict__ src, float* __restrict__ dst, long long n) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        dst[i] = static_cast<float>(src[i]);
}
template <typename T>
__global__ void narrow16_kernel(const float* __restrict__ src, T* __restrict__ dst, long long n) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        dst[i] = static_cast<T>(src[i]);
}

// Stream-ordered FP32 staging buffers of one call (separate from the library's scratch buffer, which
// the FP32 kernels underneath use themselves).
struct Staging {
    cudaStream_t stream;
    std::vector<void*> ptrs;
    explicit Staging(cudaStream_t s) : stream(s) {}
    int make(float** out, int64_t n) {
        *out = nullptr;
        if (n <= 0) n = 1;
        TFB_CUDA_OK(cudaMallocAsync(reinterpret_cast<void**>(out), (size_t)n * 4, stream));
        ptrs.push_back(*out);
        return TFB_OK;
    }
    ~Staging() {
        for (void* p : ptrs) (void)cudaFreeAsync(p, stream);
        (void)cudaGetLastError();
    }
};

int grid_1d(int64_t n) {
    int64_t g = (n + 255) / 256;
    if (g > 148 * 16) g = 148 * 16;
    return (int)(g < 1 ? 1 : g);
}

int widen(const void* src, float* dst, int64_t n, int dtype, cudaStream_t stream) {
    if (n <= 0) return TFB_OK;
    if (dtype == TFB_DTYPE_BF16)
        widen16_kernel<__nv_bfloat16><<<grid_1d(n), 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(src), dst, n);
    else
        widen16_kernel<__half><<<grid_1d(n), 256, 0, stream>>>(static_cast<const __half*>(src), dst, n);
    TFB_CUDA_OK(cudaGetLastError());
    return TFB_OK;
}

int narrow(const float* src, void* dst, int64_t n, int dtype, cudaStream_t stream) {
    if (n <= 0) return TFB_OK;
    if (dtype == TFB_DTYPE_BF16)
        narrow16_kernel<__nv_bfloat16><<<grid_1d(n), 256, 0, stream>>>(src, static_cast<__nv_bfloat16*>(dst), n);
    else
        narrow16_kernel<__half><<<grid_1d(n), 256, 0, stream>>>(src, static_cast<__half*>(dst), n);
    TFB_CUDA_OK(cudaGetLastError());
    return TFB_OK;
}

int conv2d_forward_16(const void* x, const void* w, const float* bias, void* out, const tfb::ConvShape& s, bool relu,
                      int dtype, cudaStream_t stream) {
    const int64_t nx = s.N * s.Cin * s.H * s.W, nw = s.Cout * s.Cin * s.kH * s.kW, ny = s.N * s.Cout * s.outH * s.outW;
    Staging st(stream);
    float *xf, *wf, *yf;
    int rc;
    if ((rc = st.make(&xf, nx)) != TFB_OK || (rc = st.make(&wf, nw)) != TFB_OK || (rc = st.make(&yf, ny)) != TFB_OK) return rc;
    if ((rc = widen(x, xf, nx, dtype, stream)) != TFB_OK || (rc = widen(w, wf, nw, dtype, stream)) != TFB_OK) return rc;
    rc = tfb::conv2d_forward(xf, wf, bias, yf, s, relu, stream);
    if (rc != TFB_OK) return rc;
    return narrow(yf, out, ny, dtype, stream);
}

int conv2d_backward_16(const void* x, const void* w, const void* dY, void* dX, void* dW, float* db,
                       const tfb::ConvShape& s, int dtype, cudaStream_t stream) {
    const int64_t nx = s.N * s.Cin * s.H * s.W, nw = s.Cout * s.Cin * s.kH * s.kW, ny = s.N * s.Cout * s.outH * s.outW;
    Staging st(stream);
    float *xf = nullptr, *wf = nullptr, *gf = nullptr, *dxf = nullptr, *dwf = nullptr;
    int rc;
    if ((rc = st.make(&gf, ny)) != TFB_OK || (rc = widen(dY, gf, ny, dtype, stream)) != TFB_OK) return rc;
    if (x != nullptr && ((rc = st.make(&xf, nx)) != TFB_OK || (rc = widen(x, xf, nx, dtype, stream)) != TFB_OK)) return rc;
    if (w != nullptr && ((rc = st.make(&wf, nw)) != TFB_OK || (rc = widen(w, wf, nw, dtype, stream)) != TFB_OK)) return rc;
    if (dX != nullptr && (rc = st.make(&dxf, nx)) != TFB_OK) return rc;
    if (dW != nullptr && (rc = st.make(&dwf, nw)) != TFB_OK) return rc;
    rc = tfb::conv2d_backward(xf, wf, gf, dxf, dwf, db, s, stream);
    if (rc != TFB_OK) return rc;
    if (dX != nullptr && (rc = narrow(dxf, dX, nx, dtype, stream)) != TFB_OK) return rc;
    if (dW != nullptr && (rc = narrow(dwf, dW, nw, dtype, stream)) != TFB_OK) return rc;
    return TFB_OK;
}

}  // namespace

extern "C" {

using tfb::fail;

static int make_shape(tfb::ConvShape& s, int64_t N, int64_t Cin, int64_t H, int64_t W, int64_t Cout, int64_t kH,
                      int64_t kW, int64_t sh, int64_t sw, int64_t ph, int64_t pw, int64_t dh, int64_t dw) {
    if (sh <= 0 || sw <= 0 || kH <= 0 || kW <= 0 || dh <= 0 || dw <= 0)
        return fail(TFB_ERR_INVALID_ARG, "conv2d: non-positive kernel size, stride or dilation");
    s = tfb::ConvShape{N, Cin, H, W, Cout, kH, kW, sh, sw, ph, pw, dh, dw,
                       tfb_conv_out_dim(H, kH, sh, ph, dh), tfb_conv_out_dim(W, kW, sw, pw, dw)};
    return TFB_OK;
}

int64_t tfb_conv_out_dim(int64_t in, int64_t k, int64_t stride, int64_t pad, int64_t dilation) {
    if (stride <= 0) return 0;
    return (in + 2 * pad - dilation * (k - 1) - 1) / stride + 1;
}

int tfb_conv2d_forward(const void* x, const void* w, const float* bias, void* out, int64_t N, int64_t Cin,
                       int64_t H, int64_t W, int64_t Cout, int64_t kH, int64_t kW, int64_t stride_h,
                       int64_t stride_w, int64_t pad_h, int64_t pad_w, int64_t dil_h, int64_t dil_w, int relu,
                       int dtype, void* stream) {
    if (tfb::dtype_size(dtype) == 0) return fail(TFB_ERR_UNSUPPORTED, "conv2d_forward: unknown dtype %d", dtype);
    if (x == nullptr || w == nullptr || out == nullptr) return fail(TFB_ERR_INVALID_ARG, "conv2d_forward: null pointer");
    tfb::ConvShape s;
    int rc = make_shape(s, N, Cin, H, W, Cout, kH, kW, stride_h, stride_w, pad_h, pad_w, dil_h, dil_w);
    if (rc != TFB_OK) return rc;
    if (dtype != TFB_DTYPE_F32) {
        rc = tfb::check_shape(s);
        if (rc != TFB_OK) return rc;
        return conv2d_forward_16(x, w, bias, out, s, relu != 0, dtype, static_cast<cudaStream_t>(stream));
    }
    return tfb::conv2d_forward(static_cast<const float*>(x), static_cast<const float*>(w), bias,
                               static_cast<float*>(out), s, relu != 0, static_cast<cudaStream_t>(stream));
}

int tfb_conv2d_backward(const void* x, const void* w, const void* grad_out, void* grad_input, void* grad_weight,
                        float* grad_bias, int64_t N, int64_t Cin, int64_t H, int64_t W, int64_t Cout, int64_t kH,
                        int64_t kW, int64_t stride_h, int64_t stride_w, int64_t pad_h, int64_t pad_w,
                        int64_t dil_h, int64_t dil_w, int dtype, void* stream) {
    if (tfb::dtype_size(dtype) == 0) return fail(TFB_ERR_UNSUPPORTED, "conv2d_backward: unknown dtype %d", dtype);
    if (grad_out == nullptr) return fail(TFB_ERR_INVALID_ARG, "conv2d_backward: null upstream gradient");
    if (grad_input != nullptr && w == nullptr) return fail(TFB_ERR_INVALID_ARG, "conv2d_backward: grad_input needs the weights");
    if ((grad_weight != nullptr || grad_bias != nullptr) && x == nullptr)
        return fail(TFB_ERR_INVALID_ARG, "conv2d_backward: grad_weight needs the input");
    tfb::ConvShape s;
    int rc = make_shape(s, N, Cin, H, W, Cout, kH, kW, stride_h, stride_w, pad_h, pad_w, dil_h, dil_w);
    if (rc != TFB_OK) return rc;
    if (dtype != TFB_DTYPE_F32) {
        rc = tfb::check_shape(s);
        if (rc != TFB_OK) return rc;
        return conv2d_backward_16(x, w, grad_out, grad_input, grad_weight, grad_bias, s, dtype,
                                  static_cast<cudaStream_t>(stream));
    }
    return tfb::conv2d_backward(static_cast<const float*>(x), static_cast<const float*>(w),
                                static_cast<const float*>(grad_out), static_cast<float*>(grad_input),
                                static_cast<float*>(grad_weight), grad_bias, s, static_cast<cudaStream_t>(stream));
}

int tfb_im2col_index_map(int64_t* out, int64_t n_first, int64_t n_count, int64_t Cin, int64_t H, int64_t W,
                         int64_t kH, int64_t kW, int64_t stride_h, int64_t stride_w, int64_t pad_h, int64_t pad_w,
                         int64_t dil_h, int64_t dil_w, void* stream_v) {
    using namespace tfb;
    if (out == nullptr || n_first < 0 || n_count < 0) return fail(TFB_ERR_INVALID_ARG, "im2col_index_map: bad argument");
    ConvShape s;
    int rc = make_shape(s, n_first + n_count, Cin, H, W, 1, kH, kW, stride_h, stride_w, pad_h, pad_w, dil_h, dil_w);
    if (rc != TFB_OK) return rc;
    rc = check_shape(s);
    if (rc != TFB_OK) return rc;
    if (n_count == 0) return TFB_OK;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    DeviceState* st = nullptr;
    rc = device_state(&st);
    if (rc != TFB_OK) return rc;
    const int64_t taps = Cin * kH * kW, table_len = round_up(taps, 128);
    void* ws = nullptr;
    rc = workspace_get(stream, (size_t)table_len * sizeof(TapInfo), &ws);
    if (rc != TFB_OK) return rc;
    rc = build_taps(static_cast<TapInfo*>(ws), Cin, H * W, W, s, false, false, table_len, stream);
    if (rc != TFB_OK) return rc;
    ConvArgs a;
    memset(&a, 0, sizeof(a));
    fill_forward_geometry(a, s, nullptr);
    index_map_kernel<<<st->sm_count * 8, 256, 0, stream>>>(reinterpret_cast<long long*>(out),
                                                            static_cast<const TapInfo*>(ws), a, (int)n_first,
                                                            (int)n_count, (int)taps, Cin * H * W);
    TFB_CUDA_OK(cudaGetLastError());
    return TFB_OK;
}

}  // extern "C"
