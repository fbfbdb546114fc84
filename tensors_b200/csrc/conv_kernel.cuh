// Implicit-GEMM convolution on tcgen05 (FP32 in/out through the 3xTF32 split).
//
// The column matrix of im2col is never written to memory. Producer warps gather input
// elements straight from the NCHW tensor with the im2col index map, split each into TF32
// hi + lo and store both into the shared-memory operand tile in the layout the tensor core
// reads; the other operand (weights, or the upstream gradient for wgrad) arrives by TMA.
//
// One kernel, three contractions (D is always [128 "rows" x BN "columns"] per tile):
//   fprop  rows = output positions of one sample, columns = output channels,
//          contraction over taps t = (c, ki, kj):      out[n, co, p]  = Σ_t col[n][t, p] · W[co, t]
//   dgrad  rows = input positions of one sample, columns = input channels,
//          contraction over taps t = (co, ki, kj):     dX[n, c, q]    = Σ_t colT[n][t, q] · Wd[c, t]
//          (gather form: each input pixel pulls the output pixels that touched it, so there
//          is no scatter, no atomics and a fixed summation order)
//   wgrad  rows = taps t = (c, ki, kj), columns = output channels, contraction over (n, p),
//          split over CTAs:                            dW[co, t]     += Σ_{n,p} col[n][t, p] · dY[n, co, p]
//          one extra all-ones tap makes the same product deliver the bias gradient.
//
// In all three the producer's lanes run over 32 consecutive spatial positions (coalesced global
// reads, conflict-free shared-memory writes) for one tap at a time.
//
// Warp roles (448 threads): 0 = TMA for the B operand, 1 = MMA issuer + TMEM owner,
// 2..9 = gather producers, 10..13 = epilogue. The TMEM accumulator is closed every `chunk_kb`
// K blocks and summed in registers with round-to-nearest adds (see gemm_kernel.cuh).
#pragma once

#include "ptx.cuh"

namespace tfb {

enum ConvMode : int { kConvFprop = 0, kConvDgrad = 1, kConvWgrad = 2 };

// Where tap t reads relative to a position: plane offset inside one sample and the two
// coordinate offsets. plane_off < 0 marks taps that do not exist (-1) or the all-ones tap (-2).
// `delta` = plane_off + ay * src_W + ax and `kidx` = ki | kj << 8 | (ki * kW + kj) << 16 serve the
// separable fast paths; the flat filter index is 31 for taps that do not exist and 30 for the ones tap.
struct TapInfo {
    int plane_off;
    short ay, ax;
    int delta;
    int kidx;
};

struct ConvArgs {
    const float* src;          // tensor the producers gather from (x for fprop / wgrad, dY for dgrad)
    long long src_sample;      // elements per sample of src
    int src_H, src_W;          // plane extents of src
    int div_h, div_w;          // dgrad with stride > 1: coordinates must divide by these (else 1)
    int kH, kW;                // filter extents
    int ay0, ay_step, ax0, ax_step;   // tap (ki, kj) reads at y0 + ay0 + ki*ay_step, x0 + ax0 + kj*ax_step
    int mul_h, mul_w;          // position -> coordinate scale (stride for fprop / wgrad, 1 for dgrad)
    int pos_W, pos_count;      // width of the position grid and positions per sample
    int n_samples;
    int taps;                  // entries of the tap table that may be valid (incl. the ones tap)
    int taps_table;            // table length (multiple of 128)
    const TapInfo* tap_table;  // device copy of the tap table
    float* dst;                // output: dst[(outer * J + j) * rows_ext + row]
    int J;                     // valid columns (output channels / input channels)
    int rows_ext;              // row extent of the output (positions per sample, or taps for wgrad)
    const float* bias;         // fprop: per-column bias or nullptr
    int relu;
    // tiling
    int row_tiles, col_tiles, num_tiles;
    int k_blocks;              // fprop / dgrad: tap blocks; wgrad: n_samples * pos_blocks
    int pos_blocks;            // wgrad: 32-position blocks per sample
    int splits;                // wgrad: CTAs sharing one output tile
    int chunk_kb;
    int b_rows_per_sample;     // wgrad: rows of the B matrix per sample (Cout)
    int* status;
};

// Warps: 0 TMA, 1 MMA, kConvProducerWarps gather producers, then 4 epilogue warps.
constexpr int kConvProducerWarps = 8;
// The producers form two groups of four warps that take alternate K blocks (stages), so the global-load
// latency of one block overlaps with the shared-memory stores of the other.
constexpr int kConvElems = 32;   // operand elements per producer thread and K block
constexpr int kConvThreads = 32 * (2 + kConvProducerWarps + 4);

template <int BN, int STAGES>
struct ConvSmem {
    static constexpr int A_TILE = 128 * 128;          // 128 rows x 32 fp32, per plane
    static constexpr int B_TILE = BN * 128;
    static constexpr int STAGE_BYTES = 2 * (A_TILE + B_TILE);
    static constexpr int BAR_BYTES = 256;
    static constexpr int fixed() { return 1024 + STAGES * STAGE_BYTES + BAR_BYTES; }
};

__device__ __forceinline__ float tf32_rna_dev(float x) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return __uint_as_float(r);
}

// The im2col index map as the producers evaluate it: source element (offset inside one sample)
// that tap `ti` reads for the position whose scaled coordinates are (y0, x0), or -1 for padding.
// fprop / wgrad: (u, v) = (oh*stride + ki*dil - pad, ow*stride + kj*dil - pad).
// dgrad: (u, v) = ((ih + pad - ki*dil) / stride, ...) and only where the division is exact.
template <int MODE>
__device__ __forceinline__ int conv_src_offset(const TapInfo& ti, int y0, int x0, const ConvArgs& args) {
    int u = y0 + ti.ay, v = x0 + ti.ax;
    if (MODE == kConvDgrad && (args.div_h != 1 || args.div_w != 1)) {
        if (u < 0 || v < 0 || (u % args.div_h) != 0 || (v % args.div_w) != 0) return -1;
        u /= args.div_h;
        v /= args.div_w;
    }
    if ((unsigned)u >= (unsigned)args.src_H || (unsigned)v >= (unsigned)args.src_W) return -1;
    return ti.plane_off + u * args.src_W + v;
}

// Separable form of the same map, valid whenever no stride division is involved (fprop, wgrad, and
// dgrad with stride 1): row validity depends only on (y0, ki) and column validity only on (x0, kj),
// so a thread keeps one bit mask per axis and its own base offset y0 * src_W + x0; a tap then costs
// one add (`delta`) and two bit tests. Kernels up to 32 x 32.
__device__ __forceinline__ uint32_t conv_axis_mask(int c0, int a0, int a_step, int taps, int extent) {
    uint32_t m = 0;
    for (int k = 0; k < taps; ++k) {
        const int u = c0 + a0 + k * a_step;
        if ((unsigned)u < (unsigned)extent) m |= 1u << k;
    }
    return m;
}
__device__ __forceinline__ int conv_src_offset_fast(const TapInfo& ti, int thread_off, uint32_t ymask, uint32_t xmask) {
    const uint32_t ok = (ymask >> (ti.kidx & 0xff)) & (xmask >> ((ti.kidx >> 8) & 0xff)) & 1u;
    return ok ? thread_off + ti.delta : -1;
}

// Filters of at most 30 taps per channel (3x3, 5x5): one combined validity mask per thread, bit
// ki * kW + kj, bit 30 = "position exists" (the ones tap), bit 31 = 0 (absent taps). A tap then costs
// one shift-and-test and one add.
__device__ __forceinline__ uint32_t conv_combined_mask(uint32_t ymask, uint32_t xmask, int kH, int kW, bool pos_ok) {
    uint32_t m = pos_ok ? (1u << 30) : 0u;
    for (int ki = 0; ki < kH; ++ki)
        if ((ymask >> ki) & 1u) m |= (xmask & ((1u << kW) - 1u)) << (ki * kW);
    return m;
}

template <int MODE, int BN, int STAGES>
__global__ void __launch_bounds__(kConvThreads, 1)
conv_igemm_kernel(const __grid_constant__ CUtensorMap tmB, const __grid_constant__ CUtensorMap tmB2,
                  const ConvArgs args) {
    using S = ConvSmem<BN, STAGES>;
    constexpr bool WGRAD = (MODE == kConvWgrad);
    constexpr uint32_t TMEM_COLS = (2 * BN <= 64) ? 64 : (2 * BN <= 128) ? 128 : (2 * BN <= 256) ? 256 : 512;

    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

    const uint32_t bars = smem_base + STAGES * S::STAGE_BYTES;
    auto full_a = [&](int s) { return bars + 8u * s; };
    auto full_b = [&](int s) { return bars + 8u * (STAGES + s); };
    auto empty_bar = [&](int s) { return bars + 8u * (2 * STAGES + s); };
    auto tfull_bar = [&](int b) { return bars + 8u * (3 * STAGES + b); };
    auto tempty_bar = [&](int b) { return bars + 8u * (3 * STAGES + 2 + b); };
    uint8_t* after_bars = smem_gen + STAGES * S::STAGE_BYTES + 8 * (3 * STAGES + 4);
    volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(after_bars);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(after_bars + 4);
    TapInfo* taps_sm = reinterpret_cast<TapInfo*>(smem_gen + STAGES * S::STAGE_BYTES + S::BAR_BYTES);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_a(s), 4);     // one arrival per warp of a producer group
            mbar_init(full_b(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(tfull_bar(b), 1);
            mbar_init(tempty_bar(b), 4);     // one arrival per epilogue warp
        }
        *abort_flag = 0;
        fence_mbar_init();
        tma_prefetch_desc(&tmB);
        tma_prefetch_desc(&tmB2);
    }
    for (int i = threadIdx.x; i < args.taps_table; i += blockDim.x) taps_sm[i] = args.tap_table[i];
    if (warp == 1) {
        tmem_alloc<1>(smem_u32(const_cast<uint32_t*>(tmem_holder)), TMEM_COLS);
        tmem_relinquish<1>();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_holder;

    // Tile -> (row tile, column tile, outer index). fprop / dgrad: outer = sample; wgrad: outer = split.
    auto decode_tile = [&](int t, int& rt, int& ct, int& outer) {
        ct = t % args.col_tiles;
        const int r = t / args.col_tiles;
        rt = r % args.row_tiles;
        outer = r / args.row_tiles;
    };
    // K-block range of a tile.
    auto k_range = [&](int outer, int& kb0, int& kb1) {
        if constexpr (WGRAD) {
            const int per = (args.k_blocks + args.splits - 1) / args.splits;
            kb0 = outer * per;
            kb1 = min(kb0 + per, args.k_blocks);
            if (kb0 > kb1) kb0 = kb1;
        } else {
            kb0 = 0;
            kb1 = args.k_blocks;
        }
    };

    if (warp == 0) {
        // ------------------------------ TMA producer for B -----------------------------
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < args.num_tiles && ok; t += gridDim.x) {
                int rt, ct, outer, kb0, kb1;
                decode_tile(t, rt, ct, outer);
                k_range(outer, kb0, kb1);
                for (int kb = kb0; kb < kb1; ++kb) {
                    ok = mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, args.status, kDevTimeoutEmpty);
                    if (!ok) break;
                    const uint32_t b_hi = smem_base + s * S::STAGE_BYTES + 2 * S::A_TILE;
                    const uint32_t b_lo = b_hi + S::B_TILE;
                    mbar_arrive_expect_tx(full_b(s), 2 * S::B_TILE);
                    int x, y;
                    if constexpr (WGRAD) {
                        const int n = kb / args.pos_blocks, pb = kb - n * args.pos_blocks;
                        x = pb * 32;
                        y = n * args.b_rows_per_sample + ct * BN;
                    } else {
                        x = kb * 32;
                        y = ct * BN;
                    }
                    tma_load_2d(b_hi, &tmB, x, y, full_b(s));
                    tma_load_2d(b_lo, &tmB2, x, y, full_b(s));
                    if (++s == STAGES) { s = 0; ph ^= 1u; }
                }
            }
            if (!ok || *abort_flag != 0) {
                for (int i = 0; i < STAGES; ++i) {
                    const uint64_t t0 = global_timer_ns();
                    while (!mbar_try_wait(full_b(i), 0) && !mbar_try_wait(full_b(i), 1)) {
                        if (global_timer_ns() - t0 > 100000000ull) {
                            if (args.status != nullptr) atomicCAS(args.status, 0, kDevTimeoutDrain);
                            break;
                        }
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ---------------------------------------
        if (lane == 0) {
            // A: fprop / dgrad tiles are MN-major (rows = positions contiguous) in the 128-byte
            //    swizzle with 32-byte atoms: 32-row groups 4096 B apart, 4-tap groups 512 B apart,
            //    one K step = 8 taps = 1024 B.  wgrad tiles are K-major (positions = contraction
            //    contiguous), plain 128-byte swizzle, 8-row groups 1024 B apart, K step = 32 B.
            // B: always K-major, 128-byte swizzle.
            constexpr uint32_t A_MN = WGRAD ? 0u : 1u;
            constexpr uint32_t A_LBO = WGRAD ? 16u : 4096u;
            constexpr uint32_t A_SBO = WGRAD ? 1024u : 512u;
            constexpr uint32_t A_SWZ = WGRAD ? 2u : 1u;
            constexpr uint32_t A_KSTEP = WGRAD ? 32u : 1024u;
            const uint32_t idesc = make_idesc(2u, A_MN, 0u, 128, BN);
            int s = 0;
            uint32_t ph = 0;
            uint32_t cit = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < args.num_tiles && ok; t += gridDim.x) {
                int rt, ct, outer, kb0, kb1;
                decode_tile(t, rt, ct, outer);
                k_range(outer, kb0, kb1);
                // Every tile has at least one K block (the host sizes the wgrad splits that way).
                for (int c0 = kb0; c0 < kb1 && ok; c0 += args.chunk_kb, ++cit) {
                    const uint32_t buf = cit & 1u;
                    const uint32_t use = cit >> 1;
                    ok = mbar_wait(tempty_bar(buf), (use & 1u) ^ 1u, abort_flag, args.status, kDevTimeoutTmemEmpty);
                    if (!ok) break;
                    tc_fence_after_sync();
                    const uint32_t d_tmem = tmem_base + buf * (uint32_t)BN;
                    const int c1 = min(c0 + args.chunk_kb, kb1);
                    for (int kb = c0; kb < c1; ++kb) {
                        ok = mbar_wait(full_a(s), ph, abort_flag, args.status, kDevTimeoutFull) &&
                             mbar_wait(full_b(s), ph, abort_flag, args.status, kDevTimeoutFull);
                        if (!ok) break;
                        tc_fence_after_sync();
                        const uint32_t st = smem_base + s * S::STAGE_BYTES;
                        const uint32_t a_hi = st, a_lo = st + S::A_TILE;
                        const uint32_t b_hi = st + 2 * S::A_TILE, b_lo = b_hi + S::B_TILE;
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const uint32_t acc = (kb > c0 || j > 0) ? 1u : 0u;
                            const uint64_t da = make_smem_desc(a_hi + j * A_KSTEP, A_LBO, A_SBO, A_SWZ);
                            const uint64_t dal = make_smem_desc(a_lo + j * A_KSTEP, A_LBO, A_SBO, A_SWZ);
                            const uint64_t db = make_smem_desc(b_hi + j * 32u, 16u, 1024u, 2u);
                            const uint64_t dbl = make_smem_desc(b_lo + j * 32u, 16u, 1024u, 2u);
                            umma_ss<1, true>(d_tmem, dal, db, idesc, acc);
                            umma_ss<1, true>(d_tmem, da, dbl, idesc, 1u);
                            umma_ss<1, true>(d_tmem, da, db, idesc, 1u);
                        }
                        umma_commit<1>(empty_bar(s));
                        if (++s == STAGES) { s = 0; ph ^= 1u; }
                    }
                    if (!ok) break;
                    umma_commit<1>(tfull_bar(buf));
                }
            }
        }
    } else if (warp < 2 + kConvProducerWarps) {
        // ------------------------------ gather producers ------------------------------------
        const int pw = warp - 2;                       // producer warp
        const int pgrp = pw & 3;                       // which 32 rows of the tile this warp writes
        const uint32_t group = (uint32_t)(pw >> 2);    // which of the alternating K blocks this warp takes
        uint32_t seq = 0;   // K blocks so far, over all tiles: block seq lives in stage seq % STAGES
        bool ok = true;
        for (int t = blockIdx.x; t < args.num_tiles && ok; t += gridDim.x) {
            int rt, ct, outer, kb0, kb1;
            decode_tile(t, rt, ct, outer);
            k_range(outer, kb0, kb1);
            // fprop / dgrad: this thread's position is fixed for the tile.
            int pos = 0, y0 = 0, x0 = 0, thread_off = 0;
            uint32_t ymask = 0, xmask = 0, vmask = 0;
            bool pos_ok = false;
            const float* base = args.src;
            const bool fast = (args.div_h == 1 && args.div_w == 1 && args.kH <= 32 && args.kW <= 32);
            const bool fast2 = fast && args.kH * args.kW <= 30;
            auto locate = [&]() {
                pos_ok = pos < args.pos_count;
                const int oy = pos / args.pos_W, ox = pos - oy * args.pos_W;
                y0 = oy * args.mul_h;
                x0 = ox * args.mul_w;
                thread_off = y0 * args.src_W + x0;
                if (fast) {
                    ymask = pos_ok ? conv_axis_mask(y0, args.ay0, args.ay_step, args.kH, args.src_H) : 0u;
                    xmask = pos_ok ? conv_axis_mask(x0, args.ax0, args.ax_step, args.kW, args.src_W) : 0u;
                    if (fast2) vmask = conv_combined_mask(ymask, xmask, args.kH, args.kW, pos_ok);
                }
            };
            if constexpr (!WGRAD) {
                pos = rt * 128 + pgrp * 32 + lane;
                locate();
                base = args.src + (long long)outer * args.src_sample;
            }
            // gather(kb, v): issue this thread's 32 loads of K block kb into registers, all in flight
            // together and before the wait for a free stage, so their latencies overlap.
            auto gather = [&](int kb, float (&v)[kConvElems]) {
                int tap0;
                if constexpr (WGRAD) {
                    const int n = kb / args.pos_blocks, pb = kb - n * args.pos_blocks;
                    pos = pb * 32 + lane;
                    locate();
                    base = args.src + (long long)n * args.src_sample;
                    tap0 = rt * 128 + pgrp * 32;   // rows (taps) of the tile this warp writes
                } else {
                    tap0 = kb * 32;                // K index = tap
                }
                if (fast2) {
#pragma unroll
                    for (int i = 0; i < kConvElems; ++i) {
                        const TapInfo ti = taps_sm[tap0 + i];
                        const uint32_t kf = (uint32_t)ti.kidx >> 16;
                        const bool valid = ((vmask >> kf) & 1u) != 0;
                        float val = 0.f;
                        if (WGRAD && kf == 30u) val = valid ? 1.f : 0.f;
                        else if (valid) val = __ldg(base + thread_off + ti.delta);
                        v[i] = val;
                    }
                } else if (fast) {
#pragma unroll
                    for (int i = 0; i < kConvElems; ++i) {
                        const TapInfo ti = taps_sm[tap0 + i];
                        const int off = conv_src_offset_fast(ti, thread_off, ymask, xmask);
                        float val = (ti.plane_off == -2 && pos_ok) ? 1.f : 0.f;
                        if (ti.plane_off >= 0 && off >= 0) val = __ldg(base + off);
                        v[i] = val;
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < kConvElems; ++i) {   // fully unrolled so that v[] stays in registers
                        const TapInfo ti = taps_sm[tap0 + i];
                        float val = 0.f;
                        if (ti.plane_off >= 0) {
                            const int off = pos_ok ? conv_src_offset<MODE>(ti, y0, x0, args) : -1;
                            if (off >= 0) val = __ldg(base + off);
                        } else if (ti.plane_off == -2) {
                            val = pos_ok ? 1.f : 0.f;
                        }
                        v[i] = val;
                    }
                }
            };
            // emit(v): wait for a free stage, split into hi / lo, write the operand tile, signal.
            auto emit = [&](int s, uint32_t ph, const float (&v)[kConvElems]) -> bool {
                // One lane polls (a barrier polled and arrived on by 128 threads serialises on its word).
                bool good = true;
                if (lane == 0) good = mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, args.status, kDevTimeoutEmpty);
                good = __all_sync(0xffffffffu, good);
                if (!good) return false;
                uint8_t* a_hi = smem_gen + s * S::STAGE_BYTES;
                uint8_t* a_lo = a_hi + S::A_TILE;
#pragma unroll
                for (int i = 0; i < kConvElems; ++i) {
                    const float hi = tf32_rna_dev(v[i]);
                    const float lo = v[i] - hi;
                    uint32_t off;
                    if constexpr (WGRAD) {
                        // row m = tap, contraction index kk = lane: K-major, 128-byte swizzle
                        const uint32_t m = (uint32_t)(pgrp * 32 + i);
                        off = m * 128u + ((((uint32_t)lane >> 2) ^ (m & 7u)) << 4) + ((uint32_t)lane & 3u) * 4u;
                    } else {
                        // row = position (lane), contraction index kk: MN-major, 32-byte atoms
                        const uint32_t kk = (uint32_t)i;
                        off = (uint32_t)pgrp * 4096u + (uint32_t)(lane & 7) * 4u + kk * 128u +
                              ((((uint32_t)lane >> 3) ^ (kk & 3u)) << 5);
                    }
                    *reinterpret_cast<float*>(a_hi + off) = hi;
                    *reinterpret_cast<float*>(a_lo + off) = lo;
                }
                fence_proxy_async_smem();   // every writer makes its stores visible to the tensor core's proxy
                __syncwarp();
                if (lane == 0) mbar_arrive(full_a(s));
                return true;
            };
            // (Issuing the gathers of block kb+1 before writing block kb was tried and measured slower.)
            float va[kConvElems];
            for (int kb = kb0; kb < kb1 && ok; ++kb, ++seq) {
                if ((seq & 1u) != group) continue;
                gather(kb, va);
                ok = emit((int)(seq % STAGES), (seq / STAGES) & 1u, va);
            }
        }
    } else {
        // ------------------------------ epilogue ----------------------------------------------
        const int q = warp & 3;   // TMEM lane quarter this warp may read
        uint32_t cit = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < args.num_tiles && ok; t += gridDim.x) {
            int rt, ct, outer, kb0, kb1;
            decode_tile(t, rt, ct, outer);
            k_range(outer, kb0, kb1);
            const int row = rt * 128 + q * 32 + lane;
            const bool row_ok = row < args.rows_ext;
            const int j0 = ct * BN;
            const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
            float acc[BN];
#pragma unroll
            for (int i = 0; i < BN; ++i) acc[i] = 0.f;
            for (int c0 = kb0; c0 < kb1; c0 += args.chunk_kb, ++cit) {
                const uint32_t buf = cit & 1u;
                const uint32_t use = cit >> 1;
                if (lane == 0) ok = mbar_wait(tfull_bar(buf), use & 1u, abort_flag, args.status, kDevTimeoutTmemFull);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after_sync();
#pragma unroll
                for (int c = 0; c < BN / 32; ++c) {
                    if (j0 + c * 32 < args.J) {
                        uint32_t r[32];
                        tmem_ld_32x32(lane_addr + buf * (uint32_t)BN + (uint32_t)(c * 32), r);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; ++i) acc[c * 32 + i] += __uint_as_float(r[i]);
                    }
                }
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(tempty_bar(buf));
            }
            if (!ok) break;
            if (row_ok) {
                // Lanes hold consecutive rows, so each column is one coalesced 128-byte store.
                float* dst = args.dst + ((long long)outer * args.J + j0) * args.rows_ext + row;
#pragma unroll
                for (int i = 0; i < BN; ++i) {
                    if (j0 + i < args.J) {
                        float v = acc[i];
                        if (args.bias != nullptr) v += __ldg(args.bias + j0 + i);
                        if (args.relu) v = v > 0.f ? v : 0.f;
                        dst[(long long)i * args.rows_ext] = v;
                    }
                }
            }
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc<1>(tmem_base, TMEM_COLS);
    }
}

}  // namespace tfb
