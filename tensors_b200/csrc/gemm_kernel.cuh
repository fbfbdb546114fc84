// Persistent, warp-specialised tcgen05 GEMM for sm_100a.
//
//   D[M,N] (+bias, ReLU) = A · B      with FP32 accumulation in tensor memory.
//
// Roles inside one CTA (192 threads):
//   warp 0      TMA producer: fills a ring of shared-memory stages with 128-byte-swizzled
//               operand tiles and signals `full[s]` by transaction bytes.
//   warp 1      MMA issuer: one lane issues tcgen05.mma per 32-byte K step, releases a
//               stage with tcgen05.commit -> `empty[s]`, and hands a finished accumulator
//               to the epilogue with tcgen05.commit -> `tmem_full[b]`.  Also owns the
//               TMEM allocation.
//   warps 2..5  epilogue: tcgen05.ld the accumulator (each warp its own 32 TMEM lanes),
//               apply bias / ReLU, convert and store, then release the accumulator with
//               `tmem_empty[b]`.  Two accumulators let the epilogue of tile i overlap the
//               main loop of tile i+1.
//
// Operand layouts.  "K-major": the contraction index is contiguous in memory (A[M,K]
// row-major, B given as [N,K] row-major).  "MN-major": the M (resp. N) index is
// contiguous (A given as [K,M] row-major, B as [K,N] row-major).  Both are fed to the
// tensor core straight from the TMA tiles through the matching shared-memory
// descriptor, so transposed products need no transpose copy.
//
// kTF32x3: every FP32 operand arrives pre-split as hi + lo (hi = x rounded to TF32,
// lo = x - hi).  Each K step issues lo·hi, hi·lo and hi·hi into the same FP32
// accumulator, which restores FP32-level accuracy from TF32 tensor-core products.
// The tensor core adds into its accumulator with truncation, an error that grows linearly
// with the number of accumulating instructions; the FP32 path therefore closes the TMEM
// accumulator every `chunk_kb` K blocks and the (eight) epilogue warps sum those chunk
// results in registers with round-to-nearest adds, which keeps the result within FP32
// rounding noise of a sequential FP32 dot product for any K.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "ptx.cuh"

namespace tfb {

// kKind16: f16 or bf16 operands (which one is a run-time flag); kKindTF32x3: split FP32.
enum GemmKind : int { kKind16 = 0, kKindTF32x3 = 2 };
enum OutType : int { kOutF32 = 0, kOutF16 = 1, kOutBF16 = 2 };
enum BiasMode : int { kBiasNone = 0, kBiasPerCol = 1, kBiasPerRow = 2 };

struct GemmArgs {
    int M, N, K;
    int tiles_m, tiles_n, num_tiles, k_blocks;
    int chunk_kb;         // K blocks accumulated in TMEM before the epilogue drains them
    int group_m;          // M-tiles per rasterisation group (L2 reuse of B tiles)
    void* C;
    long long ldc;        // elements
    int out_type;         // OutType
    const float* bias;
    int bias_mode;        // BiasMode
    int relu;
    int is_bf16;          // kKind16 only: 1 = bf16 operands, 0 = f16
    int* status;          // device error word (0 = ok)
};

constexpr int kBlockM = 128;
// Two control warps (TMA, MMA) plus four epilogue warps, eight on the FP32 path.
__host__ __device__ constexpr int gemm_threads(int kind) { return kind == kKindTF32x3 ? 320 : 192; }

template <int KIND, int BN, int STAGES>
struct GemmSmem {
    static constexpr int ES = (KIND == kKindTF32x3) ? 4 : 2;   // operand element bytes
    static constexpr int NSPLIT = (KIND == kKindTF32x3) ? 2 : 1;
    static constexpr int BK = 128 / ES;                         // K elements per stage
    static constexpr int A_TILE = kBlockM * 128;                // bytes
    static constexpr int B_TILE = BN * 128;
    static constexpr int STAGE_BYTES = NSPLIT * (A_TILE + B_TILE);
    static constexpr int BAR_BYTES = 256;
    static constexpr int TOTAL = 1024 + STAGES * STAGE_BYTES + BAR_BYTES;
};

// Bias, ReLU, conversion and store of 32 consecutive output columns of one row.
__device__ __forceinline__ void epilogue_store32(float (&v)[32], const GemmArgs& args, int row, int col0,
                                                 float row_bias) {
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

__device__ __forceinline__ void tile_coords(int t, const GemmArgs& a, int& tm, int& tn) {
    const int group_sz = a.group_m * a.tiles_n;
    const int g = t / group_sz;
    const int first_m = g * a.group_m;
    const int gm = min(a.tiles_m - first_m, a.group_m);
    const int r = t - g * group_sz;
    tm = first_m + r % gm;
    tn = r / gm;
}

template <int KIND, int BN, int STAGES, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(gemm_threads(KIND), 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmA2,
                    const __grid_constant__ CUtensorMap tmB, const __grid_constant__ CUtensorMap tmB2,
                    const GemmArgs args) {
    using S = GemmSmem<KIND, BN, STAGES>;
    constexpr int ES = S::ES;
    constexpr int BK = S::BK;
    constexpr bool TF32 = (KIND == kKindTF32x3);
    constexpr int UMMA_K = 32 / ES;          // K elements per tcgen05.mma
    constexpr int KSTEPS = BK / UMMA_K;      // 4
    constexpr int T_MN = 128 / ES;           // M/N elements per 128-byte swizzle row
    constexpr uint32_t TMEM_COLS = (2 * BN <= 32) ? 32 : (2 * BN <= 64) ? 64 : (2 * BN <= 128) ? 128
                                   : (2 * BN <= 256) ? 256 : 512;
    static_assert(BN % 32 == 0 && BN >= 32 && BN <= 256, "BN must be a multiple of 32 up to 256");
    static_assert(!A_MN || (kBlockM % T_MN == 0), "tile M must hold whole swizzle rows");
    static_assert(!B_MN || (BN % T_MN == 0), "tile N must hold whole swizzle rows");
    constexpr int EPI_WARPS = TF32 ? 8 : 4;
    constexpr int COLS = BN / (EPI_WARPS / 4);   // accumulator columns handled per epilogue thread
    static_assert(COLS % 32 == 0, "each epilogue thread handles whole 32-column groups");

    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

    const uint32_t bars = smem_base + STAGES * S::STAGE_BYTES;
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
    auto tfull_bar = [&](int b) { return bars + 8u * (2 * STAGES + b); };
    auto tempty_bar = [&](int b) { return bars + 8u * (2 * STAGES + 2 + b); };
    volatile uint32_t* tmem_holder =
        reinterpret_cast<volatile uint32_t*>(smem_gen + STAGES * S::STAGE_BYTES + 8 * (2 * STAGES + 4));
    volatile int* abort_flag =
        reinterpret_cast<volatile int*>(smem_gen + STAGES * S::STAGE_BYTES + 8 * (2 * STAGES + 4) + 4);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(tfull_bar(b), 1);
            mbar_init(tempty_bar(b), 32 * EPI_WARPS);
        }
        *abort_flag = 0;
        fence_mbar_init();
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmB);
        if constexpr (TF32) {
            tma_prefetch_desc(&tmA2);
            tma_prefetch_desc(&tmB2);
        }
    }
    if (warp == 1) {
        tmem_alloc<1>(smem_u32(const_cast<uint32_t*>(tmem_holder)), TMEM_COLS);
        tmem_relinquish<1>();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_holder;

    const int k_blocks = args.k_blocks;

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < args.num_tiles && ok; t += gridDim.x) {
                int tm, tn;
                tile_coords(t, args, tm, tn);
                const int m0 = tm * kBlockM, n0 = tn * BN;
                for (int kb = 0; kb < k_blocks; ++kb) {
                    ok = mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, args.status, kDevTimeoutEmpty);
                    if (!ok) break;
                    const uint32_t st = smem_base + s * S::STAGE_BYTES;
                    const uint32_t a_hi = st;
                    const uint32_t a_lo = st + S::A_TILE;
                    const uint32_t b_hi = st + S::NSPLIT * S::A_TILE;
                    const uint32_t b_lo = b_hi + S::B_TILE;
                    const uint32_t fb = full_bar(s);
                    mbar_arrive_expect_tx(fb, S::STAGE_BYTES);
                    const int k0 = kb * BK;
                    if constexpr (!A_MN) {
                        tma_load_2d(a_hi, &tmA, k0, m0, fb);
                        if constexpr (TF32) tma_load_2d(a_lo, &tmA2, k0, m0, fb);
                    } else {
#pragma unroll
                        for (int i = 0; i < kBlockM / T_MN; ++i) {
                            tma_load_2d(a_hi + i * (BK * 128), &tmA, m0 + i * T_MN, k0, fb);
                            if constexpr (TF32)
                                tma_load_2d(a_lo + i * (BK * 128), &tmA2, m0 + i * T_MN, k0, fb);
                        }
                    }
                    if constexpr (!B_MN) {
                        tma_load_2d(b_hi, &tmB, k0, n0, fb);
                        if constexpr (TF32) tma_load_2d(b_lo, &tmB2, k0, n0, fb);
                    } else {
#pragma unroll
                        for (int i = 0; i < BN / T_MN; ++i) {
                            tma_load_2d(b_hi + i * (BK * 128), &tmB, n0 + i * T_MN, k0, fb);
                            if constexpr (TF32)
                                tma_load_2d(b_lo + i * (BK * 128), &tmB2, n0 + i * T_MN, k0, fb);
                        }
                    }
                    if (++s == STAGES) { s = 0; ph ^= 1u; }
                }
            }
            // Drain: every load this thread issued has landed once the stage it targeted
            // was consumed; on the normal path the final __syncthreads implies that. On an
            // aborted run wait (bounded) for the stages still in flight.
            if (!ok || *abort_flag != 0) {
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
        if (lane == 0) {
            const uint32_t idesc = make_idesc(TF32 ? 2u : (args.is_bf16 ? 1u : 0u),
                                              A_MN ? 1u : 0u, B_MN ? 1u : 0u, kBlockM, BN);
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
            int s = 0;
            uint32_t ph = 0;
            uint32_t cit = 0;   // accumulator hand-offs so far (chunks, over all tiles)
            bool ok = true;
            for (int t = blockIdx.x; t < args.num_tiles && ok; t += gridDim.x) {
                for (int kb0 = 0; kb0 < k_blocks && ok; kb0 += args.chunk_kb, ++cit) {
                    const uint32_t buf = cit & 1u;
                    const uint32_t use = cit >> 1;
                    ok = mbar_wait(tempty_bar(buf), (use & 1u) ^ 1u, abort_flag, args.status,
                                   kDevTimeoutTmemEmpty);
                    if (!ok) break;
                    tc_fence_after_sync();
                    const uint32_t d_tmem = tmem_base + buf * (uint32_t)BN;
                    const int kb1 = min(kb0 + args.chunk_kb, k_blocks);
                    for (int kb = kb0; kb < kb1; ++kb) {
                        ok = mbar_wait(full_bar(s), ph, abort_flag, args.status, kDevTimeoutFull);
                        if (!ok) break;
                        tc_fence_after_sync();
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
                                umma_ss<1, true>(d_tmem, dal, db, idesc, acc);
                                umma_ss<1, true>(d_tmem, da, dbl, idesc, 1u);
                                umma_ss<1, true>(d_tmem, da, db, idesc, 1u);
                            } else {
                                umma_ss<1, false>(d_tmem, da, db, idesc, acc);
                            }
                        }
                        umma_commit<1>(empty_bar(s));
                        if (++s == STAGES) { s = 0; ph ^= 1u; }
                    }
                    if (!ok) break;
                    umma_commit<1>(tfull_bar(buf));
                }
            }
        }
    } else {
        // ------------------------------ epilogue ----------------------------------
        const int ew = warp - 2;
        const int q = warp & 3;            // TMEM lanes [32q, 32q+32) are the ones this warp may read
        const int cbase = (ew >> 2) * COLS; // first accumulator column of this warp
        uint32_t cit = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < args.num_tiles && ok; t += gridDim.x) {
            int tm, tn;
            tile_coords(t, args, tm, tn);
            const int m0 = tm * kBlockM, n0 = tn * BN + cbase;
            const int row = m0 + q * 32 + lane;
            const bool row_ok = row < args.M;
            float row_bias = 0.f;
            if (args.bias_mode == kBiasPerRow && row_ok) row_bias = __ldg(args.bias + row);
            const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)cbase;

            if constexpr (TF32) {
                float acc[COLS];
#pragma unroll
                for (int i = 0; i < COLS; ++i) acc[i] = 0.f;
                for (int kb0 = 0; kb0 < k_blocks; kb0 += args.chunk_kb, ++cit) {
                    const uint32_t buf = cit & 1u;
                    const uint32_t use = cit >> 1;
                    ok = mbar_wait(tfull_bar(buf), use & 1u, abort_flag, args.status, kDevTimeoutTmemFull);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    tc_fence_after_sync();
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
                    tc_fence_before_sync();
                    mbar_arrive(tempty_bar(buf));
                }
                if (!ok) break;
                if (row_ok) {
#pragma unroll
                    for (int c = 0; c < COLS / 32; ++c) {
                        if (n0 + c * 32 < args.N) {
                            float v[32];
#pragma unroll
                            for (int i = 0; i < 32; ++i) v[i] = acc[c * 32 + i];
                            epilogue_store32(v, args, row, n0 + c * 32, row_bias);
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
                    if (!row_ok) continue;
                    float v[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
                    epilogue_store32(v, args, row, col0, row_bias);
                }
                tc_fence_before_sync();
                mbar_arrive(tempty_bar(buf));
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
