// Thin inline-PTX wrappers for the sm_100a features the contraction kernels use:
// mbarrier, TMA (cp.async.bulk.tensor), tcgen05 (TMEM alloc, MMA, commit, ld) and
// the shared-memory / instruction descriptors that tcgen05.mma consumes.
//
// Every wait in this file is bounded: after a wall-clock limit the waiter records
// an error code and returns false, so a broken pipeline ends the kernel instead of
// hanging the GPU.
#pragma once

#include <cstdint>
#include <cuda.h>

namespace tfb {

// ---------------------------------------------------------------------------
// Error codes written by kernels into the per-device status word.
// ---------------------------------------------------------------------------
enum DeviceError : int {
    kDevOk = 0,
    kDevTimeoutFull = 101,     // consumer gave up waiting for a TMA-filled stage
    kDevTimeoutEmpty = 102,    // producer gave up waiting for a free stage
    kDevTimeoutTmemFull = 103, // epilogue gave up waiting for an accumulator
    kDevTimeoutTmemEmpty = 104,// MMA issuer gave up waiting for a drained accumulator
    kDevTimeoutDrain = 105,    // producer gave up waiting for its own copies in flight
    kDevTimeoutPeer = 106,     // a CTA gave up waiting for its cluster peer
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// ---------------------------------------------------------------------------
// Programmatic dependent launch. A kernel launched with the programmatic-serialization attribute
// may start while the kernel before it on the stream is still running; pdl_wait() blocks until that
// kernel has completed and its memory is visible, so it must come before the first access to global
// memory. pdl_launch_dependents() lets the NEXT kernel start its own prologue early; since that
// kernel waits for this whole grid in its own pdl_wait(), triggering early is always safe. Both are
// no-ops in a kernel that was launched the ordinary way.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// ---------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}

// Arrive on a barrier that lives in another CTA of the cluster (address from mapa).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar)
                 : "memory");
}

// One poll. The warp may be suspended by the hardware for up to `kSuspendNs` while the phase is
// incomplete (it is woken as soon as the phase completes), so waiting warps do not burn the issue
// slots that working warps of the same SM partition need.
constexpr uint32_t kSuspendNs = 20000;
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(done)
        : "r"(bar), "r"(parity), "r"(kSuspendNs)
        : "memory");
    return done;
}

// Non-suspending poll (mbarrier.test_wait): for the few waits on a latency-critical handshake path.
__device__ __forceinline__ uint32_t mbar_test_wait(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done;
}

// Wall-clock budget of one wait. The longest legitimate wait is one output tile of
// the largest supported problem (milliseconds); two seconds is far beyond that and
// still short enough for a broken run to end quickly.
constexpr uint64_t kWaitBudgetNs = 2000000000ull;

// Bounded wait. `abort_flag` is a shared-memory word that any role sets when it gives
// up; every other role sees it on its next poll and leaves too. Returns false when
// the wait was abandoned.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          int* status, int err_code) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = global_timer_ns();
    uint32_t polls = 0;
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if (((++polls) & 0xfu) == 0) {
            if (*abort_flag != 0) return false;
            if (global_timer_ns() - t0 > kWaitBudgetNs) {
                *abort_flag = err_code;
                if (status != nullptr) atomicCAS(status, 0, err_code);
                return false;
            }
        }
    }
}

// Same contract as mbar_wait, polling without suspension.
__device__ __forceinline__ bool mbar_wait_spin(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                               int* status, int err_code) {
    if (mbar_test_wait(bar, parity)) return true;
    const uint64_t t0 = global_timer_ns();
    uint32_t polls = 0;
    while (true) {
        if (mbar_test_wait(bar, parity)) return true;
        if (((++polls) & 0xfffu) == 0) {
            if (*abort_flag != 0) return false;
            if (global_timer_ns() - t0 > kWaitBudgetNs) {
                *abort_flag = err_code;
                if (status != nullptr) atomicCAS(status, 0, err_code);
                return false;
            }
        }
    }
}

// ---------------------------------------------------------------------------
// Proxy / tcgen05 fences
// ---------------------------------------------------------------------------
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ---------------------------------------------------------------------------
// TMA
// ---------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* desc) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(desc)) : "memory");
}

// 2-D tiled load global -> shared, completion counted in bytes on `bar`.
// x is the innermost coordinate; x * element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* desc, int x, int y,
                                            uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(desc)), "r"(x), "r"(y), "r"(bar)
        : "memory");
}

// Same load issued from either CTA of a pair; `bar` may live in the pair leader's
// shared memory (a shared::cluster address).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* desc, int x,
                                                 int y, uint32_t cluster_bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(desc)), "r"(x), "r"(y), "r"(cluster_bar)
        : "memory");
}

// 3-D and 4-D tiled loads (x innermost, 16-byte rule as above; the outer coordinates may lie outside
// the tensor, where the load delivers zeros). PAIR selects the form a CTA pair uses.
template <bool PAIR>
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* desc, int x, int y, int z,
                                            uint32_t bar) {
    if constexpr (PAIR)
        asm volatile(
            "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
            " [%0], [%1, {%2, %3, %4}], [%5];"
            ::"r"(dst), "l"(reinterpret_cast<uint64_t>(desc)), "r"(x), "r"(y), "r"(z), "r"(bar)
            : "memory");
    else
        asm volatile(
            "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
            " [%0], [%1, {%2, %3, %4}], [%5];"
            ::"r"(dst), "l"(reinterpret_cast<uint64_t>(desc)), "r"(x), "r"(y), "r"(z), "r"(bar)
            : "memory");
}
template <bool PAIR>
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* desc, int x, int y, int z, int w,
                                            uint32_t bar) {
    if constexpr (PAIR)
        asm volatile(
            "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
            " [%0], [%1, {%2, %3, %4, %5}], [%6];"
            ::"r"(dst), "l"(reinterpret_cast<uint64_t>(desc)), "r"(x), "r"(y), "r"(z), "r"(w), "r"(bar)
            : "memory");
    else
        asm volatile(
            "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes"
            " [%0], [%1, {%2, %3, %4, %5}], [%6];"
            ::"r"(dst), "l"(reinterpret_cast<uint64_t>(desc)), "r"(x), "r"(y), "r"(z), "r"(w), "r"(bar)
            : "memory");
}

// 2-D tiled store shared -> global (bulk-group completion).
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* desc, uint32_t src, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(reinterpret_cast<uint64_t>(desc)), "r"(src), "r"(x), "r"(y)
                 : "memory");
}
__device__ __forceinline__ void tma_store_commit() {
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait_all() {
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// ---------------------------------------------------------------------------
// Cluster helpers
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t cta_rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(cta_rank));
    return r;
}
// Orders this thread's earlier memory accesses before its later ones as seen by the other CTAs of the
// cluster (used around a hand-off through distributed shared memory).
__device__ __forceinline__ void fence_acq_rel_cluster() { asm volatile("fence.acq_rel.cluster;" ::: "memory"); }
// 16-byte store into the shared memory of a CTA of the cluster (address from mapa).
__device__ __forceinline__ void st_shared_cluster_v4(uint32_t cluster_addr, float a, float b, float c, float d) {
    asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(cluster_addr), "f"(a), "f"(b), "f"(c), "f"(d)
                 : "memory");
}
__device__ __forceinline__ void cluster_arrive() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// ---------------------------------------------------------------------------
// TMEM allocation (whole-warp instructions)
// ---------------------------------------------------------------------------
template <int CTA_GROUP>
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
    if constexpr (CTA_GROUP == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(dst_smem), "r"(ncols) : "memory");
    } else {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(dst_smem), "r"(ncols) : "memory");
    }
}
template <int CTA_GROUP>
__device__ __forceinline__ void tmem_relinquish() {
    if constexpr (CTA_GROUP == 1) {
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    } else {
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
}
template <int CTA_GROUP>
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    if constexpr (CTA_GROUP == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
                     : "memory");
    } else {
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
                     : "memory");
    }
}

// ---------------------------------------------------------------------------
// tcgen05.mma (single-thread issue), operands A and B from shared memory.
// KIND_TF32 = true -> kind::tf32 (fp32 containers), else kind::f16 (f16 / bf16).
// ---------------------------------------------------------------------------
template <int CTA_GROUP, bool KIND_TF32>
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                        uint32_t idesc, uint32_t accumulate) {
    if constexpr (CTA_GROUP == 1 && KIND_TF32) {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}\n"
            ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
    } else if constexpr (CTA_GROUP == 1 && !KIND_TF32) {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
            ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
    } else if constexpr (CTA_GROUP == 2 && KIND_TF32) {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}\n"
            ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
    } else {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
            ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
    }
}

// Make `bar` complete one arrival once every tcgen05.mma issued so far by this
// thread has finished (implies tcgen05.fence::before_thread_sync).
template <int CTA_GROUP>
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    if constexpr (CTA_GROUP == 1) {
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                     ::"r"(bar) : "memory");
    } else {
        asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                     ::"r"(bar) : "memory");
    }
}
// TMEM -> registers: this warp's 32 lanes x 32 consecutive 32-bit columns.
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
          "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
          "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ---------------------------------------------------------------------------
// Descriptors
// ---------------------------------------------------------------------------
// 64-bit shared-memory matrix descriptor: start address, leading / stride byte
// offsets (all >> 4), descriptor version 1 at bit 46, swizzle mode at bits 61..63
// (0 none, 2 = 128-byte, 4 = 64-byte, 6 = 32-byte).
__host__ __device__ constexpr uint64_t make_smem_desc(uint32_t saddr, uint32_t lbo_bytes,
                                                      uint32_t sbo_bytes, uint32_t swizzle_code) {
    return (uint64_t)((saddr & 0x3ffffu) >> 4) | ((uint64_t)((lbo_bytes >> 4) & 0x3fffu) << 16) |
           ((uint64_t)((sbo_bytes >> 4) & 0x3fffu) << 32) | ((uint64_t)1 << 46) |
           ((uint64_t)(swizzle_code & 7u) << 61);
}

// 32-bit instruction descriptor for kind::f16 / kind::tf32 with an FP32 accumulator.
// fmt: 0 = f16, 1 = bf16, 2 = tf32. a_mn / b_mn: 1 when the operand's M/N dimension
// (rather than K) is contiguous in shared memory.
__host__ __device__ constexpr uint32_t make_idesc(uint32_t fmt, uint32_t a_mn, uint32_t b_mn,
                                                  uint32_t umma_m, uint32_t umma_n) {
    return (1u << 4) | (fmt << 7) | (fmt << 10) | (a_mn << 15) | (b_mn << 16) |
           ((umma_n >> 3) << 17) | ((umma_m >> 4) << 24);
}

}  // namespace tfb
