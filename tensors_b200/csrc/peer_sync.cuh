// Device-side pieces shared by the kernels that exchange data between GPUs through peer memory
// (ordinary loads and stores over NVLink; nothing here uses cluster multicast or multimem).
//
// Synchronisation is by flags in each rank's own region: monotonic step counters, one word per
// (CTA, source rank) and barrier, written with release and polled with acquire semantics at system
// scope. CTA b of a rank only ever waits for CTA b of the other ranks. Every wait is bounded by a
// wall-clock limit; a waiter that gives up returns false and its kernel records kDevTimeoutExchange.
#pragma once

#include <cstdint>

#include "ptx.cuh"

namespace tfb {

constexpr int kMaxWorld = 8;               // ranks of one group (the GPUs of one NVSwitch box)
constexpr int kMaxExchangeCtas = 256;      // flag rows reserved per region
constexpr int kDevTimeoutExchange = 107;   // a rank gave up waiting for a peer's flag

// Flag area of a region: epoch[kMaxExchangeCtas], then two barriers of [kMaxExchangeCtas][kMaxWorld] words.
constexpr size_t kFlagBytes = sizeof(uint32_t) * (kMaxExchangeCtas + 2 * kMaxExchangeCtas * kMaxWorld);

__device__ __forceinline__ uint32_t* flag_word(uint8_t* region, long long flags_off, int barrier, int cta, int src) {
    return reinterpret_cast<uint32_t*>(region + flags_off) + kMaxExchangeCtas +
           (barrier * kMaxExchangeCtas + cta) * kMaxWorld + src;
}

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// Loads of data another GPU wrote: served by the owning GPU's L2, never by this SM's L1.
__device__ __forceinline__ float4 ld_peer(const float4* p) {
    float4 v;
    asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_peer(float4* p, const float4& v) {
    asm volatile("st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
                 ::"l"(p), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}

__device__ __forceinline__ void st_relaxed_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_relaxed_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Waits until *flag has reached `epoch` (wrap-safe) or the wall-clock limit runs out. The polls are
// relaxed loads; one acquire fence at system scope after the flag has been seen orders everything the
// waiter reads afterwards behind the writer's release.
__device__ __forceinline__ bool wait_flag(const uint32_t* flag, uint32_t epoch, unsigned long long limit_ns) {
    bool seen = (int32_t)(ld_relaxed_sys(flag) - epoch) >= 0;
    if (!seen) {
        const uint64_t t0 = global_timer_ns();
        uint32_t polls = 0;
        while (true) {
            if ((int32_t)(ld_relaxed_sys(flag) - epoch) >= 0) { seen = true; break; }
            if (((++polls) & 15u) == 0 && global_timer_ns() - t0 > limit_ns) break;
        }
    }
    if (seen) asm volatile("fence.acquire.sys;" ::: "memory");
    return seen;
}

}  // namespace tfb
