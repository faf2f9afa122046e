// Shared host/device helpers of libhidet_b200q.so: error state, launch checks and the sm_100a PTX
// wrappers (mbarrier, TMA, tcgen05) the kernels are written with.
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/hidet_b200q.h"

namespace b200q {

// ---------------------------------------------------------------------------------------------
// host side: error state
// ---------------------------------------------------------------------------------------------

// Stores a printf-formatted message in the calling thread's error slot and returns `code`.
int set_error(int code, const char *fmt, ...);

#define B200Q_CUDA_TRY(expr)                                                                        \
    do {                                                                                            \
        cudaError_t err__ = (expr);                                                                 \
        if (err__ != cudaSuccess) {                                                                 \
            return ::b200q::set_error(B200Q_CUDA_ERROR, "%s failed: %s (%s:%d)", #expr,             \
                                      cudaGetErrorString(err__), __FILE__, __LINE__);               \
        }                                                                                           \
    } while (0)

// After a kernel launch: reports launch-configuration errors without synchronising.
#define B200Q_CHECK_LAUNCH(name)                                                                    \
    do {                                                                                            \
        cudaError_t err__ = cudaGetLastError();                                                     \
        if (err__ != cudaSuccess) {                                                                 \
            return ::b200q::set_error(B200Q_CUDA_ERROR, "launch of %s failed: %s", name,            \
                                      cudaGetErrorString(err__));                                   \
        }                                                                                           \
    } while (0)

// Device-global status word: a kernel whose bounded wait runs out ORs a code into it and returns.
// Code layout: bits 0..7 kernel id, bits 8..15 wait site, bit 31 set.
unsigned int *device_status_word();  // device address for the current device (nullptr on failure)

constexpr unsigned int kKernelDecode = 1;
constexpr unsigned int kKernelPrefill = 2;

// Number of SMs of the current device (cached per device).
int sm_count();

// Encodes a 2-D tiled tensor map.  `inner`/`outer` are the tensor extents in elements, `row_bytes`
// the stride between consecutive outer indices, box_* the tile extents.  swizzle is a
// CUtensorMapSwizzle value.  Returns a b200q_status.
int make_tensor_map_2d(CUtensorMap *map, CUtensorMapDataType dtype, const void *base, uint64_t inner, uint64_t outer,
                       uint64_t row_bytes, uint32_t box_inner, uint32_t box_outer, CUtensorMapSwizzle swizzle,
                       CUtensorMapL2promotion promo);

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }
inline int64_t round_up(int64_t a, int64_t b) { return ceil_div(a, b) * b; }

// ---------------------------------------------------------------------------------------------
// device side: PTX wrappers
// ---------------------------------------------------------------------------------------------
#ifdef __CUDACC__

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ uint32_t lane_id() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%laneid;" : "=r"(r));
    return r;
}

// One lane of the (fully converged) warp.
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(pred));
    return pred != 0;
}

// ---- mbarrier ----
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// One poll: returns true once the phase with the given parity has completed.  The thread may be
// suspended inside the instruction for up to about `kWaitHintNs` while the phase is pending, so a
// polling loop spends few issue slots.
constexpr uint32_t kWaitHintNs = 2000;
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(kWaitHintNs)
        : "memory");
    return ok != 0;
}

// Bounded wait on an mbarrier phase.  Returns false if `limit` polls passed without the phase
// completing; the caller then records the failure and leaves.  Each poll of try_wait already
// blocks for a hardware-defined interval, so the limit is a time bound of the order of a second.
constexpr uint32_t kSpinLimit = 1u << 20;
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, uint32_t limit = kSpinLimit) {
    for (uint32_t i = 0; i < limit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
    }
    return false;
}

// status[0] collects every wait that ran out (codes or-ed together: one failure starves the other
// roles, whose waits then run out too); status[1] keeps the first one.
__device__ __forceinline__ void report_timeout(unsigned int *status, unsigned int kernel, unsigned int site) {
    if (status != nullptr) {
        const unsigned int code = 0x80000000u | (site << 8) | kernel;
        atomicOr(status, code);
        atomicCAS(status + 1, 0u, code);
    }
}

// ---- TMA ----
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap *map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// 2-D tiled load global -> shared, completion counted in bytes on `bar`.  x is the inner
// (contiguous) coordinate in elements and must make x * element_size a multiple of 16.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int32_t x, int32_t y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tma_load_2d_hint(uint32_t dst, const CUtensorMap *map, int32_t x, int32_t y,
                                                 uint32_t bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint"
        " [%0], [%1, {%3, %4}], [%2], %5;"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y), "l"(policy)
        : "memory");
}
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
    return p;
}

// Makes generic-proxy writes to shared memory visible to the async proxy (TMA, tcgen05.mma).
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---- programmatic dependent launch ----
// launch_dependents: the next kernel in the stream may start its prologue once every CTA of this grid
// has said so.  wait: blocks until the previous kernel in the stream has completed and its writes are
// visible; a no-op when the kernel was not launched as a programmatic dependent.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// ---- int8 -> f16 ----
// Four signed bytes packed in `v` -> (b0, b2) in lo and (b1, b3) in hi as exact f16 values.
// 0x6400 | u is the f16 number 1024 + u for u in [0, 256); with u = b ^ 0x80 = b + 128 the
// subtraction of 1152 leaves b exactly.
__device__ __forceinline__ void cvt_s8x4_to_f16x4(uint32_t v, uint32_t &lo, uint32_t &hi) {
    const uint32_t magic = 0x64806480u;           // per half: 0x6400 | 0x80 folds the sign flip in
    const uint32_t bias = 0x64806480u;            // f16x2 (1152, 1152)
    uint32_t l = (v & 0x00ff00ffu) ^ magic;
    uint32_t h = ((v >> 8) & 0x00ff00ffu) ^ magic;
    asm("sub.f16x2 %0, %1, %2;" : "=r"(lo) : "r"(l), "r"(bias));
    asm("sub.f16x2 %0, %1, %2;" : "=r"(hi) : "r"(h), "r"(bias));
}

#endif  // __CUDACC__

}  // namespace b200q
