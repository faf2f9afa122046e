// b200q_qlinear_f16_i8_static: the quantized linear for callers that have no way to obtain scratch
// memory.
//
// Who that is: code that is handed nothing but device pointers and a stream -- the launch function of
// an already compiled graph, a plugin running inside another runtime's execution loop, a serving
// process whose device memory was carved up once at start-up and is fully committed.  Such a caller
// has no allocator to ask, and it must not reach for cudaMalloc itself: that call synchronises the
// whole device, may fail when memory is committed, and breaks the host runtime's accounting.
//
// What it gets instead: the scratch lives in a fixed array that is part of this library's device
// image.  Every GPU that loads the library holds kStaticScratchBytes (512 KiB) for it until the process
// exits.  Nothing here allocates or frees: no cudaMalloc / cudaFree, no allocating library call.
#include <mutex>

#include "common.cuh"
#include "qlinear.h"

namespace b200q {
namespace {

constexpr size_t kStaticScratchBytes = 512u << 10;

// The scratch itself.  In host code this name is only a handle for the runtime: it is not a device
// address and must never be passed to a kernel.  The address each device uses is looked up below.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
void *g_scratch_ptr[kMaxDevices] = {nullptr};
cudaError_t g_scratch_err[kMaxDevices];
std::once_flag g_scratch_once[kMaxDevices];

// Device address of the scratch on the calling thread's current device.  The first call on a device
// asks the runtime for it (with that device current) and keeps the answer.
int static_scratch(void **out) {
    int dev = -1;
    B200Q_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return set_error(B200Q_UNSUPPORTED, "qlinear_f16_i8_static: device index %d out of range", dev);
    std::call_once(g_scratch_once[dev], [dev]() {
        void *p = nullptr;
        g_scratch_err[dev] = cudaGetSymbolAddress(&p, g_static_scratch);
        g_scratch_ptr[dev] = p;
    });
    if (g_scratch_err[dev] != cudaSuccess || g_scratch_ptr[dev] == nullptr) {
        return set_error(B200Q_CUDA_ERROR, "qlinear_f16_i8_static: cudaGetSymbolAddress failed on device %d: %s", dev,
                         cudaGetErrorString(g_scratch_err[dev]));
    }
    *out = g_scratch_ptr[dev];
    return B200Q_OK;
}

}  // namespace
}  // namespace b200q

extern "C" {

B200Q_API size_t b200q_qlinear_static_scratch_bytes(void) { return b200q::kStaticScratchBytes; }

B200Q_API int b200q_qlinear_f16_i8_static(const void *a, const void *wq, const void *scale, void *c, int64_t M, int64_t N,
                                          int64_t K, int w_layout, void *stream) {
    using namespace b200q;
    if (M < 0 || N < 0 || K < 0) return set_error(B200Q_INVALID_ARGUMENT, "qlinear_f16_i8_static: negative size M=%lld N=%lld K=%lld", (long long)M, (long long)N, (long long)K);
    if (w_layout != B200Q_LAYOUT_KN) return set_error(B200Q_UNSUPPORTED, "qlinear_f16_i8_static: only the [K, N] weight layout is served here");
    if (M > 2147483647LL || N > 2147483647LL || K > 2147483647LL) return set_error(B200Q_UNSUPPORTED, "qlinear_f16_i8_static: sizes beyond 2^31-1 are not supported");
    if (M == 0 || N == 0) return B200Q_OK;
    if (scale == nullptr || c == nullptr) return set_error(B200Q_INVALID_ARGUMENT, "qlinear_f16_i8_static: null output or scale pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (K == 0) {  // an empty sum, as in b200q_qlinear_f16_i8
        B200Q_CUDA_TRY(cudaMemsetAsync(c, 0, (size_t)M * N * sizeof(__half), s));
        return B200Q_OK;
    }
    if (a == nullptr || wq == nullptr) return set_error(B200Q_INVALID_ARGUMENT, "qlinear_f16_i8_static: null input pointer");
    if (!decode_kn_supported(a, wq, N, K)) {
        return set_error(B200Q_UNSUPPORTED, "qlinear_f16_i8_static: operands need 16-byte aligned bases and rows (N %% 16 == 0, K %% 8 == 0); "
                                            "got N=%lld K=%lld", (long long)N, (long long)K);
    }
    if (use_prefill_kernel(M, N, K)) return launch_prefill_kn(a, wq, scale, c, M, N, K, s);  // needs no scratch at all

    const DecodePlan plan = plan_decode(M, N, K);
    const size_t need = plan.counter_bytes + plan.partial_bytes;
    if (need > kStaticScratchBytes) {
        return set_error(B200Q_WORKSPACE_TOO_SMALL,
                         "qlinear_f16_i8_static: M=%lld N=%lld K=%lld needs %zu bytes of scratch, the built-in scratch holds %zu; "
                         "use b200q_qlinear_f16_i8 with a caller-provided workspace",
                         (long long)M, (long long)N, (long long)K, need, kStaticScratchBytes);
    }
    void *scratch = nullptr;
    if (need > 0) {
        int rc = static_scratch(&scratch);
        if (rc != B200Q_OK) return rc;
        // The arrival counters must read zero when the kernel starts.  A completed call leaves them
        // zero, but the array is shared by every caller and survives failed calls, so clear the ones
        // this problem uses (one per output tile and cluster rank) here.
        const size_t used = (size_t)plan.n_tiles * plan.m_tiles * plan.cluster * sizeof(unsigned int);
        B200Q_CUDA_TRY(cudaMemsetAsync(scratch, 0, used < plan.counter_bytes ? used : plan.counter_bytes, s));
    }
    return launch_decode_kn(a, wq, scale, c, M, N, K, 0, K, true, scratch, need, s);
}

}  // extern "C"
