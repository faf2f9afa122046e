// Host-side runtime of libhidet_b200q.so: thread-local error state, per-device cached properties,
// the device status word and tensor-map encoding.
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "common.cuh"

namespace b200q {

namespace {

thread_local char g_last_error[1024] = {0};
thread_local char g_returned_error[1024] = {0};

constexpr int kMaxDevices = 64;

struct DeviceState {
    std::once_flag once;
    int sm_count = 0;
    unsigned int *status_word = nullptr;
    cudaError_t init_error = cudaSuccess;
};
DeviceState g_devices[kMaxDevices];

// Two status words per device, part of the loaded module image (no allocation at run time): every
// wait that ran out, or-ed together, and the first one.
__device__ unsigned int g_status_word[2] = {0, 0};

DeviceState *current_device_state() {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
    DeviceState *st = &g_devices[dev];
    std::call_once(st->once, [st, dev]() {
        st->init_error = cudaDeviceGetAttribute(&st->sm_count, cudaDevAttrMultiProcessorCount, dev);
        if (st->init_error != cudaSuccess) return;
        void *p = nullptr;
        st->init_error = cudaGetSymbolAddress(&p, g_status_word);
        st->status_word = static_cast<unsigned int *>(p);
    });
    if (st->init_error != cudaSuccess) return nullptr;
    return st;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, []() {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess) {
            fn = reinterpret_cast<EncodeTiledFn>(p);
        }
    });
    return fn;
}

}  // namespace

int set_error(int code, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
    va_end(ap);
    return code;
}

unsigned int *device_status_word() {
    DeviceState *st = current_device_state();
    return st ? st->status_word : nullptr;
}

int sm_count() {
    DeviceState *st = current_device_state();
    return st ? st->sm_count : 0;
}

int make_tensor_map_2d(CUtensorMap *map, CUtensorMapDataType dtype, const void *base, uint64_t inner, uint64_t outer,
                       uint64_t row_bytes, uint32_t box_inner, uint32_t box_outer, CUtensorMapSwizzle swizzle,
                       CUtensorMapL2promotion promo) {
    EncodeTiledFn fn = get_encode_fn();
    if (fn == nullptr) return set_error(B200Q_CUDA_ERROR, "cuTensorMapEncodeTiled is not available from the driver");
    if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0 || (row_bytes & 15u) != 0) {
        return set_error(B200Q_INVALID_ARGUMENT, "tensor map needs a 16-byte aligned base and row stride (base %p, stride %llu)",
                         base, (unsigned long long)row_bytes);
    }
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {row_bytes};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t elem_strides[2] = {1, 1};
    CUresult r = fn(map, dtype, 2, const_cast<void *>(base), dims, strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    swizzle, promo, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        return set_error(B200Q_CUDA_ERROR, "cuTensorMapEncodeTiled failed with CUresult %d (dims %llu x %llu, stride %llu, box %u x %u)",
                         (int)r, (unsigned long long)inner, (unsigned long long)outer, (unsigned long long)row_bytes, box_inner,
                         box_outer);
    }
    return B200Q_OK;
}

}  // namespace b200q

extern "C" {

B200Q_API int b200q_version(void) { return 100; }

B200Q_API const char *b200q_get_last_error(void) {
    std::memcpy(b200q::g_returned_error, b200q::g_last_error, sizeof(b200q::g_last_error));
    b200q::g_last_error[0] = 0;
    return b200q::g_returned_error;
}

B200Q_API int b200q_check_status(void) {
    unsigned int *word = b200q::device_status_word();
    if (word == nullptr) return b200q::set_error(B200Q_CUDA_ERROR, "no usable CUDA device for the calling thread");
    B200Q_CUDA_TRY(cudaDeviceSynchronize());
    unsigned int v[2] = {0, 0};
    B200Q_CUDA_TRY(cudaMemcpy(v, word, sizeof(v), cudaMemcpyDeviceToHost));
    if (v[0] == 0) return B200Q_OK;
    const unsigned int zero[2] = {0, 0};
    B200Q_CUDA_TRY(cudaMemcpy(word, zero, sizeof(zero), cudaMemcpyHostToDevice));
    if ((v[0] & 0xbfffffffu) == 0) {
        return b200q::set_error(B200Q_INVALID_ARGUMENT, "an embedding lookup met an index outside its table (that row was written as zeros)");
    }
    return b200q::set_error(B200Q_KERNEL_TIMEOUT,
                            "a bounded device-side wait ran out: first in kernel id %u at wait site %u; all that ran out, or-ed: 0x%08x",
                            v[1] & 0xffu, (v[1] >> 8) & 0xffu, v[0]);
}

}  // extern "C"
