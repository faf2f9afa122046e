// Delivery of one rank's columns of a column-parallel layer's output to the other ranks.
//
// The large-M kernel writes its [rows, cols] result into the column range it owns of this rank's
// [rows, ld] output.  This entry point then copies that range into the same place of every other
// rank's output, given as peer-mapped pointers, with one strided device-to-device copy per
// destination: the copy engines move the data over NVLink while the SMs run the next rows' kernel
// on another stream.  Takes the place of the all-gather op that follows the matmul in the reference
// (python/hidet/graph/ops/distributed.py:63-97), without its staging buffer and reshuffle.
#include "common.cuh"

extern "C" {

B200Q_API int b200q_push_columns(const void *src, void *const *dst, int n_dst, int64_t rows, int64_t cols, int64_t ld,
                                 int64_t col_offset, void *stream) {
    using namespace b200q;
    if (n_dst < 0 || n_dst > 64) return set_error(B200Q_INVALID_ARGUMENT, "push_columns: n_dst must be 0..64, got %d", n_dst);
    if (rows < 0 || cols < 0 || col_offset < 0 || ld < col_offset + cols) {
        return set_error(B200Q_INVALID_ARGUMENT, "push_columns: columns [%lld, %lld) do not fit rows of %lld elements", (long long)col_offset,
                         (long long)(col_offset + cols), (long long)ld);
    }
    if (rows == 0 || cols == 0 || n_dst == 0) return B200Q_OK;
    if (src == nullptr || dst == nullptr) return set_error(B200Q_INVALID_ARGUMENT, "push_columns: null pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const size_t pitch = (size_t)ld * sizeof(__half);
    const size_t width = (size_t)cols * sizeof(__half);
    const char *from = static_cast<const char *>(src) + (size_t)col_offset * sizeof(__half);
    for (int i = 0; i < n_dst; ++i) {
        if (dst[i] == nullptr) return set_error(B200Q_INVALID_ARGUMENT, "push_columns: destination %d is null", i);
        if (dst[i] == src) continue;  // this rank's own buffer
        char *to = static_cast<char *>(dst[i]) + (size_t)col_offset * sizeof(__half);
        B200Q_CUDA_TRY(cudaMemcpy2DAsync(to, pitch, from, pitch, width, (size_t)rows, cudaMemcpyDefault, s));
    }
    return B200Q_OK;
}

}  // extern "C"
