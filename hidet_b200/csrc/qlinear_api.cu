// Entry points of the f16 x int8 quantized linear and the shape-agnostic kernel that serves operands
// the TMA kernels cannot take (rows that are not 16-byte multiples, unaligned bases).
#include "common.cuh"
#include "qlinear.h"

namespace b200q {
namespace {

constexpr int kGenericThreads = 128;

// One thread per output element, fp32 accumulation over k in [k_begin, k_end), one rounding.
// Adjacent threads take adjacent columns, so [K, N] weights are read coalesced; [N, K] weights are
// read with a stride and rely on the caches.  Correctness net, not a tuned path.
__global__ void __launch_bounds__(kGenericThreads) qlinear_generic_kernel(const __half *__restrict__ a,
                                                                          const int8_t *__restrict__ wq,
                                                                          const __half *__restrict__ scale,
                                                                          __half *__restrict__ c, int64_t M, int64_t N,
                                                                          int64_t K, int64_t k_begin, int64_t k_end,
                                                                          int layout) {
    const int64_t n = (int64_t)blockIdx.x * kGenericThreads + threadIdx.x;
    const int64_t m = blockIdx.y;
    if (n >= N || m >= M) return;
    const __half *arow = a + m * K;
    float acc = 0.0f;
    if (layout == B200Q_LAYOUT_KN) {
        for (int64_t k = k_begin; k < k_end; ++k) acc = fmaf(__half2float(arow[k]), (float)wq[k * N + n], acc);
    } else {
        const int8_t *wrow = wq + n * K;
        for (int64_t k = k_begin; k < k_end; ++k) acc = fmaf(__half2float(arow[k]), (float)wrow[k], acc);
    }
    c[m * N + n] = __float2half_rn(acc * __half2float(scale[n]));
}

int launch_generic(const void *a, const void *wq, const void *scale, void *c, int64_t M, int64_t N, int64_t K,
                   int64_t k_begin, int64_t k_end, int layout, cudaStream_t stream) {
    if (M > 65535) return set_error(B200Q_UNSUPPORTED, "qlinear: M=%lld is too large for the unaligned-operand kernel", (long long)M);
    dim3 grid((unsigned)ceil_div(N, kGenericThreads), (unsigned)M, 1);
    qlinear_generic_kernel<<<grid, kGenericThreads, 0, stream>>>(static_cast<const __half *>(a), static_cast<const int8_t *>(wq),
                                                                 static_cast<const __half *>(scale), static_cast<__half *>(c), M, N,
                                                                 K, k_begin, k_end, layout);
    B200Q_CHECK_LAUNCH("qlinear_generic_kernel");
    return B200Q_OK;
}

int check_qlinear_args(const char *op, const void *a, const void *wq, const void *scale, const void *c, int64_t M, int64_t N,
                       int64_t K, int layout) {
    if (M < 0 || N < 0 || K < 0) return set_error(B200Q_INVALID_ARGUMENT, "%s: negative size M=%lld N=%lld K=%lld", op, (long long)M, (long long)N, (long long)K);
    if (layout != B200Q_LAYOUT_KN && layout != B200Q_LAYOUT_NK) return set_error(B200Q_INVALID_ARGUMENT, "%s: unknown weight layout %d", op, layout);
    if (M > 0 && N > 0 && (c == nullptr || scale == nullptr)) return set_error(B200Q_INVALID_ARGUMENT, "%s: null output or scale pointer", op);
    if (M > 0 && N > 0 && K > 0 && (a == nullptr || wq == nullptr)) return set_error(B200Q_INVALID_ARGUMENT, "%s: null input pointer", op);
    if (M > 2147483647LL || N > 2147483647LL || K > 2147483647LL) return set_error(B200Q_UNSUPPORTED, "%s: sizes beyond 2^31-1 are not supported", op);
    return B200Q_OK;
}

}  // namespace
}  // namespace b200q

extern "C" {

B200Q_API size_t b200q_qlinear_workspace_bytes(int64_t M, int64_t N, int64_t K, int w_layout) {
    using namespace b200q;
    (void)w_layout;
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    const DecodePlan pl = plan_decode(M, N, K);
    size_t need = pl.counter_bytes + pl.partial_bytes;
    if (use_prefill_kernel(M, N, K)) {
        // the tensor-memory kernel needs scratch only when it splits K; operands it cannot take (alignment is not
        // known here) go to the small-M kernel, so its need is covered as well
        const size_t split = plan_prefill_split(M, N, K).workspace_bytes;
        if (split > need) need = split;
    }
    return need;
}

B200Q_API int b200q_qlinear_f16_i8(const void *a, const void *wq, const void *scale, void *c, int64_t M, int64_t N,
                                   int64_t K, int w_layout, void *workspace, size_t workspace_bytes, void *stream) {
    using namespace b200q;
    int rc = check_qlinear_args("qlinear_f16_i8", a, wq, scale, c, M, N, K, w_layout);
    if (rc != B200Q_OK) return rc;
    if (M == 0 || N == 0) return B200Q_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (K == 0) {  // an empty sum
        B200Q_CUDA_TRY(cudaMemsetAsync(c, 0, (size_t)M * N * sizeof(__half), s));
        return B200Q_OK;
    }
    if (w_layout == B200Q_LAYOUT_KN && use_prefill_kernel(M, N, K) && prefill_kn_supported(a, wq, N, K)) {
        return launch_prefill_kn(a, wq, scale, c, M, N, K, s, nullptr, nullptr, false, 0, workspace, workspace_bytes);
    }
    if (w_layout == B200Q_LAYOUT_NK && use_prefill_kernel(M, N, K) && prefill_nk_supported(a, wq, N, K)) {
        return launch_prefill_kn(a, wq, scale, c, M, N, K, s, nullptr, nullptr, true, 0, workspace, workspace_bytes);
    }
    if (w_layout == B200Q_LAYOUT_KN && decode_kn_supported(a, wq, N, K)) {
        return launch_decode_kn(a, wq, scale, c, M, N, K, 0, K, true, workspace, workspace_bytes, s);
    }
    if (w_layout == B200Q_LAYOUT_NK && decode_nk_supported(a, wq, N, K)) {
        return launch_decode_kn(a, wq, scale, c, M, N, K, 0, K, true, workspace, workspace_bytes, s, nullptr, nullptr, true);
    }
    return launch_generic(a, wq, scale, c, M, N, K, 0, K, w_layout, s);
}

B200Q_API int b200q_qlinear_f16_i8_fused(const void *a, const void *wq, const void *scale, void *c, int64_t M, int64_t N, int64_t K,
                                         int w_layout, const b200q_epilogue *epilogue, void *workspace, size_t workspace_bytes, void *stream) {
    using namespace b200q;
    if (epilogue == nullptr) return b200q_qlinear_f16_i8(a, wq, scale, c, M, N, K, w_layout, workspace, workspace_bytes, stream);
    int rc = check_qlinear_args("qlinear_f16_i8_fused", a, wq, scale, c, M, N, K, w_layout);
    if (rc != B200Q_OK) return rc;
    if (epilogue->activation != B200Q_ACT_NONE && epilogue->activation != B200Q_ACT_SILU_MUL) {
        return set_error(B200Q_INVALID_ARGUMENT, "qlinear_f16_i8_fused: unknown activation %d", epilogue->activation);
    }
    const bool pairs = epilogue->activation == B200Q_ACT_SILU_MUL;
    if (pairs && N % 2 != 0) return set_error(B200Q_INVALID_ARGUMENT, "qlinear_f16_i8_fused: the gate / up pairing needs an even N, got %lld", (long long)N);
    const int64_t n_out = pairs ? N / 2 : N;
    if (epilogue->residual != nullptr && epilogue->ldr < n_out) {
        return set_error(B200Q_INVALID_ARGUMENT, "qlinear_f16_i8_fused: residual rows of %lld elements are shorter than the result's %lld", (long long)epilogue->ldr, (long long)n_out);
    }
    if (M == 0 || N == 0) return B200Q_OK;
    if (w_layout != B200Q_LAYOUT_KN || K == 0 || !decode_kn_supported(a, wq, N, K)) {
        return set_error(B200Q_UNSUPPORTED, "qlinear_f16_i8_fused: the fused epilogue is served for [K, N] weights with 16-byte aligned bases and rows "
                                            "(N %% 16 == 0, K %% 8 == 0, K > 0); got layout %d N=%lld K=%lld", w_layout, (long long)N, (long long)K);
    }
    Epilogue ep;
    ep.bias = epilogue->bias;
    ep.residual = epilogue->residual;
    ep.ldr = epilogue->ldr;
    ep.act = pairs ? kActSiluMul : kActNone;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (use_prefill_kernel(M, N, K)) return launch_prefill_kn(a, wq, scale, c, M, N, K, s, nullptr, &ep, false, 0, workspace, workspace_bytes);
    return launch_decode_kn(a, wq, scale, c, M, N, K, 0, K, true, workspace, workspace_bytes, s, nullptr, &ep);
}

B200Q_API int b200q_qlinear_f16_i8_to_peers(const void *a, const void *wq, const void *scale, void *const *dst, int n_dst,
                                            int64_t ldc, int64_t col_offset, int64_t M, int64_t N, int64_t K, void *workspace,
                                            size_t workspace_bytes, void *stream) {
    using namespace b200q;
    if (n_dst < 1 || n_dst > kMaxOutTargets) return set_error(B200Q_INVALID_ARGUMENT, "qlinear_f16_i8_to_peers: n_dst must be 1..%d, got %d", kMaxOutTargets, n_dst);
    if (dst == nullptr) return set_error(B200Q_INVALID_ARGUMENT, "qlinear_f16_i8_to_peers: null destination table");
    if (col_offset < 0 || ldc < col_offset + N) return set_error(B200Q_INVALID_ARGUMENT, "qlinear_f16_i8_to_peers: columns [%lld, %lld) do not fit rows of %lld elements", (long long)col_offset, (long long)(col_offset + N), (long long)ldc);
    int rc = check_qlinear_args("qlinear_f16_i8_to_peers", a, wq, scale, dst[0], M, N, K, B200Q_LAYOUT_KN);
    if (rc != B200Q_OK) return rc;
    if (M == 0 || N == 0) return B200Q_OK;
    if (K == 0) return set_error(B200Q_INVALID_ARGUMENT, "qlinear_f16_i8_to_peers: K must be positive");
    OutTargets t;
    t.count = n_dst;
    t.ldc = ldc;
    t.col0 = col_offset;
    for (int i = 0; i < n_dst; ++i) {
        if (dst[i] == nullptr) return set_error(B200Q_INVALID_ARGUMENT, "qlinear_f16_i8_to_peers: destination %d is null", i);
        t.ptr[i] = dst[i];
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (!decode_kn_supported(a, wq, N, K)) {
        return set_error(B200Q_UNSUPPORTED, "qlinear_f16_i8_to_peers: operands need 16-byte aligned bases and rows (N %% 16 == 0, K %% 8 == 0)");
    }
    if (use_prefill_kernel(M, N, K)) return launch_prefill_kn(a, wq, scale, dst[0], M, N, K, s, &t, nullptr, false, 0, workspace, workspace_bytes);
    return launch_decode_kn(a, wq, scale, dst[0], M, N, K, 0, K, true, workspace, workspace_bytes, s, &t);
}

B200Q_API int b200q_qlinear_f16_i8_to_multicast(const void *a, const void *wq, const void *scale, void *multicast_dst, int64_t ldc,
                                                int64_t col_offset, int64_t M, int64_t N, int64_t K, void *workspace, size_t workspace_bytes,
                                                void *stream) {
    using namespace b200q;
    if (multicast_dst == nullptr) return set_error(B200Q_INVALID_ARGUMENT, "qlinear_f16_i8_to_multicast: null destination");
    if (col_offset < 0 || ldc < col_offset + N) return set_error(B200Q_INVALID_ARGUMENT, "qlinear_f16_i8_to_multicast: columns [%lld, %lld) do not fit rows of %lld elements", (long long)col_offset, (long long)(col_offset + N), (long long)ldc);
    int rc = check_qlinear_args("qlinear_f16_i8_to_multicast", a, wq, scale, multicast_dst, M, N, K, B200Q_LAYOUT_KN);
    if (rc != B200Q_OK) return rc;
    if (M == 0 || N == 0) return B200Q_OK;
    if (K == 0) return set_error(B200Q_INVALID_ARGUMENT, "qlinear_f16_i8_to_multicast: K must be positive");
    if (!use_prefill_kernel(M, N, K) || !prefill_kn_supported(a, wq, N, K)) {
        return set_error(B200Q_UNSUPPORTED, "qlinear_f16_i8_to_multicast: served by the large-M kernel only (M >= %lld, 16-byte aligned operands, "
                                            "N %% 16 == 0, K %% 8 == 0); use b200q_qlinear_f16_i8_to_peers for M=%lld N=%lld K=%lld",
                         (long long)kPrefillMinM, (long long)M, (long long)N, (long long)K);
    }
    OutTargets t;
    t.ptr[0] = multicast_dst;
    t.count = 1;
    t.ldc = ldc;
    t.col0 = col_offset;
    t.multicast = 1;
    return launch_prefill_kn(a, wq, scale, multicast_dst, M, N, K, static_cast<cudaStream_t>(stream), &t, nullptr, false, 0, workspace, workspace_bytes);
}

B200Q_API int b200q_qlinear_f16_i8_parts(const void *a, const void *wq, const void *scale, void *c, int64_t M,
                                         int64_t N, int64_t K, int k_parts, void *stream) {
    using namespace b200q;
    int rc = check_qlinear_args("qlinear_f16_i8_parts", a, wq, scale, c, M, N, K, B200Q_LAYOUT_KN);
    if (rc != B200Q_OK) return rc;
    if (k_parts < 1) return set_error(B200Q_INVALID_ARGUMENT, "qlinear_f16_i8_parts: k_parts must be >= 1, got %d", k_parts);
    if (M == 0 || N == 0) return B200Q_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // Part extent of the reference's schedule: ceil(ceil(K / parts) / 8) * 8
    // (python/hidet/graph/ops/quant/matmul_f16_i8.py:165).
    const int64_t extent = round_up(ceil_div(K, k_parts), 8);
    const bool fast = decode_kn_supported(a, wq, N, K);
    for (int part = 0; part < k_parts; ++part) {
        __half *cp = static_cast<__half *>(c) + (size_t)part * M * N;
        const int64_t k_begin = (int64_t)part * extent;
        int64_t k_end = k_begin + extent;
        if (k_end > K) k_end = K;
        if (k_begin >= K) {
            B200Q_CUDA_TRY(cudaMemsetAsync(cp, 0, (size_t)M * N * sizeof(__half), s));
            continue;
        }
        // Large M: the tensor-memory kernel on the k range as a problem of its own (activation columns k_begin ..
        // of rows that stay K long, weight rows k_begin ..); small M: the streaming kernel on the range.
        const __half *a_part = static_cast<const __half *>(a) + k_begin;
        const int8_t *w_part = static_cast<const int8_t *>(wq) + (size_t)k_begin * N;
        if (fast && use_prefill_kernel(M, N, k_end - k_begin) && prefill_kn_supported(a_part, w_part, N, k_end - k_begin)) {
            rc = launch_prefill_kn(a_part, w_part, scale, cp, M, N, k_end - k_begin, s, nullptr, nullptr, false, K);
        } else {
            rc = fast ? launch_decode_kn(a, wq, scale, cp, M, N, K, k_begin, k_end, false, nullptr, 0, s)
                      : launch_generic(a, wq, scale, cp, M, N, K, k_begin, k_end, B200Q_LAYOUT_KN, s);
        }
        if (rc != B200Q_OK) return rc;
    }
    return B200Q_OK;
}

}  // extern "C"
