// Sub-byte weights: 4-bit unsigned codes with per-group scales and zero points (w4a16), the format of the
// reference's CuTe test programs (tests/cute_kernel/quantized_linear.py:494-517, tests/cute_kernel/test_quant_linear.py:36-85):
//
//     c[M, N] = a[M, K] x w[K, N],   w[k, n] = scale[k / G, n] * (q[k, n] - zeros[k / G, n])     (zeros optional)
//
// with a, scale, zeros in f16 and q a u4 matrix [K, N] packed as the reference packs sub-byte types: element i of
// a row sits in bits 4 (i % 2) .. 4 (i % 2) + 3 of byte i / 2 (python/hidet/transforms/lower_integer_subbyte.py:103-113).
// The weight is taken in that plain row-major form; the reference's tests first permute it into a layout private to
// their kernel (preprocess_weight), which has no meaning outside that kernel.
//
// The op is bound by streaming q (half a byte per weight) once.  A thread owns eight adjacent columns (one 32-bit
// word per k row; a warp reads 128 contiguous bytes per row) and a slice of k.  Inside a group the scale and the zero
// point of a column are constant, so the inner loop multiplies activations with the bare codes and keeps the sum of
// the activations beside it; at the end of the group
//     out[m, n] += scale[n] * (sum_k a[m, k] q[k, n] - zeros[n] * sum_k a[m, k]),
// all in fp32 (the codes are exact in fp32; the reference multiplies every weight by its scale in f16 first and
// accumulates the products, tests/cute_kernel/quantized_linear.py:1044-1047: same value up to rounding).  The k slices
// of a CTA meet in shared memory; the CTAs that split K further write fp32 partial sums to the caller's workspace,
// and a second kernel adds them in slice order and rounds to f16 once: the same result on every run.
#include "common.cuh"

namespace b200q {
namespace u4 {

constexpr int COLS_PER_THREAD = 8;   // one 32-bit word of packed codes
constexpr int WORDS_X = 32;          // threads along N: a warp covers 256 columns
constexpr int K_SLICES = 8;          // warps of a CTA, each on its own k rows
constexpr int THREADS = WORDS_X * K_SLICES;
// The head of a workspace is where the int8 kernels keep their arrival counters (all-zero between calls); this op
// leaves it alone, so one workspace can serve both.
constexpr size_t kReservedHead = (size_t)65536 * 4;

struct Params {
    const __half *a;        // [M, K]
    const uint32_t *q;      // [K, N / 8] words
    const __half *scale;    // [K / G, N]
    const __half *zeros;    // [K / G, N] or null
    float *partial;         // [splits][M, N] fp32
    int M, N, K, G;
    int k_per_split;        // a multiple of G
};

// Codes of one word as exact floats: 0x4B000000 | code is 8388608 + code.
__device__ __forceinline__ void unpack8(uint32_t w, float (&v)[8]) {
#pragma unroll
    for (int c = 0; c < 8; ++c) v[c] = __uint_as_float(((w >> (4 * c)) & 0xFu) | 0x4B000000u) - 8388608.0f;
}

// MT: activation rows per pass (1, 2 or 4: the smallest that covers M, so that a single row costs a single row's
// multiplications).  The k loop is taken 4 to 16 rows at a time with all loads issued first: a thread has only a few
// dozen rows, and one load per iteration would leave it waiting for memory most of the time.
template <int MT>
__global__ void __launch_bounds__(THREADS) qlinear_u4_partial_kernel(const Params p) {
    __shared__ float red[K_SLICES][MT][WORDS_X * COLS_PER_THREAD + 8];
    const int word = blockIdx.x * WORDS_X + threadIdx.x;  // which group of eight columns
    const int n0 = word * COLS_PER_THREAD;
    const int slice = threadIdx.y;
    const int split = blockIdx.y;
    const int k_begin = split * p.k_per_split;
    const int k_end = min(p.K, k_begin + p.k_per_split);
    const int words_per_row = p.N / COLS_PER_THREAD;
    const bool in = n0 < p.N;
    float *out = p.partial + (size_t)split * p.M * p.N;
    constexpr int UNROLL = MT == 1 ? 16 : (MT == 2 ? 8 : 4);  // rows whose loads are in flight together

    for (int m0 = 0; m0 < p.M; m0 += MT) {
        float acc[MT][8];
#pragma unroll
        for (int m = 0; m < MT; ++m)
#pragma unroll
            for (int c = 0; c < 8; ++c) acc[m][c] = 0.0f;
        if (in) {
            const __half *arow[MT];
#pragma unroll
            for (int m = 0; m < MT; ++m) arow[m] = p.a + (size_t)min(m0 + m, p.M - 1) * p.K;  // rows beyond M repeat the last one and are not stored
            for (int g0 = k_begin; g0 < k_end; g0 += p.G) {
                float gs[MT][8], asum[MT];
#pragma unroll
                for (int m = 0; m < MT; ++m) {
                    asum[m] = 0.0f;
#pragma unroll
                    for (int c = 0; c < 8; ++c) gs[m][c] = 0.0f;
                }
                const int g_end = min(k_end, g0 + p.G);
                for (int kb = g0 + slice; kb < g_end; kb += UNROLL * K_SLICES) {
                    uint32_t w[UNROLL];
                    float av[UNROLL][MT];
#pragma unroll
                    for (int u = 0; u < UNROLL; ++u) {
                        const int k = kb + u * K_SLICES;
                        const bool ok = k < g_end;
                        w[u] = ok ? __ldg(p.q + (size_t)k * words_per_row + word) : 0u;
#pragma unroll
                        for (int m = 0; m < MT; ++m) av[u][m] = ok ? __half2float(__ldg(arow[m] + k)) : 0.0f;
                    }
#pragma unroll
                    for (int u = 0; u < UNROLL; ++u) {
                        float v[8];
                        unpack8(w[u], v);
#pragma unroll
                        for (int m = 0; m < MT; ++m) {
                            asum[m] += av[u][m];
#pragma unroll
                            for (int c = 0; c < 8; ++c) gs[m][c] = fmaf(av[u][m], v[c], gs[m][c]);
                        }
                    }
                }
                const size_t grow = (size_t)(g0 / p.G) * p.N + n0;
                const uint4 sraw = __ldg(reinterpret_cast<const uint4 *>(p.scale + grow));
                const __half *sh = reinterpret_cast<const __half *>(&sraw);
                uint4 zraw = make_uint4(0, 0, 0, 0);
                if (p.zeros != nullptr) zraw = __ldg(reinterpret_cast<const uint4 *>(p.zeros + grow));
                const __half *zh = reinterpret_cast<const __half *>(&zraw);
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const float s = __half2float(sh[c]), z = __half2float(zh[c]);
#pragma unroll
                    for (int m = 0; m < MT; ++m) acc[m][c] = fmaf(s, gs[m][c] - z * asum[m], acc[m][c]);
                }
            }
        }
        // the k slices of the CTA meet in shared memory, slice order
#pragma unroll
        for (int m = 0; m < MT; ++m)
#pragma unroll
            for (int c = 0; c < 8; ++c) red[slice][m][threadIdx.x * COLS_PER_THREAD + c] = acc[m][c];
        __syncthreads();
        for (int idx = threadIdx.y * WORDS_X + threadIdx.x; idx < MT * WORDS_X * COLS_PER_THREAD; idx += THREADS) {
            const int m = idx / (WORDS_X * COLS_PER_THREAD);
            const int col = idx - m * (WORDS_X * COLS_PER_THREAD);
            const int n = blockIdx.x * WORDS_X * COLS_PER_THREAD + col;
            if (m0 + m < p.M && n < p.N) {
                float s = 0.0f;
#pragma unroll
                for (int sl = 0; sl < K_SLICES; ++sl) s += red[sl][m][col];
                out[(size_t)(m0 + m) * p.N + n] = s;
            }
        }
        __syncthreads();
    }
}

__global__ void qlinear_u4_reduce_kernel(const float *partial, __half *c, int64_t mn, int splits) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= mn) return;
    float s = 0.0f;
    for (int sp = 0; sp < splits; ++sp) s += partial[(size_t)sp * mn + i];
    c[i] = __float2half_rn(s);
}

// f16 (integral values) -> u4 codes, two per byte; C conversion to int, low four bits kept.
__global__ void u4_pack_kernel(const __half *w, uint8_t *out, int64_t bytes) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= bytes) return;
    const __half2 v = reinterpret_cast<const __half2 *>(w)[i];
    const int lo = (int)__low2float(v), hi = (int)__high2float(v);
    out[i] = (uint8_t)((lo & 15) | ((hi & 15) << 4));
}

__global__ void u4_unpack_kernel(const uint8_t *packed, __half *out, int64_t bytes) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= bytes) return;
    const uint8_t b = packed[i];
    reinterpret_cast<__half2 *>(out)[i] = __floats2half2_rn((float)(b & 15), (float)(b >> 4));
}

struct Plan {
    int splits;
    int k_per_split;
};

Plan plan(int64_t M, int64_t N, int64_t K, int64_t G) {
    (void)M;
    int sms = sm_count();
    if (sms <= 0) sms = 148;
    const int64_t col_blocks = ceil_div(N, (int64_t)WORDS_X * COLS_PER_THREAD);
    const int64_t groups = ceil_div(K, G);
    int64_t splits = ceil_div((int64_t)4 * sms, col_blocks);  // four CTAs per SM: the loads of many rows in flight
    if (splits > groups) splits = groups;
    if (splits < 1) splits = 1;
    Plan pl;
    pl.k_per_split = (int)(ceil_div(groups, splits) * G);
    pl.splits = (int)ceil_div(K, pl.k_per_split);
    return pl;
}

}  // namespace u4
}  // namespace b200q

extern "C" {

B200Q_API size_t b200q_qlinear_f16_u4_workspace_bytes(int64_t M, int64_t N, int64_t K, int64_t group_size) {
    using namespace b200q;
    if (M <= 0 || N <= 0 || K <= 0 || group_size <= 0) return 0;
    return u4::kReservedHead + (size_t)u4::plan(M, N, K, group_size).splits * M * N * sizeof(float);
}

B200Q_API int b200q_qlinear_f16_u4(const void *a, const void *q, const void *scale, const void *zeros, void *c, int64_t M, int64_t N, int64_t K,
                                   int64_t group_size, void *workspace, size_t workspace_bytes, void *stream) {
    using namespace b200q;
    if (M < 0 || N < 0 || K < 0) return set_error(B200Q_INVALID_ARGUMENT, "qlinear_f16_u4: negative size M=%lld N=%lld K=%lld", (long long)M, (long long)N, (long long)K);
    if (group_size <= 0 || K % group_size != 0) {
        return set_error(B200Q_INVALID_ARGUMENT, "qlinear_f16_u4: K=%lld is not a multiple of the group size %lld", (long long)K, (long long)group_size);
    }
    if (N % 8 != 0) return set_error(B200Q_UNSUPPORTED, "qlinear_f16_u4: N=%lld is not a multiple of 8 (whole 32-bit words of codes per row)", (long long)N);
    if (M > 2147483647LL || N > 2147483647LL || K > 2147483647LL) return set_error(B200Q_UNSUPPORTED, "qlinear_f16_u4: sizes beyond 2^31-1 are not supported");
    if (M == 0 || N == 0) return B200Q_OK;
    if (c == nullptr) return set_error(B200Q_INVALID_ARGUMENT, "qlinear_f16_u4: null output pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (K == 0) {
        B200Q_CUDA_TRY(cudaMemsetAsync(c, 0, (size_t)M * N * sizeof(__half), s));
        return B200Q_OK;
    }
    if (a == nullptr || q == nullptr || scale == nullptr) return set_error(B200Q_INVALID_ARGUMENT, "qlinear_f16_u4: null input pointer");
    if ((reinterpret_cast<uintptr_t>(q) & 3u) != 0 || (reinterpret_cast<uintptr_t>(scale) & 15u) != 0 || (reinterpret_cast<uintptr_t>(zeros) & 15u) != 0) {
        return set_error(B200Q_UNSUPPORTED, "qlinear_f16_u4: codes need a 4-byte aligned base, scales and zero points 16-byte aligned bases");
    }
    const u4::Plan pl = u4::plan(M, N, K, group_size);
    const size_t need = u4::kReservedHead + (size_t)pl.splits * M * N * sizeof(float);
    if (workspace == nullptr || workspace_bytes < need) {
        return set_error(B200Q_WORKSPACE_TOO_SMALL, "qlinear_f16_u4: workspace of %zu bytes given, %zu needed for M=%lld N=%lld K=%lld", workspace_bytes, need,
                         (long long)M, (long long)N, (long long)K);
    }
    u4::Params p;
    p.a = static_cast<const __half *>(a);
    p.q = static_cast<const uint32_t *>(q);
    p.scale = static_cast<const __half *>(scale);
    p.zeros = static_cast<const __half *>(zeros);
    p.partial = reinterpret_cast<float *>(static_cast<unsigned char *>(workspace) + u4::kReservedHead);
    p.M = (int)M;
    p.N = (int)N;
    p.K = (int)K;
    p.G = (int)group_size;
    p.k_per_split = pl.k_per_split;
    const dim3 grid((unsigned)ceil_div(N, (int64_t)u4::WORDS_X * u4::COLS_PER_THREAD), (unsigned)pl.splits, 1);
    const dim3 block(u4::WORDS_X, u4::K_SLICES, 1);
    if (M == 1) {
        u4::qlinear_u4_partial_kernel<1><<<grid, block, 0, s>>>(p);
    } else if (M == 2) {
        u4::qlinear_u4_partial_kernel<2><<<grid, block, 0, s>>>(p);
    } else {
        u4::qlinear_u4_partial_kernel<4><<<grid, block, 0, s>>>(p);
    }
    B200Q_CHECK_LAUNCH("qlinear_u4_partial_kernel");
    const int64_t mn = M * N;
    u4::qlinear_u4_reduce_kernel<<<(unsigned)ceil_div(mn, 256), 256, 0, s>>>(p.partial, static_cast<__half *>(c), mn, pl.splits);
    B200Q_CHECK_LAUNCH("qlinear_u4_reduce_kernel");
    return B200Q_OK;
}

B200Q_API int b200q_u4_pack(const void *w, void *packed, int64_t rows, int64_t cols, void *stream) {
    using namespace b200q;
    if (rows < 0 || cols < 0 || cols % 2 != 0) return set_error(B200Q_INVALID_ARGUMENT, "u4_pack: rows=%lld cols=%lld (cols must be even)", (long long)rows, (long long)cols);
    const int64_t bytes = rows * cols / 2;
    if (bytes == 0) return B200Q_OK;
    if (w == nullptr || packed == nullptr) return set_error(B200Q_INVALID_ARGUMENT, "u4_pack: null pointer");
    u4::u4_pack_kernel<<<(unsigned)ceil_div(bytes, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const __half *>(w), static_cast<uint8_t *>(packed), bytes);
    B200Q_CHECK_LAUNCH("u4_pack_kernel");
    return B200Q_OK;
}

B200Q_API int b200q_u4_unpack(const void *packed, void *w, int64_t rows, int64_t cols, void *stream) {
    using namespace b200q;
    if (rows < 0 || cols < 0 || cols % 2 != 0) return set_error(B200Q_INVALID_ARGUMENT, "u4_unpack: rows=%lld cols=%lld (cols must be even)", (long long)rows, (long long)cols);
    const int64_t bytes = rows * cols / 2;
    if (bytes == 0) return B200Q_OK;
    if (w == nullptr || packed == nullptr) return set_error(B200Q_INVALID_ARGUMENT, "u4_unpack: null pointer");
    u4::u4_unpack_kernel<<<(unsigned)ceil_div(bytes, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const uint8_t *>(packed), static_cast<__half *>(w), bytes);
    B200Q_CHECK_LAUNCH("u4_unpack_kernel");
    return B200Q_OK;
}

}  // extern "C"
