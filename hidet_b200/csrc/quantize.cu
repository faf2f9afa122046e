// Symmetric quantize / dequantize kernels.
//
// The arithmetic repeats, operation for operation, what the reference's generated kernels do for
// SymmetricQuantizationTask / SymmetricDeQuantizationTask (python/hidet/graph/ops/quant/symmetric.py:23-61):
//
//     x     = (0 <= w) ? w : -w
//     amax  = max over the reduced dimension of x, starting from the lowest finite value
//     scale = amax / (T)qmax
//     wq    = (Q) round(w / scale)          round = hrint for f16 / bf16, roundf for f32
//     w'    = (T) wq * scale
//
// in w's own type T, with CUDA's own operators for __half / __nv_bfloat16 (their division is an
// approximate reciprocal times the dividend, rounded once; that is part of the result).  This file
// is compiled with -ftz=true -prec-div=false, the flags the reference compiles its kernels with
// (python/hidet/backend/build.py:142-177), because they decide the f32 division.
//
// What differs from the reference is the schedule: the reference reads the weight twice from HBM
// with one thread per column walking K serially; here a thread-block cluster owns a panel of
// columns, each CTA keeps its slice of the panel in shared memory, partial maxima are written into
// the other CTAs' shared memory, and the slice is quantized from shared memory, so the weight
// crosses HBM once.  max is exact and order-independent, so the result does not depend on the
// schedule.
#include <cooperative_groups.h>
#include <cfloat>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace b200q {
namespace {

// ---------------------------------------------------------------------------------------------
// per-type arithmetic, spelled the way the reference's generated code spells it
// ---------------------------------------------------------------------------------------------
template <typename T>
struct Arith;

template <>
struct Arith<__half> {
    static __device__ __forceinline__ __half lowest() { return (__half)-65504.0f; }
    static __device__ __forceinline__ __half abs_(__half w) { return ((__half)0.0f <= w) ? w : (-w); }
    static __device__ __forceinline__ __half max_(__half a, __half b) { return __hmax(a, b); }
    static __device__ __forceinline__ __half div_(__half a, __half b) { return a / b; }
    static __device__ __forceinline__ __half qmax(int q) { return (__half)(float)q; }
    // w / scale for many w and one scale.  CUDA's __half division (cuda_fp16.hpp, __hdiv) converts both
    // operands to f32, takes rcp.approx.ftz.f32 of the divisor, multiplies, rounds to half, and redoes
    // the last steps with one correction when the result is a non-zero value below 0x008F.  The
    // reciprocal depends on the divisor only, so it is taken once per scale; every other operation is
    // the same one, in the same order, which keeps the quotient bit-identical to `w / scale`.
    struct Divisor {
        float fb;
        float rcp;
    };
    static __device__ __forceinline__ Divisor prepare(__half scale) {
        Divisor d;
        d.fb = __half2float(scale);
        asm("{rcp.approx.ftz.f32 %0, %1;\n}" : "=f"(d.rcp) : "f"(d.fb));
        return d;
    }
    static __device__ __forceinline__ __half div_prepared(__half a, const Divisor &d) {
        const float fa = __half2float(a);
        float fv = d.rcp * fa;
        __half v = __float2half(fv);
        const __half av = __habs(v);
        if (__hlt(av, __ushort_as_half((unsigned short)0x008FU)) && __hlt(__float2half(0.0f), av)) {
            const float err = __fmaf_rn(-d.fb, fv, fa);
            fv = __fmaf_rn(d.rcp, err, fv);
            v = __float2half(fv);
        }
        return v;
    }
    template <typename Q>
    static __device__ __forceinline__ Q quant(__half w, const Divisor &d) {
        return (Q)(short)(hrint(div_prepared(w, d)));
    }
    template <typename Q>
    static __device__ __forceinline__ __half dequant(Q q, __half scale) {
        return __short2half_rn((short)q) * scale;
    }
};

template <>
struct Arith<__nv_bfloat16> {
    static __device__ __forceinline__ __nv_bfloat16 lowest() { return (__nv_bfloat16)-3.4e+38f; }
    static __device__ __forceinline__ __nv_bfloat16 abs_(__nv_bfloat16 w) { return ((__nv_bfloat16)0.0f <= w) ? w : (-w); }
    static __device__ __forceinline__ __nv_bfloat16 max_(__nv_bfloat16 a, __nv_bfloat16 b) { return __hmax(a, b); }
    static __device__ __forceinline__ __nv_bfloat16 div_(__nv_bfloat16 a, __nv_bfloat16 b) { return a / b; }
    static __device__ __forceinline__ __nv_bfloat16 qmax(int q) { return (__nv_bfloat16)(float)q; }
    typedef __nv_bfloat16 Divisor;
    static __device__ __forceinline__ Divisor prepare(__nv_bfloat16 scale) { return scale; }
    template <typename Q>
    static __device__ __forceinline__ Q quant(__nv_bfloat16 w, __nv_bfloat16 scale) {
        return (Q)(hrint(w / scale));
    }
    template <typename Q>
    static __device__ __forceinline__ __nv_bfloat16 dequant(Q q, __nv_bfloat16 scale) {
        return __short2bfloat16_rn((short)q) * scale;
    }
};

template <>
struct Arith<float> {
    static __device__ __forceinline__ float lowest() { return -3.4028234663852886e+38f; }
    static __device__ __forceinline__ float abs_(float w) { return (0.0f <= w) ? w : (-w); }
    static __device__ __forceinline__ float max_(float a, float b) { return fmaxf(a, b); }
    static __device__ __forceinline__ float div_(float a, float b) { return a / b; }
    static __device__ __forceinline__ float qmax(int q) { return (float)q; }
    typedef float Divisor;
    static __device__ __forceinline__ Divisor prepare(float scale) { return scale; }
    template <typename Q>
    static __device__ __forceinline__ Q quant(float w, float scale) {
        return (Q)(roundf(w / scale));
    }
    template <typename Q>
    static __device__ __forceinline__ float dequant(Q q, float scale) {
        return ((float)q) * scale;
    }
};

template <typename Q>
struct QMax;
template <>
struct QMax<int8_t> {
    static constexpr int value = 127;
};
template <>
struct QMax<int16_t> {
    static constexpr int value = 32767;
};

// N elements of T moved as one naturally aligned vector.
template <typename T, int N>
struct alignas(sizeof(T) * N) Vec {
    T v[N];
};

template <typename T, int N>
__device__ __forceinline__ Vec<T, N> load_vec(const T *p) {
    return *reinterpret_cast<const Vec<T, N> *>(p);
}
template <typename T, int N>
__device__ __forceinline__ void store_vec(T *p, const Vec<T, N> &x) {
    *reinterpret_cast<Vec<T, N> *>(p) = x;
}

// VEC quotients -> codes.  The general form applies Arith<T>::quant element by element.
template <typename T, typename Q, int VEC, typename D>
struct QuantVec {
    // scales: one divisor per element (PER_ELEMENT) or one for all
    template <bool PER_ELEMENT>
    static __device__ __forceinline__ void run(const Vec<T, VEC> &x, const D *s, Vec<Q, VEC> &q) {
        run_n<PER_ELEMENT, VEC>(x.v, s, q.v);
    }
    template <bool PER_ELEMENT, int N>
    static __device__ __forceinline__ void run_n(const T *x, const D *s, Q *q) {
#pragma unroll
        for (int i = 0; i < N; ++i) q[i] = Arith<T>::template quant<Q>(x[i], s[PER_ELEMENT ? i : 0]);
    }
};

// f16 -> int8, eight at a time, two per instruction where the arithmetic allows it, with the same bits as the
// general form:
//   * the quotient v is f16(rcp * f32(w)) as in Arith<__half>::div_prepared; the correction step there only touches
//     non-zero quotients below 0x008F (8.5e-6), which round to zero either way, so it is left out;
//   * b = v + 1536 in f16 (1536 = 0x6600, where one ulp is 1) is v rounded to an integer, ties to even, plus 1536
//     for |v| < 512: the same integer hrint gives, and 1536 being even the same ties.  For |hrint(v)| <= 127 the
//     low mantissa byte of b is that integer's two's-complement byte, which replaces hrint and the two conversions
//     (short)(r), (int8_t)(short);
//   * b - 1536 is exact; where its magnitude is not a number <= 127 for one of the eight (|v| >= 512 lands there too,
//     and so do the NaN and infinities a zero scale produces) all eight take the general form, whose conversions
//     define the result.
template <>
struct QuantVec<__half, int8_t, 8, Arith<__half>::Divisor> {
    template <bool PER_ELEMENT>
    static __device__ __forceinline__ void run(const Vec<__half, 8> &x, const Arith<__half>::Divisor *s, Vec<int8_t, 8> &q) {
        const __half2 *x2 = reinterpret_cast<const __half2 *>(x.v);
        const __half2 magic = __floats2half2_rn(1536.0f, 1536.0f);
        __half2 b[4], far[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const Arith<__half>::Divisor &d0 = s[PER_ELEMENT ? 2 * j : 0], &d1 = s[PER_ELEMENT ? 2 * j + 1 : 0];
            const float2 f = __half22float2(x2[j]);
            b[j] = __hadd2(__floats2half2_rn(d0.rcp * f.x, d1.rcp * f.y), magic);
            far[j] = __habs2(__hsub2(b[j], magic));
        }
        // one test for the eight: the largest magnitude, a NaN if there is any
        const __half2 worst = __hmax2_nan(__hmax2_nan(far[0], far[1]), __hmax2_nan(far[2], far[3]));
        const __half2 in_range = __hle2(worst, __floats2half2_rn(127.0f, 127.0f));  // 1.0 where true; false for NaN
        if (*reinterpret_cast<const uint32_t *>(&in_range) != 0x3C003C00u) {
            QuantVec<__half, int8_t, 1, Arith<__half>::Divisor>::template run_n<PER_ELEMENT, 8>(x.v, s, q.v);
            return;
        }
        const uint32_t *bits = reinterpret_cast<const uint32_t *>(b);
        uint32_t *out = reinterpret_cast<uint32_t *>(q.v);
        out[0] = __byte_perm(bits[0], bits[1], 0x6420);  // the low byte of each half, in order
        out[1] = __byte_perm(bits[2], bits[3], 0x6420);
    }
};

// The running absmax of VEC columns, in the reference's sense: max over abs_(w), starting from lowest().
template <typename T, int VEC>
struct AbsMaxVec {
    T m[VEC];
    __device__ __forceinline__ void init() {
#pragma unroll
        for (int i = 0; i < VEC; ++i) m[i] = Arith<T>::lowest();
    }
    __device__ __forceinline__ void add(const Vec<T, VEC> &x) {
#pragma unroll
        for (int i = 0; i < VEC; ++i) m[i] = Arith<T>::max_(m[i], Arith<T>::abs_(x.v[i]));
    }
    // The maxima over this thread's values and those of the lanes `TX`, `2 TX`, ... away in its warp (TX = 32: its own).
    template <int TX>
    __device__ __forceinline__ void finish(T *out) {
#pragma unroll
        for (int off = TX; off < 32; off <<= 1) {
#pragma unroll
            for (int i = 0; i < VEC; ++i) m[i] = Arith<T>::max_(m[i], __shfl_xor_sync(0xffffffffu, m[i], off));
        }
#pragma unroll
        for (int i = 0; i < VEC; ++i) out[i] = m[i];
    }
};

// f16, two columns per instruction: the running maximum `hi` and minimum `lo` of the values themselves (__hmax2 /
// __hmin2 skip a NaN operand and order -0 below +0, exactly as the __hmax of the element-wise form does), folded
// at the end.  abs_ leaves w >= 0 (both zeros and +inf included) as it is, negates w < 0, and turns a NaN into a
// NaN, which max_ skips; so the element-wise result over a set of values is
//     max(lowest, the largest non-NaN value, -(the smallest value) if that one is below zero)
// and hi starts at lowest.  The zero cases: only -0 (and NaN) seen gives hi = lo = -0 and the result -0, as the
// element-wise form gives; one +0 makes hi = +0.  Nothing seen, or only NaN, leaves lowest.
template <>
struct AbsMaxVec<__half, 8> {
    __half2 hi[4], lo[4];
    __device__ __forceinline__ void init() {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            hi[j] = __floats2half2_rn(-65504.0f, -65504.0f);
            lo[j] = __floats2half2_rn(65504.0f, 65504.0f);
        }
    }
    __device__ __forceinline__ void add(const Vec<__half, 8> &x) {
        const __half2 *x2 = reinterpret_cast<const __half2 *>(x.v);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            hi[j] = __hmax2(hi[j], x2[j]);
            lo[j] = __hmin2(lo[j], x2[j]);
        }
    }
    template <int TX>
    __device__ __forceinline__ void finish(__half *out) {
        const __half2 zero = __floats2half2_rn(0.0f, 0.0f);
        const uint32_t lowest2 = 0xFBFFFBFFu;  // (-65504, -65504)
        __half2 m[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            // per half: lo < 0 ? max(hi, -lo) : hi, written as max(hi, lo < 0 ? -lo : lowest); hi >= lowest always
            const uint32_t below = __hlt2_mask(lo[j], zero);
            const __half2 neg = __hneg2(lo[j]);
            const uint32_t cand = (*reinterpret_cast<const uint32_t *>(&neg) & below) | (lowest2 & ~below);
            m[j] = __hmax2(hi[j], *reinterpret_cast<const __half2 *>(&cand));
        }
#pragma unroll
        for (int off = TX; off < 32; off <<= 1) {
#pragma unroll
            for (int j = 0; j < 4; ++j) m[j] = __hmax2(m[j], __shfl_xor_sync(0xffffffffu, m[j], off));
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            out[2 * j] = __low2half(m[j]);
            out[2 * j + 1] = __high2half(m[j]);
        }
    }
};

constexpr int kThreads = 256;
constexpr int kMaxCluster = 8;   // the largest portable cluster

// ---------------------------------------------------------------------------------------------
// reduce over rows (Hidet dims=0): scale[cols]
// ---------------------------------------------------------------------------------------------
// 16 bytes global -> shared without passing through registers.
__device__ __forceinline__ void copy_async_16(uint32_t dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
// All of this thread's earlier asynchronous copies have landed.
__device__ __forceinline__ void copy_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
// The two halves of a cluster barrier that publishes nothing: it only tells that every CTA of the cluster runs.
__device__ __forceinline__ void cluster_arrive_relaxed() { asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.aligned;" ::: "memory"); }

// grid = (cluster_size, panels); the CTAs of one cluster share blockIdx.y (a panel of PW = TX*VEC
// columns) and split the rows.  TX threads lie across a panel row, kThreads / TX rows make a sweep.
// cache != 0: the CTA's rows of the panel are kept in dynamic shared memory between the two phases
// (with VEC > 1 they are brought there by asynchronous 16-byte copies, all in flight at once, and the
// absmax is taken from shared memory); cache == 0: phase 2 reads them again from global memory.
// Each thread reads back only what it copied itself, so the copies need no barrier.
template <typename T, typename Q, int VEC, int TX>
__global__ void __launch_bounds__(kThreads) quantize_cols_kernel(const T *__restrict__ w, Q *__restrict__ wq,
                                                                 T *__restrict__ scale, int64_t rows, int64_t cols,
                                                                 int64_t rows_per_cta, int cache) {
    constexpr int TY = kThreads / TX;          // rows per sweep
    constexpr int PW = TX * VEC;               // panel width in elements
    constexpr int WARPS = kThreads / 32;
    constexpr bool ASYNC = VEC > 1;            // a vector is 16 bytes whenever VEC > 1
    using A = Arith<T>;

    extern __shared__ __align__(16) unsigned char smem_raw[];
    __shared__ __align__(16) T red[WARPS][PW];
    __shared__ T recv[kMaxCluster][PW];        // recv[r]: the partial maxima of the cluster's CTA r
    __shared__ __align__(16) typename A::Divisor div_s[PW];

    T *tile = reinterpret_cast<T *>(smem_raw);

    cg::cluster_group cluster = cg::this_cluster();
    cluster_arrive_relaxed();                  // waited for before the first store into a peer's shared memory
    const int tx = threadIdx.x % TX;
    const int ty = threadIdx.x / TX;
    const int64_t col = (int64_t)blockIdx.y * PW + (int64_t)tx * VEC;
    const bool col_ok = col < cols;            // cols % VEC == 0 whenever VEC > 1
    const int64_t row0 = (int64_t)blockIdx.x * rows_per_cta;
    int64_t nrows64 = rows - row0;
    if (nrows64 > rows_per_cta) nrows64 = rows_per_cta;
    if (nrows64 < 0) nrows64 = 0;
    const int nrows = (int)nrows64;            // at most rows_per_cta, which the launcher keeps below 2^31
    const int64_t sweep = (int64_t)TY * cols;  // elements between two rows of this thread

    // ---- phase 1: partial absmax of this CTA's rows ----
    AbsMaxVec<T, VEC> acc;
    acc.init();
    if (col_ok) {
        const T *src = w + (row0 + ty) * cols + col;
        if (ASYNC && cache) {
            uint32_t dst = smem_u32(tile) + (uint32_t)((ty * PW + tx * VEC) * sizeof(T));
            for (int r = ty; r < nrows; r += TY, src += sweep, dst += (uint32_t)(TY * PW * sizeof(T))) copy_async_16(dst, src);
            copy_async_wait_all();
            const T *t = tile + ty * PW + tx * VEC;
#pragma unroll 4
            for (int r = ty; r < nrows; r += TY, t += TY * PW) acc.add(load_vec<T, VEC>(t));
        } else {
            T *t = tile + ty * PW + tx * VEC;
#pragma unroll 4
            for (int r = ty; r < nrows; r += TY, src += sweep, t += TY * PW) {
                Vec<T, VEC> x = load_vec<T, VEC>(src);
                if (cache) store_vec<T, VEC>(t, x);
                acc.add(x);
            }
        }
    }
    T m[VEC];
    acc.template finish<TX>(m);                // over the rows of a sweep that this warp holds: lanes tx, tx + TX, ...
    if ((threadIdx.x & 31) < TX) {
#pragma unroll
        for (int i = 0; i < VEC; ++i) red[threadIdx.x >> 5][tx * VEC + i] = m[i];
    }
    __syncthreads();
    // ---- exchange inside the cluster: every CTA writes its partial maxima into all the others' shared memory ----
    cluster_wait();                            // every CTA of the cluster has started
    const unsigned int n_cta = cluster.num_blocks();
    if (threadIdx.x < PW) {
        T a = A::lowest();
#pragma unroll
        for (int j = 0; j < WARPS; ++j) a = A::max_(a, red[j][threadIdx.x]);
        const unsigned int me = cluster.block_rank();
        for (unsigned int r = 0; r < n_cta; ++r) cluster.map_shared_rank(&recv[0][0], r)[me * PW + threadIdx.x] = a;
    }
    cluster.sync();  // the stores above are visible after it; nobody reads or writes a peer's memory from here on
    // one thread per column makes its scale and divisor
    if (threadIdx.x < PW) {
        T v[kMaxCluster];
#pragma unroll
        for (int r = 0; r < kMaxCluster; ++r) v[r] = ((unsigned)r < n_cta) ? recv[r][threadIdx.x] : A::lowest();
        T a = A::lowest();
#pragma unroll
        for (int r = 0; r < kMaxCluster; ++r) a = A::max_(a, v[r]);
        const T s = A::div_(a, A::qmax(QMax<Q>::value));
        div_s[threadIdx.x] = A::prepare(s);
        const int64_t c = (int64_t)blockIdx.y * PW + threadIdx.x;
        if (blockIdx.x == 0 && c < cols) scale[c] = s;
    }
    __syncthreads();

    // ---- phase 2: quantize ----
    if (col_ok) {
        typename A::Divisor s[VEC];
#pragma unroll
        for (int i = 0; i < VEC; ++i) s[i] = div_s[tx * VEC + i];
        const T *src = w + (row0 + ty) * cols + col;
        Q *dst = wq + (row0 + ty) * cols + col;
        const T *t = tile + ty * PW + tx * VEC;
#pragma unroll 4
        for (int r = ty; r < nrows; r += TY, src += sweep, dst += sweep, t += TY * PW) {
            Vec<T, VEC> x = cache ? load_vec<T, VEC>(t) : load_vec<T, VEC>(src);
            Vec<Q, VEC> q;
            QuantVec<T, Q, VEC, typename A::Divisor>::template run<true>(x, s, q);
            store_vec<Q, VEC>(dst, q);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// reduce over columns (Hidet dims=-1): scale[rows]; one CTA per row, warp-shuffle reduction
// ---------------------------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ T warp_max(T a) {
    using A = Arith<T>;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) a = A::max_(a, __shfl_xor_sync(0xffffffffu, a, off));
    return a;
}

// REG_CHUNKS: vectors of the row each thread keeps in registers between the two phases; rows longer
// than blockDim * VEC * REG_CHUNKS read the remainder again (it is in L1/L2 by then).
template <typename T, typename Q, int VEC, int REG_CHUNKS>
__global__ void __launch_bounds__(kThreads) quantize_rows_kernel(const T *__restrict__ w, Q *__restrict__ wq,
                                                                 T *__restrict__ scale, int64_t rows, int64_t cols) {
    using A = Arith<T>;
    __shared__ T warp_part[kThreads / 32];
    __shared__ T amax_s;

    const int64_t row = blockIdx.x;
    const T *src = w + row * cols;
    Q *dst = wq + row * cols;
    const int64_t nvec = cols / VEC;  // cols % VEC == 0 whenever VEC > 1
    const int64_t stride = blockDim.x;

    Vec<T, VEC> keep[REG_CHUNKS];
    AbsMaxVec<T, VEC> acc;
    acc.init();
#pragma unroll
    for (int j = 0; j < REG_CHUNKS; ++j) {
        const int64_t i = threadIdx.x + j * stride;
        if (i < nvec) {
            keep[j] = load_vec<T, VEC>(src + i * VEC);
            acc.add(keep[j]);
        }
    }
    for (int64_t i = threadIdx.x + REG_CHUNKS * stride; i < nvec; i += stride) acc.add(load_vec<T, VEC>(src + i * VEC));
    T each[VEC];
    acc.template finish<32>(each);
    T m = A::lowest();
#pragma unroll
    for (int e = 0; e < VEC; ++e) m = A::max_(m, each[e]);
    m = warp_max<T>(m);
    if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x < 32) {
        const int nwarps = (blockDim.x + 31) >> 5;
        T a = (threadIdx.x < nwarps) ? warp_part[threadIdx.x] : A::lowest();
        a = warp_max<T>(a);
        if (threadIdx.x == 0) amax_s = a;
    }
    __syncthreads();
    const T s_val = A::div_(amax_s, A::qmax(QMax<Q>::value));
    if (threadIdx.x == 0) scale[row] = s_val;
    const typename A::Divisor s = A::prepare(s_val);

#pragma unroll
    for (int j = 0; j < REG_CHUNKS; ++j) {
        const int64_t i = threadIdx.x + j * stride;
        if (i < nvec) {
            Vec<Q, VEC> q;
            QuantVec<T, Q, VEC, typename A::Divisor>::template run<false>(keep[j], &s, q);
            store_vec<Q, VEC>(dst + i * VEC, q);
        }
    }
    for (int64_t i = threadIdx.x + REG_CHUNKS * stride; i < nvec; i += stride) {
        Vec<T, VEC> x = load_vec<T, VEC>(src + i * VEC);
        Vec<Q, VEC> q;
        QuantVec<T, Q, VEC, typename A::Divisor>::template run<false>(x, &s, q);
        store_vec<Q, VEC>(dst + i * VEC, q);
    }
}

// A warp per row, for rows of at most kWarpRowBytes: the row is brought into the warp's part of shared memory by
// asynchronous 16-byte copies, all in flight at once, and both phases read it from there.  A lane reads back only
// what it copied itself and the warps of a CTA share nothing, so there is no barrier; the reduction is one round
// of warp shuffles instead of a CTA's.  grid = ceil(rows / W) CTAs of W <= kRowWarps warps (fewer for long rows, so
// that a CTA's rows stay near kRowCtaBytes and several CTAs fit an SM).
constexpr int kRowWarps = 4;
constexpr size_t kWarpRowBytes = 48 * 1024;
constexpr size_t kRowCtaBytes = 48 * 1024;

template <typename T, typename Q, int VEC>
__global__ void __launch_bounds__(kRowWarps * 32) quantize_rows_warp_kernel(const T *__restrict__ w, Q *__restrict__ wq,
                                                                            T *__restrict__ scale, int64_t rows, int64_t cols) {
    using A = Arith<T>;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + warp;
    if (row >= rows) return;
    const int nvec = (int)(cols / VEC);       // cols % VEC == 0, and a row is at most kWarpRowBytes
    T *mine = reinterpret_cast<T *>(smem_raw) + (size_t)warp * cols;
    const T *src = w + row * cols;
    Q *dst = wq + row * cols;

    {
        const uint32_t base = smem_u32(mine);
        for (int i = lane; i < nvec; i += 32) copy_async_16(base + (uint32_t)(i * VEC * sizeof(T)), src + (size_t)i * VEC);
        copy_async_wait_all();
    }
    AbsMaxVec<T, VEC> acc;
    acc.init();
#pragma unroll 4
    for (int i = lane; i < nvec; i += 32) acc.add(load_vec<T, VEC>(mine + (size_t)i * VEC));
    T each[VEC];
    acc.template finish<32>(each);
    T m = A::lowest();
#pragma unroll
    for (int e = 0; e < VEC; ++e) m = A::max_(m, each[e]);
    m = warp_max<T>(m);
    const T s_val = A::div_(m, A::qmax(QMax<Q>::value));
    if (lane == 0) scale[row] = s_val;
    const typename A::Divisor s = A::prepare(s_val);
#pragma unroll 4
    for (int i = lane; i < nvec; i += 32) {
        Vec<Q, VEC> q;
        QuantVec<T, Q, VEC, typename A::Divisor>::template run<false>(load_vec<T, VEC>(mine + (size_t)i * VEC), &s, q);
        store_vec<Q, VEC>(dst + (size_t)i * VEC, q);
    }
}

// ---------------------------------------------------------------------------------------------
// dequantize: a CTA covers kDqRows rows of kDqVecs vectors; a thread keeps its column and walks the rows
// ---------------------------------------------------------------------------------------------
// VEC codes -> values.  The general form applies Arith<T>::dequant element by element.
template <typename T, typename Q, int VEC>
struct DequantVec {
    template <bool PER_ELEMENT>
    static __device__ __forceinline__ void run(const Vec<Q, VEC> &q, const T *s, Vec<T, VEC> &out) {
#pragma unroll
        for (int e = 0; e < VEC; ++e) out.v[e] = Arith<T>::template dequant<Q>(q.v[e], s[PER_ELEMENT ? e : 0]);
    }
};

// int8 -> f16, two per instruction with the same bits: 0x6400 | (b ^ 0x80) is the f16 number 1024 + (b + 128), and
// subtracting 1152 leaves b exactly, the value __short2half_rn gives; the product with the scale is then the same
// single f16 multiplication.
template <>
struct DequantVec<__half, int8_t, 8> {
    template <bool PER_ELEMENT>
    static __device__ __forceinline__ void run(const Vec<int8_t, 8> &q, const __half *s, Vec<__half, 8> &out) {
        const uint32_t *qw = reinterpret_cast<const uint32_t *>(q.v);
        const __half2 *s2 = reinterpret_cast<const __half2 *>(s);
        const __half2 s_all = PER_ELEMENT ? __half2() : __half2half2(s[0]);
        __half2 *o2 = reinterpret_cast<__half2 *>(out.v);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            // bytes (2j, 2j+1) of the vector into the low bytes of the two halves, 0x64 above each, sign bit flipped
            const uint32_t placed = __byte_perm(qw[j >> 1], 0x64646464u, (j & 1) ? 0x4342 : 0x4140) ^ 0x00800080u;
            uint32_t exact;
            asm("sub.f16x2 %0, %1, %2;" : "=r"(exact) : "r"(placed), "r"(0x64806480u));
            o2[j] = __hmul2(*reinterpret_cast<const __half2 *>(&exact), PER_ELEMENT ? s2[j] : s_all);
        }
    }
};

constexpr int kDqVecs = 32;                       // vectors across a CTA (one warp wide)
constexpr int kDqSweep = kThreads / kDqVecs;      // rows per sweep
constexpr int kDqRows = 4 * kDqSweep;             // rows per CTA

// grid = (row blocks, column blocks)
template <typename T, typename Q, int VEC>
__global__ void __launch_bounds__(kThreads) dequantize_kernel(const Q *__restrict__ wq, const T *__restrict__ scale,
                                                              T *__restrict__ w, int64_t rows, int64_t cols,
                                                              int reduce_dim) {
    const int64_t c = ((int64_t)blockIdx.y * kDqVecs + (threadIdx.x % kDqVecs)) * VEC;
    if (c >= cols) return;                        // cols % VEC == 0 whenever VEC > 1
    const int64_t r0 = (int64_t)blockIdx.x * kDqRows + threadIdx.x / kDqVecs;
    const Q *src = wq + r0 * cols + c;
    T *dst = w + r0 * cols + c;
    const int64_t sweep = (int64_t)kDqSweep * cols;
    if (reduce_dim == 0) {
        const Vec<T, VEC> s = load_vec<T, VEC>(scale + c);
#pragma unroll
        for (int i = 0; i < kDqRows / kDqSweep; ++i) {
            if (r0 + i * kDqSweep < rows) {
                Vec<T, VEC> out;
                DequantVec<T, Q, VEC>::template run<true>(load_vec<Q, VEC>(src + i * sweep), s.v, out);
                store_vec<T, VEC>(dst + i * sweep, out);
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < kDqRows / kDqSweep; ++i) {
            if (r0 + i * kDqSweep < rows) {
                const T s = scale[r0 + i * kDqSweep];
                Vec<T, VEC> out;
                DequantVec<T, Q, VEC>::template run<false>(load_vec<Q, VEC>(src + i * sweep), &s, out);
                store_vec<T, VEC>(dst + i * sweep, out);
            }
        }
    }
}

bool aligned(const void *p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

// ---------------------------------------------------------------------------------------------
// embedding lookup in a row-quantized table: out[i, :] = T(table[idx[i], :]) * scale[idx[i]]
// ---------------------------------------------------------------------------------------------
// The tiling of dequantize_kernel over the looked-up rows: a thread keeps its column and walks kDqRows / kDqSweep
// indices.  The arithmetic is that of dequantize_kernel with reduce_dim = 1, so a lookup equals the row of the
// dequantized table bit for bit.  An index outside [0, vocab) (after adding vocab to a negative one) yields a row of
// zeros and sets bit 30 of the device status word.  grid = (index blocks, column blocks)
template <typename T, typename Q, typename I, int VEC>
__global__ void __launch_bounds__(kThreads) embedding_dequant_kernel(const Q *__restrict__ table, const T *__restrict__ scale,
                                                                     const I *__restrict__ idx, T *__restrict__ out, int64_t vocab,
                                                                     int64_t dim, int64_t n_idx, unsigned int *status) {
    const int64_t c = ((int64_t)blockIdx.y * kDqVecs + (threadIdx.x % kDqVecs)) * VEC;
    if (c >= dim) return;                         // dim % VEC == 0 whenever VEC > 1
    const int64_t r0 = (int64_t)blockIdx.x * kDqRows + threadIdx.x / kDqVecs;
#pragma unroll
    for (int i = 0; i < kDqRows / kDqSweep; ++i) {
        const int64_t r = r0 + i * kDqSweep;
        if (r >= n_idx) break;
        int64_t row = (int64_t)idx[r];
        if (row < 0) row += vocab;
        Vec<T, VEC> o;
        if (row < 0 || row >= vocab) {
#pragma unroll
            for (int e = 0; e < VEC; ++e) o.v[e] = (T)0.0f;
            if (c == 0 && status != nullptr) atomicOr(status, 0x40000000u);
        } else {
            const T s = scale[row];
            DequantVec<T, Q, VEC>::template run<false>(load_vec<Q, VEC>(table + row * dim + c), &s, o);
        }
        store_vec<T, VEC>(out + r * dim + c, o);
    }
}

// Largest dynamic shared memory a quantize_cols CTA may ask for (the static arrays need a little).
constexpr size_t kMaxTileBytes = 200 * 1024;

// Threads across a panel row when a thread moves a 16-byte vector: 4 make a panel of 64 bytes per row (32 f16
// columns), so that a [4096, 4096] weight gives 1024 CTAs of 32 KB, several to an SM and more than one wave.
constexpr int kPanelThreads = 4;

template <typename T, typename Q, int VEC, int TX>
int launch_quantize_cols(const T *w, Q *wq, T *scale, int64_t rows, int64_t cols, cudaStream_t stream) {
    constexpr int TY = kThreads / TX;
    constexpr int PW = TX * VEC;
    const int64_t panels = ceil_div(cols, PW);
    if (panels > 65535) return set_error(B200Q_UNSUPPORTED, "symmetric_quantize: %lld columns exceed the grid limit", (long long)cols);

    // Split the rows over the largest portable cluster that still leaves every CTA a full sweep,
    // and keep the slice in shared memory when it fits.
    int cluster = kMaxCluster;
    while (cluster > 1 && ceil_div(rows, cluster) < TY) cluster >>= 1;
    const int64_t rows_per_cta = ceil_div(rows, cluster);
    size_t tile_bytes = (size_t)rows_per_cta * PW * sizeof(T);
    int cache = 1;
    if (tile_bytes > kMaxTileBytes) {
        cache = 0;
        tile_bytes = 0;
    }
    auto kernel = quantize_cols_kernel<T, Q, VEC, TX>;
    if (tile_bytes > 48 * 1024) {
        B200Q_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMaxTileBytes));
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)cluster, (unsigned)panels, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = tile_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)cluster;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    B200Q_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, w, wq, scale, rows, cols, rows_per_cta, cache));
    return B200Q_OK;
}

template <typename T, typename Q, int VEC>
int launch_quantize_rows(const T *w, Q *wq, T *scale, int64_t rows, int64_t cols, cudaStream_t stream) {
    if (rows > 2147483647LL) return set_error(B200Q_UNSUPPORTED, "symmetric_quantize: %lld rows exceed the grid limit", (long long)rows);
    if (VEC > 1 && (size_t)cols * sizeof(T) <= kWarpRowBytes) {
        const size_t row_bytes = (size_t)cols * sizeof(T);
        int warps = (int)(kRowCtaBytes / row_bytes);
        warps = warps < 1 ? 1 : (warps > kRowWarps ? kRowWarps : warps);
        const size_t smem = warps * row_bytes;  // at most kRowCtaBytes, the default limit for dynamic shared memory
        auto kernel = quantize_rows_warp_kernel<T, Q, VEC>;
        kernel<<<(unsigned)ceil_div(rows, warps), warps * 32, smem, stream>>>(w, wq, scale, rows, cols);
        B200Q_CHECK_LAUNCH("quantize_rows_warp_kernel");
        return B200Q_OK;
    }
    const int64_t nvec = cols / VEC;
    int threads = (int)round_up(nvec < 32 ? 32 : nvec, 32);
    if (threads > kThreads) threads = kThreads;
    quantize_rows_kernel<T, Q, VEC, 4><<<(unsigned)rows, threads, 0, stream>>>(w, wq, scale, rows, cols);
    B200Q_CHECK_LAUNCH("quantize_rows_kernel");
    return B200Q_OK;
}

template <typename T, typename Q>
int quantize_typed(const void *w_, void *wq_, void *scale_, int64_t rows, int64_t cols, int reduce_dim, cudaStream_t stream) {
    const T *w = static_cast<const T *>(w_);
    Q *wq = static_cast<Q *>(wq_);
    T *scale = static_cast<T *>(scale_);
    constexpr int VEC = 16 / sizeof(T);
    const bool vec_ok = (cols % VEC == 0) && aligned(w, 16) && aligned(wq, VEC * sizeof(Q));
    if (reduce_dim == 0) {
        return vec_ok ? launch_quantize_cols<T, Q, VEC, kPanelThreads>(w, wq, scale, rows, cols, stream)
                      : launch_quantize_cols<T, Q, 1, 32>(w, wq, scale, rows, cols, stream);
    }
    return vec_ok ? launch_quantize_rows<T, Q, VEC>(w, wq, scale, rows, cols, stream)
                  : launch_quantize_rows<T, Q, 1>(w, wq, scale, rows, cols, stream);
}

template <typename T, typename Q>
int dequantize_typed(const void *wq_, const void *scale_, void *w_, int64_t rows, int64_t cols, int reduce_dim,
                     cudaStream_t stream) {
    const Q *wq = static_cast<const Q *>(wq_);
    const T *scale = static_cast<const T *>(scale_);
    T *w = static_cast<T *>(w_);
    constexpr int VEC = 16 / sizeof(T);  // 16-byte scale / output vectors; input vector is VEC * sizeof(Q)
    const bool vec_ok = (cols % VEC == 0) && aligned(w, 16) && aligned(wq, VEC * sizeof(Q)) && aligned(scale, 16);
    if (rows == 0 || cols == 0) return B200Q_OK;
    const int64_t row_blocks = ceil_div(rows, kDqRows);
    const int64_t col_blocks = ceil_div(vec_ok ? cols / VEC : cols, kDqVecs);
    if (row_blocks > 2147483647LL || col_blocks > 65535) {
        return set_error(B200Q_UNSUPPORTED, "symmetric_dequantize: [%lld, %lld] exceeds the grid limit", (long long)rows, (long long)cols);
    }
    const dim3 grid((unsigned)row_blocks, (unsigned)col_blocks, 1);
    if (vec_ok) {
        dequantize_kernel<T, Q, VEC><<<grid, kThreads, 0, stream>>>(wq, scale, w, rows, cols, reduce_dim);
    } else {
        dequantize_kernel<T, Q, 1><<<grid, kThreads, 0, stream>>>(wq, scale, w, rows, cols, reduce_dim);
    }
    B200Q_CHECK_LAUNCH("dequantize_kernel");
    return B200Q_OK;
}

template <typename T, typename Q, typename I>
int embedding_typed(const void *table_, const void *scale_, const void *idx_, void *out_, int64_t vocab, int64_t dim, int64_t n_idx,
                    cudaStream_t stream) {
    const Q *table = static_cast<const Q *>(table_);
    const T *scale = static_cast<const T *>(scale_);
    const I *idx = static_cast<const I *>(idx_);
    T *out = static_cast<T *>(out_);
    constexpr int VEC = 16 / sizeof(T);
    const bool vec_ok = (dim % VEC == 0) && aligned(out, 16) && aligned(table, VEC * sizeof(Q));
    if (n_idx == 0 || dim == 0) return B200Q_OK;
    const int64_t row_blocks = ceil_div(n_idx, kDqRows);
    const int64_t col_blocks = ceil_div(vec_ok ? dim / VEC : dim, kDqVecs);
    if (row_blocks > 2147483647LL || col_blocks > 65535) {
        return set_error(B200Q_UNSUPPORTED, "embedding_dequantize: %lld indices of %lld values exceed the grid limit", (long long)n_idx, (long long)dim);
    }
    const dim3 grid((unsigned)row_blocks, (unsigned)col_blocks, 1);
    unsigned int *status = device_status_word();
    if (vec_ok) {
        embedding_dequant_kernel<T, Q, I, VEC><<<grid, kThreads, 0, stream>>>(table, scale, idx, out, vocab, dim, n_idx, status);
    } else {
        embedding_dequant_kernel<T, Q, I, 1><<<grid, kThreads, 0, stream>>>(table, scale, idx, out, vocab, dim, n_idx, status);
    }
    B200Q_CHECK_LAUNCH("embedding_dequant_kernel");
    return B200Q_OK;
}

int check_common(const char *op, const void *a, const void *b, const void *c, int64_t rows, int64_t cols, int f_type,
                 int q_type, int reduce_dim) {
    if (rows < 0 || cols < 0) return set_error(B200Q_INVALID_ARGUMENT, "%s: negative shape [%lld, %lld]", op, (long long)rows, (long long)cols);
    if (f_type < B200Q_F16 || f_type > B200Q_F32) return set_error(B200Q_INVALID_ARGUMENT, "%s: unknown float type %d", op, f_type);
    if (q_type < B200Q_I8 || q_type > B200Q_I16) return set_error(B200Q_INVALID_ARGUMENT, "%s: unknown quantized type %d", op, q_type);
    if (reduce_dim != 0 && reduce_dim != 1) return set_error(B200Q_INVALID_ARGUMENT, "%s: reduce_dim must be 0 or 1, got %d", op, reduce_dim);
    if (rows > 0 && cols > 0 && (a == nullptr || b == nullptr || c == nullptr)) return set_error(B200Q_INVALID_ARGUMENT, "%s: null pointer argument", op);
    return B200Q_OK;
}

}  // namespace
}  // namespace b200q

extern "C" {

B200Q_API int b200q_symmetric_quantize(const void *w, void *wq, void *scale, int64_t rows, int64_t cols, int w_type,
                                       int q_type, int reduce_dim, void *stream) {
    using namespace b200q;
    int rc = check_common("symmetric_quantize", w, wq, scale, rows, cols, w_type, q_type, reduce_dim);
    if (rc != B200Q_OK) return rc;
    // An empty reduced dimension has no maximum; the reference cannot build that task either.
    if (rows == 0 || cols == 0) {
        if ((reduce_dim == 0 ? cols : rows) == 0) return B200Q_OK;  // no outputs at all
        return set_error(B200Q_INVALID_ARGUMENT, "symmetric_quantize: empty reduction over shape [%lld, %lld]", (long long)rows, (long long)cols);
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
#define B200Q_DISPATCH_Q(T)                                                                                    \
    (q_type == B200Q_I8 ? quantize_typed<T, int8_t>(w, wq, scale, rows, cols, reduce_dim, s)                   \
                        : quantize_typed<T, int16_t>(w, wq, scale, rows, cols, reduce_dim, s))
    switch (w_type) {
        case B200Q_F16: return B200Q_DISPATCH_Q(__half);
        case B200Q_BF16: return B200Q_DISPATCH_Q(__nv_bfloat16);
        default: return B200Q_DISPATCH_Q(float);
    }
#undef B200Q_DISPATCH_Q
}

B200Q_API int b200q_symmetric_dequantize(const void *wq, const void *scale, void *w, int64_t rows, int64_t cols,
                                         int scale_type, int q_type, int reduce_dim, void *stream) {
    using namespace b200q;
    int rc = check_common("symmetric_dequantize", wq, scale, w, rows, cols, scale_type, q_type, reduce_dim);
    if (rc != B200Q_OK) return rc;
    if (rows == 0 || cols == 0) return B200Q_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
#define B200Q_DISPATCH_DQ(T)                                                                                   \
    (q_type == B200Q_I8 ? dequantize_typed<T, int8_t>(wq, scale, w, rows, cols, reduce_dim, s)                 \
                        : dequantize_typed<T, int16_t>(wq, scale, w, rows, cols, reduce_dim, s))
    switch (scale_type) {
        case B200Q_F16: return B200Q_DISPATCH_DQ(__half);
        case B200Q_BF16: return B200Q_DISPATCH_DQ(__nv_bfloat16);
        default: return B200Q_DISPATCH_DQ(float);
    }
#undef B200Q_DISPATCH_DQ
}

B200Q_API int b200q_embedding_dequantize(const void *table, const void *scale, const void *indices, void *out, int64_t vocab,
                                         int64_t dim, int64_t n_indices, int scale_type, int q_type, int index_bytes, void *stream) {
    using namespace b200q;
    int rc = check_common("embedding_dequantize", table, scale, table, vocab, dim, scale_type, q_type, 1);
    if (rc != B200Q_OK) return rc;
    if (n_indices < 0) return set_error(B200Q_INVALID_ARGUMENT, "embedding_dequantize: negative index count %lld", (long long)n_indices);
    if (index_bytes != 4 && index_bytes != 8) return set_error(B200Q_INVALID_ARGUMENT, "embedding_dequantize: indices must be int32 or int64 (4 or 8 bytes), got %d", index_bytes);
    if (n_indices == 0 || dim == 0) return B200Q_OK;
    if (indices == nullptr || out == nullptr || table == nullptr || scale == nullptr) return set_error(B200Q_INVALID_ARGUMENT, "embedding_dequantize: null pointer argument");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
#define B200Q_DISPATCH_E2(T, Q)                                                                                    \
    (index_bytes == 8 ? embedding_typed<T, Q, int64_t>(table, scale, indices, out, vocab, dim, n_indices, s)      \
                      : embedding_typed<T, Q, int32_t>(table, scale, indices, out, vocab, dim, n_indices, s))
#define B200Q_DISPATCH_E(T) (q_type == B200Q_I8 ? B200Q_DISPATCH_E2(T, int8_t) : B200Q_DISPATCH_E2(T, int16_t))
    switch (scale_type) {
        case B200Q_F16: return B200Q_DISPATCH_E(__half);
        case B200Q_BF16: return B200Q_DISPATCH_E(__nv_bfloat16);
        default: return B200Q_DISPATCH_E(float);
    }
#undef B200Q_DISPATCH_E
#undef B200Q_DISPATCH_E2
}

}  // extern "C"
