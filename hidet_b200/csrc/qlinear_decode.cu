// Small-M (decode) f16 x int8 quantized linear for weights in the reference's [K, N] layout.
//
// The op is bound by streaming the int8 weight from HBM once, so the kernel is built around that
// stream.  A producer warp keeps a ring of TMA tile loads in flight: 64 k-rows x 128 columns of int8,
// 128B-swizzled, and copies the matching 16 x 64 f16 slice of the activations beside each with
// cp.async.  Four consumer warps own 32 columns each, so no sum ever crosses a warp.  A consumer
// fetches its slice with transposing matrix loads (four consecutive k of one column per register),
// turns the bytes into exact f16 pairs in registers and feeds warp-level m16n8k16 tensor-core MMAs
// with fp32 accumulators; the weight is the MMA's 16-row operand and the activations its 8-column operand, so up to 8 activation rows
// cost one MMA per 16 x 16 weight block and up to 16 rows two (rows beyond M are zero-filled).
//
// K is split across CTAs to fill the machine.  Up to 8 splits of one output tile form a thread-block
// cluster: every CTA sends its partial tile into the shared memory of the CTA that owns those columns
// with asynchronous remote stores that count bytes on an mbarrier of the owner (no cluster barrier
// round trip); the owner waits for the byte count, adds the partials in rank order, applies the
// per-column scale and rounds to f16 once.  More splits than a cluster holds go through a
// caller-provided fp32 workspace, where the last CTA of a tile to arrive does the same.  Either way
// the order of every sum is fixed, so results are the same on every run.
//
// The kernel is launched as a programmatic dependent of the kernel before it in the stream: weight
// tiles and scales do not depend on that kernel, so they are requested before waiting for it, and the
// kernel after this one is allowed to start once the main loop is over.  (Letting it start earlier was
// measured and is slower: its weight requests then queue in front of this kernel's own.)
//
// Replaces the generated mma.sync kernel of python/hidet/graph/ops/quant/matmul_f16_i8.py:136-485
// (f16 accumulation, 64x128 tiles, no split-K by default) for M <= 16, and serves larger M by
// tiling M over blockIdx.z.
#include <atomic>

#include "common.cuh"
#include "qlinear.h"

namespace b200q {
namespace decode {

constexpr int BN = 128;                      // columns per CTA
constexpr int BK = 64;                       // k rows per pipeline stage
constexpr int BM = 16;                       // activation rows per CTA
constexpr int STAGES = 4;
constexpr int CONSUMER_WARPS = 4;            // each owns BN / 4 = 32 columns
constexpr int THREADS = 32 * (CONSUMER_WARPS + 1);
constexpr int W_STAGE_BYTES = BK * BN;       // 8192
constexpr int A_STAGE_BYTES = BM * BK * 2;   // 2048
constexpr int PIPE_BYTES = STAGES * (W_STAGE_BYTES + A_STAGE_BYTES);
constexpr int RECV_COLS = 168;               // most columns the slices of a cluster cover together (7 ranks x 24 columns)
constexpr int RECV_BYTES = BM * RECV_COLS * 4; // partial tiles sent by the CTAs of the cluster: [rank][row][cols_per] fp32
constexpr int STAGING_ROW = 36;              // floats per row of a warp's 32-column staging block (padded: conflict-free)
constexpr int SMEM_BYTES = PIPE_BYTES + RECV_BYTES + 1024;  // + alignment slack
static_assert(CONSUMER_WARPS * BM * STAGING_ROW * 4 <= STAGES * W_STAGE_BYTES, "the staging blocks reuse the weight ring");
constexpr int kCtasPerSm = 4;                // resident CTAs per SM the plan aims at
constexpr int64_t kMaxCounters = 65536;      // arrival counters at the head of the workspace
constexpr int kMaxCluster = 8;               // largest cluster of the plan (8 is the portable limit; the reduction reads up to eight partials)

__device__ __forceinline__ uint2 lds64(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.b32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}

// Two 16 x 16 byte tiles, transposed on the way to registers.  Lanes 0-15 give the addresses of the 16
// rows (16 bytes each) of the first tile, lanes 16-31 those of the second.  With a tile stored as
// [k][column], lane (g = lane / 4, t = lane % 4) receives, for tile i, in r[2i] the bytes
// (k = 4t .. 4t+3, column g) and in r[2i+1] the bytes (k = 4t .. 4t+3, column g + 8): four consecutive
// k of one column per register, the packing an MMA operand wants.
__device__ __forceinline__ void ldmatrix_x2_trans_b8(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m16n16.x2.trans.shared.b8 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}

// Four signed bytes (b0 .. b3) -> f16 pairs (b0, b1) and (b2, b3), exactly.  b ^ 0x80 = b + 128 as an
// unsigned byte u; the half with bits 0x6400 | u is 1024 + u; subtracting 1152 leaves b.
__device__ __forceinline__ void cvt_s8x4_to_f16_pairs(uint32_t v, uint32_t &p01, uint32_t &p23) {
    const uint32_t u = v ^ 0x80808080u;
    const uint32_t e01 = __byte_perm(u, 0x64646464u, 0x4140);  // u0 0x64 u1 0x64
    const uint32_t e23 = __byte_perm(u, 0x64646464u, 0x4342);  // u2 0x64 u3 0x64
    const uint32_t bias = 0x64806480u;                          // f16x2 (1152, 1152)
    asm("sub.f16x2 %0, %1, %2;" : "=r"(p01) : "r"(e01), "r"(bias));
    asm("sub.f16x2 %0, %1, %2;" : "=r"(p23) : "r"(e23), "r"(bias));
}

// Four 8 x 16 byte tiles as they lie.  Lanes 8i .. 8i+7 give the addresses of the rows of tile i; lane
// (g = lane / 4, t = lane % 4) receives in r[i] the bytes 4t .. 4t+3 of row g of tile i.  With a weight
// stored as [column][k] that is again four consecutive k of one column per register.
__device__ __forceinline__ void ldmatrix_x4_b16(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}

// D[16 x 8] += A[16 x 16] * B[16 x 8]: A row-major (here: 16 weight columns x 16 k), B column-major
// (here: 16 k x 8 activation rows).
__device__ __forceinline__ void mma_m16n8k16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                             uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// ---- cluster primitives (a kernel launched without a cluster is a cluster of one) ----
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t cluster_nctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_arrive_release() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait_acquire() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
// Address of the same shared-memory location in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_rank(uint32_t local_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
    return r;
}
// Asynchronous stores into the shared memory of a CTA of the cluster; each adds its size to the transaction
// count of an mbarrier of that CTA once the data is there.
__device__ __forceinline__ void st_async_f32(uint32_t addr, float v, uint32_t bar) {
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.b32 [%0], %1, [%2];" ::"r"(addr), "r"(__float_as_uint(v)), "r"(bar) : "memory");
}
__device__ __forceinline__ void st_async_v4f32(uint32_t addr, float4 v, uint32_t bar) {
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.b32 [%0], {%1, %2, %3, %4}, [%5];" ::"r"(addr),
                 "r"(__float_as_uint(v.x)), "r"(__float_as_uint(v.y)), "r"(__float_as_uint(v.z)), "r"(__float_as_uint(v.w)), "r"(bar)
                 : "memory");
}
// Bounded wait on an mbarrier phase that remote CTAs complete (acquire at cluster scope).
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < kSpinLimit; ++i) {
        uint32_t ok;
        asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2, %3;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t"
            "}\n"
            : "=r"(ok)
            : "r"(bar), "r"(parity), "r"(kWaitHintNs)
            : "memory");
        if (ok) return true;
    }
    return false;
}
__device__ __forceinline__ float4 lds128f(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ void sts32f(uint32_t addr, float v) { asm volatile("st.shared.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory"); }

// 16 bytes global -> shared without passing through registers; src_bytes = 0 writes zeros instead.
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void *src, uint32_t src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
// The barrier gets one arrival from this thread once all its earlier cp.async copies have landed.
__device__ __forceinline__ void cp_async_arrive(uint32_t bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}

constexpr int kModeDirect = 0;  // one CTA per output tile
constexpr int kModeSplit = 1;   // `splits` CTAs per tile: clusters of `cluster` CTAs, `groups` clusters per tile

// One result element to every destination.
__device__ __forceinline__ void store_out(const OutTargets &o, int row, int col, __half v) {
    const size_t off = (size_t)row * o.ldc + o.col0 + col;
#pragma unroll 1
    for (int i = 0; i < o.count; ++i) static_cast<__half *>(o.ptr[i])[off] = v;
}

__device__ __forceinline__ float silu(float x) { return x / (1.0f + __expf(-x)); }

// The end of every path: y is the scaled fp32 sum of column nn (in range or not), row `row`.  Adds the bias,
// applies the activation (the value of the partner column nn ^ 1 sits in lane ^ partner_xor; every lane
// of the calling warp that is active takes part), adds the residual, rounds once and stores.
__device__ __forceinline__ void finish(const OutTargets &o, const Epilogue &ep, int row, int nn, int n_limit, bool valid, float y, int partner_xor) {
    if (valid && ep.bias != nullptr) y += __half2float(__ldg(static_cast<const __half *>(ep.bias) + nn));
    int col = nn;
    if (ep.act == kActSiluMul) {
        const float other = __shfl_xor_sync(__activemask(), y, partner_xor);
        if (nn & 1) valid = false;  // the even column of a pair finishes both
        y = silu(y) * other;
        col = nn >> 1;
    }
    if (!valid || nn >= n_limit) return;
    if (ep.residual != nullptr) y += __half2float(__ldg(static_cast<const __half *>(ep.residual) + (size_t)row * ep.ldr + col));
    store_out(o, row, col, __float2half_rn(y));
}

struct Params {
    const __half *a;          // activations [M, lda]
    int64_t lda;
    const __half *scale;
    OutTargets out;
    Epilogue ep;
    float *partial;           // [groups][M][N] fp32 in the workspace, used when groups > 1
    unsigned int *counters;   // [m_tiles * n_tiles * cluster] in the workspace, zero on entry, zero on exit
    unsigned int *status;
    int M, N;
    int k_begin, k_end;       // the k range this launch sums over (k_end is also the tensor maps' K extent)
    int iters_per_split;      // BK-sized k steps per split
    int groups;               // clusters per output tile (splits = groups * cluster size)
    int cols_per;             // columns of a tile each CTA of the cluster owns in the reduction (a multiple of 8)
    int mode;                 // kModeDirect or kModeSplit
};

// MT: 8-row blocks of activations per CTA (1: up to 8 rows, 2: up to 16).
// NK: the weight is [N, K] with K contiguous (the layout torch.nn.Linear keeps) instead of the reference's
//     [K, N]: a stage is then 128 weight rows of 64 k-bytes (64-byte swizzle) and the fragments come from
//     plain matrix loads; everything else is shared.
template <int MT, bool NK>
__global__ void __launch_bounds__(THREADS) qlinear_decode_kn_kernel(const __grid_constant__ CUtensorMap map_w, const Params p) {
    extern __shared__ unsigned char smem_dyn[];
    __shared__ __align__(8) uint64_t full_bar[STAGES];
    __shared__ __align__(8) uint64_t empty_bar[STAGES];
    __shared__ __align__(8) uint64_t recv_bar;  // the partial tiles of this CTA's columns have landed
    __shared__ unsigned int is_last;

    // 128B-swizzled TMA tiles need 1024-byte aligned bases.
    const uint32_t smem_base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
    unsigned char *smem_gen = smem_dyn + (smem_base - smem_u32(smem_dyn));
    const uint32_t w_base = smem_base;
    const uint32_t a_base = smem_base + STAGES * W_STAGE_BYTES;
    const uint32_t recv_base = smem_base + PIPE_BYTES;
    float *recv = reinterpret_cast<float *>(smem_gen + PIPE_BYTES);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int g = lane >> 2;  // MMA group id
    const int t = lane & 3;   // thread in group
    const int n0 = blockIdx.x * BN;
    const int split = blockIdx.y;
    const int m0 = blockIdx.z * BM;
    const int total_iters = (p.k_end - p.k_begin + BK - 1) / BK;
    const int it_begin = split * p.iters_per_split;
    int n_iters = total_iters - it_begin;
    if (n_iters > p.iters_per_split) n_iters = p.iters_per_split;
    if (n_iters < 0) n_iters = 0;
    int rows = p.M - m0;
    if (rows > BM) rows = BM;
    const uint32_t nranks = cluster_nctarank();
    const uint32_t rank = cluster_ctarank();
    const int cols_per = p.cols_per;
    // Columns of the tile this CTA sums in the reduction: [own_first, own_first + own_cols).
    const int own_first = (int)rank * cols_per;
    int own_cols = BN - own_first;
    if (own_cols > cols_per) own_cols = cols_per;
    if (own_cols < 0) own_cols = 0;
    if (threadIdx.x == 0) {
#pragma unroll
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1 + 32);  // the weight tile (TMA bytes) and the producer warp's 32 lanes, each when its activation copies have landed
            mbar_init(smem_u32(&empty_bar[s]), CONSUMER_WARPS);
        }
        mbar_init(smem_u32(&recv_bar), 1);
        mbar_fence_init();
        // Bytes the cluster will send here: every rank, `rows` rows of this CTA's columns.
        if (p.mode == kModeSplit && own_cols > 0) mbar_expect_tx(smem_u32(&recv_bar), nranks * (uint32_t)rows * (uint32_t)own_cols * 4u);
    }
    __syncthreads();
    // First half of a cluster barrier whose second half sits in front of the first remote store: by
    // then every CTA of the cluster has started and set up its barriers, which remote access requires.
    cluster_arrive_release();

    // The result element this thread finishes in the split-K reduction, and its scale.  Like the weight, the
    // scale does not depend on the kernel before this one, so it is fetched now, far from where it is used.
    float sc_own = 0.0f;
    if (p.mode == kModeSplit) {
        const int cc = (int)threadIdx.x % cols_per;
        if (cc < own_cols && n0 + own_first + cc < p.N) sc_own = __half2float(__ldg(p.scale + n0 + own_first + cc));
    }

    // acc[j][mt][.]: 16 x 8 tile j of this warp's 32 columns, activation rows 8 * mt ... 8 * mt + 7.
    // Element (column 16 j + 8 h + g, row 8 mt + 2t + e) is acc[j][mt][2h + e].
    float acc[2][MT][4];
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) acc[j][mt][0] = acc[j][mt][1] = acc[j][mt][2] = acc[j][mt][3] = 0.0f;

    if (warp == CONSUMER_WARPS) {
        // ---------------- producer warp ----------------
        // Lane 0 drives the TMA loads of the weight tiles.  The activation slices (8 MT rows x 64 k of f16 per stage,
        // 128-byte rows, 16-byte chunk c of row r at chunk c ^ (r & 7), the layout a 128B-swizzled TMA tile would have)
        // are copied by all 32 lanes with cp.async: they are a few hundred bytes that sit in L2, and on the load/store
        // path they do not wait in the TMA queue behind weight tiles that are still on their way from HBM.
        uint32_t dst_off[2 * MT];
        const __half *src_row[2 * MT];
        int kc[2 * MT];
#pragma unroll
        for (int q = 0; q < 2 * MT; ++q) {
            const int chunk = lane + 32 * q;  // 8 chunks per row
            const int r = chunk >> 3, c = chunk & 7;
            dst_off[q] = r * 128 + ((c ^ (r & 7)) << 4);
            src_row[q] = m0 + r < p.M ? p.a + (size_t)(m0 + r) * p.lda : nullptr;  // rows beyond M are zero-filled
            kc[q] = 8 * c;
        }
        auto copy_activations = [&](int s, int k0) {
#pragma unroll
            for (int q = 0; q < 2 * MT; ++q) {
                const int k = k0 + kc[q];
                const bool in = src_row[q] != nullptr && k < p.k_end;  // k_end is a multiple of 8 or the row's end: a chunk is in or out as a whole
                cp_async_16(a_base + s * A_STAGE_BYTES + dst_off[q], in ? static_cast<const void *>(src_row[q] + k) : static_cast<const void *>(p.a), in ? 16u : 0u);
            }
            cp_async_arrive(smem_u32(&full_bar[s]));
        };
        const int prologue = n_iters < STAGES ? n_iters : STAGES;
        uint64_t stream_policy = 0;
        if (lane == 0) {
            tma_prefetch_desc(&map_w);
            stream_policy = l2_policy_evict_first();  // the weight is read once
            // The weight does not depend on the kernel before this one in the stream; the activations
            // may.  Ask for the first weight tiles, then wait for that kernel, then ask for activations.
            for (int it = 0; it < prologue; ++it) {
                const uint32_t bar = smem_u32(&full_bar[it]);
                mbar_expect_tx(bar, W_STAGE_BYTES);
                tma_load_2d_hint(w_base + it * W_STAGE_BYTES, &map_w, NK ? p.k_begin + (it_begin + it) * BK : n0, NK ? n0 : p.k_begin + (it_begin + it) * BK, bar, stream_policy);
            }
        }
        __syncwarp();
        pdl_wait();
        for (int it = 0; it < prologue; ++it) copy_activations(it, p.k_begin + (it_begin + it) * BK);
        for (int it = STAGES; it < n_iters; ++it) {
            const int s = it % STAGES;
            if (!mbar_wait(smem_u32(&empty_bar[s]), ((it / STAGES) - 1) & 1)) {
                if (lane == 0) report_timeout(p.status, kKernelDecode, 1);
                break;
            }
            const int k0 = p.k_begin + (it_begin + it) * BK;
            if (lane == 0) {
                const uint32_t bar = smem_u32(&full_bar[s]);
                mbar_expect_tx(bar, W_STAGE_BYTES);
                tma_load_2d_hint(w_base + s * W_STAGE_BYTES, &map_w, NK ? k0 : n0, NK ? n0 : k0, bar, stream_policy);
            }
            copy_activations(s, k0);
        }
    } else {
        // ---------------- consumers ----------------
        pdl_wait();
        // Weights: one transposing matrix load per 16 k-rows brings this warp's 32 columns (16-byte
        // chunks 2 warp and 2 warp + 1 of each row).  Lane l addresses row (l & 15) of chunk
        // 2 warp + (l >> 4); under the 128B swizzle chunk c of row r sits at chunk c ^ (r & 7).
        const uint32_t off_w = (lane & 15) * 128 + (((2 * warp + (lane >> 4)) ^ (lane & 7)) << 4);
        // [N, K] weights: lane l addresses row 32 warp + 8 (l / 8 % 2) + l % 8 (+ 16 j) of the stage, 16-byte
        // chunk l / 16 (+ 2 per 32 k); rows are 64 bytes, chunk c of row r sits at chunk c ^ (r / 2 % 4).
        const uint32_t nk_row = 32 * warp + 8 * ((lane >> 3) & 1) + (lane & 7);
        const uint32_t nk_chunk = (uint32_t)lane >> 4;
        // Activations: row g (and g + 8, same swizzle phase), k = 16 ks + 4t .. 4t+3: bytes 8 (t & 1) of
        // chunk 2 ks + (t >> 1).
        const uint32_t off_a = g * 128 + 8 * (t & 1);
        const uint32_t a_chunk = (uint32_t)(t >> 1) ^ (uint32_t)g;  // chunk index is (2 ks) ^ a_chunk: bit 0 of 2 ks is free
        for (int it = 0; it < n_iters; ++it) {
            const int s = it % STAGES;
            if (!mbar_wait(smem_u32(&full_bar[s]), (it / STAGES) & 1)) {
                report_timeout(p.status, kKernelDecode, 2);
                break;
            }
            const uint32_t wb = w_base + s * W_STAGE_BYTES + off_w;
            const uint32_t ab = a_base + s * A_STAGE_BYTES + off_a;
            uint32_t q[4][4];
            uint2 b[4][MT];
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
                if (!NK) ldmatrix_x2_trans_b8(q[ks], wb + ks * 2048);
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) b[ks][mt] = lds64(ab + mt * 1024 + (((2 * ks) ^ a_chunk) << 4));
            }
            if (NK) {
#pragma unroll
                for (int j = 0; j < 2; ++j)
#pragma unroll
                    for (int kh = 0; kh < 2; ++kh) {
                        const uint32_t row = nk_row + 16 * j;
                        uint32_t r[4];
                        ldmatrix_x4_b16(r, w_base + s * W_STAGE_BYTES + row * 64 + (((2 * kh + nk_chunk) ^ ((row >> 1) & 3)) << 4));
                        q[2 * kh][2 * j] = r[0];
                        q[2 * kh][2 * j + 1] = r[1];
                        q[2 * kh + 1][2 * j] = r[2];
                        q[2 * kh + 1][2 * j + 1] = r[3];
                    }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&empty_bar[s]));  // the stage is in registers now
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    // tile j: MMA rows g / g + 8 are columns 32 warp + 16 j + g / + 8 + g;
                    // k slots (2t, 2t+1) and (2t+8, 2t+9) carry k = 4t, 4t+1 and 4t+2, 4t+3
                    uint32_t a0, a1, a2, a3;
                    cvt_s8x4_to_f16_pairs(q[ks][2 * j], a0, a2);
                    cvt_s8x4_to_f16_pairs(q[ks][2 * j + 1], a1, a3);
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) mma_m16n8k16(acc[j][mt], a0, a1, a2, a3, b[ks][mt].x, b[ks][mt].y);
                }
            }
        }
    }
    __syncwarp();  // the role branches above are lane-divergent; the cluster barrier below wants whole warps
    pdl_launch_dependents();  // the next kernel may start streaming its weight

    const bool consumer = warp < CONSUMER_WARPS;
    // This thread's four columns inside the tile: 32 warp + 16 j + 8 h + g.
    const int col_base = 32 * warp + g;

    if (p.mode == kModeDirect) {
        cluster_wait_acquire();
        if (consumer) {
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int nn = n0 + col_base + 16 * j + 8 * h;
                    const float sc = nn < p.N ? __half2float(p.scale[nn]) : 0.0f;
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            const int r = 8 * mt + 2 * t + e;  // columns nn and nn ^ 1 live in lanes that differ in g by one
                            finish(p.out, p.ep, m0 + r, nn, p.N, r < rows, acc[j][mt][2 * h + e] * sc, 4);
                        }
                }
        }
        return;
    }

    // ---------------- split-K ----------------
    // Level 1, inside a cluster: every CTA sends its partial tile into the shared memory of the CTA that
    // owns those columns, counted in bytes on the owner's barrier; the owner then holds the partials of all
    // ranks.  (Without a cluster the CTA is its own owner and the same code runs on local shared memory.)
    // recv layout: [rank][row][cols_per] fp32.
    cluster_wait_acquire();  // every CTA of the cluster is running
    if (consumer) {
        if (rows <= 2) {
            // One or two rows live in the lanes with t == 0: a few scalar remote stores, no staging.
            if (t == 0) {
#pragma unroll
                for (int j = 0; j < 2; ++j)
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int col = col_base + 16 * j + 8 * h;
                        const uint32_t owner = (uint32_t)(col / cols_per);
                        const int col_in = col - (int)owner * cols_per;
                        const uint32_t remote = map_to_rank(recv_base, owner);
                        const uint32_t rbar = map_to_rank(smem_u32(&recv_bar), owner);
#pragma unroll
                        for (int e = 0; e < 2; ++e)
                            if (e < rows) st_async_f32(remote + (((int)rank * BM + e) * cols_per + col_in) * 4, acc[j][0][2 * h + e], rbar);
                    }
            }
        } else {
            // More rows: transpose through a staging block in the (now idle) weight ring, then 16-byte remote stores.
            asm volatile("bar.sync 1, %0;" ::"n"(32 * CONSUMER_WARPS) : "memory");  // every consumer warp is done with the ring
            const uint32_t stage_w = w_base + warp * (BM * STAGING_ROW * 4);
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                        for (int e = 0; e < 2; ++e) sts32f(stage_w + ((8 * mt + 2 * t + e) * STAGING_ROW + 16 * j + 8 * h + g) * 4, acc[j][mt][2 * h + e]);
            __syncwarp();
            // lane -> row lane / 8 of each pass of four rows, columns 4 (lane % 8) .. + 3
            const int rr = lane >> 3, v4 = lane & 7;
            const int col = 32 * warp + 4 * v4;
            const uint32_t owner = (uint32_t)(col / cols_per);
            const int col_in = col - (int)owner * cols_per;
            const uint32_t remote = map_to_rank(recv_base, owner) + (((int)rank * BM) * cols_per + col_in) * 4;
            const uint32_t rbar = map_to_rank(smem_u32(&recv_bar), owner);
#pragma unroll
            for (int pass = 0; pass < BM / 4; ++pass) {
                const int r = pass * 4 + rr;
                if (r < rows) st_async_v4f32(remote + r * cols_per * 4, lds128f(stage_w + (r * STAGING_ROW + 4 * v4) * 4), rbar);
            }
        }
    }
    if (own_cols > 0) {
        if (!mbar_wait_cluster(smem_u32(&recv_bar), 0)) report_timeout(p.status, kKernelDecode, 4);
    }
    // Owner: one result element per thread and round; element i is row i / cols_per, column i % cols_per of
    // the slice.  The partials of the (at most eight) ranks are read together and added in rank order.
    const int col_first = n0 + own_first;  // first column this CTA owns
    auto sum_ranks = [&](int r, int cc) {
        float v[8];
#pragma unroll
        for (int jr = 0; jr < 8; ++jr) v[jr] = jr < (int)nranks ? recv[(jr * BM + r) * cols_per + cc] : 0.0f;
        float sum = v[0];
#pragma unroll
        for (int jr = 1; jr < 8; ++jr) sum += v[jr];
        return sum;
    };
    if (p.groups == 1) {
        for (int idx = threadIdx.x; idx < rows * cols_per; idx += THREADS) {
            const int r = idx / cols_per;
            const int cc = idx - r * cols_per;
            const int nn = col_first + cc;
            const bool valid = nn < p.N && cc < own_cols;  // N and own_cols are even: the two columns of a pair agree
            const float sc = idx < THREADS ? sc_own : (valid ? __half2float(p.scale[nn]) : 0.0f);
            finish(p.out, p.ep, m0 + r, nn, p.N, valid, valid ? sum_ranks(r, cc) * sc : 0.0f, 1);
        }
        return;
    }

    // Level 2, across the `groups` clusters of a tile: each owner publishes its cluster's sum in the
    // caller's workspace; the last of the `groups` owners of a column slice to arrive adds them in
    // group order and finishes.
    const int group = (int)(blockIdx.y / nranks);
    for (int idx = threadIdx.x; idx < rows * cols_per; idx += THREADS) {
        const int r = idx / cols_per;
        const int cc = idx - r * cols_per;
        const int nn = col_first + cc;
        if (nn < p.N && cc < own_cols) __stcg(&p.partial[((size_t)group * p.M + (m0 + r)) * p.N + nn], sum_ranks(r, cc));
    }
    __threadfence();
    __syncthreads();
    const unsigned int slot = (blockIdx.z * gridDim.x + blockIdx.x) * nranks + rank;
    if (threadIdx.x == 0) {
        const unsigned int prev = atomicAdd(&p.counters[slot], 1u);
        is_last = (prev == (unsigned int)(p.groups - 1)) ? 1u : 0u;
    }
    __syncthreads();
    if (is_last == 0) return;
    __threadfence();
    for (int idx = threadIdx.x; idx < rows * cols_per; idx += THREADS) {
        const int r = idx / cols_per;
        const int cc = idx - r * cols_per;
        const int nn = col_first + cc;
        const bool valid = nn < p.N && cc < own_cols;
        float v = 0.0f;
        if (valid) {
#pragma unroll 4
            for (int gr = 0; gr < p.groups; ++gr) v += __ldcg(&p.partial[((size_t)gr * p.M + (m0 + r)) * p.N + nn]);
            v *= idx < THREADS ? sc_own : __half2float(p.scale[nn]);
        }
        finish(p.out, p.ep, m0 + r, nn, p.N, valid, v, 1);
    }
    if (threadIdx.x == 0) p.counters[slot] = 0;  // leave the workspace ready for the next call
}

}  // namespace decode

// Split plan shared by the workspace query and the launch.
DecodePlan plan_decode(int64_t M, int64_t N, int64_t K) {
    using namespace decode;
    DecodePlan pl;
    pl.n_tiles = (int)ceil_div(N, BN);
    pl.m_tiles = (int)ceil_div(M, BM);
    const int k_iters = (int)ceil_div(K, BK);
    int sms = sm_count();
    if (sms <= 0) sms = 148;
    const int64_t target = (int64_t)sms * kCtasPerSm;
    const int64_t tiles = (int64_t)pl.n_tiles * pl.m_tiles;
    // CTAs per tile that fill the machine once, each with at least eight 64-row steps of work.
    int64_t splits = tiles > 0 ? target / tiles : 1;
    const int max_splits = k_iters / 8 > 0 ? k_iters / 8 : 1;
    if (splits > max_splits) splits = max_splits;
    if (splits > 64) splits = 64;
    if (splits < 1) splits = 1;
    // The splits of a tile form clusters of up to eight CTAs (partials meet in distributed shared
    // memory); more splits than a cluster holds become several full clusters per tile that meet in the
    // workspace.
    int c = (int)(splits < kMaxCluster ? splits : kMaxCluster);
    int groups = (int)(splits / c);
    if (groups < 1 || tiles * c > kMaxCounters) groups = 1;
    // Clusters that meet in the workspace pay three dependent trips through L2 at the end of the launch (publish,
    // count, read back), about 3 us more than partials that meet in distributed shared memory.  That is worth it only
    // when one cluster per tile would leave most of the machine idle.
    if (groups > 1 && tiles * c * 2 >= sms) groups = 1;
    pl.cluster = c;
    pl.groups = groups;
    pl.splits = c * groups;  // the grid holds whole clusters; a split may get fewer steps than others, or none
    pl.iters_per_split = (int)ceil_div(k_iters, pl.splits);
    // The counter region has one fixed size, so that counters never land on bytes an earlier call of
    // another shape used for partial sums: the region stays all-zero between calls.
    pl.counter_bytes = groups > 1 ? (size_t)kMaxCounters * 4 : 0;
    pl.partial_bytes = groups > 1 ? (size_t)groups * M * N * 4 : 0;
    return pl;
}

bool decode_kn_supported(const void *a, const void *wq, int64_t N, int64_t K) {
    return (N % 16 == 0) && (K % 8 == 0) && ((reinterpret_cast<uintptr_t>(a) & 15u) == 0) &&
           ((reinterpret_cast<uintptr_t>(wq) & 15u) == 0);
}

bool decode_nk_supported(const void *a, const void *wq, int64_t N, int64_t K) {
    (void)N;
    return (K % 16 == 0) && ((reinterpret_cast<uintptr_t>(a) & 15u) == 0) && ((reinterpret_cast<uintptr_t>(wq) & 15u) == 0);
}

int launch_decode_kn(const void *a, const void *wq, const void *scale, void *c, int64_t M, int64_t N, int64_t K,
                     int64_t k_begin, int64_t k_end, bool allow_split, void *workspace, size_t workspace_bytes,
                     cudaStream_t stream, const OutTargets *targets, const Epilogue *epilogue, bool weight_nk) {
    using namespace decode;
    DecodePlan pl = plan_decode(M, N, k_end - k_begin);
    if (!allow_split) {
        pl.iters_per_split = (int)ceil_div(k_end - k_begin, BK);
        pl.splits = 1;
        pl.cluster = 1;
        pl.groups = 1;
        pl.partial_bytes = 0;
        pl.counter_bytes = 0;
    }
    if (pl.partial_bytes > 0 && (workspace == nullptr || workspace_bytes < pl.counter_bytes + pl.partial_bytes)) {
        return set_error(B200Q_WORKSPACE_TOO_SMALL, "qlinear: workspace of %zu bytes given, %zu needed for M=%lld N=%lld K=%lld",
                         workspace_bytes, pl.counter_bytes + pl.partial_bytes, (long long)M, (long long)N, (long long)K);
    }
    if (pl.m_tiles > 65535 || pl.splits > 65535) return set_error(B200Q_UNSUPPORTED, "qlinear: M=%lld is too large for the small-M kernel", (long long)M);

    CUtensorMap map_w;
    int rc = weight_nk ? make_tensor_map_2d(&map_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, wq, (uint64_t)k_end, (uint64_t)N, (uint64_t)K, BK, BN,
                                            CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B)
                       : make_tensor_map_2d(&map_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, wq, (uint64_t)N, (uint64_t)k_end, (uint64_t)N, BN, BK,
                                            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
    if (rc != B200Q_OK) return rc;

    Params p;
    p.a = static_cast<const __half *>(a);
    p.lda = K;
    p.scale = static_cast<const __half *>(scale);
    if (targets != nullptr) {
        p.out = *targets;
    } else {
        p.out.ptr[0] = c;
        p.out.count = 1;
        p.out.ldc = (epilogue != nullptr && epilogue->act == kActSiluMul) ? N / 2 : N;
        p.out.col0 = 0;
    }
    if (epilogue != nullptr) p.ep = *epilogue;
    p.counters = static_cast<unsigned int *>(workspace);
    p.partial = pl.partial_bytes > 0 ? reinterpret_cast<float *>(static_cast<unsigned char *>(workspace) + pl.counter_bytes) : nullptr;
    p.status = device_status_word();
    p.M = (int)M;
    p.N = (int)N;
    p.k_begin = (int)k_begin;
    p.k_end = (int)k_end;
    p.iters_per_split = pl.iters_per_split;
    p.groups = pl.groups;
    p.cols_per = (int)round_up(ceil_div(BN, pl.cluster), 8);
    p.mode = pl.splits == 1 ? kModeDirect : kModeSplit;

    const bool one_block = M - (int64_t)(pl.m_tiles - 1) * BM <= 8 && pl.m_tiles == 1;
    auto kernel = weight_nk ? (one_block ? qlinear_decode_kn_kernel<1, true> : qlinear_decode_kn_kernel<2, true>)
                            : (one_block ? qlinear_decode_kn_kernel<1, false> : qlinear_decode_kn_kernel<2, false>);
    static std::atomic<bool> attr_set[64];  // per device, zero-initialised; a repeated set by a racing thread is harmless
    int dev = 0;
    B200Q_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !attr_set[dev].load(std::memory_order_acquire)) {
        const void *all[4] = {reinterpret_cast<const void *>(qlinear_decode_kn_kernel<1, false>), reinterpret_cast<const void *>(qlinear_decode_kn_kernel<2, false>),
                              reinterpret_cast<const void *>(qlinear_decode_kn_kernel<1, true>), reinterpret_cast<const void *>(qlinear_decode_kn_kernel<2, true>)};
        for (const void *f : all) {
            B200Q_CUDA_TRY(cudaFuncSetAttribute(f, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
            B200Q_CUDA_TRY(cudaFuncSetAttribute(f, cudaFuncAttributeNonPortableClusterSizeAllowed, 1));
        }
        if (dev >= 0 && dev < 64) attr_set[dev].store(true, std::memory_order_release);
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)pl.n_tiles, (unsigned)pl.splits, (unsigned)pl.m_tiles);
    cfg.blockDim = dim3(THREADS, 1, 1);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attrs[2];
    attrs[0].id = cudaLaunchAttributeClusterDimension;
    attrs[0].val.clusterDim.x = 1;
    attrs[0].val.clusterDim.y = (unsigned)pl.cluster;
    attrs[0].val.clusterDim.z = 1;
    attrs[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attrs;
    cfg.numAttrs = 2;
    B200Q_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, map_w, p));
    return B200Q_OK;
}

}  // namespace b200q
