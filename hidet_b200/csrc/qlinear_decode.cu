// Small-M (decode) f16 x int8 quantized linear for weights in the reference's [K, N] layout.
//
// The op is bound by streaming the int8 weight from HBM once, so the kernel is built around that
// stream: a producer warp keeps a ring of TMA tile loads in flight (64 k-rows x 128 columns of
// int8, 128B-swizzled, plus the matching 16 x 64 f16 slice of the activations), four consumer warps
// take 16 k-rows each, turn int8 pairs into exact f16 pairs in registers and feed warp-level
// m16n8k16 tensor-core MMAs with fp32 accumulators (M <= 16 fills one MMA row block; rows beyond M
// are zero-filled by TMA).  K is split across CTAs to fill the machine; partial sums meet in a
// caller-provided fp32 workspace and the last CTA of a column tile adds them in a fixed order,
// applies the per-column scale and rounds to f16 once.  The result is deterministic.
//
// Replaces the generated mma.sync kernel of python/hidet/graph/ops/quant/matmul_f16_i8.py:136-485
// (f16 accumulation, 64x128 tiles, no split-K by default) for M <= 16, and serves larger M by
// tiling M over blockIdx.z.
#include <cooperative_groups.h>

#include "common.cuh"
#include "qlinear.h"

namespace cg = cooperative_groups;

namespace b200q {
namespace decode {

constexpr int BN = 128;                      // columns per CTA
constexpr int BK = 64;                       // k rows per pipeline stage
constexpr int BM = 16;                       // activation rows per CTA (one MMA row block)
constexpr int STAGES = 4;
constexpr int CONSUMER_WARPS = 4;            // each takes BK / 4 = 16 k-rows of a stage
constexpr int THREADS = 32 * (CONSUMER_WARPS + 1);
constexpr int W_STAGE_BYTES = BK * BN;       // 8192
constexpr int A_STAGE_BYTES = BM * BK * 2;   // 2048
constexpr int STAGE_TX_BYTES = W_STAGE_BYTES + A_STAGE_BYTES;
constexpr int RED_STRIDE = BN + 4;           // fp32 words per row of the cross-warp reduction buffer
constexpr int RED_BYTES = CONSUMER_WARPS * BM * RED_STRIDE * 4;
constexpr int PIPE_BYTES = STAGES * STAGE_TX_BYTES;
constexpr int SMEM_BYTES = (PIPE_BYTES > RED_BYTES ? PIPE_BYTES : RED_BYTES) + 1024;  // + alignment slack
constexpr int64_t kMaxCounters = 65536;       // arrival counters at the head of the workspace
constexpr int kMaxCluster = 8;               // largest portable cluster

__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

__device__ __forceinline__ void mma_m16n8k16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Two k-rows of 16 int8 columns each (x: row k, y: row k+1) -> for every column i of the 16 the f16
// pair (w[k][i], w[k+1][i]), which is one B-fragment register of an m16n8k16 MMA.
__device__ __forceinline__ void rows_to_pairs(const uint4 &x, const uint4 &y, uint32_t (&out)[16]) {
    const uint32_t xs[4] = {x.x, x.y, x.z, x.w};
    const uint32_t ys[4] = {y.x, y.y, y.z, y.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const uint32_t p = __byte_perm(xs[j], ys[j], 0x5410);  // x.b0 x.b1 y.b0 y.b1
        const uint32_t q = __byte_perm(xs[j], ys[j], 0x7632);  // x.b2 x.b3 y.b2 y.b3
        cvt_s8x4_to_f16x4(p, out[4 * j + 0], out[4 * j + 1]);
        cvt_s8x4_to_f16x4(q, out[4 * j + 2], out[4 * j + 3]);
    }
}

struct Params {
    const __half *scale;
    __half *c;
    float *partial;           // [splits][M][N] fp32, used when splits > 1
    unsigned int *counters;   // [m_tiles * n_tiles], zero on entry, zero on exit
    unsigned int *status;
    int M, N;
    int k_begin, k_end;       // the k range this launch sums over (k_end is also the tensor maps' K extent)
    int iters_per_split;      // BK-sized k steps per split
    int splits;
    int mode;                 // how the splits of one output tile are combined
};

constexpr int kModeDirect = 0;     // splits == 1
constexpr int kModeCluster = 1;    // the splits of a tile form one thread-block cluster (splits <= 16)
constexpr int kModeWorkspace = 2;  // partial tiles in the caller's workspace, last arriver sums them

__global__ void __launch_bounds__(THREADS) qlinear_decode_kn_kernel(const __grid_constant__ CUtensorMap map_w,
                                                                    const __grid_constant__ CUtensorMap map_a,
                                                                    const Params p) {
    extern __shared__ unsigned char smem_dyn[];
    __shared__ __align__(8) uint64_t full_bar[STAGES];
    __shared__ __align__(8) uint64_t empty_bar[STAGES];
    __shared__ unsigned int is_last;

    // 128B-swizzled TMA tiles need 1024-byte aligned bases.
    const uint32_t smem_base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
    unsigned char *smem_gen = smem_dyn + (smem_base - smem_u32(smem_dyn));
    const uint32_t w_base = smem_base;
    const uint32_t a_base = smem_base + STAGES * W_STAGE_BYTES;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * BN;
    const int split = blockIdx.y;
    const int m0 = blockIdx.z * BM;
    const int total_iters = (p.k_end - p.k_begin + BK - 1) / BK;
    const int it_begin = split * p.iters_per_split;
    int n_iters = total_iters - it_begin;
    if (n_iters > p.iters_per_split) n_iters = p.iters_per_split;
    if (n_iters < 0) n_iters = 0;

    if (threadIdx.x == 0) {
#pragma unroll
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), CONSUMER_WARPS);
        }
        mbar_fence_init();
    }
    __syncthreads();

    float acc[16][4];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.0f;
    }

    if (warp == CONSUMER_WARPS) {
        // ---------------- producer: one lane drives TMA ----------------
        if (lane == 0) {
            tma_prefetch_desc(&map_w);
            tma_prefetch_desc(&map_a);
            const uint64_t stream_policy = l2_policy_evict_first();  // the weight is read once
            for (int it = 0; it < n_iters; ++it) {
                const int s = it % STAGES;
                if (it >= STAGES) {
                    if (!mbar_wait(smem_u32(&empty_bar[s]), ((it / STAGES) - 1) & 1)) {
                        report_timeout(p.status, kKernelDecode, 1);
                        break;
                    }
                }
                const uint32_t bar = smem_u32(&full_bar[s]);
                const int k0 = p.k_begin + (it_begin + it) * BK;
                mbar_expect_tx(bar, STAGE_TX_BYTES);
                tma_load_2d_hint(w_base + s * W_STAGE_BYTES, &map_w, n0, k0, bar, stream_policy);
                tma_load_2d(a_base + s * A_STAGE_BYTES, &map_a, k0, m0, bar);
            }
        }
    } else {
        // ---------------- consumers ----------------
        const int g = lane >> 2;  // MMA group id: activation row / B column
        const int t = lane & 3;   // thread in group: k pair
        const int r_lo = warp * 16 + 2 * t;  // this thread's k-rows inside a stage: r_lo, +1, +8, +9
        // 16-byte chunk g of row r sits at chunk (g ^ (r & 7)) under the 128B swizzle.
        const uint32_t off_x0 = (r_lo + 0) * 128 + ((g ^ ((r_lo + 0) & 7)) << 4);
        const uint32_t off_y0 = (r_lo + 1) * 128 + ((g ^ ((r_lo + 1) & 7)) << 4);
        const uint32_t off_x1 = (r_lo + 8) * 128 + ((g ^ ((r_lo + 8) & 7)) << 4);
        const uint32_t off_y1 = (r_lo + 9) * 128 + ((g ^ ((r_lo + 9) & 7)) << 4);
        // activations: rows g and g+8 (both have row & 7 == g), k = 16*warp + 2t (+8): chunks 2*warp, 2*warp+1
        const uint32_t off_a0 = g * 128 + (((2 * warp + 0) ^ g) << 4) + 4 * t;
        const uint32_t off_a2 = g * 128 + (((2 * warp + 1) ^ g) << 4) + 4 * t;
        bool ok = true;
        for (int it = 0; it < n_iters; ++it) {
            const int s = it % STAGES;
            if (!mbar_wait(smem_u32(&full_bar[s]), (it / STAGES) & 1)) {
                report_timeout(p.status, kKernelDecode, 2);
                ok = false;
                break;
            }
            const uint32_t wb = w_base + s * W_STAGE_BYTES;
            const uint32_t ab = a_base + s * A_STAGE_BYTES;
            const uint4 x0 = lds128(wb + off_x0);
            const uint4 y0 = lds128(wb + off_y0);
            const uint4 x1 = lds128(wb + off_x1);
            const uint4 y1 = lds128(wb + off_y1);
            uint32_t a[4];
            a[0] = lds32(ab + off_a0);
            a[1] = lds32(ab + off_a0 + 8 * 128);
            a[2] = lds32(ab + off_a2);
            a[3] = lds32(ab + off_a2 + 8 * 128);
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&empty_bar[s]));  // stage is in registers now
            uint32_t b_lo[16], b_hi[16];
            rows_to_pairs(x0, y0, b_lo);
            rows_to_pairs(x1, y1, b_hi);
#pragma unroll
            for (int i = 0; i < 16; ++i) mma_m16n8k16(acc[i], a, b_lo[i], b_hi[i]);
        }
        (void)ok;
    }

    // ---------------- cross-warp reduction through shared memory ----------------
    __syncthreads();  // every issued stage has landed and been consumed: the ring can be reused
    float *red = reinterpret_cast<float *>(smem_gen);
    if (warp < CONSUMER_WARPS) {
        const int g = lane >> 2;
        const int t = lane & 3;
        float *mine = red + warp * BM * RED_STRIDE;
        // MMA i holds columns {16 * j + i}; this thread has j = 2t, 2t+1 for rows g and g+8.  One
        // word of skew per 32 columns keeps the 32 lanes on 32 banks.
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const int c0 = 32 * t + i, c1 = c0 + 16;
            mine[g * RED_STRIDE + c0 + (c0 >> 5)] = acc[i][0];
            mine[g * RED_STRIDE + c1 + (c1 >> 5)] = acc[i][1];
            mine[(g + 8) * RED_STRIDE + c0 + (c0 >> 5)] = acc[i][2];
            mine[(g + 8) * RED_STRIDE + c1 + (c1 >> 5)] = acc[i][3];
        }
    }
    __syncthreads();

    const int col = threadIdx.x;          // column of the tile this thread finishes (threads 0..127)
    const int n = n0 + col;
    int rows = p.M - m0;
    if (rows > BM) rows = BM;
    const bool active = (col < BN) && (n < p.N);
    const int skew = col + (col >> 5);

    if (p.mode == kModeDirect) {
        if (active) {
            const float sc = __half2float(p.scale[n]);
            for (int r = 0; r < rows; ++r) {
                float v = 0.0f;
#pragma unroll
                for (int w = 0; w < CONSUMER_WARPS; ++w) v += red[(w * BM + r) * RED_STRIDE + skew];
                p.c[(size_t)(m0 + r) * p.N + n] = __float2half_rn(v * sc);
            }
        }
        return;
    }

    if (p.mode == kModeCluster) {
        // ---------------- split-K inside a cluster: partial tiles meet through distributed shared memory ----------------
        // The CTAs of a cluster are the `splits` CTAs of one output tile.  Each first folds its four
        // warp slabs into slab 0, then CTA `rank` sums columns [rank * BN / splits, ...) over all CTAs
        // in rank order (a fixed order: the result does not depend on timing).
        cg::cluster_group cluster = cg::this_cluster();
        if (col < BN) {
            for (int r = 0; r < rows; ++r) {
                float v = 0.0f;
#pragma unroll
                for (int w = 0; w < CONSUMER_WARPS; ++w) v += red[(w * BM + r) * RED_STRIDE + skew];
                red[r * RED_STRIDE + skew] = v;
            }
        }
        cluster.sync();
        const unsigned int csize = cluster.num_blocks();
        const unsigned int rank = cluster.block_rank();
        const int cols_per = BN / (int)csize;
        for (int idx = threadIdx.x; idx < rows * cols_per; idx += THREADS) {
            const int r = idx / cols_per;
            const int cc = (int)rank * cols_per + (idx - r * cols_per);
            const int nn = n0 + cc;
            if (nn < p.N) {
                const int off = r * RED_STRIDE + cc + (cc >> 5);
                float v = 0.0f;
                for (unsigned int j = 0; j < csize; ++j) v += cluster.map_shared_rank(red, j)[off];
                p.c[(size_t)(m0 + r) * p.N + nn] = __float2half_rn(v * __half2float(p.scale[nn]));
            }
        }
        cluster.sync();  // nobody leaves while a peer may still read its shared memory
        return;
    }

    // ---------------- split-K through the workspace: publish the partial tile, last CTA of the tile finishes ----------------
    if (active) {
        for (int r = 0; r < rows; ++r) {
            float v = 0.0f;
#pragma unroll
            for (int w = 0; w < CONSUMER_WARPS; ++w) v += red[(w * BM + r) * RED_STRIDE + skew];
            p.partial[((size_t)split * p.M + (m0 + r)) * p.N + n] = v;
        }
    }
    __threadfence();
    __syncthreads();
    const unsigned int tile_id = blockIdx.z * gridDim.x + blockIdx.x;
    if (threadIdx.x == 0) {
        const unsigned int prev = atomicAdd(&p.counters[tile_id], 1u);
        is_last = (prev == (unsigned int)(p.splits - 1)) ? 1u : 0u;
    }
    __syncthreads();
    if (is_last == 0) return;
    __threadfence();
    if (active) {
        const float sc = __half2float(p.scale[n]);
        for (int r = 0; r < rows; ++r) {
            float v = 0.0f;
#pragma unroll 4
            for (int s = 0; s < p.splits; ++s) v += __ldcg(&p.partial[((size_t)s * p.M + (m0 + r)) * p.N + n]);
            p.c[(size_t)(m0 + r) * p.N + n] = __float2half_rn(v * sc);
        }
    }
    if (threadIdx.x == 0) p.counters[tile_id] = 0;  // leave the workspace ready for the next call
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
    const int64_t target = (int64_t)sms * 3;  // three CTAs of this kernel share an SM
    const int64_t tiles = (int64_t)pl.n_tiles * pl.m_tiles;
    int64_t splits = tiles > 0 ? target / tiles : 1;
    const int max_splits = k_iters / 4 > 0 ? k_iters / 4 : 1;  // at least four stages of work per CTA
    if (splits > max_splits) splits = max_splits;
    if (splits > 64) splits = 64;
    if (splits < 1) splits = 1;
    if (splits <= 2 * kMaxCluster) {
        // Up to a cluster's worth (and a little beyond: a full cluster beats a few more CTAs that need
        // the workspace): the splits of a tile form a cluster and meet in distributed shared memory.
        int c = 1;
        while (c * 2 <= splits && c * 2 <= kMaxCluster) c *= 2;
        splits = c;
        pl.cluster = c;
    } else {
        pl.cluster = 1;
        if (tiles > kMaxCounters) splits = 1;
    }
    pl.iters_per_split = (int)ceil_div(k_iters, splits);
    if (pl.cluster > 1) {
        pl.splits = pl.cluster;  // the grid must hold whole clusters; a split may have fewer steps, or none
    } else {
        pl.splits = (int)ceil_div(k_iters, pl.iters_per_split);
        if (pl.splits < 1) pl.splits = 1;
    }
    const bool workspace = pl.cluster == 1 && pl.splits > 1;
    // The counter region has one fixed size, so that counters never land on bytes an earlier call of
    // another shape used for partial sums: the region stays all-zero between calls.
    pl.counter_bytes = workspace ? (size_t)kMaxCounters * 4 : 0;
    pl.partial_bytes = workspace ? (size_t)pl.splits * M * N * 4 : 0;
    return pl;
}

bool decode_kn_supported(const void *a, const void *wq, int64_t N, int64_t K) {
    return (N % 16 == 0) && (K % 8 == 0) && ((reinterpret_cast<uintptr_t>(a) & 15u) == 0) &&
           ((reinterpret_cast<uintptr_t>(wq) & 15u) == 0);
}

int launch_decode_kn(const void *a, const void *wq, const void *scale, void *c, int64_t M, int64_t N, int64_t K,
                     int64_t k_begin, int64_t k_end, bool allow_split, void *workspace, size_t workspace_bytes,
                     cudaStream_t stream) {
    using namespace decode;
    DecodePlan pl = plan_decode(M, N, k_end - k_begin);
    if (!allow_split) {
        pl.iters_per_split = (int)ceil_div(k_end - k_begin, BK);
        pl.splits = 1;
        pl.cluster = 1;
        pl.partial_bytes = 0;
        pl.counter_bytes = 0;
    }
    if (pl.partial_bytes > 0 && (workspace == nullptr || workspace_bytes < pl.counter_bytes + pl.partial_bytes)) {
        return set_error(B200Q_WORKSPACE_TOO_SMALL, "qlinear: workspace of %zu bytes given, %zu needed for M=%lld N=%lld K=%lld",
                         workspace_bytes, pl.counter_bytes + pl.partial_bytes, (long long)M, (long long)N, (long long)K);
    }
    if (pl.m_tiles > 65535 || pl.splits > 65535) return set_error(B200Q_UNSUPPORTED, "qlinear: M=%lld is too large for the small-M kernel", (long long)M);

    CUtensorMap map_w, map_a;
    int rc = make_tensor_map_2d(&map_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, wq, (uint64_t)N, (uint64_t)k_end, (uint64_t)N, BN, BK,
                                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
    if (rc != B200Q_OK) return rc;
    rc = make_tensor_map_2d(&map_a, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, a, (uint64_t)k_end, (uint64_t)M, (uint64_t)K * 2, BK, BM,
                            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B);
    if (rc != B200Q_OK) return rc;

    Params p;
    p.scale = static_cast<const __half *>(scale);
    p.c = static_cast<__half *>(c);
    p.counters = static_cast<unsigned int *>(workspace);
    p.partial = pl.partial_bytes > 0 ? reinterpret_cast<float *>(static_cast<unsigned char *>(workspace) + pl.counter_bytes) : nullptr;
    p.status = device_status_word();
    p.M = (int)M;
    p.N = (int)N;
    p.k_begin = (int)k_begin;
    p.k_end = (int)k_end;
    p.iters_per_split = pl.iters_per_split;
    p.splits = pl.splits;
    p.mode = pl.splits == 1 ? kModeDirect : (pl.cluster > 1 ? kModeCluster : kModeWorkspace);

    static bool attr_set[64] = {false};  // per device; a repeated set is harmless
    int dev = 0;
    B200Q_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !attr_set[dev]) {
        B200Q_CUDA_TRY(cudaFuncSetAttribute(qlinear_decode_kn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        if (dev >= 0 && dev < 64) attr_set[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)pl.n_tiles, (unsigned)pl.splits, (unsigned)pl.m_tiles);
    cfg.blockDim = dim3(THREADS, 1, 1);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attrs[1];
    attrs[0].id = cudaLaunchAttributeClusterDimension;
    attrs[0].val.clusterDim.x = 1;
    attrs[0].val.clusterDim.y = (unsigned)pl.cluster;
    attrs[0].val.clusterDim.z = 1;
    cfg.attrs = attrs;
    cfg.numAttrs = 1;
    B200Q_CUDA_TRY(cudaLaunchKernelEx(&cfg, qlinear_decode_kn_kernel, map_w, map_a, p));
    return B200Q_OK;
}

}  // namespace b200q
