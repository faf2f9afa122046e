// Large-M (prefill) f16 x int8 quantized linear for weights in the reference's [K, N] layout, on the
// fifth-generation tensor cores: tcgen05.mma with fp32 accumulators in tensor memory.
//
// The product is computed transposed, D[n, m] = sum_k W[k, n] * A[m, k], so that the operand that needs
// work before the MMA -- the int8 weight -- is the 128-row operand and the activations, which TMA can
// deliver in final form, are the 256-column operand: per 128 x 256 x 16 MMA the tensor core reads
// 4 KB + 8 KB of shared memory, the converters read 2 KB and write 4 KB, which leaves shared-memory
// bandwidth headroom that the opposite assignment would not.
//
// One persistent CTA per SM, fourteen warps:
//   warp 12     TMA producer: per 64-k stage one int8 tile [64 k][128 n] (128B swizzle, its own short
//               ring) and one activation tile [TM m][64 k] f16 (128B swizzle = K-major MMA operand as is);
//               TM = 256, or 64 when that fills more SMs
//   warps 4-11  converters: transposing matrix loads of the int8 tile (four consecutive k of one column per
//               register), int8 -> exact f16 in registers, written as the K-major, 128B-swizzled MMA
//               operand ([128 n][64 k], the same as for weights stored [N, K]) with 8-byte stores that
//               touch every bank once, then a proxy fence and an mbarrier
//   warp 13     MMA issuer (one lane): four K=16 MMAs per stage into one of two 256-column TMEM
//               accumulators; tcgen05.commit frees the stage / publishes the accumulator
//   warps 0-3   epilogue: tcgen05.ld of the accumulator (lane = weight column n, column = row m),
//               times scale[n], one rounding to f16, transposed through a small staging buffer and
//               written as 256-byte rows with 16-byte stores to C[m, n] of every destination (each may be a
//               column range of a wider matrix; the destinations of a column-parallel layer are the
//               peer-mapped outputs of all ranks); overlaps the next tile's MMAs
// Rows beyond M, columns beyond N and k beyond K are zero-filled by TMA and never stored.
//
// Every wait is bounded.  A wait that runs out records where in the device status word and raises a
// CTA-wide abort flag that every other wait watches, so all roles leave their loops at once instead of
// each running into its own limit.  Before the CTA gives back its tensor memory and retires, the producer
// waits (bounded again) for every copy it has armed and the MMA lane for a final commit, so that nothing
// still writes to shared memory or reads tensor memory when the CTA is gone.
//
// Replaces, for large M, the generated mma.sync kernel of
// python/hidet/graph/ops/quant/matmul_f16_i8.py:136-485 (f16 accumulation) and the separate sum over
// split-K parts that follows it (python/hidet/graph/ops/quant/resolve.py:99).
#include <atomic>

#include "common.cuh"
#include "qlinear.h"

namespace b200q {
namespace prefill {

constexpr int TN = 128;                     // weight columns per tile = MMA M
constexpr int BK = 64;                      // k per stage = four MMAs of K = 16
constexpr int RAW_BYTES = BK * TN;          // int8 tile
constexpr int WF_BYTES = BK * TN * 2;       // converted f16 tile
constexpr int CONV_WARPS = 8;
constexpr int EPI_WARP0 = 0, CONV_WARP0 = 4, PRODUCER_WARP = CONV_WARP0 + CONV_WARPS, MMA_WARP = PRODUCER_WARP + 1;
constexpr int THREADS = 32 * (MMA_WARP + 1);
constexpr int STAGE_ROW_BYTES = TN * 2 + 16; // one output row of a tile in the epilogue's staging buffer, padded
constexpr int STAGING_BYTES = 32 * STAGE_ROW_BYTES;

// Per activation-tile height TM (= MMA N): ring depths and the shared-memory budget.
template <int TM>
struct Config {
    static constexpr int ACT_BYTES = TM * BK * 2;
    static constexpr int STAGES = TM == 256 ? 4 : 6;         // f16 weight + activation ring, consumed by the MMAs
    static constexpr int RAW_SLOTS = TM == 256 ? 3 : 4;      // int8 ring, consumed by the converters
    // Converter warps form groups that take stages in turn, so that the load-convert-store-fence latency
    // of one stage overlaps that of the next ones (the ring must hold the stages being converted plus two).
    static constexpr int CONV_GROUPS = TM == 256 ? 2 : 4;
    static constexpr int GROUP_WARPS = CONV_WARPS / CONV_GROUPS;
    // Stages after which the same converter group meets the same int8 slot again: lcm(RAW_SLOTS, CONV_GROUPS).
    static constexpr int RAW_PERIOD = TM == 256 ? 6 : 4;
    static_assert(RAW_PERIOD % RAW_SLOTS == 0 && RAW_PERIOD % CONV_GROUPS == 0, "RAW_PERIOD must be a common multiple");
    static constexpr int CONV_ROWS = GROUP_WARPS * 4;        // k-rows a group covers per pass (8 threads per row)
    static constexpr int MAIN_BYTES = ACT_BYTES + WF_BYTES;
    static constexpr int SMEM_BYTES = STAGES * MAIN_BYTES + RAW_SLOTS * RAW_BYTES + STAGING_BYTES + 1024;  // + alignment slack
    static constexpr uint32_t TMEM_COLS = 2 * TM;            // two accumulators of TM fp32 columns (a power of two >= 32)
    // tcgen05 instruction descriptor, kind::f16: D = f32, A = B = f16, both K-major,
    // N = TM (bits 17..22 hold N / 8), M = 128 (bits 24..28 hold M / 16).
    static constexpr uint32_t kInstrDesc = (1u << 4) | ((uint32_t)(TM >> 3) << 17) | ((uint32_t)(TN >> 4) << 24);
};

// Shared-memory matrix descriptor: start address, leading / stride byte offsets (all in 16-byte
// units), descriptor version 1, 128-byte swizzle.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t leading_bytes, uint32_t stride_bytes) {
    return (uint64_t)((addr >> 4) & 0x3fffu) | ((uint64_t)((leading_bytes >> 4) & 0x3fffu) << 16) |
           ((uint64_t)((stride_bytes >> 4) & 0x3fffu) << 32) | (1ull << 46) | (2ull << 61);
}

__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] (+)= A[smem] * B[smem]; accumulate == 0 overwrites D.
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}\n"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
// The mbarrier gets one arrival when every MMA issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// 32 consecutive fp32 columns of this warp's 32 TMEM lanes: thread i gets lane (base lane + i).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
          "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]),
          "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
          "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Two 16 x 16 byte tiles, transposed on the way to registers.  Lanes 0-15 give the addresses of the 16 rows (16 bytes
// each) of the first tile, lanes 16-31 those of the second.  With a tile stored as [k][column], lane (g = lane / 4,
// t = lane % 4) receives, for tile i, in r[2i] the bytes (k = 4t .. 4t+3, column g) and in r[2i+1] the bytes
// (k = 4t .. 4t+3, column g + 8).
__device__ __forceinline__ void ldmatrix_x2_trans_b8(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m16n16.x2.trans.shared.b8 {%0, %1, %2, %3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void sts64(uint32_t addr, uint32_t a, uint32_t b) {
    asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(addr), "r"(a), "r"(b) : "memory");
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ void sts128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

// Four signed bytes (b0 .. b3) -> f16 pairs (b0, b1) and (b2, b3), exactly (0x6400 | u is 1024 + u).
__device__ __forceinline__ void cvt_s8x4_to_f16_pairs(uint32_t v, uint32_t &p01, uint32_t &p23) {
    const uint32_t u = v ^ 0x80808080u;
    const uint32_t e01 = __byte_perm(u, 0x64646464u, 0x4140);
    const uint32_t e23 = __byte_perm(u, 0x64646464u, 0x4342);
    const uint32_t bias = 0x64806480u;
    asm("sub.f16x2 %0, %1, %2;" : "=r"(p01) : "r"(e01), "r"(bias));
    asm("sub.f16x2 %0, %1, %2;" : "=r"(p23) : "r"(e23), "r"(bias));
}

struct Params {
    const __half *scale;
    OutTargets out;
    Epilogue ep;
    unsigned int *status;
    int M, N, K;
    int n_tiles, m_tiles;
    // K split over several CTAs per output tile (narrow problems that would leave most SMs idle): a tile index is
    // (output tile, split); split s sums k blocks [s * kb_per_split, ...) and writes raw fp32 sums to
    // partial[s][M][N]; qlinear_prefill_reduce_kernel adds the splits and finishes.  k_splits == 1: no partial.
    int k_splits, kb_per_split;
    float *partial;
};

// FUSED: the epilogue of p.ep (bias, gate / up pairing, residual) is compiled in.
// NK: the weight is [N, K] with K contiguous: the int8 tile is 128 weight rows of 64 k-bytes and its f16
//     image is the K-major MMA operand (rows of 128 bytes, 128B swizzle), like the activation tile.
constexpr uint32_t kFastPolls = 4096;
// The rest of a bounded wait: polls on, looking at the CTA's abort flag between runs of polls; when its own
// limit runs out it records the site and raises the flag for the other roles.
__device__ __noinline__ bool wait_or_abort(uint32_t bar, uint32_t parity, unsigned int site, int *abort_flag, unsigned int *status) {
    for (uint32_t round = 0; round < kSpinLimit / 1024u; ++round) {
        if (mbar_wait(bar, parity, 1024u)) return true;
        if (*reinterpret_cast<volatile int *>(abort_flag) != 0) return false;
    }
    report_timeout(status, kKernelPrefill, site);
    atomicExch(abort_flag, 1);
    return false;
}

template <int TM, bool FUSED, bool NK>
__global__ void __launch_bounds__(THREADS, 1) qlinear_prefill_kn_kernel(const __grid_constant__ CUtensorMap map_w,
                                                                        const __grid_constant__ CUtensorMap map_a,
                                                                        const Params p) {
    using Cfg = Config<TM>;
    constexpr int STAGES = Cfg::STAGES, RAW_SLOTS = Cfg::RAW_SLOTS;
    constexpr int CONV_GROUPS = Cfg::CONV_GROUPS, GROUP_WARPS = Cfg::GROUP_WARPS, CONV_ROWS = Cfg::CONV_ROWS;
    constexpr int RAW_PERIOD = Cfg::RAW_PERIOD;
    extern __shared__ unsigned char smem_dyn[];
    // An int8 tile has landed.  A parity wait tells a phase only from its neighbours, so a waiter has to
    // see every phase of its barrier; successive uses of a slot can belong to different converter groups,
    // hence one barrier per slot and group: the pair (slot, group) recurs every RAW_PERIOD stages.
    __shared__ __align__(8) uint64_t raw_full[RAW_SLOTS][CONV_GROUPS];
    __shared__ __align__(8) uint64_t raw_empty[RAW_SLOTS];  // the converter group of that stage has read it
    __shared__ __align__(8) uint64_t act_full[STAGES];      // an activation tile has landed
    __shared__ __align__(8) uint64_t conv_full[STAGES];     // the converter group of that stage has written the f16 tile
    __shared__ __align__(8) uint64_t slot_free[STAGES];     // the MMAs that read the stage have completed
    __shared__ __align__(8) uint64_t acc_full[2];           // an accumulator holds a finished tile
    __shared__ __align__(8) uint64_t acc_empty[2];          // the four epilogue warps have read it out
    __shared__ __align__(8) uint64_t drain_bar;             // every MMA issued has completed (teardown)
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;                               // a wait ran out somewhere in this CTA

    const uint32_t smem_base = (smem_u32(smem_dyn) + 1023u) & ~1023u;  // swizzled operands need 1024-byte alignment
    unsigned char *smem_gen = smem_dyn + (smem_base - smem_u32(smem_dyn));
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int total_tiles = p.n_tiles * p.m_tiles * p.k_splits;
    const int k_blocks = (p.K + BK - 1) / BK;
    // tile index -> output tile and k-block range
    auto kb_first = [&](int tile) { return (tile % p.k_splits) * p.kb_per_split; };
    auto kb_last = [&](int tile) { return min(k_blocks, (tile % p.k_splits + 1) * p.kb_per_split); };

    // layout: STAGES x [activations][f16 weights], RAW_SLOTS x [int8 weights], epilogue staging
    auto act_addr = [&](int s) { return smem_base + s * Cfg::MAIN_BYTES; };
    auto wf_addr = [&](int s) { return smem_base + s * Cfg::MAIN_BYTES + Cfg::ACT_BYTES; };
    auto raw_addr = [&](int r) { return smem_base + STAGES * Cfg::MAIN_BYTES + r * RAW_BYTES; };
    constexpr int STAGING_OFF = STAGES * Cfg::MAIN_BYTES + RAW_SLOTS * RAW_BYTES;

    if (threadIdx.x == 0) {
        for (int r = 0; r < RAW_SLOTS; ++r) {
            for (int g = 0; g < CONV_GROUPS; ++g) mbar_init(smem_u32(&raw_full[r][g]), 1);
            mbar_init(smem_u32(&raw_empty[r]), GROUP_WARPS);
        }
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&act_full[s]), 1);
            mbar_init(smem_u32(&conv_full[s]), GROUP_WARPS);
            mbar_init(smem_u32(&slot_free[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&acc_full[b]), 1);
            mbar_init(smem_u32(&acc_empty[b]), 4);
        }
        mbar_init(smem_u32(&drain_bar), 1);
        abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == MMA_WARP) {
        tmem_alloc(smem_u32(&tmem_base_slot), Cfg::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = tmem_base_slot;
    // Bounded wait that also ends when another role has given up; the role whose own limit runs out reports it.
    // The first polls are the plain inlined loop; everything else lives in a function of its own, so that the
    // code around the hot loops stays what it is without the flag (with the flag test inlined at every wait the
    // kernel lost a tenth of its speed, although the test never ran).
    auto wait = [&](uint32_t bar, uint32_t parity, unsigned int site) -> bool {
        if (mbar_wait(bar, parity, kFastPolls)) return true;
        return wait_or_abort(bar, parity, site, &abort_flag, p.status);
    };

    if (warp == PRODUCER_WARP) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            tma_prefetch_desc(&map_w);
            tma_prefetch_desc(&map_a);
            const uint64_t keep = l2_policy_evict_last();  // both operands are re-read by other tiles: keep them in L2
            uint32_t i = 0;
            bool ok = true;
            uint32_t n_raw = 0, n_act = 0;  // copies armed so far (stages 0 .. n - 1), for the teardown
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                const int otile = tile / p.k_splits;
                const int n0 = (otile % p.n_tiles) * TN;
                const int m0 = (otile / p.n_tiles) * TM;
                for (int kb = kb_first(tile), kb_end = kb_last(tile); kb < kb_end; ++kb, ++i) {
                    const int r = i % RAW_SLOTS;
                    const uint32_t use_r = i / RAW_SLOTS;
                    if (use_r >= 1 && !wait(smem_u32(&raw_empty[r]), (use_r - 1) & 1, 1)) {
                        ok = false;
                        break;
                    }
                    const uint32_t raw_bar = smem_u32(&raw_full[r][i % CONV_GROUPS]);  // the group that converts stage i
                    mbar_expect_tx(raw_bar, RAW_BYTES);
                    tma_load_2d_hint(raw_addr(r), &map_w, NK ? kb * BK : n0, NK ? n0 : kb * BK, raw_bar, keep);
                    n_raw = i + 1;
                    const int s = i % STAGES;
                    const uint32_t use = i / STAGES;
                    if (use >= 1 && !wait(smem_u32(&slot_free[s]), (use - 1) & 1, 6)) {
                        ok = false;
                        break;
                    }
                    mbar_expect_tx(smem_u32(&act_full[s]), Cfg::ACT_BYTES);
                    tma_load_2d_hint(act_addr(s), &map_a, kb * BK, m0, smem_u32(&act_full[s]), keep);
                    n_act = i + 1;
                }
            }
            // Teardown: every copy this lane has armed must have landed before the CTA may retire.  After a
            // normal run they all have (their stages were consumed); after an abort this waits for the stragglers.
            // The latest stage copied into slot x of a ring of n slots, of c copies: the largest j < c with j % n == x.
            for (uint32_t r = 0; r < (uint32_t)RAW_SLOTS; ++r) {
                if (n_raw <= r) continue;
                const uint32_t j = n_raw - 1 - (n_raw - 1 - r) % RAW_SLOTS;
                if (!mbar_wait(smem_u32(&raw_full[r][j % CONV_GROUPS]), (j / RAW_PERIOD) & 1)) report_timeout(p.status, kKernelPrefill, 7);
            }
            for (uint32_t s = 0; s < (uint32_t)STAGES; ++s) {
                if (n_act <= s) continue;
                const uint32_t j = n_act - 1 - (n_act - 1 - s) % STAGES;
                if (!mbar_wait(smem_u32(&act_full[s]), (j / STAGES) & 1)) report_timeout(p.status, kKernelPrefill, 7);
            }
        }
    } else if (warp == MMA_WARP) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            uint32_t i = 0, t_iter = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++t_iter) {
                const uint32_t buf = t_iter & 1, acc_use = t_iter >> 1;
                if (acc_use >= 1 && !wait(smem_u32(&acc_empty[buf]), (acc_use - 1) & 1, 2)) break;
                tc_fence_after_sync();
                const uint32_t d_addr = tmem_base + buf * TM;
                const int kb_begin = kb_first(tile);
                for (int kb = kb_begin, kb_end = kb_last(tile); kb < kb_end; ++kb, ++i) {
                    const int s = i % STAGES;
                    const uint32_t use = i / STAGES;
                    if (!wait(smem_u32(&act_full[s]), use & 1, 3) || !wait(smem_u32(&conv_full[s]), use & 1, 3)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
#pragma unroll
                    for (int ks = 0; ks < BK / 16; ++ks) {
                        // A: K-major f16 weights (whichever way the int8 weight is stored), like B
                        const uint64_t da = smem_desc(wf_addr(s) + ks * 32, 16, 1024);
                        // B: K-major activations, 8-row groups 1024 B apart; K = 16 is 32 bytes along the swizzled row.
                        const uint64_t db = smem_desc(act_addr(s) + ks * 32, 16, 1024);
                        umma_f16(d_addr, da, db, Cfg::kInstrDesc, (kb > kb_begin || ks > 0) ? 1u : 0u);
                    }
                    umma_commit(smem_u32(&slot_free[s]));
                }
                if (ok) umma_commit(smem_u32(&acc_full[buf]));
            }
            // Teardown: no MMA may still be running when the tensor memory is given back.
            umma_commit(smem_u32(&drain_bar));
            if (!mbar_wait(smem_u32(&drain_bar), 0)) report_timeout(p.status, kKernelPrefill, 8);
        }
    } else if (warp >= CONV_WARP0 && warp < CONV_WARP0 + CONV_WARPS) {
        // ---------------- converters ----------------
        const int cw = warp - CONV_WARP0;
        const int group = cw % CONV_GROUPS;            // this warp's group converts stages group, group + CONV_GROUPS, ...
        const int gw = cw / CONV_GROUPS;               // this warp inside its group
        const int ct = (cw / CONV_GROUPS) * 32 + lane; // 0 .. 32 * GROUP_WARPS - 1 inside the group
        uint32_t i = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
            for (int kb = kb_first(tile), kb_end = kb_last(tile); kb < kb_end; ++kb, ++i) {
                if ((int)(i % CONV_GROUPS) != group) continue;
                const int r = i % RAW_SLOTS;
                const uint32_t use_r = i / RAW_SLOTS;
                const int s = i % STAGES;
                const uint32_t use = i / STAGES;
                // The int8 tile must have landed (on the barrier of this slot that belongs to this group),
                // and the MMAs that read the f16 slot last time must be done.
                if (!wait(smem_u32(&raw_full[r][group]), (i / RAW_PERIOD) & 1, 4) || (use >= 1 && !wait(smem_u32(&slot_free[s]), (use - 1) & 1, 4))) {
                    ok = false;
                    break;
                }
                const uint32_t raw = raw_addr(r), wf = wf_addr(s);
                if (NK) {
                    uint4 v[BK / CONV_ROWS];
#pragma unroll
                    for (int pass = 0; pass < BK / CONV_ROWS; ++pass) v[pass] = lds128(raw + (pass * (32 * GROUP_WARPS) + ct) * 16);
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&raw_empty[r]));  // the int8 tile is in registers
                    // 16-byte piece `id` of the tile is 16 k of weight row id / 4: two 8-k chunks of that row's 128 f16 bytes
#pragma unroll
                    for (int pass = 0; pass < BK / CONV_ROWS; ++pass) {
                        const int id = pass * (32 * GROUP_WARPS) + ct;
                        const int n = id >> 2, c2 = (id & 3) * 2;
                        uint32_t h[8];
                        cvt_s8x4_to_f16_pairs(v[pass].x, h[0], h[1]);
                        cvt_s8x4_to_f16_pairs(v[pass].y, h[2], h[3]);
                        cvt_s8x4_to_f16_pairs(v[pass].z, h[4], h[5]);
                        cvt_s8x4_to_f16_pairs(v[pass].w, h[6], h[7]);
                        const uint32_t row = wf + n * 128;
                        sts128(row + ((c2 ^ (n & 7)) << 4), h[0], h[1], h[2], h[3]);
                        sts128(row + (((c2 + 1) ^ (n & 7)) << 4), h[4], h[5], h[6], h[7]);
                    }
                } else {
                    // [K, N] weights: the int8 tile is [64 k][128 n], 128B-swizzled.  Transposing matrix loads hand every
                    // lane four consecutive k of one column per register (column g / g + 8 of a 16-column block, k = 4t ..
                    // 4t + 3 of a 16-row block); converted, that is 8 bytes of the column's row in the K-major operand
                    // (rows of 64 k = 128 bytes, 16-byte chunk c of row n at chunk c ^ (n % 8)): the same operand as for
                    // [N, K] weights, and stores that touch every bank once.
                    constexpr int PAIRS = 4 / GROUP_WARPS;  // pairs of 16-column blocks per warp (the group covers 8 blocks)
                    uint32_t q[PAIRS][4][4];
#pragma unroll
                    for (int pr = 0; pr < PAIRS; ++pr)
#pragma unroll
                        for (int ks = 0; ks < 4; ++ks) {
                            const int chunk = 2 * (gw * PAIRS + pr) + (lane >> 4);  // 16-column block addressed by this lane
                            ldmatrix_x2_trans_b8(q[pr][ks], raw + (ks * 16 + (lane & 15)) * 128 + ((chunk ^ (lane & 7)) << 4));
                        }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&raw_empty[r]));  // the int8 tile is in registers
                    const int g = lane >> 2, t = lane & 3;
#pragma unroll
                    for (int pr = 0; pr < PAIRS; ++pr)
#pragma unroll
                        for (int ks = 0; ks < 4; ++ks)
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const int n = 32 * (gw * PAIRS + pr) + 8 * i + g;  // register i: columns g, g + 8 of the first block, then of the second
                                uint32_t lo, hi;
                                cvt_s8x4_to_f16_pairs(q[pr][ks][i], lo, hi);
                                sts64(wf + n * 128 + (((2 * ks + (t >> 1)) ^ (n & 7)) << 4) + 8 * (t & 1), lo, hi);
                            }
                }
                fence_proxy_async_smem();  // the tensor core reads these bytes through the async proxy
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&conv_full[s]));
            }
        }
    } else if (warp < 4) {
        // ---------------- epilogue ----------------
        // Per 32 activation rows: each warp reads its 32 weight columns x 32 rows from tensor memory
        // (one column per lane), scales, rounds and transposes them through the staging buffer; then the
        // four warps together write the 32 x 128 block row by row with 16-byte stores, 256 contiguous bytes
        // per row, to every destination.
        const int q = warp;       // TMEM lanes 32 q .. 32 q + 31
        const int et = threadIdx.x;  // 0 .. 127
        unsigned char *staging = smem_gen + STAGING_OFF;
        const int chunk = et & 15;   // 16-byte piece of a 256-byte output row
        const int row_in_pass = et >> 4;
        uint32_t t_iter = 0;
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++t_iter) {
            const int otile = tile / p.k_splits;
            const int n0 = (otile % p.n_tiles) * TN;
            const int m0 = (otile / p.n_tiles) * TM;
            const uint32_t buf = t_iter & 1, acc_use = t_iter >> 1;
            if (!wait(smem_u32(&acc_full[buf]), acc_use & 1, 5)) break;
            tc_fence_after_sync();
            const int n = n0 + 32 * q + lane;
            if (p.k_splits > 1) {
                // Split K: the raw fp32 sums of this split go to the workspace (lane = column, so every store of a warp is
                // 128 contiguous bytes); scales, epilogue and rounding happen once, in the reduce kernel.
                float *dst = p.partial + ((size_t)(tile % p.k_splits) * p.M + m0) * p.N + n;
                const int m_left = p.M - m0;
#pragma unroll 1
                for (int cb = 0; cb < TM / 32; ++cb) {
                    if (cb * 32 >= m_left) break;
                    uint32_t v[32];
                    tmem_ld_32x32(tmem_base + ((uint32_t)(32 * q) << 16) + buf * TM + cb * 32, v);
                    tmem_ld_wait();
                    if (n < p.N) {
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (cb * 32 + j < m_left) __stcg(dst + (size_t)(cb * 32 + j) * p.N, __uint_as_float(v[j]));
                    }
                }
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&acc_empty[buf]));
                continue;
            }
            const float sc = n < p.N ? __half2float(p.scale[n]) : 0.0f;
            const float bias = (FUSED && n < p.N && p.ep.bias != nullptr) ? __half2float(__ldg(static_cast<const __half *>(p.ep.bias) + n)) : 0.0f;
            const bool pairs = FUSED && p.ep.act == kActSiluMul;  // columns (2j, 2j + 1) = (gate, up): the even lane finishes both
            const int out_n = pairs ? p.N >> 1 : p.N;    // width of the result
            const int out_n0 = pairs ? n0 >> 1 : n0;     // first result column of this tile
            const int out_col = pairs ? n >> 1 : n;      // this lane's result column
            const bool writer = n < p.N && !(pairs && (lane & 1));
            const __half *res = FUSED ? static_cast<const __half *>(p.ep.residual) : nullptr;
            const int m_left = p.M - m0;
            const bool cols_ok = out_n0 + chunk * 8 < out_n && !(pairs && chunk >= 8);  // widths are multiples of 8: eight columns are in or out together
            const size_t col_off = (size_t)p.out.col0 + out_n0 + chunk * 8;
#pragma unroll 1
            for (int cb = 0; cb < TM / 32; ++cb) {
                if (cb * 32 >= m_left) break;  // rows beyond M: nothing to store (uniform across the four warps)
                uint32_t v[32];
                tmem_ld_32x32(tmem_base + ((uint32_t)(32 * q) << 16) + buf * TM + cb * 32, v);
                tmem_ld_wait();
                __half *col = reinterpret_cast<__half *>(staging) + (pairs ? (32 * q + lane) >> 1 : 32 * q + lane);
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    float y = __uint_as_float(v[j]) * sc;
                    if (FUSED) y += bias;
                    if (pairs) {
                        const float up = __shfl_xor_sync(0xffffffffu, y, 1);
                        y = y / (1.0f + __expf(-y)) * up;
                    }
                    if (res != nullptr && writer && cb * 32 + j < m_left) y += __half2float(__ldg(res + (size_t)(m0 + cb * 32 + j) * p.ep.ldr + out_col));
                    if (writer) col[j * (STAGE_ROW_BYTES / 2)] = __float2half_rn(y);
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");  // the four epilogue warps: block complete
#pragma unroll
                for (int pass = 0; pass < 4; ++pass) {
                    const int r = pass * 8 + row_in_pass;
                    const int m = cb * 32 + r;
                    if (m < m_left && cols_ok) {
                        const uint4 val = *reinterpret_cast<const uint4 *>(staging + r * STAGE_ROW_BYTES + chunk * 16);
                        const size_t off = (size_t)(m0 + m) * p.out.ldc + col_off;
                        // every destination: this GPU's output and, for a column-parallel layer, the peer-mapped
                        // outputs of the other ranks (plain 16-byte stores over NVLink, no loads)
                        if (p.out.multicast) {
                            // one store to the multicast address: the switch delivers it to every GPU of the group
                            asm volatile("multimem.st.weak.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(static_cast<__half *>(p.out.ptr[0]) + off),
                                         "f"(__uint_as_float(val.x)), "f"(__uint_as_float(val.y)), "f"(__uint_as_float(val.z)), "f"(__uint_as_float(val.w))
                                         : "memory");
                        } else {
#pragma unroll 1
                            for (int d = 0; d < p.out.count; ++d) *reinterpret_cast<uint4 *>(static_cast<__half *>(p.out.ptr[d]) + off) = val;
                        }
                    }
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");  // staging may be overwritten
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&acc_empty[buf]));
        }
    }

    // ---------------- teardown: everyone is done with tensor memory ----------------
    tc_fence_before_sync();
    __syncthreads();
    if (warp == MMA_WARP) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
    }
}

// Adds the k_splits partial sums of every output element in split order, then does what the epilogue does: scale,
// bias, gate / up pairing, residual, one rounding, 16-byte stores to every destination.  A thread owns eight adjacent
// columns of one row.
__global__ void __launch_bounds__(256) qlinear_prefill_reduce_kernel(const float *__restrict__ partial, const __half *__restrict__ scale,
                                                                     OutTargets out, Epilogue ep, int M, int N, int k_splits) {
    const int64_t groups_per_row = N / 8;
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (int64_t)M * groups_per_row) return;
    const int m = (int)(idx / groups_per_row);
    const int n = (int)(idx - (int64_t)m * groups_per_row) * 8;
    float y[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) y[c] = 0.0f;
    const float *src = partial + (size_t)m * N + n;
    for (int sp = 0; sp < k_splits; ++sp) {
        const float4 v0 = __ldcg(reinterpret_cast<const float4 *>(src + (size_t)sp * M * N));
        const float4 v1 = __ldcg(reinterpret_cast<const float4 *>(src + (size_t)sp * M * N + 4));
        y[0] += v0.x, y[1] += v0.y, y[2] += v0.z, y[3] += v0.w;
        y[4] += v1.x, y[5] += v1.y, y[6] += v1.z, y[7] += v1.w;
    }
    const uint4 sraw = __ldg(reinterpret_cast<const uint4 *>(scale + n));
    const __half *sh = reinterpret_cast<const __half *>(&sraw);
#pragma unroll
    for (int c = 0; c < 8; ++c) y[c] *= __half2float(sh[c]);
    if (ep.bias != nullptr) {
        const uint4 braw = __ldg(reinterpret_cast<const uint4 *>(static_cast<const __half *>(ep.bias) + n));
        const __half *bh = reinterpret_cast<const __half *>(&braw);
#pragma unroll
        for (int c = 0; c < 8; ++c) y[c] += __half2float(bh[c]);
    }
    if (ep.act == kActSiluMul) {
        // columns (2j, 2j + 1) = (gate, up): four results per thread, result column n / 2 + j
        __half2 r2[2];
        float z[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            z[j] = y[2 * j] / (1.0f + __expf(-y[2 * j])) * y[2 * j + 1];
            if (ep.residual != nullptr) z[j] += __half2float(__ldg(static_cast<const __half *>(ep.residual) + (size_t)m * ep.ldr + (n >> 1) + j));
        }
        r2[0] = __floats2half2_rn(z[0], z[1]);
        r2[1] = __floats2half2_rn(z[2], z[3]);
        const uint2 val = *reinterpret_cast<const uint2 *>(r2);
        const size_t off = (size_t)m * out.ldc + out.col0 + (n >> 1);
        for (int d = 0; d < out.count; ++d) *reinterpret_cast<uint2 *>(static_cast<__half *>(out.ptr[d]) + off) = val;
        return;
    }
    if (ep.residual != nullptr) {
        const uint4 rraw = __ldg(reinterpret_cast<const uint4 *>(static_cast<const __half *>(ep.residual) + (size_t)m * ep.ldr + n));
        const __half *rh = reinterpret_cast<const __half *>(&rraw);
#pragma unroll
        for (int c = 0; c < 8; ++c) y[c] += __half2float(rh[c]);
    }
    __half2 h2[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) h2[c] = __floats2half2_rn(y[2 * c], y[2 * c + 1]);
    const uint4 val = *reinterpret_cast<const uint4 *>(h2);
    const size_t off = (size_t)m * out.ldc + out.col0 + n;
    if (out.multicast) {
        asm volatile("multimem.st.weak.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(static_cast<__half *>(out.ptr[0]) + off), "f"(__uint_as_float(val.x)),
                     "f"(__uint_as_float(val.y)), "f"(__uint_as_float(val.z)), "f"(__uint_as_float(val.w))
                     : "memory");
    } else {
        for (int d = 0; d < out.count; ++d) *reinterpret_cast<uint4 *>(static_cast<__half *>(out.ptr[d]) + off) = val;
    }
}

}  // namespace prefill

bool prefill_kn_supported(const void *a, const void *wq, int64_t N, int64_t K) {
    return (N % 16 == 0) && (K % 8 == 0) && ((reinterpret_cast<uintptr_t>(a) & 15u) == 0) &&
           ((reinterpret_cast<uintptr_t>(wq) & 15u) == 0);
}

// Height of the activation tile: 256 rows unless 64 rows fill more of
// the machine.  Cost model: waves of tiles over the SMs times the time of one tile, where the shorter
// tiles run the tensor core below its rate (more shared-memory traffic per flop).
static int choose_tile_m(int64_t M, int64_t N, int sms) {
    const int64_t n_tiles = ceil_div(N, prefill::TN);
    const int cand[2] = {256, 64};
    const double cost_per_row[2] = {1.0, 1.0 / 0.5};
    int best = 256;
    double best_cost = 0.0;
    for (int i = 0; i < 2; ++i) {
        const int64_t tiles = n_tiles * ceil_div(M, cand[i]);
        const double cost = (double)ceil_div(tiles, sms) * cand[i] * cost_per_row[i];
        if (i == 0 || cost < best_cost * 0.98) {
            best = cand[i];
            best_cost = cost;
        }
    }
    return best;
}

// Split K over several CTAs per output tile when 256-row tiles alone would occupy less than half of the SMs and
// there are enough k blocks to share out (a narrow column shard at a few hundred rows).  Splits come with 256-row
// tiles; every split gets at least eight k blocks.
PrefillSplit plan_prefill_split(int64_t M, int64_t N, int64_t K) {
    PrefillSplit ps;
    int sms = sm_count();
    if (sms <= 0) sms = 148;
    const int64_t tiles = ceil_div(N, prefill::TN) * ceil_div(M, 256);
    const int64_t k_blocks = ceil_div(K, prefill::BK);
    if (tiles * 2 > sms || k_blocks < 16 || N % 8 != 0) return ps;
    int64_t splits = sms / tiles;
    if (splits > k_blocks / 8) splits = k_blocks / 8;
    if (splits < 2) return ps;
    ps.kb_per_split = (int)ceil_div(k_blocks, splits);
    ps.k_splits = (int)ceil_div(k_blocks, ps.kb_per_split);
    if (ps.k_splits < 2) return PrefillSplit();
    ps.workspace_bytes = kSplitWorkspaceHead + (size_t)ps.k_splits * M * N * sizeof(float);
    return ps;
}

template <int TM>
static int launch_prefill_tm(const void *a, const void *wq, const void *scale, void *c, int64_t M, int64_t N, int64_t K,
                             cudaStream_t stream, const OutTargets *targets, const Epilogue *epilogue, int sms, bool weight_nk, int64_t lda,
                             const PrefillSplit &split, void *workspace) {
    using namespace prefill;
    using Cfg = Config<TM>;
    CUtensorMap map_w, map_a;
    int rc = weight_nk ? make_tensor_map_2d(&map_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, wq, (uint64_t)K, (uint64_t)N, (uint64_t)K, BK, TN,
                                            CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B)
                       : make_tensor_map_2d(&map_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, wq, (uint64_t)N, (uint64_t)K, (uint64_t)N, TN, BK,
                                            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
    if (rc != B200Q_OK) return rc;
    rc = make_tensor_map_2d(&map_a, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, a, (uint64_t)K, (uint64_t)M, (uint64_t)lda * 2, BK, TM,
                            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
    if (rc != B200Q_OK) return rc;

    Params p;
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
    if (p.ep.act == kActSiluMul && N % 16 != 0) return set_error(B200Q_INVALID_ARGUMENT, "qlinear: the gate / up pairing needs N to be a multiple of 16, got %lld", (long long)N);
    for (int d = 0; d < p.out.count; ++d)
        if ((reinterpret_cast<uintptr_t>(p.out.ptr[d]) & 15u) != 0) return set_error(B200Q_INVALID_ARGUMENT, "qlinear: output %d is not 16-byte aligned", d);
    if (p.out.ldc % 8 != 0 || p.out.col0 % 8 != 0) return set_error(B200Q_INVALID_ARGUMENT, "qlinear: output row length and column offset must be multiples of 8 elements");
    p.status = device_status_word();
    p.M = (int)M;
    p.N = (int)N;
    p.K = (int)K;
    p.n_tiles = (int)ceil_div(N, TN);
    p.m_tiles = (int)ceil_div(M, TM);
    p.k_splits = split.k_splits;
    p.kb_per_split = split.k_splits > 1 ? split.kb_per_split : (int)ceil_div(K, BK);
    p.partial = split.k_splits > 1 ? reinterpret_cast<float *>(static_cast<unsigned char *>(workspace) + kSplitWorkspaceHead) : nullptr;
    const int64_t total = (int64_t)p.n_tiles * p.m_tiles * p.k_splits;
    if (total > 2147483647LL) return set_error(B200Q_UNSUPPORTED, "qlinear: problem too large for the tile counter");
    const unsigned grid = (unsigned)(total < sms ? total : sms);

    static std::atomic<bool> attr_set[64];  // per device and instantiation, zero-initialised; a repeated set by a racing thread is harmless
    int dev = 0;
    B200Q_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !attr_set[dev].load(std::memory_order_acquire)) {
        B200Q_CUDA_TRY(cudaFuncSetAttribute(qlinear_prefill_kn_kernel<TM, false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
        B200Q_CUDA_TRY(cudaFuncSetAttribute(qlinear_prefill_kn_kernel<TM, true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
        B200Q_CUDA_TRY(cudaFuncSetAttribute(qlinear_prefill_kn_kernel<TM, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
        if (dev >= 0 && dev < 64) attr_set[dev].store(true, std::memory_order_release);
    }
    const bool fused = p.ep.bias != nullptr || p.ep.residual != nullptr || p.ep.act != kActNone;
    if (p.k_splits > 1) {
        // the splits write raw sums; the reduce kernel scales, applies the epilogue and delivers
        if (weight_nk) {
            qlinear_prefill_kn_kernel<TM, false, true><<<grid, THREADS, Cfg::SMEM_BYTES, stream>>>(map_w, map_a, p);
        } else {
            qlinear_prefill_kn_kernel<TM, false, false><<<grid, THREADS, Cfg::SMEM_BYTES, stream>>>(map_w, map_a, p);
        }
        B200Q_CHECK_LAUNCH("qlinear_prefill_kn_kernel");
        const int64_t threads = M * (N / 8);
        qlinear_prefill_reduce_kernel<<<(unsigned)ceil_div(threads, 256), 256, 0, stream>>>(p.partial, p.scale, p.out, p.ep, (int)M, (int)N, p.k_splits);
        B200Q_CHECK_LAUNCH("qlinear_prefill_reduce_kernel");
        return B200Q_OK;
    }
    if (weight_nk) {
        if (fused) return set_error(B200Q_UNSUPPORTED, "qlinear: the fused epilogue is served for [K, N] weights");
        qlinear_prefill_kn_kernel<TM, false, true><<<grid, THREADS, Cfg::SMEM_BYTES, stream>>>(map_w, map_a, p);
    } else if (fused) {
        qlinear_prefill_kn_kernel<TM, true, false><<<grid, THREADS, Cfg::SMEM_BYTES, stream>>>(map_w, map_a, p);
    } else {
        qlinear_prefill_kn_kernel<TM, false, false><<<grid, THREADS, Cfg::SMEM_BYTES, stream>>>(map_w, map_a, p);
    }
    B200Q_CHECK_LAUNCH("qlinear_prefill_kn_kernel");
    return B200Q_OK;
}

bool prefill_nk_supported(const void *a, const void *wq, int64_t N, int64_t K) {
    return (N % 8 == 0) && (K % 16 == 0) && ((reinterpret_cast<uintptr_t>(a) & 15u) == 0) && ((reinterpret_cast<uintptr_t>(wq) & 15u) == 0);
}

int launch_prefill_kn(const void *a, const void *wq, const void *scale, void *c, int64_t M, int64_t N, int64_t K,
                      cudaStream_t stream, const OutTargets *targets, const Epilogue *epilogue, bool weight_nk, int64_t lda,
                      void *workspace, size_t workspace_bytes) {
    if (lda <= 0) lda = K;
    int sms = sm_count();
    if (sms <= 0) sms = 148;
    // K is split only when the caller brought the scratch for it (the entry points without a workspace do not split).
    PrefillSplit split = plan_prefill_split(M, N, K);
    if (split.k_splits > 1 && (workspace == nullptr || workspace_bytes < split.workspace_bytes)) split = PrefillSplit();
    if (split.k_splits > 1 && targets != nullptr && targets->multicast && epilogue != nullptr && epilogue->act == kActSiluMul) split = PrefillSplit();
    if (split.k_splits > 1) {
        return launch_prefill_tm<256>(a, wq, scale, c, M, N, K, stream, targets, epilogue, sms, weight_nk, lda, split, workspace);
    }
    const int tm = choose_tile_m(M, N, sms);
    switch (tm) {
        case 64: return launch_prefill_tm<64>(a, wq, scale, c, M, N, K, stream, targets, epilogue, sms, weight_nk, lda, split, workspace);
        default: return launch_prefill_tm<256>(a, wq, scale, c, M, N, K, stream, targets, epilogue, sms, weight_nk, lda, split, workspace);
    }
}

}  // namespace b200q
