// Internal interface between the quantized-linear entry points and the kernels behind them.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace b200q {

// Where a kernel writes its result.  Element (m, n) of the result goes to
// ptr[i][m * ldc + col0 + n] for every i < count: one entry is the ordinary output; several entries
// are the same column block of output buffers on several GPUs (peer-mapped pointers), which is how a
// column-parallel layer delivers its slice to every rank without a separate all-gather.
constexpr int kMaxOutTargets = 8;
struct OutTargets {
    void *ptr[kMaxOutTargets] = {};
    int count = 0;
    int64_t ldc = 0;   // elements between consecutive rows of the destination
    int64_t col0 = 0;  // first destination column
    // ptr[0] is an NVLink multicast address (one store reaches the same place of every GPU bound to it, this one
    // included); count is 1.  Served by the large-M kernel only, whose epilogue then stores with multimem.st.
    int multicast = 0;
};

// What a kernel does to the scaled fp32 sums y[m, n] before the one rounding to f16:
//   y += bias[n];  activation (silu_mul: the weight's columns come in pairs (gate_j, up_j) = (2j, 2j + 1), and
//   z[m, j] = silu(y[m, 2j]) * y[m, 2j + 1] is the result, half as wide);  z += residual[m, j].
// Takes the place of the element-wise operators the reference fuses into its matmul by IR rewriting
// (python/hidet/graph/transforms/fuse_operator.py, python/hidet/graph/ops/quant/matmul_f16_i8.py:95-99).
constexpr int kActNone = 0;
constexpr int kActSiluMul = 1;
struct Epilogue {
    const void *bias = nullptr;      // f16 [N]
    const void *residual = nullptr;  // f16 [M, ldr]
    int64_t ldr = 0;                 // elements between rows of residual
    int act = kActNone;
};

// How the small-M kernel splits a problem over CTAs, and the scratch that split needs.
struct DecodePlan {
    int n_tiles = 0;
    int m_tiles = 0;
    int splits = 1;            // CTAs along K per output tile
    int cluster = 1;           // of them, this many form a thread-block cluster that needs no workspace
    int groups = 1;            // clusters per tile; > 1: the clusters meet in the workspace
    int iters_per_split = 0;   // 64-row k steps each of them takes
    size_t counter_bytes = 0;  // head of the workspace: one arrival counter per output tile
    size_t partial_bytes = 0;  // then [groups][M][N] fp32 partial sums (0 when groups == 1)
};

DecodePlan plan_decode(int64_t M, int64_t N, int64_t K);

// True when the TMA-based [K, N] kernel can take these operands (16-byte aligned bases and rows).
bool decode_kn_supported(const void *a, const void *wq, int64_t N, int64_t K);

// c[M, N] = scale * (a[:, k_begin:k_end] x wq[k_begin:k_end, :]).  K is the row length of `a`.
int launch_decode_kn(const void *a, const void *wq, const void *scale, void *c, int64_t M, int64_t N, int64_t K,
                     int64_t k_begin, int64_t k_end, bool allow_split, void *workspace, size_t workspace_bytes,
                     cudaStream_t stream, const OutTargets *targets = nullptr, const Epilogue *epilogue = nullptr, bool weight_nk = false);
// The same kernel on a weight stored [N, K] (weight_nk = true): needs 16-byte aligned bases and K % 16 == 0.
bool decode_nk_supported(const void *a, const void *wq, int64_t N, int64_t K);

// The tensor-memory kernel for large M: same operand requirements as the small-M kernel.
bool prefill_kn_supported(const void *a, const void *wq, int64_t N, int64_t K);
// How the tensor-memory kernel splits K (narrow problems only) and the scratch that takes: fp32 partial sums
// [k_splits][M][N] behind an untouched head of kSplitWorkspaceHead bytes (the small-M kernel's counters live there).
constexpr size_t kSplitWorkspaceHead = (size_t)65536 * 4;
struct PrefillSplit {
    int k_splits = 1;
    int kb_per_split = 0;
    size_t workspace_bytes = 0;
};
PrefillSplit plan_prefill_split(int64_t M, int64_t N, int64_t K);
// lda: elements between rows of `a` when they are longer than K (a k range of wider activations); 0 = K.
// workspace: where K may be split (see plan_prefill_split); without it the kernel runs one CTA per output tile.
int launch_prefill_kn(const void *a, const void *wq, const void *scale, void *c, int64_t M, int64_t N, int64_t K,
                      cudaStream_t stream, const OutTargets *targets = nullptr, const Epilogue *epilogue = nullptr, bool weight_nk = false,
                      int64_t lda = 0, void *workspace = nullptr, size_t workspace_bytes = 0);
// The same kernel on a weight stored [N, K] (weight_nk = true): 16-byte aligned bases, K % 16 == 0, N % 8 == 0.
bool prefill_nk_supported(const void *a, const void *wq, int64_t N, int64_t K);

// Which kernel serves M activation rows.  The tensor-memory kernel's tiles span 64 or 256 rows and it
// streams every weight tile once per row block; the small-M kernel re-streams the weight once per 16
// rows (from L2 after the first pass).  Up to 32 rows the small-M kernel always wins, up to 64 rows it
// still wins on weights of a few tens of MB.
constexpr int64_t kPrefillMinM = 33;
inline bool use_prefill_kernel(int64_t M, int64_t N, int64_t K) {
    if (M < kPrefillMinM) return false;
    if (M <= 64) return K * N > (int64_t)24 * 1024 * 1024;
    return true;
}

}  // namespace b200q
