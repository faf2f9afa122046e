/*
 * hidet_b200q.h -- C ABI of libhidet_b200q.so
 *
 * Hand-written sm_100a (B200) kernels for Hidet's weight-only int8 quantized linear path:
 * symmetric quantize / dequantize, the absmax reduction behind them, and the f16 x int8
 * matmul that Hidet's quantization pass substitutes for fp16 matmul / linear.
 *
 * Conventions (they follow the reference's native runtime, src/hidet/runtime/logging.cpp:14-36
 * and include/hidet/runtime/common.h:16-18):
 *   - every entry point is extern "C" with default visibility, takes plain pointers and sizes,
 *     and launches asynchronously on the CUDA stream passed as `stream` (a cudaStream_t; NULL
 *     means the legacy default stream).  No entry point synchronises (b200q_check_status
 *     excepted), and none allocates or frees device memory;
 *   - the caller owns every buffer, outputs included (the reference allocates outputs before the
 *     call too: python/hidet/runtime/compiled_task.py:146-173);
 *   - every entry point returns a b200q_status.  On failure a thread-local message is kept and
 *     b200q_get_last_error() returns it and clears it (read-and-clear, like
 *     hidet_get_last_error).  Nothing aborts the process and no kernel traps.
 *   - the quantized-linear kernels are launched as programmatic dependents of the kernel in front of them
 *     in the stream: they request `wq` and `scale` BEFORE the stream dependency on that kernel is
 *     honoured (activations, outputs and scratch are touched only after it).  `wq` and `scale` must
 *     therefore be complete when the kernel in front may let its dependents start.  Ordinary kernels
 *     (every other kernel of this library, memcpy / memset nodes, anything that does not itself execute
 *     griddepcontrol.launch_dependents) let dependents start only when they have finished, so producing a
 *     weight with b200q_symmetric_quantize and using it in the next call on the same stream is safe.  Not
 *     safe: writing `wq` or `scale` from a kernel that triggers its dependents early when nothing but
 *     kernels of that kind lie between it and the quantized linear that reads them on the same stream (the
 *     quantized-linear kernels are themselves of that kind: they let the next kernel start while they
 *     run); put an event or any ordinary kernel between the two.
 *   - matrices are dense row-major.  "KN" weight layout = [K, N] with N contiguous, the layout of
 *     the reference operator (python/hidet/graph/ops/quant/matmul.py:30-32); "NK" = [N, K] with K
 *     contiguous, the layout torch.nn.Linear stores.
 */
#ifndef HIDET_B200Q_H
#define HIDET_B200Q_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define B200Q_API __attribute__((visibility("default")))
#else
#define B200Q_API
#endif

typedef enum b200q_status {
    B200Q_OK = 0,
    B200Q_INVALID_ARGUMENT = 1, /* null pointer, negative size, unknown enum value            */
    B200Q_UNSUPPORTED = 2,      /* a legal request that this build has no kernel for          */
    B200Q_WORKSPACE_TOO_SMALL = 3,
    B200Q_CUDA_ERROR = 4,       /* a CUDA runtime / driver call failed; message has the text  */
    B200Q_KERNEL_TIMEOUT = 5    /* a bounded device-side wait ran out (see b200q_check_status) */
} b200q_status;

/* element types of the floating-point side (weight before quantization, scale, dequantized weight) */
typedef enum b200q_float_type { B200Q_F16 = 0, B200Q_BF16 = 1, B200Q_F32 = 2 } b200q_float_type;
/* element types of the quantized side */
typedef enum b200q_quant_type { B200Q_I8 = 0, B200Q_I16 = 1 } b200q_quant_type;
/* memory layout of the int8 weight given to the matmul */
typedef enum b200q_weight_layout { B200Q_LAYOUT_KN = 0, B200Q_LAYOUT_NK = 1 } b200q_weight_layout;

/* Library version as major*10000 + minor*100 + patch. */
B200Q_API int b200q_version(void);

/* Message of the last failed call on this thread, or "" if none; clears it.
 * Counterpart of hidet_get_last_error (src/hidet/runtime/logging.cpp:29-36). */
B200Q_API const char *b200q_get_last_error(void);

/*
 * Symmetric quantization of a 2-D tensor w[rows, cols].
 * Replaces the three generated kernels of SymmetricQuantizationTask
 * (python/hidet/graph/ops/quant/symmetric.py:23-47): absmax reduction, scale, quantize.
 *
 *   reduce_dim = 0 : absmax over rows   -> scale[cols]  (Hidet dims=0, "per output channel" for a
 *                                                         [K, N] weight; the linear rewrite uses it)
 *   reduce_dim = 1 : absmax over cols   -> scale[rows]  (Hidet dims=-1, row-wise)
 *
 *   amax  = max |w|                      in w's own type
 *   scale = amax / qmax                  qmax = 127 (int8) or 32767 (int16), in w's own type
 *   wq    = (q_type) round(w / scale)    round = hrint (ties to even) for f16 / bf16,
 *                                                roundf (ties away from zero) for f32
 *
 * The arithmetic is the reference's, operation for operation, so wq and scale are bit-identical
 * to what the reference's kernels write.  scale has w's element type.
 */
B200Q_API int b200q_symmetric_quantize(const void *w, void *wq, void *scale, int64_t rows, int64_t cols,
                                       int w_type /* b200q_float_type */, int q_type /* b200q_quant_type */,
                                       int reduce_dim, void *stream);

/*
 * Symmetric dequantization w[r, c] = (scale_type) wq[r, c] * scale[reduce_dim == 0 ? c : r].
 * Replaces SymmetricDeQuantizationTask (python/hidet/graph/ops/quant/symmetric.py:50-61).
 */
B200Q_API int b200q_symmetric_dequantize(const void *wq, const void *scale, void *w, int64_t rows, int64_t cols,
                                         int scale_type /* b200q_float_type */, int q_type /* b200q_quant_type */,
                                         int reduce_dim, void *stream);

/*
 * Embedding lookup in a row-quantized table: out[i, :] = (scale_type) table[indices[i], :] * scale[indices[i]]
 * for table int8 / int16 [vocab, dim] quantized per row (b200q_symmetric_quantize with reduce_dim = 1) and
 * scale [vocab].  Replaces take(symmetric_dequantize(wq, scale, dims=-1), indices, axis=0), the graph the
 * reference's embedding rule builds (python/hidet/graph/transforms/graph_patterns/quant/embedding.py:22-39),
 * without materialising the dequantized table; every output row equals the row of the dequantized table
 * bit for bit.  index_bytes is 4 (int32) or 8 (int64), the index types the reference's rule accepts; a
 * negative index counts from the end; an index outside the table yields a row of zeros and is reported
 * by b200q_check_status.
 */
B200Q_API int b200q_embedding_dequantize(const void *table, const void *scale, const void *indices, void *out, int64_t vocab,
                                         int64_t dim, int64_t n_indices, int scale_type /* b200q_float_type */,
                                         int q_type /* b200q_quant_type */, int index_bytes, void *stream);

/*
 * Sub-byte weights (w4a16): 4-bit unsigned codes with per-group scales and optional zero points, the format of the
 * reference's CuTe test programs (tests/cute_kernel/quantized_linear.py:494-517, its check at
 * tests/cute_kernel/test_quant_linear.py:68-85):
 *     c[M, N] = a[M, K] x w[K, N],   w[k, n] = scale[k / G, n] * (q[k, n] - zeros[k / G, n])
 * a f16 [M, K]; q u4 [K, N] packed two codes per byte, element i of a row in bits 4 (i % 2) .. + 3 of byte i / 2
 * (the reference's sub-byte storage, python/hidet/transforms/lower_integer_subbyte.py:103-113), row-major, as
 * b200q_u4_pack / the reference's cast_f16_to_u4 produce it (not the kernel-private layout of its
 * preprocess_weight); scale, zeros f16 [K / G, N] (zeros may be NULL: w = scale * q); c f16 [M, N].
 * K must be a multiple of the group size G, N a multiple of 8.  Sums are fp32, the order of every sum is fixed.
 * The workspace (b200q_qlinear_f16_u4_workspace_bytes) holds fp32 partial sums behind an untouched head of 256 KB
 * (where b200q_qlinear_f16_i8 keeps its counters, so that one workspace can serve both) and needs no initialisation.
 */
B200Q_API size_t b200q_qlinear_f16_u4_workspace_bytes(int64_t M, int64_t N, int64_t K, int64_t group_size);
B200Q_API int b200q_qlinear_f16_u4(const void *a, const void *q, const void *scale, const void *zeros, void *c, int64_t M, int64_t N,
                                   int64_t K, int64_t group_size, void *workspace, size_t workspace_bytes, void *stream);

/*
 * u4 codes <-> f16: b200q_u4_pack converts f16 [rows, cols] to int the way C does and keeps the low four bits
 * (the reference's cast_f16_to_u4, tests/cute_kernel/quantized_linear.py:226-267), two codes per byte as above;
 * b200q_u4_unpack is the inverse (cast_u4_to_f16, :181-223).  cols must be even.
 */
B200Q_API int b200q_u4_pack(const void *w, void *packed, int64_t rows, int64_t cols, void *stream);
B200Q_API int b200q_u4_unpack(const void *packed, void *w, int64_t rows, int64_t cols, void *stream);

/*
 * Bytes of scratch b200q_qlinear_f16_i8 needs for this problem (0 is a valid answer).
 * The scratch must be zero-filled once before its first use; every call leaves it zero-filled in
 * the part that has to be (its tile counters), so the same buffer can serve later calls of any
 * shape whose requirement it covers.  Two calls that may overlap on the GPU need two buffers.
 * Counterpart of request_cuda_workspace(nbytes, require_clean)
 * (src/hidet/runtime/cuda/context.cpp:90-104).
 */
B200Q_API size_t b200q_qlinear_workspace_bytes(int64_t M, int64_t N, int64_t K, int w_layout);

/*
 * c[M, N] (f16) = a[M, K] (f16) x dequant(wq, scale), fp32 accumulation, scale applied to the fp32
 * sum, one rounding to f16.
 * Replaces symmetric_quant_matmul together with the resolve rule's
 * symmetric_quant_matmul_f16_i8(...).sum(0) (python/hidet/graph/ops/quant/matmul.py:83-93,
 * python/hidet/graph/ops/quant/resolve.py:23-100).  Leading batch dimensions of `a` are folded
 * into M by the caller (the weight is 2-D).
 *
 *   wq    : int8, [K, N] if w_layout == B200Q_LAYOUT_KN, [N, K] if B200Q_LAYOUT_NK
 *   scale : f16 [N]
 * Picks the small-M streaming kernel or the large-M tensor-core kernel from M.
 */
B200Q_API int b200q_qlinear_f16_i8(const void *a, const void *wq, const void *scale, void *c, int64_t M, int64_t N,
                                   int64_t K, int w_layout, void *workspace, size_t workspace_bytes, void *stream);

/*
 * What b200q_qlinear_f16_i8_fused does to the scaled fp32 sums y[m, n] before the one rounding to f16, in
 * this order:  y += bias[n];  the activation;  + residual[m, .].
 * B200Q_ACT_SILU_MUL is the SwiGLU pairing: the N columns of the weight come in pairs (gate_j, up_j) at
 * (2j, 2j + 1) -- a gate and an up projection [K, F] each, interleaved column by column into one [K, 2F]
 * weight (quantization is per column, so codes and scales are those of the two separate weights) -- and
 * the result is z[m, j] = silu(y[m, 2j]) * y[m, 2j + 1], N / 2 columns wide.
 */
typedef enum b200q_activation { B200Q_ACT_NONE = 0, B200Q_ACT_SILU_MUL = 1 } b200q_activation;
typedef struct b200q_epilogue {
    const void *bias;     /* f16 [N], or NULL                                                     */
    const void *residual; /* f16 [M, ldr], added to the result (after the activation), or NULL    */
    int64_t ldr;          /* elements between rows of residual; at least the width of the result  */
    int activation;       /* b200q_activation                                                     */
} b200q_epilogue;

/*
 * b200q_qlinear_f16_i8 with the element-wise operators that follow a linear layer applied inside the
 * kernel: c[M, N or N / 2] = epilogue(a x dequant(wq, scale)).  Takes the place of the reference's fusion of
 * those operators into its matmul by IR rewriting (python/hidet/graph/transforms/fuse_operator.py,
 * python/hidet/graph/ops/quant/matmul_f16_i8.py:95-99: the task allows an epilogue); the intermediate
 * values stay in fp32, so the result is rounded once where the unfused graph rounds after every operator.
 * [K, N] weights with 16-byte aligned bases and rows; workspace as for b200q_qlinear_f16_i8 with the same
 * M, N, K.  epilogue == NULL is b200q_qlinear_f16_i8.
 */
B200Q_API int b200q_qlinear_f16_i8_fused(const void *a, const void *wq, const void *scale, void *c, int64_t M, int64_t N,
                                         int64_t K, int w_layout, const b200q_epilogue *epilogue, void *workspace,
                                         size_t workspace_bytes, void *stream);

/*
 * The reference's explicit split-K form: c[p, M, N] (f16) = scale[n] * sum over the p-th K part of
 * a[m, k] * wq[k, n], parts of ceil(K / k_parts) consecutive k (the last may be short or empty).
 * The caller sums over p.  Replaces symmetric_quant_matmul_f16_i8
 * (python/hidet/graph/ops/quant/matmul_f16_i8.py:28-93, 501-511).  Each part is accumulated in
 * fp32 and rounded to f16 once.  KN layout only (the reference has no other).
 */
B200Q_API int b200q_qlinear_f16_i8_parts(const void *a, const void *wq, const void *scale, void *c, int64_t M,
                                         int64_t N, int64_t K, int k_parts, void *stream);

/*
 * The quantized linear of one rank of a column-parallel layer, delivering its result to every rank:
 * element (m, n) of a[M, K] x dequant(wq[K, N], scale[N]) is stored to
 * dst[i][m * ldc + col_offset + n] for each of the n_dst destinations (1 <= n_dst <= 8).  The
 * destinations are the [M, ldc] output buffers of the ranks, this rank's own included, given as
 * pointers valid on this device (peer-mapped for the other GPUs); the stores are plain peer stores
 * from the kernel's epilogue.  Replaces the matmul followed by the all-gather op of
 * python/hidet/graph/ops/distributed.py:63-97 (whose result is rank-major and needs a reshuffle).
 * The caller orders the ranks afterwards (a barrier between "all kernels done" and "outputs read").
 * `dst` is a host array.  KN layout; workspace as for b200q_qlinear_f16_i8 with the same M, N, K.
 * Both kernels store to every destination from their epilogue, tile by tile, so the delivery overlaps
 * the rest of the product; ldc and col_offset must be multiples of 8 and the destinations 16-byte aligned
 * when the large-M kernel serves the call.
 */
B200Q_API int b200q_qlinear_f16_i8_to_peers(const void *a, const void *wq, const void *scale, void *const *dst, int n_dst,
                                            int64_t ldc, int64_t col_offset, int64_t M, int64_t N, int64_t K, void *workspace,
                                            size_t workspace_bytes, void *stream);

/*
 * The same for large M through an NVLink multicast address: `multicast_dst` maps the [M, ldc] output buffers of all
 * ranks of the group at once (a multicast object over symmetric allocations, e.g. the multicast pointer of a
 * torch symmetric-memory handle), and the large-M kernel's epilogue stores every 16 bytes once with multimem.st;
 * the switch delivers them to every GPU, this one included.  The bytes that leave this GPU are 1 / (ranks - 1) of
 * what b200q_qlinear_f16_i8_to_peers sends.  M >= 33 and operands the large-M kernel accepts, else
 * B200Q_UNSUPPORTED (use b200q_qlinear_f16_i8_to_peers); workspace as for b200q_qlinear_f16_i8.  The caller orders the ranks
 * afterwards, as above.  No counterpart in the reference beyond the all-gather op named above.
 */
B200Q_API int b200q_qlinear_f16_i8_to_multicast(const void *a, const void *wq, const void *scale, void *multicast_dst, int64_t ldc,
                                                int64_t col_offset, int64_t M, int64_t N, int64_t K, void *workspace, size_t workspace_bytes,
                                                void *stream);

/*
 * Delivery by copies instead of epilogue stores (an alternative, not what the layer uses): copies columns
 * [col_offset, col_offset + cols) of the fp16 matrix src[rows, ld] into the same place of every
 * dst[i][rows, ld] (pointers valid on this device, peer-mapped for other GPUs; an entry equal to src
 * is skipped).  One strided device-to-device copy per destination, executed by the copy engines in
 * stream order; `dst` is a host array.  With b200q_qlinear_f16_i8_to_peers(n_dst = 1) in front it
 * takes the place of the all-gather op of python/hidet/graph/ops/distributed.py:63-97
 * (ncclAllGather, python/hidet/ir/primitives/cuda/nccl.py:62-73).
 */
B200Q_API int b200q_push_columns(const void *src, void *const *dst, int n_dst, int64_t rows, int64_t cols, int64_t ld,
                                 int64_t col_offset, void *stream);

/*
 * Bytes of the scratch array built into the library for b200q_qlinear_f16_i8_static (512 KiB).
 * No counterpart in the reference.
 */
B200Q_API size_t b200q_qlinear_static_scratch_bytes(void);

/*
 * b200q_qlinear_f16_i8 for callers that cannot provide scratch memory and cannot allocate any.
 * No counterpart in the reference (its generated launch functions ask the runtime for a workspace).
 *
 * Meant for code that only holds device pointers and a stream: the launch function of a compiled
 * graph, a plugin called from inside another runtime's loop, a process whose device memory is fully
 * pre-partitioned.  Such code has no allocator to turn to and must not call cudaMalloc itself (it
 * synchronises the device, can fail once memory is committed, and bypasses the host runtime's
 * bookkeeping).  This entry point allocates nothing: the scratch is a fixed 512 KiB array inside the
 * library's device image, held by every GPU that loads the library until the process exits.
 *
 *   - same operands and result as b200q_qlinear_f16_i8 with w_layout = B200Q_LAYOUT_KN; operands must
 *     have 16-byte aligned bases and rows (N % 16 == 0, K % 8 == 0).  (One exception to "same result": a
 *     narrow weight at M >= 33, where b200q_qlinear_f16_i8 splits K over several CTAs per tile and needs MBs
 *     of scratch for it, is computed here without the split: same value, fp32 sums grouped differently);
 *   - a problem whose scratch requirement (b200q_qlinear_workspace_bytes) exceeds the built-in array
 *     is refused with B200Q_WORKSPACE_TOO_SMALL and a message naming both sizes (most shapes need no
 *     scratch; narrow, deep weights with 16 or more activation rows can exceed the array);
 *   - the first call on a device looks up the array's device address (cudaGetSymbolAddress, with that
 *     device current) and sets kernel attributes: make that first call before any stream capture;
 *   - all calls on a device share the one array: calls that may overlap on the GPU (different
 *     streams, or host threads launching concurrently) race on it.  Calls ordered on one stream are safe.
 */
B200Q_API int b200q_qlinear_f16_i8_static(const void *a, const void *wq, const void *scale, void *c, int64_t M, int64_t N,
                                          int64_t K, int w_layout, void *stream);

/*
 * Device-side status word of the calling thread's current device: 0 if no bounded wait of any
 * kernel launched so far has run out.  Synchronises the device.  A non-zero value is returned as
 * B200Q_KERNEL_TIMEOUT with the details in the error message, and the word is cleared.
 */
B200Q_API int b200q_check_status(void);

#ifdef __cplusplus
}
#endif
#endif /* HIDET_B200Q_H */
