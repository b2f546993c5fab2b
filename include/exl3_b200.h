/*
 * exl3_b200 — C ABI of the B200 (sm_100a) EXL3 fused dequant-matmul path.
 *
 * Drop-in boundary for the EXL3 linear-module path of PonyExl3: a host program
 * (PyTorch via ctypes, or any FFI) owns every buffer and passes plain device
 * pointers, sizes and a CUDA stream; nothing is allocated or freed in here and
 * there is no CPU fallback.  Every entry point validates its arguments on the
 * host before launching and returns 0 or a negative EXL3_E* code; kernels are
 * enqueued on `stream` and the call returns without synchronising.
 *
 * Data formats are the reference's (paths are inside the reference project):
 *   trellis  (in/16, out/16, 16*K) uint16, C order   ponyexl3/ref/layer.py:12-44
 *   suh/svh  (in,) / (out,) fp16 multipliers or NULL  ponyexl3/ref/signs.py:22-27
 *   bias     (out,) fp16 or NULL
 *   K        1..8 bits per weight; cb 0 = 3INST, 1 = MCG, 2 = MUL1
 *                                                      ponyexl3/ref/codebook.py:9-12,94-99
 * All fp16 buffers are passed as uint16_t* (bit patterns).
 */
#ifndef EXL3_B200_H
#define EXL3_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define EXL3_B200_VERSION 100

#if defined(__GNUC__)
#define EXL3_API __attribute__((visibility("default")))
#else
#define EXL3_API
#endif

/* error codes */
#define EXL3_OK 0
#define EXL3_E_NULL (-1)        /* a required pointer is NULL */
#define EXL3_E_K (-2)           /* K outside 1..8 */
#define EXL3_E_CODEBOOK (-3)    /* cb outside 0..2 */
#define EXL3_E_SHAPE (-4)       /* a dimension is zero, negative or not a multiple of 16 / 128 */
#define EXL3_E_ROWS (-5)        /* row count outside what the entry point supports */
#define EXL3_E_ALIGN (-6)       /* a pointer or stride is not aligned as required */
#define EXL3_E_WORKSPACE (-7)   /* workspace missing or too small */
#define EXL3_E_DTYPE (-8)       /* unknown activation dtype */
#define EXL3_E_CUDA (-9)        /* a CUDA runtime call failed (see exl3_last_cuda_error) */
#define EXL3_E_RANGE (-10)      /* an index or slice is out of range */
#define EXL3_E_UNSUPPORTED (-11)

/* activation dtypes */
#define EXL3_DT_F16 0
#define EXL3_DT_BF16 1
#define EXL3_DT_F32 2

/* flags */
#define EXL3_FLAG_PDL 1u        /* launch with programmatic stream serialisation so the next
                                   kernel's weight prefetch overlaps this kernel's tail */

#define EXL3_FLAG_FAST_ACCUM 2u /* 3INST / MCG only: keep the two fp16 halves of a codebook value
                                   apart and let the fp32 tensor-core accumulation add them,
                                   instead of rounding their sum to fp16 first.  Saves one
                                   instruction per weight; outputs move by < 2e-4 relative */

#define EXL3_FLAG_GLU_SILU 4u   /* exl3_gemv, exl3_gemv_blocks, exl3_gemv_noalloc, exl3_gemm_tiles: every x row holds */
#define EXL3_FLAG_GLU_GELU 8u   /* [gate (in) | up (in)] (x_row_stride >= 2*in) and the layer's input is
                                   fp16(silu(gate) * up) / fp16(gelu_tanh(gate) * up), computed while x
                                   is read: the down projection of a gated MLP or of a SwitchGLU takes
                                   the gate|up output as it is, with no activation launch in between
                                   (the reference folds the GLU into its down kernel the same way,
                                   ponyexl3/mlx/exl3_moe.py:374-422; activations :62-75) */

typedef void* exl3_stream_t;    /* cudaStream_t */

EXL3_API int exl3_version(void);
EXL3_API const char* exl3_error_string(int code);
/* Text of the last CUDA runtime error seen by this thread inside the library. */
EXL3_API const char* exl3_last_cuda_error(void);

/* ---- codec pieces (tests, debugging; reference: ponyexl3/ref) ------------------------- */

/* Packed tiles -> 256 uint16 codewords per tile.
 * Replaces unpack_trellis, ponyexl3/ref/trellis.py:205-214 (Metal twin
 * exl3_unpack_trellis_k{K}_v2, ponyexl3/mlx/metal_kernels.py:59-87). */
EXL3_API int exl3_unpack(const uint16_t* trellis, int64_t n_tiles, int k, uint16_t* codewords,
                exl3_stream_t stream);

/* Packed trellis -> inner weight matrix W (16*t_in rows, ld columns) fp16, out-tiles
 * [tn0, tn0+tn_count).  Bit-exact with decode_packed_trellis, ponyexl3/ref/decode.py:32-81 /
 * reconstruct_inner, ponyexl3/ref/reconstruct.py:13-23.  A test and debugging aid: the
 * matmul entry points never materialise W. */
EXL3_API int exl3_decode(const uint16_t* trellis, int64_t t_in, int64_t t_out, int k, int cb, int64_t tn0,
                int64_t tn_count, uint16_t* w, int64_t ld, exl3_stream_t stream);

/* All 65,536 codewords of a codebook -> fp16.  decode_3inst, ponyexl3/ref/codebook.py:66-91. */
EXL3_API int exl3_codebook_table(int cb, uint16_t* table65536, exl3_stream_t stream);

/* out = fp16( ((x * pre) @ H128 / sqrt(128)) * post ) per 128-wide block of the last
 * dimension; pre/post fp16 vectors of length n or NULL; x rows are x_row_stride elements
 * apart.  Replaces had_r_128, ponyexl3/ref/hadamard.py:50-80 (runtime twin prepare_xh /
 * finish_y, ponyexl3/mlx/layer_state.py:121-141). */
EXL3_API int exl3_hadamard128(const void* x, int x_dtype, int64_t rows, int64_t n, int64_t x_row_stride,
                     const uint16_t* pre, const uint16_t* post, uint16_t* out,
                     exl3_stream_t stream);

/* ---- workspace ------------------------------------------------------------------------- */

/* Bytes of scratch the matmul entry points need for activations of up to `max_rows` rows
 * (counting every member of a sibling group and every MoE slot) and `max_in` input
 * features: a status word, the arrival counters and fp32 partial sums of column blocks that
 * the streamed GEMV splits over several CTAs, and the rotated activations.  The caller
 * allocates it (256-byte aligned) and calls exl3_workspace_init once before first use (the
 * counters must start at zero; every launch leaves them at zero); calls that share a
 * workspace must be ordered on one stream.  A workspace larger than asked for is fine; one
 * that is smaller but still holds the activations only makes the GEMV use fewer CTAs. */
EXL3_API size_t exl3_workspace_bytes(int64_t max_rows, int64_t max_in);
EXL3_API int exl3_workspace_init(void* workspace, size_t bytes, exl3_stream_t stream);
/* Device-side status word of the workspace (0 = no kernel reported a bounded wait giving
 * up); copies it to *status_out after synchronising the stream. */
EXL3_API int exl3_workspace_status(const void* workspace, int* status_out, exl3_stream_t stream);

/* ---- the linear forward ------------------------------------------------------------------ */

/* y[rows, out] = fp16( had( fp16( fp16(had(x * suh)) @ W ) ) * svh ) + bias, rows 1..16:
 * the decode-time GEMV (rows = 1) and the small-batch verify GEMV (2..16).  The packed
 * trellis is streamed once, decoded in registers, accumulated in fp32.
 * Replaces EXL3Linear.__call__ rows<=16, ponyexl3/mlx/exl3_linear.py:98-136, i.e.
 * prepare_xh + inner_gemv_mlx / inner_gemm_mlx (ponyexl3/mlx/gemv_metal.py:1340-1478) +
 * finish_y; contract linear_forward_reconstruct, ponyexl3/ref/forward.py:14-49.
 * x rows are x_row_stride elements apart; y rows are y_row_stride elements apart. */
EXL3_API int exl3_gemv(const void* x, int x_dtype, int rows, int64_t x_row_stride, const uint16_t* trellis,
              int64_t t_in, int64_t t_out, int k, int cb, const uint16_t* suh, const uint16_t* svh,
              const uint16_t* bias, uint16_t* y, int64_t y_row_stride, void* workspace,
              size_t workspace_bytes, unsigned flags, exl3_stream_t stream);

/* The streamed GEMV over a TABLE of 128-column blocks, for sibling groups and stacked MoE
 * experts: block b multiplies `rows` rows of the rotated activations starting at row
 * blocks[b].xrow with the trellis columns of physical block blocks[b].phys, scales with
 * svh / adds bias at element offset blocks[b].sv_off (-1 = none) and stores its 128 outputs at
 * element offset blocks[b].y_off of each y row.  `blocks` is a device array of n_blocks x
 * {int32 phys, xrow, sv_off, y_off}.
 * The rotated activations are xh_rows rows: row i = had(x[row_src[i]] * suh[suh_row[i]]),
 * row_src / suh_row device int32 arrays or NULL (identity / row 0); suh is a (n, in) matrix.
 * raw_out != 0 stores fp16(x @ W) without output rotation.
 * Replaces the tile_map / tile_sub indirection of the reference's mapped GEMV:
 * FusedEXL3Group.forward_all, ponyexl3/mlx/exl3_fused.py:136-202, and
 * EXL3SwitchGLU._decode, ponyexl3/mlx/exl3_moe.py:634-683 (_mapped_gemv). */
EXL3_API int exl3_gemv_blocks(const void* x, int x_dtype, int64_t x_row_stride, int64_t xh_rows,
                     const int32_t* row_src, const uint16_t* suh, const int32_t* suh_row,
                     const uint16_t* trellis, int64_t t_in, int64_t t_out_total, int k, int cb,
                     const int32_t* blocks, int64_t n_blocks, int rows, const uint16_t* svh,
                     const uint16_t* bias, uint16_t* y, int64_t y_row_stride, int raw_out,
                     void* workspace, size_t workspace_bytes, unsigned flags, exl3_stream_t stream);

/* exl3_gemv_blocks with the number of blocks in use read from the device: *n_blocks_dev
 * (int32, written by an earlier kernel of the stream, clamped to 0..max_blocks) blocks of the
 * table are computed; the launch is planned for max_blocks, so nothing about it depends on a
 * value the host has not seen (expert-parallel SwitchGLU, exl3_moe_decode_tables_range). */
EXL3_API int exl3_gemv_blocks_counted(const void* x, int x_dtype, int64_t x_row_stride, int64_t xh_rows,
                             const int32_t* row_src, const uint16_t* suh, const int32_t* suh_row,
                             const uint16_t* trellis, int64_t t_in, int64_t t_out_total, int k, int cb,
                             const int32_t* blocks, int64_t max_blocks, const int32_t* n_blocks_dev, int rows,
                             const uint16_t* svh, const uint16_t* bias, uint16_t* y, int64_t y_row_stride,
                             int raw_out, void* workspace, size_t workspace_bytes, unsigned flags,
                             exl3_stream_t stream);

/* Same contract for any number of rows (prefill): the packed tiles are decoded to fp16 in
 * shared memory and multiplied on the tensor cores (tcgen05.mma, fp32 accumulators in tensor
 * memory) against TMA-staged rotated activations; W is never materialised in global memory.
 * Replaces the rows > 16 branches of EXL3Linear.__call__, ponyexl3/mlx/exl3_linear.py:137-161
 * (decode_full_mlx + matmul, ponyexl3/mlx/gemv_metal.py:630-774, and the striped path).
 * The workspace holds the rotated activations: exl3_gemm_workspace_bytes(rows, in). */
EXL3_API size_t exl3_gemm_workspace_bytes(int64_t rows, int64_t in);
EXL3_API int exl3_gemm(const void* x, int x_dtype, int64_t rows, int64_t x_row_stride, const uint16_t* trellis,
              int64_t t_in, int64_t t_out, int k, int cb, const uint16_t* suh, const uint16_t* svh,
              const uint16_t* bias, uint16_t* y, int64_t y_row_stride, void* workspace,
              size_t workspace_bytes, unsigned flags, exl3_stream_t stream);

/* The tensor-core GEMM over a TABLE of output tiles, for stacked MoE experts at prefill:
 * (token, slot) pairs are sorted by expert, so each expert owns a contiguous run of rows of
 * the rotated activations; tile t multiplies rows [row0, row_end) (at most 256) with the 256
 * trellis columns starting at tile column tn0, scales with svh at element offset sv_off and
 * stores ncols (128 or 256) outputs at column y_col of y rows (row + y_row_delta).
 * `tiles` is a device array of n_tiles x {int32 row0, row_end, tn0, sv_off, y_col, ncols,
 * y_row_delta, 0}; a slot with row0 >= row_end is skipped, so the table can be built on the
 * device with a fixed upper bound and no host synchronisation.  Rotated row i =
 * had(x[row_src[i]] * suh[suh_row[i]]) as in exl3_gemv_blocks.  y_row_map (may be NULL): the
 * y row that computed row r + y_row_delta is stored to — the last projection of a MoE call
 * writes straight back into (token, slot) order instead of sorted order.
 * Replaces the segmented trellis GEMM of the reference, inner_mm_seg_mlx with its expert block
 * table, ponyexl3/mlx/gemv_metal.py:1519-1741 and ponyexl3/mlx/exl3_moe.py:79-99,685-768. */
EXL3_API int exl3_gemm_tiles(const void* x, int x_dtype, int64_t x_row_stride, int64_t xh_rows,
                    const int32_t* row_src, const uint16_t* suh, const int32_t* suh_row,
                    const uint16_t* trellis, int64_t t_in, int64_t t_out_total, int k, int cb,
                    const int32_t* tiles, int64_t n_tiles, const uint16_t* svh, uint16_t* y,
                    int64_t y_row_stride, const int32_t* y_row_map, void* workspace, size_t workspace_bytes,
                    unsigned flags, exl3_stream_t stream);

/* exl3_gemm_tiles for expert parallelism.  xh_rows_dev (may be NULL): device int32 with the
 * number of rotated rows in use, at most xh_rows (only those are rotated; the tile table refers
 * to no others).  n_peers > 0: the output rows are spread over n_peers GPUs — y_row_map is
 * required and gives a GLOBAL row, row r lives in row r % rows_per_peer of the buffer
 * y_peers[r / rows_per_peer] (host array of device addresses, peer-mapped, y_row_stride apart);
 * the epilogue stores straight into the owner's memory, and when the whole grid has stored its
 * tiles every GPU's arrival counter (counter_peers, as in exl3_gemv_peers) gets one arrival, so
 * a GPU's rows are complete after n_peers arrivals (exl3_peer_wait).  y is ignored then.
 * EXL3_FLAG_GLU_* as in exl3_gemv: x rows are [gate | up]. */
EXL3_API int exl3_gemm_tiles_peers(const void* x, int x_dtype, int64_t x_row_stride, int64_t xh_rows,
                          const int32_t* xh_rows_dev, const int32_t* row_src, const uint16_t* suh,
                          const int32_t* suh_row, const uint16_t* trellis, int64_t t_in, int64_t t_out_total, int k,
                          int cb, const int32_t* tiles, int64_t n_tiles, const uint16_t* svh, uint16_t* y,
                          int64_t y_row_stride, const int32_t* y_row_map, const uint64_t* y_peers,
                          const uint64_t* counter_peers, int n_peers, int64_t rows_per_peer, void* workspace,
                          size_t workspace_bytes, unsigned flags, exl3_stream_t stream);

/* exl3_gemv without a caller-supplied workspace, for callers that cannot allocate device
 * memory: operator slots of a serving framework or thin language bindings that are handed
 * input and output buffers but own no allocator, and decode loops where cudaMalloc is
 * forbidden or all free memory already belongs to someone else's pool.
 * This entry point has no counterpart in the reference (unified memory there makes the
 * question moot); it is an addition of this library.
 *   - The scratch (status word, split-block counters and partial sums, rotated activations)
 *     is a fixed device array inside the library, 5.75 MiB + 2304 B per GPU, held from
 *     library load until the process exits.
 *   - Limit: rows * in_features <= 262,144 (e.g. 16 rows x 16,384 features); larger calls
 *     return EXL3_E_RANGE and launch nothing.
 *   - The first call on each device looks up the array's device address; make that first
 *     call outside any stream capture.
 *   - No cudaMalloc / cudaFree or allocating library routine is called.
 *   - All calls on a device share the one array: calls that overlap on the GPU (different
 *     streams) race on it; order them on one stream.  The array keeps the previous call's
 *     contents; each call rewrites what it reads, and the status word stays sticky.
 * Arguments and results are those of exl3_gemv. */
EXL3_API int exl3_gemv_noalloc(const void* x, int x_dtype, int rows, int64_t x_row_stride,
                               const uint16_t* trellis, int64_t t_in, int64_t t_out, int k, int cb,
                               const uint16_t* suh, const uint16_t* svh, const uint16_t* bias,
                               uint16_t* y, int64_t y_row_stride, unsigned flags,
                               exl3_stream_t stream);
/* Status word of that built-in scratch (the caller never sees the array, so
 * exl3_workspace_status cannot be used): 0 = no bounded wait of an exl3_gemv_noalloc kernel
 * ever gave up on this device.  Synchronises the stream.  No counterpart in the reference. */
EXL3_API int exl3_gemv_noalloc_status(int* status_out, exl3_stream_t stream);

/* ---- the caller's side of a decode step --------------------------------------------------
 * What sits between the EXL3 linears of a transformer layer during generation.  The reference
 * leaves these to its array framework inside the model graphs it patches (mlx.fast.rms_norm,
 * mlx.fast.rope, mlx.fast.scaled_dot_product_attention; linears installed at
 * ponyexl3/mlx/model.py:628-634), so they replace no reference code of the path; they exist so
 * that a whole decode step can run as a short train of launches.  fp16 tensors, fp32 math,
 * head_dim 128, device pointers, nothing allocated.  flags: EXL3_FLAG_PDL launches the kernel
 * with programmatic stream serialization (it may start while its predecessor drains; it waits
 * for the predecessor's results before touching memory). */

/* x <- fp16(x + delta) (delta NULL: no add); h <- fp16(x * rsqrt(mean(x^2) + eps) * weight).
 * rows x n, n a multiple of 8, pointers 16-byte aligned, strides in elements (multiples of 8). */
EXL3_API int exl3_add_rmsnorm(uint16_t* x, const uint16_t* delta, const uint16_t* weight, uint16_t* h,
                              int rows, int64_t n, int64_t x_row_stride, int64_t delta_row_stride,
                              int64_t h_row_stride, float eps, unsigned flags, exl3_stream_t stream);

/* qkv row r = [q_heads | kv_heads | kv_heads] x 128.  q and k get the rotate-half rotary
 * embedding with rows r of cos_table / sin_table (rows x 128); q -> q_out (rows, q_heads, 128),
 * k and v -> row pos0 + r of their head in the caches (kv_heads, cache_len, 128). */
EXL3_API int exl3_rope_append(const uint16_t* qkv, int64_t qkv_row_stride, const uint16_t* cos_table,
                              const uint16_t* sin_table, uint16_t* q_out, uint16_t* k_cache,
                              uint16_t* v_cache, int rows, int q_heads, int kv_heads, int64_t cache_len,
                              int pos0, unsigned flags, exl3_stream_t stream);

/* Grouped-query attention of `rows` (1..16) new positions over caches that already hold them:
 * position r sees keys 0 .. ctx + r.  q (rows, q_heads, 128) -> out (rows, q_heads * 128).
 * (q_heads / kv_heads) * rows <= 128.  Workspace from exl3_attn_workspace_bytes, 16-byte aligned;
 * the size does not grow with total_keys (it is the bound over all context lengths), so one
 * workspace sized once serves a whole generation. */
EXL3_API size_t exl3_attn_workspace_bytes(int rows, int q_heads, int kv_heads, int64_t total_keys);
EXL3_API int exl3_attn_decode(const uint16_t* q, const uint16_t* k_cache, const uint16_t* v_cache,
                              uint16_t* out, int rows, int q_heads, int kv_heads, int64_t cache_len, int ctx,
                              void* workspace, size_t workspace_bytes, unsigned flags, exl3_stream_t stream);

/* gate_up row = [gate (h) | up (h)]; out = fp16(silu(gate) * up).  h a multiple of 8. */
EXL3_API int exl3_swiglu(const uint16_t* gate_up, int64_t gu_row_stride, uint16_t* out, int64_t out_row_stride,
                         int rows, int64_t h, unsigned flags, exl3_stream_t stream);

/* ---- output exchange over peer memory (tensor parallel by output tile) -------------------
 * The reference is single-device; sharding a linear by output tile (ponyexl3/ref/reconstruct.py:13-23
 * decodes any 128-aligned column range on its own) needs the slices of a row gathered on every GPU
 * before the next layer.  These entry points do that with plain loads and stores over NVLink: the
 * caller maps every rank's full-row buffer and arrival counter into every process (one process per
 * GPU) and passes the W device pointers as HOST arrays.
 *
 * exl3_gemv_peers: exl3_gemv whose epilogue stores each finished 128-column block at column
 *   col0 + block * 128 of EVERY rank's (rows, full_row_stride) buffer; the CTA that finishes the
 *   rank's last block then adds 1 to every rank's counter (one system-scope release per launch).
 *   A rank's full row is complete when its counter has grown by n_peers.
 * exl3_peer_allgather: the same exchange for a (rows, cols) slice computed by other kernels;
 *   one arrival per rank, so the full row is complete after n_peers arrivals.
 * exl3_peer_wait: one-thread kernel that polls this rank's counter until `target` arrivals are
 *   there, subtracts them again and ends.  The poll gives up after about a second and sets the
 *   value 16 (mask 0x10) in the status word of `workspace` (exl3_workspace_status).  A (buffer, counter) pair must not be
 *   the target of two consecutive exchanges: rotate over at least two pairs. */
EXL3_API int exl3_gemv_peers(const void* x, int x_dtype, int rows, int64_t x_row_stride,
                             const uint16_t* trellis, int64_t t_in, int64_t t_out, int k, int cb,
                             const uint16_t* suh, const uint16_t* svh, const uint16_t* bias,
                             const uint64_t* y_peers, const uint64_t* counter_peers, int n_peers,
                             int64_t full_row_stride, int64_t col0, void* workspace, size_t workspace_bytes,
                             unsigned flags, exl3_stream_t stream);
/* exl3_gemv_peers that FIRST waits for its own input: x is a row that the previous exchange
 * completes on this rank, and instead of a separate exl3_peer_wait launch the kernel itself waits
 * (bounded, same status value 16) until *wait_counter has grown by wait_target, then takes the
 * arrivals off again; one kernel boundary per layer less.  Only the kernel that reads x can do
 * that: when the call needs the separate rotation kernel (more rows than the fused rotation takes)
 * the function launches nothing and returns EXL3_E_UNSUPPORTED — run exl3_peer_wait and
 * exl3_gemv_peers instead.  No counterpart in the reference (single device). */
EXL3_API int exl3_gemv_peers_after(const void* x, int x_dtype, int rows, int64_t x_row_stride,
                                   const uint16_t* trellis, int64_t t_in, int64_t t_out, int k, int cb,
                                   const uint16_t* suh, const uint16_t* svh, const uint16_t* bias,
                                   const uint64_t* y_peers, const uint64_t* counter_peers, int n_peers,
                                   int64_t full_row_stride, int64_t col0, uint32_t* wait_counter,
                                   uint32_t wait_target, void* workspace, size_t workspace_bytes,
                                   unsigned flags, exl3_stream_t stream);
EXL3_API int exl3_peer_allgather(const uint16_t* src, int rows, int64_t cols, int64_t src_row_stride,
                                 const uint64_t* dst_peers, const uint64_t* counter_peers, int n_peers,
                                 int64_t dst_row_stride, int64_t col0, unsigned flags, exl3_stream_t stream);
EXL3_API int exl3_peer_wait(uint32_t* counter, uint32_t target, void* workspace, unsigned flags,
                            exl3_stream_t stream);

/* ---- stacked-expert SwitchGLU, decode-class calls -------------------------------------------
 * Builds, on the device, the tables exl3_gemv_blocks takes for the two launches of a
 * SwitchGLU call with few tokens (the reference maps (token, slot) pairs to experts for its
 * mapped GEMV in the same way, ponyexl3/mlx/exl3_moe.py:634-683).  indices: n_pairs expert ids
 * (int32 or int64: index_bytes 4 or 8), pair s = token s / top_k.  Stacked layouts as in the
 * reference: gu_trellis (d/16, E*2*h/16, 16K) = all gates then all ups, gu_suh (E*2, d),
 * gu_svh (E, 2h), dn_trellis (h/16, E*d/16, 16K), dn_suh (E, h), dn_svh (E, d).
 *   blocks_gu (n_pairs*2*h/128, 4), row_src_gu (2*n_pairs), suh_row_gu (2*n_pairs): the gate/up
 *     launch over 2*n_pairs rotated rows (row 2s+p = pair s, p = 0 gate / 1 up), output
 *     (n_pairs, 2h) = [gate | up] per pair;
 *   blocks_dn (n_pairs*d/128, 4), suh_row_dn (n_pairs): the down launch, output (n_pairs, d). */
EXL3_API int exl3_moe_decode_tables(const void* indices, int index_bytes, int n_pairs, int top_k,
                                    int num_experts, int64_t d, int64_t h, int32_t* blocks_gu,
                                    int32_t* row_src_gu, int32_t* suh_row_gu, int32_t* blocks_dn,
                                    int32_t* suh_row_dn, unsigned flags, exl3_stream_t stream);

/* Expert parallelism (the stacked tensors passed to the GEMV hold only experts expert_lo ..
 * expert_hi-1 of num_experts; indices stay global): only the pairs routed to a held expert get
 * blocks, packed to the front of both tables in pair order, and the numbers of blocks in use are
 * left in counts[0] (gate/up) and counts[1] (down), a device int32[2], for
 * exl3_gemv_blocks_counted.  Rows and output offsets keep the numbering of ALL pairs, so the
 * output rows of pairs computed on another GPU are never written (the caller zero-fills them
 * and sums the ranks' outputs).  n_pairs <= 2048.  Nothing comes back to the host: the whole
 * call can be captured in a CUDA graph.  The reference has no multi-device path; the pair ->
 * expert mapping is the one of ponyexl3/mlx/exl3_moe.py:634-683. */
EXL3_API int exl3_moe_decode_tables_range(const void* indices, int index_bytes, int n_pairs, int top_k,
                                          int num_experts, int expert_lo, int expert_hi, int64_t d, int64_t h,
                                          int32_t* blocks_gu, int32_t* row_src_gu, int32_t* suh_row_gu,
                                          int32_t* blocks_dn, int32_t* suh_row_dn, int32_t* counts,
                                          unsigned flags, exl3_stream_t stream);

/* Prefill-class SwitchGLU tables, built on the device by one kernel (no host round trip): the
 * n_pairs (token, slot) pairs are grouped by expert (a counting sort; the order inside an expert
 * is not fixed, rows are independent), cut into row tiles of at most 256 pairs that never straddle
 * two experts, and expanded into the tile tables exl3_gemm_tiles takes — the reference builds the
 * same expert block table on the host, ponyexl3/mlx/exl3_moe.py:79-99,685-768.
 *   order (n_pairs): sorted position -> pair (the y_row_map of the down launch);
 *   row_src_gu, suh_row_gu (2*n_pairs): the rotated rows of the gate/up launch; an expert with
 *     sorted positions [seg, seg + cnt) has its gate rows at [2 seg, 2 seg + cnt) and its up rows
 *     at [2 seg + cnt, 2 seg + 2 cnt), and both kinds of tiles store to the [gate | up] row of
 *     the sorted position;
 *   suh_row_dn (n_pairs); tiles_gu (2 * slots * ceil(h/256), 8): gate tiles then up tiles;
 *   tiles_dn (slots * ceil(d/256), 8); slots = n_pairs / 256 + num_experts (unused ones are empty).
 * n_pairs <= 2^20, num_experts <= 1024. */
EXL3_API int exl3_moe_prefill_tables(const void* indices, int index_bytes, int n_pairs, int top_k,
                                     int num_experts, int64_t d, int64_t h, int32_t* order,
                                     int32_t* row_src_gu, int32_t* suh_row_gu, int32_t* suh_row_dn,
                                     int32_t* tiles_gu, int32_t* tiles_dn, unsigned flags,
                                     exl3_stream_t stream);

/* Expert parallelism, many tokens (every GPU sees all tokens' routing, the stacked tensors hold
 * experts expert_lo .. expert_hi-1 of num_experts): only the pairs routed to a held expert are
 * sorted and tiled; counts (device int32[2]) receives the rotated gate/up rows in use (2 x held
 * pairs) and the sorted positions in use, for exl3_gemm_tiles_peers.  slots = n_pairs / 256 +
 * (expert_hi - expert_lo). */
EXL3_API int exl3_moe_prefill_tables_range(const void* indices, int index_bytes, int n_pairs, int top_k,
                                           int num_experts, int expert_lo, int expert_hi, int64_t d, int64_t h,
                                           int32_t* order, int32_t* row_src_gu, int32_t* suh_row_gu,
                                           int32_t* suh_row_dn, int32_t* tiles_gu, int32_t* tiles_dn,
                                           int32_t* counts, unsigned flags, exl3_stream_t stream);

/* ---- trellis encoder (the converter's side of the format) -----------------------------------
 * Exact Viterbi search of 16x16 tiles over the bitshift trellis with tail-biting closure:
 * quantize_tile_reference, ponyexl3/convert/reference_search.py:30-87 (float64 path costs, first
 * minimum wins: the chosen states are bit-identical to the reference's).
 * w: (n_tiles, 256) float32 in codeword order (ponyexl3/convert/direct.py:409-420 maps a weight
 * matrix to it); states: (n_tiles, 256) the 16-bit window of every codeword; packed (may be
 * NULL): (n_tiles, 16K) the packed tiles as stored on disk (pack_trellis_tile,
 * ponyexl3/ref/trellis.py:12-50).  max_pins: pinned passes after the free one (the reference's
 * default is 4).  The workspace holds float64 costs and back-pointers of the tiles in flight,
 * 17 MiB each: exl3_encode_workspace_bytes(n_tiles) is enough for one tile per SM; a smaller
 * workspace (at least one slot) only lowers the number of tiles in flight. */
EXL3_API size_t exl3_encode_workspace_bytes(int64_t n_tiles);
EXL3_API int exl3_encode_tiles(const float* w, int64_t n_tiles, int k, int cb, int max_pins, uint16_t* states,
                               uint16_t* packed, void* workspace, size_t workspace_bytes, exl3_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* EXL3_B200_H */
