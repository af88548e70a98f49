/*
 * wush_b200 -- C ABI of the B200 (sm_100a) kernels for the WUSH quantized-linear hot path.
 *
 * Every entry point takes caller-owned DEVICE pointers plus sizes and a CUDA stream
 * (passed as void*, i.e. a cudaStream_t / CUstream handle; NULL is the legacy default
 * stream).  Calls are asynchronous with respect to the host unless stated otherwise.
 * Return value: 0 on success, a negative WUSH_ERR_* code for a rejected argument, or a
 * positive cudaError_t value reported by the CUDA runtime for the launch.
 *
 * Reference interfaces are cited by their path inside the WUSH project
 * (https://github.com/IST-DASLab/WUSH).
 */
#ifndef WUSH_B200_H_
#define WUSH_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define WUSH_API __attribute__((visibility("default")))
#else
#define WUSH_API
#endif

#define WUSH_OK 0
#define WUSH_ERR_NULL_POINTER (-1)
#define WUSH_ERR_BAD_SHAPE (-2)
#define WUSH_ERR_BAD_ALIGNMENT (-3)
#define WUSH_ERR_BAD_FLAG (-4)
#define WUSH_ERR_WORKSPACE_TOO_SMALL (-5)
#define WUSH_ERR_NOT_SM100 (-6)
#define WUSH_ERR_DEVICE_TIMEOUT (-7) /* a bounded wait inside a kernel ran out (reported through `status`) */
#define WUSH_ERR_TOO_LARGE (-8)      /* problem exceeds a fixed capacity of the entry point */

/* Layout of the per-group scale bytes written by the fused quantize kernels. */
#define WUSH_SF_ROW_MAJOR 0 /* sf[row * sf_cols + group], sf_cols = ceil(C/G/4)*4 */
#define WUSH_SF_BLOCKED 1   /* 128x4 tiles of 512 bytes: ((row/128)*(sf_cols/4) + group/4)*512
                               + (row%32)*16 + ((row%128)/32)*4 + group%4 -- the layout the
                               block-scaled tensor-core MMA consumes */

/* flags of the fused quantize entry points */
#define WUSH_QUANT_ROUND_BF16 1 /* round the transformed values to bf16 before quantizing, as the
                                   reference's runtime module does between its einsum and its
                                   quantizer (src/utils/wush_utils.py:140-149) */
#define WUSH_QUANT_WIDE_MATRIX 2 /* `mat` is one square bf16 matrix [mat_cols, mat_cols] shared by every block of
                                   mat_cols channels, wider than the quantization group: mat_cols 64 or 128 (and 32
                                   for NVFP4); cols % mat_cols == 0.  y_block = x_block @ mat, then groups of 32 / 16
                                   as usual: the shared Hadamard sizes of FPQuantConfig.hadamard_group_size
                                   (inference_lib/src/fp_quant/utils/config.py:35-50).  Not with ROUND_BF16, the
                                   debug or the strided entry. */

/* quantization formats of the entry points that take a `format` argument */
#define WUSH_FORMAT_MXFP4 0 /* groups of 32, E8M0 scales */
#define WUSH_FORMAT_NVFP4 1 /* groups of 16, E4M3 scales, fp32 tensor scale */

/* Library / build information: compute capability the kernels were compiled for (100). */
WUSH_API int wush_b200_arch(void);

/*
 * Device-side errors.  The entry points that take a `status` argument (a DEVICE int, may be NULL) run kernels
 * whose waits on asynchronous copies and tensor-core completions are bounded; if one runs out, the kernel
 * unwinds, frees what it holds and sets *status = 1 (its output is then invalid).  One word may be shared by any
 * number of calls.  wush_status_check synchronizes `stream`, reads the word and returns WUSH_ERR_DEVICE_TIMEOUT
 * (clearing the word) if it was set, WUSH_OK otherwise.  The reference has no error codes; its host code raises
 * Python exceptions (e.g. src/quantization/accumulate_hessian.py:126-127), which is what the Python layer does
 * with this return value.
 * wush_selftest_bounded_wait launches one tiny kernel that waits, with a limit of `max_polls` polls (at most
 * 65536), on a barrier nothing arrives on, so that callers can test their handling of the status word; the
 * kernel returns by itself within microseconds.
 * Every launching entry point returns WUSH_ERR_NOT_SM100 when the current device is not compute capability 10.x.
 */
WUSH_API int wush_status_check(int* status_dev, void* stream);
WUSH_API int wush_selftest_bounded_wait(int* status_dev, int max_polls, void* stream);

/*
 * Fused per-group transform + MXFP4 quantization of activations or weights.
 *
 * Replaces qutlass.fusedQuantizeWushMx / qutlass.fusedQuantizeMx (abs_max method) as bound at
 * inference_lib/src/fp_quant/module/qutlass_ops.py:37-72 and :110-143, and the three-kernel
 * pseudo-quant path of src/utils/wush_utils.py:124-150.
 *
 *   x        bf16 [rows, cols] row-major, cols % 32 == 0, 16-byte aligned
 *   mat      bf16 [32, mat_cols] row-major; mat_cols == cols: column block n holds the transposed
 *            32x32 transform of channel group n (y_n = x_n @ mat[:, 32n:32n+32]);
 *            mat_cols == 32: one matrix shared by every group (e.g. a Hadamard matrix)
 *   q        u8 [rows, cols/2]: E2M1 codes, element 2i in the low nibble; 16-byte aligned
 *   sf       u8 E8M0 scale bytes, one per 32 channels, in `sf_layout` with `sf_cols` bytes per
 *            row (sf_cols % 4 == 0, sf_cols >= cols/32; 4-byte aligned); only entries of real rows and groups
 *            are written, padding is left untouched
 * Scale = 2^floor(log2(absmax)); code = RNE_e2m1(3 * y / scale); an all-zero group gives scale
 * byte 0 and codes 0x88.
 */
WUSH_API int wush_fused_quantize_mx(const void* x, const void* mat, int64_t mat_cols, uint8_t* q, uint8_t* sf,
                           int64_t sf_cols, int sf_layout, int64_t rows, int64_t cols, int flags,
                           void* stream);

/*
 * The same kernel with the "quest" scale (MXFP4 only): replaces qutlass.fusedQuantizeMx(method="quest",
 * return_mask) as bound at inference_lib/src/fp_quant/module/qutlass_ops.py:37-52; the arithmetic is that of the
 * reference's Triton kernel, inference_lib/src/fp_quant/module/triton/mxfp4.py:64-124.
 *
 *   scale = 2^floor(log2(c * std + 1e-8)), std = sqrt(E[y^2] - E[y]^2) over the group's 32 values in fp32,
 *   c = 2.92247856 / 6;  code = RNE_e2m1(y / scale) saturated at +-6 (no factor 3: the layer's global scales are 1).
 *   clip_mask  null, or u8 [rows, cols/8]: bit i of byte b is set when element 8b + i was not clipped
 *              (|y / scale| < 6), the packing the reference's _unpack_mask (linear_fns.py:78-88) reads.
 * Other arguments as for wush_fused_quantize_mx.
 */
WUSH_API int wush_fused_quantize_mx_quest(const void* x, const void* mat, int64_t mat_cols, uint8_t* q, uint8_t* sf,
                                 int64_t sf_cols, int sf_layout, uint8_t* clip_mask, int64_t rows, int64_t cols,
                                 int flags, void* stream);

/*
 * Fused per-group transform + NVFP4 quantization (groups of 16, E4M3 scales, fp32 tensor scale).
 *
 * Replaces qutlass.fusedQuantizeNv as bound at
 * inference_lib/src/fp_quant/module/qutlass_ops.py:75-106.
 *
 *   mat           bf16 [16, mat_cols]; mat_cols == cols (per-group 16x16 transforms, laid out as
 *                 above) or mat_cols == 16 (shared)
 *   global_scale  device pointer to one fp32 (10.0 in the reference's exported checkpoints)
 *   sf            u8 E4M3 scale bytes, one per 16 channels; sf_cols >= cols/16
 * Scale = RN_e4m3(absmax * global_scale / 6), saturated at 448; code = RNE_e2m1(y * global_scale
 * / scale).
 */
WUSH_API int wush_fused_quantize_nv(const void* x, const void* mat, int64_t mat_cols, const float* global_scale,
                           uint8_t* q, uint8_t* sf, int64_t sf_cols, int sf_layout, int64_t rows,
                           int64_t cols, int flags, void* stream);

/*
 * The same kernels for operands that are column slices of wider tensors: the activations may be a slice of a wider
 * row-major tensor (row stride ldx elements), and the codes and scales are written into the operand buffers of a
 * GEMM whose K dimension is wider than this call's columns -- how a tensor-parallel layer assembles the quantized
 * input of its next GEMM from column shards that were produced on different GPUs (every GPU quantizes the columns it
 * holds; scale groups never straddle a shard).  No counterpart in the reference, which is single-GPU and always
 * quantizes whole rows (inference_lib/src/fp_quant/module/linear_fns.py:29-62).
 *
 *   format     WUSH_FORMAT_MXFP4 / WUSH_FORMAT_NVFP4 (global_scale is ignored for MXFP4 and may be NULL)
 *   x, ldx     bf16 [rows, cols], row stride ldx >= cols elements, ldx % 8 == 0
 *   q, ldq     first byte of this call's codes inside the destination, row stride ldq >= cols / 2 bytes, ldq % 16 == 0
 *   sf, sf_cols, sf_layout   the destination's scale tensor (sf_cols scale bytes per row, all columns of the GEMM)
 *   sf_group0  index of this call's first scale group inside a row of sf; a multiple of 4
 *   row_scale, col_scale   both NULL, or fp32 [rows] and bf16 [cols]: the activations are replaced by
 *              bf16(bf16(x * row_scale[row]) * col_scale[col]) before the transform -- RMSNorm folded into the
 *              quantizer of the layer that follows it (row_scale = rsqrt(mean(x^2) + eps) of the WHOLE row, which
 *              with column shards is formed from wush_row_sumsq partial sums of all GPUs; col_scale = the norm's
 *              weight), with the roundings of the separate bf16 steps.  Not with WUSH_QUANT_ROUND_BF16.
 */
WUSH_API int wush_fused_quantize_strided(int format, const void* x, int64_t ldx, const void* mat, int64_t mat_cols,
                                         const float* global_scale, uint8_t* q, int64_t ldq, uint8_t* sf,
                                         int64_t sf_cols, int sf_layout, int64_t sf_group0, const float* row_scale,
                                         const void* col_scale, int64_t rows, int64_t cols, int flags, void* stream);

/*
 * Element-wise neighbours of the quantized layers in a decoder block, one pass over HBM each.  No counterpart in
 * the reference, whose layers (inference_lib/src/fp_quant/module/linear.py) leave them to the model code.
 *   wush_row_sumsq  out[r] = sum_c x[r, c]^2 in fp32 (bf16 x [rows, cols], row stride ldx; cols % 8 == 0)
 *   wush_swiglu     out = bf16(silu(gate)) * up, all bf16 [rows, cols]; gate and up share the row stride ld_in (e.g.
 *                   the two halves of a fused gate/up projection's output); silu uses the hardware exponential
 */
WUSH_API int wush_row_sumsq(const void* x, int64_t ldx, float* out, int64_t rows, int64_t cols, void* stream);
WUSH_API int wush_swiglu(const void* gate, const void* up, int64_t ld_in, void* out, int64_t ld_out, int64_t rows,
                         int64_t cols, void* stream);

/*
 * Debug/validation variant of the two calls above: same arithmetic, but also stores the
 * transformed values (after the optional bf16 rounding) as fp32 [rows, cols].  `fmt` is 0 for
 * MXFP4 and 1 for NVFP4 (global_scale may be NULL for MXFP4).  Used by the parity tests for the
 * 1e-5 bound on transformed values; has no counterpart in the reference's FFI.
 */
WUSH_API int wush_fused_quantize_debug(int fmt, const void* x, const void* mat, int64_t mat_cols,
                              const float* global_scale, uint8_t* q, uint8_t* sf, int64_t sf_cols,
                              int sf_layout, float* transformed, int64_t rows, int64_t cols, int flags,
                              void* stream);

/*
 * Row-major padded scales -> 128x4 blocked layout (see WUSH_SF_BLOCKED).
 * Replaces qutlass.utils.to_blocked as called at
 * inference_lib/src/fp_quant/module/qutlass_ops.py:160-161,198-199,372-373.
 *   in   u8 [rows, cols]   out  u8, ceil(rows/128)*128 * ceil(cols/4)*4 bytes, zero in the padding
 */
WUSH_API int wush_sf_to_blocked(const uint8_t* in, uint8_t* out, int64_t rows, int64_t cols, void* stream);

/* flags of wush_hessian_accumulate */
#define WUSH_HESSIAN_LOWER_ONLY 1 /* update the lower triangle (and diagonal) only, do not mirror */
#define WUSH_HESSIAN_INPUT_F32 2  /* x is fp32 [tokens, hidden]; products are formed in TF32 (top 19 bits of each
                                     operand), as the reference's Triton kernel does for fp32 inputs */
#define WUSH_HESSIAN_OVERWRITE 4  /* H = X^T X instead of H += X^T X: the previous contents of the updated entries are
                                     not read, so the buffer needs no zeroing (what WUSH.update does on its first call,
                                     src/quantization/wush_gptq.py:464-465, without the torch.zeros pass) */

/*
 * GPTQ Hessian accumulation, in place:  H += X^T X.
 *
 * Replaces the Triton kernel behind accumulate_hessian(mat_hessian, mat_input, save_lower_only,
 * compute_lower_only) at src/quantization/accumulate_hessian.py:26-148 (called from WUSH.update,
 * src/quantization/wush_gptq.py:456-469).
 *
 *   h       fp32 [hidden, hidden] row-major, 16-byte aligned, read and written
 *   x       bf16 (or fp32 with WUSH_HESSIAN_INPUT_F32) [tokens, hidden] row-major, 16-byte aligned, hidden % 8 == 0
 *   flags   bitwise OR of WUSH_HESSIAN_LOWER_ONLY (the reference's save_lower_only=True), WUSH_HESSIAN_INPUT_F32 and
           WUSH_HESSIAN_OVERWRITE
 *   status  optional device int, set to 1 if a bounded wait inside the kernel ran out (the result
 *           is then invalid); may be NULL
 * bf16 products are exact in fp32 and are summed in fp32 tensor-core accumulators over the tokens
 * of the call, then added to H with one fp32 rounding per element.  Only tiles that touch the
 * lower triangle are computed; the upper triangle is written as a mirror image.
 */
WUSH_API int wush_hessian_accumulate(float* h, const void* x, int64_t tokens, int64_t hidden, int flags, int* status,
                                     void* stream);

/*
 * The same update restricted to rows [row_begin, row_end) of H (row_begin % 128 == 0; row_end % 128 == 0 or
 * row_end == hidden).  Lets a caller finish H one row panel at a time, e.g. to all-reduce a finished panel
 * across GPUs while the next one is being computed.  With the mirror enabled the matching columns of the
 * upper triangle are written too.  No counterpart in the reference, which is single-GPU.
 */
WUSH_API int wush_hessian_accumulate_rows(float* h, const void* x, int64_t tokens, int64_t hidden, int64_t row_begin,
                                          int64_t row_end, int flags, int* status, void* stream);

/*
 * The lower triangle as a list of 256 x 256 tiles, in the order the accumulation kernel walks them (bands of 8
 * row blocks, column block by column block inside a band).  Ranges of this list are the unit in which a
 * multi-GPU job overlaps the combine of finished tiles with the accumulation of later ones.  No counterpart in
 * the reference, which is single-GPU.
 *   wush_hessian_tile_count      number of tiles: n (n + 1) / 2 with n = ceil(hidden / 256)
 *   wush_hessian_tiles_per_wave  tiles the current device works on side by side (resident CTA pairs); a launch
 *                                over a multiple of this many tiles has no partly filled last wave
 *   wush_hessian_tile_coords     row / column block (units of 256) of entry `tile`
 */
WUSH_API int64_t wush_hessian_tile_count(int64_t hidden);
WUSH_API int wush_hessian_tiles_per_wave(void);
WUSH_API int wush_hessian_tile_coords(int64_t hidden, int64_t tile, int* row_block, int* col_block);

/*
 * H += X^T X restricted to entries [tile_begin, tile_end) of the tile list; always the CTA-pair kernel.
 * Same arguments and flags as wush_hessian_accumulate.
 */
WUSH_API int wush_hessian_accumulate_tiles(float* h, const void* x, int64_t tokens, int64_t hidden, int64_t tile_begin,
                                           int64_t tile_end, int flags, int* status, void* stream);

/*
 * Writes the mirror image (upper triangle) of the tiles [tile_begin, tile_end) from their lower-triangle values.
 * barrier_slots / barrier_epoch / rank / world: as for wush_hessian_peer_reduce (NULL slots: no barrier).
 */
WUSH_API int wush_hessian_mirror_tiles(float* h, int64_t hidden, int64_t tile_begin, int64_t tile_end, int rank, int world,
                                       uint32_t* const* barrier_slots, uint32_t barrier_epoch, int* status, void* stream);

/*
 * h[i][j] <- scale * h[i][j] for j <= i, and h[j][i] <- the same value: turns a lower-triangular raw sum
 * into the symmetric running mean that WUSH.update maintains (src/quantization/wush_gptq.py:467-468 applies
 * the 1/N factor on every call; applying it once here is algebraically the same).  hidden % 4 == 0.
 * With scale == 1 the lower triangle is not rewritten (mirror only).
 */
WUSH_API int wush_hessian_finalize(float* h, int64_t hidden, float scale, void* stream);
/* The same with scale = 1 / *count, `count` being a device int64 (e.g. the all-reduced token count): keeps a
 * multi-GPU job free of host synchronisation.  No counterpart in the reference, which is single-GPU. */
WUSH_API int wush_hessian_finalize_count(float* h, int64_t hidden, const int64_t* count, void* stream);

/*
 * Multi-GPU combine of the Hessian over NVLink / NVSwitch (one process per GPU), for a range of the tile list.
 * No counterpart in the reference, which is single-GPU.
 *
 *   bufs    DEVICE array of `world` pointers: every rank's fp32 [hidden, hidden] buffer holding its raw
 *           lower-triangle sum, all addressable from this GPU (e.g. torch symmetric memory)
 *   mc_buf  multicast address of the same buffers (one address that reaches all of them through the NVSwitch),
 *           or NULL.  Given: the sums are formed by multimem.ld_reduce inside the switch and delivered by
 *           multimem.st; NULL: plain peer loads and stores
 *   counts  DEVICE array of `world` pointers to each rank's int64 local token count (peer-addressable)
 * The range is cut into sub-tiles of 8 rows x 128 columns that are dealt round-robin to the ranks.  On return (stream order) every
 * rank's buffer holds, for the sub-tiles this rank owns, the sum over ranks divided by the total token count
 * (lower triangle only; wush_hessian_mirror_tiles rebuilds the rest locally).  Once EVERY rank has run it, all
 * buffers hold the same bits for the range.  The launches must be separated from the producers and consumers of
 * the range by cross-rank barriers: all ranks' partial sums of the range complete before any rank starts, all
 * ranks done before the result is read.  hidden % 4 == 0, world <= 16.
 *   barrier_slots  NULL: the caller runs those barriers.  Otherwise a DEVICE array of `world` pointers to every
 *           rank's array of 16 uint32 slots in peer-addressable memory (zero before the first use): the kernel then
 *           starts with a barrier of its own -- it stores barrier_epoch into its slot on every rank and waits until
 *           all of its own slots have reached it -- which says "the previous kernel of my stream is complete" to
 *           the other ranks at the cost of one NVLink round trip instead of a separate barrier kernel.  Every use
 *           (of this call or of wush_hessian_mirror_tiles) on the same slots takes the next barrier_epoch, the
 *           same on all ranks.  The wait is bounded; on expiry *status (DEVICE int, may be NULL) is set to 1.
 */
WUSH_API int wush_hessian_peer_reduce(float* const* bufs, float* mc_buf, const int64_t* const* counts, int rank,
                                      int world, int64_t hidden, int64_t tile_begin, int64_t tile_end,
                                      uint32_t* const* barrier_slots, uint32_t barrier_epoch, int* status, void* stream);

/*
 * One rank's piece of a buffer that exists on every GPU (symmetric memory) delivered to all of them in one launch:
 * the exchange of FP4 codes + scale bytes between the ranks of a column-sharded decoder block (this build's
 * multi-GPU form of the activation path of FPQuant4x16NoMasterFn.forward, inference_lib/src/fp_quant/module/
 * linear_fns.py:494-539; the reference has no multi-GPU path of its own).
 *
 *   src     this rank's data, 16-byte aligned, `bytes` a multiple of 16
 *   mc_dst  the multicast address of the destination range (every 16 bytes leave this GPU once, the NVSwitch writes
 *           them into all ranks' buffers, this rank's included), or NULL
 *   dst     when mc_dst is NULL: the destination addresses in the n_dst other ranks' buffers (HOST array of device
 *           pointers, at most 16), written one after the other with plain peer stores
 * The caller orders the stores against their readers (a barrier across the ranks after the launch).
 */
WUSH_API int wush_peer_broadcast(const void* src, void* mc_dst, void* const* dst, int n_dst, int64_t bytes,
                                 void* stream);

/*
 * Block-scaled FP4 GEMM, "TN":  y[m, n] (bf16) = alpha * deq(a)[m, k] . deq(b)[n, k]^T.
 *
 * Replace qutlass.matmul_mxf4_bf16_tn / qutlass.matmul_nvf4_bf16_tn as bound at
 * inference_lib/src/fp_quant/module/qutlass_ops.py:149-168 and :187-206 (called from forward_gemm,
 * inference_lib/src/fp_quant/module/linear_fns.py:65-76).
 *
 *   a, b       u8 [m, k/2], [n, k/2]: packed E2M1, element 2i in the low nibble; 16-byte aligned
 *   sfa, sfb   scale bytes in the WUSH_SF_BLOCKED layout, covering ceil(rows/128)*128 rows and
 *              ceil(k/G/4)*4 groups (G = 32, E8M0 for mxf4; G = 16, E4M3 for nvf4); padding entries must
 *              hold finite scale bytes (zero is fine)
 *   alpha      device pointer to one fp32 (1 / (weight_global_scale * act_global_scale) in the reference)
 *   y          bf16 [m, n] row-major, 16-byte aligned; n % 8 == 0, k % 128 == 0
 *   splits     0 = choose automatically.  m <= 4 and k <= 8192 (decode; WUSH_B200_GEMV_MAX_M / _MAX_K move the limits, 0 rows
 *              switches it off):
 *              a matrix-vector kernel streams the weight bytes once with plain loads and multiplies on the CUDA cores
 *              (exact fp16 sums of 8 products, fp32 from there on), 16 weight rows per CTA, no K splits.
 *              Otherwise, when few output tiles exist (small m: the GEMM streams the weights once and is bound by
 *              memory) the K range is split over 2, 4 or 8 CTAs that form a thread-block cluster;
 *              their fp32 partial tiles meet in distributed shared memory and are added in split order, in the same
 *              launch, without scratch memory.
 *              > 0 forces that many K splits the other way: fp32 partial tiles [splits, m, n] in `workspace` and a
 *              second kernel that adds them (fails with WUSH_ERR_WORKSPACE_TOO_SMALL if the workspace is too small).
 *   workspace  device scratch for forced splits only (16-byte aligned, contents irrelevant,
 *              wush_gemm_workspace_bytes() bytes); may be NULL when splits <= 1
 *   status     optional device int set to 1 if a bounded wait inside the kernel ran out; may be NULL
 * fp32 accumulation over the whole K range; one rounding to bf16 at the end.
 */
WUSH_API int wush_gemm_mxf4_bf16_tn(const uint8_t* a, const uint8_t* b, const uint8_t* sfa, const uint8_t* sfb,
                                    const float* alpha, void* y, int64_t m, int64_t n, int64_t k, void* workspace,
                                    size_t workspace_bytes, int splits, int* status, void* stream);
WUSH_API int wush_gemm_nvf4_bf16_tn(const uint8_t* a, const uint8_t* b, const uint8_t* sfa, const uint8_t* sfb,
                                    const float* alpha, void* y, int64_t m, int64_t n, int64_t k, void* workspace,
                                    size_t workspace_bytes, int splits, int* status, void* stream);
/*
 * The same GEMM with the neighbouring element-wise steps of the layer folded into its epilogue, and explicit row
 * strides.  Replaces, in FPQuant4x16NoMasterFn.forward (inference_lib/src/fp_quant/module/linear_fns.py:514-525),
 * the sequence forward_gemm(...) ; y += bias, and the residual addition that follows the o_proj / down_proj layers
 * of a decoder block.  The roundings of the unfused sequence are kept, so the result is bit-identical to it:
 *   y = bf16(alpha * acc);  if bias: y = bf16(y + bias[col]);  if residual: y = bf16(y + residual[row, col])
 *
 *   format     WUSH_FORMAT_MXFP4 / WUSH_FORMAT_NVFP4
 *   bias       bf16 [n] or NULL;  residual  bf16 [m, ldr] or NULL (may be y itself: every element is read before it
 *              is written, by the same thread);  ldr, ldy  row strides in elements (0 = n); multiples of 8
 *   a_shards   1: `a` is [m, k/2] as above.  > 1: the K dimension of the activations arrives in `a_shards` pieces
 *              that were quantized separately (e.g. column shards produced on different GPUs and copied side by
 *              side): `a` is a stack of a_shards matrices [a_shard_rows, k/a_shards/2] (a_shard_rows >= m), and
 *              `sfa` a stack of their blocked scale tensors, a_sf_shard_bytes apart (0 = densely stacked:
 *              ceil(a_shard_rows/128)*128 rows x k/a_shards/G groups each; otherwise a multiple of 16);
 *              k/a_shards must be a multiple of 256.  The weights are unaffected: piece s multiplies the weight
 *              columns [s, s+1) * k/a_shards.
 * Everything else as for wush_gemm_mxf4_bf16_tn.
 */
WUSH_API int wush_gemm_fp4_bf16_tn_fused(int format, const uint8_t* a, int a_shards, int64_t a_shard_rows,
                                         int64_t a_sf_shard_bytes, const uint8_t* b, const uint8_t* sfa,
                                         const uint8_t* sfb, const float* alpha,
                                         const void* bias, const void* residual, int64_t ldr, void* y, int64_t ldy,
                                         int64_t m, int64_t n, int64_t k, void* workspace, size_t workspace_bytes,
                                         int splits, int* status, void* stream);

/*
 * Split-K MXFP4 GEMM for callers that must not allocate device memory.  (No counterpart in the reference.)
 *
 * Some hosts of this library cannot call cudaMalloc on the path where the GEMM runs: a serving loop whose
 * memory is fully carved up at start-up, a plugin running inside another framework's stream-ordered pool, code
 * replayed from a captured graph.  For small-M (decode) shapes the GEMM wants scratch for its split-K partial
 * tiles; this entry point keeps that scratch in a fixed array inside the library (WUSH_GEMM_STATIC_SCRATCH_BYTES
 * of device memory per GPU that loads the library, held until the process exits), so the caller passes inputs and
 * the output only.  Same arithmetic and argument meaning as
 * wush_gemm_mxf4_bf16_tn with a workspace.
 *
 *   splits   0 = choose (at least 2, reduced until the partial tiles fit); >= 2 forces a value
 * Returns WUSH_ERR_TOO_LARGE when splits * m * n fp32 values do not fit in the array (or the problem has more than
 * 256 output tiles), WUSH_ERR_BAD_FLAG when K is too short to be split (fewer than 2 blocks of 256) or `splits`
 * is out of range.
 * Rules: (1) the first call on each device looks up the array's device address (cudaGetSymbolAddress) and caches
 * it; make that first call outside any stream capture.  (2) Every call on a device uses the same array: calls
 * that can overlap on the GPU (different streams without ordering) race and corrupt each other; serialize them.
 * (3) Nothing needs zeroing: each call overwrites every partial value it later reads.  It calls no cudaMalloc,
 * cudaFree or other allocating routine.
 */
#define WUSH_GEMM_STATIC_SCRATCH_BYTES (16u << 20)
WUSH_API int wush_gemm_mxf4_bf16_tn_noalloc(const uint8_t* a, const uint8_t* b, const uint8_t* sfa, const uint8_t* sfb,
                                            const float* alpha, void* y, int64_t m, int64_t n, int64_t k, int splits,
                                            int* status, void* stream);

/* Thread-block clusters of `splits` (2, 4 or 8) CTAs of the split-K kernel that the current device can run side by
 * side (0: none, or no sm_100 device); the automatic split choice keeps one cluster per output tile within it. */
WUSH_API int wush_gemm_cluster_capacity(int format, int splits);

/* Scratch bytes a GEMM with `splits` forced K splits needs (0 for splits <= 1; the automatic choice needs none). */
WUSH_API size_t wush_gemm_workspace_bytes(int64_t m, int64_t n, int64_t k, int splits);

/*
 * Block-scaled FP4 GEMM with column-sharded weights: y[:, col0 : col0 + n] = alpha * A . B_shard^T, stored into the
 * same place of EVERY GPU's output buffer, so that after all `world` GPUs have run it each holds the complete
 * [m, ldy] output -- the GEMM and the all-gather of its columns in one kernel (the epilogue's whole-line stores
 * go to peer-addressable memory over NVLink; no multicast, no collective call).
 *
 * Replaces, for weights split by output features over GPUs, the pair matmul_*_bf16_tn_op
 * (inference_lib/src/fp_quant/module/qutlass_ops.py:149-206) + an all-gather of the output; the reference is
 * single-GPU and has no counterpart.
 *
 *   format   WUSH_FORMAT_MXFP4 / WUSH_FORMAT_NVFP4
 *   a        packed E2M1 [m, k/2] (replicated activations); sfa blocked scales, as for wush_gemm_*_bf16_tn
 *   b, sfb   THIS GPU's shard of the weights: packed E2M1 [n, k/2] and its blocked scales
 *   y_all    HOST array of `world` DEVICE pointers to bf16 [m, ldy] buffers, all addressable from this GPU (e.g.
 *            torch symmetric memory); entry `rank` is this GPU's own buffer
 *   ldy      row stride of the buffers in elements (the unsharded N); col0 first column of this shard;
 *            ldy % 8 == col0 % 8 == n % 8 == 0, world <= 8
 * The caller separates the launches from the readers of the buffers with cross-GPU barriers: nobody still reads
 * the previous contents when any GPU starts, every GPU has finished before the result is read.  Always unsplit
 * (no workspace).
 */
WUSH_API int wush_gemm_fp4_bf16_tn_sharded(int format, const uint8_t* a, const uint8_t* b, const uint8_t* sfa,
                                           const uint8_t* sfb, const float* alpha, void* const* y_all, int world,
                                           int rank, int64_t ldy, int64_t col0, int64_t m, int64_t n, int64_t k,
                                           int* status, void* stream);

/*
 * One block of the GPTQ / Babai column sweep, all weight rows at once.
 *
 * Replaces the part of block_transform_gptq_babai_inner after its QR factorization
 * (src/quantization/wush_gptq.py:254-274): the triangular solve for the transformed coefficients, the
 * quantizer call rtn_xxfp4 (:91-138, constants of :388-407), the nearest-plane loop that re-quantizes with
 * frozen scales and updates the remaining targets (:266-272), and the coefficient product transform^T . x
 * (:274); it also writes what collate_xxfp4 (:280-301) assembles.  With nblocks > 1 it handles independent
 * blocks in one launch (round-to-nearest mode, where no block depends on another).
 *
 *   rn       float64 [nblocks, G, G]   upper-triangular factor of basis . transform^T
 *   ynew     float64 [nblocks, G, rows] rotated targets Q^T y -- or the raw targets y when qt is given
 *   qt       float64 [nblocks, G, G]   Q^T; the kernel then rotates the targets itself (:252).  NULL: ynew is rotated
 *   tmat     float64 [nblocks, G, G]   block transforms (already rounded to the model dtype)
 *   codes    u8 [rows, cols/2]  packed E2M1 (element 2i in the low nibble); this call writes columns
 *            [(col_block0 + b) * G/2, +G/2) of every row for b < nblocks
 *   scales   u8 [rows, cols/G]  E8M0 / E4M3 bytes, column col_block0 + b
 *   fake     bf16 (or fp32 with WUSH_SWEEP_FAKE_F32) [rows, cols] dequantized transformed weights, or NULL
 *   coef     float64 [nblocks, G, rows] transform^T . x_quantized, or NULL
 *   format   WUSH_FORMAT_MXFP4 (G = 32, E8M0 scales) / WUSH_FORMAT_NVFP4 (G = 16, E4M3, tensor scale 10)
 *   flags    WUSH_SWEEP_RTN_ONLY: round to nearest only (force_rtn), no nearest-plane loop
 * Float64 arithmetic in the reference's operation order; ties round to the even code; exact zeros encode
 * as -0 like the reference's quantizer does.
 */
#define WUSH_SWEEP_RTN_ONLY 1
#define WUSH_SWEEP_FAKE_F32 2
WUSH_API int wush_gptq_block_step(const double* rn, const double* ynew, const double* qt, const double* tmat,
                                  int nblocks, int col_block0, int64_t rows, int64_t cols, int format, int flags,
                                  uint8_t* codes, uint8_t* scales, void* fake, double* coef, void* stream);

/*
 * The G x G dense algebra of one sweep block (or of nblocks independent blocks), one CTA per block.
 *
 * Replaces get_transform (src/quantization/wush_gptq.py:304-347) and the QR factorization at the top of
 * block_transform_gptq_babai_inner (:251-252):
 *   'wush': V, s = left singular vectors / values of the block's targets y, taken from the eigen-decomposition
 *   of gram = y y^T (cyclic Jacobi); s *= rows^-1/2; s += 1 % of mean(s); T = Had diag(s^1/2) V^T basis^-T
 *   (:331-341; 'wus': identity instead of the Hadamard matrix); T is rounded to the model dtype (:345);
 *   then Q R = basis T^T by Householder reflections.
 * The sign of every singular vector is fixed by making its largest component positive (an SVD leaves it open).
 *
 *   gram        float64 [nblocks, G, G] (read for WUSH / WUS only)
 *   basis       float64 G x G upper-triangular diagonal block of the Cholesky factor, row stride ldb; block b
 *               starts basis_step * b elements further (G * ldb + G walks down the diagonal of one factor)
 *   transform   WUSH_TRANSFORM_*; GIVEN reads tmat instead of computing it
 *   flags       WUSH_SWEEP_FAKE_F32: the model dtype is fp32 (round T to fp32 instead of bf16)
 *   rows        number of weight rows R (for the R^-1/2 factor)
 *   tmat, rn, qt  float64 [nblocks, G, G] out: transform, R (upper triangular), Q^T -- the inputs of
 *               wush_gptq_block_step (which rotates the raw targets itself when given qt)
 *   status      optional DEVICE int, set to 1 if a transform is not finite
 */
#define WUSH_TRANSFORM_IDENTITY 0
#define WUSH_TRANSFORM_HADAMARD 1
#define WUSH_TRANSFORM_WUSH 2
#define WUSH_TRANSFORM_WUS 3
#define WUSH_TRANSFORM_GIVEN 4
WUSH_API int wush_gptq_block_prepare(const double* gram, const double* basis, int64_t ldb, int64_t basis_step,
                                     int nblocks, int format, int transform, int flags, int64_t rows, double* tmat,
                                     double* rn, double* qt, int* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* WUSH_B200_H_ */
