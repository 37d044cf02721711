/* lockstep_b200 -- C ABI of the B200 (sm_100a) MXFP4 hot path.
 *
 * Drop-in boundary for lockstep's data-parallel hot path: MXFP4 quantize /
 * pack / unpack / dequantize, the packed (dual-batch) MXFP4 GEMM and the
 * FP4-compressed gradient all-reduce.  Plain pointers and sizes only; every
 * pointer is a DEVICE pointer unless its comment says "host".  Kernels are
 * enqueued on the CUDA stream passed as `stream` (a cudaStream_t cast to
 * void*, NULL = default stream) and the call returns without synchronising
 * unless stated otherwise.
 *
 * Return value: 0 on success, a negative LS_E* code otherwise;
 * ls_last_error() gives the message of the calling thread's last failure.
 * Nothing in this library computes on the CPU: without a CUDA device of
 * compute capability 10.x every compute entry point returns LS_EARCH.
 *
 * "Replaces" comments cite the lockstep source (path:line within that
 * project) whose behaviour the entry point reproduces.
 */
#ifndef LOCKSTEP_B200_H
#define LOCKSTEP_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LS_OK        0
#define LS_EINVAL   -1   /* bad argument (shape, block size, null pointer)   */
#define LS_EALIGN   -2   /* pointer or size not aligned as documented        */
#define LS_ECUDA    -3   /* a CUDA runtime/driver call failed                */
#define LS_ETIMEOUT -4   /* a bounded device-side wait ran out               */
#define LS_EARCH    -5   /* no sm_100 device                                 */
#define LS_ESTATE   -6   /* handle used in the wrong state                   */

/* element types of floating-point buffers */
#define LS_F32  0
#define LS_BF16 1

/* rounding of a value exactly halfway between two E2M1 grid points */
#define LS_ROUND_REF 0   /* keep the smaller magnitude: lockstep fp4.py:43-54 */
#define LS_ROUND_RNE 1   /* OCP MX ties-to-even (no lockstep counterpart)     */

int ls_version(void);
const char *ls_last_error(void);

/* Number of bytes of the tensor-core scale-factor ("SF") buffer for a
 * [rows, K] operand quantized in blocks of 32: 512 bytes per 128 rows x 128
 * columns, rows rounded up to 128.  K must be a multiple of 128. */
int64_t ls_sf_bytes(int64_t rows, int64_t K);
/* The same for blocks of `block` = 32 or 16 elements: a 512-byte tile holds 128
 * rows x 4 scales, so blocks of 16 take twice the bytes.  -1 for a bad argument. */
int64_t ls_sf_bytes_block(int64_t rows, int64_t K, int block);

/* Fused MXFP4 quantizer along the last dimension.
 * Replaces fp4.py:57-72 (quantize_mxfp4), :43-54 (_round_to_e2m1) and,
 * through `packed`, :91-94 (pack_fp4).
 *   x        [rows, K] row-major, LS_F32 or LS_BF16; 32-byte aligned
 *   block    32 or 16; K % block == 0
 * Outputs, each may be NULL (at least one must not be):
 *   codes    [rows, K] one E2M1 code per byte (bit 3 = sign)
 *   packed   [rows, K/2] two codes per byte, even index in the low nibble
 *   scale    [rows, K/block] fp32 power of two 2^E
 *   e8m0     [rows, K/block] biased exponent E+127 (0xFF for a NaN block)
 *   sf       e8m0 bytes in the tcgen05 scale-factor layout
 *            (ls_sf_bytes_block(rows, K, block)); needs K % 128 == 0 */
int ls_quantize_mxfp4(const void *x, int x_dtype, int64_t rows, int64_t K, int block,
                      int rounding, uint8_t *codes, uint8_t *packed, float *scale,
                      uint8_t *e8m0, uint8_t *sf, void *stream);

/* Transposed form: x [R, C] row-major -> MXFP4 of x^T, i.e. blocks of 32 run down
 * the columns of x.  Same arithmetic as ls_quantize_mxfp4 applied to a
 * transposed copy (lockstep composes fp4.quantize_mxfp4(x.t().contiguous()) for
 * GEMMs that contract over rows); no copy is made here.  R % 128 == 0.
 *   packed [C, R/2], scale fp32 [C, R/32], sf = scale-factor layout of a
 *   [C, R] operand (ls_sf_bytes(C, R)); each may be NULL. */
int ls_quantize_mxfp4_t(const void *x, int x_dtype, int64_t R, int64_t C, int rounding,
                        uint8_t *packed, float *scale, uint8_t *sf, void *stream);

/* ls_quantize_mxfp4_t of act(x): act = 1 quantizes GELU(x) (0.5 x (1 + erf(x / sqrt 2)), computed
 * in fp32 and rounded to bf16 as an elementwise pass would leave it) without that pass: the
 * activation of lockstep's feed-forward block (train.py:53) is needed transposed for the
 * weight gradient of the projection after it and need not exist in HBM.  bf16 input only;
 * act = 0 is ls_quantize_mxfp4_t.  No single lockstep function does this. */
int ls_quantize_mxfp4_t_act(const void *x, int x_dtype, int64_t R, int64_t C, int rounding, int act,
                            uint8_t *packed, float *scale, uint8_t *sf, void *stream);
/* Likewise ls_quantize_mxfp4_both of act(x): both orientations of GELU(x) from one read of x. */
int ls_quantize_mxfp4_both_act(const void *x, int x_dtype, int64_t R, int64_t C, int rounding, int act,
                               uint8_t *row_packed, uint8_t *row_sf, uint8_t *t_packed, uint8_t *t_sf,
                               void *stream);

/* LayerNorm over the last dimension fused with ls_quantize_mxfp4 of its output: the input of
 * the qkv and fc projections of lockstep's block (train.py:50,53: linear(ln(x))) in one pass.
 *   x       [rows, D] LS_F32 or LS_BF16;  gamma, beta [D] fp32 (NULL: 1 and 0)
 *   y_bf16  [rows, D] the normalized rows rounded to bf16 (what the backward pass needs), or NULL
 *   packed  [rows, D/2], sf: MXFP4 of exactly those bf16 values (block 32, reference rounding)
 *   mean, rstd [rows] fp32 statistics for LayerNorm's backward, or NULL
 * D % 256 == 0, D <= 8192.  LayerNorm is computed in fp32 (as torch does under autocast).
 * No single lockstep function does this. */
int ls_layernorm_quantize(const void *x, int x_dtype, const float *gamma, const float *beta, float eps,
                          int64_t rows, int64_t D, void *y_bf16, uint8_t *packed, uint8_t *sf, float *mean,
                          float *rstd, void *stream);

/* Backward of that LayerNorm from the statistics ls_layernorm_quantize kept (what
 * torch.native_layer_norm_backward computes; lockstep leaves it to torch, train.py:50,53):
 *   gx [rows, D] in x's type = rstd (g - mean_D(g) - xhat mean_D(g xhat)),  g = gy gamma,
 *   ggamma [D] = sum over rows of gy xhat,  gbeta [D] = sum over rows of gy  (fp32; either may be NULL)
 *   gy [rows, D] LS_F32 or LS_BF16 (the incoming gradient as the GEMM left it: no cast pass);
 *   gamma NULL means 1.  scratch: ls_layernorm_backward_scratch(rows, D) floats, 16-byte aligned;
 *   the column sums are added in a fixed order (no atomics).  D % 256 == 0, D <= 8192. */
int64_t ls_layernorm_backward_scratch(int64_t rows, int64_t D);
int ls_layernorm_backward(const void *gy, int gy_dtype, const void *x, int x_dtype, const float *mean,
                          const float *rstd, const float *gamma, int64_t rows, int64_t D, void *gx,
                          float *ggamma, float *gbeta, float *scratch, void *stream);

/* Both orientations of one tensor from one read of x [R, C]: what
 * ls_quantize_mxfp4 (packed + scale-factor bytes of x, blocks along C) and
 * ls_quantize_mxfp4_t (of x^T, blocks along R) would write.  For a linear layer
 * whose forward GEMM contracts over C and whose weight-gradient GEMM contracts
 * over R (lockstep quantizes x and x.t().contiguous() separately).
 * R % 128 == 0, C % 128 == 0; all four outputs required.
 *   row_packed [R, C/2], row_sf ls_sf_bytes(R, C); t_packed [C, R/2], t_sf ls_sf_bytes(C, R) */
int ls_quantize_mxfp4_both(const void *x, int x_dtype, int64_t R, int64_t C, int rounding,
                           uint8_t *row_packed, uint8_t *row_sf, uint8_t *t_packed, uint8_t *t_sf,
                           void *stream);

/* Replaces fp4.py:43-54 (_round_to_e2m1) on values already divided by their
 * scale: q fp32 [n] -> codes [n]. */
int ls_round_e2m1(const float *q, int64_t n, int rounding, uint8_t *codes, void *stream);

/* Replaces fp4.py:91-94 (pack_fp4).  n_codes even; 16-byte aligned buffers. */
int ls_pack_fp4(const uint8_t *codes, uint8_t *packed, int64_t n_codes, void *stream);

/* Replaces fp4.py:97-99 (unpack_fp4). */
int ls_unpack_fp4(const uint8_t *packed, uint8_t *codes, int64_t n_bytes, void *stream);

/* Replaces fp4.py:75-78 (dequantize_mxfp4): out = value[code] * scale.
 *   q        codes [rows, K] (is_packed = 0) or packed bytes [rows, K/2] (1)
 *   scale    fp32 [rows, K/block], or NULL when e8m0 is given
 *   e8m0     exponent bytes [rows, K/block], or NULL
 *   out      [rows, K], LS_F32 or LS_BF16 */
int ls_dequantize_mxfp4(const uint8_t *q, int is_packed, const float *scale,
                        const uint8_t *e8m0, int64_t rows, int64_t K, int block,
                        void *out, int out_dtype, void *stream);

/* fp32 power-of-two scales [rows, K/32] -> scale-factor layout bytes.
 * Serves callers of mxfp4_gemm.py:161 that hold fp32 scales.  `bad` (device
 * int32, may be NULL) is incremented for every scale that is not a power of
 * two in [2^-127, 2^127]. */
int ls_scales_to_sf(const float *scale, int64_t rows, int64_t K, uint8_t *sf, int32_t *bad,
                    void *stream);
/* The same for scales [rows, K/block], block = 32 or 16. */
int ls_scales_to_sf_block(const float *scale, int64_t rows, int64_t K, int block, uint8_t *sf,
                          int32_t *bad, void *stream);

/* Packed MXFP4 GEMM  C[M,N] = A[M,K] * W[N,K]^T  with fp32 accumulation.
 * Replaces mxfp4_gemm.py:161-174 (mxfp4_gemm_packed) and the kernel behind it
 * (:116-158); same math as the reference's dequantize + F.linear path
 * (fp4_linear.py:40).
 *   a_pk   [M, K/2] packed E2M1, K-contiguous          bt_pk  [N, K/2] likewise
 *   sfa    scale bytes of A in the scale-factor layout  sfb    likewise for W
 *   c      [M, N] row-major, LS_BF16 (round to nearest even) or LS_F32
 * K % 128 == 0; M and N are free.  All buffers 16-byte aligned.
 * Entry points may be called from several host threads and streams.  A product
 * that the library splits along K (few output tiles, long K; see
 * ls_gemm_set_splits) puts its partial sums in one scratch buffer per device;
 * the library orders such calls on different streams with an event (the later
 * call waits for the earlier one's summation), so they are safe but do not
 * overlap.  On a stream that is being captured into a CUDA graph the product is
 * never split (the capture cannot wait for a user outside it).  Encoded TMA
 * descriptors are cached per host thread. */
int ls_mxfp4_gemm(const uint8_t *a_pk, const uint8_t *bt_pk, const uint8_t *sfa, const uint8_t *sfb,
                  void *c, int out_dtype, int64_t M, int64_t N, int64_t K, void *stream);

/* Dual-batch form: two activation batches against one weight stream, one
 * launch, two outputs.  Replaces dual_gemm.py:244-255 (dual_separate) for the
 * shared-weight case b1 is b2 (train_step.py:52-53) on MXFP4 operands. */
int ls_mxfp4_gemm_dual(const uint8_t *a1_pk, const uint8_t *a2_pk, const uint8_t *bt_pk,
                       const uint8_t *sfa1, const uint8_t *sfa2, const uint8_t *sfb, void *c1,
                       void *c2, int out_dtype, int64_t M, int64_t N, int64_t K, void *stream);

/* ls_mxfp4_gemm and ls_mxfp4_gemm_dual for operands quantized in blocks of 16
 * (fp4.py:57, quantize_mxfp4(x, 16)): scale-factor buffers of
 * ls_sf_bytes_block(rows, K, 16) bytes, everything else as above.  lockstep's own
 * GEMM takes 32 values per scale only (mxfp4_gemm.py:136), so this form has no
 * counterpart there; the tensor core takes it natively
 * (tcgen05.mma.kind::mxf4nvf4.block_scale.block16 with UE8M0 scales). */
int ls_mxfp4_gemm_block16(const uint8_t *a_pk, const uint8_t *bt_pk, const uint8_t *sfa,
                          const uint8_t *sfb, void *c, int out_dtype, int64_t M, int64_t N, int64_t K,
                          void *stream);
int ls_mxfp4_gemm_dual_block16(const uint8_t *a1_pk, const uint8_t *a2_pk, const uint8_t *bt_pk,
                               const uint8_t *sfa1, const uint8_t *sfa2, const uint8_t *sfb, void *c1,
                               void *c2, int out_dtype, int64_t M, int64_t N, int64_t K, void *stream);

/* NVFP4: blocks of 16 E2M1 values under one E4M3 scale.  lockstep states the format in its
 * study of block formats (rig_sm75/quant_sim.cuh:90-97 nv_scale_e2m1, :20-33 quant_e4m3,
 * :57-69 quant_e2m1_code, applied per block as rig_q.cu:348-363) but has no kernel for it.
 *   scale = E4M3(amax / 6) (half-even, saturating at 448; 2^-9 where that is 0; 1.0 for a block
 *   with no positive maximum), code = E2M1 nearest to v / scale, ties to the smaller magnitude.
 *   x         [rows, K] LS_F32 or LS_BF16, 32-byte aligned;  K % 128 == 0
 *   packed    [rows, K/2]
 *   scale_u8  [rows, K/16] E4M3 bytes, or NULL;  scale_f32 the same scales as fp32, or NULL
 *   sf        the scale bytes in the scale-factor layout (ls_sf_bytes_block(rows, K, 16)), or NULL */
int ls_quantize_nvfp4(const void *x, int x_dtype, int64_t rows, int64_t K, uint8_t *packed,
                      uint8_t *scale_u8, float *scale_f32, uint8_t *sf, void *stream);
/* value[code] * scale for NVFP4 operands: out [rows, K] LS_F32 or LS_BF16; K % 16 == 0. */
int ls_dequantize_nvfp4(const uint8_t *packed, const uint8_t *scale_u8, int64_t rows, int64_t K,
                        void *out, int out_dtype, void *stream);
/* ls_mxfp4_gemm_block16 / ls_mxfp4_gemm_dual_block16 with E4M3 scale bytes (the `sf` output of
 * ls_quantize_nvfp4): C = A W^T on tcgen05.mma.kind::mxf4nvf4.block_scale.block16, fp32
 * accumulation.  No counterpart in lockstep. */
int ls_nvfp4_gemm(const uint8_t *a_pk, const uint8_t *bt_pk, const uint8_t *sfa, const uint8_t *sfb,
                  void *c, int out_dtype, int64_t M, int64_t N, int64_t K, void *stream);
int ls_nvfp4_gemm_dual(const uint8_t *a1_pk, const uint8_t *a2_pk, const uint8_t *bt_pk,
                       const uint8_t *sfa1, const uint8_t *sfa2, const uint8_t *sfb, void *c1, void *c2,
                       int out_dtype, int64_t M, int64_t N, int64_t K, void *stream);

/* GEMM whose epilogue also emits MXFP4 of act(C) for a following MXFP4 GEMM
 * (scale blocks of 32 along N), so that C is not re-read by a quantize pass.
 * Covers the chain  _MXFP4Matmul -> F.gelu -> _MXFP4Matmul  of lockstep's
 * block (fp4_linear.py:33-40 twice, train.py:53); no single lockstep function
 * does this.  The quantized values are those a separate pass would see: C
 * rounded to out_dtype, act in fp32, rounded to out_dtype, then
 * ls_quantize_mxfp4's arithmetic.
 *   c         [M, N] or NULL (then only the quantized form is written)
 *   act       0 = none, 1 = GELU, 0.5 x (1 + erf(x / sqrt 2))
 *   q_packed  [M, N/2];  q_sf  ls_sf_bytes(M, N) bytes;  N % 128 == 0 */
int ls_mxfp4_gemm_quant(const uint8_t *a_pk, const uint8_t *bt_pk, const uint8_t *sfa, const uint8_t *sfb,
                        void *c, int out_dtype, int act, uint8_t *q_packed, uint8_t *q_sf, int64_t M,
                        int64_t N, int64_t K, void *stream);

/* Operands in the form of mxfp4_gemm.py:74-87 (mxfp4_gemm_fp8): E4M3 bytes that
 * hold E2M1 values, a [M, K] K-contiguous, b [K, N] N-contiguous, b_scale
 * [K/32, N].  Hopper needs that expansion; the B200 tensor cores take E2M1
 * directly at twice the FP8 rate, so these re-encode the bytes (exactly) to the
 * packed form ls_mxfp4_gemm reads:
 *   ls_e4m3_to_packed    src [rows, K]          -> packed [rows, K/2]   K % 16 == 0
 *   ls_e4m3_to_packed_t  src [K, N]             -> packed [N, K/2]      K % 32 == 0
 *   ls_scales_to_sf_t    scale [K/32, rows] f32 -> scale-factor bytes of a [rows, K] operand
 * A byte that is not one of the 16 images sets bit 1 of the error word that
 * ls_gemm_status reports (LS_EINVAL); the call itself does not synchronise. */
int ls_e4m3_to_packed(const uint8_t *src, int64_t rows, int64_t K, uint8_t *packed, void *stream);
int ls_e4m3_to_packed_t(const uint8_t *src, int64_t K, int64_t N, uint8_t *packed, void *stream);
int ls_scales_to_sf_t(const float *scale, int64_t rows, int64_t K, uint8_t *sf, int32_t *bad, void *stream);

/* Which GEMM kernel the two entry points above launch: 0 = by shape (default),
 * 1 = one CTA per 128 x 256 tile, 2 = CTA pairs on 256 x 256 tiles
 * (cta_group::2), 3 / 5 = one CTA per 128 x 128 / 128 x 64 tile, 6 = CTA pairs
 * on 256 x 192 tiles (accumulators that share no tensor-memory columns).
 * Results are identical; for measurements and tests.  The block-16 and NVFP4
 * entry points follow it too (1 there means 128-column tiles). */
int ls_gemm_set_variant(int variant);

/* Measurement aid, no reference counterpart: launches a kernel that issues only
 * the MMA instruction stream of the CTA-pair GEMM (`rounds` pipeline stages of
 * four 256 x 256 x 64 block-scaled FP4 MMAs per CTA pair, operands resident in
 * shared memory, no loads, copies or epilogue) on every CTA pair of the device.
 * *flop_out (host, may be NULL) receives the FLOPs of the launch; the caller
 * times it with events on `stream`.  The rate it reaches is the ceiling of the
 * tensor pipe at the clock the power cap allows. */
int ls_fp4_mma_peak(int rounds, double *flop_out, void *stream);

/* The GEMM kernels are launched with programmatic stream serialization (default
 * on): a kernel's set-up overlaps the tail of the kernel before it in the
 * stream (this library's quantizers release their dependents at once), and it
 * waits for that kernel before its first load.  0 switches this off (ordinary
 * launches).  For measurements. */
int ls_gemm_set_pdl(int on);

/* K-splitting of the two GEMM entry points: 0 = by shape (default: products of
 * more than 128 rows with few output tiles and a long K, i.e. weight gradients
 * of small layers), 1 = never, 2..16 = that many splits.  A split product
 * accumulates each K range in fp32 on the tensor cores and sums the ranges in
 * ascending order in fp32 before the one rounding to out_dtype.  No reference
 * counterpart (dual_gemm.py:261-289 splits K with atomics); for measurements
 * and tests. */
int ls_gemm_set_splits(int splits);

/* Synchronises the device's error word to the host: returns LS_ETIMEOUT (and
 * clears the word) if any GEMM kernel since the last call abandoned a bounded
 * wait, LS_EINVAL if an E4M3 operand was off the E2M1 grid, LS_OK otherwise.  `status_host` (host int, may be NULL) receives the
 * raw word.  Blocks until prior work on the default stream is done. */
int ls_gemm_status(int *status_host);

/* ---- FP4-compressed gradient all-reduce --------------------------------------
 * Replaces the transport of wire.py:104-138 (Wire._integer: quantize, send each
 * chunk to its owner, owner sums and re-encodes, gather) with the fp4.py codec
 * as payload (block 32, 16 packed bytes + 1 UE8M0 byte): a reduce-scatter and
 * an all-gather done by direct peer stores over NVLink.  One handle per Wire
 * object and rank; at most 8 ranks, one process per GPU.
 *   padded   elements covered, a positive multiple of world * 256
 * Set-up: ls_wire_create, exchange ls_wire_local_handle blobs
 * (ls_wire_handle_bytes each) through the process group, ls_wire_map_peers with
 * all blobs in rank order.  ls_wire_map_local instead connects handles created
 * in one process (single-GPU emulation of several ranks, used by the tests).
 * ls_wire_create allocates the rank's receive arena and synchronises. */
int64_t ls_wire_handle_bytes(void);
int ls_wire_create(int rank, int world, int64_t padded, void **handle);
int ls_wire_destroy(void *handle);
int ls_wire_local_handle(void *handle, void *blob_host);
int ls_wire_map_peers(void *handle, const void *all_blobs_host);
int ls_wire_map_local(void *handle, void *const *handles_host);

/* In-place average of g[numel] (fp32) over the ranks, enqueued on `stream`.
 * res [padded] / ores [padded / world] are the sender / owner error-feedback
 * residuals (wire.py:109-111,128-135), updated in place; NULL disables error
 * feedback.  reverse != 0 sums senders in descending order (wire.py:122-123).
 * Every rank must make the same calls in the same order.
 * ls_wire_send / _reduce / _finish are the three phases of one step as separate
 * launches (a kernel then only waits for kernels of other GPUs; callers that
 * interleave ranks in one process, or that want to start the send early, use
 * them).  ls_wire_allreduce runs the step either as those three launches or as
 * ONE cooperative launch that pipelines sub-ranges of the shards through the
 * three phases (see ls_wire_set_mode); results and wire bytes are the same.
 * A step cannot be captured into a CUDA graph (its epoch advances on the host and
 * travels as a kernel argument): on a capturing stream these calls, and the
 * integer wire's, return LS_ESTATE and launch nothing. */
int ls_wire_send(void *handle, const float *g, int64_t numel, float *res, void *stream);
int ls_wire_reduce(void *handle, float *ores, int reverse, void *stream);
int ls_wire_finish(void *handle, float *g, int64_t numel, void *stream);
int ls_wire_allreduce(void *handle, float *g, int64_t numel, float *res, float *ores, int reverse,
                      void *stream);

/* One step of ALL ranks of a group created in one process on one GPU
 * (ls_wire_map_local) as a single cooperative launch: every rank's CTAs are
 * resident together, so the waits between ranks are met inside the launch.
 * handles / gs / ress / oress: host arrays of `world` entries in rank order
 * (ress / oress may be NULL).  Used by the single-GPU tests of the pipelined
 * kernel; no reference counterpart. */
int ls_wire_allreduce_group(void *const *handles, float *const *gs, int64_t numel, float *const *ress,
                            float *const *oress, int reverse, void *stream);

/* The reference's integer wires (wire.py:104-138: int16, int8, int8 with error
 * feedback) on the same transport: a shared grid per chunk of 64 from the
 * maximum over ranks, exact int32 sum at the owner, owner re-encodes, gather.
 * bits = 8 or 16.  Set-up as for the MXFP4 wire (handles, map).  One step is
 * four launches; ls_wire_int_phase runs one of them (0 publish chunk maxima,
 * 1 quantize and send, 2 owner, 3 decode) for callers that interleave ranks in
 * one process.  res [padded] / ores [padded / world]: residuals or NULL. */
int ls_wire_create_int(int rank, int world, int64_t padded, int bits, void **handle);
int ls_wire_int_phase(void *handle, int phase, float *g, int64_t numel, float *res, float *ores, void *stream);
int ls_wire_int_allreduce(void *handle, float *g, int64_t numel, float *res, float *ores, void *stream);

/* How ls_wire_allreduce runs a step on this handle.  mode: 0 = default (the
 * cooperative launch), 1 = three launches, 2 = one cooperative launch.  subs:
 * sub-ranges each shard is cut into by the cooperative launch (0 = default: 2,
 * 1 on two ranks; else 1..8; lowered until the shard divides into multiples of
 * 256 elements).
 * stagger != 0: the CTAs take the three items of a pipeline step in rotated
 * orders (also the default from three ranks up when subs is 0).  The
 * cooperative launch needs the whole grid resident at once: do not run it
 * beside other kernels that occupy the SMs for long.  ls_wire_mode
 * returns the mode in force (1 or 2).  No reference counterpart. */
int ls_wire_set_mode(void *handle, int mode, int subs, int stagger);
int ls_wire_mode(void *handle);

/* How the groups of a phase are spread over the warps: 0 = fixed shares (the
 * default up to seven ranks), 1 = chunks of 256 groups handed out from a counter
 * in the arena (the default from eight ranks up, where it measured 9 % faster).
 * Results do not depend on it. */
int ls_wire_set_dynamic(void *handle, int on);

/* How long (default 20 s) a kernel waits for a peer's flag before it gives up.
 * A CTA whose wait ran out records it in the status word, stores nothing more
 * (g, the owner residual and the peers' slots keep what they held) and raises
 * no further flag, so every rank that depends on it runs out as well and the
 * step fails on all ranks; the context stays usable.  The sender residual of
 * that step has already been updated: after a time-out call ls_wire_reset on
 * every rank and clear or restore the residuals. */
int ls_wire_set_timeout_us(void *handle, int64_t microseconds);

/* Non-blocking status: a kernel whose wait ran out also sets a word in mapped
 * pinned host memory; this returns LS_ETIMEOUT if that word is set (cleared by
 * ls_wire_status and ls_wire_reset).  Kernels in flight are not waited for. */
int ls_wire_poll_status(void *handle, int *status_host);

/* After a time-out: synchronises this device, clears flags, counters and the
 * status word and rewinds the epoch.  Collective by contract: every rank calls
 * it between two host-side barriers. */
int ls_wire_reset(void *handle);

/* Synchronising: LS_ETIMEOUT (and clears it) if a wire kernel gave up waiting
 * for a peer since the last call.  status_host (host int) may be NULL. */
int ls_wire_status(void *handle, int *status_host);

/* Copies the raw receive slots (which = 0) or gather slots (1) of this rank,
 * world x slot bytes, to a device buffer; *slot_bytes_host receives the slot
 * size.  For byte-exact checks of the wire format. */
int ls_wire_debug_slots(void *handle, int which, uint8_t *out, int64_t *slot_bytes_host, void *stream);

/* MXFP4 linear forward without any allocation: quantizes x [M, K] (LS_BF16 or
 * LS_F32) to MXFP4 and multiplies by a pre-quantized weight (w_pk [N, K/2],
 * w_sf its scale-factor buffer), c [M, N] as in ls_mxfp4_gemm.  x must be
 * 32-byte aligned (the quantizer reads 32-byte words), the other buffers
 * 16-byte aligned, as in ls_quantize_mxfp4 / ls_mxfp4_gemm.  No counterpart
 * in lockstep; added for callers that may not call cudaMalloc (a plugin
 * inside a host's fixed memory plan, a loop that cannot afford an
 * allocation's device-wide synchronisation).  The temporaries between the
 * two kernels live in a 9.3 MB array inside the library image instead:
 *   - limit: M * K <= 2^24 elements and ls_sf_bytes(M, K) <= 2^20; larger
 *     shapes return LS_EINVAL;
 *   - the first call on each device looks the array's address up
 *     (cudaGetSymbolAddress); make that call before any stream capture;
 *   - all calls on a device share the array: calls that may overlap on the GPU
 *     (different streams) race; calls on one stream are safe.
 * status (device int32, may be NULL) receives 0, or non-zero if the GEMM kernel
 * abandoned a bounded wait.  Results equal ls_quantize_mxfp4 + ls_mxfp4_gemm
 * bit for bit. */
int ls_mxfp4_linear_noalloc(const void *x, int x_dtype, const uint8_t *w_pk, const uint8_t *w_sf,
                            void *c, int out_dtype, int64_t M, int64_t N, int64_t K,
                            int32_t *status, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* LOCKSTEP_B200_H */
