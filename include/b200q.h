/*
 * b200q — C ABI of the B200 (sm_100a) calibrate-and-quantize kernels.
 *
 * Every entry point replaces one piece of the llm-compressor hot path; the comment
 * above each declaration cites the reference code it stands in for.  Prefixes:
 *   src/  = src/llmcompressor/ of llm-compressor
 *   CT/   = the compressed_tensors package that llm-compressor calls for the arithmetic
 *
 * Conventions
 *   - plain C, no torch types; tensors are raw DEVICE pointers + shapes + leading
 *     dimensions (in elements) + a dtype code; `stream` is a cudaStream_t passed as void*.
 *   - every function returns int: 0 = ok, <0 = argument / launch error
 *     (see b200q_status), >0 = numeric status reported by the routine.
 *   - nothing is allocated inside unless stated; scratch is passed in by the caller and
 *     sized by the matching *_workspace_bytes query.
 *   - row-major matrices; W is [N rows = output features, K cols = input features].
 */
#ifndef B200Q_H_
#define B200Q_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  B200Q_OK = 0,
  B200Q_ERR_ARG = -1,         /* bad pointer / shape / alignment */
  B200Q_ERR_UNSUPPORTED = -2, /* combination not implemented */
  B200Q_ERR_CUDA = -3,        /* a CUDA call failed; see b200q_last_error */
  B200Q_ERR_DEVICE = -4,      /* kernel reported an internal error (bounded wait expired) */
  B200Q_NOT_POSITIVE_DEFINITE = 1 /* Cholesky met a pivot <= 0 */
} b200q_status;

typedef enum { B200Q_BF16 = 0, B200Q_F32 = 1, B200Q_F16 = 2 } b200q_dtype;
typedef enum { B200Q_QINT = 0, B200Q_QFLOAT = 1 } b200q_qtype;
typedef enum {
  B200Q_TENSOR = 0,
  B200Q_CHANNEL = 1,
  B200Q_GROUP = 2,
  B200Q_TENSOR_GROUP = 3,
  B200Q_BLOCK = 4
} b200q_strategy;
typedef enum { B200Q_SCALE_PLAIN = 0, B200Q_SCALE_FP8 = 1, B200Q_SCALE_E8M0 = 2 } b200q_scale_kind;
typedef enum { B200Q_ZP_INT8 = 0, B200Q_ZP_FP8 = 1, B200Q_ZP_UINT8 = 2 } b200q_zp_kind;

/* Mirror of the weight-side QuantizationArgs (CT/quantization/quant_args.py:157-330). */
typedef struct {
  int32_t num_bits;   /* 4 or 8 */
  int32_t qtype;      /* b200q_qtype */
  int32_t symmetric;  /* 0 / 1 */
  int32_t strategy;   /* b200q_strategy */
  int32_t group_size; /* GROUP / TENSOR_GROUP */
  int32_t block_h;    /* BLOCK */
  int32_t block_w;
  int32_t scale_kind; /* b200q_scale_kind: rounding applied to the scale */
  int32_t zp_kind;    /* b200q_zp_kind: storage type of the zero point */
} b200q_qargs;

const char* b200q_version(void);
/* Text of the last CUDA error seen by the calling thread ("" if none). */
const char* b200q_last_error(void);
/* Number of kernels this library has launched in the process so far (diagnostic; no
 * counterpart in the reference). */
long long b200q_launch_count(void);
/* The streaming quantize / pack kernels that are fed by TMA copies wait for them with a bound.  If
 * such a wait ever ran out on the current device since the last call, this returns
 * B200Q_ERR_DEVICE once (the affected launch left its output incomplete), otherwise B200Q_OK.
 * Synchronises the device.  No counterpart in the reference. */
int b200q_take_wait_status(void);

/* ------------------------------------------------------------------ observers */

/* Per-group / per-channel / per-tensor / per-block min and max of a weight matrix.
 * Replaces flatten_for_calibration + _get_min_max
 * (src/observers/helpers.py:28-102, src/observers/min_max.py:70-74).
 * W: [N,K] of dtype `wdtype`; outputs have W's dtype and the qparam shape
 * ([1], [N,1], [N,K/g], [ceil(N/bh), K/bw]).  TENSOR uses `scratch`
 * (b200q_observe_minmax_workspace_bytes) for the cross-CTA reduction. */
size_t b200q_observe_minmax_workspace_bytes(int64_t N, int64_t K, const b200q_qargs* qa);
int b200q_observe_minmax(const void* W, int wdtype, int64_t N, int64_t K, int64_t ldw,
                         const b200q_qargs* qa, void* min_out, void* max_out, void* scratch,
                         void* stream);

/* Largest magnitude over `count` min/max statistics, folded into *absmax (float, device);
 * call once per member of a fused q/k/v or gate/up group, with *absmax zeroed before the
 * first call.  Then b200q_global_scale_finalize turns it into the NVFP4 tensor scale
 * 448*6/absmax computed in the statistics' dtype, NaN/Inf -> 1, stored as float.
 * Replaces Observer.get_global_scale + generate_gparam
 * (src/observers/base.py:78-96, CT/quantization/utils/helpers.py:309-338). */
int b200q_absmax_accumulate(const void* min_vals, const void* max_vals, int dtype, int64_t count,
                            float* absmax, void* stream);
int b200q_global_scale_finalize(const float* absmax, int stat_dtype, float* global_scale,
                                void* stream);
/* Same accumulation straight from a weight matrix (bf16, K % 8 == 0, 16-byte aligned rows; other
 * inputs return B200Q_ERR_UNSUPPORTED and go through b200q_observe_minmax): the first pass of
 * NVFP4 weight quantisation when no per-group statistics are wanted
 * (src/observers/base.py:78-96 followed by CT/quantization/utils/helpers.py:309-338). */
int b200q_absmax_accumulate_weight(const void* W, int wdtype, int64_t N, int64_t K, int64_t ldw,
                                   float* absmax, void* stream);

/* scale / zero point from statistics.  Replaces calculate_qparams
 * (CT/quantization/utils/helpers.py:50-137) including the MX exponent rule
 * (CT/quantization/utils/mxfp_utils.py:68-128).  `global_scale` may be NULL.
 * scale_out dtype: the statistics' dtype when global_scale is NULL, float otherwise
 * (torch type promotion).  zp_out: 1 byte per entry of kind qa->zp_kind. */
int b200q_qparams(const void* min_vals, const void* max_vals, int stat_dtype, int64_t count,
                  const b200q_qargs* qa, const float* global_scale, void* scale_out,
                  void* zp_out, void* stream);

/* MSE shrink-grid search over per-group ranges.  Replaces _grid_search_mse /
 * _grid_search_eager / _calculate_error (src/observers/mse_quant.py:19-141,255-284).
 * Writes the best min/max per group (W's dtype).  Strategies: GROUP / TENSOR_GROUP (group a power
 * of two, 8..256), CHANNEL and BLOCK (a row / block of up to 51200 elements per CTA, ragged blocks
 * completed with zeros) and TENSOR (one launch per candidate).  scratch:
 * b200q_observe_mse_workspace_bytes (per-candidate "some group improved" flags that reproduce the
 * reference's global early stop; for TENSOR also the search state and per-CTA partial sums). */
int b200q_observe_mse_steps(double maxshrink, double grid); /* int(maxshrink * grid), -1 if invalid */
size_t b200q_observe_mse_workspace_bytes(int64_t N, int64_t K, const b200q_qargs* qa, int steps);
int b200q_observe_mse(const void* W, int wdtype, int64_t N, int64_t K, int64_t ldw,
                      const b200q_qargs* qa, double maxshrink, int patience, double grid,
                      float norm, float expand, void* min_out, void* max_out, void* scratch,
                      void* stream);

/* Same search as b200q_observe_mse for callers that cannot allocate device memory (a process
 * whose memory is already committed to a cache pool, code inside an allocator callback, a
 * plain C host with no allocator).  It has no counterpart in the reference.  The scratch lives
 * in a 4 KiB array inside the library image, which every GPU that loads the library holds
 * until exit; nothing is allocated or freed by this call.
 *   - limit: int(maxshrink * grid) <= 1023 candidates, otherwise B200Q_ERR_ARG is returned
 *     (text in b200q_last_error) and nothing is launched; the TENSOR strategy, whose search needs
 *     more scratch than the array holds, returns B200Q_ERR_UNSUPPORTED;
 *   - the first call on each device looks the array's device address up
 *     (cudaGetSymbolAddress); make that first call outside any stream capture;
 *   - all calls on a device share the one array: calls that overlap on the GPU (different
 *     streams) race on it, so issue them on one stream or order them yourself.  The previous
 *     call's contents are cleared by the search itself. */
int b200q_observe_mse_noalloc(const void* W, int wdtype, int64_t N, int64_t K, int64_t ldw,
                              const b200q_qargs* qa, double maxshrink, int patience, double grid,
                              float norm, float expand, void* min_out, void* max_out, void* stream);

/* ------------------------------------------------------------- quantize / pack */

/* Quantize-dequantize.  Replaces fake_quantize (CT/quantization/lifecycle/forward.py:149-181,
 * forward_helpers.py:113-210).  scale: [qparam shape] of dtype sdtype; zp may be NULL;
 * g_idx (int32 [K], group of each column) may be NULL; global_scale may be NULL.
 * out has W's dtype. */
int b200q_fake_quantize(const void* W, int wdtype, int64_t N, int64_t K, int64_t ldw,
                        const void* scale, int sdtype, const void* zp, const int32_t* g_idx,
                        const float* global_scale, const b200q_qargs* qa, void* out,
                        int64_t ldo, void* stream);

/* Quantize to storage codes and pack.  Replaces quantize() + pack_to_int32 /
 * pack_fp4_to_uint8 / the FP8 / int8 cast of the compressors
 * (CT/quantization/lifecycle/forward.py:37-78, CT/compressors/pack_quantized/helpers.py:20-89,
 *  CT/compressors/nvfp4/helpers.py:34-74, CT/compressors/naive_quantized/base.py:34-82).
 * Output by scheme:  int4 -> int32 [N, ceil(K/8)] ; int8 -> int8 [N,K] when pack_int8==0 or
 * int32 [N, ceil(K/4)] when pack_int8==1 ; fp8 -> e4m3 bytes [N,K] ; fp4 -> uint8 [N,K/2]. */
int b200q_quantize_pack(const void* W, int wdtype, int64_t N, int64_t K, int64_t ldw,
                        const void* scale, int sdtype, const void* zp, const int32_t* g_idx,
                        const float* global_scale, const b200q_qargs* qa, int pack_int8,
                        void* out, void* stream);

/* Asymmetric zero points packed along dim 0 (pack_to_int32(zp, bits, packed_dim=0),
 * CT/compressors/pack_quantized/base.py:70-73): zp int8 [N,G] -> int32 [ceil(N*bits/32), G]. */
int b200q_pack_zero_points(const int8_t* zp, int64_t N, int64_t G, int num_bits, int32_t* out,
                           void* stream);

/* Scale storage: kind FP8 -> e4m3 bytes (NVFP4PackedCompressor._compress_scale,
 * CT/compressors/nvfp4/base.py:33-38); kind E8M0 -> 127+floor(log2 s) (compress_mx_scale,
 * CT/compressors/mx_utils.py:18-30). */
int b200q_compress_scale(const void* scale, int sdtype, int64_t count, int scale_kind,
                         uint8_t* out, void* stream);

/* One pass over W for round-to-nearest weight quantisation without a global scale
 * (int4/int8 group or channel, FP8 channel, MXFP4, MXFP8): statistics, qparams, codes and
 * packing fused, W read once.  Equivalent to memoryless_minmax observer -> calculate_qparams
 * -> compressor.compress (src/modifiers/quantization/quantization/base.py:83-108 followed by
 * CT/compressors/base.py:145-168).  scale_out has W's dtype; scale_store (may be NULL)
 * receives the compressed scale bytes for MX formats; zp_out may be NULL when symmetric. */
int b200q_rtn_quantize_pack(const void* W, int wdtype, int64_t N, int64_t K, int64_t ldw,
                            const b200q_qargs* qa, void* scale_out, void* zp_out,
                            uint8_t* scale_store, void* out, void* stream);

/* NVFP4 with a known global scale, one pass: per-16 amax -> FP8 block scale -> E2M1 codes.
 * Same result as observer -> calculate_qparams(global_scale) -> NVFP4PackedCompressor.compress
 * (CT/compressors/nvfp4/base.py:40-72).  scale_out: W-dtype values on the FP8 grid [N,K/16];
 * scale_store: e4m3 bytes [N,K/16]; out: uint8 [N,K/2]. */
int b200q_nvfp4_quantize_pack(const void* W, int wdtype, int64_t N, int64_t K, int64_t ldw,
                              const float* global_scale, void* scale_out, uint8_t* scale_store,
                              void* out, void* stream);

/* ------------------------------------------------------------------ GPTQ: Hessian */

/* H_lower += alpha * X^T X  (fp32 accumulate, bf16 X [T,K] row-major, K contiguous).
 * Only tiles on or below the diagonal are written; b200q_hessian_finalize mirrors them.
 * Replaces accumulate_hessian (src/modifiers/gptq/gptq_quantize.py:28-64; alpha = 2).
 * Requires K % 8 == 0 and 16-byte aligned X, ldx % 8 == 0 (the Python front end pads other
 * widths).  `status` (device int, may be NULL; never cleared by the call) receives non-zero if
 * a bounded wait inside the kernel expired: H is then incomplete.  Launches clusters of
 * two CTAs (tcgen05.mma.cta_group::2); B200Q_SYRK_SINGLE_CTA=1 in the environment selects the
 * single-CTA kernel. */
int b200q_hessian_syrk(const void* X, int64_t T, int64_t K, int64_t ldx, float* H, int64_t ldh,
                       float alpha, int* status, void* stream);

/* H[i][j] = H[j][i] = H_lower[i][j] * scale for j <= i.  The division of
 * src/modifiers/gptq/base.py:336 (H / num_samples) is scale = 1/n. */
int b200q_hessian_finalize(float* H, int64_t K, int64_t ldh, float scale, void* stream);

/* b200q_hessian_syrk splits long token ranges over several thread blocks per tile and adds the
 * partial tiles with floating-point atomics: H is then reproducible to rounding error (about 1e-7
 * relative), not bit for bit, and a GPTQ solve on it may differ in a few codes from run to run.
 * b200q_set_reproducible(1) makes every later call give whole tiles to a thread-block pair, which
 * adds the token splits of its tile one after the other without atomics (bitwise reproducible
 * results for equal inputs and call sequences; slower for narrow Hessians).  Process-wide. */
void b200q_set_reproducible(int on);
int b200q_get_reproducible(void);

/* ------------------------------------------------------------------ GPTQ: solve */

/* perm = stable argsort(diag(H), descending)  (gptq_quantize.py:267-278). */
int b200q_actorder_perm(const float* H, int64_t K, int64_t ldh, int32_t* perm, void* stream);
/* Wf[:, j] = float(W[:, perm[j]]) (perm NULL = identity): the fp32 working copy of
 * gptq_quantize.py:92-96,107-108. */
int b200q_gather_columns_f32(const void* W, int wdtype, int64_t N, int64_t K, int64_t ldw,
                             const int32_t* perm, float* Wf, int64_t ldf, void* stream);
/* Hp[i][j] = H[perm[i]][perm[j]]  (gptq_quantize.py:278). */
int b200q_permute_hessian(const float* H, int64_t K, int64_t ldh, const int32_t* perm, float* Hp,
                          int64_t ldp, void* stream);
/* out[:, perm[j]] = cast(Wf[:, j]) (perm NULL = identity): un-permute and cast back
 * (gptq_quantize.py:247-252). */
int b200q_scatter_columns_cast(const float* Wf, int64_t N, int64_t K, int64_t ldf,
                               const int32_t* perm, void* out, int odtype, int64_t ldo,
                               void* stream);

/* Dead columns and dampening (gptq_quantize.py:143-152): where diag(H)==0 set H_ii=1 and
 * W[:,i]=0; then H_ii += percdamp * mean(diag H). */
int b200q_gptq_prepare(float* H, int64_t K, int64_t ldh, float* Wf, int64_t N, int64_t ldf,
                       float percdamp, void* stream);
/* W[:, i] = 0 where diag[i * diag_stride] == 0 (gptq_quantize.py:144-146), for modules that
 * share one Hessian (q/k/v, gate/up): `diag` is the diagonal saved before b200q_gptq_prepare. */
int b200q_gptq_zero_dead_columns(const float* diag, int64_t diag_stride, int64_t K, float* Wf,
                                 int64_t N, int64_t ldf, void* stream);

/* In place: H (symmetric positive definite, full storage) -> upper-triangular U with
 * U^T U = H^-1, strictly-lower part zeroed.  Stands in for cholesky -> cholesky_inverse ->
 * cholesky(upper=True) (gptq_quantize.py:153-156).  status: four device ints, zeroed by the
 * caller; status[0] is set to B200Q_NOT_POSITIVE_DEFINITE (status[1] to the first bad column
 * + 1) if a pivot is <= 0, status[2] to B200Q_ERR_DEVICE if a bounded wait expired; the
 * caller then takes the reference's identity fallback (:157-164).  workspace:
 * b200q_gptq_factor_workspace_bytes(K) bytes.
 *
 * Streams: all work is ordered on `stream`.  Unless the environment has B200Q_LOOKAHEAD=0, the
 * bulk of each rank-128 update is launched on a helper stream that the library creates once per
 * (device, `stream`) and keeps; it is forked from and joined to `stream` with events before the
 * call returns, so callers see ordinary stream semantics (b200q_gptq_sweep does the same).  The
 * helper streams and the per-thread cache of TMA descriptors are the library's only hidden
 * state; they hold no device memory. */
size_t b200q_gptq_factor_workspace_bytes(int64_t K);
int b200q_gptq_factor(float* H, int64_t K, int64_t ldh, void* workspace, int* status,
                      void* stream);

/* The float32-accurate tensor-core GEMM that the factorisation and the sweep use for their
 * rank-128 updates (tcgen05 kind::tf32, three MMAs per product on hi/lo splits of the operands):
 *   C[M,N] = beta*C + alpha * A[M,Kd] * (trans_b ? B[N,Kd]^T : B[Kd,N]),   Kd <= 128.
 * Stands in for the torch.matmul calls of gptq_quantize.py:236,244 and the cuSOLVER updates
 * behind :153-155.  lower_tiles != 0 restricts the update to 128x128 tiles with column block <=
 * row block.  status (device int, may be NULL) receives B200Q_ERR_DEVICE if a bounded wait
 * expired.  workspace: b200q_gemm_tf32x3_workspace_bytes. */
size_t b200q_gemm_tf32x3_workspace_bytes(int64_t M, int64_t N, int64_t Kd);
int b200q_gemm_tf32x3(int trans_b, const float* A, int64_t lda, const float* B, int64_t ldb, float* C,
                      int64_t ldc, int64_t M, int64_t N, int64_t Kd, float alpha, float beta,
                      int lower_tiles, void* workspace, int* status, void* stream);

/* Blockwise column sweep (gptq_quantize.py:166-245): for each block of `blocksize` columns,
 * column by column: q = fake_quantize(w); loss += (w-q)^2/d^2/2; err = (w-q)/d;
 * W_block[:, i:] -= err x U[i, i:]; then W[:, after] -= Err @ U[block, after].
 * Wf fp32 [N,K] in/out (ends as the fake-quantised weight); U from b200q_gptq_factor
 * (NULL = identity: round to nearest); scale [N,G] / [N,1] / [1] of dtype sdtype; zp may be
 * NULL; col_group int32 [K] (group of each column; NULL = column/group_size); losses float [N]
 * (overwritten).  workspace: b200q_gptq_sweep_workspace_bytes(N, K, blocksize) bytes, 16-byte
 * aligned.  Its first int32 is a status word: the call clears it, and a bounded wait that ran
 * out inside one of the trailing-update GEMMs sets it to B200Q_ERR_DEVICE (W is then
 * incomplete); read it after the stream has reached the end of the call. */
size_t b200q_gptq_sweep_workspace_bytes(int64_t N, int64_t K, int blocksize);
int b200q_gptq_sweep(float* Wf, int64_t N, int64_t K, int64_t ldf, const float* U, int64_t ldu,
                     const void* scale, int sdtype, const void* zp, const int32_t* col_group,
                     const float* global_scale, const b200q_qargs* qa, int blocksize,
                     float* losses, void* workspace, void* stream);

/* Many small problems of one shape per launch (the experts of a mixture-of-experts layer, whose
 * per-module calls of gptq_quantize.py:67-264 are otherwise bound by launch overhead).  Every
 * pointer argument is a DEVICE array of `count` device pointers.
 *
 * b200q_gptq_factor_batched: H[i] (K x K floats, leading dimension ldh) -> U[i] in place, as
 * b200q_gptq_factor does, one thread block per problem; K <= 4096 (meant for K <= 2048).
 * scratch[i]: K*K floats each (b200q_gptq_factor_batched_workspace_bytes(K, count) in total).
 * status: int32 [count][4], cleared by the call; status[i][0] = B200Q_NOT_POSITIVE_DEFINITE and
 * status[i][1] = first bad column + 1 (in reversed column order) when problem i failed.
 *
 * b200q_gptq_sweep_batched: the sweep of b200q_gptq_sweep for `count` weights of one shape
 * [N, K], one quantisation scheme and one scale dtype, blocksize 128.  A thread block carries 64
 * rows of one weight through every column block, trailing updates included (float32 FMA).
 * U may be NULL (identity for all) and so may zp, col_group and global_scale (absent for all);
 * losses[i]: float [N]. */
/* The gather / scatter around the batched sweep, for `count` weights of one shape (device arrays
 * of device pointers): Wf[i] = float32 copy of W[i] with its columns permuted by perm[i] (perm
 * NULL: identity for all) and the columns whose dead_diag[i][c] is 0 zeroed (dead_diag NULL: none),
 * as b200q_gather_columns_f32 followed by b200q_gptq_zero_dead_columns; and the way back,
 * out[i][:, perm[i][c]] = cast(Wf[i][:, c]), as b200q_scatter_columns_cast. */
int b200q_gather_columns_f32_batched(const void* const* W, int wdtype, const int32_t* const* perm,
                                     const float* const* dead_diag, float* const* Wf, int count, int64_t N,
                                     int64_t K, int64_t ldw, int64_t ldf, void* stream);
int b200q_scatter_columns_cast_batched(const float* const* Wf, const int32_t* const* perm, void* const* out,
                                       int odtype, int count, int64_t N, int64_t K, int64_t ldf, int64_t ldo,
                                       void* stream);
size_t b200q_gptq_factor_batched_workspace_bytes(int64_t K, int count);
int b200q_gptq_factor_batched(float* const* H, float* const* scratch, int count, int64_t K, int64_t ldh,
                              int* status, void* stream);
int b200q_gptq_sweep_batched(float* const* W, const float* const* U, const void* const* scale, int sdtype,
                             const void* const* zp, const int32_t* const* col_group,
                             const float* const* global_scale, float* const* losses, int count, int64_t N,
                             int64_t K, int64_t ldw, int64_t ldu, const b200q_qargs* qa, int blocksize,
                             void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200Q_H_ */
