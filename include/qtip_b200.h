/*
 * qtip_b200 -- C ABI of the B200 (sm_100a) implementation of the QTIP 2-bit trellis codec hot path.
 *
 * Every entry point takes plain pointers and sizes, launches on the caller's stream, allocates nothing unless it
 * says so, never synchronises the host unless it says so, and returns an int status: 0 = success,
 * QTIP_E_* (< 0) = argument / geometry violation detected before any launch, > 0 = a cudaError_t.
 * qtip_last_error() gives the message of the calling thread's last failure.
 *
 * Device pointers are marked `_d`, host pointers `_h` in the comments. `stream` is a cudaStream_t passed as void*.
 * The comments cite the reference interface (file:line in the reference project) that each function replaces.
 */
#ifndef QTIP_B200_H
#define QTIP_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define QTIP_OK 0
#define QTIP_E_ARG (-1)       /* null pointer, negative size, ... */
#define QTIP_E_GEOMETRY (-2)  /* shape not supported by the codec (multiples of 16/32/128, Hadamard order, ...) */
#define QTIP_E_WORKSPACE (-3) /* workspace too small */
#define QTIP_E_DEVICE (-4)    /* device is not sm_100 or cannot run the cluster kernel */
#define QTIP_E_KERNEL (-5)    /* a kernel reported a bounded wait that ran out (status word set) */
#define QTIP_E_NUMERIC (-6)   /* a factorisation met a matrix that is not positive definite, or produced non-finite values */

const char* qtip_last_error(void);
/* Version of this ABI (bumped on any signature change). */
int qtip_abi_version(void);

/* ------------------------------------------------------------------------------------------------------------
 * Per-device set-up. Uploads the order-12/20/28 Hadamard factors to constant memory, sets the opt-in
 * shared-memory sizes and cluster attributes of the kernels and reads the SM count. Call once per device, with
 * that device current, before any other call and before any stream capture. Idempotent.
 * Replaces initialize_tables() (runtime/cuda/kernels.cu:398-401), device_had() (src/kernels.hip:271-291) and the
 * lazy cudaFuncSetAttribute of launch_fused (runtime/cuda/kernels.cu:201-210).
 */
int qtip_init(void);

/* ------------------------------------------------------------------------------------------------------------
 * Codebook. tlut_h: [512][2] fp16 bits on the HOST (the checkpoint's `tlut` tensor).
 */
/* Encoder table: lut_h2_d[65536] packed half2 (lo = component 0) by quantlut_sym; *lut_rms_h (may be NULL) gets
 * sqrt(mean(lut^2)) in fp64. Synchronous host computation + one H2D copy of the table (the call returns after the copy has been issued from pageable memory, i.e. the host buffer may be reused).
 * Replaces build_codebook()/device_lut() (src/qtip_core.cpp:18-50, src/quantizer.cpp:14-28), with the table as a
 * parameter instead of a compiled-in constant. */
int qtip_encoder_lut(const uint16_t* tlut_h, uint32_t* lut_h2_d, double* lut_rms_h, void* stream);
/* Runtime table: lut_d[1024] bf16x2 words (entry e = sign<<9 | idx, RNE from the fp16 values). Rejects non-finite
 * entries with QTIP_E_ARG. Replaces make_codebook() (runtime/src/qtip.cpp:62-80). */
int qtip_runtime_lut(const uint16_t* tlut_h, uint32_t* lut_d, void* stream);

/* ------------------------------------------------------------------------------------------------------------
 * Encode side: kernel-level interface, argument for argument the k_* wrappers of src/gpu.hpp:276-292.
 */
/* X_d [B][256] f32 -> the 16 x-column feedback step of one LDLQ block. src/viterbi.hip:241-274 (k_ldlq_prep). */
int qtip_k_ldlq_prep(const float* WT_d, const float* hatWT_d, const float* prod_d, const float* L_d, long n, long m,
                     int col0, int bufend, float* X_d, void* stream);
/* One Viterbi forward pass over B sequences. A_d [B][127][1024] u16, final_state_d [B] u16, overlap_d [B] i32 or
 * NULL, roll = 1 reads X rolled by 128. src/viterbi.hip:49-188,275-279 (k_viterbi_fwd). */
int qtip_k_viterbi_fwd(const float* X_d, const int* overlap_d, int roll, int B, uint16_t* A_d,
                       uint16_t* final_state_d, const uint32_t* lut_h2_d, void* stream);
/* Pass-1 backtrace: overlap[b] = state(step 64) >> 4. src/viterbi.hip:197-205,280-283 (k_viterbi_overlap). */
int qtip_k_viterbi_overlap(const uint16_t* A_d, const uint16_t* final_state_d, int B, int* overlap_d, void* stream);
/* Pass-2 backtrace: states into Q_d[(b0+b)*nblk+blk][128] (may be NULL) and decoded values scattered into
 * hatWT_d[(col0+c)*m + 16(b0+b)+r] (may be NULL). src/viterbi.hip:207-229,284-289 (k_viterbi_finish). */
int qtip_k_viterbi_finish(const uint16_t* A_d, const uint16_t* final_state_d, int B, int b0, uint16_t* Q_d, int nblk,
                          int blk, float* hatWT_d, long m, int col0, const uint32_t* lut_h2_d, void* stream);
/* hat_d[b][2i..2i+1] = lut[states_d[b][i]]. src/viterbi.hip:231-238,290-294 (k_decode_states). */
int qtip_k_decode_states(const uint16_t* states_d, int B, float* hat_d, const uint32_t* lut_h2_d, void* stream);

/* Elementwise / layout kernels used around LDLQ and the weight rotation. src/gpu.hpp:222-259, src/kernels.hip:66-314. */
int qtip_k_hadamard_rows(float* X_d, long rows, int n, long ld, int transpose, void* stream);
int qtip_k_transpose(const float* in_d, long rows, long cols, long ld_in, float* out_d, long ld_out, void* stream);
int qtip_k_scale_rows_cols(float* X_d, long rows, long cols, long ld, const float* rs_d, const float* cs_d,
                           void* stream);
int qtip_k_scale(float* X_d, long rows, long cols, long ld, float a, void* stream);
int qtip_k_sub(const float* A_d, const float* B_d, float* D_d, long rows, long cols, long ld, void* stream);
int qtip_k_sumsq(const float* X_d, long rows, long cols, long ld, double* out_d, void* stream);
int qtip_k_dot(const float* A_d, long lda, const float* B_d, long ldb, long rows, long cols, double* out_d,
               void* stream);
int qtip_k_add_diag(float* H_d, long n, float a, void* stream);
int qtip_k_diag_sum(const float* H_d, long n, double* out_d, void* stream);
int qtip_k_split_bf16(const float* X_d, long rows, long cols, long ld_in, uint16_t* hi_d, uint16_t* lo_d,
                      long ld_out, void* stream);
int qtip_k_diff_split_bf16(const float* A_d, const float* B_d, long rows, long cols, long ld, uint16_t* hi_d,
                           uint16_t* lo_d, long ld_out, void* stream);

/* ------------------------------------------------------------------------------------------------------------
 * Encode side: fused interface (what a caller of ldlq_gpu / quantize_group switches to).
 */
/* Bytes of device workspace qtip_quantize_tiles needs for up to max_tiles sequences per call. A batch larger than
 * half the workspace's capacity is processed in chunks that alternate between `stream` and a side stream owned by the
 * library (created on first use per device; joined back into `stream` before the call returns to the host), so that
 * one chunk's backtraces run under the other's forward pass. qtip_ldlq uses side streams the same way for row slices.
 * Consequence: on one device, calls of these entry points from different host threads must not overlap in time. */
size_t qtip_quantize_workspace_bytes(int max_tiles);
/* Two-pass tail-biting quantisation of B sequences: forward(roll) -> overlap -> forward(overlap) -> backtrace, the
 * call sequence of src/quantizer.cpp:59-62 in one entry point. X_d [B][256] f32 -> states_d [B][128] u16 (may be
 * NULL) and hat_d [B][256] f32 decoded values in sequence order (may be NULL). Bit-identical to the four k_* calls. */
int qtip_quantize_tiles(const float* X_d, int B, const uint32_t* lut_h2_d, uint16_t* states_d, float* hat_d,
                        void* workspace_d, size_t workspace_bytes, void* stream);
/* Same, with the outputs of k_viterbi_finish: states into Q_d[(b0+b)*nblk+blk][128] and decoded values scattered
 * through the tile permutation into hatWT_d[(col0+c)*m + 16(b0+b)+r]. Either may be NULL. */
int qtip_quantize_tiles_scatter(const float* X_d, int B, int b0, const uint32_t* lut_h2_d, uint16_t* Q_d, int nblk,
                                int blk, float* hatWT_d, long m, int col0, void* workspace_d, size_t workspace_bytes,
                                void* stream);

/* qtip_quantize_tiles for callers that must not allocate device memory (a process with a frozen memory pool, a plugin
 * working inside an arena it was given, a loop where cudaMalloc's device-wide synchronisation is not acceptable): the
 * scratch is a 16 MiB array inside the library's device module, so no workspace is passed and nothing is allocated,
 * here or by the caller. Limit: B <= 64 sequences per call (QTIP_E_WORKSPACE above that; split the batch). Outputs are
 * bit-identical to qtip_quantize_tiles. The first call on a device looks the array's device address up
 * (cudaGetSymbolAddress): make that first call outside any stream capture, with the device current. All calls on a
 * device share the one array, so two calls whose kernels can overlap on the GPU (different streams) race; calls on
 * one stream are safe. A hand-shake between thread blocks that timed out (outputs then invalid) is reported by
 * qtip_kernel_status(), which reads and clears the status word kept in the array; the call itself does not clear it.
 * This entry point has no counterpart in the reference. */
int qtip_quantize_tiles_noalloc(const float* X_d, int B, const uint32_t* lut_h2_d, uint16_t* states_d, float* hat_d,
                                void* stream);

/* Synchronises `stream`, then returns QTIP_E_KERNEL if a fused call that used this workspace since its last reset
 * reported a timed-out hand-shake between thread blocks (its outputs are then invalid), else QTIP_OK. Each fused call
 * resets the status word when it starts. The reference has no counterpart: its kernels have no inter-block waits. */
int qtip_workspace_status(const void* workspace_d, void* stream);

/* Building blocks of the fused path, exported for profiling and for callers that keep their own scratch: the
 * forward pass of k_viterbi_fwd (src/viterbi.hip:49-188) with the back-pointers stored as one 32-bit word per
 * (8 steps, group): bp_d [B][16][4096] u32, word (b, i >> 3, j) holds step i of group j in bits [4 (7 - (i & 7)), +4);
 * 8-step blocks below first_block are not written (pass 1 needs blocks 8..15 only). status_d: one int, set to 1 if a
 * hand-shake timed out (zero it first). The two backtraces read that layout (k_viterbi_overlap / k_viterbi_finish,
 * src/viterbi.hip:197-229); finish can also write the decoded values in sequence order to hat_d [B][256]. */
int qtip_k_viterbi_fwd_words(const float* X_d, const int* overlap_d, int roll, int B, uint32_t* bp_d, int first_block,
                             uint16_t* final_state_d, const uint32_t* lut_h2_d, int* status_d, void* stream);
int qtip_k_viterbi_overlap_words(const uint32_t* bp_d, const uint16_t* final_state_d, int B, int* overlap_d,
                                 void* stream);
int qtip_k_viterbi_finish_words(const uint32_t* bp_d, const uint16_t* final_state_d, int B, int b0, uint16_t* Q_d,
                                int nblk, int blk, float* hat_d, float* hatWT_d, long m, int col0,
                                const uint32_t* lut_h2_d, void* stream);

/* One linear of a Hessian group, end to end on one stream: the per-linear body of quantize_group
 * (src/quantizer.cpp:236-320). W_d [m][n] f32 (overwritten), L_d [n][n] f32 strictly block-lower (block LDL of the
 * rotated, damped Hessian), su_d [n] / sv_d [m] sign vectors, lut_h2_d / lut_rms from qtip_encoder_lut.
 * Steps: Wr = T_m^T diag(SV) W diag(SU) T_n kept transposed in WT_d [n][m]; Wscale = rms(Wr) / (float(lut_rms) *
 * scale_override), returned in *wscale_out (host) and divided out of WT_d; LDLQ + Viterbi (hatWT_d [n][m], Q_d
 * [(m/16)(n/16)][128] states); bit packing and kernel layout into trellis_d [(m/16)(n/16)][32]. Synchronises the
 * stream once, where the reference reads the rms back. The checkpoint tensors are trellis_d, SU as bf16 and
 * SV * Wscale (src/pipeline.cpp:329-340). Needs m % 32 == 0, n % 128 == 0. */
size_t qtip_quantize_linear_workspace_bytes(long m, long n);
int qtip_quantize_linear(float* W_d, const float* L_d, long m, long n, const float* su_d, const float* sv_d,
                         const uint32_t* lut_h2_d, double lut_rms, double scale_override, float* WT_d, float* hatWT_d,
                         uint16_t* Q_d, uint16_t* trellis_d, float* wscale_out, void* workspace_d, size_t workspace_bytes,
                         void* stream);

/* A whole Hessian group as one call: quantize_group(s, gemm, lins, hp, opt, ...) of src/quantizer.cpp:166-346 on device
 * buffers. The `count` linears share the rotated, damped Hessian HR_d [n][n] (qtip_rotate_hessian), its block LDL factor
 * L_d [n][n] (qtip_block_ldl), the sign vector su_d [n] and creg; each brings its weight W_d [m][n] f32 (overwritten) and
 * its sign vector sv_d [m]. All are rotated into WT_d [n][mt] (mt = sum of the m), quantised by ONE LDLQ + Viterbi run
 * (hatWT_d [n][mt]; states Q_d [(mt/16)(n/16)][128], linear i's tiles starting at tile row (rows before it) / 16), and
 * every linear gets back its Wscale, its trellis words in kernel layout, proxy_rot_reg = tr(D HR D^T) / tr(W HR W^T)
 * and the unregularised proxy (LinearOut, src/quantizer.hpp:34-46). The traces use bf16 hi/lo splits with three partial
 * products on the tensor cores, as the reference does with its library GEMM. Needs n % 128 == 0, every m % 32 == 0.
 * Synchronises the stream several times (rms and traces are read back, as in the reference). Checkpoint tensors per
 * linear: trellis_d, SU as bf16, SV * wscale (src/pipeline.cpp:329-340). */
typedef struct qtip_group_linear {
  float* W_d;           /* in: [m][n] f32, overwritten */
  long m;               /* in: rows */
  const float* sv_d;    /* in: [m] +-1 */
  uint16_t* trellis_d;  /* out: [(m/16)(n/16)][32] u16, kernel layout */
  float wscale;         /* out */
  double proxy;         /* out: unregularised Hessian */
  double proxy_rot_reg; /* out: rotated, regularised Hessian */
} qtip_group_linear;
size_t qtip_quantize_group_workspace_bytes(long n, long mt, long m_max);
int qtip_quantize_group(qtip_group_linear* lins, int count, long n, const float* HR_d, const float* L_d, const float* su_d,
                        double creg, const uint32_t* lut_h2_d, double lut_rms, double scale_override, float* WT_d,
                        float* hatWT_d, uint16_t* Q_d, void* workspace_d, size_t workspace_bytes, void* stream);

/* Hessian side of a group as one call (src/quantizer.cpp:124-152): H_d [n][n] f32 is damped in place by
 * creg = sigma_reg * mean(diag(H)) (returned through creg_out, host) and rotated, HR_d = T_n^T diag(SU) (H + creg I)
 * diag(SU) T_n. scratch_d: one double on the device. Synchronises the stream once (the trace is read back). The block LDL
 * of HR_d is the next step: qtip_block_ldl below, or the reference's host routine (src/qtip_core.cpp:444-487). */
int qtip_rotate_hessian(float* H_d, long n, const float* su_d, double sigma_reg, float* HR_d, double* creg_out,
                        double* scratch_d, void* stream);

/* Block LDL of the rotated, damped Hessian on the GPU in fp64 (the reference does this step on the host:
 * block_ldl_to_L / cholesky_inplace, src/qtip_core.cpp:321-487, called from ldl_hessian, src/quantizer.cpp:154-165).
 * HR_d [n][n] f32 (the output of qtip_rotate_hessian) is symmetrised in fp64, A = (HR + HR^T) / 2, factored A = C C^T by a
 * blocked right-looking Cholesky (128-column panels), and L_d [n][n] f32 receives the strictly block-lower factor with
 * 16 x 16 blocks: L[:, block b] = C[:, block b] inv(C[b, b]) below the diagonal block, zero on and above it -- the L
 * argument of qtip_ldlq. L64_d (may be NULL): the same values before the rounding to fp32. n % 16 == 0.
 * Asynchronous on `stream`; qtip_block_ldl_status then synchronises and returns QTIP_E_NUMERIC if a pivot was not
 * positive or the factor is not finite (the reference's `false`). */
size_t qtip_block_ldl_workspace_bytes(long n);
int qtip_block_ldl(const float* HR_d, long n, float* L_d, double* L64_d, void* workspace_d, size_t workspace_bytes,
                   void* stream);
int qtip_block_ldl_status(const void* workspace_d, void* stream);

/* X_d[(tr * (n/16) + tc)][p] = W_d[16 tr + r][16 tc + c], 16 r + c = perm(p): the sequences of every 16x16 tile of a
 * row-major m x n matrix (row stride ld), i.e. what k_ldlq_prep produces block by block when the Hessian is the
 * identity (L = 0, prod = 0; src/viterbi.hip:241-267). */
int qtip_tiles_from_matrix(const float* W_d, long m, long n, long ld, float* X_d, void* stream);

/* Bytes of device workspace qtip_ldlq needs for an n x m problem (prod, X, Viterbi scratch). */
size_t qtip_ldlq_workspace_bytes(long n, long m);
/* LDLQ with 128-column buffers over WT_d (n x m f32, already scaled) and L_d (n x n f32, strictly block-lower):
 * writes hatWT_d (n x m) and Q_d [(m/16)(n/16)][128]. Replaces ldlq_gpu (src/quantizer.cpp:30-89); the cross-buffer
 * update is an fp32 FMA kernel instead of the split-bf16 library GEMM. Rows of W (columns j of WT) are independent:
 * [j0, j0+mj) restricts the call to that slice of rows (multiple of 16) for row-block sharding over GPUs; pass
 * j0 = 0, mj = m for the whole matrix. */
int qtip_ldlq(const float* WT_d, const float* L_d, long n, long m, long j0, long mj, float* hatWT_d, uint16_t* Q_d,
              const uint32_t* lut_h2_d, void* workspace_d, size_t workspace_bytes, void* stream);

/* Bitstream and kernel layout on the device. src/qtip_core.cpp:194-253 (pack_trellis, unpack_trellis,
 * swizzle_for_kernel, unswizzle_for_kernel; CPU code in the reference, src/quantizer.cpp:306-320). */
int qtip_pack_trellis(const uint16_t* states_d, long B, uint16_t* packed_d, void* stream);
int qtip_unpack_trellis(const uint16_t* packed_d, long B, uint16_t* states_d, void* stream);
int qtip_swizzle_for_kernel(const uint16_t* packed_d, int m, int n, uint16_t* out_d, void* stream);
int qtip_unswizzle_for_kernel(const uint16_t* in_d, int m, int n, uint16_t* packed_d, void* stream);

/* ------------------------------------------------------------------------------------------------------------
 * Layer files of a QTIP checkpoint (safetensors container), host side. Writer: the tensors the quantizer emits per linear
 * (write_layer_file, src/pipeline.cpp:314-352, container src/safetensors.cpp:93-136): `model.layers.<layer>.<name>.`
 * trellis I16 [(m/16)(n/16), 32] (kernel layout), SU BF16 [n], SV F32 [m] (sign * Wscale), tlut F16 [512, 2], rcp I64 = 0,
 * tp_rank I64 = 8; written to <path>.tmp and renamed. Reader: one linear with the loader's checks (load_linear,
 * runtime/src/qtip.cpp:231-289): dtypes, shapes for the expected m x n, finite SU / SV / tlut, rcp == 0; SU comes back
 * as fp32. All pointers are HOST pointers. */
typedef struct qtip_checkpoint_linear {
  const char* name;          /* e.g. "self_attn.q_proj" */
  int m, n;                  /* out features, in features */
  const uint16_t* trellis_h; /* (m/16)(n/16)*32 words */
  const uint16_t* su_bf16_h; /* [n] bf16 bits */
  const float* sv_h;         /* [m] */
  const uint16_t* tlut_h;    /* [512][2] fp16 bits */
} qtip_checkpoint_linear;
int qtip_write_layer_file(const char* path, int layer, const qtip_checkpoint_linear* lins, int count);
int qtip_read_layer_linear(const char* path, int layer, const char* name, int m, int n, uint16_t* trellis_h, float* su_h,
                           float* sv_h, uint16_t* tlut_h);

/* ------------------------------------------------------------------------------------------------------------
 * Decode side: the runtime's QTIP linear operator. runtime/cuda/kernels.hpp:5-24, batch_kernels.hpp:5-8,22-23.
 * bf16 values are passed as uint16_t bit patterns (the reference's B16).
 */
typedef struct qtip_matrix {
  const uint16_t* trellis; /* _d kernel-layout words, (out/16)(in/16)*32 */
  const float* su;         /* _d [in]  +-1 */
  const float* sv;         /* _d [out] sign * Wscale */
  const uint32_t* lut;     /* _d [1024] bf16x2 (qtip_runtime_lut) */
  int in, out;
} qtip_matrix; /* field for field runtime/cuda/kernels.hpp:5-10 (QtipMatrix) */

/* rotated = bf16(hadUt_in(x * SU)). scratch_d >= max(in,out)*tokens f32, rotated_d >= in*tokens bf16.
 * runtime/cuda/kernels.cu:412-427 (qtip_prepare). */
int qtip_prepare(qtip_matrix w, const uint16_t* x_d, float* scratch_d, uint16_t* rotated_d, void* stream, int tokens,
                 int rank_major);
/* z[split][token][stride] = What . rotated (fp32 accumulate, bf16 LUT values), K split into `splits` slices.
 * runtime/cuda/kernels.cu:428-436 (qtip_multiply). */
int qtip_multiply(qtip_matrix w, const uint16_t* rotated_d, float* z_d, int stride, int splits, void* stream,
                  int tokens);
/* y = bf16(SV * hadU_out(sum_splits z)), optional bf16 rounding of z first.
 * runtime/cuda/kernels.cu:437-456 (qtip_finish). */
int qtip_finish(qtip_matrix w, const float* z_d, uint16_t* y_d, float* scratch_d, int round_z, int splits,
                void* stream, int tokens, int rank_major);
/* Same from bf16 z. runtime/cuda/kernels.cu:457-470 (qtip_finish_b16). */
int qtip_finish_b16(qtip_matrix w, const uint16_t* z_d, uint16_t* y_d, float* scratch_d, int tokens, void* stream,
                    int rank_major);
/* prepare + multiply + finish for one token. runtime/cuda/kernels.cu:471-476 (qtip_forward). */
int qtip_forward(qtip_matrix w, const uint16_t* x_d, uint16_t* y_d, float* scratch_d, uint16_t* rotated_d,
                 float* z_d, int round_z, void* stream, int splits);
/* Token-major activations, split-major fp32 products. runtime/cuda/batch_kernels.cu:701-736 (qtip_multiply_batch).
 * `implementation` is accepted for signature compatibility and ignored (one code path per batch regime). */
int qtip_multiply_batch(qtip_matrix w, const uint16_t* x_d, float* z_d, int stride, int splits, int tokens,
                        void* stream, int implementation);
/* Dense bf16 decode of the whole matrix, row-major [out][in]. runtime/cuda/batch_kernels.cu:23-46,737-740. */
int qtip_decode_matrix(qtip_matrix w, uint16_t* out_d, void* stream);
/* x[i] = sum over splits of x[split*n + i]. runtime/cuda/batch_kernels.cu:670-678,831-835 (reduce_products). */
int qtip_reduce_products(float* x_d, size_t elements, int splits, void* stream);
/* y = bf16(sum over splits * scale[i % width]) (scale may be NULL). batch_kernels.cu:684-693,836-839. */
int qtip_reduce_to_b16(const float* x_d, const float* scale_d, uint16_t* y_d, size_t elements, int width, int splits,
                       void* stream);

/* ------------------------------------------------------------------------------------------------------------
 * Fused epilogues of a decode step: the transforms either side of the products with the element-wise work of the
 * residual stream folded in, one kernel each. They take the place of input_transform, output_residual, output_gateup
 * and output_residual_input of the reference's ROCm operator (runtime/include/behemoth/qtip_gpu.hpp:199-285, kernels
 * runtime/src/qtip.hip:713-1163), with the gathered products in this library's layouts ([split][row][n], or rank-major
 * as qtip_finish). Hadamard orders 1, 12 and 28 (widths such as 1024, 8192, 12288, 28672). With few rows every row is
 * spread over K CTAs (one per 1024-chunk), with many rows one CTA holds a whole row; both give the same bits.
 *
 * qtip_input_transform: u[r] = bf16(hadUt_n(SU (.) x'[r])), x' = bf16(x * rsqrt(mean(x^2) + epsilon) * norm) when
 * norm_d (bf16 [n]) is given (the runtime's RMSNorm rounding), else x' = x (then it equals qtip_prepare). x_d bf16
 * [rows][ldx], u_d bf16 [rows][ldu]; xn_d (may be NULL, needs norm_d): x' written out as bf16 [rows][n], the input of the
 * FP8 K/V projections. */
int qtip_input_transform(const uint16_t* x_d, long ldx, const uint16_t* norm_d, float epsilon, const float* su_d, int n,
                         int rows, uint16_t* u_d, long ldu, uint16_t* xn_d, void* stream);
/* qtip_output_residual: state[r] = bf16(state[r] + bf16(SV (.) hadU_n(sum over splits of z))), the o / down epilogue.
 * z_d fp32 [splits][rows][n] (rank_major as qtip_finish), state_d bf16 [rows][n]. */
int qtip_output_residual(const float* z_d, int splits, int rows, int rank_major, const float* sv_d, int n,
                         uint16_t* state_d, void* stream);
/* qtip_output_gateup: h[r] = bf16(silu(g) * u), g = bf16(SVg (.) hadU_F(bf16(zg))), u = bf16(SVu (.) hadU_F(bf16(zu))),
 * silu(g) = g / (1 + exp(-g)). z_d fp32 [splits][rows][2 F] holds the gate products in columns [0, F) and the up
 * products in [F, 2 F) (the stacked gate/up matrix); the sum over splits is rounded to bf16 first (the exchange
 * rounding of these two projections). h_d bf16 [rows][F]. */
int qtip_output_gateup(const float* z_d, int splits, int rows, const float* sv_gate_d, const float* sv_up_d, int features,
                       uint16_t* h_d, void* stream);
/* qtip_output_residual_input: qtip_output_residual followed by qtip_input_transform of the updated state (same width n,
 * with the next block's norm): one kernel when the batch is large enough for whole-row CTAs, else two launches;
 * identical results either way. */
int qtip_output_residual_input(const float* z_d, int splits, int rows, int rank_major, const float* sv_d, int n,
                               uint16_t* state_d, const uint16_t* norm_d, float epsilon, const float* su_d, uint16_t* u_d,
                               long ldu, uint16_t* xn_d, void* stream);

/* Prefill product on the tcgen05 tensor cores: z_d[token][row] (fp32, row stride `stride`) = sum_k w_dense_d[row][k] *
 * x_d[token][k], bf16 operands (w_dense_d is the output of qtip_decode_matrix, x_d the rotated activations). Needs
 * in % 64 == 0 and out % 128 == 0. status_d (one int, may be NULL): set to 2 if a bounded pipeline wait timed out.
 * Replaces the cublasGemmEx call of the >= 128-token path (runtime/cuda/tensor_model.cpp:210-222).
 * Products of more than a few tiles run as one persistent cooperative launch (one CTA per SM) in which the tiles of the
 * last, partial round are split by K ranges and summed in z in a fixed order, so results are reproducible run to run;
 * the per-tile counters of that sum live in a ring of 32 state blocks inside the library, one per launch, so up to 32
 * such products may be in flight on one GPU at a time (streams, graph branches). Capturable; no allocation. */
int qtip_prefill_gemm(const uint16_t* w_dense_d, const uint16_t* x_d, float* z_d, int stride, int in, int out, int tokens,
                      int* status_d, void* stream);
/* The same product with the K range split `splits` ways over the grid, for weights with few rows (the FP8 K/V
 * projections: 1,024 rows are 4 row tiles): z_d[(split * tokens + token) * stride + row] holds the partial sums, to be
 * added by qtip_reduce_to_b16 / qtip_reduce_products / qtip_finish. */
int qtip_prefill_gemm_splitk(const uint16_t* w_dense_d, const uint16_t* x_d, float* z_d, int stride, int in, int out,
                             int tokens, int splits, int* status_d, void* stream);

/* Products for 17 .. a few hundred tokens with the decode fused into the tcgen05 product: the codes are decoded straight
 * into the shared-memory A operand (no dense copy of the weights), 128 rows x 64/128/256 tokens per CTA, K split
 * `splits` ways (z_d[(split * tokens + token) * stride + row], summed by qtip_finish / qtip_reduce_products). Needs
 * in % 64 == 0 and out % 128 == 0. status_d (one int, may be NULL: then a word inside the library, read by
 * qtip_kernel_status) is set to 2 if a bounded pipeline wait timed out. qtip_multiply_batch takes this path by itself
 * above 16 tokens, and from 9 tokens for matrices of up to 16,384 rows (implementation = 0 keeps the 16-tokens-per-pass
 * kernel, 2 forces this one). Takes the place of the
 * 17..127-token kernel of runtime/cuda/batch_kernels.cu:23-288 (launch<0>) and, up to a few hundred tokens, of the dense
 * decode + library GEMM of runtime/cuda/tensor_model.cpp:210-222. */
int qtip_multiply_tc(qtip_matrix w, const uint16_t* rotated_d, float* z_d, int stride, int splits, int tokens,
                     int* status_d, void* stream);
/* Synchronises `stream`; QTIP_E_KERNEL if a kernel launched through an entry point without a status argument
 * (qtip_multiply_batch's tensor-core path, qtip_k_viterbi_fwd, qtip_quantize_tiles_noalloc) reported a bounded wait
 * that ran out since the last call. The status words live inside the library, one set per device; this call reads
 * them on the current device and clears them (clear on read), so an error is reported once. */
int qtip_kernel_status(void* stream);
/* Test hook: stores `value` into one of those status words on the current device (which: 0 = tensor-core kernels,
 * 1 = kernel-level cluster Viterbi, 2 = built-in scratch of qtip_quantize_tiles_noalloc; the last needs one earlier
 * call of that entry point on the device). Lets a test drive the reporting path without making any kernel wait. */
int qtip_debug_set_status(int which, int value, void* stream);

/* FP8 (e4m3) W8A16 projection of the K/V weights kept beside the QTIP linears: y[t][o] = bf16((sum_i fp8(w[o][i]) *
 * bf16(x[t][i])) * scale[o]), fp32 accumulation. w_d [out][in] bytes, scale_d [out], x_d [tokens][in] bf16, y_d
 * [tokens][out] bf16. runtime/cuda/kernels.cu:279-289,477-480 (fp8_forward) and batch_kernels.cu:750-763
 * (fp8_multiply_batch), with the token count as a parameter. */
int qtip_fp8_forward(const uint8_t* w_d, const float* scale_d, const uint16_t* x_d, uint16_t* y_d, int in, int out,
                     int tokens, void* stream);

/* Exact bf16 copy of an e4m3 weight matrix for the prefill product (then qtip_prefill_gemm and qtip_reduce_to_b16 with
 * the per-row scale). runtime/cuda/batch_kernels.cu:694-698,845-848 (decode_fp8_matrix). */
int qtip_decode_fp8_matrix(const uint8_t* w_d, uint16_t* out_d, size_t elements, void* stream);

/* ---- Tensor-parallel decode: rotated-row sharding with the gather fused into the product kernel --------------------
 * Replaces, for the <= 16-token path, Rank::multiply + the ncclAllGather of z of runtime/cuda/tensor_model.cpp:444-502
 * (sharding rule :105-124) and the peer_store copy of runtime/cuda/kernels.cu:402-411. Rank r holds the trellis words of
 * output rows [r out/R, (r+1) out/R) (whole 32-row block-rows, see qtip_matrix) and the full SU / SV / LUT.
 *
 * Every rank owns one exchange buffer of qtip_tp_exchange_bytes() bytes that all ranks can address: base[p] is rank p's
 * buffer as mapped in the calling process (peer access inside one process, or qtip_tp_export / qtip_tp_import between
 * processes). It holds a 256-byte control block and two gathered-product slots, [split][token][out_full] fp32 each.
 *
 * qtip_multiply_push computes this rank's products and stores every finished 32-row piece directly into the slot of ALL
 * ranks (plain peer stores, no staging copy, no collective call); the last CTA then raises this rank's flag on every
 * rank. The wait for the peers (at most about a second, until every rank's flag shows the slot's next epoch) is done by
 * the last CTA of the push kernel itself (wait = 1) or by the one-warp kernel of qtip_gather_wait (wait = 0); the local
 * slot then holds the gathered z for qtip_finish (full matrix geometry, splits as pushed). Epochs live on the device, so the calls can be captured in a CUDA graph and replayed.
 * Rule: consecutive uses of one exchange alternate slot 0 and 1 (also across graph replays), and every rank makes the
 * same sequence of calls. A wait that runs out raises the status word (qtip_tp_status) and leaves the context usable.
 * These entry points allocate nothing and do not synchronise the host; qtip_tp_alloc / qtip_tp_free / qtip_tp_export /
 * qtip_tp_import / qtip_tp_close are set-up calls. */
#define QTIP_TP_MAX_RANKS 8
typedef struct qtip_tp_exchange {
  void* base[QTIP_TP_MAX_RANKS]; /* every rank's exchange buffer (device addresses valid in this process) */
  size_t bytes;                  /* size of each buffer */
  int rank, ranks;
} qtip_tp_exchange;
size_t qtip_tp_exchange_bytes(int out_full, int max_tokens, int max_splits);
/* cudaMalloc + zero fill of an exchange buffer (an allocation of its own, so that it can be exported). */
int qtip_tp_alloc(size_t bytes, void** buf_d);
int qtip_tp_free(void* buf_d);
/* Inter-process handle (64 bytes) of a buffer from qtip_tp_alloc, and its mapping in another process of the same node. */
int qtip_tp_export(void* buf_d, unsigned char handle[64]);
int qtip_tp_import(const unsigned char handle[64], void** peer_d);
int qtip_tp_close(void* peer_d);
/* Zeroes the local control block (epochs, flags, status). All ranks call it, then synchronise with one another on the
 * host, before the first push. */
int qtip_tp_reset(const qtip_tp_exchange* ex, void* stream);
/* Products of w_shard (rows [row0, row0 + w_shard.out) of a matrix of out_full rows) pushed to every rank. tokens <= the
 * max_tokens the exchange was sized for; rotated_d as for qtip_multiply. */
int qtip_multiply_push(qtip_matrix w_shard, const uint16_t* rotated_d, const qtip_tp_exchange* ex, int slot, int out_full,
                       int row0, int splits, void* stream, int tokens, int wait);
/* wait = 0 above: the wait as a kernel of its own (required when several ranks share one GPU: a kernel must never wait
 * for a kernel that is queued behind it). wait = 1: done by the push kernel's last CTA; then only ask for the address. */
int qtip_gather_wait(const qtip_tp_exchange* ex, int slot, const float** z_gathered_d, void* stream);
int qtip_gathered_products(const qtip_tp_exchange* ex, int slot, const float** z_gathered_d);
/* Synchronises `stream`; QTIP_E_KERNEL if a wait of this rank ran out since the last reset. */
int qtip_tp_status(const qtip_tp_exchange* ex, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* QTIP_B200_H */
