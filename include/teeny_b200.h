/*
 * teeny_b200 -- C ABI of the sm_100a (B200) backend for teenygrad's GEMM / attention / Qwen3-forward path.
 *
 * Every entry point
 *   - takes DEVICE pointers owned by the caller, sizes as plain ints, and a CUDA stream last;
 *   - enqueues its kernels on that stream and returns without synchronising;
 *   - allocates nothing (kernels that need scratch take it as an argument, like the `global_scratch` pointer the
 *     reference's launcher appends to every kernel's arguments, drivers/teeny-cuda/src/device/mod.rs:336-362);
 *   - returns 0 on success, a negative TEENY_ERR_* code for a rejected call, or a positive cudaError_t value.
 *
 * Names and leading argument order are those of the reference's kernel entry points (symbol
 * "{kernel_fn}_entry_point", macros/teeny-macros/src/macros/kernel.rs:544,600-615); the reference monomorphises per
 * dtype, C has no generics, hence the _f32 / _bf16 suffixes.  bf16 values are raw 16-bit patterns (uint16_t here).
 * Reference paths below are relative to the teenygrad repository root.
 */
#ifndef TEENY_B200_H_
#define TEENY_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* teeny_stream_t; /* cudaStream_t / CUstream */
typedef uint16_t teeny_bf16;

enum {
  TEENY_OK = 0,
  TEENY_ERR_BAD_ARG = -1,     /* null pointer, non-positive size, unsupported shape */
  TEENY_ERR_ALIGNMENT = -2,   /* pointer / stride alignment the kernel needs is not met */
  TEENY_ERR_SCRATCH = -3,     /* scratch missing or too small */
  TEENY_ERR_DRIVER = -4,      /* CUDA driver entry point unavailable or tensor-map encode failed */
  TEENY_ERR_DEVICE_WAIT = -5, /* a bounded wait inside a kernel expired (see teeny_device_error) */
  TEENY_ERR_NCCL = -6,
  TEENY_ERR_STATIC_LIMIT = -7 /* shape needs more scratch than a no-allocation entry point has built in */
};

int teeny_version(void);
const char* teeny_status_string(int status);
/* Synchronises the device and returns the error word kernels set when one of their bounded waits expires
 * (0 = none).  clear != 0 resets it.  The reference surfaces device faults by cuCtxSynchronize after each launch
 * (drivers/teeny-cuda/src/device/mod.rs:369-381); here launches stay asynchronous and this is the explicit check. */
int teeny_device_error(int clear);
/* Kernels this library has launched in this process so far (a kernel recorded into a CUDA graph counts when it is
 * recorded and again on every replay by teeny_qwen3_decode_replay); reset != 0 returns the count and zeroes it.
 * Library kernels of others (NCCL) are not counted.  For callers that want to see that the CUDA path ran, as the
 * reference's launcher can by counting its cuLaunchKernel calls (drivers/teeny-cuda/src/device/mod.rs:315-388). */
unsigned long long teeny_launch_count(int reset);

/* ---------------------------------------------------------------------------------------------------------------
 * GEMM
 * ------------------------------------------------------------------------------------------------------------- */
/* C[M,N] = A[M,K] @ B[K,N], all row-major.  Replaces matmul_forward, kernels/teeny-kernels/src/math/gemm.rs:44-108
 * (arguments a_ptr, b_ptr, c_ptr, M, N, K, :52-59).  bf16: f32 accumulate.  f32: f32 accuracy either way -- with
 * global_scratch of at least teeny_matmul_f32_scratch_bytes(M, N, K) bytes (and K, N multiples of 8, 16-byte aligned
 * pointers) on the tensor cores, every operand split into two bf16 terms and three products accumulated in f32 (the
 * split the reference's DSL calls TF32x3, kernels/teeny-triton/src/triton/mod.rs:76-83; its kernel uses one TF32 pass,
 * math/gemm.rs:95, which the 1e-4 bar rules out); with global_scratch NULL by f32 FMAs on the CUDA cores. */
int matmul_forward_entry_point_f32(const float* a, const float* b, float* c, int M, int N, int K,
                                   void* global_scratch, size_t global_scratch_bytes, teeny_stream_t stream);
int matmul_forward_entry_point_bf16(const teeny_bf16* a, const teeny_bf16* b, teeny_bf16* c, int M, int N, int K,
                                    void* global_scratch, size_t global_scratch_bytes, teeny_stream_t stream);

/* Y[M,N] = X[M,K] @ W[N,K]^T (+ bias[N], NULL for none); strides in elements.  Replaces linear_forward,
 * kernels/teeny-kernels/src/nn/mlp/linear.rs:22-116 (arguments :31-45, packed by RuntimeOp for LinearForward
 * :275-307).  bf16: when stride_xk == stride_wk == stride_yn == 1 and rows are 16-byte aligned the tcgen05 kernel
 * runs; other layouts run on a CUDA-core kernel.  With M <= 128 the tcgen05 kernel splits K across the CTAs of a
 * thread-block cluster and sums the partial tiles through distributed shared memory, so it needs no global scratch:
 * global_scratch is accepted for signature parity with the reference and may be NULL. */
int linear_forward_entry_point_f32(const float* x, const float* w, const float* bias, float* y, int M, int N, int K,
                                   int stride_xm, int stride_xk, int stride_wn, int stride_wk, int stride_ym,
                                   int stride_yn, void* global_scratch, size_t global_scratch_bytes,
                                   teeny_stream_t stream);
int linear_forward_entry_point_bf16(const teeny_bf16* x, const teeny_bf16* w, const teeny_bf16* bias, teeny_bf16* y,
                                    int M, int N, int K, int stride_xm, int stride_xk, int stride_wn, int stride_wk,
                                    int stride_ym, int stride_yn, void* global_scratch, size_t global_scratch_bytes,
                                    teeny_stream_t stream);
size_t teeny_matmul_f32_scratch_bytes(int M, int N, int K);
/* Global scratch the bf16 GEMM wants at this shape.  Always 0 (split-K is reduced on chip); kept so hosts that size
 * a scratch arena per shape, as the reference's launcher does, have one call to ask. */
size_t teeny_gemm_scratch_bytes(int M, int N, int K);

/* ---------------------------------------------------------------------------------------------------------------
 * Attention
 * ------------------------------------------------------------------------------------------------------------- */
/* O = softmax(Q K^T * scale) V, L = logsumexp; q/k/v/o [BH, n_ctx, head_dim] contiguous, l [BH, n_ctx_q] f32;
 * non-causal, one KV head per query head.  Replaces flash_attention2_forward,
 * kernels/teeny-kernels/src/nn/attention/flash_attn2.rs:53-156 (arguments :54-63).  In the reference BH is the
 * launch grid's y extent and HEAD_DIM a const generic (tests/test_flash_attn2.rs:120-124); here they are the two
 * arguments after neg_inf.  neg_inf is accepted for ABI parity and ignored.  l may be NULL. */
int flash_attention2_forward_entry_point_f32(const float* q, const float* k, const float* v, float* o, float* l,
                                             int n_ctx_q, int n_ctx_k, float softmax_scale, float neg_inf, int bh,
                                             int head_dim, teeny_stream_t stream);
int flash_attention2_forward_entry_point_bf16(const teeny_bf16* q, const teeny_bf16* k, const teeny_bf16* v,
                                              teeny_bf16* o, float* l, int n_ctx_q, int n_ctx_k, float softmax_scale,
                                              float neg_inf, int bh, int head_dim, teeny_stream_t stream);

/* Strided, grouped-query, optionally causal attention.  The graph op it implements is
 * Op::MultiHeadAttention{q_num_heads, kv_num_heads} (core/teeny-core/src/graph/mod.rs:1278), which the reference
 * leaves unlowered (kernels/teeny-kernels/src/graph/mod.rs:2603-2607).  Element strides for (batch, head, sequence);
 * head_dim is contiguous.  Causal masks are aligned to the end of the keys: query i sees keys j <= i + Skv - Sq. */
typedef struct {
  int B, Hq, Hkv, Sq, Skv, D;
  long long q_sb, q_sh, q_ss;
  long long k_sb, k_sh, k_ss;
  long long v_sb, v_sh, v_ss;
  long long o_sb, o_sh, o_ss;
  float scale;
  int causal;
} teeny_attn_shape;
/* Prefill: D == 128 runs the tcgen05 kernel; other head dims (<= 256) a CUDA-core kernel.  lse [B, Hq, Sq] or NULL. */
int teeny_flash_attn_fwd_bf16(const teeny_bf16* q, const teeny_bf16* k, const teeny_bf16* v, teeny_bf16* o,
                              float* lse, const teeny_attn_shape* shape, teeny_stream_t stream);
/* Decode: Sq == 1, D == 128.  shape->Skv is the cache capacity; the live length is *kv_len_dev (device int, lets a
 * captured CUDA graph advance) or kv_len when kv_len_dev is NULL.  scratch >= teeny_attn_decode_scratch_bytes(). */
int teeny_flash_attn_decode_bf16(const teeny_bf16* q, const teeny_bf16* k, const teeny_bf16* v, teeny_bf16* o,
                                 const teeny_attn_shape* shape, int kv_len, const int* kv_len_dev, void* scratch,
                                 size_t scratch_bytes, teeny_stream_t stream);
size_t teeny_attn_decode_scratch_bytes(int B, int Hq, int D, int max_kv);
/* Decode attention for callers that cannot provide scratch memory.  (No counterpart in the reference, whose launcher
 * allocates scratch for every launch.)  Meant for hosts where a device allocation is not an option once serving has
 * started: the framework's pool already owns all of HBM, or a cudaMalloc -- which synchronises the device -- would
 * stall every stream in the decode loop.  Same arguments and result as teeny_flash_attn_decode_bf16 minus the scratch:
 * the split-KV partials go to an 8 MiB array that is part of the library image (each GPU that loads the library keeps
 * those 8 MiB until the process ends).  Shapes with teeny_attn_decode_scratch_bytes(B, Hq, D, shape->Skv) above
 * teeny_attn_decode_static_limit() return TEENY_ERR_STATIC_LIMIT.  The call allocates nothing.  Its first call on a
 * device looks up the array's device address (one runtime query); make that first call before any stream capture.
 * Every call on a device uses the same array (contents are whatever the previous call left; none of it has to be
 * zero), so calls that could run at the same time on the GPU, e.g. on two streams, race: serialise them. */
int teeny_flash_attn_decode_bf16_static(const teeny_bf16* q, const teeny_bf16* k, const teeny_bf16* v, teeny_bf16* o,
                                        const teeny_attn_shape* shape, int kv_len, const int* kv_len_dev,
                                        teeny_stream_t stream);
size_t teeny_attn_decode_static_limit(void);

/* ---------------------------------------------------------------------------------------------------------------
 * Normalisation and elementwise
 * ------------------------------------------------------------------------------------------------------------- */
/* rrms[r] = 1/sqrt(mean(x[r,:]^2) + eps); y = x * rrms * weight.  Replaces rms_norm_forward,
 * kernels/teeny-kernels/src/nn/norm/rmsnorm.rs:40-118 (arguments :41-48).  rrms may be NULL.
 * bf16 variant: statistics in f32, normalised row rounded to bf16, then multiplied by the bf16 weight (the cast
 * points of the Qwen3 graph the reference records, support/teeny-torch/tests/data/qwen3_1.bin.gz). */
int rms_norm_forward_entry_point_f32(const float* x, float* y, const float* weight, float* rrms, int M, int N,
                                     float eps, teeny_stream_t stream);
int rms_norm_forward_entry_point_bf16(const teeny_bf16* x, teeny_bf16* y, const teeny_bf16* weight, float* rrms,
                                      int M, int N, float eps, teeny_stream_t stream);
/* y = x / (1 + exp(-x)).  Replaces silu_forward, kernels/teeny-kernels/src/nn/activation/sigmoid.rs:120-156. */
int silu_forward_entry_point_f32(const float* x, float* y, int n, teeny_stream_t stream);
int silu_forward_entry_point_bf16(const teeny_bf16* x, teeny_bf16* y, int n, teeny_stream_t stream);
/* out = a * b.  Replaces elemwise_mul_forward, kernels/teeny-kernels/src/nn/tensor/elemwise_binary.rs:206-250. */
int elemwise_mul_forward_entry_point_f32(const float* a, const float* b, float* out, int n, teeny_stream_t stream);
int elemwise_mul_forward_entry_point_bf16(const teeny_bf16* a, const teeny_bf16* b, teeny_bf16* out, int n,
                                          teeny_stream_t stream);
/* out = a + b.  Replaces elemwise_add_forward, kernels/teeny-kernels/src/nn/tensor/elemwise_add.rs:29-69. */
int elemwise_add_forward_entry_point_f32(const float* a, const float* b, float* out, int n, teeny_stream_t stream);
int elemwise_add_forward_entry_point_bf16(const teeny_bf16* a, const teeny_bf16* b, teeny_bf16* out, int n,
                                          teeny_stream_t stream);
/* Row softmax.  Replaces softmax_forward, kernels/teeny-kernels/src/nn/activation/softmax.rs:39-69. */
int softmax_forward_entry_point_f32(const float* x, float* y, int n_rows, int n_cols, teeny_stream_t stream);
int softmax_forward_entry_point_bf16(const teeny_bf16* x, teeny_bf16* y, int n_rows, int n_cols,
                                     teeny_stream_t stream);

/* Fused kernels of the Qwen3 layer.  The reference has no fused forms: Op::Fused and Op::RotaryEmbedding do not lower
 * (kernels/teeny-kernels/src/graph/mod.rs:2953-2966, 2598-2602); each fuses the ops named. */
/* residual <- residual + x (bf16 add); y <- rms_norm(residual).  Fuses elemwise_add_forward + rms_norm_forward. */
int teeny_add_rms_norm_bf16(const teeny_bf16* x, teeny_bf16* residual, teeny_bf16* y, const teeny_bf16* weight, int M,
                            int N, float eps, teeny_stream_t stream);
/* out[t, i] = silu(gate_up[t, i]) * gate_up[t, inter + i].  Fuses silu_forward + elemwise_mul_forward. */
int teeny_silu_mul_bf16(const teeny_bf16* gate_up, long long ld, teeny_bf16* out, int T, int inter,
                        teeny_stream_t stream);
/* Y[M, N/2] = silu(X Wg^T) * (X Wu^T) in one GEMM: w is [N, K] with the gate and up projection rows interleaved in
 * blocks of 64 channels (rows 128b .. 128b+63 = gate channels 64b .., rows 128b+64 .. 128b+127 = up channels 64b ..),
 * N a multiple of 128.  Fuses linear_forward (twice) + silu_forward + elemwise_mul_forward; rounding points are those
 * of the unfused bf16 graph.  Strides in elements; unit inner strides, 16-byte aligned rows. */
int teeny_linear_swiglu_bf16(const teeny_bf16* x, long long ldx, const teeny_bf16* w, long long ldw, teeny_bf16* y,
                             long long ldy, int M, int N, int K, teeny_stream_t stream);
/* Weight-only FP8 linear: Y[M, N] = X[M, K] @ W^T (+ bias) with X, Y bf16 and W in the "float-quantized"
 * compressed-tensors layout the reference's quantiser writes (utilities/teeny-quant/src/format.rs:215-240): w_fp8 holds
 * OCP FP8 E4M3 bytes in the weight's own [N, K] shape (row stride ldw bytes, a multiple of 16) and w_scale the f32
 * scales of `foo.weight_scale`, one per group as utilities/teeny-quant/src/quant/groups.rs:84-110 numbers them:
 * scale_kind 0 = "tensor" (1 scale), 1 = "channel" with axis 0 (N scales), 2 = "group" with axis 1 (row-major
 * [N][ceil(K / group_size)], group_size a multiple of 64).  An element's value is f8_to_f32(byte) * scale
 * (utilities/teeny-quant/src/quant/fp8.rs:175-206, 262-268); the products are accumulated in f32.  The reference has
 * no kernel that consumes these files (its Linear is f32, nn/linear.rs:226-335); this is the weight-only GEMM its
 * quantiser feeds.  M <= 128 streams the bytes (half the traffic of bf16 weights), converts them next to the tensor
 * core and applies kinds 0 and 1 to the f32 sums; larger M first converts W into global_scratch
 * (teeny_linear_w8a16_scratch_bytes) as bf16(value * scale) and runs the bf16 GEMM.  swiglu != 0: rows interleaved
 * and output as in teeny_linear_swiglu_bf16 (scales in the same interleaved row order, no bias).  The two NaN bytes
 * (0x7f, 0xff) are not reproduced by the M <= 128 path: check a tensor once with teeny_fp8_e4m3_count_nan. */
int teeny_linear_w8a16_forward(const teeny_bf16* x, long long ldx, const void* w_fp8, long long ldw, const float* w_scale,
                               int scale_kind, int group_size, const teeny_bf16* bias, teeny_bf16* y, long long ldy, int M,
                               int N, int K, int swiglu, void* global_scratch, size_t global_scratch_bytes,
                               teeny_stream_t stream);
size_t teeny_linear_w8a16_scratch_bytes(int M, int N, int K);
/* The same product with the ACTIVATIONS in FP8 too, for the projections whose input a norm kernel writes anyway: every
 * bf16 activation is split into two E4M3 terms, x * s = hi + lo with s the power of two that brings the row's largest
 * magnitude into [128, 256).  A bf16 value has 8 significant bits and an E4M3 number 4, so the split is exact while both
 * terms are normal numbers: for every element within 2^10 of its row's maximum (lo is stored times 16); smaller
 * elements keep fewer bits (4 down to 2^-13 of the maximum, none below 2^-17).  teeny_split_fp8_e4m3 writes
 * out[2 * M, K] bytes (the hi rows, then the lo rows; row stride ldo bytes, a multiple of 16) and x_scale[M] = 1 / s;
 * teeny_linear_w8a8x2_forward multiplies them with FP8 weights as they are (tcgen05.mma kind::f8f6f4, no conversion
 * inside the kernel): Y[m, n] = x_scale[m] * w_scale[n] * sum_k w[n, k] * (hi[m, k] + lo[m, k] / 16), M <= 128,
 * scale_kind 0 or 1.  Where the split is exact this is teeny_linear_w8a16_forward's result. */
int teeny_split_fp8_e4m3(const teeny_bf16* x, long long ldx, void* out, long long ldo, float* x_scale, int M, int K,
                         teeny_stream_t stream);
int teeny_linear_w8a8x2_forward(const void* x_fp8, long long ldx, const float* x_scale, const void* w_fp8, long long ldw,
                                const float* w_scale, int scale_kind, const teeny_bf16* bias, teeny_bf16* y, long long ldy,
                                int M, int N, int K, int swiglu, teeny_stream_t stream);
/* out[N, K] (bf16, row stride ldo elements) = bf16(f8_to_f32(w_fp8) * scale): dequantize_fp8 of
 * utilities/teeny-quant/src/quant/fp8.rs:262-268 with one rounding to bf16, every byte value handled (NaN included). */
int teeny_dequant_fp8_e4m3_bf16(const void* w_fp8, long long ldw, const float* w_scale, int scale_kind, int group_size,
                                teeny_bf16* out, long long ldo, int N, int K, teeny_stream_t stream);
/* The quantiser's integer schemes ("int-quantized": I8 in the weight's shape; "pack-quantized": 4-bit values two per
 * byte over the flattened tensor, the first in the low nibble, utilities/teeny-quant/src/quant/pack4.rs:31-40) back to
 * bf16: out[N, K] = bf16((q - zero_point) * scale), dequantize_affine of utilities/teeny-quant/src/quant/affine.rs:151-161
 * with one rounding.  bits = 8 or 4; zero_point = the I32 vector of `foo.weight_zero_point` or NULL for a symmetric
 * scheme; scale kinds as above, any group_size.  There is no streaming integer GEMM: such weights are converted once
 * when they are loaded and run through the bf16 kernels. */
int teeny_dequant_int_bf16(const void* q, int bits, const float* w_scale, const int* zero_point, int scale_kind,
                           int group_size, teeny_bf16* out, long long ldo, int N, int K, teeny_stream_t stream);
/* *count (device word) <- how many of the n bytes are E4M3 NaN encodings. */
int teeny_fp8_e4m3_count_nan(const void* bytes, size_t n, unsigned* count, teeny_stream_t stream);
/* cos/sin tables [max_pos, D] from inv_freq[D/2] (f32 angles, one rounding to bf16). */
int teeny_rope_table_bf16(const float* inv_freq, teeny_bf16* cos_table, teeny_bf16* sin_table, int max_pos, int D,
                          teeny_stream_t stream);
/* Per-head RMSNorm of q and k (D == 128), rotary embedding (rotate-half), KV-cache append.  qkv is the fused
 * projection [T, (Hq + 2 Hkv) * D] with row stride ld; token t is sequence t / S at position pos0 + t % S
 * (pos0 = *pos0_dev when non-NULL).  q is rewritten in place; caches are [B, Hkv, max_len, D]. */
int teeny_qk_norm_rope_kv_bf16(teeny_bf16* qkv, long long ld, const teeny_bf16* q_norm_w, const teeny_bf16* k_norm_w,
                               const teeny_bf16* cos_table, const teeny_bf16* sin_table, teeny_bf16* k_cache,
                               teeny_bf16* v_cache, int T, int S, int Hq, int Hkv, int D, int max_len, int pos0,
                               const int* pos0_dev, float eps, teeny_stream_t stream);
/* out[t, :] = table[ids[t], :] */
int teeny_embedding_bf16(const int* ids, const teeny_bf16* table, teeny_bf16* out, int T, int hidden, int vocab,
                         teeny_stream_t stream);
/* Row argmax, lowest index on ties: best_val[r] (f32), best_idx[r] = index + idx_offset. */
int teeny_argmax_bf16(const teeny_bf16* logits, long long ld, float* best_val, int* best_idx, int rows, int cols,
                      int idx_offset, teeny_stream_t stream);
/* Merge `parts` candidates per row (vals / idx laid out [parts, rows]) into out_idx[rows]. */
int teeny_argmax_combine(const float* vals, const int* idx, int* out_idx, int parts, int rows,
                         teeny_stream_t stream);
/* Sampling behind the LM head: temperature, top-k (1..1024) and top-p over each row of bf16 logits [rows, cols]
 * (row stride ld).  Candidates are the top_k entries by (logit descending, index ascending); e_i = exp((l_i - l_0) /
 * temperature) in f32, summed sequentially in that order; the nucleus is the shortest prefix whose mass reaches
 * top_p of the total; out_idx[r] is the first candidate whose running mass exceeds u[r] times the nucleus mass
 * (u[r] in [0, 1) is the caller's random number, so the call is deterministic); out_prob (optional) receives the
 * sampled token's probability within the nucleus.  The reference has only the row softmax next to the logits
 * (kernels/teeny-kernels/src/nn/activation/softmax.rs:39-69; Op::TopK is not lowered,
 * kernels/teeny-kernels/src/graph/mod.rs:2784). */
int teeny_sample_top_k_top_p_bf16(const teeny_bf16* logits, long long ld, int rows, int cols, float temperature,
                                  int top_k, float top_p, const float* u, int* out_idx, float* out_prob,
                                  teeny_stream_t stream);
/* The same sampler over a vocabulary that is split in shards (vocabulary-parallel LM head).  Per shard,
 * teeny_sample_candidates_bf16 writes the shard's top_k candidates of every row, sorted, as 64-bit words
 * (order key << 32 | 0xFFFFFFFF - (index + idx_offset); zero = empty slot) to cand_out[row * top_k + i].
 * teeny_sample_merge takes `parts` such lists per row (shard p's at lists + p * list_stride words: the layout an
 * all-gather of the shards' outputs has), finds the top_k of their union and finishes as the unsharded call does: given
 * the same u it returns the token teeny_sample_top_k_top_p_bf16 returns on the concatenated row.  parts <= 8. */
int teeny_sample_candidates_bf16(const teeny_bf16* logits, long long ld, int rows, int cols, int top_k, int idx_offset,
                                 unsigned long long* cand_out, teeny_stream_t stream);
int teeny_sample_merge(const unsigned long long* lists, int parts, size_t list_stride, int rows, float temperature,
                       int top_k, float top_p, const float* u, int* out_idx, float* out_prob, teeny_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* TEENY_B200_H_ */
