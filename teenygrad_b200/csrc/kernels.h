// Internal launch functions behind the C ABI (include/teeny_b200.h).  Every function enqueues work on
// `stream` and returns 0, a negative TEENY_ERR_* code, or a positive cudaError_t.  None allocates memory.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace teeny {

typedef __nv_bfloat16 bf16;

unsigned long long launches_so_far();  // see count_launches (common.cuh)

// ---- GEMM --------------------------------------------------------------------------------------
constexpr int kGemmMaxSplitK = 16;     // most k-splits per output tile
constexpr int kGemmMaxWorkPerSm = 8;   // split-K is only used while tiles*splits <= this * SM count

size_t gemm_bf16_scratch_bytes(int M, int N, int K);
// Set function attributes for every kernel variant on the current device (also done lazily at first launch).
int gemm_bf16_prepare();
int attention_prefill_prepare();
int attention_decode_prepare();
// swiglu: W is [N, K] with rows interleaved in blocks of 64 gate channels / 64 up channels (N = 2 * channels) and
// Y is [M, N / 2] = silu(gate) * up, rounded as the unfused bf16 graph rounds (both projections, silu, product).
// Tensor-parallel push mode of the decode GEMM (M <= 128): y is not written; every rank receives this rank's f32
// result in its receive buffer as {value, stamp} pairs (8 bytes per element, element (row, col) at row * N + col),
// stamp = *epoch * 1024 + round + 1.  The receiver recognises arrived data by the stamp, so the sender needs no
// fence, flag or counter; a buffer must not be written again with the same stamp.
struct GemmPush {
  uint2* const* recv;     // device array [world]: this rank's slot inside every rank's buffer
  int world;
  const unsigned* epoch;  // device word, constant while the kernel runs
  unsigned round;         // < 1023
  int owner_rows;         // 0: every rank receives every row; > 0: row r goes only to rank r / owner_rows, which sums it
};
int gemm_bf16(const bf16* x, int ldx, const bf16* w, int ldw, bool w_is_kn, const bf16* bias, bf16* y, int ldy,
              int M, int N, int K, void* scratch, size_t scratch_bytes, cudaStream_t stream, bool swiglu = false,
              const GemmPush* push = nullptr, float* y32 = nullptr, int l2_ahead = -1);
// y32 (w_is_kn only): store the f32 accumulators to y32[M, ldy] instead of rounding them to bf16 into y.
// l2_ahead (decode-shaped GEMMs, M <= 128): how many of its 16 KB weight tiles beyond the shared-memory ring each CTA
// asks into L2 before it waits for its predecessor (-1: the library default, none).  Worth it only where the
// predecessor leaves HBM idle, e.g. a norm kernel that waits for other ranks' partial sums.
// Row-parallel epilogue of tensor parallelism: sums the `world` f32 partial rows [M][N] that the ranks' GEMMs pushed
// as {value, stamp} pairs (slot_elems elements between ranks), waiting for each element until it carries the stamp
// *epoch * 1024 + round + 1; rounds the sum to bf16 (the all-reduced projection), adds it into the bf16 residual and
// RMS-normalises it: residual <- residual + sum; y <- norm(residual).  Waits are bounded (device error word;
// wait_limit_ns = 0 means the library's 2 s limit).
int gather_add_rms_norm_bf16(const uint2* recv, size_t slot_elems, int world, const unsigned* epoch, unsigned round,
                             bf16* residual, long long ldr, bf16* y, long long ldy, const bf16* w, int M, int N,
                             float eps, cudaStream_t st, unsigned long long wait_limit_ns = 0);
// The same in two hops: row r is summed and normalised only by rank r / owner_rows (the GEMMs pushed it only there,
// GemmPush::owner_rows), which then stores the new residual row and the normed row, stamped, into every other rank's
// broadcast buffer bcast[p] (device array [world], own entry unused); the other ranks' CTAs wait for their copy.
int gather_add_rms_norm_owner_bf16(const uint2* recv, size_t slot_elems, int world, int rank, int owner_rows,
                                   uint4* const* bcast, const unsigned* epoch, unsigned round, bf16* residual,
                                   long long ldr, bf16* y, long long ldy, const bf16* w, int M, int N, float eps,
                                   cudaStream_t st, unsigned long long wait_limit_ns = 0);
// ---- FP8 (E4M3) weight-only linear ----
// W as bytes [N, K] (row stride ldw bytes) plus f32 scales: kind 0 = one scale, 1 = one per weight row (N), 2 = one per
// `group` consecutive k of a row ([N][ceil(K / group)], group a multiple of 64).  value = decode(byte) * scale.
// M <= 128: the bytes are streamed and converted inside the GEMM (swiglu and the tensor-parallel push as in gemm_bf16);
// larger M: converted once into `scratch` (linear_w8a16_scratch_bytes) as bf16(value * scale), then the bf16 GEMM.
int gemm_w8a16_skinny(const bf16* x, int ldx, const uint8_t* wq, int ldw, const float* w_scale, int scale_kind,
                      int group, const bf16* bias, bf16* y, int ldy, int M, int N, int K, cudaStream_t stream,
                      bool swiglu = false, const GemmPush* push = nullptr);
// FP8 weights AND two-term FP8 activations (split_e4m3 writes them: x = (hi + lo / 16) * x_scale[row], exact for
// elements within 2^10 of their row's maximum): kind::f8f6f4 on the bytes as they are, M <= 128, scale kinds 0 and 1.
int split_e4m3(const bf16* x, long long ldx, uint8_t* out, long long ldo, float* scale, int M, int K, cudaStream_t st);
int gemm_w8a8x2_skinny(const uint8_t* x8, int ldx8, const float* x_scale, const uint8_t* wq, int ldw, const float* w_scale,
                       int scale_kind, const bf16* bias, bf16* y, int ldy, int M, int N, int K, cudaStream_t stream,
                       bool swiglu = false, const GemmPush* push = nullptr);
int dequant_e4m3_bf16(const uint8_t* wq, long long ldw, const float* scale, int kind, int group, bf16* out, long long ldo,
                      int N, int K, cudaStream_t st);
// out[N, K] = bf16((q - zero point) * scale) for the integer schemes: bits 8 (int8 [N, K]) or 4 (nibbles packed two per
// byte over the flattened tensor, low nibble first); zero_point null for symmetric schemes; scale kinds as above (any
// group size).
int dequant_int_bf16(const void* q, int bits, const float* scale, const int* zero_point, int kind, int group, bf16* out,
                     long long ldo, int N, int K, cudaStream_t st);
// *count <- number of NaN encodings (0x7f, 0xff) among n bytes; the in-GEMM conversion does not reproduce them
int e4m3_count_nan(const uint8_t* p, size_t n, unsigned* count, cudaStream_t st);
size_t linear_w8a16_scratch_bytes(int M, int N, int K);
int linear_w8a16(const bf16* x, int ldx, const uint8_t* wq, int ldw, const float* scale, int kind, int group,
                 const bf16* bias, bf16* y, int ldy, int M, int N, int K, void* scratch, size_t scratch_bytes,
                 cudaStream_t st, bool swiglu = false, const GemmPush* push = nullptr);

// Large-M path on CTA pairs (tcgen05 cta_group::2, 256 x 256 tiles); same contract as gemm_bf16 without the options.
// With `qkv` the GEMM is the fused [q | k | v] projection of a prefill (N = (Hq + 2 Hkv) * 128, token t = sequence
// t / S at position pos0 + t % S) and its epilogue does what qk_norm_rope_kv_bf16 does in a pass of its own: per-head
// RMSNorm of q and k, rotary embedding, q written to y (k / v columns of y are NOT written), k and v rows appended
// to the caches [B, Hkv, max_len, 128].
struct QkvEpilogue {
  const bf16* q_w;     // [128] head-norm weights
  const bf16* k_w;
  const bf16* cos_t;   // [max_len, 128] tables
  const bf16* sin_t;
  bf16* k_cache;
  bf16* v_cache;
  int S, Hq, Hkv, max_len, pos0;
  float eps;
};
int gemm_bf16_2cta_prepare();
int gemm_bf16_2cta(const bf16* x, int ldx, const bf16* w, int ldw, const bf16* bias, bf16* y, int ldy, int M, int N,
                   int K, cudaStream_t stream, bool swiglu = false, const QkvEpilogue* qkv = nullptr);
// Whether gemm_bf16 hands an [M, N] problem to the CTA-pair kernel (enough 256 x 256 tiles for every SM pair).
bool gemm_bf16_uses_2cta(int M, int N);
// C[M, N] = A[M, K] B[K, N], all f32 row-major and contiguous, on the tensor cores at f32 accuracy: each operand is
// split into two bf16 terms (x = hi + mid + O(2^-16 x)) and hi*hi + mid*hi + hi*mid is accumulated in f32 by ONE bf16
// GEMM over the concatenated K (A' = [hi | mid | hi], B' = [hi ; hi ; mid]).  scratch holds A' and B':
// gemm_f32_split_scratch_bytes(M, N, K).  Needs K and N multiples of 8 and 16-byte aligned pointers.
size_t gemm_f32_split_scratch_bytes(int M, int N, int K);
int gemm_f32_split(const float* a, const float* b, float* c, int M, int N, int K, void* scratch, size_t scratch_bytes,
                   cudaStream_t stream);
// f32 GEMM with true f32 accuracy.  b_is_nk: B given as [N, K] (linear layout) instead of [K, N].
int gemm_f32(const float* a, long long sam, long long sak, const float* b, long long sbk, long long sbn,
             const float* bias, float* c, long long scm, long long scn, int M, int N, int K, cudaStream_t stream);
// bf16 GEMM on CUDA cores for shapes the TMA path cannot take (unaligned strides / pointers).
int gemm_bf16_generic(const bf16* a, long long sam, long long sak, const bf16* b, long long sbk, long long sbn,
                      const bf16* bias, bf16* c, long long scm, long long scn, int M, int N, int K,
                      cudaStream_t stream);

// ---- attention ---------------------------------------------------------------------------------
struct AttnShape {
  int B, Hq, Hkv, Sq, Skv, D;
  long long q_sb, q_sh, q_ss;   // element strides of Q (batch, head, sequence); D is contiguous
  long long k_sb, k_sh, k_ss;
  long long v_sb, v_sh, v_ss;
  long long o_sb, o_sh, o_ss;
  float scale;
  int causal;
};
int attention_prefill_bf16(const bf16* q, const bf16* k, const bf16* v, bf16* o, float* lse, const AttnShape& s,
                           cudaStream_t stream);
size_t attention_decode_scratch_bytes(int B, int Hq, int D, int max_kv);
// Optional front end of the decode attention kernel: per-head RMSNorm + RoPE of the step's q / k heads and the append
// of the new k / v rows to the caches, done by the CTA that attends over them instead of by a kernel of its own.
// q (the attention call's argument) then holds the raw projection and is left untouched.
struct DecodeRope {
  const bf16* k_new;   // raw K projection of the new token: k_new + b * new_sb + kv_head * 128; V likewise
  const bf16* v_new;
  long long new_sb;
  bf16* k_cache;       // the caches the call attends over (same strides as in the AttnShape), writable
  bf16* v_cache;
  const bf16* q_w;     // [128] head-norm weights
  const bf16* k_w;
  const bf16* cos_t;   // [max_len, 128] tables
  const bf16* sin_t;
  const int* pos_dev;  // position of the new token (device word), or pos if null; the live length must be pos + 1
  int pos;
  int max_len;
  float eps;
};
// One query token per sequence against the first *kv_len_dev (or kv_len if the pointer is null) cache entries.
// fresh_rows >= 0 is a promise that matters only under programmatic dependent launch: the kernel launched just before
// this one writes nothing this call reads except q (and rope->k_new / v_new) and the last fresh_rows live cache rows,
// and *kv_len_dev is older still; the kernel then starts streaming the older rows before its predecessor has finished.
// counters: B * Hkv words, zero before the first call and left zero by every call; with them a split sequence is merged
// by the last CTA to finish instead of by a second kernel (calls sharing the counters must not overlap).
int attention_decode_bf16(const bf16* q, const bf16* k, const bf16* v, bf16* o, const AttnShape& s, int kv_len,
                          const int* kv_len_dev, void* scratch, size_t scratch_bytes, cudaStream_t stream,
                          int fresh_rows = -1, const DecodeRope* rope = nullptr, unsigned* counters = nullptr);
// Same as attention_decode_bf16 with the partials in a fixed-size array inside the library image (no caller scratch).
size_t attention_decode_static_scratch_limit();
int attention_decode_bf16_static(const bf16* q, const bf16* k, const bf16* v, bf16* o, const AttnShape& s, int kv_len,
                                 const int* kv_len_dev, cudaStream_t stream);
template <typename T>
int attention_generic(const T* q, const T* k, const T* v, T* o, float* lse, const AttnShape& s, cudaStream_t stream);

// ---- normalisation / elementwise ----------------------------------------------------------------
int rms_norm_f32(const float* x, float* y, const float* w, float* rrms, int M, int N, float eps, cudaStream_t st);
// bf16 with the Qwen3 rounding points: f32 statistics, round to bf16, then multiply by the bf16 weight.
// y8 != null: y is also written as two-term FP8 activations (hi rows, then M lo rows; row stride ld8 bytes;
// y8_scale[M]), as split_e4m3 would split it.
int rms_norm_bf16(const bf16* x, long long ldx, bf16* y, long long ldy, const bf16* w, float* rrms, int M, int N,
                  float eps, cudaStream_t st, uint8_t* y8 = nullptr, long long ld8 = 0, float* y8_scale = nullptr);
// residual <- bf16(residual + x); y <- rms_norm(residual) (same rounding as rms_norm_bf16).
int add_rms_norm_bf16(const bf16* x, long long ldx, bf16* residual, long long ldr, bf16* y, long long ldy,
                      const bf16* w, int M, int N, float eps, cudaStream_t st, uint8_t* y8 = nullptr, long long ld8 = 0,
                      float* y8_scale = nullptr);
int silu_f32(const float* x, float* y, long long n, cudaStream_t st);
int silu_bf16(const bf16* x, bf16* y, long long n, cudaStream_t st);
int mul_f32(const float* a, const float* b, float* o, long long n, cudaStream_t st);
int mul_bf16(const bf16* a, const bf16* b, bf16* o, long long n, cudaStream_t st);
int add_f32(const float* a, const float* b, float* o, long long n, cudaStream_t st);
int add_bf16(const bf16* a, const bf16* b, bf16* o, long long n, cudaStream_t st);
int softmax_f32(const float* x, float* y, int rows, int cols, cudaStream_t st);
int softmax_bf16(const bf16* x, bf16* y, int rows, int cols, cudaStream_t st);
// out[t, i] = bf16(bf16(silu(gate_up[t, i])) * gate_up[t, inter + i])
int silu_mul_bf16(const bf16* gate_up, long long ld, bf16* out, int T, int inter, cudaStream_t st);
int embedding_bf16(const int* ids, const bf16* table, bf16* out, int T, int hidden, int vocab, cudaStream_t st);
// cos/sin tables [max_pos, D] bf16 from f32 inv_freq[D/2]: angle = pos * inv_freq in f32, cos/sin, one rounding.
int rope_table_bf16(const float* inv_freq, bf16* cos_t, bf16* sin_t, int max_pos, int D, cudaStream_t st);
// Per-head RMSNorm of q and k, rotary embedding, and KV-cache append, reading the fused QKV projection.
//   qkv [T, (Hq + 2 Hkv) * D]; token t belongs to sequence t / S at position pos0 + t % S, where
//   pos0 = *pos0_dev if the pointer is non-null else pos0.  q is rewritten in place; k (normed + rotated) and v go
//   to the caches laid out [B, Hkv, max_len, D].
int qk_norm_rope_kv_bf16(bf16* qkv, long long ld, const bf16* q_w, const bf16* k_w, const bf16* cos_t,
                         const bf16* sin_t, bf16* k_cache, bf16* v_cache, int T, int S, int Hq, int Hkv, int D,
                         int max_len, int pos0, const int* pos0_dev, float eps, cudaStream_t st);
// Row argmax with lowest index on ties; writes value (f32) and index + idx_offset.
int argmax_bf16(const bf16* logits, long long ld, float* best_val, int* best_idx, int rows, int cols, int idx_offset,
                cudaStream_t st);
// Combine `parts` candidate (value, index) pairs per row: vals/idx [parts, rows] -> out_idx [rows].
int argmax_combine(const float* vals, const int* idx, int* out_idx, int parts, int rows, cudaStream_t st);
// Temperature / top-k / top-p sampling, one row of bf16 logits per CTA (csrc/sampling.cu): out_idx[r] = sampled column,
// out_prob[r] (optional) = its probability inside the nucleus.  u[r] in [0, 1) is the caller's random number.
int sample_top_k_top_p_bf16(const bf16* logits, long long ld, int rows, int cols, float temperature, int top_k,
                            float top_p, const float* u, int* out_idx, float* out_prob, cudaStream_t st);
// The same sampler over a vocabulary split in `parts` shards (tensor parallelism): sample_candidates_bf16 writes a
// shard's top_k candidates per row, sorted, as 64-bit words (order key << 32 | 0xFFFFFFFF - global index, zero = empty) to
// cand_out[row * top_k + i]; sample_merge takes the shards' lists (lists + p * list_stride, e.g. straight out of an
// all-gather) and finishes: same token as the unsharded call on the concatenated row, on every rank.
int sample_candidates_bf16(const bf16* logits, long long ld, int rows, int cols, int top_k, int idx_offset,
                           unsigned long long* cand_out, cudaStream_t st);
int sample_merge_prepare();
int sample_merge(const unsigned long long* lists, int parts, size_t list_stride, int rows, float temperature, int top_k,
                 float top_p, const float* u, int* out_idx, float* out_prob, cudaStream_t st);
// u[row] = uniform in [0, 1) from (seed, step, row) by a stateless hash; step from *step_dev when given.
int sampling_uniform(unsigned long long seed, int step, const int* step_dev, float* u, int rows, cudaStream_t st);

}  // namespace teeny
