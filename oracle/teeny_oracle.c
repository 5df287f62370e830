/*
 * TEST INFRASTRUCTURE ONLY -- CPU restatement of the reference's kernels for the
 * GEMM / attention / Qwen3-forward path.  Nothing in the product path may call this file:
 * only tests, the smoke check and the benchmark's CPU-baseline leg link it.
 *
 * Each function restates, in plain sequential C with f32 arithmetic, what the reference's
 * kernel (a Triton-like Rust DSL source) or its test-side host loop computes.  Parity is
 * pinned: tests/test_oracle_golden.py checks every function here against the reference's own
 * committed fixtures (tests/golden/reference_fixtures.npz).
 *
 * Build: make -C oracle   (gcc -O2 -shared -fPIC; no -ffast-math so the f32 summation
 * order written here is the order that runs).
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* C = A @ B, all row-major f32, sequential k accumulation.
 * Follows matmul_reference, kernels/teeny-kernels/tests/test_gemm.rs:183-196, which is the
 * expectation for matmul_forward (kernels/teeny-kernels/src/math/gemm.rs:44-108). */
void oracle_matmul_f32(const float* a, const float* b, float* c, int M, int N, int K) {
  for (int mi = 0; mi < M; ++mi)
    for (int ni = 0; ni < N; ++ni) {
      float acc = 0.0f;
      for (int ki = 0; ki < K; ++ki) acc += a[(size_t)mi * K + ki] * b[(size_t)ki * N + ni];
      c[(size_t)mi * N + ni] = acc;
    }
}

/* Y = X @ W^T (+ bias); X is [M,K], W is [N,K] (out_features first), Y is [M,N].
 * Follows linear_reference, kernels/teeny-kernels/tests/test_linear.rs:62-84, the expectation
 * for linear_forward (kernels/teeny-kernels/src/nn/mlp/linear.rs:22-116).  bias may be NULL. */
void oracle_linear_f32(const float* x, const float* w, const float* bias, float* y, int M, int N,
                       int K) {
  for (int mi = 0; mi < M; ++mi)
    for (int ni = 0; ni < N; ++ni) {
      float acc = 0.0f;
      for (int ki = 0; ki < K; ++ki) acc += x[(size_t)mi * K + ki] * w[(size_t)ni * K + ki];
      if (bias) acc += bias[ni];
      y[(size_t)mi * N + ni] = acc;
    }
}

/* Attention forward with the reference kernel's online-softmax recurrence, one query row at a
 * time and one key at a time: m' = max(m, s); l = exp(m-m')*l + exp(s-m'); acc likewise;
 * O = acc / l; L = m + log(l).  Follows flash_attention2_forward,
 * kernels/teeny-kernels/src/nn/attention/flash_attn2.rs:53-156 (layout [BH, n_ctx, D]).
 *
 * Extensions the hot path needs beyond that kernel (PyTorch SDPA semantics, which is how the
 * reference's Qwen3 trace calls attention): grouped-query heads (kv head = q head / group) and a
 * causal mask aligned to the end of the key sequence (query i sees keys j <= i + n_ctx_k - n_ctx_q).
 * With Hq == Hkv and causal == 0 this is exactly the reference kernel.
 *   q,o: [B, Hq, n_ctx_q, D]   k,v: [B, Hkv, n_ctx_k, D]   lse: [B, Hq, n_ctx_q] (may be NULL) */
void oracle_attention_f32(const float* q, const float* k, const float* v, float* o, float* lse,
                          int B, int Hq, int Hkv, int n_ctx_q, int n_ctx_k, int D,
                          float softmax_scale, int causal) {
  const int group = Hq / Hkv;
  for (int b = 0; b < B; ++b)
    for (int h = 0; h < Hq; ++h) {
      const int hk = h / group;
      const float* kb = k + ((size_t)b * Hkv + hk) * n_ctx_k * D;
      const float* vb = v + ((size_t)b * Hkv + hk) * n_ctx_k * D;
      for (int i = 0; i < n_ctx_q; ++i) {
        const float* qr = q + (((size_t)b * Hq + h) * n_ctx_q + i) * D;
        float* orow = o + (((size_t)b * Hq + h) * n_ctx_q + i) * D;
        float m_i = -INFINITY, l_i = 0.0f;
        for (int d = 0; d < D; ++d) orow[d] = 0.0f;
        const int last = causal ? i + (n_ctx_k - n_ctx_q) : n_ctx_k - 1;
        for (int j = 0; j <= last && j < n_ctx_k; ++j) {
          float s = 0.0f;
          for (int d = 0; d < D; ++d) s += qr[d] * kb[(size_t)j * D + d];
          s *= softmax_scale;
          const float m_new = s > m_i ? s : m_i;
          const float corr = expf(m_i - m_new);
          const float p = expf(s - m_new);
          l_i = corr * l_i + p;
          for (int d = 0; d < D; ++d) orow[d] = corr * orow[d] + p * vb[(size_t)j * D + d];
          m_i = m_new;
        }
        for (int d = 0; d < D; ++d) orow[d] /= l_i;
        if (lse) lse[((size_t)b * Hq + h) * n_ctx_q + i] = m_i + logf(l_i);
      }
    }
}

/* rrms = 1/sqrt(mean(x^2) + eps) (eps inside the root); y = x * rrms * weight; rrms stored per row.
 * Follows rms_norm_forward, kernels/teeny-kernels/src/nn/norm/rmsnorm.rs:40-118 and
 * tests/fixtures/generate.py:541-556.  rrms may be NULL. */
void oracle_rms_norm_f32(const float* x, float* y, const float* weight, float* rrms, int M, int N,
                         float eps) {
  for (int r = 0; r < M; ++r) {
    float sq = 0.0f;
    for (int c = 0; c < N; ++c) sq += x[(size_t)r * N + c] * x[(size_t)r * N + c];
    const float rr = 1.0f / sqrtf(sq * (1.0f / (float)N) + eps);
    if (rrms) rrms[r] = rr;
    for (int c = 0; c < N; ++c) y[(size_t)r * N + c] = x[(size_t)r * N + c] * rr * weight[c];
  }
}

/* y = x * (1 / (1 + exp(-x))).  Follows silu_forward,
 * kernels/teeny-kernels/src/nn/activation/sigmoid.rs:120-156 (multiply by the reciprocal). */
void oracle_silu_f32(const float* x, float* y, int n) {
  for (int i = 0; i < n; ++i) y[i] = x[i] * (1.0f / (1.0f + expf(-x[i])));
}

/* out = a * b.  Follows elemwise_mul_forward, kernels/teeny-kernels/src/nn/tensor/elemwise_binary.rs:206. */
void oracle_mul_f32(const float* a, const float* b, float* out, int n) {
  for (int i = 0; i < n; ++i) out[i] = a[i] * b[i];
}

/* out = a + b.  Follows elemwise_add_forward, kernels/teeny-kernels/src/nn/tensor/elemwise_add.rs:29-69. */
void oracle_add_f32(const float* a, const float* b, float* out, int n) {
  for (int i = 0; i < n; ++i) out[i] = a[i] + b[i];
}

/* Row softmax with max subtraction.  Follows softmax_forward,
 * kernels/teeny-kernels/src/nn/activation/softmax.rs:39-69. */
void oracle_softmax_f32(const float* x, float* y, int n_rows, int n_cols) {
  for (int r = 0; r < n_rows; ++r) {
    const float* xr = x + (size_t)r * n_cols;
    float* yr = y + (size_t)r * n_cols;
    float mx = -INFINITY, sum = 0.0f;
    for (int c = 0; c < n_cols; ++c) mx = xr[c] > mx ? xr[c] : mx;
    for (int c = 0; c < n_cols; ++c) { yr[c] = expf(xr[c] - mx); sum += yr[c]; }
    for (int c = 0; c < n_cols; ++c) yr[c] /= sum;
  }
}

#ifdef __cplusplus
}
#endif
