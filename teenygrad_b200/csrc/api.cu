// C ABI (include/teeny_b200.h): argument checks, dtype / layout dispatch, and the few process-wide helpers
// (tensor-map encoding through the driver entry point, per-device error word, SM count).
#include <atomic>
#include <mutex>

#include "../../include/teeny_b200.h"
#include "common.cuh"
#include "kernels.h"

namespace teeny {

namespace {

constexpr int kMaxDevices = 64;
__device__ int g_error_word = 0;  // one instance per device that loads this module

std::mutex g_mutex;
int* g_error_ptr[kMaxDevices] = {};
int g_sm_count[kMaxDevices] = {};

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;

int current_device() {
  int d = 0;
  cudaGetDevice(&d);
  return (d >= 0 && d < kMaxDevices) ? d : 0;
}

}  // namespace

namespace {
thread_local bool t_pdl_enabled = false;
}
bool pdl_enabled() { return t_pdl_enabled; }
void pdl_set_enabled(bool on) { t_pdl_enabled = on; }

int* device_error_word() {
  const int d = current_device();
  std::lock_guard<std::mutex> lock(g_mutex);
  if (!g_error_ptr[d]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_error_word) != cudaSuccess) return nullptr;
    g_error_ptr[d] = static_cast<int*>(p);
  }
  return g_error_ptr[d];
}

namespace { std::atomic<unsigned long long> g_launches{0}; }
void count_launches(unsigned long long n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
unsigned long long launches_so_far() { return g_launches.load(std::memory_order_relaxed); }

namespace { thread_local int t_sm_limit = 0; }
void set_sm_limit(int n) { t_sm_limit = n > 0 ? n : 0; }

int sm_count() {
  const int d = current_device();
  std::lock_guard<std::mutex> lock(g_mutex);
  if (!g_sm_count[d]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, d) != cudaSuccess || n <= 0) n = 148;
    g_sm_count[d] = n;
  }
  const int n = g_sm_count[d];
  return (t_sm_limit > 0 && t_sm_limit < n) ? t_sm_limit : n;
}

namespace {
int encode_tensor_map(CUtensorMap* out, CUtensorMapDataType type, CUtensorMapSwizzle swizzle, const void* base, int rank,
                      const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box) {
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    if (!g_encode) {
      void* fn = nullptr;
      cudaDriverEntryPointQueryResult qres;
      if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess ||
          qres != cudaDriverEntryPointSuccess || !fn)
        return TEENY_ERR_DRIVER;
      g_encode = reinterpret_cast<EncodeTiledFn>(fn);
    }
  }
  if (rank < 1 || rank > 5) return TEENY_ERR_BAD_ARG;
  cuuint64_t gdim[5], gstr[4];
  cuuint32_t gbox[5], estr[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    gbox[i] = box[i];
    estr[i] = 1;
  }
  for (int i = 0; i + 1 < rank; ++i) {
    if (strides_bytes[i] == 0 || (strides_bytes[i] & 15)) return TEENY_ERR_ALIGNMENT;
    gstr[i] = strides_bytes[i];
  }
  if (reinterpret_cast<uintptr_t>(base) & 15) return TEENY_ERR_ALIGNMENT;
  const CUresult r = g_encode(out, type, static_cast<cuuint32_t>(rank),
                              const_cast<void*>(base), gdim, gstr, gbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? TEENY_OK : TEENY_ERR_DRIVER;
}
}  // namespace

int encode_tensor_map_bf16(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                           const uint64_t* strides_bytes, const uint32_t* box) {
  return encode_tensor_map(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, CU_TENSOR_MAP_SWIZZLE_128B, base, rank, dims,
                           strides_bytes, box);
}

// Bytes in the same 128-byte swizzle: the FP8 weight tiles that warps convert before the MMA reads them.
int encode_tensor_map_u8(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                         const uint64_t* strides_bytes, const uint32_t* box) {
  return encode_tensor_map(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, CU_TENSOR_MAP_SWIZZLE_128B, base, rank, dims, strides_bytes,
                           box);
}

}  // namespace teeny

using namespace teeny;

namespace {
inline const bf16* B(const teeny_bf16* p) { return reinterpret_cast<const bf16*>(p); }
inline bf16* B(teeny_bf16* p) { return reinterpret_cast<bf16*>(p); }
inline cudaStream_t S(teeny_stream_t s) { return reinterpret_cast<cudaStream_t>(s); }

AttnShape to_shape(const teeny_attn_shape& t) {
  AttnShape s;
  s.B = t.B; s.Hq = t.Hq; s.Hkv = t.Hkv; s.Sq = t.Sq; s.Skv = t.Skv; s.D = t.D;
  s.q_sb = t.q_sb; s.q_sh = t.q_sh; s.q_ss = t.q_ss;
  s.k_sb = t.k_sb; s.k_sh = t.k_sh; s.k_ss = t.k_ss;
  s.v_sb = t.v_sb; s.v_sh = t.v_sh; s.v_ss = t.v_ss;
  s.o_sb = t.o_sb; s.o_sh = t.o_sh; s.o_ss = t.o_ss;
  s.scale = t.scale; s.causal = t.causal;
  return s;
}

AttnShape contiguous_shape(int bh, int nq, int nk, int d, float scale) {
  AttnShape s;
  s.B = 1; s.Hq = bh; s.Hkv = bh; s.Sq = nq; s.Skv = nk; s.D = d;
  s.q_sb = static_cast<long long>(bh) * nq * d; s.q_sh = static_cast<long long>(nq) * d; s.q_ss = d;
  s.k_sb = static_cast<long long>(bh) * nk * d; s.k_sh = static_cast<long long>(nk) * d; s.k_ss = d;
  s.v_sb = s.k_sb; s.v_sh = s.k_sh; s.v_ss = d;
  s.o_sb = s.q_sb; s.o_sh = s.q_sh; s.o_ss = d;
  s.scale = scale; s.causal = 0;
  return s;
}
}  // namespace

extern "C" {

int teeny_version(void) { return 100; }

const char* teeny_status_string(int status) {
  switch (status) {
    case TEENY_OK: return "ok";
    case TEENY_ERR_BAD_ARG: return "bad argument (null pointer, non-positive size or unsupported shape)";
    case TEENY_ERR_ALIGNMENT: return "pointer or stride alignment not met";
    case TEENY_ERR_SCRATCH: return "scratch missing or too small";
    case TEENY_ERR_DRIVER: return "CUDA driver entry point unavailable or tensor-map encode failed";
    case TEENY_ERR_DEVICE_WAIT: return "a bounded wait inside a kernel expired";
    case TEENY_ERR_NCCL: return "NCCL error";
    case TEENY_ERR_STATIC_LIMIT: return "shape needs more scratch than the no-allocation entry point has built in";
    default: return status > 0 ? cudaGetErrorString(static_cast<cudaError_t>(status)) : "unknown status";
  }
}

unsigned long long teeny_launch_count(int reset) {
  return reset ? g_launches.exchange(0, std::memory_order_relaxed) : g_launches.load(std::memory_order_relaxed);
}

int teeny_device_error(int clear) {
  int* p = device_error_word();
  if (!p) return TEENY_ERR_DRIVER;
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return static_cast<int>(e);
  int v = 0;
  e = cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (clear && v != 0) {
    const int zero = 0;
    cudaMemcpy(p, &zero, sizeof(int), cudaMemcpyHostToDevice);
  }
  return v;
}

// ---- GEMM ----
int matmul_forward_entry_point_f32(const float* a, const float* b, float* c, int M, int N, int K, void* scratch,
                                   size_t scratch_bytes, teeny_stream_t stream) {
  // with scratch for the split operands: the tensor-core path (bf16 x 3, f32 accuracy); else f32 FMAs on the CUDA cores
  if (a && b && c && scratch && M > 0 && N > 0 && K > 0 && !(K & 7) && !(N & 7) &&
      !((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(c) |
         reinterpret_cast<uintptr_t>(scratch)) & 15) &&
      scratch_bytes >= gemm_f32_split_scratch_bytes(M, N, K))
    return gemm_f32_split(a, b, c, M, N, K, scratch, scratch_bytes, S(stream));
  return gemm_f32(a, K, 1, b, N, 1, nullptr, c, N, 1, M, N, K, S(stream));
}

size_t teeny_matmul_f32_scratch_bytes(int M, int N, int K) { return gemm_f32_split_scratch_bytes(M, N, K); }

int matmul_forward_entry_point_bf16(const teeny_bf16* a, const teeny_bf16* b, teeny_bf16* c, int M, int N, int K,
                                    void* scratch, size_t scratch_bytes, teeny_stream_t stream) {
  if (!a || !b || !c || M <= 0 || N <= 0 || K <= 0) return TEENY_ERR_BAD_ARG;
  const bool tma_ok = (K % 8 == 0) && (N % 8 == 0) &&
                      !((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b)) & 15);
  if (tma_ok) return gemm_bf16(B(a), K, B(b), N, /*w_is_kn=*/true, nullptr, B(c), N, M, N, K, scratch, scratch_bytes, S(stream));
  return gemm_bf16_generic(B(a), K, 1, B(b), N, 1, nullptr, B(c), N, 1, M, N, K, S(stream));
}

int linear_forward_entry_point_f32(const float* x, const float* w, const float* bias, float* y, int M, int N, int K,
                                   int sxm, int sxk, int swn, int swk, int sym, int syn, void*, size_t,
                                   teeny_stream_t stream) {
  return gemm_f32(x, sxm, sxk, w, swk, swn, bias, y, sym, syn, M, N, K, S(stream));
}

int linear_forward_entry_point_bf16(const teeny_bf16* x, const teeny_bf16* w, const teeny_bf16* bias, teeny_bf16* y,
                                    int M, int N, int K, int sxm, int sxk, int swn, int swk, int sym, int syn,
                                    void* scratch, size_t scratch_bytes, teeny_stream_t stream) {
  if (!x || !w || !y || M <= 0 || N <= 0 || K <= 0) return TEENY_ERR_BAD_ARG;
  const bool tma_ok = sxk == 1 && swk == 1 && syn == 1 && (sxm % 8 == 0) && (swn % 8 == 0) && sxm >= K && swn >= K &&
                      !((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) & 15);
  if (tma_ok)
    return gemm_bf16(B(x), sxm, B(w), swn, /*w_is_kn=*/false, B(bias), B(y), sym, M, N, K, scratch, scratch_bytes, S(stream));
  return gemm_bf16_generic(B(x), sxm, sxk, B(w), swk, swn, B(bias), B(y), sym, syn, M, N, K, S(stream));
}

size_t teeny_gemm_scratch_bytes(int M, int N, int K) { return gemm_bf16_scratch_bytes(M, N, K); }

// ---- attention ----
int flash_attention2_forward_entry_point_f32(const float* q, const float* k, const float* v, float* o, float* l,
                                             int n_ctx_q, int n_ctx_k, float softmax_scale, float, int bh,
                                             int head_dim, teeny_stream_t stream) {
  if (bh <= 0 || n_ctx_q <= 0 || n_ctx_k <= 0 || head_dim <= 0) return TEENY_ERR_BAD_ARG;
  return attention_generic<float>(q, k, v, o, l, contiguous_shape(bh, n_ctx_q, n_ctx_k, head_dim, softmax_scale), S(stream));
}

int flash_attention2_forward_entry_point_bf16(const teeny_bf16* q, const teeny_bf16* k, const teeny_bf16* v,
                                              teeny_bf16* o, float* l, int n_ctx_q, int n_ctx_k, float softmax_scale,
                                              float, int bh, int head_dim, teeny_stream_t stream) {
  if (bh <= 0 || n_ctx_q <= 0 || n_ctx_k <= 0 || head_dim <= 0) return TEENY_ERR_BAD_ARG;
  teeny_attn_shape t;
  const AttnShape s = contiguous_shape(bh, n_ctx_q, n_ctx_k, head_dim, softmax_scale);
  t.B = s.B; t.Hq = s.Hq; t.Hkv = s.Hkv; t.Sq = s.Sq; t.Skv = s.Skv; t.D = s.D;
  t.q_sb = s.q_sb; t.q_sh = s.q_sh; t.q_ss = s.q_ss; t.k_sb = s.k_sb; t.k_sh = s.k_sh; t.k_ss = s.k_ss;
  t.v_sb = s.v_sb; t.v_sh = s.v_sh; t.v_ss = s.v_ss; t.o_sb = s.o_sb; t.o_sh = s.o_sh; t.o_ss = s.o_ss;
  t.scale = s.scale; t.causal = 0;
  return teeny_flash_attn_fwd_bf16(q, k, v, o, l, &t, stream);
}

int teeny_flash_attn_fwd_bf16(const teeny_bf16* q, const teeny_bf16* k, const teeny_bf16* v, teeny_bf16* o, float* lse,
                              const teeny_attn_shape* shape, teeny_stream_t stream) {
  if (!shape) return TEENY_ERR_BAD_ARG;
  const AttnShape s = to_shape(*shape);
  if (s.D == 128) {
    const int rc = attention_prefill_bf16(B(q), B(k), B(v), B(o), lse, s, S(stream));
    if (rc != TEENY_ERR_ALIGNMENT) return rc;  // unaligned views fall through to the CUDA-core kernel
  }
  return attention_generic<bf16>(B(q), B(k), B(v), B(o), lse, s, S(stream));
}

int teeny_flash_attn_decode_bf16(const teeny_bf16* q, const teeny_bf16* k, const teeny_bf16* v, teeny_bf16* o,
                                 const teeny_attn_shape* shape, int kv_len, const int* kv_len_dev, void* scratch,
                                 size_t scratch_bytes, teeny_stream_t stream) {
  if (!shape) return TEENY_ERR_BAD_ARG;
  return attention_decode_bf16(B(q), B(k), B(v), B(o), to_shape(*shape), kv_len, kv_len_dev, scratch, scratch_bytes, S(stream));
}

int teeny_flash_attn_decode_bf16_static(const teeny_bf16* q, const teeny_bf16* k, const teeny_bf16* v, teeny_bf16* o,
                                        const teeny_attn_shape* shape, int kv_len, const int* kv_len_dev,
                                        teeny_stream_t stream) {
  if (!shape) return TEENY_ERR_BAD_ARG;
  return attention_decode_bf16_static(B(q), B(k), B(v), B(o), to_shape(*shape), kv_len, kv_len_dev, S(stream));
}

size_t teeny_attn_decode_static_limit(void) { return attention_decode_static_scratch_limit(); }

size_t teeny_attn_decode_scratch_bytes(int Bn, int Hq, int D, int max_kv) {
  return attention_decode_scratch_bytes(Bn, Hq, D, max_kv);
}

// ---- normalisation / elementwise ----
int rms_norm_forward_entry_point_f32(const float* x, float* y, const float* w, float* rrms, int M, int N, float eps,
                                     teeny_stream_t stream) {
  return rms_norm_f32(x, y, w, rrms, M, N, eps, S(stream));
}
int rms_norm_forward_entry_point_bf16(const teeny_bf16* x, teeny_bf16* y, const teeny_bf16* w, float* rrms, int M,
                                      int N, float eps, teeny_stream_t stream) {
  return rms_norm_bf16(B(x), N, B(y), N, B(w), rrms, M, N, eps, S(stream));
}
int silu_forward_entry_point_f32(const float* x, float* y, int n, teeny_stream_t s) { return silu_f32(x, y, n, S(s)); }
int silu_forward_entry_point_bf16(const teeny_bf16* x, teeny_bf16* y, int n, teeny_stream_t s) { return silu_bf16(B(x), B(y), n, S(s)); }
int elemwise_mul_forward_entry_point_f32(const float* a, const float* b, float* o, int n, teeny_stream_t s) { return mul_f32(a, b, o, n, S(s)); }
int elemwise_mul_forward_entry_point_bf16(const teeny_bf16* a, const teeny_bf16* b, teeny_bf16* o, int n, teeny_stream_t s) { return mul_bf16(B(a), B(b), B(o), n, S(s)); }
int elemwise_add_forward_entry_point_f32(const float* a, const float* b, float* o, int n, teeny_stream_t s) { return add_f32(a, b, o, n, S(s)); }
int elemwise_add_forward_entry_point_bf16(const teeny_bf16* a, const teeny_bf16* b, teeny_bf16* o, int n, teeny_stream_t s) { return add_bf16(B(a), B(b), B(o), n, S(s)); }
int softmax_forward_entry_point_f32(const float* x, float* y, int r, int c, teeny_stream_t s) { return softmax_f32(x, y, r, c, S(s)); }
int softmax_forward_entry_point_bf16(const teeny_bf16* x, teeny_bf16* y, int r, int c, teeny_stream_t s) { return softmax_bf16(B(x), B(y), r, c, S(s)); }

int teeny_add_rms_norm_bf16(const teeny_bf16* x, teeny_bf16* residual, teeny_bf16* y, const teeny_bf16* w, int M, int N,
                            float eps, teeny_stream_t s) {
  return add_rms_norm_bf16(B(x), N, B(residual), N, B(y), N, B(w), M, N, eps, S(s));
}
int teeny_silu_mul_bf16(const teeny_bf16* gate_up, long long ld, teeny_bf16* out, int T, int inter, teeny_stream_t s) {
  return silu_mul_bf16(B(gate_up), ld, B(out), T, inter, S(s));
}
int teeny_linear_swiglu_bf16(const teeny_bf16* x, long long ldx, const teeny_bf16* w, long long ldw, teeny_bf16* y,
                             long long ldy, int M, int N, int K, teeny_stream_t s) {
  if (ldx > 0x7fffffffLL || ldw > 0x7fffffffLL || ldy > 0x7fffffffLL || ldx < K || ldw < K) return TEENY_ERR_BAD_ARG;
  return gemm_bf16(B(x), static_cast<int>(ldx), B(w), static_cast<int>(ldw), false, nullptr, B(y),
                   static_cast<int>(ldy), M, N, K, nullptr, 0, S(s), /*swiglu=*/true);
}
int teeny_linear_w8a16_forward(const teeny_bf16* x, long long ldx, const void* w_fp8, long long ldw, const float* w_scale,
                               int scale_kind, int group_size, const teeny_bf16* bias, teeny_bf16* y, long long ldy, int M,
                               int N, int K, int swiglu, void* global_scratch, size_t global_scratch_bytes,
                               teeny_stream_t s) {
  if (ldx > 0x7fffffffLL || ldw > 0x7fffffffLL || ldy > 0x7fffffffLL || ldx < K || ldw < K) return TEENY_ERR_BAD_ARG;
  return linear_w8a16(B(x), static_cast<int>(ldx), static_cast<const uint8_t*>(w_fp8), static_cast<int>(ldw), w_scale,
                      scale_kind, group_size, B(bias), B(y), static_cast<int>(ldy), M, N, K, global_scratch,
                      global_scratch_bytes, S(s), swiglu != 0);
}
int teeny_split_fp8_e4m3(const teeny_bf16* x, long long ldx, void* out, long long ldo, float* x_scale, int M, int K,
                         teeny_stream_t s) {
  return split_e4m3(B(x), ldx, static_cast<uint8_t*>(out), ldo, x_scale, M, K, S(s));
}
int teeny_linear_w8a8x2_forward(const void* x_fp8, long long ldx, const float* x_scale, const void* w_fp8, long long ldw,
                                const float* w_scale, int scale_kind, const teeny_bf16* bias, teeny_bf16* y, long long ldy,
                                int M, int N, int K, int swiglu, teeny_stream_t s) {
  if (ldx > 0x7fffffffLL || ldw > 0x7fffffffLL || ldy > 0x7fffffffLL || ldx < K || ldw < K) return TEENY_ERR_BAD_ARG;
  return gemm_w8a8x2_skinny(static_cast<const uint8_t*>(x_fp8), static_cast<int>(ldx), x_scale,
                            static_cast<const uint8_t*>(w_fp8), static_cast<int>(ldw), w_scale, scale_kind, B(bias), B(y),
                            static_cast<int>(ldy), M, N, K, S(s), swiglu != 0);
}
size_t teeny_linear_w8a16_scratch_bytes(int M, int N, int K) { return linear_w8a16_scratch_bytes(M, N, K); }
int teeny_dequant_fp8_e4m3_bf16(const void* w_fp8, long long ldw, const float* w_scale, int scale_kind, int group_size,
                                teeny_bf16* out, long long ldo, int N, int K, teeny_stream_t s) {
  return dequant_e4m3_bf16(static_cast<const uint8_t*>(w_fp8), ldw, w_scale, scale_kind, group_size, B(out), ldo, N, K, S(s));
}
int teeny_dequant_int_bf16(const void* q, int bits, const float* w_scale, const int* zero_point, int scale_kind,
                           int group_size, teeny_bf16* out, long long ldo, int N, int K, teeny_stream_t s) {
  return dequant_int_bf16(q, bits, w_scale, zero_point, scale_kind, group_size, B(out), ldo, N, K, S(s));
}
int teeny_fp8_e4m3_count_nan(const void* bytes, size_t n, unsigned* count, teeny_stream_t s) {
  return e4m3_count_nan(static_cast<const uint8_t*>(bytes), n, count, S(s));
}
int teeny_rope_table_bf16(const float* inv_freq, teeny_bf16* c, teeny_bf16* sn, int max_pos, int D, teeny_stream_t s) {
  return rope_table_bf16(inv_freq, B(c), B(sn), max_pos, D, S(s));
}
int teeny_qk_norm_rope_kv_bf16(teeny_bf16* qkv, long long ld, const teeny_bf16* qw, const teeny_bf16* kw,
                               const teeny_bf16* c, const teeny_bf16* sn, teeny_bf16* kc, teeny_bf16* vc, int T, int Sx,
                               int Hq, int Hkv, int D, int max_len, int pos0, const int* pos0_dev, float eps,
                               teeny_stream_t s) {
  return qk_norm_rope_kv_bf16(B(qkv), ld, B(qw), B(kw), B(c), B(sn), B(kc), B(vc), T, Sx, Hq, Hkv, D, max_len, pos0,
                              pos0_dev, eps, S(s));
}
int teeny_embedding_bf16(const int* ids, const teeny_bf16* table, teeny_bf16* out, int T, int hidden, int vocab,
                         teeny_stream_t s) {
  return embedding_bf16(ids, B(table), B(out), T, hidden, vocab, S(s));
}
int teeny_argmax_bf16(const teeny_bf16* logits, long long ld, float* bv, int* bi, int rows, int cols, int off,
                      teeny_stream_t s) {
  return argmax_bf16(B(logits), ld, bv, bi, rows, cols, off, S(s));
}
int teeny_argmax_combine(const float* vals, const int* idx, int* out_idx, int parts, int rows, teeny_stream_t s) {
  return argmax_combine(vals, idx, out_idx, parts, rows, S(s));
}
int teeny_sample_top_k_top_p_bf16(const teeny_bf16* logits, long long ld, int rows, int cols, float temperature,
                                  int top_k, float top_p, const float* u, int* out_idx, float* out_prob,
                                  teeny_stream_t s) {
  return sample_top_k_top_p_bf16(B(logits), ld, rows, cols, temperature, top_k, top_p, u, out_idx, out_prob, S(s));
}
int teeny_sample_candidates_bf16(const teeny_bf16* logits, long long ld, int rows, int cols, int top_k, int idx_offset,
                                 unsigned long long* cand_out, teeny_stream_t stream) {
  return sample_candidates_bf16(B(logits), ld, rows, cols, top_k, idx_offset, cand_out, S(stream));
}
int teeny_sample_merge(const unsigned long long* lists, int parts, size_t list_stride, int rows, float temperature,
                       int top_k, float top_p, const float* u, int* out_idx, float* out_prob, teeny_stream_t stream) {
  return sample_merge(lists, parts, list_stride, rows, temperature, top_k, top_p, u, out_idx, out_prob, S(stream));
}

}  // extern "C"

// Kernel-timeline registry of development builds (-DTEENY_TRACE): one dump function per translation unit.
#ifdef TEENY_TRACE
namespace { struct TraceTu { const char* name; teeny_trace_dump_fn fn; }; TraceTu g_tus[16]; int g_ntu = 0; }
extern "C" void teeny_trace_register(const char* tu, teeny_trace_dump_fn fn) { if (g_ntu < 16) g_tus[g_ntu++] = {tu, fn}; }
extern "C" int teeny_trace_count() { return g_ntu; }
extern "C" const char* teeny_trace_name(int i) { return g_tus[i].name; }
extern "C" int teeny_trace_dump(int i, unsigned long long* out, unsigned cap, int reset) { return g_tus[i].fn(out, cap, reset); }
#endif
