// Attention kernels that are not tcgen05-shaped.
//
// 1. attention_decode_bf16: one query token per sequence against a long KV cache.  HBM-bound (every K and V byte is
//    read once, the query heads of a KV group share it), so the design goal is streaming the cache with 16-byte
//    coalesced loads and enough loads in flight; the arithmetic runs on warp-level mma.sync tiles fed straight from
//    registers (a 128-row tcgen05 tile would be 97 % padding for 4 query heads).  Split over the sequence: each CTA
//    takes kDecChunk keys of one (batch, kv head), every warp a 16-key slice at a time with an online softmax, warps
//    are merged through shared memory, per-chunk partials (m, l, O) go to scratch and a second kernel merges chunks.
// 2. attention_generic<T>: any head_dim <= 256, f32 or bf16, one warp per query row, sequential online softmax --
//    the reference kernel's own recurrence; used for the f32 entry point and for shapes the tcgen05 kernel
//    does not cover.
#include "common.cuh"
#include "kernels.h"

namespace teeny {

namespace {

constexpr int kDecChunk = 512;
constexpr int kDecWarps = 4;
constexpr int kDecThreads = kDecWarps * 32;
constexpr int kHD = 128;

struct DecodeArgs {
  const bf16 *q, *k, *v;
  float* part_o;   // [B, Hkv, chunks, G, 128]
  float* part_ml;  // [B, Hkv, chunks, G, 2]
  long long q_sb, q_sh, k_sb, k_sh, k_ss, v_sb, v_sh, v_ss;
  int Hkv, G, max_chunks;
  int kv_len;
  const int* kv_len_dev;
  float scale_log2;
};

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint4 ldg_nc(const bf16* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}

// Fragment conventions (mma.m16n8k16, g = lane / 4, c = lane % 4):
//   A (16 x 16, rows = query heads of the group, rows >= G are zero): a0 = (row g, k 2c..2c+1), a2 = (row g, k 2c+8..)
//   B (16 x 8): b0 = (k 2c..2c+1, col g), b1 = (k 2c+8.., col g)
//   C (16 x 8): c0,c1 = (row g, cols 2c, 2c+1); c2,c3 = rows g+8 (padding, stays zero)
// The contraction index of Q K^T is d, and any permutation of d may be used as long as A and B agree: lane (g, c)
// loads the 16 contiguous bytes d = 32p + 8c .. +8 of "its" key (B side) or head (A side), p = 0..3, and feeds the
// first four values to k-step 2p and the last four to k-step 2p+1.  Each warp-wide load therefore covers 8 key rows
// x 64 contiguous bytes.
// For P V the contraction index is the key and the output column is d (again any labelling works): lane (g, c) loads
// d = 64 ps + 8g .. +8 of keys 2c, 2c+1, 2c+8, 2c+9 and byte-permutes pairs of keys into one register; MMA (ps, i)
// then produces O[head][d = 64 ps + 8 n + i] in column n.
template <int G>
__global__ void __launch_bounds__(kDecThreads)
attention_decode_kernel(const DecodeArgs a) {
  pdl_wait();
  const int chunk = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  const int L = a.kv_len_dev ? *a.kv_len_dev : a.kv_len;
  const int key_begin = chunk * kDecChunk;
  if (key_begin >= L) return;
  const int key_end = min(L, key_begin + kDecChunk);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, c = lane & 3;

  // Q fragments: head = hk * G + g (zero rows beyond G)
  uint4 qf[4];
  if (g < G) {
    const bf16* qp = a.q + b * a.q_sb + (hk * G + g) * a.q_sh;
#pragma unroll
    for (int p = 0; p < 4; ++p) qf[p] = *reinterpret_cast<const uint4*>(qp + 32 * p + 8 * c);
  } else {
#pragma unroll
    for (int p = 0; p < 4; ++p) qf[p] = make_uint4(0, 0, 0, 0);
  }
  const bf16* kbase = a.k + b * a.k_sb + hk * a.k_sh;
  const bf16* vbase = a.v + b * a.v_sb + hk * a.v_sh;

  float acc[2][8][4];
#pragma unroll
  for (int ps = 0; ps < 2; ++ps)
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[ps][i][e] = 0.0f;
  float m = -INFINITY, l = 0.0f;  // per row g (replicated over the 4 lanes of the group)

  // K and V fragments of one 16-key slice (64 registers).  The slice after the current one is loaded before the
  // current one is consumed, so every warp keeps 8 KB of cache reads in flight while its tensor-core work runs.
  struct Slice { uint4 kf[2][4]; uint4 vf[2][4]; };
  auto load_slice = [&](Slice& f, int kb) {
#pragma unroll
    for (int nb = 0; nb < 2; ++nb) {
      const int key = min(kb + nb * 8 + g, L - 1);  // clamp: masked later, but the load must stay in valid rows
      const bf16* kp = kbase + static_cast<long long>(key) * a.k_ss + 8 * c;
#pragma unroll
      for (int p = 0; p < 4; ++p) f.kf[nb][p] = ldg_nc(kp + 32 * p);
    }
    const int k0 = min(kb + 2 * c, L - 1), k1 = min(kb + 2 * c + 1, L - 1);
    const int k2 = min(kb + 8 + 2 * c, L - 1), k3 = min(kb + 9 + 2 * c, L - 1);
#pragma unroll
    for (int ps = 0; ps < 2; ++ps) {
      const int d0 = 64 * ps + 8 * g;
      f.vf[ps][0] = ldg_nc(vbase + static_cast<long long>(k0) * a.v_ss + d0);
      f.vf[ps][1] = ldg_nc(vbase + static_cast<long long>(k1) * a.v_ss + d0);
      f.vf[ps][2] = ldg_nc(vbase + static_cast<long long>(k2) * a.v_ss + d0);
      f.vf[ps][3] = ldg_nc(vbase + static_cast<long long>(k3) * a.v_ss + d0);
    }
  };
  constexpr int kStride = kDecWarps * 16;
  Slice cur;
  if (key_begin + warp * 16 < key_end) load_slice(cur, key_begin + warp * 16);
#pragma unroll 2
  for (int kb = key_begin + warp * 16; kb < key_end; kb += kStride) {
    Slice nxt;
    if (kb + kStride < key_end) load_slice(nxt, kb + kStride);
    // ---- S = Q K^T for 16 keys (two 8-key column blocks) ----
    float s[2][4];
#pragma unroll
    for (int nb = 0; nb < 2; ++nb) {
      s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.0f;
#pragma unroll
      for (int p = 0; p < 4; ++p) {
        mma_bf16_16816(s[nb], qf[p].x, 0u, qf[p].y, 0u, cur.kf[nb][p].x, cur.kf[nb][p].y);
        mma_bf16_16816(s[nb], qf[p].z, 0u, qf[p].w, 0u, cur.kf[nb][p].z, cur.kf[nb][p].w);
      }
    }
    // ---- online softmax on row g: this lane holds keys kb + nb*8 + 2c + {0,1} ----
    float tmax = -INFINITY;
#pragma unroll
    for (int nb = 0; nb < 2; ++nb)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int key = kb + nb * 8 + 2 * c + e;
        s[nb][e] = key < key_end ? s[nb][e] * a.scale_log2 : -INFINITY;
        tmax = fmaxf(tmax, s[nb][e]);
      }
    tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 1));
    tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 2));
    const float m_new = fmaxf(m, tmax);  // finite: key kb itself is always < key_end
    const float alpha = ex2(m - m_new);  // m = -inf on the first slice -> 0
    m = m_new;
    float p[2][2], psum = 0.0f;
#pragma unroll
    for (int nb = 0; nb < 2; ++nb)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        p[nb][e] = ex2(s[nb][e] - m);
        psum += p[nb][e];
      }
    psum += __shfl_xor_sync(0xffffffffu, psum, 1);
    psum += __shfl_xor_sync(0xffffffffu, psum, 2);
    l = l * alpha + psum;
#pragma unroll
    for (int ps = 0; ps < 2; ++ps)
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        acc[ps][i][0] *= alpha;
        acc[ps][i][1] *= alpha;
      }
    const uint32_t pa0 = pack_bf16x2(p[0][0], p[0][1]);  // keys 2c, 2c+1
    const uint32_t pa2 = pack_bf16x2(p[1][0], p[1][1]);  // keys 2c+8, 2c+9
    // ---- O += P V ----
#pragma unroll
    for (int ps = 0; ps < 2; ++ps) {
      const uint32_t w0[4] = {cur.vf[ps][0].x, cur.vf[ps][0].y, cur.vf[ps][0].z, cur.vf[ps][0].w};
      const uint32_t w1[4] = {cur.vf[ps][1].x, cur.vf[ps][1].y, cur.vf[ps][1].z, cur.vf[ps][1].w};
      const uint32_t w2[4] = {cur.vf[ps][2].x, cur.vf[ps][2].y, cur.vf[ps][2].z, cur.vf[ps][2].w};
      const uint32_t w3[4] = {cur.vf[ps][3].x, cur.vf[ps][3].y, cur.vf[ps][3].z, cur.vf[ps][3].w};
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const uint32_t sel = (i & 1) ? 0x7632u : 0x5410u;
        const uint32_t b0 = prmt(w0[i >> 1], w1[i >> 1], sel);  // (key 2c, key 2c+1) at d index i
        const uint32_t b1 = prmt(w2[i >> 1], w3[i >> 1], sel);  // (key 2c+8, key 2c+9)
        mma_bf16_16816(acc[ps][i], pa0, 0u, pa2, 0u, b0, b1);
      }
    }
    cur = nxt;
  }

  pdl_trigger();  // cache streaming done; what follows is the small merge
  // ---- merge the warps of this CTA ----
  __shared__ float sm_ml[kDecWarps][8][2];
  __shared__ float sm_o[kDecWarps][G][kHD];
  if (c == 0 && g < G) {
    sm_ml[warp][g][0] = m;
    sm_ml[warp][g][1] = l;
  }
  if (g < G) {
#pragma unroll
    for (int ps = 0; ps < 2; ++ps)
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        sm_o[warp][g][64 * ps + 8 * (2 * c) + i] = acc[ps][i][0];
        sm_o[warp][g][64 * ps + 8 * (2 * c + 1) + i] = acc[ps][i][1];
      }
  }
  __syncthreads();
  const size_t slot = (static_cast<size_t>(b) * a.Hkv + hk) * a.max_chunks + chunk;
  for (int idx = threadIdx.x; idx < G * kHD; idx += kDecThreads) {
    const int gg = idx / kHD, d = idx - gg * kHD;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) mm = fmaxf(mm, sm_ml[w][gg][0]);  // warps without keys hold -inf
    float ll = 0.0f, oo = 0.0f;
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) {
      const float wm = sm_ml[w][gg][0];
      const float sc = (wm == -INFINITY) ? 0.0f : ex2(wm - mm);
      ll += sm_ml[w][gg][1] * sc;
      oo += sm_o[w][gg][d] * sc;
    }
    a.part_o[(slot * G + gg) * kHD + d] = oo;
    if (d == 0) {
      a.part_ml[(slot * G + gg) * 2 + 0] = mm;
      a.part_ml[(slot * G + gg) * 2 + 1] = ll;
    }
  }
}

// grid (Hq, B), 128 threads: thread d merges the valid chunks of head h.
__global__ void attention_decode_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                                bf16* __restrict__ o, long long o_sb, long long o_sh, int Hkv, int G,
                                                int max_chunks, int kv_len, const int* __restrict__ kv_len_dev) {
  pdl_wait();
  const int h = blockIdx.x, b = blockIdx.y, d = threadIdx.x;
  const int L = kv_len_dev ? *kv_len_dev : kv_len;
  const int chunks = (L + kDecChunk - 1) / kDecChunk;
  const int hk = h / G, gg = h - hk * G;
  const size_t slot0 = (static_cast<size_t>(b) * Hkv + hk) * max_chunks;
  float mm = -INFINITY;
  for (int ch = 0; ch < chunks; ++ch) mm = fmaxf(mm, part_ml[((slot0 + ch) * G + gg) * 2]);
  float ll = 0.0f, oo = 0.0f;
  for (int ch = 0; ch < chunks; ++ch) {
    const size_t s = (slot0 + ch) * G + gg;
    const float sc = ex2(part_ml[s * 2] - mm);
    ll += part_ml[s * 2 + 1] * sc;
    oo += part_o[s * kHD + d] * sc;
  }
  o[b * o_sb + h * o_sh + d] = __float2bfloat16_rn(oo / ll);
}

// ------------------------------------------------------------------------------------------------
template <typename T> __device__ __forceinline__ float ld_as_f(const T* p);
template <> __device__ __forceinline__ float ld_as_f<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ld_as_f<bf16>(const bf16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void st_from_f(float* p, float v) { *p = v; }
__device__ __forceinline__ void st_from_f(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

// one warp per (query row, head, batch); lane owns d = lane, lane + 32, ... (up to 8 values: D <= 256)
template <typename T>
__global__ void attention_generic_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                                         T* __restrict__ o, float* __restrict__ lse, const AttnShape s) {
  pdl_wait();
  const long long wid = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long rows = static_cast<long long>(s.B) * s.Hq * s.Sq;
  if (wid >= rows) return;
  const int i = static_cast<int>(wid % s.Sq);
  const int h = static_cast<int>((wid / s.Sq) % s.Hq);
  const int b = static_cast<int>(wid / (static_cast<long long>(s.Sq) * s.Hq));
  const int hk = h / (s.Hq / s.Hkv);
  const T* qr = q + b * s.q_sb + h * s.q_sh + i * s.q_ss;
  const T* kb = k + b * s.k_sb + hk * s.k_sh;
  const T* vb = v + b * s.v_sb + hk * s.v_sh;
  float qv[8], acc[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const int d = lane + 32 * e;
    qv[e] = d < s.D ? ld_as_f(qr + d) : 0.0f;
    acc[e] = 0.0f;
  }
  float m = -INFINITY, l = 0.0f;
  const int last = s.causal ? min(s.Skv - 1, i + (s.Skv - s.Sq)) : s.Skv - 1;
  for (int j = 0; j <= last; ++j) {
    const T* kr = kb + j * s.k_ss;
    const T* vr = vb + j * s.v_ss;
    float dot = 0.0f;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const int d = lane + 32 * e;
      if (d < s.D) dot += qv[e] * ld_as_f(kr + d);
    }
    dot = warp_sum(dot) * s.scale;
    const float m_new = fmaxf(m, dot);
    const float corr = expf(m - m_new);
    const float p = expf(dot - m_new);
    l = corr * l + p;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const int d = lane + 32 * e;
      if (d < s.D) acc[e] = corr * acc[e] + p * ld_as_f(vr + d);
    }
    m = m_new;
  }
  T* orow = o + b * s.o_sb + h * s.o_sh + i * s.o_ss;
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const int d = lane + 32 * e;
    if (d < s.D) st_from_f(orow + d, acc[e] / l);
  }
  if (lse && lane == 0) lse[(static_cast<long long>(b) * s.Hq + h) * s.Sq + i] = m + logf(l);
}

}  // namespace

size_t attention_decode_scratch_bytes(int B, int Hq, int D, int max_kv) {
  if (B <= 0 || Hq <= 0 || D <= 0 || max_kv <= 0) return 0;
  const size_t chunks = (static_cast<size_t>(max_kv) + kDecChunk - 1) / kDecChunk;
  return static_cast<size_t>(B) * Hq * chunks * (D + 2) * sizeof(float);
}

int attention_decode_bf16(const bf16* q, const bf16* k, const bf16* v, bf16* o, const AttnShape& s, int kv_len,
                          const int* kv_len_dev, void* scratch, size_t scratch_bytes, cudaStream_t stream) {
  if (!q || !k || !v || !o || !scratch || s.B <= 0 || s.Hq <= 0 || s.Hkv <= 0 || s.Skv <= 0) return TEENY_ERR_BAD_ARG;
  if (s.D != kHD || s.Hq % s.Hkv != 0 || s.Sq != 1) return TEENY_ERR_BAD_ARG;
  if (!kv_len_dev && (kv_len <= 0 || kv_len > s.Skv)) return TEENY_ERR_BAD_ARG;
  const int G = s.Hq / s.Hkv;
  if (G != 1 && G != 2 && G != 4 && G != 8) return TEENY_ERR_BAD_ARG;
  const long long strides[] = {s.q_sb, s.q_sh, s.k_sb, s.k_sh, s.k_ss, s.v_sb, s.v_sh, s.v_ss};
  for (long long st : strides)
    if (st % 8 != 0) return TEENY_ERR_ALIGNMENT;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v)) & 15)
    return TEENY_ERR_ALIGNMENT;
  // s.Skv is the cache capacity the grid is sized for; the live length comes from kv_len / kv_len_dev
  if (scratch_bytes < attention_decode_scratch_bytes(s.B, s.Hq, s.D, s.Skv)) return TEENY_ERR_SCRATCH;
  const int max_chunks = (s.Skv + kDecChunk - 1) / kDecChunk;
  if (s.Hkv > 65535 || s.B > 65535) return TEENY_ERR_BAD_ARG;

  DecodeArgs a{};
  a.q = q; a.k = k; a.v = v;
  a.part_o = static_cast<float*>(scratch);
  a.part_ml = a.part_o + static_cast<size_t>(s.B) * s.Hq * max_chunks * kHD;
  a.q_sb = s.q_sb; a.q_sh = s.q_sh;
  a.k_sb = s.k_sb; a.k_sh = s.k_sh; a.k_ss = s.k_ss;
  a.v_sb = s.v_sb; a.v_sh = s.v_sh; a.v_ss = s.v_ss;
  a.Hkv = s.Hkv; a.G = G; a.max_chunks = max_chunks;
  a.kv_len = kv_len; a.kv_len_dev = kv_len_dev;
  a.scale_log2 = s.scale * 1.4426950408889634f;
  dim3 grid(max_chunks, s.Hkv, s.B);
  switch (G) {
    case 1: launch_kernel(attention_decode_kernel<1>, dim3(grid), dim3(kDecThreads), 0, stream, 1, a); break;
    case 2: launch_kernel(attention_decode_kernel<2>, dim3(grid), dim3(kDecThreads), 0, stream, 1, a); break;
    case 4: launch_kernel(attention_decode_kernel<4>, dim3(grid), dim3(kDecThreads), 0, stream, 1, a); break;
    default: launch_kernel(attention_decode_kernel<8>, dim3(grid), dim3(kDecThreads), 0, stream, 1, a); break;
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return static_cast<int>(e);
  launch_kernel(attention_decode_combine_kernel, dim3(dim3(s.Hq, s.B)), dim3(kHD), 0, stream, 1, a.part_o, a.part_ml, o, s.o_sb, s.o_sh, s.Hkv,
                                                                       G, max_chunks, kv_len, kv_len_dev);
  return static_cast<int>(cudaGetLastError());
}

// ------------------------------------------------------------------------------------------------
// Decode attention without a caller-provided scratch buffer.
//
// Some hosts cannot hand this library device memory beyond the tensors themselves: an inference server whose
// allocator reserved every byte of HBM at start-up, or a steady-state decode loop in which a driver allocation is
// forbidden because cudaMalloc synchronises the whole device.  For them the split-KV partials live in the
// fixed-size device array below (part of the library image: every GPU that loads the library holds these bytes
// until the process exits).  Shapes whose partials do not fit are rejected, not truncated.
//
// All calls on one device share the array.  Nothing in it needs to start at zero -- every partial that the
// combine step reads was written by the same call -- but two calls that overlap on the GPU (different streams)
// would write the same slots, so such calls race and must be serialised by the caller.
// ------------------------------------------------------------------------------------------------
namespace {
constexpr size_t kStaticDecodeScratchBytes = size_t(8) << 20;  // 8 MiB, e.g. B=32, Hq=32, cache capacity 4096
static __device__ __align__(256) unsigned char g_static_decode_scratch[kStaticDecodeScratchBytes];
void* g_static_decode_scratch_ptr[64] = {};  // per device: resolved address of the array
}  // namespace

size_t attention_decode_static_scratch_limit() { return kStaticDecodeScratchBytes; }

int attention_decode_bf16_static(const bf16* q, const bf16* k, const bf16* v, bf16* o, const AttnShape& s, int kv_len,
                                 const int* kv_len_dev, cudaStream_t stream) {
  const size_t need = attention_decode_scratch_bytes(s.B, s.Hq, s.D, s.Skv);
  if (need == 0) return TEENY_ERR_BAD_ARG;
  if (need > kStaticDecodeScratchBytes) return TEENY_ERR_STATIC_LIMIT;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 0 || dev >= 64) return TEENY_ERR_BAD_ARG;
  if (!g_static_decode_scratch_ptr[dev]) {
    // In host code the array's name is only a handle: the address a kernel can use comes from the runtime, once
    // per device, with that device current.
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_decode_scratch);
    if (e != cudaSuccess) return static_cast<int>(e);
    g_static_decode_scratch_ptr[dev] = p;
  }
  return attention_decode_bf16(q, k, v, o, s, kv_len, kv_len_dev, g_static_decode_scratch_ptr[dev],
                               kStaticDecodeScratchBytes, stream);
}

template <typename T>
int attention_generic(const T* q, const T* k, const T* v, T* o, float* lse, const AttnShape& s, cudaStream_t stream) {
  if (!q || !k || !v || !o || s.B <= 0 || s.Hq <= 0 || s.Hkv <= 0 || s.Sq <= 0 || s.Skv <= 0 || s.D <= 0)
    return TEENY_ERR_BAD_ARG;
  if (s.D > 256 || s.Hq % s.Hkv != 0 || (s.causal && s.Skv < s.Sq)) return TEENY_ERR_BAD_ARG;
  const long long rows = static_cast<long long>(s.B) * s.Hq * s.Sq;
  const long long blocks = (rows + 3) / 4;
  if (blocks > 0x7fffffffLL) return TEENY_ERR_BAD_ARG;
  launch_kernel(attention_generic_kernel<T>, dim3(static_cast<int>(blocks)), dim3(128), 0, stream, 1, q, k, v, o, lse, s);
  return static_cast<int>(cudaGetLastError());
}
template int attention_generic<float>(const float*, const float*, const float*, float*, float*, const AttnShape&, cudaStream_t);
template int attention_generic<bf16>(const bf16*, const bf16*, const bf16*, bf16*, float*, const AttnShape&, cudaStream_t);

}  // namespace teeny
