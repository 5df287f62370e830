// Bandwidth-bound kernels of the Qwen3 forward path: RMSNorm (+ fused residual add), per-head QK-norm + RoPE +
// KV-cache append, SiLU*up, residual add, embedding gather, softmax, argmax.  All use 128-bit coalesced global
// accesses where alignment allows and warp shuffles for the row reductions; arithmetic is f32 with the same
// rounding points as the PyTorch graph the reference records for Qwen3 (bf16 tensors between ops).
#include "common.cuh"
#include "kernels.h"

namespace teeny {

namespace {

constexpr int kEwThreads = 256;

inline int ew_grid(long long work_items, int per_block) {
  long long g = (work_items + per_block - 1) / per_block;
  const long long cap = static_cast<long long>(sm_count()) * 16;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  return static_cast<int>(g);
}

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : 0.0f;
  t = warp_sum(t);
  __syncthreads();
  return t;
}

__device__ __forceinline__ float block_max(float v, float* red) {  // of non-negative values
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : 0.0f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) t = fmaxf(t, __shfl_xor_sync(0xffffffffu, t, o));
  __syncthreads();
  return t;
}

__device__ __forceinline__ float silu_f(float x) { return x * (1.0f / (1.0f + expf(-x))); }

struct OpSilu { __device__ float operator()(float a, float) const { return silu_f(a); } };
struct OpMul { __device__ float operator()(float a, float b) const { return a * b; } };
struct OpAdd { __device__ float operator()(float a, float b) const { return a + b; } };

// ---- flat elementwise, f32 ----
template <typename Op, bool BINARY>
__global__ void ew_f32_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ o,
                              long long n, bool vec) {
  pdl_wait();
  Op op;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (vec) {
    const long long n4 = n >> 2;
    for (long long v = i; v < n4; v += stride) {
      const float4 x = reinterpret_cast<const float4*>(a)[v];
      float4 y = BINARY ? reinterpret_cast<const float4*>(b)[v] : make_float4(0, 0, 0, 0);
      float4 r;
      r.x = op(x.x, y.x); r.y = op(x.y, y.y); r.z = op(x.z, y.z); r.w = op(x.w, y.w);
      reinterpret_cast<float4*>(o)[v] = r;
    }
    for (long long t = (n4 << 2) + i; t < n; t += stride) o[t] = op(a[t], BINARY ? b[t] : 0.0f);
  } else {
    for (; i < n; i += stride) o[i] = op(a[i], BINARY ? b[i] : 0.0f);
  }
}

// ---- flat elementwise, bf16 (f32 math, one rounding) ----
template <typename Op, bool BINARY>
__global__ void ew_bf16_kernel(const bf16* __restrict__ a, const bf16* __restrict__ b, bf16* __restrict__ o,
                               long long n, bool vec) {
  pdl_wait();
  Op op;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (vec) {
    const long long n8 = n >> 3;
    for (long long v = i; v < n8; v += stride) {
      const uint4 x = reinterpret_cast<const uint4*>(a)[v];
      const uint4 y = BINARY ? reinterpret_cast<const uint4*>(b)[v] : make_uint4(0, 0, 0, 0);
      uint4 r;
      r.x = pack_bf16x2(op(bf16_lo(x.x), bf16_lo(y.x)), op(bf16_hi(x.x), bf16_hi(y.x)));
      r.y = pack_bf16x2(op(bf16_lo(x.y), bf16_lo(y.y)), op(bf16_hi(x.y), bf16_hi(y.y)));
      r.z = pack_bf16x2(op(bf16_lo(x.z), bf16_lo(y.z)), op(bf16_hi(x.z), bf16_hi(y.z)));
      r.w = pack_bf16x2(op(bf16_lo(x.w), bf16_lo(y.w)), op(bf16_hi(x.w), bf16_hi(y.w)));
      reinterpret_cast<uint4*>(o)[v] = r;
    }
    for (long long t = (n8 << 3) + i; t < n; t += stride)
      o[t] = __float2bfloat16_rn(op(__bfloat162float(a[t]), BINARY ? __bfloat162float(b[t]) : 0.0f));
  } else {
    for (; i < n; i += stride)
      o[i] = __float2bfloat16_rn(op(__bfloat162float(a[i]), BINARY ? __bfloat162float(b[i]) : 0.0f));
  }
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

template <typename Op, bool BINARY>
int launch_ew_f32(const float* a, const float* b, float* o, long long n, cudaStream_t st) {
  if (!a || !o || (BINARY && !b) || n < 0) return TEENY_ERR_BAD_ARG;
  if (n == 0) return TEENY_OK;
  const bool vec = aligned16(a) && aligned16(o) && (!BINARY || aligned16(b));
  launch_kernel(ew_f32_kernel<Op, BINARY>, dim3(ew_grid((n + 3) / 4, kEwThreads)), dim3(kEwThreads), 0, st, 1, a, b, o, n, vec);
  return static_cast<int>(cudaGetLastError());
}
template <typename Op, bool BINARY>
int launch_ew_bf16(const bf16* a, const bf16* b, bf16* o, long long n, cudaStream_t st) {
  if (!a || !o || (BINARY && !b) || n < 0) return TEENY_ERR_BAD_ARG;
  if (n == 0) return TEENY_OK;
  const bool vec = aligned16(a) && aligned16(o) && (!BINARY || aligned16(b));
  launch_kernel(ew_bf16_kernel<Op, BINARY>, dim3(ew_grid((n + 7) / 8, kEwThreads)), dim3(kEwThreads), 0, st, 1, a, b, o, n, vec);
  return static_cast<int>(cudaGetLastError());
}

// ---- RMSNorm, f32, one CTA per row (reference semantics: y = x * rrms * w) ----
__global__ void rms_norm_f32_kernel(const float* __restrict__ x, float* __restrict__ y, const float* __restrict__ w,
                                    float* __restrict__ rrms, int N, float eps) {
  pdl_wait();
  __shared__ float red[32];
  const float* xr = x + static_cast<size_t>(blockIdx.x) * N;
  float* yr = y + static_cast<size_t>(blockIdx.x) * N;
  float sq = 0.0f;
  for (int c = threadIdx.x; c < N; c += blockDim.x) sq += xr[c] * xr[c];
  sq = block_sum(sq, red);
  const float rr = 1.0f / sqrtf(sq * (1.0f / static_cast<float>(N)) + eps);
  if (threadIdx.x == 0 && rrms) rrms[blockIdx.x] = rr;
  for (int c = threadIdx.x; c < N; c += blockDim.x) yr[c] = xr[c] * rr * w[c];
}

// ---- RMSNorm, bf16, Qwen3 rounding.  One CTA per row; the row stays in registers between the two phases. ----
// VPT = 16-byte vectors per thread (N <= VPT * 8 * blockDim).  ADD: x is added into `res` first (bf16 add).
// y8 != null: the normed row is ALSO written as two-term FP8 (hi bytes to row `row` of y8, lo bytes to row gridDim.x +
// row; row stride ld8 bytes; y8_scale[row] = 1 / s), what split_e4m3_kernel would make of y, for the GEMM variant that
// takes its activations that way.
template <int VPT, bool ADD>
__global__ void rms_norm_bf16_kernel(const bf16* __restrict__ x, long long ldx, bf16* __restrict__ res,
                                     long long ldr, bf16* __restrict__ y, long long ldy, const bf16* __restrict__ w,
                                     float* __restrict__ rrms, int N, float eps, uint8_t* __restrict__ y8 = nullptr,
                                     long long ld8 = 0, float* __restrict__ y8_scale = nullptr) {
  // the norm weights are written by no kernel: fetch them while the producer of x is still running, and let the
  // consumer of y become resident (and fetch its own weights) as soon as this kernel's input is complete
  const int nv = N >> 3;
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  uint4 g[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = threadIdx.x + i * blockDim.x;
    g[i] = idx < nv ? __ldg(wr + idx) : make_uint4(0u, 0u, 0u, 0u);
  }
  pdl_wait();
  pdl_trigger();
  __shared__ float red[32];
  const int row = blockIdx.x;
  const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * ldx);
  uint4* rr4 = ADD ? reinterpret_cast<uint4*>(res + static_cast<size_t>(row) * ldr) : nullptr;
  float v[VPT][8];
  float sq = 0.0f;
  // all loads first: the stores into `res` below would otherwise order every later load of it behind them
  uint4 xa[VPT], xb[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = threadIdx.x + i * blockDim.x;
    xa[i] = idx < nv ? xr[idx] : make_uint4(0u, 0u, 0u, 0u);
    if (ADD) xb[i] = idx < nv ? rr4[idx] : make_uint4(0u, 0u, 0u, 0u);
  }
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = threadIdx.x + i * blockDim.x;
    if (idx < nv) {
      const uint32_t aw[4] = {xa[i].x, xa[i].y, xa[i].z, xa[i].w};
      if (ADD) {
        const uint32_t bw[4] = {xb[i].x, xb[i].y, xb[i].z, xb[i].w};
        uint32_t ow[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          // bf16 + bf16 rounded to bf16: the residual stream stays a bf16 tensor
          const float lo = bf16_round(bf16_lo(aw[e]) + bf16_lo(bw[e]));
          const float hi = bf16_round(bf16_hi(aw[e]) + bf16_hi(bw[e]));
          v[i][2 * e] = lo;
          v[i][2 * e + 1] = hi;
          ow[e] = pack_bf16x2(lo, hi);
        }
        rr4[idx] = make_uint4(ow[0], ow[1], ow[2], ow[3]);
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          v[i][2 * e] = bf16_lo(aw[e]);
          v[i][2 * e + 1] = bf16_hi(aw[e]);
        }
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) sq += v[i][e] * v[i][e];
    }
  }
  sq = block_sum(sq, red);
  const float rr = 1.0f / sqrtf(sq * (1.0f / static_cast<float>(N)) + eps);
  if (threadIdx.x == 0 && rrms) rrms[row] = rr;
  uint4* yr = reinterpret_cast<uint4*>(y + static_cast<size_t>(row) * ldy);
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = threadIdx.x + i * blockDim.x;
    if (idx < nv) {
      const uint32_t gw[4] = {g[i].x, g[i].y, g[i].z, g[i].w};
      uint32_t ow[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float lo = bf16_round(v[i][2 * e] * rr) * bf16_lo(gw[e]);
        const float hi = bf16_round(v[i][2 * e + 1] * rr) * bf16_hi(gw[e]);
        ow[e] = pack_bf16x2(lo, hi);
        // the bf16 values just stored, for the FP8 copy below
        v[i][2 * e] = bf16_lo(ow[e]);
        v[i][2 * e + 1] = bf16_hi(ow[e]);
        amax = fmaxf(amax, fmaxf(fabsf(v[i][2 * e]), fabsf(v[i][2 * e + 1])));
      }
      yr[idx] = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    }
  }
  if (y8) {
    amax = block_max(amax, red);
    const int p = split_scale_exponent(amax);
    const float s = ldexpf(1.0f, p);
    if (threadIdx.x == 0) y8_scale[row] = ldexpf(1.0f, -p);
    uint2* hr = reinterpret_cast<uint2*>(y8 + static_cast<size_t>(row) * ld8);
    uint2* lr = reinterpret_cast<uint2*>(y8 + (static_cast<size_t>(gridDim.x) + row) * ld8);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int idx = threadIdx.x + i * blockDim.x;
      if (idx < nv) {
        unsigned short h[4], l[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) split_e4m3_pair(v[i][2 * e] * s, v[i][2 * e + 1] * s, h[e], l[e]);
        hr[idx] = make_uint2(h[0] | (static_cast<uint32_t>(h[1]) << 16), h[2] | (static_cast<uint32_t>(h[3]) << 16));
        lr[idx] = make_uint2(l[0] | (static_cast<uint32_t>(l[1]) << 16), l[2] | (static_cast<uint32_t>(l[3]) << 16));
      }
    }
  }
  TRACE_END();
}

// Any N / alignment: scalar accesses, row re-read from L2 in the second phase.
template <bool ADD>
__global__ void rms_norm_bf16_scalar_kernel(const bf16* __restrict__ x, long long ldx, bf16* __restrict__ res,
                                            long long ldr, bf16* __restrict__ y, long long ldy, const bf16* __restrict__ w,
                                            float* __restrict__ rrms, int N, float eps) {
  pdl_wait();
  __shared__ float red[32];
  const int row = blockIdx.x;
  const bf16* xr = x + static_cast<size_t>(row) * ldx;
  bf16* rs = ADD ? res + static_cast<size_t>(row) * ldr : nullptr;
  float sq = 0.0f;
  for (int c = threadIdx.x; c < N; c += blockDim.x) {
    float h = __bfloat162float(xr[c]);
    if (ADD) {
      h = bf16_round(h + __bfloat162float(rs[c]));
      rs[c] = __float2bfloat16_rn(h);
    }
    sq += h * h;
  }
  sq = block_sum(sq, red);
  const float rr = 1.0f / sqrtf(sq * (1.0f / static_cast<float>(N)) + eps);
  if (threadIdx.x == 0 && rrms) rrms[row] = rr;
  bf16* yr = y + static_cast<size_t>(row) * ldy;
  for (int c = threadIdx.x; c < N; c += blockDim.x) {
    const float h = __bfloat162float(ADD ? rs[c] : xr[c]);
    yr[c] = __float2bfloat16_rn(bf16_round(h * rr) * __bfloat162float(w[c]));
  }
}

template <bool ADD>
int launch_rms_bf16(const bf16* x, long long ldx, bf16* res, long long ldr, bf16* y, long long ldy, const bf16* w, float* rrms,
                    int M, int N, float eps, cudaStream_t st, uint8_t* y8 = nullptr, long long ld8 = 0, float* y8_scale = nullptr) {
  if (!x || !y || !w || (ADD && !res) || M < 0 || N <= 0) return TEENY_ERR_BAD_ARG;
  if (y8 && (!y8_scale || (ld8 & 7) || ld8 < N || (reinterpret_cast<uintptr_t>(y8) & 7))) return TEENY_ERR_BAD_ARG;
  if (M == 0) return TEENY_OK;
  const bool vec = (N % 8 == 0) && (ldx % 8 == 0) && (ldy % 8 == 0) && aligned16(x) && aligned16(y) && aligned16(w) &&
                   (!ADD || (aligned16(res) && ldr % 8 == 0));
  const int nv = N / 8;
  if (vec && nv <= 8 * 256) {
    int threads = 128;
    if (nv <= 32) threads = 32;
    else if (nv <= 64) threads = 64;
    else if (nv > 4 * 128) threads = 256;
    // a few rows (decode): the kernel is one chain of latencies, so one vector per thread
    if (M <= 512 && nv > threads) threads = nv >= 512 ? 512 : (nv + 31) / 32 * 32;
    const int vpt = (nv + threads - 1) / threads;
#define TEENY_RMS_CASE(V)                                                                                    \
  launch_kernel(rms_norm_bf16_kernel<V, ADD>, dim3(M), dim3(threads), 0, st, 1, x, ldx, res, ldr, y, ldy, w, rrms, N, eps, y8, \
                ld8, y8_scale)
    if (vpt <= 1) TEENY_RMS_CASE(1);
    else if (vpt <= 2) TEENY_RMS_CASE(2);
    else if (vpt <= 4) TEENY_RMS_CASE(4);
    else TEENY_RMS_CASE(8);
#undef TEENY_RMS_CASE
  } else {
    if (y8) return TEENY_ERR_ALIGNMENT;  // the FP8 copy exists only in the vector kernel
    launch_kernel(rms_norm_bf16_scalar_kernel<ADD>, dim3(M), dim3(256), 0, st, 1, x, ldx, res, ldr, y, ldy, w, rrms, N, eps);
  }
  return static_cast<int>(cudaGetLastError());
}

// ---- tensor-parallel row-parallel epilogue: take every rank's pushed partial rows as they arrive, sum, add, normalise ----
// One CTA per token row (decode batches: a few dozen rows).  recv holds `world` copies of the projection as
// {f32 value, stamp} pairs, slot_elems elements apart; an element has arrived when its stamp equals this round's.
// A pair is one 64-bit word, written with one 64-bit store and read with one 64-bit load (st_stamped / ld_stamped,
// common.cuh): single-copy atomic, so a reader never sees a new stamp beside an old value.

// Bounded polling state of one thread: gives up `limit_ns` after its first unsuccessful poll, or as soon as another
// thread has reported an error.
struct PollState {
  uint64_t t0 = 0, limit_ns;
  int* err;
  bool live = true;
  __device__ PollState(int* e, uint64_t limit) : limit_ns(limit), err(e) {}
  __device__ __forceinline__ void tick(uint32_t it) {
    if ((it & 0x3f) != 0x3f) return;
    if (*reinterpret_cast<volatile int*>(err) != 0) { live = false; return; }
    const uint64_t now = global_timer_ns();
    if (t0 == 0) t0 = now;
    else if (now - t0 > limit_ns) { atomicCAS(err, 0, DEVERR_TP_GATHER); live = false; }
  }
};

// Eight consecutive stamped words from each of `nr` <= NR sources (src[r] + k), every request in flight together;
// words that do not carry `stamp` yet are asked for again until they do (or the poll state gives up).
template <int NR>
__device__ __forceinline__ void poll_words(const uint2* const (&src)[NR], int nr, unsigned stamp, unsigned long long (&q)[NR][8],
                                           PollState& ps) {
#pragma unroll
  for (int r = 0; r < NR; ++r)
#pragma unroll
    for (int k = 0; k < 8; k += 2) {  // 16-byte accesses, each 64-bit word of which is atomic on its own
      if (r < nr) ld_stamped_x2(src[r] + k, q[r][k], q[r][k + 1]);
      else q[r][k] = q[r][k + 1] = static_cast<unsigned long long>(stamp) << 32;
    }
  for (uint32_t it = 0;; ++it) {
    bool all = true;
#pragma unroll
    for (int r = 0; r < NR; ++r)
#pragma unroll
      for (int k = 0; k < 8; k += 2)
        if (static_cast<unsigned>(q[r][k] >> 32) != stamp || static_cast<unsigned>(q[r][k + 1] >> 32) != stamp) {
          ld_stamped_x2(src[r] + k, q[r][k], q[r][k + 1]);
          all = false;
        }
    if (all || !ps.live) break;
    ps.tick(it);
  }
}

// sum[e] += the `world` ranks' values of this thread's eight columns, in rank order (every rank adds in the same order,
// so all ranks hold identical results), four ranks' requests in flight at a time
__device__ __forceinline__ void gather_sum8(const uint2* recv, size_t slot_elems, int world, size_t elem, unsigned stamp,
                                            float (&sum)[8], PollState& ps) {
  for (int p0 = 0; p0 < world; p0 += 4) {
    const int nr = min(4, world - p0);
    const uint2* src[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) src[r] = recv + static_cast<size_t>(p0 + (r < nr ? r : 0)) * slot_elems + elem;
    unsigned long long q[4][8];
    poll_words<4>(src, nr, stamp, q, ps);
#pragma unroll
    for (int r = 0; r < 4; ++r)
      if (r < nr) {
#pragma unroll
        for (int k = 0; k < 8; ++k) sum[k] += __uint_as_float(static_cast<unsigned>(q[r][k]));
      }
  }
}

template <int VPT>
__global__ void __launch_bounds__(512) gather_add_rms_norm_kernel(const uint2* __restrict__ recv, size_t slot_elems, int world,
                                           const unsigned* __restrict__ epoch, unsigned round,
                                           bf16* __restrict__ res, long long ldr, bf16* __restrict__ y, long long ldy,
                                           const bf16* __restrict__ w, int N, float eps, int* err, uint64_t limit_ns) {
  const int nv = N >> 3;
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  uint4 g[VPT];  // norm weights: constant, fetched ahead of the wait
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = threadIdx.x + i * blockDim.x;
    g[i] = idx < nv ? __ldg(wr + idx) : make_uint4(0u, 0u, 0u, 0u);
  }
  // Nothing this kernel READS comes from its immediate predecessor in the stream (the GEMM that pushes) except the
  // pushed words themselves, and those carry their own stamps: the residual and the step counter were written by
  // kernels older than that, which are complete when this one starts.  So the partial sums are gathered BEFORE the
  // dependency wait -- while the GEMM's epilogue and the acknowledgement of its NVLink stores are still under way --
  // and only the writes come after it (so a later kernel that waits for this one still finds everything before it
  // complete).  The GEMM behind this kernel is let in at once: it fetches weights while this kernel waits for peers.
  pdl_trigger();
  __shared__ float red[32];
  const unsigned stamp = __ldcg(epoch) * 1024u + round + 1u;
  const int row = blockIdx.x;
  uint4* rr4 = reinterpret_cast<uint4*>(res + static_cast<size_t>(row) * ldr);
  float v[VPT][8];
  float sq = 0.0f;
  uint4 hb[VPT];  // the residual row as loaded; overwritten below with the new residual, stored after the wait
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = threadIdx.x + i * blockDim.x;
    hb[i] = idx < nv ? rr4[idx] : make_uint4(0u, 0u, 0u, 0u);
  }
  PollState ps(err, limit_ns);
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = threadIdx.x + i * blockDim.x;
    if (idx < nv) {
      float sum[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      gather_sum8(recv, slot_elems, world, static_cast<size_t>(row) * N + 8 * static_cast<size_t>(idx), stamp, sum, ps);
      const uint32_t hw[4] = {hb[i].x, hb[i].y, hb[i].z, hb[i].w};
      uint32_t ow[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float lo = bf16_round(bf16_lo(hw[e]) + bf16_round(sum[2 * e]));      // projection is a bf16 tensor
        const float hi = bf16_round(bf16_hi(hw[e]) + bf16_round(sum[2 * e + 1]));
        v[i][2 * e] = lo;
        v[i][2 * e + 1] = hi;
        ow[e] = pack_bf16x2(lo, hi);
      }
      hb[i] = make_uint4(ow[0], ow[1], ow[2], ow[3]);
#pragma unroll
      for (int e = 0; e < 8; ++e) sq += v[i][e] * v[i][e];
    }
  }
  sq = block_sum(sq, red);
  const float rr = 1.0f / sqrtf(sq * (1.0f / static_cast<float>(N)) + eps);
  uint4* yr = reinterpret_cast<uint4*>(y + static_cast<size_t>(row) * ldy);
  pdl_wait();
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = threadIdx.x + i * blockDim.x;
    if (idx < nv) {
      rr4[idx] = hb[i];
      const uint32_t gw[4] = {g[i].x, g[i].y, g[i].z, g[i].w};
      uint32_t ow[4];
#pragma unroll
      for (int e = 0; e < 4; ++e)
        ow[e] = pack_bf16x2(bf16_round(v[i][2 * e] * rr) * bf16_lo(gw[e]), bf16_round(v[i][2 * e + 1] * rr) * bf16_hi(gw[e]));
      yr[idx] = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    }
  }
}

// ---- the same epilogue in two hops, for wider tensor parallelism ----
// Pushing every rank's partial rows to every rank costs world x the tensor per rank.  Here token row r has one owner
// (rank r / owner_rows): the GEMMs push row r only to its owner; the owner's CTA sums the world partials, adds the
// residual, normalises, keeps the new residual and the normed row and stores both, stamped, into every other rank's
// broadcast buffer; every other rank's CTA for row r waits for that row and unpacks it.  Traffic per rank is about
// twice the tensor instead of world times it, for one more NVLink latency.
// bcast[p]: rank p's broadcast buffer (this rank's own entry = local); a row is N words of
// {bf16 pair, stamp}: per two columns one word with the residual pair, then one with the normed pair.
template <int VPT>
__global__ void __launch_bounds__(512) gather_add_rms_norm_owner_kernel(const uint2* __restrict__ recv, size_t slot_elems, int world, int rank,
                                                 int owner_rows, uint4* const* __restrict__ bcast,
                                                 const unsigned* __restrict__ epoch, unsigned round,
                                                 bf16* __restrict__ res, long long ldr, bf16* __restrict__ y,
                                                 long long ldy, const bf16* __restrict__ w, int N, float eps, int* err,
                                                 uint64_t limit_ns) {
  const int nv = N >> 3;
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  uint4 g[VPT];  // norm weights: constant, fetched ahead of the wait
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = threadIdx.x + i * blockDim.x;
    g[i] = idx < nv ? __ldg(wr + idx) : make_uint4(0u, 0u, 0u, 0u);
  }
  // as in gather_add_rms_norm_kernel: gather (and, for a row owned elsewhere, the wait for its broadcast) before the
  // dependency wait, local writes after it; the stores into OTHER ranks' broadcast buffers need no such order
  pdl_trigger();
  __shared__ float red[32];
  const unsigned stamp = __ldcg(epoch) * 1024u + round + 1u;
  const int row = blockIdx.x;
  const int owner = row / owner_rows;
  uint4* rr4 = reinterpret_cast<uint4*>(res + static_cast<size_t>(row) * ldr);
  uint4* yr = reinterpret_cast<uint4*>(y + static_cast<size_t>(row) * ldy);
  const size_t brow = static_cast<size_t>(row) * (N >> 1);  // 16-byte lines per row in a broadcast buffer
  PollState ps(err, limit_ns);
  if (owner != rank) {
    // this row is reduced elsewhere: take the finished residual and normed row from the owner's broadcast
    const uint2* src0 = reinterpret_cast<const uint2*>(bcast[rank] + brow);
    uint4 got_r[VPT], got_y[VPT];
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int idx = threadIdx.x + i * blockDim.x;
      if (idx < nv) {
        const uint2* src[1] = {src0 + 8 * idx};
        unsigned long long q[1][8];
        poll_words<1>(src, 1, stamp, q, ps);
        got_r[i] = make_uint4(static_cast<unsigned>(q[0][0]), static_cast<unsigned>(q[0][2]), static_cast<unsigned>(q[0][4]),
                              static_cast<unsigned>(q[0][6]));
        got_y[i] = make_uint4(static_cast<unsigned>(q[0][1]), static_cast<unsigned>(q[0][3]), static_cast<unsigned>(q[0][5]),
                              static_cast<unsigned>(q[0][7]));
      }
    }
    TRACE_MARK(3, threadIdx.x == 0);  // a row owned elsewhere: its broadcast has arrived
    pdl_wait();
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int idx = threadIdx.x + i * blockDim.x;
      if (idx < nv) {
        rr4[idx] = got_r[i];
        yr[idx] = got_y[i];
      }
    }
    TRACE_END();
    return;
  }
  float v[VPT][8];
  float sq = 0.0f;
  uint32_t hp[VPT][4];
  uint4 hb[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = threadIdx.x + i * blockDim.x;
    hb[i] = idx < nv ? rr4[idx] : make_uint4(0u, 0u, 0u, 0u);
  }
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = threadIdx.x + i * blockDim.x;
    if (idx < nv) {
      float sum[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      // rank order: the one owner's result is what every rank gets
      gather_sum8(recv, slot_elems, world, static_cast<size_t>(row) * N + 8 * static_cast<size_t>(idx), stamp, sum, ps);
      const uint32_t hw[4] = {hb[i].x, hb[i].y, hb[i].z, hb[i].w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float lo = bf16_round(bf16_lo(hw[e]) + bf16_round(sum[2 * e]));      // projection is a bf16 tensor
        const float hi = bf16_round(bf16_hi(hw[e]) + bf16_round(sum[2 * e + 1]));
        v[i][2 * e] = lo;
        v[i][2 * e + 1] = hi;
        hp[i][e] = pack_bf16x2(lo, hi);
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) sq += v[i][e] * v[i][e];
    }
  }
  TRACE_MARK(1, threadIdx.x == 0);  // an owned row: every rank's partial has arrived
  sq = block_sum(sq, red);
  const float rr = 1.0f / sqrtf(sq * (1.0f / static_cast<float>(N)) + eps);
  uint32_t yw[VPT][4];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = threadIdx.x + i * blockDim.x;
    if (idx < nv) {
      const uint32_t gw[4] = {g[i].x, g[i].y, g[i].z, g[i].w};
      uint32_t ow[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        ow[e] = pack_bf16x2(bf16_round(v[i][2 * e] * rr) * bf16_lo(gw[e]), bf16_round(v[i][2 * e + 1] * rr) * bf16_hi(gw[e]));
        yw[i][e] = ow[e];
      }
      for (int p = 0; p < world; ++p) {  // NVLink stores to the other ranks: 16 bytes = {residual pair, stamp}, {normed pair, stamp}
        if (p == rank) continue;
        uint2* dst = reinterpret_cast<uint2*>(bcast[p] + brow) + 8 * idx;
#pragma unroll
        for (int e = 0; e < 4; ++e) st_stamped_x2(dst + 2 * e, hp[i][e], ow[e], stamp);
      }
    }
  }
  TRACE_MARK(2, threadIdx.x == 0);  // ... and its broadcast is on its way
  pdl_wait();
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = threadIdx.x + i * blockDim.x;
    if (idx < nv) {
      rr4[idx] = make_uint4(hp[i][0], hp[i][1], hp[i][2], hp[i][3]);
      yr[idx] = make_uint4(yw[i][0], yw[i][1], yw[i][2], yw[i][3]);
    }
  }
  TRACE_END();
}

// ---- SiLU(gate) * up on the fused [T, 2*inter] projection ----
__global__ void silu_mul_bf16_kernel(const bf16* __restrict__ gu, long long ld, bf16* __restrict__ out, int T,
                                     int inter) {
  pdl_wait();
  const int vec_per_row = inter >> 3;
  const long long total = static_cast<long long>(T) * vec_per_row;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const long long t = i / vec_per_row;
    const int c = static_cast<int>(i - t * vec_per_row) * 8;
    const uint4 g = *reinterpret_cast<const uint4*>(gu + t * ld + c);
    const uint4 u = *reinterpret_cast<const uint4*>(gu + t * ld + inter + c);
    const uint32_t gw[4] = {g.x, g.y, g.z, g.w}, uw[4] = {u.x, u.y, u.z, u.w};
    uint32_t ow[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float lo = bf16_round(silu_f(bf16_lo(gw[e]))) * bf16_lo(uw[e]);
      const float hi = bf16_round(silu_f(bf16_hi(gw[e]))) * bf16_hi(uw[e]);
      ow[e] = pack_bf16x2(lo, hi);
    }
    *reinterpret_cast<uint4*>(out + t * inter + c) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
  }
}
__global__ void silu_mul_bf16_scalar_kernel(const bf16* __restrict__ gu, long long ld, bf16* __restrict__ out, int T,
                                            int inter) {
  pdl_wait();
  const long long total = static_cast<long long>(T) * inter;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const long long t = i / inter;
    const int c = static_cast<int>(i - t * inter);
    const float g = __bfloat162float(gu[t * ld + c]), u = __bfloat162float(gu[t * ld + inter + c]);
    out[t * inter + c] = __float2bfloat16_rn(bf16_round(silu_f(g)) * u);
  }
}

// ---- embedding gather: one warp per 16-byte vector strip ----
__global__ void embedding_bf16_kernel(const int* __restrict__ ids, const bf16* __restrict__ table,
                                      bf16* __restrict__ out, int T, int hidden, int vocab, bool vec) {
  pdl_wait();
  const int row = blockIdx.x;
  if (row >= T) return;
  int id = ids[row];
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);  // ids are validated on the host; clamp keeps loads in range
  const bf16* src = table + static_cast<size_t>(id) * hidden;
  bf16* dst = out + static_cast<size_t>(row) * hidden;
  if (vec) {
    for (int c = threadIdx.x; c < (hidden >> 3); c += blockDim.x)
      reinterpret_cast<uint4*>(dst)[c] = reinterpret_cast<const uint4*>(src)[c];
  } else {
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) dst[c] = src[c];
  }
}

// ---- RoPE tables ----
__global__ void rope_table_kernel(const float* __restrict__ inv_freq, bf16* __restrict__ cos_t,
                                  bf16* __restrict__ sin_t, int max_pos, int D) {
  pdl_wait();
  const int half = D >> 1;
  const long long total = static_cast<long long>(max_pos) * half;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int pos = static_cast<int>(i / half), j = static_cast<int>(i % half);
    const float angle = inv_freq[j] * static_cast<float>(pos);  // f32 product, as the traced graph computes it
    // cos/sin of the f32 angle evaluated in double and rounded once: stays within half an ulp of the f32 result
    const bf16 c = __float2bfloat16_rn(static_cast<float>(cos(static_cast<double>(angle))));
    const bf16 s = __float2bfloat16_rn(static_cast<float>(sin(static_cast<double>(angle))));
    cos_t[static_cast<size_t>(pos) * D + j] = c;
    cos_t[static_cast<size_t>(pos) * D + half + j] = c;
    sin_t[static_cast<size_t>(pos) * D + j] = s;
    sin_t[static_cast<size_t>(pos) * D + half + j] = s;
  }
}

// ---- per-head RMSNorm + RoPE + KV-cache append; D == 128, one half-warp per (token, head) ----
// Lane s (0..15) of the half-warp holds elements [8s, 8s+8) as one 16-byte vector; its rotate-half partner elements
// (d +- 64) live in lane s ^ 8.  V heads are copied into the cache unchanged.  A half-warp takes kRopeUnits
// consecutive (token, head) units and issues all their loads before it computes, so a short-lived CTA still keeps
// enough bytes in flight.
constexpr int kRopeUnits = 4;

__global__ void qk_norm_rope_kv_kernel(bf16* __restrict__ qkv, long long ld, const bf16* __restrict__ q_w,
                                       const bf16* __restrict__ k_w, const bf16* __restrict__ cos_t,
                                       const bf16* __restrict__ sin_t, bf16* __restrict__ k_cache,
                                       bf16* __restrict__ v_cache, int T, int S, int Hq, int Hkv, int max_len,
                                       int pos0, const int* __restrict__ pos0_dev, float eps) {
  constexpr int D = 128;
  const int heads = Hq + 2 * Hkv;
  const long long total = static_cast<long long>(T) * heads;
  const long long unit0 = ((static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 4) * kRopeUnits;
  const int sub = threadIdx.x & 15;
  // head-norm weights are constants: fetched ahead of the wait for the projection
  const uint4 wq = __ldg(reinterpret_cast<const uint4*>(q_w + sub * 8));
  const uint4 wk = __ldg(reinterpret_cast<const uint4*>(k_w + sub * 8));
  pdl_wait();
  pdl_trigger();
  const int base_pos = pos0_dev ? *pos0_dev : pos0;
  uint4 raw[kRopeUnits], craw[kRopeUnits], sraw[kRopeUnits];
  int tok[kRopeUnits], head[kRopeUnits], pos[kRopeUnits], bidx[kRopeUnits];
  bool valid[kRopeUnits];
  // one division for the first unit; the following units step through heads and tokens
  const long long first = unit0 < total ? unit0 : total - 1;  // units past the end shadow the last one (no stores)
  int t_cur = static_cast<int>(first / heads);
  int h_cur = static_cast<int>(first - static_cast<long long>(t_cur) * heads);
  int b_cur = t_cur / S;
  int s_cur = t_cur - b_cur * S;
#pragma unroll
  for (int u = 0; u < kRopeUnits; ++u) {
    valid[u] = unit0 + u < total;
    tok[u] = t_cur;
    head[u] = h_cur;
    bidx[u] = b_cur;
    pos[u] = base_pos + s_cur;
    const int tp = pos[u] < max_len ? pos[u] : max_len - 1;  // table has max_len rows
    raw[u] = *reinterpret_cast<const uint4*>(qkv + static_cast<size_t>(t_cur) * ld + static_cast<size_t>(h_cur) * D + sub * 8);
    craw[u] = __ldg(reinterpret_cast<const uint4*>(cos_t + static_cast<size_t>(tp) * D + sub * 8));
    sraw[u] = __ldg(reinterpret_cast<const uint4*>(sin_t + static_cast<size_t>(tp) * D + sub * 8));
    if (unit0 + u + 1 < total) {  // advance (stays on the last unit at the end)
      if (++h_cur == heads) {
        h_cur = 0;
        ++t_cur;
        if (++s_cur == S) { s_cur = 0; ++b_cur; }
      }
    }
  }
#pragma unroll
  for (int u = 0; u < kRopeUnits; ++u) {
    const int h = head[u];
    const bool is_v = h >= Hq + Hkv, is_q = h < Hq;
    const uint4 outv = head_norm_rope(raw[u], is_q ? wq : wk, craw[u], sraw[u], sub, eps);
    if (!valid[u]) continue;
    if (is_q) {
      *reinterpret_cast<uint4*>(qkv + static_cast<size_t>(tok[u]) * ld + static_cast<size_t>(h) * D + sub * 8) = outv;
    } else if (pos[u] < max_len) {
      bf16* cache = is_v ? v_cache : k_cache;
      const int hh = is_v ? h - Hq - Hkv : h - Hq;
      bf16* dst = cache + ((static_cast<size_t>(bidx[u]) * Hkv + hh) * max_len + pos[u]) * D + sub * 8;
      *reinterpret_cast<uint4*>(dst) = is_v ? raw[u] : outv;
    }
  }
}

// ---- softmax rows (f32 math) ----
template <typename T>
__device__ __forceinline__ float ldf(const T* p);
template <> __device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldf<bf16>(const bf16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void stf(float* p, float v) { *p = v; }
__device__ __forceinline__ void stf(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

template <typename T>
__global__ void softmax_kernel(const T* __restrict__ x, T* __restrict__ y, int cols) {
  pdl_wait();
  __shared__ float red[32];
  const T* xr = x + static_cast<size_t>(blockIdx.x) * cols;
  T* yr = y + static_cast<size_t>(blockIdx.x) * cols;
  float mx = -INFINITY;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) mx = fmaxf(mx, ldf(xr + c));
  mx = warp_max(mx);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (lane == 0) red[warp] = mx;
  __syncthreads();
  mx = warp_max(lane < nw ? red[lane] : -INFINITY);
  __syncthreads();
  float sum = 0.0f;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) sum += expf(ldf(xr + c) - mx);
  sum = block_sum(sum, red);
  for (int c = threadIdx.x; c < cols; c += blockDim.x) stf(yr + c, expf(ldf(xr + c) - mx) / sum);
}

// ---- argmax over the last dim (lowest index wins ties) ----
__device__ __forceinline__ void argmax_merge(float& v, int& i, float ov, int oi) {
  if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
}
__global__ void argmax_bf16_kernel(const bf16* __restrict__ logits, long long ld, float* __restrict__ best_val,
                                   int* __restrict__ best_idx, int cols, int idx_offset, bool vec) {
  pdl_wait();
  __shared__ float sv[32];
  __shared__ int si[32];
  const bf16* row = logits + static_cast<size_t>(blockIdx.x) * ld;
  float v = -INFINITY;
  int idx = 0x7fffffff;
  if (vec) {
    for (int c = threadIdx.x; c < (cols >> 3); c += blockDim.x) {
      const uint4 a = reinterpret_cast<const uint4*>(row)[c];
      const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        argmax_merge(v, idx, bf16_lo(aw[e]), c * 8 + 2 * e);
        argmax_merge(v, idx, bf16_hi(aw[e]), c * 8 + 2 * e + 1);
      }
    }
    for (int c = (cols & ~7) + threadIdx.x; c < cols; c += blockDim.x) argmax_merge(v, idx, __bfloat162float(row[c]), c);
  } else {
    for (int c = threadIdx.x; c < cols; c += blockDim.x) argmax_merge(v, idx, __bfloat162float(row[c]), c);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    argmax_merge(v, idx, ov, oi);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (lane == 0) { sv[warp] = v; si[warp] = idx; }
  __syncthreads();
  if (warp == 0) {
    v = lane < nw ? sv[lane] : -INFINITY;
    idx = lane < nw ? si[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, v, o);
      const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
      argmax_merge(v, idx, ov, oi);
    }
    if (lane == 0) {
      best_val[blockIdx.x] = v;
      best_idx[blockIdx.x] = idx + idx_offset;
    }
  }
}
__global__ void argmax_combine_kernel(const float* __restrict__ vals, const int* __restrict__ idx,
                                      int* __restrict__ out_idx, int parts, int rows) {
  pdl_wait();
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  float v = -INFINITY;
  int i = 0x7fffffff;
  for (int p = 0; p < parts; ++p) argmax_merge(v, i, vals[static_cast<size_t>(p) * rows + r], idx[static_cast<size_t>(p) * rows + r]);
  out_idx[r] = i;
}

}  // namespace

int rms_norm_f32(const float* x, float* y, const float* w, float* rrms, int M, int N, float eps, cudaStream_t st) {
  if (!x || !y || !w || M < 0 || N <= 0) return TEENY_ERR_BAD_ARG;
  if (M == 0) return TEENY_OK;
  launch_kernel(rms_norm_f32_kernel, dim3(M), dim3(128), 0, st, 1, x, y, w, rrms, N, eps);
  return static_cast<int>(cudaGetLastError());
}
int rms_norm_bf16(const bf16* x, long long ldx, bf16* y, long long ldy, const bf16* w, float* rrms, int M, int N,
                  float eps, cudaStream_t st, uint8_t* y8, long long ld8, float* y8_scale) {
  return launch_rms_bf16<false>(x, ldx, nullptr, 0, y, ldy, w, rrms, M, N, eps, st, y8, ld8, y8_scale);
}
int add_rms_norm_bf16(const bf16* x, long long ldx, bf16* residual, long long ldr, bf16* y, long long ldy,
                      const bf16* w, int M, int N, float eps, cudaStream_t st, uint8_t* y8, long long ld8, float* y8_scale) {
  return launch_rms_bf16<true>(x, ldx, residual, ldr, y, ldy, w, nullptr, M, N, eps, st, y8, ld8, y8_scale);
}
int gather_add_rms_norm_bf16(const uint2* recv, size_t slot_elems, int world, const unsigned* epoch, unsigned round,
                             bf16* residual, long long ldr, bf16* y, long long ldy, const bf16* w, int M, int N,
                             float eps, cudaStream_t st, unsigned long long wait_limit_ns) {
  const uint64_t limit = wait_limit_ns ? wait_limit_ns : kWaitLimitNs;
  if (!recv || !epoch || !residual || !y || !w || world < 2 || M <= 0 || N <= 0 || round >= 1023) return TEENY_ERR_BAD_ARG;
  if (N % 8 || ldr % 8 || ldy % 8 || N > 8 * 4 * 512) return TEENY_ERR_BAD_ARG;
  if (!aligned16(recv) || !aligned16(residual) || !aligned16(y) || !aligned16(w) || (slot_elems % 2)) return TEENY_ERR_ALIGNMENT;
  const int nv = N / 8;
  const int threads = nv >= 512 ? 512 : (nv + 31) / 32 * 32, vpt = (nv + threads - 1) / threads;
  int* err = device_error_word();
  if (!err) return TEENY_ERR_DRIVER;
#define TEENY_GATHER_CASE(V)                                                                                       \
  launch_kernel(gather_add_rms_norm_kernel<V>, dim3(M), dim3(threads), 0, st, 1, recv, slot_elems, world, epoch, round, \
                residual, ldr, y, ldy, w, N, eps, err, limit)
  if (vpt <= 1) TEENY_GATHER_CASE(1);
  else if (vpt <= 2) TEENY_GATHER_CASE(2);
  else TEENY_GATHER_CASE(4);
#undef TEENY_GATHER_CASE
  return static_cast<int>(cudaGetLastError());
}
int gather_add_rms_norm_owner_bf16(const uint2* recv, size_t slot_elems, int world, int rank, int owner_rows,
                                   uint4* const* bcast, const unsigned* epoch, unsigned round, bf16* residual,
                                   long long ldr, bf16* y, long long ldy, const bf16* w, int M, int N, float eps,
                                   cudaStream_t st, unsigned long long wait_limit_ns) {
  const uint64_t limit = wait_limit_ns ? wait_limit_ns : kWaitLimitNs;
  if (!recv || !bcast || !epoch || !residual || !y || !w || world < 2 || rank < 0 || rank >= world || owner_rows <= 0 ||
      M <= 0 || M > owner_rows * world || N <= 0 || round >= 1023)
    return TEENY_ERR_BAD_ARG;
  if (N % 8 || ldr % 8 || ldy % 8 || N > 8 * 4 * 512) return TEENY_ERR_BAD_ARG;
  if (!aligned16(recv) || !aligned16(residual) || !aligned16(y) || !aligned16(w) || (slot_elems % 2)) return TEENY_ERR_ALIGNMENT;
  const int nv = N / 8;
  const int threads = nv >= 512 ? 512 : (nv + 31) / 32 * 32, vpt = (nv + threads - 1) / threads;
  int* err = device_error_word();
  if (!err) return TEENY_ERR_DRIVER;
#define TEENY_GATHER_CASE(V)                                                                                          \
  launch_kernel(gather_add_rms_norm_owner_kernel<V>, dim3(M), dim3(threads), 0, st, 1, recv, slot_elems, world, rank, \
                owner_rows, bcast, epoch, round, residual, ldr, y, ldy, w, N, eps, err, limit)
  if (vpt <= 1) TEENY_GATHER_CASE(1);
  else if (vpt <= 2) TEENY_GATHER_CASE(2);
  else TEENY_GATHER_CASE(4);
#undef TEENY_GATHER_CASE
  return static_cast<int>(cudaGetLastError());
}
int silu_f32(const float* x, float* y, long long n, cudaStream_t st) { return launch_ew_f32<OpSilu, false>(x, nullptr, y, n, st); }
int silu_bf16(const bf16* x, bf16* y, long long n, cudaStream_t st) { return launch_ew_bf16<OpSilu, false>(x, nullptr, y, n, st); }
int mul_f32(const float* a, const float* b, float* o, long long n, cudaStream_t st) { return launch_ew_f32<OpMul, true>(a, b, o, n, st); }
int mul_bf16(const bf16* a, const bf16* b, bf16* o, long long n, cudaStream_t st) { return launch_ew_bf16<OpMul, true>(a, b, o, n, st); }
int add_f32(const float* a, const float* b, float* o, long long n, cudaStream_t st) { return launch_ew_f32<OpAdd, true>(a, b, o, n, st); }
int add_bf16(const bf16* a, const bf16* b, bf16* o, long long n, cudaStream_t st) { return launch_ew_bf16<OpAdd, true>(a, b, o, n, st); }

int softmax_f32(const float* x, float* y, int rows, int cols, cudaStream_t st) {
  if (!x || !y || rows < 0 || cols <= 0) return TEENY_ERR_BAD_ARG;
  if (rows == 0) return TEENY_OK;
  launch_kernel(softmax_kernel<float>, dim3(rows), dim3(cols >= 1024 ? 256 : 128), 0, st, 1, x, y, cols);
  return static_cast<int>(cudaGetLastError());
}
int softmax_bf16(const bf16* x, bf16* y, int rows, int cols, cudaStream_t st) {
  if (!x || !y || rows < 0 || cols <= 0) return TEENY_ERR_BAD_ARG;
  if (rows == 0) return TEENY_OK;
  launch_kernel(softmax_kernel<bf16>, dim3(rows), dim3(cols >= 1024 ? 256 : 128), 0, st, 1, x, y, cols);
  return static_cast<int>(cudaGetLastError());
}

int silu_mul_bf16(const bf16* gate_up, long long ld, bf16* out, int T, int inter, cudaStream_t st) {
  if (!gate_up || !out || T < 0 || inter <= 0) return TEENY_ERR_BAD_ARG;
  if (T == 0) return TEENY_OK;
  const bool vec = (inter % 8 == 0) && (ld % 8 == 0) && aligned16(gate_up) && aligned16(out);
  if (vec)
    launch_kernel(silu_mul_bf16_kernel, dim3(ew_grid(static_cast<long long>(T) * (inter / 8), kEwThreads)), dim3(kEwThreads), 0, st, 1, gate_up, ld, out, T, inter);
  else
    launch_kernel(silu_mul_bf16_scalar_kernel, dim3(ew_grid(static_cast<long long>(T) * inter, kEwThreads)), dim3(kEwThreads), 0, st, 1, gate_up, ld, out, T, inter);
  return static_cast<int>(cudaGetLastError());
}

int embedding_bf16(const int* ids, const bf16* table, bf16* out, int T, int hidden, int vocab, cudaStream_t st) {
  if (!ids || !table || !out || T < 0 || hidden <= 0 || vocab <= 0) return TEENY_ERR_BAD_ARG;
  if (T == 0) return TEENY_OK;
  const bool vec = (hidden % 8 == 0) && aligned16(table) && aligned16(out);
  launch_kernel(embedding_bf16_kernel, dim3(T), dim3(128), 0, st, 1, ids, table, out, T, hidden, vocab, vec);
  return static_cast<int>(cudaGetLastError());
}

int rope_table_bf16(const float* inv_freq, bf16* cos_t, bf16* sin_t, int max_pos, int D, cudaStream_t st) {
  if (!inv_freq || !cos_t || !sin_t || max_pos <= 0 || D <= 0 || (D & 1)) return TEENY_ERR_BAD_ARG;
  launch_kernel(rope_table_kernel, dim3(ew_grid(static_cast<long long>(max_pos) * (D / 2), kEwThreads)), dim3(kEwThreads), 0, st, 1, inv_freq, cos_t, sin_t, max_pos, D);
  return static_cast<int>(cudaGetLastError());
}

int qk_norm_rope_kv_bf16(bf16* qkv, long long ld, const bf16* q_w, const bf16* k_w, const bf16* cos_t,
                         const bf16* sin_t, bf16* k_cache, bf16* v_cache, int T, int S, int Hq, int Hkv, int D,
                         int max_len, int pos0, const int* pos0_dev, float eps, cudaStream_t st) {
  if (!qkv || !q_w || !k_w || !cos_t || !sin_t || !k_cache || !v_cache || T < 0 || S <= 0 || Hq <= 0 || Hkv <= 0 ||
      max_len <= 0)
    return TEENY_ERR_BAD_ARG;
  if (D != 128) return TEENY_ERR_BAD_ARG;  // head_dim of every Qwen3 size
  if ((ld % 8) || (reinterpret_cast<uintptr_t>(qkv) & 15) || (reinterpret_cast<uintptr_t>(k_cache) & 15) ||
      (reinterpret_cast<uintptr_t>(v_cache) & 15) || (reinterpret_cast<uintptr_t>(q_w) & 15) ||
      (reinterpret_cast<uintptr_t>(k_w) & 15))
    return TEENY_ERR_ALIGNMENT;
  if (T == 0) return TEENY_OK;
  const long long units = static_cast<long long>(T) * (Hq + 2 * Hkv);  // kRopeUnits per half-warp, 16 half-warps per CTA
  const long long blocks = (units + 16 * kRopeUnits - 1) / (16 * kRopeUnits);
  if (blocks > 0x7fffffffLL) return TEENY_ERR_BAD_ARG;
  launch_kernel(qk_norm_rope_kv_kernel, dim3(static_cast<int>(blocks)), dim3(256), 0, st, 1, qkv, ld, q_w, k_w, cos_t, sin_t, k_cache, v_cache,
                                                                   T, S, Hq, Hkv, max_len, pos0, pos0_dev, eps);
  return static_cast<int>(cudaGetLastError());
}

int argmax_bf16(const bf16* logits, long long ld, float* best_val, int* best_idx, int rows, int cols, int idx_offset,
                cudaStream_t st) {
  if (!logits || !best_val || !best_idx || rows < 0 || cols <= 0) return TEENY_ERR_BAD_ARG;
  if (rows == 0) return TEENY_OK;
  const bool vec = aligned16(logits) && (ld % 8 == 0);
  launch_kernel(argmax_bf16_kernel, dim3(rows), dim3(1024), 0, st, 1, logits, ld, best_val, best_idx, cols, idx_offset, vec);
  return static_cast<int>(cudaGetLastError());
}
int argmax_combine(const float* vals, const int* idx, int* out_idx, int parts, int rows, cudaStream_t st) {
  if (!vals || !idx || !out_idx || parts <= 0 || rows < 0) return TEENY_ERR_BAD_ARG;
  if (rows == 0) return TEENY_OK;
  launch_kernel(argmax_combine_kernel, dim3((rows + 127) / 128), dim3(128), 0, st, 1, vals, idx, out_idx, parts, rows);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace teeny
