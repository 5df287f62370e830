// Weight-only FP8 linear: Y[M, N] = X[M, K] (bf16) * W^T with W stored as OCP FP8 E4M3 bytes plus f32 scales, the
// "float-quantized" compressed-tensors layout the reference's quantiser writes
// (utilities/teeny-quant/src/format.rs:215-240: `foo.weight` as F8_E4M3 in the weight's own shape, `foo.weight_scale`
// as a flat F32 vector with one scale per group; groups per utilities/teeny-quant/src/quant/groups.rs:84-110; decode
// per utilities/teeny-quant/src/quant/fp8.rs:175-206: value = f8_to_f32(byte) * scale[group]).
//
// Decode-shaped calls (M <= 128) stream the bytes as they are -- half the HBM traffic of bf16 weights -- and convert
// them on the way into the tensor core (gemm_bf16_skinny_kernel's W8 variant, gemm_bf16.cu).  Larger M is compute
// bound: the weight is converted once into a bf16 scratch matrix and the ordinary bf16 GEMM runs on that.
#include "common.cuh"
#include "kernels.h"

namespace teeny {

namespace {

// One E4M3 byte as f32, every encoding (subnormals included; 0x7f / 0xff are NaN).
__device__ __forceinline__ float e4m3_to_f32(uint32_t b) {
  const uint32_t mag = b & 0x7fu;
  // magnitude bits placed at the top of an f32's exponent/mantissa give 2^-120 times the value (subnormals land on
  // f32 normals or subnormals of the same spacing), so one exact multiplication finishes it
  float v = __uint_as_float(mag << 20) * 0x1p120f;
  if (mag == 0x7fu) v = __uint_as_float(0x7fc00000u);
  return (b & 0x80u) ? -v : v;
}

// 16 bytes of one weight row per thread -> 16 bf16 = bf16_rn(value * scale of the element's group)
__global__ void __launch_bounds__(256)
dequant_e4m3_bf16_kernel(const uint8_t* __restrict__ wq, long long ldw, const float* __restrict__ scale, int kind, int group,
                         bf16* __restrict__ out, long long ldo, int N, int K) {
  pdl_wait();
  pdl_trigger();
  const int pieces = (K + 15) / 16;
  const long long total = static_cast<long long>(N) * pieces;
  const int groups_per_row = kind == 2 ? (K + group - 1) / group : 0;
  for (long long p = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; p < total;
       p += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int n = static_cast<int>(p / pieces), k0 = static_cast<int>(p % pieces) * 16;
    const uint8_t* src = wq + n * ldw + k0;
    bf16* dst = out + n * ldo + k0;
    float s = kind == 0 ? __ldg(scale) : (kind == 1 ? __ldg(scale + n) : 0.0f);
    if (k0 + 16 <= K) {
      const uint4 w = __ldg(reinterpret_cast<const uint4*>(src));
      const uint32_t words[4] = {w.x, w.y, w.z, w.w};
      uint32_t o[8];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        float v[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          if (kind == 2) s = __ldg(scale + static_cast<size_t>(n) * groups_per_row + (k0 + 4 * q + e) / group);
          v[e] = e4m3_to_f32((words[q] >> (8 * e)) & 0xffu) * s;
        }
        o[2 * q] = pack_bf16x2(v[0], v[1]);
        o[2 * q + 1] = pack_bf16x2(v[2], v[3]);
      }
      reinterpret_cast<uint4*>(dst)[0] = make_uint4(o[0], o[1], o[2], o[3]);
      reinterpret_cast<uint4*>(dst)[1] = make_uint4(o[4], o[5], o[6], o[7]);
    } else {
      for (int e = 0; k0 + e < K; ++e) {
        if (kind == 2) s = __ldg(scale + static_cast<size_t>(n) * groups_per_row + (k0 + e) / group);
        dst[e] = __float2bfloat16_rn(e4m3_to_f32(src[e]) * s);
      }
    }
  }
}

// Integer schemes (utilities/teeny-quant/src/quant/affine.rs:151-161): value = (q - zero point) * scale, q an int8 or a
// sign-extended nibble (two per byte over the flattened tensor, the first in the low nibble, pack4.rs:31-40).  One
// thread per 8 consecutive k of a row.
__global__ void __launch_bounds__(256)
dequant_int_bf16_kernel(const uint8_t* __restrict__ q, int bits, const float* __restrict__ scale,
                        const int* __restrict__ zero_point, int kind, int group, bf16* __restrict__ out, long long ldo,
                        int N, int K) {
  const int pieces = (K + 7) / 8;
  const long long total = static_cast<long long>(N) * pieces;
  const int groups_per_row = kind == 2 ? (K + group - 1) / group : 0;
  for (long long p = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; p < total;
       p += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int n = static_cast<int>(p / pieces), k0 = static_cast<int>(p % pieces) * 8;
    for (int e = 0; e < 8 && k0 + e < K; ++e) {
      const int k = k0 + e;
      const long long i = static_cast<long long>(n) * K + k;
      int v;
      if (bits == 8) {
        v = static_cast<int8_t>(q[i]);
      } else {
        const int nib = (q[i >> 1] >> ((i & 1) * 4)) & 0xf;
        v = nib >= 8 ? nib - 16 : nib;
      }
      const size_t g = kind == 0 ? 0 : (kind == 1 ? static_cast<size_t>(n) : static_cast<size_t>(n) * groups_per_row + k / group);
      const int zp = zero_point ? __ldg(zero_point + g) : 0;
      out[n * ldo + k] = __float2bfloat16_rn(static_cast<float>(v - zp) * __ldg(scale + g));
    }
  }
}

// Activations for the F8 GEMM variant: a bf16 value has 8 significant bits, an E4M3 number 4, so x * s = hi + lo with
// hi = e4m3(x * s) (round to nearest even) and lo = x * s - hi holds exactly while both terms stay normal in E4M3.  s is
// the power of two that brings the row's largest magnitude into [128, 256); lo is stored times 16 (it is at most half
// an ulp of hi, so lo * 16 <= |hi|: no overflow) which keeps it normal for |x * s| >= 2^-3, i.e. the split is EXACT for
// every element within 2^10 of its row's maximum and loses low bits gradually below (4 significant bits down to 2^-13
// of the maximum, zero below 2^-17).  out: [2 * M, K] bytes (hi rows, then the lo rows), scale[m] = 1 / s.
// One CTA per row.
__global__ void __launch_bounds__(256)
split_e4m3_kernel(const bf16* __restrict__ x, long long ldx, uint8_t* __restrict__ out, long long ldo, float* __restrict__ scale,
                  int M, int K) {
  pdl_wait();
  pdl_trigger();
  __shared__ float red[8];
  const int m = blockIdx.x;
  const bf16* row = x + m * ldx;
  float amax = 0.0f;
  for (int k = threadIdx.x; k < K; k += blockDim.x) amax = fmaxf(amax, fabsf(__bfloat162float(row[k])));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 16));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 8));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = red[0];
  for (int w = 1; w < static_cast<int>(blockDim.x >> 5); ++w) amax = fmaxf(amax, red[w]);
  const int p = split_scale_exponent(amax);
  const float s = ldexpf(1.0f, p);
  if (threadIdx.x == 0) scale[m] = ldexpf(1.0f, -p);
  uint8_t* hi_row = out + m * ldo;
  uint8_t* lo_row = out + (static_cast<long long>(M) + m) * ldo;
  for (int k = 2 * threadIdx.x; k < K; k += 2 * blockDim.x) {
    const bool two = k + 1 < K;
    const float a = __bfloat162float(row[k]) * s, b = two ? __bfloat162float(row[k + 1]) * s : 0.0f;
    unsigned short h, l;
    split_e4m3_pair(a, b, h, l);
    hi_row[k] = static_cast<uint8_t>(h & 0xff);
    lo_row[k] = static_cast<uint8_t>(l & 0xff);
    if (two) {
      hi_row[k + 1] = static_cast<uint8_t>(h >> 8);
      lo_row[k + 1] = static_cast<uint8_t>(l >> 8);
    }
  }
}

// The same for rows of whole 16-byte pieces (K % 8 == 0, aligned): eight values per load, the row read twice (the
// second pass comes out of L1), eight bytes per store.
__global__ void __launch_bounds__(256)
split_e4m3_vec_kernel(const bf16* __restrict__ x, long long ldx, uint8_t* __restrict__ out, long long ldo, float* __restrict__ scale,
                      int M, int K) {
  pdl_wait();
  pdl_trigger();
  __shared__ float red[8];
  const int m = blockIdx.x;
  const uint4* row = reinterpret_cast<const uint4*>(x + m * ldx);
  const int chunks = K >> 3;
  float amax = 0.0f;
  for (int c = threadIdx.x; c < chunks; c += blockDim.x) {
    const uint4 v = row[c];
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) amax = fmaxf(amax, fmaxf(fabsf(bf16_lo(w[i])), fabsf(bf16_hi(w[i]))));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = red[0];
  for (int w = 1; w < static_cast<int>(blockDim.x >> 5); ++w) amax = fmaxf(amax, red[w]);
  const int p = split_scale_exponent(amax);
  const float s = ldexpf(1.0f, p);
  if (threadIdx.x == 0) scale[m] = ldexpf(1.0f, -p);
  uint2* hi_row = reinterpret_cast<uint2*>(out + m * ldo);
  uint2* lo_row = reinterpret_cast<uint2*>(out + (static_cast<long long>(M) + m) * ldo);
  for (int c = threadIdx.x; c < chunks; c += blockDim.x) {
    const uint4 v = row[c];
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    unsigned short h[4], l[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) split_e4m3_pair(bf16_lo(w[i]) * s, bf16_hi(w[i]) * s, h[i], l[i]);
    hi_row[c] = make_uint2(h[0] | (static_cast<uint32_t>(h[1]) << 16), h[2] | (static_cast<uint32_t>(h[3]) << 16));
    lo_row[c] = make_uint2(l[0] | (static_cast<uint32_t>(l[1]) << 16), l[2] | (static_cast<uint32_t>(l[3]) << 16));
  }
}

__global__ void __launch_bounds__(256) e4m3_count_nan_kernel(const uint8_t* __restrict__ p, size_t n, unsigned* count) {
  unsigned found = 0;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<size_t>(gridDim.x) * blockDim.x)
    found += (p[i] & 0x7fu) == 0x7fu;
  found = __reduce_add_sync(0xffffffffu, found);
  if ((threadIdx.x & 31) == 0 && found) atomicAdd(count, found);
}

}  // namespace

int dequant_e4m3_bf16(const uint8_t* wq, long long ldw, const float* scale, int kind, int group, bf16* out, long long ldo,
                      int N, int K, cudaStream_t st) {
  if (!wq || !scale || !out || N <= 0 || K <= 0 || kind < 0 || kind > 2 || (kind == 2 && group <= 0)) return TEENY_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(wq) & 15) || (ldw & 15) || (reinterpret_cast<uintptr_t>(out) & 15) || (ldo & 7))
    return TEENY_ERR_ALIGNMENT;
  const long long total = static_cast<long long>(N) * ((K + 15) / 16);
  const long long want = (total + 255) / 256;
  const int grid = static_cast<int>(want < 148 * 16 ? want : 148 * 16);
  return launch_kernel(dequant_e4m3_bf16_kernel, dim3(grid), dim3(256), 0, st, 1, wq, ldw, scale, kind, group, out, ldo, N, K);
}

int dequant_int_bf16(const void* q, int bits, const float* scale, const int* zero_point, int kind, int group, bf16* out,
                     long long ldo, int N, int K, cudaStream_t st) {
  if (!q || !scale || !out || N <= 0 || K <= 0 || (bits != 4 && bits != 8) || kind < 0 || kind > 2 || (kind == 2 && group <= 0))
    return TEENY_ERR_BAD_ARG;
  const long long total = static_cast<long long>(N) * ((K + 7) / 8);
  const long long want = (total + 255) / 256;
  const int grid = static_cast<int>(want < 148 * 16 ? want : 148 * 16);
  return launch_kernel(dequant_int_bf16_kernel, dim3(grid), dim3(256), 0, st, 1, static_cast<const uint8_t*>(q), bits, scale,
                       zero_point, kind, group, out, ldo, N, K);
}

int split_e4m3(const bf16* x, long long ldx, uint8_t* out, long long ldo, float* scale, int M, int K, cudaStream_t st) {
  if (!x || !out || !scale || M <= 0 || K <= 0 || ldo < K) return TEENY_ERR_BAD_ARG;
  const bool vec = K % 8 == 0 && ldx % 8 == 0 && ldo % 8 == 0 && !(reinterpret_cast<uintptr_t>(x) & 15) &&
                   !(reinterpret_cast<uintptr_t>(out) & 7);
  if (vec) return launch_kernel(split_e4m3_vec_kernel, dim3(M), dim3(256), 0, st, 1, x, ldx, out, ldo, scale, M, K);
  return launch_kernel(split_e4m3_kernel, dim3(M), dim3(256), 0, st, 1, x, ldx, out, ldo, scale, M, K);
}

int e4m3_count_nan(const uint8_t* p, size_t n, unsigned* count, cudaStream_t st) {
  if (!p || !count) return TEENY_ERR_BAD_ARG;
  if (cudaMemsetAsync(count, 0, sizeof(unsigned), st) != cudaSuccess) return TEENY_ERR_DRIVER;
  if (n == 0) return 0;
  const size_t want = (n + 256 * 64 - 1) / (256 * 64);
  const int grid = static_cast<int>(want < 148 * 8 ? want : 148 * 8);
  return launch_kernel(e4m3_count_nan_kernel, dim3(grid), dim3(256), 0, st, 1, p, n, count);
}

size_t linear_w8a16_scratch_bytes(int M, int N, int K) {
  if (M <= 128 || N <= 0 || K <= 0) return 0;
  return static_cast<size_t>(N) * ((static_cast<size_t>(K) + 7) / 8 * 8) * sizeof(bf16);
}

int linear_w8a16(const bf16* x, int ldx, const uint8_t* wq, int ldw, const float* scale, int kind, int group,
                 const bf16* bias, bf16* y, int ldy, int M, int N, int K, void* scratch, size_t scratch_bytes,
                 cudaStream_t st, bool swiglu, const GemmPush* push) {
  if (M <= 128) return gemm_w8a16_skinny(x, ldx, wq, ldw, scale, kind, group, bias, y, ldy, M, N, K, st, swiglu, push);
  if (push) return TEENY_ERR_BAD_ARG;
  if (!scratch || scratch_bytes < linear_w8a16_scratch_bytes(M, N, K)) return TEENY_ERR_SCRATCH;
  if (reinterpret_cast<uintptr_t>(scratch) & 15) return TEENY_ERR_ALIGNMENT;
  const int ldo = (K + 7) / 8 * 8;
  bf16* w = static_cast<bf16*>(scratch);
  const int rc = dequant_e4m3_bf16(wq, ldw, scale, kind, group, w, ldo, N, K, st);
  if (rc) return rc;
  return gemm_bf16(x, ldx, w, ldo, false, bias, y, ldy, M, N, K, nullptr, 0, st, swiglu);
}

}  // namespace teeny
