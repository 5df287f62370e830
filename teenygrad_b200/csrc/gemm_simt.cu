// CUDA-core GEMM with genuine f32 products and accumulation (FFMA): C[m,n] = sum_k A[m,k] * B[k,n] (+ bias[n]).
// It serves (a) the f32 entry points, whose parity bar (1e-4 against an f32 CPU loop) a single-pass TF32 tensor-core
// product cannot meet, and (b) bf16 problems whose pointers or strides the TMA path cannot describe.
// 64 x 64 output tile per CTA, 16-deep k slices through shared memory, 4 x 4 register tile per thread; all operands
// are addressed through element strides so [K,N], [N,K] and padded layouts share the kernel.
#include "common.cuh"
#include "kernels.h"

namespace teeny {

namespace {

constexpr int kTM = 64, kTN = 64, kTK = 16;

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<bf16>(bf16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f<bf16>(float v) { return __float2bfloat16_rn(v); }

template <typename T>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const T* __restrict__ a, long long sam, long long sak, const T* __restrict__ b, long long sbk,
                 long long sbn, const T* __restrict__ bias, T* __restrict__ c, long long scm, long long scn, int M,
                 int N, int K) {
  pdl_wait();
  __shared__ float as[kTK][kTM + 4];
  __shared__ float bs[kTK][kTN + 4];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int m0 = blockIdx.y * kTM, n0 = blockIdx.x * kTN;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += kTK) {
    // 64 x 16 elements of each operand: 4 per thread
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int e = threadIdx.x + i * 256;
      {
        const int kk = e & 15, mm = e >> 4;  // k fastest: unit-stride reads when A is [M,K]
        const int gm = m0 + mm, gk = k0 + kk;
        as[kk][mm] = (gm < M && gk < K) ? to_f<T>(a[gm * sam + gk * sak]) : 0.0f;
      }
      {
        int kk, nn;
        if (sbn == 1) { nn = e & 63; kk = e >> 6; } else { kk = e & 15; nn = e >> 4; }
        const int gn = n0 + nn, gk = k0 + kk;
        bs[kk][nn] = (gn < N && gk < K) ? to_f<T>(b[gk * sbk + gn * sbn]) : 0.0f;
      }
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kTK; ++kk) {
      float av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = as[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) bv[j] = bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gm = m0 + ty * 4 + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tx * 4 + j;
      if (gn < N) {
        float v = acc[i][j];
        if (bias) v += to_f<T>(bias[gn]);
        c[gm * scm + gn * scn] = from_f<T>(v);
      }
    }
  }
}

template <typename T>
int launch(const T* a, long long sam, long long sak, const T* b, long long sbk, long long sbn, const T* bias, T* c,
           long long scm, long long scn, int M, int N, int K, cudaStream_t st) {
  if (!a || !b || !c || M <= 0 || N <= 0 || K <= 0) return TEENY_ERR_BAD_ARG;
  dim3 grid((N + kTN - 1) / kTN, (M + kTM - 1) / kTM);
  if (grid.y > 65535) return TEENY_ERR_BAD_ARG;
  launch_kernel(gemm_simt_kernel<T>, dim3(grid), dim3(256), 0, st, 1, a, sam, sak, b, sbk, sbn, bias, c, scm, scn, M, N, K);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace

int gemm_f32(const float* a, long long sam, long long sak, const float* b, long long sbk, long long sbn,
             const float* bias, float* c, long long scm, long long scn, int M, int N, int K, cudaStream_t stream) {
  return launch<float>(a, sam, sak, b, sbk, sbn, bias, c, scm, scn, M, N, K, stream);
}
int gemm_bf16_generic(const bf16* a, long long sam, long long sak, const bf16* b, long long sbk, long long sbn,
                      const bf16* bias, bf16* c, long long scm, long long scn, int M, int N, int K,
                      cudaStream_t stream) {
  return launch<bf16>(a, sam, sak, b, sbk, sbn, bias, c, scm, scn, M, N, K, stream);
}

}  // namespace teeny
