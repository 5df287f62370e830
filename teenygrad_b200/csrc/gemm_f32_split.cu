// f32 matmul on the tensor cores at f32 accuracy ("bf16 x 3"): C = A B with every operand split into two bf16 terms.
//
// x = hi + mid + r with hi = bf16(x), mid = bf16(x - hi), |r| <= 2^-17 |x|.  A B = sum_k a b ~ hi_a hi_b + mid_a hi_b +
// hi_a mid_b; what is dropped (mid_a mid_b and the r terms) is below 2^-15 of each product, the products themselves are
// exact in f32 (8-bit x 8-bit mantissas) and the sums run in the tensor core's f32 accumulator.  Against an f32
// reference the result is within a few 1e-6 of max|C| -- the 1e-4 bar of the f32 entry points has a wide margin, which
// one TF32 pass (10-bit mantissas, ~1e-3) does not meet.  The three products are ONE bf16 GEMM over a three times
// longer K: A' = [hi_a | mid_a | hi_a] (M x 3K), B' = [hi_b ; hi_b ; mid_b] (3K x N).
// The reference's kernel computes the same product with TF32 MMAs (kernels/teeny-kernels/src/math/gemm.rs:95) and its
// DSL names this split InputPrecision::TF32x3 (kernels/teeny-triton/src/triton/mod.rs:76-83).
#include "common.cuh"
#include "kernels.h"

namespace teeny {

namespace {

// one thread per 8 consecutive elements of a row: src [rows, cols] f32 -> dst rows of 3 * cols (A', LEFT) or three row
// blocks of `rows` (B', !LEFT) holding hi and mid in the orders above
template <bool LEFT>
__global__ void split_bf16_kernel(const float* __restrict__ src, bf16* __restrict__ dst, int rows, int cols) {
  pdl_wait();
  const long long vecs = static_cast<long long>(rows) * (cols >> 3);
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < vecs;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int r = static_cast<int>(i / (cols >> 3)), c = static_cast<int>(i % (cols >> 3)) * 8;
    const float4 lo = *reinterpret_cast<const float4*>(src + static_cast<size_t>(r) * cols + c);
    const float4 hi4 = *reinterpret_cast<const float4*>(src + static_cast<size_t>(r) * cols + c + 4);
    const float x[8] = {lo.x, lo.y, lo.z, lo.w, hi4.x, hi4.y, hi4.z, hi4.w};
    uint32_t h[4], m[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float h0 = bf16_round(x[2 * e]), h1 = bf16_round(x[2 * e + 1]);
      h[e] = pack_bf16x2(h0, h1);
      m[e] = pack_bf16x2(x[2 * e] - h0, x[2 * e + 1] - h1);
    }
    const uint4 hv = make_uint4(h[0], h[1], h[2], h[3]), mv = make_uint4(m[0], m[1], m[2], m[3]);
    if (LEFT) {  // [hi | mid | hi] along the row
      bf16* d = dst + static_cast<size_t>(r) * 3 * cols + c;
      *reinterpret_cast<uint4*>(d) = hv;
      *reinterpret_cast<uint4*>(d + cols) = mv;
      *reinterpret_cast<uint4*>(d + 2 * cols) = hv;
    } else {     // [hi ; hi ; mid] down the rows
      bf16* d = dst + static_cast<size_t>(r) * cols + c;
      const size_t block = static_cast<size_t>(rows) * cols;
      *reinterpret_cast<uint4*>(d) = hv;
      *reinterpret_cast<uint4*>(d + block) = hv;
      *reinterpret_cast<uint4*>(d + 2 * block) = mv;
    }
  }
}

size_t align256(size_t v) { return (v + 255) / 256 * 256; }

}  // namespace

size_t gemm_f32_split_scratch_bytes(int M, int N, int K) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  return align256(static_cast<size_t>(M) * 3 * K * 2) + align256(static_cast<size_t>(3) * K * N * 2);
}

int gemm_f32_split(const float* a, const float* b, float* c, int M, int N, int K, void* scratch, size_t scratch_bytes,
                   cudaStream_t stream) {
  if (!a || !b || !c || !scratch || M <= 0 || N <= 0 || K <= 0) return TEENY_ERR_BAD_ARG;
  if ((K & 7) || (N & 7)) return TEENY_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(c) |
       reinterpret_cast<uintptr_t>(scratch)) & 15)
    return TEENY_ERR_ALIGNMENT;
  if (scratch_bytes < gemm_f32_split_scratch_bytes(M, N, K)) return TEENY_ERR_SCRATCH;
  bf16* a3 = static_cast<bf16*>(scratch);
  bf16* b3 = reinterpret_cast<bf16*>(static_cast<uint8_t*>(scratch) + align256(static_cast<size_t>(M) * 3 * K * 2));
  const int threads = 256;
  auto blocks = [&](long long vecs) { return static_cast<int>(vecs / threads + 1 < 2048 ? vecs / threads + 1 : 2048); };
  launch_kernel(split_bf16_kernel<true>, dim3(blocks(static_cast<long long>(M) * (K >> 3))), dim3(threads), 0, stream, 1, a,
                a3, M, K);
  launch_kernel(split_bf16_kernel<false>, dim3(blocks(static_cast<long long>(K) * (N >> 3))), dim3(threads), 0, stream, 1, b,
                b3, K, N);
  const int rc = static_cast<int>(cudaGetLastError());
  if (rc) return rc;
  return gemm_bf16(a3, 3 * K, b3, N, /*w_is_kn=*/true, nullptr, nullptr, N, M, N, 3 * K, nullptr, 0, stream, false, nullptr, c);
}

}  // namespace teeny
