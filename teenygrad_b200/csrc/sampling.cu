// Token sampling after the LM head: temperature, top-k and top-p (nucleus) over one row of bf16 logits per CTA.
//
// The reference ships only the row softmax next to the logits (kernels/teeny-kernels/src/nn/activation/softmax.rs:39;
// Op::TopK is unlowered, kernels/teeny-kernels/src/graph/mod.rs:2784); this is the step a serving loop needs behind
// it.  Definition (oracle/sampling.py restates it on the CPU):
//   1. candidates = the top_k entries of the row by (logit descending, index ascending);
//   2. e_i = exp((l_i - l_0) / temperature) in f32 over the candidates in that order, c_i = e_0 + ... + e_i summed
//      sequentially in f32;
//   3. nucleus = the shortest prefix with c_{n-1} >= top_p * c_last (at least one candidate);
//   4. the sample is the first candidate i < n with c_i > u * c_{n-1}, u in [0, 1) given per row by the caller.
// bf16 logits have 65536 possible values, so the k-th largest value is found exactly with two 256-bin histograms
// (high byte, then low byte inside the deciding bin); ties at the threshold are resolved in index order by a third,
// ordered pass.  The <= 1024 candidates are sorted in shared memory (bitonic), exponentials are computed in parallel
// and one thread does the sequential sums so the result does not depend on a reduction tree.
#include <atomic>

#include "common.cuh"
#include "kernels.h"

namespace teeny {

namespace {

constexpr int kSampleThreads = 1024;
constexpr int kMaxTopK = 1024;

// bf16 bit pattern -> 16-bit key whose unsigned order is the float order (NaNs sort above +inf; not expected here)
__device__ __forceinline__ unsigned sort_key(unsigned short bits) {
  return (bits & 0x8000u) ? (~static_cast<unsigned>(bits) & 0xFFFFu) : (static_cast<unsigned>(bits) | 0x8000u);
}
__device__ __forceinline__ float key_to_float(unsigned key) {
  const unsigned bits = (key & 0x8000u) ? (key & 0x7FFFu) : (~key & 0xFFFFu);
  return __uint_as_float(bits << 16);
}

// Largest bin b with (number of entries in bins above b) < want <= (number in bins >= b); `above` gets the former.
__device__ void pick_bin(const unsigned* hist, unsigned want, unsigned* bin_out, unsigned* above_out) {
  unsigned above = 0;
  int b = 255;
  for (; b > 0; --b) {
    if (above + hist[b] >= want) break;
    above += hist[b];
  }
  *bin_out = static_cast<unsigned>(b);
  *above_out = above;
}

// Steps 2-4 of the definition over the K sorted candidates in cand[]: exponentials in parallel, sums by one thread in
// candidate order.  A candidate is (key << 32) | (0xFFFFFFFF - index).
__device__ __forceinline__ void pick_from_sorted(const unsigned long long* cand, float* expv, unsigned K, float inv_temperature,
                                                 float top_p, float u, int* out_idx, float* out_prob) {
  const int tid = threadIdx.x;
  const float l0 = key_to_float(static_cast<unsigned>(cand[0] >> 32));
  if (static_cast<unsigned>(tid) < K) expv[tid] = expf((key_to_float(static_cast<unsigned>(cand[tid] >> 32)) - l0) * inv_temperature);
  __syncthreads();
  if (tid == 0) {
    float total = 0.0f;
    for (unsigned i = 0; i < K; ++i) total += expv[i];
    // nucleus: shortest prefix whose mass reaches top_p of the total
    const float want = top_p * total;
    float c = 0.0f;
    unsigned n = 0;
    while (n < K) {
      c += expv[n];
      ++n;
      if (c >= want) break;
    }
    const float target = u * c;  // c = mass of the nucleus
    float run = 0.0f;
    unsigned pick = n - 1;
    for (unsigned i = 0; i < n; ++i) {
      run += expv[i];
      if (run > target) { pick = i; break; }
    }
    *out_idx = static_cast<int>(0xFFFFFFFFu - static_cast<unsigned>(cand[pick] & 0xFFFFFFFFull));
    if (out_prob) *out_prob = expv[pick] / c;
  }
}

// cand_out != null: stop after step 1 and write the K sorted candidates of the row, indices shifted by idx_offset, to
// cand_out[row * cand_stride ...] (a vocabulary shard's contribution under tensor parallelism; sample_merge_kernel
// finishes the job over all shards' lists).
__global__ void __launch_bounds__(kSampleThreads, 1)
sample_top_k_top_p_kernel(const bf16* __restrict__ logits, long long ld, int cols, float inv_temperature, int top_k,
                          float top_p, const float* __restrict__ u, int* __restrict__ out_idx,
                          float* __restrict__ out_prob, unsigned long long* __restrict__ cand_out, int cand_stride,
                          int idx_offset) {
  pdl_wait();
  __shared__ unsigned hist[256];
  __shared__ unsigned long long cand[kMaxTopK];  // (key << 32) | (0xFFFFFFFF - index): descending = value desc, index asc
  __shared__ float expv[kMaxTopK];
  __shared__ unsigned s_bin, s_above, s_count, s_eq_base;
  __shared__ unsigned warp_tot[32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const unsigned short* row = reinterpret_cast<const unsigned short*>(logits) + static_cast<size_t>(blockIdx.x) * ld;
  const unsigned K = static_cast<unsigned>(min(top_k, cols));

  // ---- pass 1: histogram of the key's high byte ----
  if (tid < 256) hist[tid] = 0;
  __syncthreads();
  for (int i = tid; i < cols; i += kSampleThreads) atomicAdd(&hist[sort_key(row[i]) >> 8], 1u);
  __syncthreads();
  if (tid == 0) pick_bin(hist, K, &s_bin, &s_above);
  __syncthreads();
  const unsigned hi_bin = s_bin, above_hi = s_above;
  __syncthreads();
  // ---- pass 2: histogram of the low byte inside that bin ----
  if (tid < 256) hist[tid] = 0;
  __syncthreads();
  for (int i = tid; i < cols; i += kSampleThreads) {
    const unsigned k = sort_key(row[i]);
    if ((k >> 8) == hi_bin) atomicAdd(&hist[k & 255u], 1u);
  }
  __syncthreads();
  if (tid == 0) pick_bin(hist, K - above_hi, &s_bin, &s_above);
  __syncthreads();
  const unsigned thresh = (hi_bin << 8) | s_bin;            // the K-th largest key
  const unsigned need_eq = K - (above_hi + s_above);        // how many entries equal to it are taken (>= 1)
  if (tid == 0) { s_count = 0; s_eq_base = 0; }
  for (int i = tid; i < kMaxTopK; i += kSampleThreads) cand[i] = 0ull;
  __syncthreads();
  // ---- pass 3, in index order: everything above the threshold, and the first need_eq entries equal to it ----
  for (int base = 0; base < cols; base += kSampleThreads) {
    const int i = base + tid;
    const unsigned k = i < cols ? sort_key(row[i]) : 0u;
    const bool gt = i < cols && k > thresh, eq = i < cols && k == thresh;
    // rank of this thread's tie among the ties of the tile (block-wide exclusive count in index order)
    const unsigned eq_mask = __ballot_sync(0xffffffffu, eq);
    if (lane == 0) warp_tot[warp] = __popc(eq_mask);
    __syncthreads();
    unsigned before = s_eq_base;
    for (int w = 0; w < warp; ++w) before += warp_tot[w];
    before += __popc(eq_mask & ((1u << lane) - 1u));
    if (gt || (eq && before < need_eq)) {
      const unsigned slot = atomicAdd(&s_count, 1u);
      if (slot < static_cast<unsigned>(kMaxTopK))
        cand[slot] = (static_cast<unsigned long long>(k) << 32) | (0xFFFFFFFFu - static_cast<unsigned>(i));
    }
    __syncthreads();
    if (tid == 0) {
      unsigned t = 0;
      for (int w = 0; w < 32; ++w) t += warp_tot[w];
      s_eq_base += t;
    }
    __syncthreads();
  }
  // ---- bitonic sort of the 1024 slots, descending (empty slots are zero and end up last) ----
  for (unsigned size = 2; size <= static_cast<unsigned>(kMaxTopK); size <<= 1) {
    for (unsigned stride = size >> 1; stride > 0; stride >>= 1) {
      const unsigned partner = tid ^ stride;
      if (partner > static_cast<unsigned>(tid)) {
        const bool descending = (tid & size) == 0;
        const unsigned long long a = cand[tid], b = cand[partner];
        if ((a < b) == descending) { cand[tid] = b; cand[partner] = a; }
      }
      __syncthreads();
    }
  }
  if (cand_out) {
    // entries past K are zero (smaller than any real candidate); the shift keeps (value desc, index asc) order
    if (tid < cand_stride) {
      const unsigned long long c = cand[tid];
      cand_out[static_cast<size_t>(blockIdx.x) * cand_stride + tid] =
          static_cast<unsigned>(tid) < K ? ((c & 0xFFFFFFFF00000000ull) | ((c & 0xFFFFFFFFull) - static_cast<unsigned>(idx_offset))) : 0ull;
    }
    return;
  }
  pick_from_sorted(cand, expv, K, inv_temperature, top_p, u[blockIdx.x], out_idx + blockIdx.x,
                   out_prob ? out_prob + blockIdx.x : nullptr);
}

// Tensor-parallel finish: lists[p * list_stride + row * K + i] is candidate i (sorted descending) of vocabulary shard p
// for this row; the top K of their union are found by rank counting -- a candidate's place in the union is the number
// of candidates above it, a binary search per list, and the keys are distinct -- and steps 2-4 follow as on one GPU,
// so every rank, given the same u, picks the same token as the unsharded kernel would.
__global__ void __launch_bounds__(kSampleThreads, 1)
sample_merge_kernel(const unsigned long long* __restrict__ lists, int parts, size_t list_stride, int K_list, int top_k,
                    float inv_temperature, float top_p, const float* __restrict__ u, int* __restrict__ out_idx,
                    float* __restrict__ out_prob) {
  pdl_wait();
  extern __shared__ unsigned long long all[];      // [parts][K_list]
  __shared__ unsigned long long cand[kMaxTopK];
  __shared__ float expv[kMaxTopK];
  const int tid = threadIdx.x;
  const int total = parts * K_list;
  for (int i = tid; i < total; i += kSampleThreads) {
    const int p = i / K_list, e = i - p * K_list;
    all[i] = lists[static_cast<size_t>(p) * list_stride + static_cast<size_t>(blockIdx.x) * K_list + e];
  }
  for (int i = tid; i < kMaxTopK; i += kSampleThreads) cand[i] = 0ull;
  __syncthreads();
  unsigned live = 0;  // real candidates in the union (empty slots are zero)
  for (int i = tid; i < total; i += kSampleThreads) {
    const unsigned long long c = all[i];
    if (c == 0ull) continue;
    unsigned above = 0;
    for (int p = 0; p < parts; ++p) {  // entries of list p greater than c: lists are sorted descending
      const unsigned long long* lp = all + p * K_list;
      int lo = 0, hi = K_list;
      while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (lp[mid] > c) lo = mid + 1; else hi = mid;
      }
      above += static_cast<unsigned>(lo);
    }
    if (above < static_cast<unsigned>(kMaxTopK)) cand[above] = c;
    ++live;
  }
  __shared__ unsigned s_live;
  if (tid == 0) s_live = 0;
  __syncthreads();
  if (live) atomicAdd(&s_live, live);
  __syncthreads();
  const unsigned K = min(static_cast<unsigned>(top_k), s_live);
  pick_from_sorted(cand, expv, K, inv_temperature, top_p, u[blockIdx.x], out_idx + blockIdx.x,
                   out_prob ? out_prob + blockIdx.x : nullptr);
}

// u[row] in [0, 1) as a pure function of (seed, step, row): a splitmix64 finaliser over the three, top 24 bits.
// (oracle/sampling.py restates it, so a generation can be replayed on the CPU.)
__global__ void sampling_uniform_kernel(unsigned long long seed, int step, const int* __restrict__ step_dev,
                                        float* __restrict__ u, int rows) {
  pdl_wait();
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  const unsigned long long t = static_cast<unsigned long long>(step_dev ? *step_dev : step);
  unsigned long long x = seed ^ (t * 0x9E3779B97F4A7C15ull) ^ (static_cast<unsigned long long>(r) * 0xBF58476D1CE4E5B9ull);
  x ^= x >> 30; x *= 0xBF58476D1CE4E5B9ull;
  x ^= x >> 27; x *= 0x94D049BB133111EBull;
  x ^= x >> 31;
  u[r] = static_cast<float>(x >> 40) * (1.0f / 16777216.0f);
}

}  // namespace

int sampling_uniform(unsigned long long seed, int step, const int* step_dev, float* u, int rows, cudaStream_t st) {
  if (!u || rows < 0) return TEENY_ERR_BAD_ARG;
  if (rows == 0) return TEENY_OK;
  launch_kernel(sampling_uniform_kernel, dim3((rows + 127) / 128), dim3(128), 0, st, 1, seed, step, step_dev, u, rows);
  return static_cast<int>(cudaGetLastError());
}

int sample_top_k_top_p_bf16(const bf16* logits, long long ld, int rows, int cols, float temperature, int top_k,
                            float top_p, const float* u, int* out_idx, float* out_prob, cudaStream_t st) {
  if (!logits || !u || !out_idx || rows < 0 || cols <= 0 || ld < cols) return TEENY_ERR_BAD_ARG;
  if (!(temperature > 0.0f) || top_k < 1 || top_k > kMaxTopK || !(top_p > 0.0f) || top_p > 1.0f) return TEENY_ERR_BAD_ARG;
  if (rows == 0) return TEENY_OK;
  launch_kernel(sample_top_k_top_p_kernel, dim3(rows), dim3(kSampleThreads), 0, st, 1, logits, ld, cols,
                1.0f / temperature, top_k, top_p, u, out_idx, out_prob, static_cast<unsigned long long*>(nullptr), 0, 0);
  return static_cast<int>(cudaGetLastError());
}

int sample_candidates_bf16(const bf16* logits, long long ld, int rows, int cols, int top_k, int idx_offset,
                           unsigned long long* cand_out, cudaStream_t st) {
  if (!logits || !cand_out || rows < 0 || cols <= 0 || ld < cols || top_k < 1 || top_k > kMaxTopK || idx_offset < 0)
    return TEENY_ERR_BAD_ARG;
  if (rows == 0) return TEENY_OK;
  launch_kernel(sample_top_k_top_p_kernel, dim3(rows), dim3(kSampleThreads), 0, st, 1, logits, ld, cols, 1.0f, top_k, 1.0f,
                static_cast<const float*>(nullptr), static_cast<int*>(nullptr), static_cast<float*>(nullptr), cand_out,
                top_k, idx_offset);
  return static_cast<int>(cudaGetLastError());
}

int sample_merge_prepare() {
  static std::atomic<unsigned long long> done{0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 64 && (done.load(std::memory_order_acquire) >> dev) & 1ull) return 0;
  cudaError_t e = cudaFuncSetAttribute(sample_merge_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 8 * kMaxTopK * 8);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 64) done.fetch_or(1ull << dev, std::memory_order_release);
  return 0;
}

int sample_merge(const unsigned long long* lists, int parts, size_t list_stride, int rows, float temperature, int top_k,
                 float top_p, const float* u, int* out_idx, float* out_prob, cudaStream_t st) {
  if (!lists || !u || !out_idx || parts < 1 || parts > 8 || rows < 0 || list_stride < static_cast<size_t>(rows) * top_k)
    return TEENY_ERR_BAD_ARG;
  if (!(temperature > 0.0f) || top_k < 1 || top_k > kMaxTopK || !(top_p > 0.0f) || top_p > 1.0f) return TEENY_ERR_BAD_ARG;
  if (rows == 0) return TEENY_OK;
  const int prc = sample_merge_prepare();
  if (prc) return prc;
  launch_kernel(sample_merge_kernel, dim3(rows), dim3(kSampleThreads), static_cast<size_t>(parts) * top_k * 8, st, 1, lists,
                parts, list_stride, top_k, top_k, 1.0f / temperature, top_p, u, out_idx, out_prob);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace teeny
