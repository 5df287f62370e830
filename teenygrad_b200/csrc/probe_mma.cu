// Development builds only (-DTEENY_TRACE): how fast can threads ISSUE tcgen05.mma?  One thread (or two, in different
// warps) per CTA issues `iters` instructions back to back from a loop with the usual per-step address arithmetic;
// `python -m teenygrad_b200.microbench probe` prints cycles per instruction for the shapes the attention and GEMM
// kernels use.  What it showed on B200: ~100 cycles per instruction from one thread whatever the shape (a 128x128x16
// step needs 64 on the pipe, a 256x256x16 pair step 128), ~70 in aggregate from two threads -- which is why the
// attention kernel issues each product's eight steps as one straight-line block from two issuer threads.
#ifdef TEENY_TRACE
#include "common.cuh"

namespace teeny {

namespace {

__device__ __forceinline__ void probe_mma_pair_ts(uint32_t d, uint32_t a, uint64_t b, uint32_t idesc) {
  asm volatile("{\n\t.reg .pred p;\n\t setp.eq.b32 p, %3, %3;\n\t tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
               ::"r"(d), "r"(a), "l"(b), "r"(idesc) : "memory");
}
__device__ __forceinline__ void probe_mma_pair_ss(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc) {
  asm volatile("{\n\t.reg .pred p;\n\t setp.eq.b32 p, %3, %3;\n\t tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
               ::"r"(d), "l"(a), "l"(b), "r"(idesc) : "memory");
}
__device__ __forceinline__ void probe_commit_pair(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"(static_cast<uint16_t>(3)) : "memory");
}

constexpr int kProbeSmem = 160 * 1024;

// mode bit 0: A from tensor memory (else shared memory); bit 1: alternate between two accumulators; bit 2: two issuers
template <int PAIR>
__global__ void __launch_bounds__(128, 1) probe_kernel(int mode, int N, int iters, long long* out) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar0 = base + kProbeSmem, slot = bar0 + 64;
  uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
  volatile uint32_t* slot_ptr = reinterpret_cast<volatile uint32_t*>(gen + kProbeSmem + 64);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint32_t rank = 0;
  if (PAIR) asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  for (int i = threadIdx.x; i < kProbeSmem / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(gen)[i] = 0x3c003c00u;
  if (warp == 0 && lane == 0) { mbar_init(bar0, 1); mbar_init(bar0 + 8, 1); mbar_fence_init(); }
  if (warp == 1) {
    if (PAIR) {
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot), "r"(512) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      tmem_alloc(slot, 512);
      tmem_relinquish();
    }
  }
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  if (PAIR) asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
  tc_fence_after();
  const uint32_t tmem = *slot_ptr;
  const bool two = mode & 4;
  if ((warp == 0 || (two && warp == 2)) && lane == 0 && rank == 0) {
    const uint32_t bar = bar0 + (warp == 2 ? 8 : 0);
    const uint32_t idesc = make_idesc_bf16(PAIR ? 256 : 128, N, false, false);
    const uint64_t adesc = make_smem_desc_sw128(base, 16, 1024);
    const uint64_t bdesc = make_smem_desc_sw128(base + 64 * 1024, 16, 1024);
    const bool ts = mode & 1, alt = mode & 2;
    const long long c0 = clock64();
    for (int i = 0; i < iters; ++i) {
      const uint32_t d = tmem + ((alt && (i & 1)) ? 128 : 0) + (warp == 2 ? 256 : 0);
      const uint64_t bd = bdesc + static_cast<uint64_t>((i & 3) * 2);
      if (PAIR) {
        if (ts) probe_mma_pair_ts(d, tmem + 448, bd, idesc); else probe_mma_pair_ss(d, adesc + (i & 3) * 2, bd, idesc);
      } else {
        if (ts) umma_bf16_ts(d, tmem + 448, bd, idesc, 1); else umma_bf16_ss(d, adesc + (i & 3) * 2, bd, idesc, 1);
      }
    }
    const long long c1 = clock64();
    if (PAIR) probe_commit_pair(bar); else umma_commit(bar);
    while (!mbar_try_wait(bar, 0)) {
      if (clock64() - c1 > 2000000000ll) break;  // bounded: about a second
    }
    if (blockIdx.x == 0 && warp == 0) { out[0] = c1 - c0; out[1] = clock64() - c0; }
  }
  __syncthreads();
  if (PAIR) asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    if (PAIR) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
    else tmem_dealloc(tmem, 512);
  }
}

template <int PAIR>
int run_probe(int mode, int N, int iters, long long* out_dev) {
  const int smem = kProbeSmem + 1024 + 256;
  cudaError_t e = cudaFuncSetAttribute(probe_kernel<PAIR>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return static_cast<int>(e);
  launch_kernel(probe_kernel<PAIR>, dim3(148), dim3(128), smem, nullptr, PAIR ? 2 : 1, mode, N, iters, out_dev);
  return static_cast<int>(cudaDeviceSynchronize());
}

}  // namespace

}  // namespace teeny

// cycles[0] = issue loop, cycles[1] = until the last instruction completed (device clocks of CTA 0's first issuer)
extern "C" int teeny_probe_mma_issue(int pair, int mode, int N, int iters, long long* cycles) {
  if (!cycles || iters <= 0 || (N != 64 && N != 128 && N != 256) || ((mode & 2) && N == 256)) return TEENY_ERR_BAD_ARG;
  long long* dev = nullptr;
  if (cudaMalloc(&dev, 16) != cudaSuccess) return TEENY_ERR_SCRATCH;
  int rc = pair ? teeny::run_probe<1>(mode, N, iters, dev) : teeny::run_probe<0>(mode, N, iters, dev);
  if (rc == 0) rc = static_cast<int>(cudaMemcpy(cycles, dev, 16, cudaMemcpyDeviceToHost));
  cudaFree(dev);
  return rc;
}
#endif  // TEENY_TRACE
