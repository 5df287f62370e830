// Shared device helpers for the sm_100a kernels: mbarrier, TMA, tcgen05 / TMEM wrappers (inline PTX),
// bounded waits that report through an error word instead of hanging, and small bf16 utilities.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/teeny_b200.h"  // status codes

namespace teeny {

typedef __nv_bfloat16 bf16;

// Codes written to the device error word by kernels (which wait gave up).
enum : int {
  DEVERR_NONE = 0,
  DEVERR_GEMM_PRODUCER = 0x101,
  DEVERR_GEMM_MMA = 0x102,
  DEVERR_GEMM_EPILOGUE = 0x103,
  DEVERR_ATTN_PRODUCER = 0x201,
  DEVERR_ATTN_MMA = 0x202,
  DEVERR_ATTN_SOFTMAX = 0x203,
  DEVERR_TP_GATHER = 0x301,
};

// Host side (defined in api.cu): device address of the per-device error word.
int* device_error_word();

// ------------------------------------------------------------------------------------------------
// generic helpers
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\t elect.sync _|p, 0xffffffff;\n\t selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

__device__ __forceinline__ void named_barrier_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// ------------------------------------------------------------------------------------------------
// programmatic dependent launch
// ------------------------------------------------------------------------------------------------
// Every kernel of this library calls pdl_wait() before it first touches memory that an earlier kernel in the
// stream may still be writing; whatever it does before that (barrier init, TMEM allocation, fetching weights,
// which no kernel writes) overlaps the tail of its predecessor.  pdl_trigger() lets the next kernel become resident:
// the long kernels call it when their main loop is done, the short ones (norms, rope) right after their own wait, so
// that the GEMM or attention kernel behind them streams its first ring of weights or cache tiles while they run.
// No kernel triggers before its own wait has returned: at most two later kernels are ever resident beside the
// running one, and when a kernel starts, everything older than its immediate predecessor is complete.  (Triggering
// at kernel entry everywhere was measured slower: CTAs of several later kernels then sit resident and waiting.)
// Both calls are no-ops for a kernel launched the ordinary way.  Every thread of every CTA executes pdl_wait(), so a
// grid never completes before its predecessor has.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
#ifndef TEENY_TRACE
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
#define TRACE_END() do {} while (0)
#define TRACE_MARK(id, cond) do {} while (0)
#define TRACE_VALUE(id, cond, value) do {} while (0)
#define TRACE_ONLY(...)
#else
// ------------------------------------------------------------------------------------------------
// Kernel timeline (development builds only: make EXTRA=-DTEENY_TRACE).  Thread 0 of every CTA records the global
// timer when it reaches pdl_wait() and when the wait returns, and kernels that call TRACE_END() also when the CTA
// is done (TRACE_MARK(id, cond) adds intermediate records); records carry the source line of the call, the SM, the CTA index and the grid size.  Each translation
// unit has its own buffer and registers a dump function with the C API (teeny_trace_count / _name / _dump), so
// `python -m teenygrad_b200.microbench trace` can print when each kernel of a decode step became resident, was
// released and finished.  The stamps cost an atomic and four stores per CTA: use the output for where time goes,
// not for absolute kernel times.
// ------------------------------------------------------------------------------------------------
static __device__ unsigned long long g_trace[4u << 18];
static __device__ unsigned g_trace_n;
__device__ __forceinline__ void trace_put(unsigned long long t0, unsigned long long t1, int line) {
  const unsigned idx = atomicAdd(&g_trace_n, 1u);
  if (idx < (1u << 18)) {
    unsigned sm;
    asm volatile("mov.u32 %0, %%smid;" : "=r"(sm));
    g_trace[idx * 4 + 0] = t0;
    g_trace[idx * 4 + 1] = t1;
    g_trace[idx * 4 + 2] = static_cast<unsigned long long>(line) | (static_cast<unsigned long long>(sm) << 32);
    g_trace[idx * 4 + 3] = (blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z)) |
                           (static_cast<unsigned long long>(gridDim.x * gridDim.y * gridDim.z) << 32);
  }
}
__device__ __forceinline__ void pdl_wait_traced(int line) {
  const unsigned long long t0 = global_timer_ns();
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (threadIdx.x == 0 && threadIdx.y == 0 && threadIdx.z == 0) trace_put(t0, global_timer_ns(), line);
}
#define pdl_wait() pdl_wait_traced(__LINE__)
// end-of-CTA record (t0 == 0 marks it)
#define TRACE_END() \
  do { if (threadIdx.x == 0 && threadIdx.y == 0 && threadIdx.z == 0) trace_put(0, global_timer_ns(), __LINE__); } while (0)
// intermediate record by the one thread for which `cond` holds (t0 = id, 1..15)
#define TRACE_MARK(id, cond) do { if (cond) trace_put(id, global_timer_ns(), __LINE__); } while (0)
// a measured quantity (e.g. cycles spent in a phase, summed by the caller) instead of a time (t0 = 16 + id, id 0..15)
#define TRACE_VALUE(id, cond, value) do { if (cond) trace_put(16 + (id), static_cast<unsigned long long>(value), __LINE__); } while (0)
#define TRACE_ONLY(...) __VA_ARGS__
typedef int (*teeny_trace_dump_fn)(unsigned long long* out, unsigned cap, int reset);
extern "C" void teeny_trace_register(const char* tu, teeny_trace_dump_fn fn);
namespace {
int trace_dump_tu(unsigned long long* out, unsigned cap, int reset) {
  unsigned n = 0;
  cudaDeviceSynchronize();
  cudaMemcpyFromSymbol(&n, g_trace_n, sizeof(n));
  if (n > (1u << 18)) n = 1u << 18;
  if (n > cap) n = cap;
  if (out && n) cudaMemcpyFromSymbol(out, g_trace, sizeof(unsigned long long) * 4 * n);
  if (reset) { unsigned z = 0; cudaMemcpyToSymbol(g_trace_n, &z, sizeof(z)); }
  return static_cast<int>(n);
}
struct TraceReg { TraceReg() { teeny_trace_register(__BASE_FILE__, trace_dump_tu); } } g_trace_reg;
}
#endif

// Host: whether launches on this thread carry the programmatic-stream-serialization attribute (the Qwen3 runner
// turns it on around its kernel sequences).
bool pdl_enabled();
void pdl_set_enabled(bool on);

// Kernel launches issued by this library since the last reset (process-wide; teeny_launch_count in the C ABI).  A
// launch recorded into a CUDA graph counts once when it is recorded; the runner adds a graph's kernel count per replay.
void count_launches(unsigned long long n);

// Launch through cudaLaunchKernelEx so the attribute can be attached; `cluster` > 1 also sets the cluster width.
template <typename... KArgs, typename... Args>
inline int launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                         unsigned cluster, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  unsigned n = 0;
  if (cluster > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = cluster;
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = 1;
    ++n;
  }
  if (pdl_enabled()) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  count_launches(1);
  return static_cast<int>(cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...));
}

// ------------------------------------------------------------------------------------------------
// mbarrier
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done != 0;
}

// Wait limit for every spin in this library.  Kernels here run for milliseconds; a wait that lasts
// this long means a protocol bug, and the kernel must give the GPU back instead of hanging it.
constexpr uint64_t kWaitLimitNs = 2000000000ull;

// Bounded mbarrier wait.  Returns false (after storing `code` in *err) when the limit expires or when
// another role of the kernel has already reported an error; the caller then leaves its loop.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* err, int code) {
  uint64_t t0 = 0;
#pragma unroll 1
  for (uint32_t it = 0;; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 0xff) == 0xff) {
      if (*reinterpret_cast<volatile int*>(err) != 0) return false;
      const uint64_t now = global_timer_ns();
      if (t0 == 0) {
        t0 = now;
      } else if (now - t0 > kWaitLimitNs) {
        atomicCAS(err, 0, code);
        return false;
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------
// TMA (tiled bulk tensor copies, no multicast anywhere)
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* m, uint32_t bar, int x,
                                            int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* m, uint32_t bar, int x,
                                            int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* m, uint32_t bar, int x,
                                            int y, int z, int w) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(y), "r"(z), "r"(w)
      : "memory");
}
// Asks for a tile to be brought into L2 only (no shared memory, no barrier): what a kernel launched early uses to
// keep HBM streaming its next weight tiles, beyond what its shared-memory ring holds, while its predecessor finishes.
__device__ __forceinline__ void tma_prefetch_l2_2d(const CUtensorMap* m, int x, int y) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];"
               ::"l"(reinterpret_cast<uint64_t>(m)), "r"(x), "r"(y)
               : "memory");
}
// generic-proxy writes to shared memory -> visible to the async proxy (TMA / tcgen05 operand reads)
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ------------------------------------------------------------------------------------------------
// tcgen05 / tensor memory
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {  // whole warp
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {  // whole warp
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// D[tmem] (+)= A[smem] * B[smem]; one thread issues.  accumulate==0 overwrites D.
__device__ __forceinline__ void umma_bf16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                             uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void umma_bf16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                             uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// mbarrier arrives once every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_st() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// 32 lanes x 32 consecutive 32-bit columns: thread t of the warp gets lane (base_lane + t).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
        "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]),
        "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]),
        "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
        "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]),
        "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]),
        "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]),
        "r"(r[31])
      : "memory");
}

__device__ __forceinline__ void tmem_st_32x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]),
        "r"(r[15])
      : "memory");
}

// Shared-memory matrix descriptor for a tile written by TMA with the 128-byte swizzle.
//   K-major operand  ([rows][64] bf16, one 128-byte row per matrix row; 8-row groups 1024 B apart):
//       leading byte offset unused (1), stride byte offset 1024.
//   MN-major operand ([k][64] bf16 per 128-byte row, i.e. 64 MN elements contiguous; 8-k groups 1024 B
//       apart; successive 64-element MN chunks `mn_chunk_bytes` apart):
//       leading byte offset = mn_chunk_bytes, stride byte offset 1024.
// Bits: [0,14) address>>4, [16,30) LBO>>4, [32,46) SBO>>4, [46,48) version=1, [61,64) layout=2 (SW128).
__device__ __forceinline__ uint64_t make_smem_desc_sw128(uint32_t smem_addr, uint32_t lbo_bytes,
                                                         uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3ffff) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3fff) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3fff) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

// Instruction descriptor for kind::f16 with bf16 A/B and f32 accumulate.
//   bits [4,6) D format (1 = f32), [7,10) A format (1 = bf16), [10,13) B format, 15 A major (1 = MN),
//   16 B major, [17,23) N>>3, [24,29) M>>4.
__host__ __device__ constexpr uint32_t make_idesc_bf16(int m, int n, bool a_mn_major, bool b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(a_mn_major) << 15) |
         (static_cast<uint32_t>(b_mn_major) << 16) | (static_cast<uint32_t>(n >> 3) << 17) |
         (static_cast<uint32_t>(m >> 4) << 24);
}

// The same descriptor for kind::f8f6f4 with both operands E4M3 (format code 0), K-major, f32 accumulate.
__host__ __device__ constexpr uint32_t make_idesc_e4m3(int m, int n) {
  return (1u << 4) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

// ------------------------------------------------------------------------------------------------
// two-term FP8 activations (see split_e4m3_kernel, gemm_w8a16.cu)
// ------------------------------------------------------------------------------------------------
// Exponent p of the row scale s = 2^p that brings a row maximum `amax` into [128, 256) (0 for a zero / non-finite row;
// clamped so that s and 1 / s are normal f32 numbers).
__device__ __forceinline__ int split_scale_exponent(float amax) {
  if (!(amax > 0.0f) || !(amax < INFINITY)) return 0;
  int e;
  frexpf(amax, &e);  // amax = f * 2^e, f in [0.5, 1): floor(log2 amax) = e - 1
  return min(100, max(-100, 8 - e));
}
// a, b (already multiplied by the row scale) -> hi = e4m3(x), lo = e4m3((x - hi) * 16), two elements per 16-bit result
// (a in the low byte), round to nearest even, saturating
__device__ __forceinline__ void split_e4m3_pair(float a, float b, unsigned short& hi, unsigned short& lo) {
  const __nv_fp8x2_storage_t h = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2(h, __NV_E4M3);
  const float2 hf = __half22float2(*reinterpret_cast<const __half2*>(&hr));
  lo = __nv_cvt_float2_to_fp8x2(make_float2((a - hf.x) * 16.0f, (b - hf.y) * 16.0f), __NV_SATFINITE, __NV_E4M3);
  hi = h;
}

// ------------------------------------------------------------------------------------------------
// small math helpers
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
__device__ __forceinline__ float bf16_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }

__device__ __forceinline__ uint32_t bf16x2_mul(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ uint32_t bf16x2_add(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("add.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

// Per-head RMSNorm followed by rotate-half RoPE for one 128-wide head spread over a half-warp: lane `sub` (0..15)
// holds elements [8 sub, 8 sub + 8) of the head (raw), of the norm weight (wraw) and of the position's cos / sin rows
// (craw, sraw); the rotate-half partner elements (d +- 64) live in lane sub ^ 8.  Every lane of the warp must call
// this (shuffles).  Rounding points follow the traced bf16 graph: the normed head, each product and the sum are
// bf16 tensors.  Returns the eight rotated elements packed as bf16.
__device__ __forceinline__ uint4 head_norm_rope(const uint4 raw, const uint4 wraw, const uint4 craw, const uint4 sraw,
                                                int sub, float eps) {
  const uint32_t rw[4] = {raw.x, raw.y, raw.z, raw.w};
  float sq = 0.0f;
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    sq += bf16_lo(rw[e]) * bf16_lo(rw[e]);
    sq += bf16_hi(rw[e]) * bf16_hi(rw[e]);
  }
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);  // stays inside the half-warp
  const float rr = 1.0f / sqrtf(sq * (1.0f / 128.0f) + eps);
  const uint32_t ww[4] = {wraw.x, wraw.y, wraw.z, wraw.w}, cw[4] = {craw.x, craw.y, craw.z, craw.w},
                 sw[4] = {sraw.x, sraw.y, sraw.z, sraw.w};
  const uint32_t flip = (sub < 8) ? 0x80008000u : 0u;  // rotate_half: the first half gets -x[d + 64]
  uint32_t out[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    // Two elements at a time.  A product of two bf16 values is exact in f32, and so is their sum unless it is far
    // below the result's rounding step, so the packed bf16 multiply / add (one rounding) equal the f32 operation
    // followed by a rounding to bf16.
    const uint32_t xn = pack_bf16x2(bf16_lo(rw[e]) * rr, bf16_hi(rw[e]) * rr);
    const uint32_t n = bf16x2_mul(xn, ww[e]);  // normed head, a bf16 tensor in the traced graph
    const uint32_t partner = __shfl_xor_sync(0xffffffffu, n, 8) ^ flip;
    out[e] = bf16x2_add(bf16x2_mul(n, cw[e]), bf16x2_mul(partner, sw[e]));
  }
  return make_uint4(out[0], out[1], out[2], out[3]);
}

// A {32-bit payload, 32-bit stamp} pair as ONE 64-bit word in (possibly another GPU's) global memory: a 64-bit scalar
// access is single-copy atomic, so a reader that sees the stamp sees the payload written with it.  (A 16-byte vector
// store of two pairs carries no such guarantee between its halves, let alone inside one.)  Layout = uint2{payload, stamp}.
__device__ __forceinline__ void st_stamped(uint2* dst, uint32_t payload, uint32_t stamp) {
  const unsigned long long word = (static_cast<unsigned long long>(stamp) << 32) | payload;
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(dst), "l"(word) : "memory");
}
__device__ __forceinline__ unsigned long long ld_stamped(const uint2* src) {
  unsigned long long word;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(word) : "l"(src) : "memory");
  return word;
}
// Two neighbouring pairs in one 16-byte access (dst / src 16-byte aligned).  A vector access counts as one access per
// element, so each 64-bit pair is still single-copy atomic on its own, and the access keeps the width that NVLink
// packets and the memory system like.
__device__ __forceinline__ void st_stamped_x2(uint2* dst, uint32_t payload0, uint32_t payload1, uint32_t stamp) {
  const unsigned long long hi = static_cast<unsigned long long>(stamp) << 32;
  asm volatile("st.relaxed.sys.global.v2.u64 [%0], {%1, %2};" ::"l"(dst), "l"(hi | payload0), "l"(hi | payload1) : "memory");
}
__device__ __forceinline__ void ld_stamped_x2(const uint2* src, unsigned long long& w0, unsigned long long& w1) {
  asm volatile("ld.relaxed.sys.global.v2.u64 {%0, %1}, [%2];" : "=l"(w0), "=l"(w1) : "l"(src) : "memory");
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// ------------------------------------------------------------------------------------------------
// host: tensor-map encoding through the driver entry point (no link-time dependency on libcuda)
// ------------------------------------------------------------------------------------------------
// Encodes a bf16 tensor of `rank` dims (dims[0] innermost, strides in BYTES for dims 1..rank-1) with the
// 128-byte swizzle; box[0] must be 64 elements.  Returns TEENY_OK or an error code.
int encode_tensor_map_bf16(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                           const uint64_t* strides_bytes, const uint32_t* box);
// the same for a tensor of bytes
int encode_tensor_map_u8(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                         const uint64_t* strides_bytes, const uint32_t* box);

// SMs of the current device that this thread's launches size their grids for: the device's count, or less while a
// limit is set (set_sm_limit(n), n <= 0 clears it) to leave SMs to kernels of another stream.
int sm_count();
void set_sm_limit(int n);

}  // namespace teeny
