// bf16 GEMM for sm_100a: D[i, j] = sum_k P[i, k] * Q[j, k] with f32 accumulation in tensor memory.
//
// Kernel 1 -- gemm_bf16_kernel: persistent, warp-specialised, one CTA per SM.
//   warp 0      TMA producer: P tile [128 x 64] and Q tile [BN x 64] per k-block into a ring of shared-memory
//               stages (128-byte swizzle), completion on `full` mbarriers;
//   warp 1      MMA issuer: one elected thread issues tcgen05.mma (M=128, N=BN, K=16) four times per k-block,
//               tcgen05.commit releases the stage (`empty`) and finally publishes the accumulator (`acc_full`);
//   warps 2-5   epilogue: tcgen05.ld the 128 x BN f32 accumulator (thread = row), convert to bf16, store.
//   The accumulator is double buffered in TMEM (2 x BN columns) so the epilogue of tile t overlaps the main loop
//   of tile t+1.
//
// Two operand assignments share the code:
//   normal  P = activations X [M, K], Q = weights W [N, K]  -> Y[m, n] tile 128 x BN
//   swapped P = weights W [N, K],     Q = activations X     -> Y^T tile; used when M is small (decode), so the
//           128-row MMA dimension is filled by weight rows and the token count only sets N of the MMA.
// B may also be MN-major ([K, N] row-major, the matmul_forward layout): its tiles are [64 k][64 n] boxes and the
// descriptor uses the MN-major canonical layout.
//
// Kernel 2 -- gemm_bf16_skinny_kernel: the swapped assignment for weight matrices with too few 128-row tiles to
// occupy the GPU (decode: M <= 128 tokens, N of a few thousand).  These GEMMs only stream weights, so the job is to
// get every SM pulling from HBM: K is split across a thread-block cluster (2, 4 or 8 CTAs per weight tile, one
// k-range each, small enough that two CTAs share an SM), every CTA accumulates its partial tile in TMEM, parks it
// in its own shared memory, and after a cluster barrier the CTAs sum the partials through distributed shared
// memory -- each CTA reduces its own slice of the token columns, in cluster-rank order, so the result is
// bit-reproducible.  No global scratch, no atomics.
#include <atomic>
#include <cstdlib>

#include "common.cuh"
#include "kernels.h"

namespace teeny {

namespace {

int ceil_div(int a, int b) { return (a + b - 1) / b; }

constexpr int kBM = 128;  // rows of P per tile (MMA M)
constexpr int kBK = 64;   // k-block: 64 bf16 = one 128-byte swizzle row
constexpr int kNumThreads = 192;
constexpr int kEpilogueThreads = 128;

struct GemmArgs {
  int M, N, K;            // Y[M, N] = X[M, K] * W[N, K]^T
  int ldy;                // row stride of Y in elements
  bf16* y;
  float* y32;             // when set (persistent kernel, unswapped): the f32 accumulators are stored as they are, to y32[M, ldy]
  const bf16* bias;       // [N] or null
  int tiles_p, tiles_q;   // tiles along P rows and along Q rows
  int k_blocks;           // ceil(K / 64)
  int group;              // persistent kernel: P-tiles per raster group
  int kb_per_split;       // skinny kernel: k-blocks per cluster rank
  int l2_ahead;           // skinny kernel: weight k-blocks asked into L2 beyond the shared-memory ring at start
  int swiglu;             // W rows interleave 64 gate / 64 up channels; Y[M, N/2] = silu(gate) * up
  // Tensor-parallel push (skinny kernel only): instead of Y, the f32 row sums go to slot `rank` of every rank's
  // receive buffer (peer-mapped memory, [M][N] f32 each) and each CTA then bumps every rank's arrival counter.
  uint2* const* push_recv;    // device array [push_world]: where this rank writes inside rank p's buffer (or null)
  const unsigned* push_epoch; // stamp of the pushed {value, stamp} pairs = *push_epoch * 1024 + push_round + 1
  unsigned push_round;
  int push_world;
  int push_owner_rows;        // > 0: token row c goes only to rank c / push_owner_rows (which reduces it); 0: to every rank
  int* err;
};

template <int BN>
struct GemmCfg {
  static constexpr int kStageP = kBM * kBK * 2;
  static constexpr int kStageQ = BN * kBK * 2;
  static constexpr int kStageBytes = kStageP + kStageQ;
  static constexpr int kStages = (BN >= 256) ? 4 : (BN >= 128 ? 6 : 8);
  static constexpr int kTmemCols = (2 * BN < 32) ? 32 : 2 * BN;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*align slack*/ + 256 /*barriers*/;
};

__device__ __forceinline__ void tile_coords(int tile, int tiles_p, int tiles_q, int kGroup, int& tp, int& tq) {
  // Grouped raster: kGroup consecutive P-tiles share each Q-tile before moving on, so the tiles in flight across
  // the SMs reuse both operands out of L2.
  const int per_group = kGroup * tiles_q;
  const int g = tile / per_group;
  const int first_p = g * kGroup;
  const int size_p = min(kGroup, tiles_p - first_p);
  const int r = tile - g * per_group;
  tp = first_p + r % size_p;
  tq = r / size_p;
}

// SwiGLU on two projections of the same channel, with the rounding points of the unfused graph: both projections
// are bf16 tensors, silu is evaluated in f32 and rounded to bf16, the product is rounded to bf16 by the caller.
__device__ __forceinline__ float swiglu_f(float gate_acc, float up_acc) {
  const float g = bf16_round(gate_acc), u = bf16_round(up_acc);
  return bf16_round(g * (1.0f / (1.0f + expf(-g)))) * u;
}

// One k-block of MMAs: four K=16 steps over the 64-wide stage.
template <int BN, bool Q_MN_MAJOR>
__device__ __forceinline__ void issue_kblock(uint32_t d_tmem, uint32_t sp, uint32_t sq, bool first) {
  constexpr uint32_t idesc = make_idesc_bf16(kBM, BN, false, Q_MN_MAJOR);
  const uint64_t pdesc = make_smem_desc_sw128(sp, 16, 1024);
  const uint64_t qdesc = Q_MN_MAJOR ? make_smem_desc_sw128(sq, kBK * 128, 1024) : make_smem_desc_sw128(sq, 16, 1024);
#pragma unroll
  for (int k = 0; k < kBK / 16; ++k) {
    // K-major: 16 elements along k = 32 bytes inside the swizzled row -> +2 in the address field.
    // MN-major: 16 k = two 8-row groups of 1024 bytes -> +128.
    const uint64_t pd = pdesc + static_cast<uint64_t>(k * 2);
    const uint64_t qd = qdesc + static_cast<uint64_t>(Q_MN_MAJOR ? k * 128 : k * 2);
    umma_bf16_ss(d_tmem, pd, qd, idesc, (!first || k > 0) ? 1u : 0u);
  }
}

template <int BN, bool SWAP, bool Q_MN_MAJOR>
__global__ void __launch_bounds__(kNumThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmap_p, const __grid_constant__ CUtensorMap tmap_q,
                 const GemmArgs args) {
  using Cfg = GemmCfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar_base = smem_base + Cfg::kStages * Cfg::kStageBytes;
  // barrier layout (8 B each): full[kStages], empty[kStages], acc_full[2], acc_empty[2], then the TMEM address
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (Cfg::kStages + s); };
  auto acc_full_bar = [&](int b) { return bar_base + 8u * (2 * Cfg::kStages + b); };
  auto acc_empty_bar = [&](int b) { return bar_base + 8u * (2 * Cfg::kStages + 2 + b); };
  const uint32_t tmem_slot = bar_base + 8u * (2 * Cfg::kStages + 4);
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  volatile uint32_t* tmem_slot_ptr =
      reinterpret_cast<volatile uint32_t*>(smem_gen + Cfg::kStages * Cfg::kStageBytes + 8 * (2 * Cfg::kStages + 4));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  int* err = args.err;

  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmap_p);
    tma_prefetch_desc(&tmap_q);
    for (int s = 0; s < Cfg::kStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full_bar(b), 1);
      mbar_init(acc_empty_bar(b), kEpilogueThreads / 32);
    }
    mbar_fence_init();
  }
  if (warp == 2) {
    tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;
  pdl_wait();  // set-up above overlapped the previous kernel; operands and outputs are touched from here on

  const int num_work = args.tiles_p * args.tiles_q;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int w = blockIdx.x; ok && w < num_work; w += gridDim.x) {
        int tp, tq;
        tile_coords(w, args.tiles_p, args.tiles_q, args.group, tp, tq);
        for (int kb = 0; kb < args.k_blocks; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1, err, DEVERR_GEMM_PRODUCER)) { ok = false; break; }
          const uint32_t sp = smem_base + stage * Cfg::kStageBytes;
          const uint32_t sq = sp + Cfg::kStageP;
          mbar_expect_tx(full_bar(stage), Cfg::kStageBytes);
          tma_load_2d(sp, &tmap_p, full_bar(stage), kb * kBK, tp * kBM);
          if constexpr (Q_MN_MAJOR) {
            // Q is [K, N] row-major: boxes of [64 k][64 n]; BN/64 boxes per stage, 8 KB each.
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              tma_load_2d(sq + c * (kBK * 128), &tmap_q, full_bar(stage), tq * BN + c * 64, kb * kBK);
          } else {
            tma_load_2d(sq, &tmap_q, full_bar(stage), kb * kBK, tq * BN);
          }
          if (++stage == Cfg::kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int local = 0;
      for (int w = blockIdx.x; ok && w < num_work; w += gridDim.x, ++local) {
        const int buf = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1;
        if (!mbar_wait(acc_empty_bar(buf), acc_phase ^ 1, err, DEVERR_GEMM_MMA)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = 0; kb < args.k_blocks; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, err, DEVERR_GEMM_MMA)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sp = smem_base + stage * Cfg::kStageBytes;
          issue_kblock<BN, Q_MN_MAJOR>(d_tmem, sp, sp + Cfg::kStageP, kb == 0);
          umma_commit(empty_bar(stage));  // stage reusable once these MMAs have read it
          if (++stage == Cfg::kStages) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit(acc_full_bar(buf));
      }
    }
  } else {
    // ---------------- epilogue (warps 2..5; TMEM lane quarter = warp % 4) ----------------
    const int quarter = warp & 3;
    const int row_in_tile = quarter * 32 + lane;
    bool ok = true;
    int local = 0;
    for (int w = blockIdx.x; ok && w < num_work; w += gridDim.x, ++local) {
      int tp, tq;
      tile_coords(w, args.tiles_p, args.tiles_q, args.group, tp, tq);
      const int buf = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      if (!mbar_wait(acc_full_bar(buf), acc_phase, err, DEVERR_GEMM_EPILOGUE)) { ok = false; break; }
      tc_fence_after();
      const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * BN;
      const int prow = tp * kBM + row_in_tile;  // index along P rows
      constexpr int kChunk = (BN >= 32) ? 32 : 16;
      if constexpr (!SWAP && BN >= 128) {
        if (args.swiglu) {
          // columns come in groups of 128 weight rows = 64 gate + 64 up channels: emit 64 outputs per group
#pragma unroll 1
          for (int c0 = 0; c0 < BN; c0 += 128) {
#pragma unroll 1
            for (int sub = 0; sub < 64; sub += 32) {
              uint32_t gr[32], ur[32];
              tmem_ld_32x32(t_addr + c0 + sub, gr);
              tmem_ld_32x32(t_addr + c0 + 64 + sub, ur);
              tmem_wait_ld();
              const int ocol0 = (tq * BN + c0) / 2 + sub;
              if (prow < args.M) {
                bf16* dst = args.y + static_cast<size_t>(prow) * args.ldy + ocol0;
                const bool vec_ok = ((reinterpret_cast<uintptr_t>(dst) & 15) == 0) && (ocol0 + 32 <= args.N / 2);
#pragma unroll
                for (int v = 0; v < 4; ++v) {
                  float f[8];
#pragma unroll
                  for (int e = 0; e < 8; ++e)
                    f[e] = swiglu_f(__uint_as_float(gr[v * 8 + e]), __uint_as_float(ur[v * 8 + e]));
                  if (vec_ok) {
                    uint4 o;
                    o.x = pack_bf16x2(f[0], f[1]); o.y = pack_bf16x2(f[2], f[3]);
                    o.z = pack_bf16x2(f[4], f[5]); o.w = pack_bf16x2(f[6], f[7]);
                    *reinterpret_cast<uint4*>(dst + v * 8) = o;
                  } else {
#pragma unroll
                    for (int e = 0; e < 8; ++e)
                      if (ocol0 + v * 8 + e < args.N / 2) dst[v * 8 + e] = __float2bfloat16_rn(f[e]);
                  }
                }
              }
            }
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(acc_empty_bar(buf));
          continue;
        }
      }
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += kChunk) {
        uint32_t r[kChunk];
        if constexpr (kChunk == 32) tmem_ld_32x32(t_addr + c0, r); else tmem_ld_32x16(t_addr + c0, r);
        tmem_wait_ld();
        const int qcol0 = tq * BN + c0;  // index along Q rows
        if constexpr (!SWAP) {
          // thread owns Y[prow, qcol0 .. qcol0+kChunk)
          if (prow < args.M && args.y32) {
            float* dst = args.y32 + static_cast<size_t>(prow) * args.ldy + qcol0;
            if (((reinterpret_cast<uintptr_t>(dst) & 15) == 0) && (qcol0 + kChunk <= args.N)) {
#pragma unroll
              for (int v = 0; v < kChunk / 4; ++v)
                *reinterpret_cast<uint4*>(dst + v * 4) = make_uint4(r[v * 4], r[v * 4 + 1], r[v * 4 + 2], r[v * 4 + 3]);
            } else {
#pragma unroll
              for (int e = 0; e < kChunk; ++e)
                if (qcol0 + e < args.N) dst[e] = __uint_as_float(r[e]);
            }
          } else if (prow < args.M) {
            bf16* dst = args.y + static_cast<size_t>(prow) * args.ldy + qcol0;
            const bool vec_ok = ((reinterpret_cast<uintptr_t>(dst) & 15) == 0) && (qcol0 + kChunk <= args.N);
            if (vec_ok) {
#pragma unroll
              for (int v = 0; v < kChunk / 8; ++v) {
                float f[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                  f[e] = __uint_as_float(r[v * 8 + e]);
                  if (args.bias) f[e] += __bfloat162float(args.bias[qcol0 + v * 8 + e]);
                }
                uint4 o;
                o.x = pack_bf16x2(f[0], f[1]); o.y = pack_bf16x2(f[2], f[3]);
                o.z = pack_bf16x2(f[4], f[5]); o.w = pack_bf16x2(f[6], f[7]);
                *reinterpret_cast<uint4*>(dst + v * 8) = o;
              }
            } else {
#pragma unroll
              for (int e = 0; e < kChunk; ++e) {
                const int n = qcol0 + e;
                if (n < args.N) {
                  float f = __uint_as_float(r[e]);
                  if (args.bias) f += __bfloat162float(args.bias[n]);
                  dst[e] = __float2bfloat16_rn(f);
                }
              }
            }
          }
        } else {
          // thread owns Y[qcol0 + e, prow] for e in the chunk (prow indexes N); lanes are consecutive in n.
          if (prow < args.N) {
            const float b = args.bias ? __bfloat162float(args.bias[prow]) : 0.0f;
#pragma unroll
            for (int e = 0; e < kChunk; ++e) {
              const int m = qcol0 + e;
              if (m < args.M)
                args.y[static_cast<size_t>(m) * args.ldy + prow] = __float2bfloat16_rn(__uint_as_float(r[e]) + b);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty_bar(buf));
    }
  }

  // ---------------- teardown ----------------
  pdl_trigger();  // this CTA has no more tiles to start: the next kernel may begin its set-up
  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    if (*reinterpret_cast<volatile int*>(err) != 0) {
      // A wait gave up: let copies / MMAs that are still in flight drain before the memory is released.
      const uint64_t t0 = global_timer_ns();
      while (global_timer_ns() - t0 < 2000000ull) __nanosleep(1000);
    }
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

// ------------------------------------------------------------------------------------------------
// Kernel 2: cluster split-K for the swapped (small-M) assignment
// ------------------------------------------------------------------------------------------------
// Weight k-blocks (16 KB each) a decode GEMM's CTA asks into L2 beyond its shared-memory ring while it waits for its
// predecessor (TEENY_L2_AHEAD overrides).  Measured on a 12-layer Qwen3-8B-shaped decode step: 1.79 / 1.80 / 1.83 / 1.85 /
// 1.88 ms with 0 / 4 / 8 / 16 / 32 blocks -- the early requests take bandwidth from the predecessor's tail instead of
// filling an idle bus -- so the default is none.
constexpr int kL2Ahead = 0;

template <int BN>
struct SkinnyCfg {
  static constexpr int kStageP = kBM * kBK * 2;
  static constexpr int kStageQ = BN * kBK * 2;
  static constexpr int kStageBytes = kStageP + kStageQ;
  // As many stages as let two CTAs share an SM (about 100 KB each): what streams the weights fast is the number of
  // bytes in flight per SM, and two short-lived CTAs overlap each other's set-up and reduction.
  static constexpr int kStages = (BN <= 32) ? 5 : (BN <= 64 ? 4 : 3);
  static constexpr int kPartialBytes = BN * kBM * 4;  // f32 partial tile, column-major [BN][128]; reuses the ring
  static_assert(kPartialBytes <= kStages * kStageBytes, "partial tile must fit in the stage ring");
  static constexpr int kTmemCols = BN < 32 ? 32 : BN;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 128;
};

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t cluster_size() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// 16 bytes of CTA `rank`'s shared memory at this CTA's address `local_addr`.  Volatile (so it stays behind the cluster
// barrier, itself a volatile asm) but without a memory clobber: consecutive loads are all in flight together.
__device__ __forceinline__ float4 ld_cluster_f32x4(uint32_t local_addr, uint32_t rank) {
  uint32_t remote;
  float4 v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(remote));
  return v;
}

// grid (S, tiles): blockIdx.x = cluster rank = k-split, blockIdx.y = 128-row weight tile.
template <int BN>
__global__ void __launch_bounds__(kNumThreads, 2)
gemm_bf16_skinny_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                        const GemmArgs args) {
  using Cfg = SkinnyCfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  // The partial tile is written after the last MMA has completed, i.e. when no stage is in use any more, so it
  // lives at the start of the ring.
  const uint32_t part_base = smem_base;
  const uint32_t bar_base = smem_base + Cfg::kStages * Cfg::kStageBytes;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (Cfg::kStages + s); };
  const uint32_t acc_full_bar = bar_base + 8u * (2 * Cfg::kStages);
  const uint32_t tmem_slot = acc_full_bar + 8;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  float* part_gen = reinterpret_cast<float*>(smem_gen);
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(
      smem_gen + Cfg::kStages * Cfg::kStageBytes + 8 * (2 * Cfg::kStages + 1));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int* err = args.err;
  const uint32_t S = cluster_size(), rank = cluster_rank();
  const int tile = blockIdx.y;
  const int kb0 = static_cast<int>(rank) * args.kb_per_split;
  const int kb1 = min(args.k_blocks, kb0 + args.kb_per_split);

  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmap_w);
    tma_prefetch_desc(&tmap_x);
    for (int s = 0; s < Cfg::kStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(acc_full_bar, 1);
    mbar_fence_init();
  }
  if (warp == 2) {
    tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;

  if (warp == 0) {
    if (lane == 0) {
      // Weights are never written by a kernel of the stream, so the first ring of weight tiles is requested while
      // the previous kernel may still be running; the activation tiles follow once it has finished.
      const int pre = min(kb1 - kb0, Cfg::kStages);
      for (int i = 0; i < pre; ++i) {
        mbar_expect_tx(full_bar(i), Cfg::kStageBytes);
        tma_load_2d(smem_base + i * Cfg::kStageBytes, &tmap_w, full_bar(i), (kb0 + i) * kBK, tile * kBM);
      }
      // ... and the weight tiles behind them are asked into L2, so that HBM keeps streaming this kernel's weights for
      // as long as the predecessor's tail lasts, not just until the ring is full
      for (int kb = kb0 + pre; kb < min(kb1, kb0 + pre + args.l2_ahead); ++kb) tma_prefetch_l2_2d(&tmap_w, kb * kBK, tile * kBM);
      pdl_wait();
      for (int i = 0; i < pre; ++i)
        tma_load_2d(smem_base + i * Cfg::kStageBytes + Cfg::kStageP, &tmap_x, full_bar(i), (kb0 + i) * kBK, 0);
      int stage = pre == Cfg::kStages ? 0 : pre;
      uint32_t phase = pre == Cfg::kStages ? 1 : 0;
      for (int kb = kb0 + pre; kb < kb1; ++kb) {
        if (!mbar_wait(empty_bar(stage), phase ^ 1, err, DEVERR_GEMM_PRODUCER)) break;
        const uint32_t sp = smem_base + stage * Cfg::kStageBytes;
        mbar_expect_tx(full_bar(stage), Cfg::kStageBytes);
        tma_load_2d(sp, &tmap_w, full_bar(stage), kb * kBK, tile * kBM);
        tma_load_2d(sp + Cfg::kStageP, &tmap_x, full_bar(stage), kb * kBK, 0);
        if (++stage == Cfg::kStages) { stage = 0; phase ^= 1; }
      }
    } else {
      pdl_wait();
    }
  } else if (warp == 1) {
    pdl_wait();
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!mbar_wait(full_bar(stage), phase, err, DEVERR_GEMM_MMA)) { ok = false; break; }
        tc_fence_after();
        const uint32_t sp = smem_base + stage * Cfg::kStageBytes;
        issue_kblock<BN, false>(tmem_base, sp, sp + Cfg::kStageP, kb == kb0);
        umma_commit(empty_bar(stage));
        if (++stage == Cfg::kStages) { stage = 0; phase ^= 1; }
      }
      if (ok) umma_commit(acc_full_bar);
    }
  } else {
    pdl_wait();
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    if (mbar_wait(acc_full_bar, 0, err, DEVERR_GEMM_EPILOGUE)) {
      TRACE_MARK(1, threadIdx.x == 64);
      tc_fence_after();
      const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
      constexpr int kChunk = (BN >= 32) ? 32 : 16;
      const bool direct = (S == 1) && !args.swiglu;
      const int n = tile * kBM + row;
      const float bias = (direct && args.bias && n < args.N) ? __bfloat162float(args.bias[n]) : 0.0f;
      const unsigned stamp = (direct && args.push_recv) ? __ldcg(args.push_epoch) * 1024u + args.push_round + 1u : 0u;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += kChunk) {
        uint32_t r[kChunk];
        if constexpr (kChunk == 32) tmem_ld_32x32(t_addr + c0, r); else tmem_ld_32x16(t_addr + c0, r);
        tmem_wait_ld();
        if (direct) {
          // the whole K range was this CTA's: registers -> global, a warp's 32 rows side by side in each token row
          if (n < args.N) {
#pragma unroll
            for (int e = 0; e < kChunk; ++e) {
              const int c = c0 + e;
              if (c < args.M) {
                const float v = __uint_as_float(r[e]) + bias;
                if (args.push_recv) {
                  const size_t off = static_cast<size_t>(c) * args.N + n;
                  const int p0 = args.push_owner_rows > 0 ? c / args.push_owner_rows : 0;
                  const int p1 = args.push_owner_rows > 0 ? p0 + 1 : args.push_world;
                  for (int p = p0; p < p1; ++p)  // NVLink stores, one 64-bit word per {value, stamp}
                    st_stamped(args.push_recv[p] + off, __float_as_uint(v), stamp);
                } else {
                  args.y[static_cast<size_t>(c) * args.ldy + n] = __float2bfloat16_rn(v);
                }
              }
            }
          }
        } else {
          // accumulator -> this CTA's partial tile in shared memory, column-major (a token column = 128 consecutive
          // words), so these stores and the 16-byte reads of the reduction are both conflict-free
#pragma unroll
          for (int e = 0; e < kChunk; ++e) part_gen[(c0 + e) * kBM + row] = __uint_as_float(r[e]);
        }
      }
      tc_fence_before();
    }
  }

  __syncwarp();
  pdl_trigger();  // main loop done: the next kernel's set-up (and weight prefetch) overlaps the reduction below
  const bool reduce = (S > 1) || args.swiglu;
  // every partial tile of the cluster is in place
  if (S > 1) cluster_sync_all(); else if (reduce) __syncthreads();
  TRACE_MARK(2, threadIdx.x == 64);

  if (warp >= 2 && reduce) {
    // CTA `rank` finishes token columns [rank * cw, (rank + 1) * cw): per 16-byte unit (4 weight rows of one token
    // column) all S partial values are requested at once and summed in rank order
    const int cw = (BN + static_cast<int>(S) - 1) / static_cast<int>(S);  // columns per rank (last rank may get fewer)
    const int c_begin = static_cast<int>(rank) * cw;
    const int ncols = min(BN, c_begin + cw) - c_begin;
    const int epi = (warp - 2) * 32 + lane;
    if (args.swiglu) {
      // the tile holds 64 gate rows then the 64 up rows of the same channels: a unit = 4 channels of one column
      const bool vec_ok = (args.ldy % 4 == 0) && ((reinterpret_cast<uintptr_t>(args.y) & 7) == 0);
      for (int u = epi; u < ncols * 16; u += kEpilogueThreads) {
        const int c = c_begin + (u >> 4), j = u & 15;
        const uint32_t ga = part_base + static_cast<uint32_t>((c * kBM + 4 * j) * 4);
        float4 gv[8], uv[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          gv[q] = (static_cast<uint32_t>(q) < S) ? ld_cluster_f32x4(ga, q) : make_float4(0.f, 0.f, 0.f, 0.f);
          uv[q] = (static_cast<uint32_t>(q) < S) ? ld_cluster_f32x4(ga + 64 * 4, q) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        float4 gs = gv[0], us = uv[0];
#pragma unroll
        for (int q = 1; q < 8; ++q) {
          gs.x += gv[q].x; gs.y += gv[q].y; gs.z += gv[q].z; gs.w += gv[q].w;
          us.x += uv[q].x; us.y += uv[q].y; us.z += uv[q].z; us.w += uv[q].w;
        }
        const int n_out = tile * 64 + 4 * j;
        if (c < args.M) {
          const float o[4] = {swiglu_f(gs.x, us.x), swiglu_f(gs.y, us.y), swiglu_f(gs.z, us.z), swiglu_f(gs.w, us.w)};
          bf16* dst = args.y + static_cast<size_t>(c) * args.ldy + n_out;
          if (vec_ok && n_out + 3 < args.N / 2) {
            *reinterpret_cast<uint2*>(dst) = make_uint2(pack_bf16x2(o[0], o[1]), pack_bf16x2(o[2], o[3]));
          } else {
            for (int e = 0; e < 4; ++e)
              if (n_out + e < args.N / 2) dst[e] = __float2bfloat16_rn(o[e]);
          }
        }
      }
    } else {
      const bool vec_ok = args.push_recv ? (args.N % 4 == 0)
                                         : ((args.ldy % 4 == 0) && ((reinterpret_cast<uintptr_t>(args.y) & 7) == 0));
      const unsigned stamp = args.push_recv ? __ldcg(args.push_epoch) * 1024u + args.push_round + 1u : 0u;
      for (int u = epi; u < ncols * 32; u += kEpilogueThreads) {
        const int c = c_begin + (u >> 5), j = u & 31;
        const uint32_t addr = part_base + static_cast<uint32_t>((c * kBM + 4 * j) * 4);
        float4 v[8];
#pragma unroll
        for (int q = 0; q < 8; ++q)
          v[q] = (static_cast<uint32_t>(q) < S) ? ld_cluster_f32x4(addr, q) : make_float4(0.f, 0.f, 0.f, 0.f);
        float4 acc = v[0];
#pragma unroll
        for (int q = 1; q < 8; ++q) { acc.x += v[q].x; acc.y += v[q].y; acc.z += v[q].z; acc.w += v[q].w; }
        const int n = tile * kBM + 4 * j;
        if (c < args.M && n < args.N) {
          float o[4] = {acc.x, acc.y, acc.z, acc.w};
          if (args.bias) {
#pragma unroll
            for (int e = 0; e < 4; ++e)
              if (n + e < args.N) o[e] += __bfloat162float(args.bias[n + e]);
          }
          if (args.push_recv) {
            const size_t off = static_cast<size_t>(c) * args.N + n;
            const int p0 = args.push_owner_rows > 0 ? c / args.push_owner_rows : 0;
            const int p1 = args.push_owner_rows > 0 ? p0 + 1 : args.push_world;
            for (int p = p0; p < p1; ++p) {  // NVLink stores: 16 bytes = two {value, stamp} words, each atomic on its own
              if (vec_ok) {
                st_stamped_x2(args.push_recv[p] + off, __float_as_uint(o[0]), __float_as_uint(o[1]), stamp);
                st_stamped_x2(args.push_recv[p] + off + 2, __float_as_uint(o[2]), __float_as_uint(o[3]), stamp);
              } else {
#pragma unroll
                for (int e = 0; e < 4; ++e)
                  if (n + e < args.N) st_stamped(args.push_recv[p] + off + e, __float_as_uint(o[e]), stamp);
              }
            }
          } else {
            bf16* dst = args.y + static_cast<size_t>(c) * args.ldy + n;
            if (vec_ok && n + 3 < args.N) {
              *reinterpret_cast<uint2*>(dst) = make_uint2(pack_bf16x2(o[0], o[1]), pack_bf16x2(o[2], o[3]));
            } else {
              for (int e = 0; e < 4; ++e)
                if (n + e < args.N) dst[e] = __float2bfloat16_rn(o[e]);
            }
          }
        }
      }
    }
  }
  TRACE_MARK(3, threadIdx.x == 64);

  // nobody leaves (and frees its shared memory) while a peer may still be reading it
  __syncwarp();
  if (S > 1) cluster_sync_all(); else __syncthreads();
  if (warp == 2) {
    if (*reinterpret_cast<volatile int*>(err) != 0) {
      const uint64_t t0 = global_timer_ns();
      while (global_timer_ns() - t0 < 2000000ull) __nanosleep(1000);
    }
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
  TRACE_END();
}

// ------------------------------------------------------------------------------------------------
// host launchers
// ------------------------------------------------------------------------------------------------
// Raises the kernel's dynamic shared-memory limit once per device (bit d of `done` = device d prepared).
template <int BN, bool SWAP, bool Q_MN>
int prepare_variant() {
  static std::atomic<unsigned long long> done{0};  // one bit per device; threads may race to set it
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 64 && (done.load(std::memory_order_acquire) >> dev) & 1ull) return 0;
  cudaError_t e = cudaFuncSetAttribute(gemm_bf16_kernel<BN, SWAP, Q_MN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       GemmCfg<BN>::kSmemBytes);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 64) done.fetch_or(1ull << dev, std::memory_order_release);
  return 0;
}

template <int BN>
int prepare_skinny() {
  static std::atomic<unsigned long long> done{0};  // one bit per device; threads may race to set it
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 64 && (done.load(std::memory_order_acquire) >> dev) & 1ull) return 0;
  cudaError_t e = cudaFuncSetAttribute(gemm_bf16_skinny_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       SkinnyCfg<BN>::kSmemBytes);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 64) done.fetch_or(1ull << dev, std::memory_order_release);
  return 0;
}

template <int BN, bool SWAP, bool Q_MN>
int launch_variant(const CUtensorMap& tp, const CUtensorMap& tq, const GemmArgs& a, int grid, cudaStream_t st) {
  const int rc = prepare_variant<BN, SWAP, Q_MN>();
  if (rc) return rc;
  launch_kernel(gemm_bf16_kernel<BN, SWAP, Q_MN>, dim3(grid), dim3(kNumThreads), GemmCfg<BN>::kSmemBytes, st, 1, tp, tq, a);
  return static_cast<int>(cudaGetLastError());
}

template <int BN>
int launch_skinny(const CUtensorMap& tw, const CUtensorMap& tx, const GemmArgs& a, int split, int tiles,
                  cudaStream_t st) {
  const int rc = prepare_skinny<BN>();
  if (rc) return rc;
  return launch_kernel(gemm_bf16_skinny_kernel<BN>, dim3(split, tiles, 1), dim3(kNumThreads, 1, 1),
                       SkinnyCfg<BN>::kSmemBytes, st, static_cast<unsigned>(split), tw, tx, a);
}

// Largest token count that takes the swapped (weights on the 128-row MMA side) assignment.
constexpr int kSwapMaxM = 128;
int swap_bn(int M) { return M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : 128)); }

}  // namespace

int gemm_bf16_prepare() {
  int rc = 0;
  if ((rc = prepare_variant<16, true, false>())) return rc;
  if ((rc = prepare_variant<32, true, false>())) return rc;
  if ((rc = prepare_variant<64, true, false>())) return rc;
  if ((rc = prepare_variant<128, true, false>())) return rc;
  if ((rc = prepare_variant<128, false, false>())) return rc;
  if ((rc = prepare_variant<256, false, false>())) return rc;
  if ((rc = prepare_variant<64, false, true>())) return rc;
  if ((rc = prepare_variant<128, false, true>())) return rc;
  if ((rc = prepare_skinny<16>())) return rc;
  if ((rc = prepare_skinny<32>())) return rc;
  if ((rc = prepare_skinny<64>())) return rc;
  return prepare_skinny<128>();
}

bool gemm_bf16_uses_2cta(int M, int N) {
  return M > kSwapMaxM && static_cast<long long>(ceil_div(M, 256)) * ceil_div(N, 256) >= sm_count() / 2;
}

// The GEMM keeps its split-K partials in distributed shared memory: no global scratch at any shape.
size_t gemm_bf16_scratch_bytes(int, int, int) { return 0; }

// Y[M,N] = X[M,K] W^T (+bias).  w_is_kn: W given as [K, N] row-major (matmul_forward's B) instead of [N, K].
int gemm_bf16(const bf16* x, int ldx, const bf16* w, int ldw, bool w_is_kn, const bf16* bias, bf16* y, int ldy,
              int M, int N, int K, void*, size_t, cudaStream_t stream, bool swiglu, const GemmPush* push, float* y32,
              int l2_ahead) {
  if (!x || !w || (!y && !y32) || M <= 0 || N <= 0 || K <= 0) return TEENY_ERR_BAD_ARG;
  if (y32 && (!w_is_kn || swiglu || push || bias)) return TEENY_ERR_BAD_ARG;  // f32 output: the [K, N] form only
  if (swiglu && (w_is_kn || bias || N % 128 != 0)) return TEENY_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15) || (ldx & 7) || (ldw & 7))
    return TEENY_ERR_ALIGNMENT;

  GemmArgs a{};
  a.M = M; a.N = N; a.K = K; a.ldy = ldy; a.y = y; a.y32 = y32; a.bias = bias;
  a.k_blocks = ceil_div(K, kBK);
  a.kb_per_split = a.k_blocks;
  a.group = 8;
  a.swiglu = swiglu ? 1 : 0;
  {
    static const int ahead = [] { const char* e = getenv("TEENY_L2_AHEAD"); return e ? atoi(e) : kL2Ahead; }();
    a.l2_ahead = l2_ahead >= 0 ? l2_ahead : (ahead < 0 ? 0 : ahead);
  }
  if (push) {
    if (swiglu || w_is_kn || M > kSwapMaxM || !push->recv || !push->epoch || push->world < 2 || push->round >= 1023)
      return TEENY_ERR_BAD_ARG;
    a.push_recv = push->recv;
    a.push_epoch = push->epoch;
    a.push_round = push->round;
    a.push_world = push->world;
    a.push_owner_rows = push->owner_rows;
  }
  a.err = device_error_word();
  if (!a.err) return TEENY_ERR_DRIVER;  // kernels report expired waits through this word: no launch without it
  const int sms = sm_count();

  CUtensorMap tmx, tmw;
  const bool swap = (!w_is_kn) && (M <= kSwapMaxM);
  int bn;
  if (swap) {
    bn = swap_bn(M);
  } else if (w_is_kn) {
    bn = (N <= 64) ? 64 : 128;
  } else {
    bn = (N <= 128 || (static_cast<long long>(ceil_div(M, kBM)) * ceil_div(N, 256) < sms)) ? 128 : 256;
  }

  // activations X: K-major rows; box = 64 k x (128 rows normally, bn rows when swapped)
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(M)};
    const uint64_t strides[1] = {static_cast<uint64_t>(ldx) * 2};
    const uint32_t box[2] = {kBK, static_cast<uint32_t>(swap ? bn : kBM)};
    int rc = encode_tensor_map_bf16(&tmx, x, 2, dims, strides, box);
    if (rc) return rc;
  }
  if (w_is_kn) {
    const uint64_t dims[2] = {static_cast<uint64_t>(N), static_cast<uint64_t>(K)};
    const uint64_t strides[1] = {static_cast<uint64_t>(ldw) * 2};
    const uint32_t box[2] = {64, kBK};
    int rc = encode_tensor_map_bf16(&tmw, w, 2, dims, strides, box);
    if (rc) return rc;
  } else {
    const uint64_t dims[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(N)};
    const uint64_t strides[1] = {static_cast<uint64_t>(ldw) * 2};
    const uint32_t box[2] = {kBK, static_cast<uint32_t>(swap ? kBM : bn)};
    int rc = encode_tensor_map_bf16(&tmw, w, 2, dims, strides, box);
    if (rc) return rc;
  }

  if (swap) {
    const int tiles = ceil_div(N, kBM);
    if ((tiles < 4 * sms || swiglu || push) && tiles <= 65535) {
      // Few weight tiles: cluster split-K.  Measured on B200 (batch 32, K = 4096 / 12288): the kernel is fastest
      // when all its CTAs are resident at once (two per SM) and share HBM evenly -- about 0.85 of the slots -- and a
      // wider cluster than that only adds barrier and reduction cost; with at least as many tiles as SMs no split.
      const int slots = sms * 2;
      int split = (slots * 85 / 100) / tiles;
      if (split > 8) split = 8;
      {  // TEENY_SKINNY_SPLIT: fixed cluster width, for measurements
        static const int forced = [] { const char* e = getenv("TEENY_SKINNY_SPLIT"); return e ? atoi(e) : 0; }();
        if (forced > 0 && forced <= 8) split = forced;
      }
      while (split > 1 && (ceil_div(a.k_blocks, split) < 4 || ceil_div(a.k_blocks, split) * (split - 1) >= a.k_blocks))
        --split;  // too thin, or a rank would be left without k-blocks
      if (split < 1) split = 1;
      a.kb_per_split = ceil_div(a.k_blocks, split);
      {  // what the CTAs ask into L2 ahead of time must stay well inside it (126 MB): at most 48 MB over the grid
        const long long per_cta = (48ll << 20) / (static_cast<long long>(kBM * kBK * 2) * split * tiles);
        if (a.l2_ahead > per_cta) a.l2_ahead = static_cast<int>(per_cta);
      }
      switch (bn) {
        case 16: return launch_skinny<16>(tmw, tmx, a, split, tiles, stream);
        case 32: return launch_skinny<32>(tmw, tmx, a, split, tiles, stream);
        case 64: return launch_skinny<64>(tmw, tmx, a, split, tiles, stream);
        default: return launch_skinny<128>(tmw, tmx, a, split, tiles, stream);
      }
    }
    a.tiles_p = tiles;
    a.tiles_q = 1;
    const int grid = tiles < sms ? tiles : sms;
    switch (bn) {
      case 16: return launch_variant<16, true, false>(tmw, tmx, a, grid, stream);
      case 32: return launch_variant<32, true, false>(tmw, tmx, a, grid, stream);
      case 64: return launch_variant<64, true, false>(tmw, tmx, a, grid, stream);
      default: return launch_variant<128, true, false>(tmw, tmx, a, grid, stream);
    }
  }

  // Enough 256 x 256 tiles to occupy every SM pair: the CTA-pair kernel (about a fifth faster at these sizes).
  if (!w_is_kn && gemm_bf16_uses_2cta(M, N))
    return gemm_bf16_2cta(x, ldx, w, ldw, bias, y, ldy, M, N, K, stream, swiglu);
  a.tiles_p = ceil_div(M, kBM);
  a.tiles_q = ceil_div(N, bn);
  const int work = a.tiles_p * a.tiles_q;
  const int grid = work < sms ? work : sms;
  if (w_is_kn) {
    if (bn == 64) return launch_variant<64, false, true>(tmx, tmw, a, grid, stream);
    return launch_variant<128, false, true>(tmx, tmw, a, grid, stream);
  }
  if (bn == 128) return launch_variant<128, false, false>(tmx, tmw, a, grid, stream);
  return launch_variant<256, false, false>(tmx, tmw, a, grid, stream);
}

}  // namespace teeny
