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
  // FP8 (E4M3) weights (skinny kernel, W8 variant): W is one byte per element, value = decode(byte) * scale of its group
  const float* w_scale;       // 1 scale (w_scale_kind 0), N scales (1: per weight row) or [N][ceil(K / group)] (2)
  int w_scale_kind;
  int w_group;                // w_scale_kind 2: elements of k per scale, a multiple of 64
  unsigned w_mul16;           // the constant 16, in a register (see e4m3x4_to_bf16x4)
  // F8 variant: the activations come as two FP8 (E4M3) terms per element, x = (hi + lo / 16) * x_scale[row]; the tensor
  // map covers both, the rows of the lo term x_lo_row rows behind those of the hi term
  const float* x_scale;
  int x_lo_row;
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

// The four K=16 steps of a 64-deep product as one block of straight-line code, D[tmem] (+)= A * B with B in shared
// memory and A in shared memory (SS) or tensor memory (TS).  Per step the address field of a K-major shared-memory
// descriptor advances by 2 (16 k = 32 bytes inside the swizzled row), that of an MN-major one by 128 (two 8-row groups
// of 1024 bytes), a tensor-memory A by 8 columns (16 bf16 as pairs); the steps are compile-time immediates because a
// lone thread that computes addresses between its tcgen05.mma issues one only every ~100 cycles.
template <int A_STEP, int B_STEP>
__device__ __forceinline__ void umma_bf16_ss_x4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                uint32_t accumulate_first) {
  asm volatile(
      "{\n\t.reg .pred p, t;\n\t.reg .b64 a, b;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "setp.eq.b32 t, %3, %3;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "add.u64 a, %1, %5;\n\t add.u64 b, %2, %6;\n\t tcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, t;\n\t"
      "add.u64 a, %1, %7;\n\t add.u64 b, %2, %8;\n\t tcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, t;\n\t"
      "add.u64 a, %1, %9;\n\t add.u64 b, %2, %10;\n\t tcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, t;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate_first), "n"(A_STEP), "n"(B_STEP), "n"(2 * A_STEP),
        "n"(2 * B_STEP), "n"(3 * A_STEP), "n"(3 * B_STEP)
      : "memory");
}
// The same for kind::f8f6f4 with both operands FP8 (E4M3) in shared memory: four K = 32 steps over 128 k, 32 bytes each.
__device__ __forceinline__ void umma_f8_ss_x4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                              uint32_t accumulate_first) {
  asm volatile(
      "{\n\t.reg .pred p, t;\n\t.reg .b64 a, b;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "setp.eq.b32 t, %3, %3;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t"
      "add.u64 a, %1, 2;\n\t add.u64 b, %2, 2;\n\t tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], a, b, %3, t;\n\t"
      "add.u64 a, %1, 4;\n\t add.u64 b, %2, 4;\n\t tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], a, b, %3, t;\n\t"
      "add.u64 a, %1, 6;\n\t add.u64 b, %2, 6;\n\t tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], a, b, %3, t;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate_first)
      : "memory");
}
template <int B_STEP>
__device__ __forceinline__ void umma_bf16_ts_x4(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                                uint32_t accumulate_first) {
  asm volatile(
      "{\n\t.reg .pred p, t;\n\t.reg .b64 b;\n\t.reg .b32 a;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "setp.eq.b32 t, %3, %3;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      "add.u32 a, %1, 8;\n\t add.u64 b, %2, %5;\n\t tcgen05.mma.cta_group::1.kind::f16 [%0], [a], b, %3, t;\n\t"
      "add.u32 a, %1, 16;\n\t add.u64 b, %2, %6;\n\t tcgen05.mma.cta_group::1.kind::f16 [%0], [a], b, %3, t;\n\t"
      "add.u32 a, %1, 24;\n\t add.u64 b, %2, %7;\n\t tcgen05.mma.cta_group::1.kind::f16 [%0], [a], b, %3, t;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate_first), "n"(B_STEP), "n"(2 * B_STEP), "n"(3 * B_STEP)
      : "memory");
}

// One k-block of MMAs: four K=16 steps over the 64-wide stage.
template <int BN, bool Q_MN_MAJOR>
__device__ __forceinline__ void issue_kblock(uint32_t d_tmem, uint32_t sp, uint32_t sq, bool first) {
  constexpr uint32_t idesc = make_idesc_bf16(kBM, BN, false, Q_MN_MAJOR);
  const uint64_t pdesc = make_smem_desc_sw128(sp, 16, 1024);
  const uint64_t qdesc = Q_MN_MAJOR ? make_smem_desc_sw128(sq, kBK * 128, 1024) : make_smem_desc_sw128(sq, 16, 1024);
  umma_bf16_ss_x4<2, Q_MN_MAJOR ? 128 : 2>(d_tmem, pdesc, qdesc, idesc, first ? 0u : 1u);
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

// W8: the weights arrive as FP8 (E4M3) bytes.  A stage holds 16 KB of them -- 128 rows of 128 k -- next to the two
// 64-k activation tiles that go with them.  Eight warps (the four epilogue warps, idle during the main loop otherwise,
// and four more) turn each 64-k half of a stage into bf16 in registers and store it into TENSOR memory, from where the
// MMA takes it as its A operand.  Converting through shared memory instead (bytes in, bf16 tile out, tile read by the
// MMA) costs six bytes of shared-memory traffic per weight byte, more than the SM has at the rate HBM delivers the
// bytes -- that version ran no faster than the bf16 kernel; this one reads every weight byte from shared memory once.
// F8 (with W8): the activations are FP8 as well -- every element split beforehand into two E4M3 terms, which represent
// a bf16 value exactly over twelve binades below its row's maximum (split_e4m3 in gemm_w8a16.cu) -- so the weight bytes
// are the MMA's A operand as TMA delivered them (kind::f8f6f4, K = 32 per instruction) and nothing is converted: two
// products per stage half, W * hi and W * lo, into two accumulators that the epilogue combines.
template <int BN, bool W8 = false, bool F8 = false>
struct SkinnyCfg {
  static_assert(W8 || !F8, "F8 activations go with FP8 weights");
  static constexpr int kKB = W8 ? 2 * kBK : kBK;       // k per stage
  static constexpr int kStageP = kBM * kBK * 2;        // 16 KB of weights either way
  static constexpr int kStageQ = BN * kKB * 2;
  static constexpr int kStageBytes = kStageP + kStageQ;
  // As many stages as let two CTAs share an SM (about 100 KB each): what streams the weights fast is the number of
  // bytes in flight per SM, and two short-lived CTAs overlap each other's set-up and reduction.
  static constexpr int kStages = W8 ? (BN <= 16 ? 5 : (BN <= 32 ? 4 : (BN <= 64 ? 3 : 2)))
                                    : ((BN <= 32) ? 5 : (BN <= 64 ? 4 : 3));
  static constexpr int kPartialBytes = BN * kBM * 4;  // f32 partial tile, column-major [BN][128]; reuses the ring
  static_assert(kPartialBytes <= kStages * kStageBytes, "partial tile must fit in the stage ring");
  // W8: 64 k of 128 weight rows as bf16 pairs are 32 columns of tensor memory; four such tiles behind the accumulator
  static constexpr int kABufs = (W8 && !F8) ? 4 : 0;
  static constexpr int kAccCols = BN < 32 ? 32 : BN;
  static constexpr int kTmemA = 128;                   // first column of the weight tiles
  static constexpr int kTmemCols = F8 ? (BN <= 64 ? 128 : 256) : (W8 ? 256 : kAccCols);
  // W8: four more warps behind the epilogue warps, all eight convert (a lone warp per scheduler cannot hide the latency
  // of its own dependent bit operations); only the first four run the epilogue
  static constexpr int kConvWarps = (W8 && !F8) ? 8 : 0;
  // W8: one thread issues a tcgen05.mma only every ~90 cycles, and a 64-k block of FP8 weights is half the bytes of a
  // bf16 one for the same four instructions: two issuing threads (a second MMA warp behind the converting warps), one
  // per half of a stage, each with its own accumulator (the epilogue adds the two); BN = 128 has no columns left for a
  // second accumulator and keeps one issuer
  static constexpr int kIssuers = (W8 && !F8 && BN <= 64) ? 2 : 1;
  static constexpr int kAcc1 = (F8 && BN > 64) ? 128 : 64;  // first column of the second accumulator (F8: of the lo products)
  static constexpr bool kTwoAcc = kIssuers == 2 || F8;
  static constexpr int kThreads = (W8 && !F8) ? 64 + 32 * kConvWarps + (kIssuers == 2 ? 32 : 0) : kNumThreads;
  static_assert(F8 || (kTmemA + kABufs * 32 <= 256 && kAccCols <= kTmemA && (kIssuers == 1 || kAcc1 + kAccCols <= kTmemA)),
                "accumulators and weight tiles share the allocation");
  static_assert(!F8 || kAcc1 + kAccCols <= kTmemCols, "two accumulators share the allocation");
  static constexpr int kBarOffset = kStages * kStageBytes;
  static constexpr int kSmemBytes = kBarOffset + 1024 + 256;
};

// Four FP8 E4M3 bytes (k ascending from the low byte) -> two bf16 pairs, exactly.  A byte's seven magnitude bits,
// placed four bits below the top of a bf16's exponent field, read as the bf16 number 2^-120 times the E4M3 value --
// also for E4M3 subnormals, which land on bf16 subnormals -- so one multiplication by 2^120 finishes the job.  (The two
// NaN bytes 0x7f / 0xff decode as +-480; the loader refuses tensors that contain them.)
// The conversion is what bounds this kernel, and the integer pipe (logic, shifts, byte permutes: half the rate of the
// FMA pipe) is what bounds the conversion.  So the placement is done by integer multiply-adds, which run on the FMA
// pipe: with the byte in the low half of a halfword (one permute), x * 16 puts the magnitude at bits 10..4 and the sign
// at bit 11, and adding 240 * (x & 0x80) carries the sign from bit 11 to bit 15 without touching the rest.  `mul16`
// is the constant 16 handed in through a register, so that the compiler keeps the multiply-add instead of turning it
// into a shift on the integer pipe.
__device__ __forceinline__ void e4m3x4_to_bf16x4(uint32_t w, uint32_t mul16, uint32_t& lo, uint32_t& hi) {
  const uint32_t x0 = __byte_perm(w, 0u, 0x4140), x1 = __byte_perm(w, 0u, 0x4342);
  const uint32_t s0 = x0 & 0x00800080u, s1 = x1 & 0x00800080u;
  uint32_t t0, t1;
  asm("mad.lo.u32 %0, %1, %2, 0;\n\tmad.lo.u32 %0, %3, 240, %0;" : "=&r"(t0) : "r"(x0), "r"(mul16), "r"(s0));
  asm("mad.lo.u32 %0, %1, %2, 0;\n\tmad.lo.u32 %0, %3, 240, %0;" : "=&r"(t1) : "r"(x1), "r"(mul16), "r"(s1));
  const __nv_bfloat162 k = __halves2bfloat162(__ushort_as_bfloat16(0x7b80), __ushort_as_bfloat16(0x7b80));  // 2^120
  const __nv_bfloat162 r0 = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&t0), k);
  const __nv_bfloat162 r1 = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&t1), k);
  lo = *reinterpret_cast<const uint32_t*>(&r0);
  hi = *reinterpret_cast<const uint32_t*>(&r1);
}

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
template <int BN, bool W8 = false, bool F8 = false>
__global__ void __launch_bounds__((SkinnyCfg<BN, W8, F8>::kThreads), 2)
gemm_bf16_skinny_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                        const GemmArgs args) {
  using Cfg = SkinnyCfg<BN, W8, F8>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  // The partial tile is written after the last MMA has completed, i.e. when no stage is in use any more, so it
  // lives at the start of the ring.
  const uint32_t part_base = smem_base;
  const uint32_t bar_base = smem_base + Cfg::kBarOffset;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (Cfg::kStages + s); };
  const uint32_t acc_full_bar = bar_base + 8u * (2 * Cfg::kStages);
  const uint32_t tmem_slot = acc_full_bar + 8;
  auto wfull_bar = [&](int b) { return acc_full_bar + 16u + 8u * b; };   // W8: weight tile b is in tensor memory
  auto wempty_bar = [&](int b) { return acc_full_bar + 48u + 8u * b; };  // W8: the MMAs that read tile b are done
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  float* part_gen = reinterpret_cast<float*>(smem_gen);
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(
      smem_gen + Cfg::kBarOffset + 8 * (2 * Cfg::kStages + 1));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int* err = args.err;
  const uint32_t S = cluster_size(), rank = cluster_rank();
  const int tile = blockIdx.y;
  const int kb0 = static_cast<int>(rank) * args.kb_per_split;
  const int kb1 = min(args.k_blocks, kb0 + args.kb_per_split);
  // W8: what the accumulator of weight row n is multiplied by on the way out (per-group scales are already in the
  // converted weights)
  auto row_scale = [&](int n) -> float {
    if constexpr (!W8) return 1.0f;
    if (args.w_scale_kind == 0) return __ldg(args.w_scale);
    return (args.w_scale_kind == 1 && n < args.N) ? __ldg(args.w_scale + n) : 1.0f;
  };

  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmap_w);
    tma_prefetch_desc(&tmap_x);
    for (int s = 0; s < Cfg::kStages; ++s) {
      mbar_init(full_bar(s), 1);
      // W8: a stage is free when the MMAs are done with its activation tile and the four converting warps with its bytes
      mbar_init(empty_bar(s), Cfg::kIssuers + Cfg::kConvWarps);
    }
    mbar_init(acc_full_bar, Cfg::kIssuers);
    if constexpr (W8 && !F8) {
      for (int b = 0; b < Cfg::kABufs; ++b) {
        mbar_init(wfull_bar(b), Cfg::kConvWarps / 2);  // a tile is written by one group of four warps
        mbar_init(wempty_bar(b), 1);
      }
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

  if (warp == 0) {
    if (lane == 0) {
      // Weights are never written by a kernel of the stream, so the first ring of weight tiles is requested while
      // the previous kernel may still be running; the activation tiles follow once it has finished.
      const int pre = min(kb1 - kb0, Cfg::kStages);
      for (int i = 0; i < pre; ++i) {
        mbar_expect_tx(full_bar(i), Cfg::kStageBytes);
        tma_load_2d(smem_base + i * Cfg::kStageBytes, &tmap_w, full_bar(i), (kb0 + i) * Cfg::kKB, tile * kBM);
      }
      // ... and the weight tiles behind them are asked into L2, so that HBM keeps streaming this kernel's weights for
      // as long as the predecessor's tail lasts, not just until the ring is full
      for (int kb = kb0 + pre; kb < min(kb1, kb0 + pre + args.l2_ahead); ++kb)
        tma_prefetch_l2_2d(&tmap_w, kb * Cfg::kKB, tile * kBM);
      pdl_wait();
      auto load_x = [&](uint32_t sq, uint32_t bar, int kb) {  // the activation tile(s) of one stage: 64 k each
        tma_load_2d(sq, &tmap_x, bar, kb * Cfg::kKB, 0);
        if constexpr (F8) tma_load_2d(sq + BN * kBK * 2, &tmap_x, bar, kb * Cfg::kKB, args.x_lo_row);  // the lo terms
        else if constexpr (W8) tma_load_2d(sq + BN * kBK * 2, &tmap_x, bar, kb * Cfg::kKB + kBK, 0);
      };
      for (int i = 0; i < pre; ++i) load_x(smem_base + i * Cfg::kStageBytes + Cfg::kStageP, full_bar(i), kb0 + i);
      int stage = pre == Cfg::kStages ? 0 : pre;
      uint32_t phase = pre == Cfg::kStages ? 1 : 0;
      for (int kb = kb0 + pre; kb < kb1; ++kb) {
        if (!mbar_wait(empty_bar(stage), phase ^ 1, err, DEVERR_GEMM_PRODUCER)) break;
        const uint32_t sp = smem_base + stage * Cfg::kStageBytes;
        mbar_expect_tx(full_bar(stage), Cfg::kStageBytes);
        tma_load_2d(sp, &tmap_w, full_bar(stage), kb * Cfg::kKB, tile * kBM);
        load_x(sp + Cfg::kStageP, full_bar(stage), kb);
        if (++stage == Cfg::kStages) { stage = 0; phase ^= 1; }
      }
    } else {
      pdl_wait();
    }
  } else if (warp == 1 || (Cfg::kIssuers == 2 && warp == 2 + Cfg::kConvWarps)) {
    pdl_wait();
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      TRACE_ONLY(long long m_full = 0, m_wfull = 0, m_issue = 0, c0; const long long m_begin = clock64();)
      // W8 with two issuers: warp 1 takes half 0 of every stage into the first accumulator, the other MMA warp half 1
      // into the second
      const int h_first = (W8 && warp != 1) ? 1 : 0, h_step = Cfg::kIssuers;
      const uint32_t acc = tmem_base + ((W8 && warp != 1) ? Cfg::kAcc1 : 0);
      for (int kb = kb0; kb < kb1; ++kb) {
        TRACE_ONLY(c0 = clock64();)
        if (!mbar_wait(full_bar(stage), phase, err, DEVERR_GEMM_MMA)) { ok = false; break; }
        TRACE_ONLY(m_full += clock64() - c0;)
        const uint32_t sp = smem_base + stage * Cfg::kStageBytes;
        if constexpr (F8) {
          tc_fence_after();
          constexpr uint32_t idesc = make_idesc_e4m3(kBM, BN);
          const uint64_t wdesc = make_smem_desc_sw128(sp, 16, 1024);
          const uint64_t hdesc = make_smem_desc_sw128(sp + Cfg::kStageP, 16, 1024);
          const uint64_t ldesc = make_smem_desc_sw128(sp + Cfg::kStageP + BN * kBK * 2, 16, 1024);
          // 128 k of the stage = four K = 32 steps of 32 bytes (+2 in both address fields); hi products, then lo
          umma_f8_ss_x4(tmem_base, wdesc, hdesc, idesc, kb == kb0 ? 0u : 1u);
          umma_f8_ss_x4(tmem_base + Cfg::kAcc1, wdesc, ldesc, idesc, kb == kb0 ? 0u : 1u);
        } else if constexpr (W8) {
          for (int h = h_first; h < 2; h += h_step) {
            const int q = 2 * (kb - kb0) + h, j = q & 3;  // the q-th 64-k block goes through weight tile q % 4
            TRACE_ONLY(c0 = clock64();)
            if (!mbar_wait(wfull_bar(j), (q >> 2) & 1, err, DEVERR_GEMM_MMA)) { ok = false; break; }
            TRACE_ONLY(m_wfull += clock64() - c0; c0 = clock64();)
            tc_fence_after();
            constexpr uint32_t idesc = make_idesc_bf16(kBM, BN, false, false);
            const uint64_t xdesc = make_smem_desc_sw128(sp + Cfg::kStageP + h * BN * kBK * 2, 16, 1024);
            const uint32_t a_tmem = tmem_base + Cfg::kTmemA + j * 32;
            umma_bf16_ts_x4<2>(acc, a_tmem, xdesc, idesc, q >= h_step ? 1u : 0u);  // an issuer's first block overwrites
            umma_commit(wempty_bar(j));
            TRACE_ONLY(m_issue += clock64() - c0;)
          }
          if (!ok) break;
        } else {
          tc_fence_after();
          issue_kblock<BN, false>(tmem_base, sp, sp + Cfg::kStageP, kb == kb0);
        }
        umma_commit(empty_bar(stage));
        if (++stage == Cfg::kStages) { stage = 0; phase ^= 1; }
      }
      if (ok) umma_commit(acc_full_bar);
      TRACE_VALUE(0, W8 && blockIdx.y == 0 && warp == 1, clock64() - m_begin);
      TRACE_VALUE(1, W8 && blockIdx.y == 0 && warp == 1, m_full);
      TRACE_VALUE(2, W8 && blockIdx.y == 0 && warp == 1, m_wfull);
      TRACE_VALUE(3, W8 && blockIdx.y == 0 && warp == 1, m_issue);
    }
  } else {
    pdl_wait();
    if constexpr (W8 && !F8) {
      // ---- main loop of the converting warps: the q-th 64-k block of weights -> weight tile q % 4 in tensor memory ----
      // Two groups of four warps: group g takes half g of every stage, so two blocks are always under way (one group's
      // loads, bit operations and tensor-memory stores overlap the other's).  A warp reaches the 32 lanes (weight rows)
      // of its quarter, warp % 4: a thread reads the 64 bytes of its row (four 16-byte chunks; the tile lies in the
      // 128-byte swizzle TMA wrote, chunk c of row r at chunk c ^ (r & 7), which also keeps a quarter warp's loads on
      // distinct banks), converts them and stores 32 columns of bf16 pairs.
      const int quarter = warp & 3, h = (warp - 2) >> 2;
      const int r = quarter * 32 + lane;
      const bool by_group = args.w_scale_kind == 2;
      const int groups_per_row = by_group ? (args.K + args.w_group - 1) / args.w_group : 0;
      const int wrow = tile * kBM + r;
      int stage = 0;
      uint32_t phase = 0;
      TRACE_ONLY(long long c_full = 0, c_empty = 0, c_conv = 0, c_sig = 0, c0; const long long c_begin = clock64();)
      for (int kb = kb0; kb < kb1; ++kb) {
        const int q = 2 * (kb - kb0) + h, j = q & 3;
        float sc = 1.0f;
        if (by_group) {  // one scale per (weight row, 64 k); requested before the wait below
          const int g = (kb * Cfg::kKB + h * kBK) / args.w_group;
          if (wrow < args.N && g < groups_per_row) sc = __ldg(args.w_scale + static_cast<size_t>(wrow) * groups_per_row + g);
        }
        TRACE_ONLY(c0 = clock64();)
        if (!mbar_wait(full_bar(stage), phase, err, DEVERR_GEMM_EPILOGUE)) break;
        TRACE_ONLY(c_full += clock64() - c0; c0 = clock64();)
        const uint8_t* row_gen = smem_gen + stage * Cfg::kStageBytes + r * 128;
        uint4 in[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) in[c] = *reinterpret_cast<const uint4*>(row_gen + (((4 * h + c) ^ (r & 7)) << 4));
        uint32_t o[32];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const uint32_t w[4] = {in[c].x, in[c].y, in[c].z, in[c].w};
#pragma unroll
          for (int e = 0; e < 4; ++e) e4m3x4_to_bf16x4(w[e], args.w_mul16, o[8 * c + 2 * e], o[8 * c + 2 * e + 1]);
        }
        if (by_group) {  // the group's scale goes into the weight: bf16(value * scale), as the large-M path stores it
#pragma unroll
          for (int e = 0; e < 32; ++e) o[e] = pack_bf16x2(bf16_lo(o[e]) * sc, bf16_hi(o[e]) * sc);
        }
        TRACE_ONLY(c_conv += clock64() - c0; c0 = clock64();)
        if (q >= 4 && !mbar_wait(wempty_bar(j), ((q >> 2) - 1) & 1, err, DEVERR_GEMM_EPILOGUE)) break;
        TRACE_ONLY(c_empty += clock64() - c0; c0 = clock64();)
        tc_fence_after();
        tmem_st_32x32(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + Cfg::kTmemA + j * 32, o);
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(wfull_bar(j));
          mbar_arrive(empty_bar(stage));
        }
        TRACE_ONLY(c_sig += clock64() - c0;)
        if (++stage == Cfg::kStages) { stage = 0; phase ^= 1; }
      }
      TRACE_VALUE(4, threadIdx.x == 64 && blockIdx.y == 0, clock64() - c_begin);
      TRACE_VALUE(5, threadIdx.x == 64 && blockIdx.y == 0, c_full);
      TRACE_VALUE(6, threadIdx.x == 64 && blockIdx.y == 0, c_empty);
      TRACE_VALUE(7, threadIdx.x == 64 && blockIdx.y == 0, c_conv);
      TRACE_VALUE(8, threadIdx.x == 64 && blockIdx.y == 0, c_sig);
    }
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    if (warp < 6 && mbar_wait(acc_full_bar, 0, err, DEVERR_GEMM_EPILOGUE)) {
      TRACE_MARK(1, threadIdx.x == 64);
      tc_fence_after();
      const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
      constexpr int kChunk = (BN >= 32) ? 32 : 16;
      const bool direct = (S == 1) && !args.swiglu;
      const int n = tile * kBM + row;
      const float bias = (direct && args.bias && n < args.N) ? __bfloat162float(args.bias[n]) : 0.0f;
      const float wsc = direct ? row_scale(n) : 1.0f;
      const unsigned stamp = (direct && args.push_recv) ? __ldcg(args.push_epoch) * 1024u + args.push_round + 1u : 0u;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += kChunk) {
        uint32_t r[kChunk];
        if constexpr (kChunk == 32) tmem_ld_32x32(t_addr + c0, r); else tmem_ld_32x16(t_addr + c0, r);
        if constexpr (Cfg::kTwoAcc) {
          // two accumulators: the two issuers' (halves 0 and halves 1 of the stages), or the hi and the lo products of the
          // F8 variant (the lo terms were stored times 16); F8 also applies the token's activation scale here
          uint32_t r1[kChunk];
          if constexpr (kChunk == 32) tmem_ld_32x32(t_addr + Cfg::kAcc1 + c0, r1); else tmem_ld_32x16(t_addr + Cfg::kAcc1 + c0, r1);
          tmem_wait_ld();
#pragma unroll
          for (int e = 0; e < kChunk; ++e) {
            if constexpr (F8) {
              const float xs = (c0 + e < args.M) ? __ldg(args.x_scale + c0 + e) : 0.0f;
              r[e] = __float_as_uint(fmaf(__uint_as_float(r1[e]), 0.0625f, __uint_as_float(r[e])) * xs);
            } else {
              r[e] = __float_as_uint(__uint_as_float(r[e]) + __uint_as_float(r1[e]));
            }
          }
        }
        tmem_wait_ld();
        if (direct) {
          // the whole K range was this CTA's: registers -> global, a warp's 32 rows side by side in each token row
          if (n < args.N) {
#pragma unroll
            for (int e = 0; e < kChunk; ++e) {
              const int c = c0 + e;
              if (c < args.M) {
                const float v = W8 ? fmaf(__uint_as_float(r[e]), wsc, bias) : __uint_as_float(r[e]) + bias;
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

  if (warp >= 2 && warp < 6 && reduce) {
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
        if constexpr (W8) {  // gate rows of this tile are weight rows tile * 128 + [0, 64), up rows the 64 behind them
          const int wr = tile * kBM + 4 * j;
          gs.x *= row_scale(wr); gs.y *= row_scale(wr + 1); gs.z *= row_scale(wr + 2); gs.w *= row_scale(wr + 3);
          us.x *= row_scale(wr + 64); us.y *= row_scale(wr + 65); us.z *= row_scale(wr + 66); us.w *= row_scale(wr + 67);
        }
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
          if constexpr (W8) {
#pragma unroll
            for (int e = 0; e < 4; ++e) o[e] *= row_scale(n + e);
          }
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

template <int BN, bool W8 = false, bool F8 = false>
int prepare_skinny() {
  static std::atomic<unsigned long long> done{0};  // one bit per device; threads may race to set it
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 64 && (done.load(std::memory_order_acquire) >> dev) & 1ull) return 0;
  cudaError_t e = cudaFuncSetAttribute(gemm_bf16_skinny_kernel<BN, W8, F8>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       SkinnyCfg<BN, W8, F8>::kSmemBytes);
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

template <int BN, bool W8 = false, bool F8 = false>
int launch_skinny(const CUtensorMap& tw, const CUtensorMap& tx, const GemmArgs& a, int split, int tiles,
                  cudaStream_t st) {
  const int rc = prepare_skinny<BN, W8, F8>();
  if (rc) return rc;
  return launch_kernel(gemm_bf16_skinny_kernel<BN, W8, F8>, dim3(split, tiles, 1),
                       dim3(SkinnyCfg<BN, W8, F8>::kThreads, 1, 1), SkinnyCfg<BN, W8, F8>::kSmemBytes, st,
                       static_cast<unsigned>(split), tw, tx, a);
}

// Cluster width (K split) of the skinny kernel for `tiles` 128-row weight tiles.
int skinny_split(int tiles, int k_blocks, int sms) {
  const int slots = sms * 2;
  int split = (slots * 85 / 100) / tiles;
  if (split > 8) split = 8;
  {  // TEENY_SKINNY_SPLIT: fixed cluster width, for measurements
    static const int forced = [] { const char* e = getenv("TEENY_SKINNY_SPLIT"); return e ? atoi(e) : 0; }();
    if (forced > 0 && forced <= 8) split = forced;
  }
  while (split > 1 && (ceil_div(k_blocks, split) < 4 || ceil_div(k_blocks, split) * (split - 1) >= k_blocks))
    --split;  // too thin, or a rank would be left without k-blocks
  return split < 1 ? 1 : split;
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
  if ((rc = prepare_skinny<128>())) return rc;
  if ((rc = prepare_skinny<16, true>())) return rc;
  if ((rc = prepare_skinny<32, true>())) return rc;
  if ((rc = prepare_skinny<64, true>())) return rc;
  if ((rc = prepare_skinny<128, true>())) return rc;
  if ((rc = prepare_skinny<16, true, true>())) return rc;
  if ((rc = prepare_skinny<32, true, true>())) return rc;
  if ((rc = prepare_skinny<64, true, true>())) return rc;
  return prepare_skinny<128, true, true>();
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
      const int split = skinny_split(tiles, a.k_blocks, sms);
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

// Y[M, N] = X[M, K] (bf16) * dequant(Wq[N, K])^T for M <= 128: the skinny kernel's W8 variant at every N (one CTA per
// weight tile where the tiles alone fill the GPU).
int gemm_w8a16_skinny(const bf16* x, int ldx, const uint8_t* wq, int ldw, const float* w_scale, int scale_kind,
                      int group, const bf16* bias, bf16* y, int ldy, int M, int N, int K, cudaStream_t stream, bool swiglu,
                      const GemmPush* push) {
  if (!x || !wq || !w_scale || !y || M <= 0 || M > kSwapMaxM || N <= 0 || K <= 0) return TEENY_ERR_BAD_ARG;
  if (scale_kind < 0 || scale_kind > 2 || (scale_kind == 2 && (group <= 0 || group % kBK != 0))) return TEENY_ERR_BAD_ARG;
  if (swiglu && (bias || N % 128 != 0)) return TEENY_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(wq) & 15) || (ldx & 7) || (ldw & 15))
    return TEENY_ERR_ALIGNMENT;
  GemmArgs a{};
  a.M = M; a.N = N; a.K = K; a.ldy = ldy; a.y = y; a.bias = bias;
  a.k_blocks = ceil_div(K, 2 * kBK);  // a stage of the W8 variant is 128 k wide
  a.swiglu = swiglu ? 1 : 0;
  a.w_scale = w_scale; a.w_scale_kind = scale_kind; a.w_group = group; a.w_mul16 = 16u;
  if (push) {
    if (swiglu || !push->recv || !push->epoch || push->world < 2 || push->round >= 1023) return TEENY_ERR_BAD_ARG;
    a.push_recv = push->recv;
    a.push_epoch = push->epoch;
    a.push_round = push->round;
    a.push_world = push->world;
    a.push_owner_rows = push->owner_rows;
  }
  a.err = device_error_word();
  if (!a.err) return TEENY_ERR_DRIVER;
  const int bn = swap_bn(M);
  CUtensorMap tmx, tmw;
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(M)};
    const uint64_t strides[1] = {static_cast<uint64_t>(ldx) * 2};
    const uint32_t box[2] = {kBK, static_cast<uint32_t>(bn)};
    const int rc = encode_tensor_map_bf16(&tmx, x, 2, dims, strides, box);
    if (rc) return rc;
  }
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(N)};
    const uint64_t strides[1] = {static_cast<uint64_t>(ldw)};
    const uint32_t box[2] = {2 * kBK, kBM};
    const int rc = encode_tensor_map_u8(&tmw, wq, 2, dims, strides, box);
    if (rc) return rc;
  }
  const int tiles = ceil_div(N, kBM);
  if (tiles > 65535) return TEENY_ERR_BAD_ARG;
  const int split = skinny_split(tiles, a.k_blocks, sm_count());
  a.kb_per_split = ceil_div(a.k_blocks, split);
  a.l2_ahead = 0;
  switch (bn) {
    case 16: return launch_skinny<16, true>(tmw, tmx, a, split, tiles, stream);
    case 32: return launch_skinny<32, true>(tmw, tmx, a, split, tiles, stream);
    case 64: return launch_skinny<64, true>(tmw, tmx, a, split, tiles, stream);
    default: return launch_skinny<128, true>(tmw, tmx, a, split, tiles, stream);
  }
}

// The same with the activations already split into two FP8 terms (split_e4m3): x8 = [2 * M, K] bytes (hi rows, then lo
// rows; row stride ldx8 bytes), x_scale[M].  Nothing is converted inside: kind::f8f6f4 on the bytes as they are.
int gemm_w8a8x2_skinny(const uint8_t* x8, int ldx8, const float* x_scale, const uint8_t* wq, int ldw, const float* w_scale,
                       int scale_kind, const bf16* bias, bf16* y, int ldy, int M, int N, int K, cudaStream_t stream,
                       bool swiglu, const GemmPush* push) {
  if (!x8 || !x_scale || !wq || !w_scale || !y || M <= 0 || M > kSwapMaxM || N <= 0 || K <= 0) return TEENY_ERR_BAD_ARG;
  if (scale_kind < 0 || scale_kind > 1) return TEENY_ERR_BAD_ARG;  // per-group weight scales need the converting variant
  if (swiglu && (bias || N % 128 != 0)) return TEENY_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(x8) & 15) || (reinterpret_cast<uintptr_t>(wq) & 15) || (ldx8 & 15) || (ldw & 15))
    return TEENY_ERR_ALIGNMENT;
  GemmArgs a{};
  a.M = M; a.N = N; a.K = K; a.ldy = ldy; a.y = y; a.bias = bias;
  a.k_blocks = ceil_div(K, 2 * kBK);
  a.swiglu = swiglu ? 1 : 0;
  a.w_scale = w_scale; a.w_scale_kind = scale_kind; a.w_group = 0; a.w_mul16 = 16u;
  a.x_scale = x_scale; a.x_lo_row = M;
  if (push) {
    if (swiglu || !push->recv || !push->epoch || push->world < 2 || push->round >= 1023) return TEENY_ERR_BAD_ARG;
    a.push_recv = push->recv;
    a.push_epoch = push->epoch;
    a.push_round = push->round;
    a.push_world = push->world;
    a.push_owner_rows = push->owner_rows;
  }
  a.err = device_error_word();
  if (!a.err) return TEENY_ERR_DRIVER;
  const int bn = swap_bn(M);
  CUtensorMap tmx, tmw;
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(2 * M)};
    const uint64_t strides[1] = {static_cast<uint64_t>(ldx8)};
    const uint32_t box[2] = {2 * kBK, static_cast<uint32_t>(bn)};
    const int rc = encode_tensor_map_u8(&tmx, x8, 2, dims, strides, box);
    if (rc) return rc;
  }
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(N)};
    const uint64_t strides[1] = {static_cast<uint64_t>(ldw)};
    const uint32_t box[2] = {2 * kBK, kBM};
    const int rc = encode_tensor_map_u8(&tmw, wq, 2, dims, strides, box);
    if (rc) return rc;
  }
  const int tiles = ceil_div(N, kBM);
  if (tiles > 65535) return TEENY_ERR_BAD_ARG;
  const int split = skinny_split(tiles, a.k_blocks, sm_count());
  a.kb_per_split = ceil_div(a.k_blocks, split);
  switch (bn) {
    case 16: return launch_skinny<16, true, true>(tmw, tmx, a, split, tiles, stream);
    case 32: return launch_skinny<32, true, true>(tmw, tmx, a, split, tiles, stream);
    case 64: return launch_skinny<64, true, true>(tmw, tmx, a, split, tiles, stream);
    default: return launch_skinny<128, true, true>(tmw, tmx, a, split, tiles, stream);
  }
}

}  // namespace teeny
