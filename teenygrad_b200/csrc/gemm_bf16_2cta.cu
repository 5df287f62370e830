// bf16 GEMM, large-M path: Y[M, N] = X[M, K] W[N, K]^T on CTA pairs (tcgen05 cta_group::2).
//
// Two CTAs of a cluster -- two neighbouring SMs -- compute one 256 x 256 output tile.  Each CTA loads only ITS half
// of both operands per k-block (128 rows of X, 128 rows of W, 64 k: 32 KB), so per SM the shared-memory fill and the
// L2 traffic are two thirds of what a lone 128 x 256 tile needs, and the ring holds six stages instead of four.  The
// leader CTA (cluster rank 0) issues every tcgen05.mma for the pair: the instruction reads rows 0-127 of A and of B
// from the leader's shared memory and rows 128-255 from the peer's (same offsets), and writes output rows 0-127 to
// the leader's tensor memory and rows 128-255 to the peer's.  No multicast loads: each CTA's TMA fetches its own
// half; only the completion (tcgen05.commit) is delivered to both CTAs' barriers.
//
//   warp 0   TMA producer (both CTAs).  Transaction bytes of both CTAs land on the leader's `full` barrier.
//   warp 1   MMA issuer (leader only).  commit -> `empty` barrier of both CTAs; after the last k-block -> `acc_full`
//            of both CTAs.
//   warp 2   allocates / frees tensor memory (both CTAs, cta_group::2).
//   warps 2-5 epilogue (both CTAs): tcgen05.ld the CTA's 128 x 256 f32 half, bf16, 16-byte stores; then arrive on
//            the leader's `acc_empty` (the peer does so through a cluster-mapped address).
// Two accumulators in tensor memory (2 x 256 columns) let the epilogue of tile t overlap the main loop of tile t+1.
#include <atomic>

#include "common.cuh"
#include "kernels.h"

namespace teeny {

namespace {

constexpr int kBM = 128;      // rows per CTA (pair: 256)
constexpr int kBNh = 128;     // W rows loaded per CTA (pair: 256)
constexpr int kBN = 256;
constexpr int kBK = 64;
constexpr int kStages = 6;
constexpr int kStageA = kBM * kBK * 2;
constexpr int kStageB = kBNh * kBK * 2;
constexpr int kStageBytes = kStageA + kStageB;   // 32 KB per CTA
constexpr int kThreads = 192;
constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 256;
constexpr uint32_t kPeerBitMask = 0xFEFFFFFFu;   // clears the CTA-rank bit of a shared::cluster address -> leader

struct Args2 {
  int M, N, K, ldy;
  bf16* y;
  const bf16* bias;
  int tiles_m, tiles_n;   // 256 x 256 tiles
  int k_blocks;
  int group;
  int swiglu;             // W rows interleave 64 gate / 64 up channels; Y[M, N/2] = silu(gate) * up
  int qkv;                // the fused QKV projection with head norms, rotary embedding and cache fill in the epilogue
  QkvEpilogue f;
  int* err;
};

__device__ __forceinline__ uint32_t cluster_rank2() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync2() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t map_to_rank(uint32_t local_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// This CTA's half tile; completion bytes are credited to the LEADER's barrier at the same offset.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* m, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar & kPeerBitMask), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void umma_bf16_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                  uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives on the barrier at this offset in BOTH CTAs of the pair once all MMAs issued so far have completed.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(bar), "h"(static_cast<uint16_t>(3))
      : "memory");
}

// SwiGLU with the rounding points of the unfused bf16 graph (both projections, silu, product).
__device__ __forceinline__ float swiglu2_f(float gate_acc, float up_acc) {
  const float g = bf16_round(gate_acc), u = bf16_round(up_acc);
  return bf16_round(g * (1.0f / (1.0f + expf(-g)))) * u;
}

__device__ __forceinline__ void tile_coords2(int tile, int tiles_m, int tiles_n, int group, int& tm, int& tn) {
  const int per_group = group * tiles_n;
  const int g = tile / per_group;
  const int first = g * group;
  const int size = min(group, tiles_m - first);
  const int r = tile - g * per_group;
  tm = first + r % size;
  tn = r / size;
}

__global__ void __launch_bounds__(kThreads, 1)
gemm_bf16_2cta_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
                      const Args2 args) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar_base = smem_base + kStages * kStageBytes;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
  auto acc_full_bar = [&](int b) { return bar_base + 8u * (2 * kStages + b); };
  auto acc_empty_bar = [&](int b) { return bar_base + 8u * (2 * kStages + 2 + b); };
  const uint32_t tmem_slot = bar_base + 8u * (2 * kStages + 4);
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  volatile uint32_t* tmem_slot_ptr =
      reinterpret_cast<volatile uint32_t*>(smem_gen + kStages * kStageBytes + 8 * (2 * kStages + 4));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank2();
  const bool leader = rank == 0;
  int* err = args.err;

  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmap_x);
    tma_prefetch_desc(&tmap_w);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full_bar(s), 1);    // leader's producer arms it; both CTAs' copies complete on it
      mbar_init(empty_bar(s), 1);   // one commit per use
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full_bar(b), 1);
      mbar_init(acc_empty_bar(b), 8);  // four epilogue warps in each CTA of the pair
    }
    mbar_fence_init();
  }
  if (warp == 2) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync2();  // both CTAs' barriers exist before either CTA can signal the other
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;
  pdl_wait();

  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int num_tiles = args.tiles_m * args.tiles_n;

  if (warp == 0) {
    // ---------------- TMA producer (both CTAs) ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = pair; ok && t < num_tiles; t += n_pairs) {
        int tm, tn;
        tile_coords2(t, args.tiles_m, args.tiles_n, args.group, tm, tn);
        const int row_x = tm * 256 + static_cast<int>(rank) * kBM;
        const int row_w = tn * 256 + static_cast<int>(rank) * kBNh;
        for (int kb = 0; kb < args.k_blocks; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1, err, DEVERR_GEMM_PRODUCER)) { ok = false; break; }
          const uint32_t sa = smem_base + stage * kStageBytes;
          if (leader) mbar_expect_tx(full_bar(stage), 2 * kStageBytes);  // both CTAs' halves
          tma_load_2d_pair(sa, &tmap_x, full_bar(stage), kb * kBK, row_x);
          tma_load_2d_pair(sa + kStageA, &tmap_w, full_bar(stage), kb * kBK, row_w);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader CTA only) ----------------
    if (leader && lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(256, kBN, false, false);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int local = 0;
      for (int t = pair; ok && t < num_tiles; t += n_pairs, ++local) {
        const int buf = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1;
        if (!mbar_wait(acc_empty_bar(buf), acc_phase ^ 1, err, DEVERR_GEMM_MMA)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * kBN;
        for (int kb = 0; kb < args.k_blocks; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, err, DEVERR_GEMM_MMA)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_base + stage * kStageBytes;
          const uint64_t adesc = make_smem_desc_sw128(sa, 16, 1024);
          const uint64_t bdesc = make_smem_desc_sw128(sa + kStageA, 16, 1024);
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k)
            umma_bf16_ss_pair(d_tmem, adesc + static_cast<uint64_t>(k * 2), bdesc + static_cast<uint64_t>(k * 2), idesc,
                              (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit_pair(empty_bar(stage));
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit_pair(acc_full_bar(buf));
      }
    }
  } else {
    // ---------------- epilogue (both CTAs; TMEM lane quarter = warp % 4) ----------------
    const int quarter = warp & 3;
    const int row_in_half = quarter * 32 + lane;
    const uint32_t acc_empty_leader0 = map_to_rank(acc_empty_bar(0), 0), acc_empty_leader1 = map_to_rank(acc_empty_bar(1), 0);
    bool ok = true;
    int local = 0;
    for (int t = pair; ok && t < num_tiles; t += n_pairs, ++local) {
      int tm, tn;
      tile_coords2(t, args.tiles_m, args.tiles_n, args.group, tm, tn);
      const int buf = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      const int row = tm * 256 + static_cast<int>(rank) * kBM + row_in_half;
      // fused QKV epilogue: the token's rotary rows are requested before the wait for the accumulator, so their latency
      // is gone by the time they are used.  cos[d + 64] == cos[d] (the angles are cat(freqs, freqs)): 64 values each.
      uint4 rope_c[8], rope_s[8];
      if (args.qkv && row < args.M) {
        const int pos = args.f.pos0 + row % args.f.S;
        const uint4* c4 = reinterpret_cast<const uint4*>(args.f.cos_t + static_cast<size_t>(pos) * 128);
        const uint4* s4 = reinterpret_cast<const uint4*>(args.f.sin_t + static_cast<size_t>(pos) * 128);
#pragma unroll
        for (int v = 0; v < 8; ++v) {
          rope_c[v] = __ldg(c4 + v);
          rope_s[v] = __ldg(s4 + v);
        }
      }
      if (!mbar_wait(acc_full_bar(buf), acc_phase, err, DEVERR_GEMM_EPILOGUE)) { ok = false; break; }
      tc_fence_after();
      const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * kBN;
      if (args.qkv) {
        // Each 128-column half of the tile is one head of the fused [q | k | v] projection and a thread holds the whole
        // head of its token: per-head RMSNorm (q, k), rotate-half rotary embedding at the token's position (q, k), then
        // q goes back into the projection buffer and k / v straight into the caches -- the rounding points are those of
        // the separate kernel (head_norm_rope, common.cuh): the projection, the normed head, each product and the sum
        // are bf16 tensors.
        const QkvEpilogue& f = args.f;
        const int seq = row / f.S, pos = f.pos0 + row % f.S;
#pragma unroll 1
        for (int hh = 0; hh < 2; ++hh) {
          const int head = tn * 2 + hh;
          if (head >= f.Hq + 2 * f.Hkv) break;  // uniform over the CTA
          uint32_t xp[64];                      // the head as bf16 pairs (the projection is a bf16 tensor)
          float sq4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t r[32];
            tmem_ld_32x32(t_addr + hh * 128 + c * 32, r);
            tmem_wait_ld();
#pragma unroll
            for (int e = 0; e < 16; ++e) {
              const uint32_t pr = pack_bf16x2(__uint_as_float(r[2 * e]), __uint_as_float(r[2 * e + 1]));
              xp[c * 16 + e] = pr;
              sq4[e & 3] = fmaf(bf16_lo(pr), bf16_lo(pr), fmaf(bf16_hi(pr), bf16_hi(pr), sq4[e & 3]));
            }
          }
          const float sq = (sq4[0] + sq4[1]) + (sq4[2] + sq4[3]);
          if (row >= args.M) continue;
          bf16* dst;
          if (head < f.Hq) {
            dst = args.y + static_cast<size_t>(row) * args.ldy + static_cast<size_t>(head) * 128;
          } else {
            const bool is_k = head < f.Hq + f.Hkv;
            const int hk = head - f.Hq - (is_k ? 0 : f.Hkv);
            dst = (is_k ? f.k_cache : f.v_cache) +
                  ((static_cast<size_t>(seq) * f.Hkv + hk) * f.max_len + pos) * 128;
          }
          uint4* dst4 = reinterpret_cast<uint4*>(dst);
          if (head >= f.Hq + f.Hkv) {  // v: no norm, no rotation
#pragma unroll
            for (int v = 0; v < 16; ++v) dst4[v] = make_uint4(xp[4 * v], xp[4 * v + 1], xp[4 * v + 2], xp[4 * v + 3]);
            continue;
          }
          const float rr = 1.0f / sqrtf(sq * (1.0f / 128.0f) + f.eps);
          const uint4* w4 = reinterpret_cast<const uint4*>(head < f.Hq ? f.q_w : f.k_w);
          // normed head n = bf16(bf16(x * rr) * w), pairs 0..31 = d 0..63, pairs 32..63 = d 64..127
#pragma unroll
          for (int v = 0; v < 16; ++v) {
            const uint4 wv = __ldg(w4 + v);
            const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const uint32_t pr = xp[4 * v + e];
              xp[4 * v + e] = bf16x2_mul(pack_bf16x2(bf16_lo(pr) * rr, bf16_hi(pr) * rr), ww[e]);
            }
          }
          // out[d] = n[d] cos[d] - n[d + 64] sin[d];  out[d + 64] = n[d + 64] cos[d + 64] + n[d] sin[d + 64]
#pragma unroll
          for (int v = 0; v < 8; ++v) {
            const uint32_t cw[4] = {rope_c[v].x, rope_c[v].y, rope_c[v].z, rope_c[v].w};
            const uint32_t sw[4] = {rope_s[v].x, rope_s[v].y, rope_s[v].z, rope_s[v].w};
            uint32_t lo[4], hi[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const uint32_t n_lo = xp[4 * v + e], n_hi = xp[32 + 4 * v + e];
              lo[e] = bf16x2_add(bf16x2_mul(n_lo, cw[e]), bf16x2_mul(n_hi ^ 0x80008000u, sw[e]));
              hi[e] = bf16x2_add(bf16x2_mul(n_hi, cw[e]), bf16x2_mul(n_lo, sw[e]));
            }
            dst4[v] = make_uint4(lo[0], lo[1], lo[2], lo[3]);
            dst4[8 + v] = make_uint4(hi[0], hi[1], hi[2], hi[3]);
          }
        }
      } else if (args.swiglu) {
        // columns come in groups of 128 weight rows = 64 gate + 64 up channels: 64 outputs per group
#pragma unroll 1
        for (int c0 = 0; c0 < kBN; c0 += 128) {
#pragma unroll 1
          for (int sub = 0; sub < 64; sub += 32) {
            uint32_t gr[32], ur[32];
            tmem_ld_32x32(t_addr + c0 + sub, gr);
            tmem_ld_32x32(t_addr + c0 + 64 + sub, ur);
            tmem_wait_ld();
            const int ocol0 = (tn * 256 + c0) / 2 + sub;
            if (row < args.M) {
              bf16* dst = args.y + static_cast<size_t>(row) * args.ldy + ocol0;
              const bool vec_ok = ((reinterpret_cast<uintptr_t>(dst) & 15) == 0) && (ocol0 + 32 <= args.N / 2);
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                float f[8];
#pragma unroll
                for (int e = 0; e < 8; ++e)
                  f[e] = swiglu2_f(__uint_as_float(gr[v * 8 + e]), __uint_as_float(ur[v * 8 + e]));
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
      } else
#pragma unroll 1
      for (int c0 = 0; c0 < kBN; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32(t_addr + c0, r);
        tmem_wait_ld();
        const int col0 = tn * 256 + c0;
        if (row < args.M) {
          bf16* dst = args.y + static_cast<size_t>(row) * args.ldy + col0;
          const bool vec_ok = ((reinterpret_cast<uintptr_t>(dst) & 15) == 0) && (col0 + 32 <= args.N);
          if (vec_ok) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              float f[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) {
                f[e] = __uint_as_float(r[v * 8 + e]);
                if (args.bias) f[e] += __bfloat162float(args.bias[col0 + v * 8 + e]);
              }
              uint4 o;
              o.x = pack_bf16x2(f[0], f[1]); o.y = pack_bf16x2(f[2], f[3]);
              o.z = pack_bf16x2(f[4], f[5]); o.w = pack_bf16x2(f[6], f[7]);
              *reinterpret_cast<uint4*>(dst + v * 8) = o;
            }
          } else {
#pragma unroll
            for (int e = 0; e < 32; ++e) {
              const int n = col0 + e;
              if (n < args.N) {
                float f = __uint_as_float(r[e]);
                if (args.bias) f += __bfloat162float(args.bias[n]);
                dst[e] = __float2bfloat16_rn(f);
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(buf ? acc_empty_leader1 : acc_empty_leader0);
    }
  }

  // ---------------- teardown ----------------
  pdl_trigger();
  tc_fence_before();
  __syncthreads();
  cluster_sync2();  // the peer may still be signalling this CTA's barriers / reading its shared memory
  if (warp == 2) {
    if (*reinterpret_cast<volatile int*>(err) != 0) {
      const uint64_t t0 = global_timer_ns();
      while (global_timer_ns() - t0 < 2000000ull) __nanosleep(1000);
    }
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
  }
}

}  // namespace

int gemm_bf16_2cta_prepare() {
  static std::atomic<unsigned long long> done{0};  // one bit per device; threads may race to set it
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 64 && (done.load(std::memory_order_acquire) >> dev) & 1ull) return 0;
  cudaError_t e = cudaFuncSetAttribute(gemm_bf16_2cta_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 64) done.fetch_or(1ull << dev, std::memory_order_release);
  return 0;
}

// Y[M, N] = X[M, K] W[N, K]^T (+ bias) for large M and N; caller has checked pointers / alignment.
int gemm_bf16_2cta(const bf16* x, int ldx, const bf16* w, int ldw, const bf16* bias, bf16* y, int ldy, int M, int N,
                   int K, cudaStream_t stream, bool swiglu, const QkvEpilogue* qkv) {
  int rc = gemm_bf16_2cta_prepare();
  if (rc) return rc;
  if (qkv) {
    if (swiglu || bias || !qkv->q_w || !qkv->k_w || !qkv->cos_t || !qkv->sin_t || !qkv->k_cache || !qkv->v_cache ||
        qkv->S <= 0 || qkv->Hq <= 0 || qkv->Hkv <= 0 || N != (qkv->Hq + 2 * qkv->Hkv) * 128 || M % qkv->S != 0 ||
        qkv->pos0 < 0 || qkv->pos0 + qkv->S > qkv->max_len || (ldy & 7))
      return TEENY_ERR_BAD_ARG;
    const uintptr_t al = reinterpret_cast<uintptr_t>(qkv->q_w) | reinterpret_cast<uintptr_t>(qkv->k_w) |
                         reinterpret_cast<uintptr_t>(qkv->cos_t) | reinterpret_cast<uintptr_t>(qkv->sin_t) |
                         reinterpret_cast<uintptr_t>(qkv->k_cache) | reinterpret_cast<uintptr_t>(qkv->v_cache) |
                         reinterpret_cast<uintptr_t>(y);
    if (al & 15) return TEENY_ERR_ALIGNMENT;
  }
  CUtensorMap tmx, tmw;
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(M)};
    const uint64_t strides[1] = {static_cast<uint64_t>(ldx) * 2};
    const uint32_t box[2] = {kBK, kBM};
    if ((rc = encode_tensor_map_bf16(&tmx, x, 2, dims, strides, box))) return rc;
  }
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(N)};
    const uint64_t strides[1] = {static_cast<uint64_t>(ldw) * 2};
    const uint32_t box[2] = {kBK, kBNh};
    if ((rc = encode_tensor_map_bf16(&tmw, w, 2, dims, strides, box))) return rc;
  }
  Args2 a{};
  a.M = M; a.N = N; a.K = K; a.ldy = ldy; a.y = y; a.bias = bias;
  a.tiles_m = (M + 255) / 256;
  a.tiles_n = (N + 255) / 256;
  a.k_blocks = (K + kBK - 1) / kBK;
  a.group = 16;  // 16 x 256 rows of X share each 256-row block of W before moving on (best of 4/8/16/32 measured)
  a.swiglu = swiglu ? 1 : 0;
  if (qkv) {
    a.qkv = 1;
    a.f = *qkv;
  }
  a.err = device_error_word();
  if (!a.err) return TEENY_ERR_DRIVER;  // kernels report expired waits through this word: no launch without it
  const int tiles = a.tiles_m * a.tiles_n;
  int pairs = sm_count() / 2;
  if (pairs > tiles) pairs = tiles;
  return launch_kernel(gemm_bf16_2cta_kernel, dim3(2 * pairs), dim3(kThreads), kSmemBytes, stream, 2, tmx, tmw, a);
}

}  // namespace teeny
