// Causal grouped-query flash-attention forward for sm_100a, head_dim 128, bf16 in/out, f32 softmax.
//
// One CTA per (128-query tile, query head, batch); keys/values stream through in tiles of 128.
//   warps 0, 3  TMA producers: warp 0 loads Q once and then the K tiles, warp 3 the V tiles, each into a two-stage ring
//               (128-byte swizzle) with its own barriers;
//   warp 1      MMA issuer: S = Q K^T (tcgen05.mma 128x128x16, both operands K-major) into one of two S buffers in
//               TMEM, and O += P V (P from tensor memory, V MN-major straight from its [key][d] tile);
//               QK^T is issued two tiles ahead of P V so the tensor pipe works while the softmax groups run;
//   warp 2      allocates / frees tensor memory;
//   warps 4-7, 8-11   two softmax warpgroups, thread = query row in both; warpgroup w takes the key tiles j = w mod 2
//               (S buffer w, P buffer w), so one group's exponentials run while the other loads and scans its next
//               tile.  Per tile: tcgen05.ld the S row in 32-column pieces for the row maximum (causal / tail mask);
//               (registers re-divided with setmaxnreg: 224 per softmax thread, 56 per service thread);
//               agree on the running maximum with the other group (it lives in shared memory; a tile's decision
//               waits for the previous tile's, a few instructions); lazy rescale (O in TMEM is only rescaled when
//               the maximum grows by more than 2^8); P = exp2(s * scale - m) as bf16
//               pairs into tensor memory, row sums in f32 per group.
// Epilogue: O / l to bf16, optional LSE = ln2 * (m + log2 l).
#include <atomic>

#include "common.cuh"
#include "kernels.h"

namespace teeny {

namespace {

constexpr int kQT = 128;
constexpr int kKT = 128;
constexpr int kHD = 128;
constexpr int kThreads = 384;  // TMA, MMA, TMEM, idle + two softmax warpgroups
constexpr int kTileBytes = kKT * kHD * 2;       // 32 KB: two 16 KB boxes of [128 rows][64 d]
constexpr int kBoxBytes = 128 * 64 * 2;         // 16 KB
constexpr int kSmemQ = 0;
constexpr int kSmemK = kSmemQ + kTileBytes;     // 2 stages
constexpr int kKV = 2;                          // stages of the K ring and of the V ring (three measured no faster)
constexpr int kSmemV = kSmemK + kKV * kTileBytes;
constexpr int kSmemBar = kSmemV + kKV * kTileBytes;
constexpr int kSmemXch = kSmemBar + 256;        // running maximum per row (128 floats), row sums of both groups (256)
constexpr int kSmemTotal = kSmemXch + 384 * 4 + 1024;
static_assert(kSmemTotal <= 232448, "exceeds the 227 KB of shared memory a CTA can have");
constexpr float kRescaleThreshold = 8.0f;       // log2 units

struct PrefillArgs {
  bf16* o;
  float* lse;
  int B, Hq, Hkv, Sq, Skv;
  long long o_sb, o_sh, o_ss;
  float scale_log2;
  int causal;
  int* err;
};

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__global__ void __launch_bounds__(kThreads, 1)
attention_prefill_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                         const __grid_constant__ CUtensorMap tmap_v, const PrefillArgs args) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t bar0 = base + kSmemBar;
  // barriers: 0 q_full | 1-3 k_full | 4-6 k_empty | 7-9 v_full | 10-12 v_empty | 13,14 s_full | 15,16 s_empty |
  //           17,18 p_full | 19,20 pv_done | 21,22 m_ready ; then the TMEM base address
  auto bar = [&](int i) { return bar0 + 8u * i; };
  constexpr int Q_FULL = 0, K_FULL = 1, K_EMPTY = K_FULL + kKV, V_FULL = K_EMPTY + kKV, V_EMPTY = V_FULL + kKV,
                S_FULL = V_EMPTY + kKV, S_EMPTY = S_FULL + 2, P_FULL = S_EMPTY + 2, PV_DONE = P_FULL + 2,
                M_READY = PV_DONE + 2, kNumBars = M_READY + 2;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gen + kSmemBar + 8 * kNumBars);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int* err = args.err;

  // heavier (later) query tiles first: with causal masking they have the most key tiles
  const int qt = gridDim.x - 1 - blockIdx.x;
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (args.Hq / args.Hkv);
  const int q0 = qt * kQT;
  const int off = args.Skv - args.Sq;  // causal: query i sees keys <= i + off
  int kv_end = args.Skv;
  if (args.causal) kv_end = min(args.Skv, q0 + kQT + off);
  const int n_tiles = (kv_end + kKT - 1) / kKT;  // >= 1 (host guarantees Skv >= Sq >= 1 when causal)

  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
    for (int i = 0; i < kNumBars; ++i) {
      const bool softmax_arrives = (i == S_EMPTY || i == S_EMPTY + 1 || i == P_FULL || i == P_FULL + 1 || i >= M_READY);
      mbar_init(bar(i), softmax_arrives ? 128 : 1);
    }
    mbar_fence_init();
  }
  if (warp == 2) {
    tmem_alloc(base + kSmemBar + 8 * kNumBars, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  // tensor memory columns: S0 0-127, S1 128-255 (f32 scores), O 256-383 (f32), P0 384-447, P1 448-511 (bf16 pairs)
  const uint32_t tmem_s0 = tmem, tmem_o = tmem + 256, tmem_p = tmem + 384;
  pdl_wait();

  // The two softmax warpgroups hold a 128-value score row per thread; the four service warps need few registers:
  // each side re-sizes its register file share at the top of its own branch.
  if (warp < 4) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
  if (warp == 0) {
    if (lane == 0) {  // Q once, then the K tiles
      mbar_expect_tx(bar(Q_FULL), kTileBytes);
      tma_load_4d(base + kSmemQ, &tmap_q, bar(Q_FULL), 0, q0, h, b);
      tma_load_4d(base + kSmemQ + kBoxBytes, &tmap_q, bar(Q_FULL), 64, q0, h, b);
      for (int j = 0; j < n_tiles; ++j) {
        const int st = j % kKV;
        const uint32_t ph = (j / kKV) & 1;
        if (!mbar_wait(bar(K_EMPTY + st), ph ^ 1, err, DEVERR_ATTN_PRODUCER)) break;
        mbar_expect_tx(bar(K_FULL + st), kTileBytes);
        tma_load_4d(base + kSmemK + st * kTileBytes, &tmap_k, bar(K_FULL + st), 0, j * kKT, hk, b);
        tma_load_4d(base + kSmemK + st * kTileBytes + kBoxBytes, &tmap_k, bar(K_FULL + st), 64, j * kKT, hk, b);
      }
    }
  } else if (warp == 3) {
    if (lane == 0) {  // the V tiles, from a thread of their own: K runs two tiles ahead of V and must not queue behind it
      for (int j = 0; j < n_tiles; ++j) {
        const int st = j % kKV;
        const uint32_t ph = (j / kKV) & 1;
        if (!mbar_wait(bar(V_EMPTY + st), ph ^ 1, err, DEVERR_ATTN_PRODUCER)) break;
        mbar_expect_tx(bar(V_FULL + st), kTileBytes);
        tma_load_4d(base + kSmemV + st * kTileBytes, &tmap_v, bar(V_FULL + st), 0, j * kKT, hk, b);
        tma_load_4d(base + kSmemV + st * kTileBytes + kBoxBytes, &tmap_v, bar(V_FULL + st), 64, j * kKT, hk, b);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_qk = make_idesc_bf16(kQT, kKT, false, false);
      constexpr uint32_t idesc_pv = make_idesc_bf16(kQT, kHD, false, true);
      bool ok = mbar_wait(bar(Q_FULL), 0, err, DEVERR_ATTN_MMA);
      // development builds: cycles this thread spends waiting for K, a free S buffer, V and P (summed over the tiles)
      TRACE_ONLY(long long w_k = 0, w_se = 0, w_v = 0, w_p = 0, c0; const long long c_begin = clock64();)
      auto issue_qk = [&](int j) -> bool {
        const int st = j & 1, kst = j % kKV;  // S buffer / K ring stage
        const uint32_t ph = (j >> 1) & 1, kph = (j / kKV) & 1;
        TRACE_ONLY(c0 = clock64();)
        if (!mbar_wait(bar(K_FULL + kst), kph, err, DEVERR_ATTN_MMA)) return false;
        TRACE_ONLY(w_k += clock64() - c0; c0 = clock64();)
        if (!mbar_wait(bar(S_EMPTY + st), ph ^ 1, err, DEVERR_ATTN_MMA)) return false;
        TRACE_ONLY(w_se += clock64() - c0;)
        tc_fence_after();
        const uint32_t qb = base + kSmemQ, kb = base + kSmemK + kst * kTileBytes;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {  // 16 d per step; 4 steps per 64-wide box
          const uint32_t o = (ks >> 2) * kBoxBytes + (ks & 3) * 32;
          umma_bf16_ss(tmem_s0 + st * 128, make_smem_desc_sw128(qb + o, 16, 1024),
                       make_smem_desc_sw128(kb + o, 16, 1024), idesc_qk, ks > 0 ? 1u : 0u);
        }
        umma_commit(bar(K_EMPTY + kst));
        umma_commit(bar(S_FULL + st));
        return true;
      };
      auto issue_pv = [&](int j) -> bool {
        const int st = j & 1, vst = j % kKV;  // P buffer / V ring stage
        const uint32_t ph = (j >> 1) & 1, vph = (j / kKV) & 1;
        TRACE_ONLY(c0 = clock64();)
        if (!mbar_wait(bar(V_FULL + vst), vph, err, DEVERR_ATTN_MMA)) return false;
        TRACE_ONLY(w_v += clock64() - c0; c0 = clock64();)
        if (!mbar_wait(bar(P_FULL + st), ph, err, DEVERR_ATTN_MMA)) return false;
        TRACE_ONLY(w_p += clock64() - c0;)
        tc_fence_after();
        const uint32_t vb = base + kSmemV + vst * kTileBytes;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {  // 16 keys per step: 8 columns of packed bf16 pairs of P in tensor memory
          // V tile: rows = keys (128 B = 64 d each), two boxes = two 64-wide d chunks (leading offset 16 KB),
          // 8-key groups 1 KB apart; 16 keys = 2 KB per step.
          const uint64_t vd = make_smem_desc_sw128(vb + ks * 2048, kBoxBytes, 1024);
          umma_bf16_ts(tmem_o, tmem_p + st * 64 + ks * 8, vd, idesc_pv, (j > 0 || ks > 0) ? 1u : 0u);
        }
        umma_commit(bar(V_EMPTY + vst));
        umma_commit(bar(PV_DONE + st));
        return true;
      };
      // QK^T runs two tiles ahead of P V: an S buffer is free again as soon as its softmax group has the row in
      // registers, and this thread must not sit in the wait for P of tile j while S of tile j+2 could be computed
      if (ok) ok = issue_qk(0);
      if (ok && n_tiles > 1) ok = issue_qk(1);
      for (int j = 0; ok && j < n_tiles; ++j) {
        if (j + 2 < n_tiles) ok = issue_qk(j + 2);
        if (ok) ok = issue_pv(j);
      }
      TRACE_VALUE(0, true, n_tiles);
      TRACE_VALUE(1, true, clock64() - c_begin);
      TRACE_VALUE(2, true, w_k);
      TRACE_VALUE(3, true, w_se);
      TRACE_VALUE(4, true, w_v);
      TRACE_VALUE(5, true, w_p);
    }
  }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 224;");
    const int quarter = warp & 3;
    const int wg = (warp - 4) >> 2;     // softmax warpgroup: key tiles j = wg, wg + 2, ...; S and P buffer wg
    const int r = quarter * 32 + lane;  // query row in the tile == TMEM lane
    const int qi = q0 + r;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t s_addr = tmem_s0 + lane_addr + wg * 128;
    float* m_sh = reinterpret_cast<float*>(gen + kSmemXch);  // [128] running maximum, log2 domain
    float* l_sh = m_sh + 128;                                // [2 groups][128] row sums
    float m_used = -INFINITY, l = 0.0f;                      // the maximum this group's sums are relative to
    bool ok = true;
    // development builds: cycles of thread 128 per phase (wait for S, scan, decision, wait for the P buffer, exp + store)
    TRACE_ONLY(long long w_s = 0, t_ld = 0, t_max = 0, w_pv = 0, t_exp = 0, c0; const long long c_begin = clock64();)
    for (int j = wg; j < n_tiles; j += 2) {
      const uint32_t ph = (j >> 1) & 1;
      TRACE_ONLY(c0 = clock64();)
      if (!mbar_wait(bar(S_FULL + wg), ph, err, DEVERR_ATTN_SOFTMAX)) { ok = false; break; }
      TRACE_ONLY(w_s += clock64() - c0; c0 = clock64();)
      tc_fence_after();
      // the S row into registers (raw scores: the scale is folded into the exponent), then the buffer is free
      float s[128];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t t[32];
        tmem_ld_32x32(s_addr + c * 32, t);
        tmem_wait_ld();
#pragma unroll
        for (int e = 0; e < 32; ++e) s[c * 32 + e] = __uint_as_float(t[e]);
      }
      tc_fence_before();
      mbar_arrive(bar(S_EMPTY + wg));  // the buffer can take QK^T of tile j+2
      const int k0 = j * kKT;
      const bool need_mask = (k0 + kKT > args.Skv) || (args.causal && (k0 + kKT - 1 > q0 + off));
      if (need_mask) {
        const int limit = args.causal ? min(args.Skv - 1, qi + off) : args.Skv - 1;  // last visible key
#pragma unroll
        for (int e = 0; e < 128; ++e)
          if (k0 + e > limit) s[e] = -INFINITY;
      }
      // row maximum: four independent chains
      float tm[4] = {s[0], s[1], s[2], s[3]};
#pragma unroll
      for (int e = 4; e < 128; e += 4) {
        tm[0] = fmaxf(tm[0], s[e]);
        tm[1] = fmaxf(tm[1], s[e + 1]);
        tm[2] = fmaxf(tm[2], s[e + 2]);
        tm[3] = fmaxf(tm[3], s[e + 3]);
      }
      const float tmax = fmaxf(fmaxf(tm[0], tm[1]), fmaxf(tm[2], tm[3])) * args.scale_log2;  // log2 domain (scale > 0)
      TRACE_ONLY(t_ld += clock64() - c0; c0 = clock64();)
      // ---- the running maximum: tile j's decision follows tile j-1's (made by the other group) ----
      float m;
      if (j == 0) {
        m = tmax;  // key 0 is visible to every row, so m is finite from here on
      } else {
        if (!mbar_wait(bar(M_READY + (wg ^ 1)), ((j - 1) >> 1) & 1, err, DEVERR_ATTN_SOFTMAX)) { ok = false; break; }
        m = m_sh[r];
        const float m_new = fmaxf(m, tmax);
        const bool grow = m_new > m + kRescaleThreshold;
        if (__any_sync(0xffffffffu, grow)) {
          // O must be final for tile j-1 before it is rescaled
          if (!mbar_wait(bar(PV_DONE + ((j - 1) & 1)), ((j - 1) >> 1) & 1, err, DEVERR_ATTN_SOFTMAX)) { ok = false; break; }
          tc_fence_after();
          const float alpha = fast_exp2(m - m_new);
          m = m_new;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t t[32];
            tmem_ld_32x32(tmem_o + lane_addr + c * 32, t);
            tmem_wait_ld();
#pragma unroll
            for (int e = 0; e < 32; ++e) t[e] = __float_as_uint(__uint_as_float(t[e]) * alpha);
            tmem_st_32x32(tmem_o + lane_addr + c * 32, t);
          }
          tmem_wait_st();
          tc_fence_before();
        }
      }
      m_sh[r] = m;
      mbar_arrive(bar(M_READY + wg));  // tile j + 1 may decide (and rescale O) now
      if (m_used != m) {                // this group's sums follow the maximum (no-op while l == 0)
        l *= fast_exp2(m_used - m);
        m_used = m;
      }
      TRACE_ONLY(t_max += clock64() - c0; c0 = clock64();)
      // the P buffer was last read by P V of tile j-2
      if (j >= 2) {
        if (!mbar_wait(bar(PV_DONE + wg), ((j - 2) >> 1) & 1, err, DEVERR_ATTN_SOFTMAX)) { ok = false; break; }
      }
      TRACE_ONLY(w_pv += clock64() - c0; c0 = clock64();)
      // probabilities as bf16 pairs straight into tensor memory (the A operand of P V): no shared-memory round trip
      float ls[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      const float neg_m = -m;
#pragma unroll
      for (int hc = 0; hc < 2; ++hc) {  // 64 keys = 32 packed columns per store
        uint32_t pk[32];
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          const float p0 = fast_exp2(fmaf(s[hc * 64 + 2 * e], args.scale_log2, neg_m));  // masked scores are -inf -> 0
          const float p1 = fast_exp2(fmaf(s[hc * 64 + 2 * e + 1], args.scale_log2, neg_m));
          ls[(2 * e) & 3] += p0;
          ls[(2 * e + 1) & 3] += p1;
          pk[e] = pack_bf16x2(p0, p1);
        }
        tmem_st_32x32(tmem_p + lane_addr + wg * 64 + hc * 32, pk);
      }
      tmem_wait_st();
      l += (ls[0] + ls[1]) + (ls[2] + ls[3]);
      tc_fence_before();
      mbar_arrive(bar(P_FULL + wg));
      TRACE_ONLY(t_exp += clock64() - c0;)
    }
    TRACE_VALUE(6, threadIdx.x == 128, clock64() - c_begin);
    TRACE_VALUE(7, threadIdx.x == 128, w_s);
    TRACE_VALUE(8, threadIdx.x == 128, t_ld);
    TRACE_VALUE(9, threadIdx.x == 128, t_max);
    TRACE_VALUE(10, threadIdx.x == 128, w_pv);
    TRACE_VALUE(11, threadIdx.x == 128, t_exp);
    // ---- both groups: final maximum, total row sum, then half of the output columns each ----
    const int last = n_tiles - 1;
    if (ok) ok = mbar_wait(bar(M_READY + (last & 1)), (last >> 1) & 1, err, DEVERR_ATTN_SOFTMAX);
    const float m_fin = m_sh[r];
    if (m_used != m_fin) l *= fast_exp2(m_used - m_fin);  // a group without tiles has l = 0 and m_used = -inf
    l_sh[wg * 128 + r] = l;
    named_barrier_sync(1, 256);  // every softmax thread gets here, also after a failed wait
    l = l_sh[r] + l_sh[128 + r];
    if (ok) ok = mbar_wait(bar(PV_DONE + (last & 1)), (last >> 1) & 1, err, DEVERR_ATTN_SOFTMAX);
    if (ok) {
      tc_fence_after();
      const float inv = 1.0f / l;
      const bool valid = qi < args.Sq;
      const int col0 = wg * 64;
      bf16* dst = args.o + b * args.o_sb + h * args.o_sh + static_cast<long long>(qi) * args.o_ss + col0;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t t[32];
        tmem_ld_32x32(tmem_o + lane_addr + col0 + c * 32, t);
        tmem_wait_ld();
        if (valid) {
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint4 o4;
            o4.x = pack_bf16x2(__uint_as_float(t[v * 8 + 0]) * inv, __uint_as_float(t[v * 8 + 1]) * inv);
            o4.y = pack_bf16x2(__uint_as_float(t[v * 8 + 2]) * inv, __uint_as_float(t[v * 8 + 3]) * inv);
            o4.z = pack_bf16x2(__uint_as_float(t[v * 8 + 4]) * inv, __uint_as_float(t[v * 8 + 5]) * inv);
            o4.w = pack_bf16x2(__uint_as_float(t[v * 8 + 6]) * inv, __uint_as_float(t[v * 8 + 7]) * inv);
            *reinterpret_cast<uint4*>(dst + c * 32 + v * 8) = o4;
          }
        }
      }
      if (valid && args.lse && wg == 0)
        args.lse[(static_cast<long long>(b) * args.Hq + h) * args.Sq + qi] = 0.6931471805599453f * (m_fin + log2f(l));
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    if (*reinterpret_cast<volatile int*>(err) != 0) {
      const uint64_t t0 = global_timer_ns();
      while (global_timer_ns() - t0 < 2000000ull) __nanosleep(1000);
    }
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

int make_map(CUtensorMap* m, const bf16* p, int S, int H, int B, long long ss, long long sh, long long sb) {
  const uint64_t dims[4] = {kHD, static_cast<uint64_t>(S), static_cast<uint64_t>(H), static_cast<uint64_t>(B)};
  const uint64_t strides[3] = {static_cast<uint64_t>(ss) * 2, static_cast<uint64_t>(sh) * 2,
                               static_cast<uint64_t>(sb) * 2};
  const uint32_t box[4] = {64, 128, 1, 1};
  return encode_tensor_map_bf16(m, p, 4, dims, strides, box);
}

}  // namespace

int attention_prefill_prepare() {
  static std::atomic<unsigned long long> done{0};  // one bit per device; threads may race to set it
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 64 && (done.load(std::memory_order_acquire) >> dev) & 1ull) return 0;
  cudaError_t e = cudaFuncSetAttribute(attention_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemTotal);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 64) done.fetch_or(1ull << dev, std::memory_order_release);
  return 0;
}

int attention_prefill_bf16(const bf16* q, const bf16* k, const bf16* v, bf16* o, float* lse, const AttnShape& s,
                           cudaStream_t stream) {
  if (!q || !k || !v || !o || s.B <= 0 || s.Hq <= 0 || s.Hkv <= 0 || s.Sq <= 0 || s.Skv <= 0) return TEENY_ERR_BAD_ARG;
  if (s.D != kHD || s.Hq % s.Hkv != 0) return TEENY_ERR_BAD_ARG;
  if (s.causal && s.Skv < s.Sq) return TEENY_ERR_BAD_ARG;
  const long long strides[] = {s.q_sb, s.q_sh, s.q_ss, s.k_sb, s.k_sh, s.k_ss, s.v_sb, s.v_sh, s.v_ss, s.o_ss, s.o_sh, s.o_sb};
  for (long long st : strides)
    if (st % 8 != 0) return TEENY_ERR_ALIGNMENT;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
       reinterpret_cast<uintptr_t>(o)) & 15)
    return TEENY_ERR_ALIGNMENT;
  if (s.Hq > 65535 || s.B > 65535) return TEENY_ERR_BAD_ARG;
  CUtensorMap mq, mk, mv;
  int rc;
  // a dimension of extent 1 still needs a legal (multiple-of-16-byte, non-zero) stride
  auto fix = [](long long st, long long fallback) { return st > 0 ? st : fallback; };
  if ((rc = make_map(&mq, q, s.Sq, s.Hq, s.B, s.q_ss, fix(s.q_sh, s.q_ss), fix(s.q_sb, s.q_ss)))) return rc;
  if ((rc = make_map(&mk, k, s.Skv, s.Hkv, s.B, s.k_ss, fix(s.k_sh, s.k_ss), fix(s.k_sb, s.k_ss)))) return rc;
  if ((rc = make_map(&mv, v, s.Skv, s.Hkv, s.B, s.v_ss, fix(s.v_sh, s.v_ss), fix(s.v_sb, s.v_ss)))) return rc;

  PrefillArgs a{};
  a.o = o; a.lse = lse; a.B = s.B; a.Hq = s.Hq; a.Hkv = s.Hkv; a.Sq = s.Sq; a.Skv = s.Skv;
  a.o_sb = s.o_sb; a.o_sh = s.o_sh; a.o_ss = s.o_ss;
  a.scale_log2 = s.scale * 1.4426950408889634f;
  a.causal = s.causal;
  a.err = device_error_word();
  if (!a.err) return TEENY_ERR_DRIVER;  // kernels report expired waits through this word: no launch without it

  {
    const int prc = attention_prefill_prepare();
    if (prc) return prc;
  }
  dim3 grid((s.Sq + kQT - 1) / kQT, s.Hq, s.B);
  launch_kernel(attention_prefill_kernel, dim3(grid), dim3(kThreads), kSmemTotal, stream, 1, mq, mk, mv, a);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace teeny
