// Attention kernels that are not tcgen05-shaped.
//
// 1. attention_decode_bf16: one query token per sequence against a long KV cache.  HBM-bound (every K and V byte is
//    read once, the query heads of a KV group share it), so the design goal is streaming the cache: a producer warp
//    keeps a ring of TMA tile copies in flight (data in flight costs no registers) and four consumer warps run the
//    arithmetic on warp-level mma.sync tiles fed by ldmatrix (a 128-row tcgen05 tile would be 97 % padding for 4 query
//    heads).  Split over the sequence only when B * Hkv alone cannot fill the GPU; every consumer warp takes 16
//    keys of each 64-key tile with an online softmax, warps are merged through shared memory, per-chunk partials
//    (m, l, O) go to scratch and a second kernel merges chunks.
// 2. attention_generic<T>: any head_dim <= 256, f32 or bf16, one warp per query row, sequential online softmax --
//    the reference kernel's own recurrence; used for the f32 entry point and for shapes the tcgen05 kernel
//    does not cover.
#include <atomic>

#include "common.cuh"
#include "kernels.h"

namespace teeny {

namespace {

constexpr int kDecChunk = 512;
constexpr int kHD = 128;

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// ---- decode kernel: TMA-fed shared-memory ring + mma.sync ----
// CTA = one (batch, kv head, share of the live keys).  Warp 4 is the producer: for every 64-key tile it requests the
// K rows and the V rows (two [64 keys][64 d] boxes each, 128-byte swizzle) into a ring of 32 KB stages (three deep with two CTAs per SM, six with one) and the copies
// signal a `full` mbarrier; nothing in flight costs registers.  Warps 0-3 each own 16 keys of a tile:
//   S = Q K^T   A = Q from registers (rows = the G query heads of the group, padded to 16), B = K fragments through
//               ldmatrix (a matrix row is one key's 16 bytes, so the swizzle makes the eight rows conflict-free);
//   softmax     online, log2 domain, in the C-fragment registers (lane group g = head, lane c = key pair);
//   O += P V    A = P straight from the S fragments, B = V fragments through ldmatrix.trans (pairs of keys per d).
// Fragment layout (mma.m16n8k16, g = lane / 4, c = lane % 4): A a0 = (row g, k 2c..2c+1), a2 = (row g, k 2c+8..);
// B b0 = (k 2c..2c+1, col g), b1 = (k 2c+8.., col g); C c0,c1 = (row g, cols 2c, 2c+1); rows 8..15 are padding.
struct DecodeArgs {
  const bf16* q;
  float* part_o;   // [B, Hkv, chunks, G, 128]
  float* part_ml;  // [B, Hkv, chunks, G, 2]
  long long q_sb, q_sh;
  bf16* o;         // final output, written directly when the sequence is not split (gridDim.x == 1)
  long long o_sb, o_sh;
  int Hkv, G, max_chunks;
  int kv_len;
  const int* kv_len_dev;
  // >= 0: only the last `fresh_rows` live cache rows (and q) come from the kernel launched just before this one;
  // the length and every older row were complete before that kernel started, so they may be read ahead of the
  // dependency wait.  < 0: nothing is known, read everything after the wait.
  int fresh_rows;
  int stages;          // ring depth of this launch
  unsigned* counters;  // [B * Hkv] arrival counters (zero between calls) for the in-kernel merge, or null
  float scale_log2;
  int* err;
  DecodeRope rope;  // rope.k_new == nullptr: q is final and the caches already hold the new rows
  long long kc_sb, kc_sh, kc_ss, vc_sb, vc_sh, vc_ss;  // cache strides for the append
};

constexpr int kDecTile = 64;                     // keys per ring stage
constexpr int kDecStagesShared = 3;  // ring depth when two CTAs share an SM
constexpr int kDecStagesAlone = 6;   // ring depth when the grid has at most one CTA per SM
constexpr int kDecBox = kDecTile * 64 * 2;       // 8 KB: [64 keys][64 d]
constexpr int kDecStageBytes = 4 * kDecBox;      // K (2 boxes) + V (2 boxes) = 32 KB
constexpr int dec_smem_bytes(int stages) { return stages * kDecStageBytes + 1024 + 128; }
constexpr int kDecThreads = 160;                 // 4 consumer warps + 1 producer warp

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

template <int G>
__global__ void __launch_bounds__(kDecThreads, 2)
attention_decode_kernel(const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                        const DecodeArgs a) {
  extern __shared__ uint8_t dec_smem_raw[];
  __shared__ float sm_ml[4][8][2];
  __shared__ float sm_o[4][G][kHD];
  __shared__ __align__(16) bf16 sm_q[4][G][kHD];  // normed, rotated q heads, one copy per consumer warp (fused front end)
  const uint32_t base = (smem_u32(dec_smem_raw) + 1023u) & ~1023u;
  uint8_t* gen = dec_smem_raw + (base - smem_u32(dec_smem_raw));
  const int n_stages = a.stages;
  const uint32_t bar0 = base + n_stages * kDecStageBytes;
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (n_stages + s); };
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int chunk = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
    for (int s = 0; s < n_stages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 4);
    }
    mbar_fence_init();
  }
  __syncthreads();
  // the live keys are divided evenly (in whole 64-key tiles) over the gridDim.x CTAs of this (batch, kv head)
  int L = 0, span = 0, key_begin = 0, key_end = 0, n_tiles = 0;
  auto plan = [&]() {
    L = a.kv_len_dev ? *a.kv_len_dev : a.kv_len;
    span = ((L + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x) + kDecTile - 1) / kDecTile * kDecTile;
    key_begin = chunk * span;
    key_end = min(L, key_begin + span);
    n_tiles = key_begin < L ? (key_end - key_begin + kDecTile - 1) / kDecTile : 0;
  };
  auto load_tile = [&](int t, int st) {
    const uint32_t dst = base + st * kDecStageBytes;
    const int key0 = key_begin + t * kDecTile;
    mbar_expect_tx(full_bar(st), kDecStageBytes);
    tma_load_4d(dst, &tmap_k, full_bar(st), 0, key0, hk, b);
    tma_load_4d(dst + kDecBox, &tmap_k, full_bar(st), 64, key0, hk, b);
    tma_load_4d(dst + 2 * kDecBox, &tmap_v, full_bar(st), 0, key0, hk, b);
    tma_load_4d(dst + 3 * kDecBox, &tmap_v, full_bar(st), 64, key0, hk, b);
  };
  int pre = 0;  // tiles requested ahead of the wait (producer thread only)
  int rope_pos = 0;
  if (a.fresh_rows >= 0) {
    plan();
    if (a.rope.k_new) rope_pos = a.rope.pos_dev ? *a.rope.pos_dev : a.rope.pos;
    if (threadIdx.x == 128) {
      // first ring of tiles that hold none of the rows the previous kernel is still writing
      while (pre < n_tiles && pre < n_stages && key_begin + (pre + 1) * kDecTile <= L - a.fresh_rows) {
        load_tile(pre, pre);
        ++pre;
      }
    }
  }
  pdl_wait();  // the cache rows of this step (and, unless declared stable, the live length) come from earlier kernels
  if (a.fresh_rows < 0) {
    plan();
    if (a.rope.k_new) rope_pos = a.rope.pos_dev ? *a.rope.pos_dev : a.rope.pos;
  }
  const int g = lane >> 2, c = lane & 3;
  float acc[16][4];
  float m = -INFINITY, l = 0.0f;
  if (n_tiles == 0) return;  // chunk lies beyond the live length (uniform for the CTA)

  // Fused front end (per-head RMSNorm + RoPE + cache append), one 128-wide head per half-warp.  No CTA-wide barrier:
  // the producer warp norms / rotates the new key, appends it and the new value to the caches and goes on streaming;
  // every consumer warp prepares its own copy of the G query heads.
  const bool fused = a.rope.k_new != nullptr;
  const int sub = lane & 15, hw = lane >> 4;
  auto rope_head = [&](const bf16* src, const bf16* w, uint4& raw) {
    raw = *reinterpret_cast<const uint4*>(src + sub * 8);
    const uint4 wraw = __ldg(reinterpret_cast<const uint4*>(w + sub * 8));
    const int tp = rope_pos < a.rope.max_len ? rope_pos : a.rope.max_len - 1;
    const uint4 craw = __ldg(reinterpret_cast<const uint4*>(a.rope.cos_t + static_cast<size_t>(tp) * kHD + sub * 8));
    const uint4 sraw = __ldg(reinterpret_cast<const uint4*>(a.rope.sin_t + static_cast<size_t>(tp) * kHD + sub * 8));
    return head_norm_rope(raw, wraw, craw, sraw, sub, a.rope.eps);
  };

  if (warp == 4) {
    // ---------------- producer ----------------
    if (fused) {
      // half-warp 0: key head (normed, rotated); half-warp 1: value head (copied)
      uint4 raw;
      const uint4 outv = rope_head((hw == 0 ? a.rope.k_new : a.rope.v_new) + b * a.rope.new_sb + hk * kHD, a.rope.k_w, raw);
      if (rope_pos >= key_begin && rope_pos < key_end && rope_pos < a.rope.max_len) {
        if (hw == 0)
          *reinterpret_cast<uint4*>(a.rope.k_cache + b * a.kc_sb + hk * a.kc_sh + rope_pos * a.kc_ss + sub * 8) = outv;
        else
          *reinterpret_cast<uint4*>(a.rope.v_cache + b * a.vc_sb + hk * a.vc_sh + rope_pos * a.vc_ss + sub * 8) = raw;
      }
      // the appended rows are read back by this warp's own TMA loads (async proxy): order them behind the stores
      __threadfence();
      asm volatile("fence.proxy.async;" ::: "memory");
      __syncwarp();
    }
    if (lane == 0) {
      int st = pre == n_stages ? 0 : pre;
      uint32_t ph = pre == n_stages ? 1 : 0;
      for (int t = pre; t < n_tiles; ++t) {
        if (!mbar_wait(empty_bar(st), ph ^ 1, a.err, DEVERR_ATTN_PRODUCER)) break;
        load_tile(t, st);
        if (++st == n_stages) { st = 0; ph ^= 1; }
      }
    }
  } else {
    // ---------------- consumers: warp w owns keys [16 w, 16 w + 16) of every tile ----------------
#pragma unroll
    for (int i = 0; i < 16; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.0f;
    // Q fragments: head hk * G + g; a0 = d 16 ks + 2c.., a2 = d 16 ks + 8 + 2c..; rows >= G are zero
    uint32_t qa[8][2];
    {
      if (fused) {
#pragma unroll
        for (int h0 = 0; h0 < G; h0 += 2) {  // two heads per pass (a lone last head is done twice)
          const int hsel = h0 + hw < G ? h0 + hw : G - 1;
          uint4 raw;
          const uint4 outv = rope_head(a.q + b * a.q_sb + (hk * G + hsel) * a.q_sh, a.rope.q_w, raw);
          *reinterpret_cast<uint4*>(&sm_q[warp][hsel][sub * 8]) = outv;
        }
        __syncwarp();
      }
      const bf16* qp = fused ? &sm_q[warp][g < G ? g : 0][0] : a.q + b * a.q_sb + (hk * G + (g < G ? g : 0)) * a.q_sh;
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        const uint32_t lo = *reinterpret_cast<const uint32_t*>(qp + 16 * ks + 2 * c);
        const uint32_t hi = *reinterpret_cast<const uint32_t*>(qp + 16 * ks + 8 + 2 * c);
        qa[ks][0] = g < G ? lo : 0u;
        qa[ks][1] = g < G ? hi : 0u;
      }
    }
    const int row_k = 16 * warp + (lane & 7);  // ldmatrix row this lane addresses for K: + 8 * n-block
    const int mat = lane >> 3;                 // which of the four 8x8 matrices this lane addresses
    bool ok = true;
    int st = 0;
    uint32_t ph = 0;
    for (int t = 0; t < n_tiles; ++t, st = (st + 1 == n_stages ? 0 : st + 1), ph ^= (st == 0 ? 1u : 0u)) {
      if (!mbar_wait(full_bar(st), ph, a.err, DEVERR_ATTN_SOFTMAX)) { ok = false; break; }
      const uint32_t kt = base + st * kDecStageBytes, vt = kt + 2 * kDecBox;
      const int kb = key_begin + t * kDecTile + 16 * warp;  // first key of this warp's slice
      if (kb < key_end) {
        if (kb + 16 > key_end) {
          // rows past the live length hold whatever the cache had (possibly NaN patterns): their probabilities are
          // zero, but 0 * NaN is NaN inside the MMA, so clear those V rows first
          uint8_t* vrow = gen + st * kDecStageBytes + 2 * kDecBox;
          for (int i = lane; i < 256; i += 32) {
            const int r = i >> 4, ch = i & 15;
            if (kb + r >= key_end)
              *reinterpret_cast<uint4*>(vrow + (ch >> 3) * kDecBox + (16 * warp + r) * 128 + (ch & 7) * 16) =
                  make_uint4(0, 0, 0, 0);
          }
          __syncwarp();
        }
        // ---- S = Q K^T: two 8-key column blocks ----
        float s[2][4];
#pragma unroll
        for (int nb = 0; nb < 2; ++nb) {
          s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.0f;
          const int row = row_k + 8 * nb;
#pragma unroll
          for (int p = 0; p < 4; ++p) {  // 32 d per ldmatrix.x4: matrices = four 8-d chunks
            uint32_t kf[4];
            ldsm_x4(kf, kt + (p >> 1) * kDecBox + row * 128 + ((((p & 1) * 4 + mat) ^ (row & 7)) << 4));
            mma_bf16_16816(s[nb], qa[2 * p][0], 0u, qa[2 * p][1], 0u, kf[0], kf[1]);
            mma_bf16_16816(s[nb], qa[2 * p + 1][0], 0u, qa[2 * p + 1][1], 0u, kf[2], kf[3]);
          }
        }
        // ---- online softmax on row g: this lane holds keys kb + nb*8 + 2c + {0,1} ----
        float tmax = -INFINITY;
#pragma unroll
        for (int nb = 0; nb < 2; ++nb)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int key = kb + nb * 8 + 2 * c + e;
            s[nb][e] = key < key_end ? s[nb][e] * a.scale_log2 : -INFINITY;
            tmax = fmaxf(tmax, s[nb][e]);
          }
        tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 1));
        tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 2));
        const float m_new = fmaxf(m, tmax);  // finite: key kb itself is < key_end
        const float alpha = ex2(m - m_new);  // m = -inf on the first slice -> 0
        m = m_new;
        float p[2][2], psum = 0.0f;
#pragma unroll
        for (int nb = 0; nb < 2; ++nb)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            p[nb][e] = ex2(s[nb][e] - m);
            psum += p[nb][e];
          }
        psum += __shfl_xor_sync(0xffffffffu, psum, 1);
        psum += __shfl_xor_sync(0xffffffffu, psum, 2);
        l = l * alpha + psum;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          acc[i][0] *= alpha;
          acc[i][1] *= alpha;
        }
        const uint32_t pa0 = pack_bf16x2(p[0][0], p[0][1]);  // keys 2c, 2c+1
        const uint32_t pa2 = pack_bf16x2(p[1][0], p[1][1]);  // keys 2c+8, 2c+9
        // ---- O += P V: ldmatrix.trans yields (key pair, d) fragments; one x4 covers two 8-wide d blocks ----
        const int row_v = 16 * warp + (mat & 1) * 8 + (lane & 7);
#pragma unroll
        for (int nbp = 0; nbp < 8; ++nbp) {
          const int chunk16 = 2 * nbp + (mat >> 1);  // 8-d chunk index 0..15
          uint32_t vf[4];
          ldsm_x4_trans(vf, vt + (chunk16 >> 3) * kDecBox + row_v * 128 + (((chunk16 & 7) ^ (row_v & 7)) << 4));
          mma_bf16_16816(acc[2 * nbp], pa0, 0u, pa2, 0u, vf[0], vf[1]);
          mma_bf16_16816(acc[2 * nbp + 1], pa0, 0u, pa2, 0u, vf[2], vf[3]);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(empty_bar(st));  // this warp has read everything it needs from the stage
    }
    (void)ok;
  }

  pdl_trigger();  // cache streaming done; what follows is the small merge
  // ---- merge the four consumer warps ----
  if (warp < 4) {
    if (c == 0 && g < G) {
      sm_ml[warp][g][0] = m;
      sm_ml[warp][g][1] = l;
    }
    if (g < G) {
#pragma unroll
      for (int nb = 0; nb < 16; ++nb) {
        sm_o[warp][g][8 * nb + 2 * c] = acc[nb][0];
        sm_o[warp][g][8 * nb + 2 * c + 1] = acc[nb][1];
      }
    }
  }
  __syncthreads();
  const size_t slot = (static_cast<size_t>(b) * a.Hkv + hk) * a.max_chunks + chunk;
  for (int idx = threadIdx.x; idx < G * kHD; idx += kDecThreads) {
    const int gg = idx / kHD, d = idx - gg * kHD;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) mm = fmaxf(mm, sm_ml[w][gg][0]);  // warps without keys hold -inf
    float ll = 0.0f, oo = 0.0f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float wm = sm_ml[w][gg][0];
      const float sc = (wm == -INFINITY) ? 0.0f : ex2(wm - mm);
      ll += sm_ml[w][gg][1] * sc;
      oo += sm_o[w][gg][d] * sc;
    }
    if (gridDim.x == 1) {  // whole sequence in this CTA: finish here, no partials
      a.o[b * a.o_sb + (hk * G + gg) * a.o_sh + d] = __float2bfloat16_rn(oo / ll);
      continue;
    }
    a.part_o[(slot * G + gg) * kHD + d] = oo;
    if (d == 0) {
      a.part_ml[(slot * G + gg) * 2 + 0] = mm;
      a.part_ml[(slot * G + gg) * 2 + 1] = ll;
    }
  }
  if (gridDim.x > 1 && a.counters) {
    // The last CTA of this (sequence, kv head) to have stored its partial merges them all: no second kernel.
    __shared__ unsigned sm_last;
    __threadfence();
    __syncthreads();
    const int chunks = (L + span - 1) / span;  // CTAs of this group that had keys
    unsigned* ctr = a.counters + static_cast<size_t>(b) * a.Hkv + hk;
    if (threadIdx.x == 0) {
      const unsigned old = atomicAdd(ctr, 1u);
      sm_last = (old == static_cast<unsigned>(chunks - 1)) ? 1u : 0u;
      if (sm_last) *ctr = 0u;  // every CTA of the group has arrived: re-arm for the next call
    }
    __syncthreads();
    if (sm_last) {
      __threadfence();
      const size_t slot0 = (static_cast<size_t>(b) * a.Hkv + hk) * a.max_chunks;
      for (int idx = threadIdx.x; idx < G * kHD; idx += kDecThreads) {
        const int gg = idx / kHD, d = idx - gg * kHD;
        float mm = -INFINITY;
        for (int ch = 0; ch < chunks; ++ch) mm = fmaxf(mm, __ldcg(a.part_ml + ((slot0 + ch) * G + gg) * 2));
        float ll = 0.0f, oo = 0.0f;
        for (int ch = 0; ch < chunks; ++ch) {
          const size_t sl = (slot0 + ch) * G + gg;
          const float sc = ex2(__ldcg(a.part_ml + sl * 2) - mm);
          ll += __ldcg(a.part_ml + sl * 2 + 1) * sc;
          oo += __ldcg(a.part_o + sl * kHD + d) * sc;
        }
        a.o[b * a.o_sb + (hk * G + gg) * a.o_sh + d] = __float2bfloat16_rn(oo / ll);
      }
    }
  }
  TRACE_END();
}

// grid (Hq, B), 128 threads: thread d merges the valid chunks of head h.
__global__ void attention_decode_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                                bf16* __restrict__ o, long long o_sb, long long o_sh, int Hkv, int G,
                                                int max_chunks, int n_split, int kv_len,
                                                const int* __restrict__ kv_len_dev) {
  pdl_wait();
  const int h = blockIdx.x, b = blockIdx.y, d = threadIdx.x;
  const int L = kv_len_dev ? *kv_len_dev : kv_len;
  const int span = ((L + n_split - 1) / n_split + kDecTile - 1) / kDecTile * kDecTile;  // as in the main kernel
  const int chunks = (L + span - 1) / span;
  const int hk = h / G, gg = h - hk * G;
  const size_t slot0 = (static_cast<size_t>(b) * Hkv + hk) * max_chunks;
  float mm = -INFINITY;
  for (int ch = 0; ch < chunks; ++ch) mm = fmaxf(mm, part_ml[((slot0 + ch) * G + gg) * 2]);
  float ll = 0.0f, oo = 0.0f;
  for (int ch = 0; ch < chunks; ++ch) {
    const size_t s = (slot0 + ch) * G + gg;
    const float sc = ex2(part_ml[s * 2] - mm);
    ll += part_ml[s * 2 + 1] * sc;
    oo += part_o[s * kHD + d] * sc;
  }
  o[b * o_sb + h * o_sh + d] = __float2bfloat16_rn(oo / ll);
}

// ------------------------------------------------------------------------------------------------
template <typename T> __device__ __forceinline__ float ld_as_f(const T* p);
template <> __device__ __forceinline__ float ld_as_f<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ld_as_f<bf16>(const bf16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void st_from_f(float* p, float v) { *p = v; }
__device__ __forceinline__ void st_from_f(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

// one warp per (query row, head, batch); lane owns d = lane, lane + 32, ... (up to 8 values: D <= 256)
template <typename T>
__global__ void attention_generic_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                                         T* __restrict__ o, float* __restrict__ lse, const AttnShape s) {
  pdl_wait();
  const long long wid = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long rows = static_cast<long long>(s.B) * s.Hq * s.Sq;
  if (wid >= rows) return;
  const int i = static_cast<int>(wid % s.Sq);
  const int h = static_cast<int>((wid / s.Sq) % s.Hq);
  const int b = static_cast<int>(wid / (static_cast<long long>(s.Sq) * s.Hq));
  const int hk = h / (s.Hq / s.Hkv);
  const T* qr = q + b * s.q_sb + h * s.q_sh + i * s.q_ss;
  const T* kb = k + b * s.k_sb + hk * s.k_sh;
  const T* vb = v + b * s.v_sb + hk * s.v_sh;
  float qv[8], acc[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const int d = lane + 32 * e;
    qv[e] = d < s.D ? ld_as_f(qr + d) : 0.0f;
    acc[e] = 0.0f;
  }
  float m = -INFINITY, l = 0.0f;
  const int last = s.causal ? min(s.Skv - 1, i + (s.Skv - s.Sq)) : s.Skv - 1;
  for (int j = 0; j <= last; ++j) {
    const T* kr = kb + j * s.k_ss;
    const T* vr = vb + j * s.v_ss;
    float dot = 0.0f;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const int d = lane + 32 * e;
      if (d < s.D) dot += qv[e] * ld_as_f(kr + d);
    }
    dot = warp_sum(dot) * s.scale;
    const float m_new = fmaxf(m, dot);
    const float corr = expf(m - m_new);
    const float p = expf(dot - m_new);
    l = corr * l + p;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const int d = lane + 32 * e;
      if (d < s.D) acc[e] = corr * acc[e] + p * ld_as_f(vr + d);
    }
    m = m_new;
  }
  T* orow = o + b * s.o_sb + h * s.o_sh + i * s.o_ss;
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const int d = lane + 32 * e;
    if (d < s.D) st_from_f(orow + d, acc[e] / l);
  }
  if (lse && lane == 0) lse[(static_cast<long long>(b) * s.Hq + h) * s.Sq + i] = m + logf(l);
}

}  // namespace

// Raises the decode kernel's dynamic shared-memory limit once per device.
int attention_decode_prepare() {
  static std::atomic<unsigned long long> done{0};  // one bit per device; threads may race to set it
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 64 && (done.load(std::memory_order_acquire) >> dev) & 1ull) return 0;
  cudaError_t e = cudaFuncSetAttribute(attention_decode_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, dec_smem_bytes(kDecStagesAlone));
  if (e == cudaSuccess) e = cudaFuncSetAttribute(attention_decode_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, dec_smem_bytes(kDecStagesAlone));
  if (e == cudaSuccess) e = cudaFuncSetAttribute(attention_decode_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, dec_smem_bytes(kDecStagesAlone));
  if (e == cudaSuccess) e = cudaFuncSetAttribute(attention_decode_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, dec_smem_bytes(kDecStagesAlone));
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 64) done.fetch_or(1ull << dev, std::memory_order_release);
  return 0;
}

size_t attention_decode_scratch_bytes(int B, int Hq, int D, int max_kv) {
  if (B <= 0 || Hq <= 0 || D <= 0 || max_kv <= 0) return 0;
  const size_t chunks = (static_cast<size_t>(max_kv) + kDecChunk - 1) / kDecChunk;
  return static_cast<size_t>(B) * Hq * chunks * (D + 2) * sizeof(float);
}

int attention_decode_bf16(const bf16* q, const bf16* k, const bf16* v, bf16* o, const AttnShape& s, int kv_len,
                          const int* kv_len_dev, void* scratch, size_t scratch_bytes, cudaStream_t stream,
                          int fresh_rows, const DecodeRope* rope, unsigned* counters) {
  if (!q || !k || !v || !o || !scratch || s.B <= 0 || s.Hq <= 0 || s.Hkv <= 0 || s.Skv <= 0) return TEENY_ERR_BAD_ARG;
  if (s.D != kHD || s.Hq % s.Hkv != 0 || s.Sq != 1) return TEENY_ERR_BAD_ARG;
  if (!kv_len_dev && (kv_len <= 0 || kv_len > s.Skv)) return TEENY_ERR_BAD_ARG;
  const int G = s.Hq / s.Hkv;
  if (G != 1 && G != 2 && G != 4 && G != 8) return TEENY_ERR_BAD_ARG;
  const long long strides[] = {s.q_sb, s.q_sh, s.k_sb, s.k_sh, s.k_ss, s.v_sb, s.v_sh, s.v_ss};
  for (long long st : strides)
    if (st % 8 != 0) return TEENY_ERR_ALIGNMENT;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v)) & 15)
    return TEENY_ERR_ALIGNMENT;
  // s.Skv is the cache capacity the grid is sized for; the live length comes from kv_len / kv_len_dev
  if (scratch_bytes < attention_decode_scratch_bytes(s.B, s.Hq, s.D, s.Skv)) return TEENY_ERR_SCRATCH;
  const int max_chunks = (s.Skv + kDecChunk - 1) / kDecChunk;
  if (s.Hkv > 65535 || s.B > 65535) return TEENY_ERR_BAD_ARG;

  // K and V caches as 4-D tensors (d, key, kv head, batch); a tile is two [64 keys][64 d] boxes
  CUtensorMap mk, mv;
  {
    const uint64_t dims[4] = {kHD, static_cast<uint64_t>(s.Skv), static_cast<uint64_t>(s.Hkv), static_cast<uint64_t>(s.B)};
    const uint32_t box[4] = {64, kDecTile, 1, 1};
    auto nz = [](long long st, long long fb) { return static_cast<uint64_t>(st > 0 ? st : fb) * 2; };
    const uint64_t ks[3] = {static_cast<uint64_t>(s.k_ss) * 2, nz(s.k_sh, s.k_ss), nz(s.k_sb, s.k_ss)};
    const uint64_t vs[3] = {static_cast<uint64_t>(s.v_ss) * 2, nz(s.v_sh, s.v_ss), nz(s.v_sb, s.v_ss)};
    int rc = encode_tensor_map_bf16(&mk, k, 4, dims, ks, box);
    if (rc) return rc;
    rc = encode_tensor_map_bf16(&mv, v, 4, dims, vs, box);
    if (rc) return rc;
  }
  {
    const int rc = attention_decode_prepare();
    if (rc) return rc;
  }
  DecodeArgs a{};
  a.q = q;
  a.part_o = static_cast<float*>(scratch);
  a.part_ml = a.part_o + static_cast<size_t>(s.B) * s.Hq * max_chunks * kHD;
  a.q_sb = s.q_sb; a.q_sh = s.q_sh;
  a.o = o; a.o_sb = s.o_sb; a.o_sh = s.o_sh;
  a.Hkv = s.Hkv; a.G = G; a.max_chunks = max_chunks;
  a.kv_len = kv_len; a.kv_len_dev = kv_len_dev;
  a.fresh_rows = fresh_rows;
  if (rope) {
    if (!rope->k_new || !rope->v_new || !rope->k_cache || !rope->v_cache || !rope->q_w || !rope->k_w || !rope->cos_t ||
        !rope->sin_t || rope->max_len <= 0)
      return TEENY_ERR_BAD_ARG;
    if ((rope->new_sb % 8) || ((reinterpret_cast<uintptr_t>(rope->k_new) | reinterpret_cast<uintptr_t>(rope->v_new) |
                                reinterpret_cast<uintptr_t>(rope->q_w) | reinterpret_cast<uintptr_t>(rope->k_w) |
                                reinterpret_cast<uintptr_t>(rope->cos_t) | reinterpret_cast<uintptr_t>(rope->sin_t)) & 15))
      return TEENY_ERR_ALIGNMENT;
    a.rope = *rope;
    a.kc_sb = s.k_sb; a.kc_sh = s.k_sh; a.kc_ss = s.k_ss;
    a.vc_sb = s.v_sb; a.vc_sh = s.v_sh; a.vc_ss = s.v_ss;
  }
  a.scale_log2 = s.scale * 1.4426950408889634f;
  a.err = device_error_word();
  if (!a.err) return TEENY_ERR_DRIVER;  // kernels report expired waits through this word: no launch without it
  // Split the sequence only as far as needed to fill the GPU.  With B * Hkv at (or near) two CTAs per SM, each CTA
  // walks its whole sequence behind a three-stage ring and writes the output itself.  With fewer, the grid is sized
  // to at most one CTA per SM and each CTA gets the whole shared memory as a six-stage ring (the same bytes in flight
  // per SM).  Split sequences are merged by the last CTA to finish when the caller provides arrival counters,
  // otherwise by a second kernel.
  const int bh = s.B * s.Hkv, sms = sm_count();
  int n_split = 1;
  a.stages = kDecStagesShared;
  if (bh * 4 < sms * 2 * 3) {  // fewer than 3/4 of the two-per-SM slots
    a.stages = kDecStagesAlone;
    n_split = sms / bh;
    if (n_split > max_chunks) n_split = max_chunks;
    if (n_split < 1) n_split = 1;
  }
  a.counters = n_split > 1 ? counters : nullptr;
  const int smem = dec_smem_bytes(a.stages);
  dim3 grid(n_split, s.Hkv, s.B);
  switch (G) {
    case 1: launch_kernel(attention_decode_kernel<1>, grid, dim3(kDecThreads), smem, stream, 1, mk, mv, a); break;
    case 2: launch_kernel(attention_decode_kernel<2>, grid, dim3(kDecThreads), smem, stream, 1, mk, mv, a); break;
    case 4: launch_kernel(attention_decode_kernel<4>, grid, dim3(kDecThreads), smem, stream, 1, mk, mv, a); break;
    default: launch_kernel(attention_decode_kernel<8>, grid, dim3(kDecThreads), smem, stream, 1, mk, mv, a); break;
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return static_cast<int>(e);
  if (n_split == 1 || a.counters) return 0;
  launch_kernel(attention_decode_combine_kernel, dim3(s.Hq, s.B), dim3(kHD), 0, stream, 1, a.part_o, a.part_ml, o,
                s.o_sb, s.o_sh, s.Hkv, G, max_chunks, n_split, kv_len, kv_len_dev);
  return static_cast<int>(cudaGetLastError());
}

// ------------------------------------------------------------------------------------------------
// Decode attention without a caller-provided scratch buffer.
//
// Some hosts cannot hand this library device memory beyond the tensors themselves: an inference server whose
// allocator reserved every byte of HBM at start-up, or a steady-state decode loop in which a driver allocation is
// forbidden because cudaMalloc synchronises the whole device.  For them the split-KV partials live in the
// fixed-size device array below (part of the library image: every GPU that loads the library holds these bytes
// until the process exits).  Shapes whose partials do not fit are rejected, not truncated.
//
// All calls on one device share the array.  Nothing in it needs to start at zero -- every partial that the
// combine step reads was written by the same call -- but two calls that overlap on the GPU (different streams)
// would write the same slots, so such calls race and must be serialised by the caller.
// ------------------------------------------------------------------------------------------------
namespace {
constexpr size_t kStaticDecodeScratchBytes = size_t(8) << 20;  // 8 MiB, e.g. B=32, Hq=32, cache capacity 4096
static __device__ __align__(256) unsigned char g_static_decode_scratch[kStaticDecodeScratchBytes];
void* g_static_decode_scratch_ptr[64] = {};  // per device: resolved address of the array
}  // namespace

size_t attention_decode_static_scratch_limit() { return kStaticDecodeScratchBytes; }

int attention_decode_bf16_static(const bf16* q, const bf16* k, const bf16* v, bf16* o, const AttnShape& s, int kv_len,
                                 const int* kv_len_dev, cudaStream_t stream) {
  const size_t need = attention_decode_scratch_bytes(s.B, s.Hq, s.D, s.Skv);
  if (need == 0) return TEENY_ERR_BAD_ARG;
  if (need > kStaticDecodeScratchBytes) return TEENY_ERR_STATIC_LIMIT;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 0 || dev >= 64) return TEENY_ERR_BAD_ARG;
  if (!g_static_decode_scratch_ptr[dev]) {
    // In host code the array's name is only a handle: the address a kernel can use comes from the runtime, once
    // per device, with that device current.
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_decode_scratch);
    if (e != cudaSuccess) return static_cast<int>(e);
    g_static_decode_scratch_ptr[dev] = p;
  }
  return attention_decode_bf16(q, k, v, o, s, kv_len, kv_len_dev, g_static_decode_scratch_ptr[dev],
                               kStaticDecodeScratchBytes, stream);
}

template <typename T>
int attention_generic(const T* q, const T* k, const T* v, T* o, float* lse, const AttnShape& s, cudaStream_t stream) {
  if (!q || !k || !v || !o || s.B <= 0 || s.Hq <= 0 || s.Hkv <= 0 || s.Sq <= 0 || s.Skv <= 0 || s.D <= 0)
    return TEENY_ERR_BAD_ARG;
  if (s.D > 256 || s.Hq % s.Hkv != 0 || (s.causal && s.Skv < s.Sq)) return TEENY_ERR_BAD_ARG;
  const long long rows = static_cast<long long>(s.B) * s.Hq * s.Sq;
  const long long blocks = (rows + 3) / 4;
  if (blocks > 0x7fffffffLL) return TEENY_ERR_BAD_ARG;
  launch_kernel(attention_generic_kernel<T>, dim3(static_cast<int>(blocks)), dim3(128), 0, stream, 1, q, k, v, o, lse, s);
  return static_cast<int>(cudaGetLastError());
}
template int attention_generic<float>(const float*, const float*, const float*, float*, float*, const AttnShape&, cudaStream_t);
template int attention_generic<bf16>(const bf16*, const bf16*, const bf16*, bf16*, float*, const AttnShape&, cudaStream_t);

}  // namespace teeny
