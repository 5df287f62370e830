// Causal grouped-query flash-attention forward for sm_100a, head_dim 128, bf16 in/out, f32 softmax, on CTA pairs.
//
// A cluster of two CTAs (two neighbouring SMs) takes 256 queries of one (head, batch): CTA r owns query rows
// [q0 + 128 r, q0 + 128 r + 128).  Keys / values stream through in tiles of 128 keys.  Every tcgen05.mma is issued by
// the leader CTA for the pair (cta_group::2, M = 256): the instruction takes rows 0-127 of its A operand and output
// from the leader's tensor memory and rows 128-255 from the peer's, and HALF of its B operand from each CTA's shared
// memory.  So each SM loads and re-reads only half of every K and V tile, and neither Q nor P is read from shared
// memory at all (both are A operands in tensor memory): per key tile an SM's shared memory sees 32 KB of TMA writes
// and 32 KB of operand reads for 1024 tensor-pipe cycles, where a lone 128 x 128 tile with Q in shared memory needs
// 64 KB + 96 KB -- more than the port delivers in that time, which is what held a single-CTA version of this kernel at
// 43 % tensor-pipe activity.  No multicast loads: each CTA's TMA fetches its own half; only completions
// (tcgen05.commit) are delivered to both CTAs.
//
//   warp 0       K producer (both CTAs): its 64 keys x 128 d of each key tile (two 8 KB boxes), ring of kKV stages;
//                transaction bytes of both CTAs are credited to the leader's barrier.
//   warp 3       V producer (both CTAs): all 128 keys x its 64 d columns (one 16 KB box), ring of its own: K runs two
//                tiles ahead of V and must not queue behind it.
//   warps 1, 2   MMA issuers (leader only), one thread each.  Warp 1: S = Q K^T (A = Q from tensor memory, B = K,
//                K-major) into one of two S buffers, as far ahead of P V as the buffers allow (an S buffer is free
//                again as soon as its softmax group of both CTAs has the rows in registers), so the tensor pipe works
//                while the softmax groups run.  Warp 2: O += P V (A = P from tensor memory, B = V MN-major straight
//                from its [key][d] tile).  Two threads because a lone thread cannot issue these 64-cycle instructions
//                fast enough, and so that neither stream waits behind the other's barriers.
//   warp 2       also allocates / frees tensor memory (cta_group::2, both CTAs).
//   warps 4-7, 8-11   two softmax warpgroups per CTA, thread = query row in both; the groups take the pair's key tiles
//                alternately (S buffer = tile parity), so one group's exponentials run while the other scans its next
//                tile.  Per tile: tcgen05.ld the S row (four loads in flight), row maximum (causal / tail mask; three-
//                input maxima), agreement on the running maximum with the other group (shared memory; a tile's
//                decision waits for the previous tile's), lazy rescale (O in tensor memory is only rescaled when the
//                maximum grows by more than 2^8), P = exp2(s * scale - m) (packed fp32 multiply-adds and adds) as bf16
//                pairs into the one P buffer in tensor memory (free once P V of the previous tile has completed), row
//                sums in f32 per group.
//                (Registers re-divided with setmaxnreg: 224 per softmax thread, 56 per service thread.)
//
// The grid is persistent: one CTA pair per SM pair walks a list of (256-query tile, head, batch) items, heaviest first;
// key tiles are counted across items, so ring stages, S-buffer parities and barrier phases carry on from one item into
// the next and the producers and the Q K^T issuer run ahead into the next item.  At an item's end the two softmax
// groups part: the one that took the last tile ("closer") adds the other's row sum to its own, waits for the last P V,
// reads O out of tensor memory, frees it for the next item at once and sends the rows out (bf16 into swizzled boxes in
// shared memory, one TMA store per warp and box; optional LSE = ln2 * (m + log2 l)); the other ("opener") hands over
// its row sum and running maximum, copies the next item's Q rows -- fetched by TMA into a staging box an item ahead --
// from shared into tensor memory as soon as the item's last Q K^T has completed, and goes on with the next item's first
// tile.  Values the groups exchange (running maximum, row sums) and the barriers that guard them alternate with the
// item, because the opener is up to one item ahead of the closer.  (Plain 16-byte-per-row loads of Q and stores of O
// kept the load/store unit busy for ~2000 cycles per item each: a warp instruction touched 32 lines.)
// Tensor memory columns per CTA: S0 0-127, S1 128-255 (f32 scores), O 256-383 (f32), Q 384-447, P 448-511 (bf16 pairs).
#include <atomic>

#include "common.cuh"
#include "kernels.h"

namespace teeny {

namespace {

constexpr int kQT = 128;                        // query rows per CTA (pair: 256)
constexpr int kKT = 128;                        // keys per tile
constexpr int kHD = 128;
constexpr int kThreads = 384;                   // TMA K, MMA QK, MMA PV + TMEM, TMA V; two softmax warpgroups
constexpr int kHalfBytes = 64 * kHD * 2;        // 16 KB: this CTA's half of a K tile (64 keys) or of a V tile (64 d)
constexpr int kKBoxBytes = 64 * 64 * 2;         // 8 KB: [64 keys][64 d]
constexpr int kKV = 4;                          // stages of the K ring and of the V ring
constexpr int kSmemK = 0;
constexpr int kSmemV = kSmemK + kKV * kHalfBytes;
constexpr int kSmemQ = kSmemV + kKV * kHalfBytes;   // 32 KB: the next item's Q rows of this CTA, two [128 rows][64 d] boxes
constexpr int kSmemO = kSmemQ + 2 * kQT * 128;      // 32 KB: output rows on their way out, per warp quarter two [32 rows][64 d] boxes
constexpr int kSmemBar = kSmemO + 2 * kQT * 128;
constexpr int kSmemXch = kSmemBar + 512;        // per item parity: running maximum per row, and the row sum / maximum the
                                                // group that leaves an item first hands to the one that finishes it
constexpr int kSmemTotal = kSmemXch + 2 * 3 * 128 * 4 + 1024;
static_assert(kSmemTotal <= 232448, "exceeds the 227 KB of shared memory a CTA can have");
constexpr float kRescaleThreshold = 8.0f;       // log2 units
constexpr uint32_t kPeerBitMask = 0xFEFFFFFFu;  // clears the CTA-rank bit of a shared::cluster address -> leader

struct PrefillArgs {  // (Q, K, V and O travel as tensor maps)
  float* lse;
  int B, Hq, Hkv, Sq, Skv;
  float scale_log2;
  int causal;
  int n_pair_tiles;  // 256-row query tiles per (batch, head)
  int n_items;       // n_pair_tiles * Hq * B work items; CTA pair p takes items p, p + pairs, ...
  int* err;
};

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Development builds: clock of event `id` at key tile g of CTA 0, for a window of twenty tiles in the middle of its list
// (kept in shared memory and written out when the CTA is done, so that the stamps cost a store each;
// `python -m teenygrad_b200.microbench timeline` prints them in order).
#ifdef TEENY_TRACE
#define TL(id, g, c) do { if ((c) && blockIdx.x == 0 && (g) >= 196 && (g) < 216) tl_sh[id][(g) - 196] = clock64(); } while (0)
#else
#define TL(id, g, c) do {} while (0)
#endif
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float y;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(y) : "f"(a), "f"(b), "f"(c));
  return y;
}
__device__ __forceinline__ uint32_t pair_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void pair_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t map_to_leader(uint32_t local_addr) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(0u));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// This CTA's half tile; completion bytes are credited to the LEADER's barrier at the same offset.
__device__ __forceinline__ void tma_load_4d_pair(uint32_t dst, const CUtensorMap* m, uint32_t bar, int x, int y, int z, int w) {
  asm volatile(
      "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar & kPeerBitMask), "r"(x), "r"(y), "r"(z), "r"(w)
      : "memory");
}
// Rows of shared memory (128-byte-swizzled boxes) -> global through the tensor map, as one bulk group of the calling thread.
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* m, uint32_t src, int x, int y, int z, int w) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(m)), "r"(src), "r"(x), "r"(y), "r"(z), "r"(w)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// every bulk store of this thread has read its shared memory (immediate for a thread that issued none)
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// The eight K-steps of one 128-deep product for the pair, D[tmem] (+)= A[tmem] * B[smem] (rows 0-127 in the leader,
// 128-255 in the peer), as one block of straight-line code: A advances eight tensor-memory columns per step, the
// address field of the B descriptor by the compile-time offsets O1..O7 (16-byte units).  One thread issues a
// tcgen05.mma only every ~100 cycles when address arithmetic sits between them (a lone lane runs a dependent
// instruction every few cycles), which is more than the 64 cycles the tensor pipe needs for one of these steps.
template <int O1, int O2, int O3, int O4, int O5, int O6, int O7>
__device__ __forceinline__ void umma_bf16_ts_pair_x8(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                                     uint32_t accumulate_first) {
  asm volatile(
      "{\n\t.reg .pred p, t;\n\t.reg .b64 b;\n\t.reg .b32 a;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "setp.eq.b32 t, %3, %3;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      "add.u32 a, %1, 8;\n\t add.u64 b, %2, %5;\n\t tcgen05.mma.cta_group::2.kind::f16 [%0], [a], b, %3, t;\n\t"
      "add.u32 a, %1, 16;\n\t add.u64 b, %2, %6;\n\t tcgen05.mma.cta_group::2.kind::f16 [%0], [a], b, %3, t;\n\t"
      "add.u32 a, %1, 24;\n\t add.u64 b, %2, %7;\n\t tcgen05.mma.cta_group::2.kind::f16 [%0], [a], b, %3, t;\n\t"
      "add.u32 a, %1, 32;\n\t add.u64 b, %2, %8;\n\t tcgen05.mma.cta_group::2.kind::f16 [%0], [a], b, %3, t;\n\t"
      "add.u32 a, %1, 40;\n\t add.u64 b, %2, %9;\n\t tcgen05.mma.cta_group::2.kind::f16 [%0], [a], b, %3, t;\n\t"
      "add.u32 a, %1, 48;\n\t add.u64 b, %2, %10;\n\t tcgen05.mma.cta_group::2.kind::f16 [%0], [a], b, %3, t;\n\t"
      "add.u32 a, %1, 56;\n\t add.u64 b, %2, %11;\n\t tcgen05.mma.cta_group::2.kind::f16 [%0], [a], b, %3, t;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate_first), "n"(O1), "n"(O2), "n"(O3), "n"(O4), "n"(O5),
        "n"(O6), "n"(O7)
      : "memory");
}
// Arrives on the barrier at this offset in BOTH CTAs of the pair once all MMAs issued so far have completed.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(bar), "h"(static_cast<uint16_t>(3))
      : "memory");
}

__global__ void __launch_bounds__(kThreads, 1)
attention_prefill_kernel(const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                         const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_o,
                         const PrefillArgs args) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t bar0 = base + kSmemBar;
  auto bar = [&](int i) { return bar0 + 8u * i; };
  // K_FULL / V_FULL / S_EMPTY / P_FULL / Q_READY are used in the leader's copy only (the peer's producers and softmax
  // threads signal them across the pair); the others exist and are used in both CTAs
  constexpr int Q_READY = 0, K_FULL = 1, K_EMPTY = K_FULL + kKV, V_FULL = K_EMPTY + kKV, V_EMPTY = V_FULL + kKV,
                S_FULL = V_EMPTY + kKV, S_EMPTY = S_FULL + 2, P_FULL = S_EMPTY + 2, PV_DONE = P_FULL + 1,
                M_READY = PV_DONE + 2, O_FREE = M_READY + 4, L_READY = O_FREE + 1, QS_FULL = L_READY + 2,
                QS_FREE = QS_FULL + 1, kNumBars = QS_FREE + 1;
  static_assert(8 * kNumBars + 8 <= 512, "barrier block");
  const uint32_t tmem_slot = bar0 + 8u * kNumBars;
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(gen + kSmemBar + 8 * kNumBars);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = pair_rank();
  const bool leader = rank == 0;
  int* err = args.err;

  // Work items = (query tile of 256 rows, head, batch), the heavier (later) query tiles first: with causal masking they
  // have the most key tiles.  The pair walks items pair_id, pair_id + n_pairs, ...; every role walks the same list and
  // counts key tiles across items (`g`), so ring stages, buffer parities and barrier phases simply continue from one
  // item into the next: the loads of the next item's keys and values, and its first products, overlap the current
  // item's last softmax steps and output.
  const int pair_id = static_cast<int>(blockIdx.x >> 1), n_pairs = static_cast<int>(gridDim.x >> 1);
  const int off = args.Skv - args.Sq;                           // causal: query i sees keys <= i + off
  const int heads_x_batch = args.Hq * args.B;
  struct Item { int pt, h, b, hk, n_tiles; };
  auto item_at = [&](int item) {
    Item it;
    it.pt = args.n_pair_tiles - 1 - item / heads_x_batch;
    const int rest = item % heads_x_batch;
    it.b = rest / args.Hq;
    it.h = rest % args.Hq;
    it.hk = it.h / (args.Hq / args.Hkv);
    int kv_end = args.Skv;
    if (args.causal) kv_end = min(args.Skv, it.pt * 2 * kQT + 2 * kQT + off);   // of the pair's last row
    it.n_tiles = (kv_end + kKT - 1) / kKT;  // >= 1 (host guarantees Skv >= Sq >= 1 when causal)
    return it;
  };

  TRACE_ONLY(__shared__ long long tl_sh[12][20]; if (threadIdx.x < 240) (&tl_sh[0][0])[threadIdx.x] = 0;)
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_o);
    for (int i = 0; i < kNumBars; ++i) {
      uint32_t count = 1;
      if (i == Q_READY || i == O_FREE) count = 256;         // one softmax group of each CTA
      else if (i == S_EMPTY || i == S_EMPTY + 1 || i == P_FULL) count = 256;
      else if ((i >= M_READY && i < M_READY + 4) || i == L_READY || i == L_READY + 1 || i == QS_FREE) count = 128;
      mbar_init(bar(i), count);
    }
    mbar_fence_init();
  }
  if (warp == 2) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  pair_sync();  // both CTAs' barriers exist before either CTA can signal the other
  tc_fence_after();
  const uint32_t tmem = *tmem_slot_ptr;
  const uint32_t tmem_s0 = tmem, tmem_o = tmem + 256, tmem_q = tmem + 384, tmem_p = tmem + 448;
  pdl_wait();

  // The two softmax warpgroups hold a 128-value score row per thread; the four service warps need few registers:
  // each side re-sizes its register file share at the top of its own branch.
  if (warp < 4) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
  if (warp == 0) {
    if (lane == 0) {  // this CTA's 64 keys of every K tile
      bool ok = true;
      for (int item = pair_id, g = 0; ok && item < args.n_items; item += n_pairs) {
        const Item it = item_at(item);
        for (int j = 0; j < it.n_tiles; ++j, ++g) {
          const int st = g % kKV;
          const uint32_t ph = (g / kKV) & 1;
          if (!mbar_wait(bar(K_EMPTY + st), ph ^ 1, err, DEVERR_ATTN_PRODUCER)) { ok = false; break; }
          if (leader) mbar_expect_tx(bar(K_FULL + st), 2 * kHalfBytes);  // both CTAs' halves
          const uint32_t dst = base + kSmemK + st * kHalfBytes;
          const int key0 = j * kKT + static_cast<int>(rank) * 64;
          tma_load_4d_pair(dst, &tmap_k, bar(K_FULL + st), 0, key0, it.hk, it.b);
          tma_load_4d_pair(dst + kKBoxBytes, &tmap_k, bar(K_FULL + st), 64, key0, it.hk, it.b);
        }
      }
    }
  } else if (warp == 3) {
    if (lane == 0) {  // this CTA's 64 d columns of every V tile
      bool ok = true;
      for (int item = pair_id, g = 0; ok && item < args.n_items; item += n_pairs) {
        const Item it = item_at(item);
        for (int j = 0; j < it.n_tiles; ++j, ++g) {
          const int st = g % kKV;
          const uint32_t ph = (g / kKV) & 1;
          if (!mbar_wait(bar(V_EMPTY + st), ph ^ 1, err, DEVERR_ATTN_PRODUCER)) { ok = false; break; }
          if (leader) mbar_expect_tx(bar(V_FULL + st), 2 * kHalfBytes);
          tma_load_4d_pair(base + kSmemV + st * kHalfBytes, &tmap_v, bar(V_FULL + st), static_cast<int>(rank) * 64, j * kKT,
                           it.hk, it.b);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- QK^T issuer (leader only) ----------------
    // Two issuing threads, this one and warp 2's: their instruction streams are independent (S buffers here, O there),
    // neither waits for the other's barriers, and together they keep the tensor pipe fed.
    if (leader && lane == 0) {
      constexpr uint32_t idesc_qk = make_idesc_bf16(2 * kQT, kKT, false, false);
      // K-major B: 8-row groups 1 KB apart; ring stage s is kHalfBytes further on
      const uint64_t kdesc0 = make_smem_desc_sw128(base + kSmemK, 16, 1024);
      // development builds: cycles this thread spends waiting for K and for a free S buffer (summed over the tiles)
      TRACE_ONLY(long long w_k = 0, w_se = 0, c0; const long long c_begin = clock64();)
      bool ok = true;
      int g = 0;
      for (int item = pair_id, seq = 0; ok && item < args.n_items; item += n_pairs, ++seq) {
        const Item it = item_at(item);
        if (!mbar_wait(bar(Q_READY), seq & 1, err, DEVERR_ATTN_MMA)) break;  // this item's Q is in tensor memory
        for (int j = 0; j < it.n_tiles; ++j, ++g) {
          const int sb = g & 1, kst = g % kKV;  // S buffer / K ring stage
          const uint32_t ph = (g >> 1) & 1, kph = (g / kKV) & 1;
          TRACE_ONLY(c0 = clock64();)
          if (!mbar_wait(bar(K_FULL + kst), kph, err, DEVERR_ATTN_MMA)) { ok = false; break; }
          TRACE_ONLY(w_k += clock64() - c0; c0 = clock64();)
          // an S buffer is free again as soon as its softmax groups (of both CTAs) have the rows in registers
          if (!mbar_wait(bar(S_EMPTY + sb), ph ^ 1, err, DEVERR_ATTN_MMA)) { ok = false; break; }
          TRACE_ONLY(w_se += clock64() - c0;)
          TL(0, g, true);
          tc_fence_after();
          // 16 d per step: 8 tensor-memory columns of Q; 32 bytes along a K box row, the second box 8 KB further on
          constexpr int B2 = kKBoxBytes >> 4;
          umma_bf16_ts_pair_x8<2, 4, 6, B2, B2 + 2, B2 + 4, B2 + 6>(tmem_s0 + sb * 128, tmem_q,
                                                                     kdesc0 + static_cast<uint64_t>(kst * (kHalfBytes >> 4)),
                                                                     idesc_qk, 0u);
          umma_commit_pair(bar(K_EMPTY + kst));
          umma_commit_pair(bar(S_FULL + sb));
          TL(1, g, true);
        }
      }
      TRACE_VALUE(0, true, g);
      TRACE_VALUE(1, true, clock64() - c_begin);
      TRACE_VALUE(2, true, w_k);
      TRACE_VALUE(3, true, w_se);
    }
  } else {
    // ---------------- P V issuer (warp 2, leader only) ----------------
    if (leader && lane == 0) {
      constexpr uint32_t idesc_pv = make_idesc_bf16(2 * kQT, kHD, false, true);
      // MN-major B, this CTA's V half: rows = keys (128 B = its 64 d each), 8-key groups 1 KB apart; 16 keys = 2 KB per step
      const uint64_t vdesc0 = make_smem_desc_sw128(base + kSmemV, kHalfBytes, 1024);
      TRACE_ONLY(long long w_v = 0, w_p = 0, c0; const long long c_begin = clock64();)
      bool ok = true;
      int g = 0;
      for (int item = pair_id, seq = 0; ok && item < args.n_items; item += n_pairs, ++seq) {
        const Item it = item_at(item);
        // the output accumulator is free once the softmax threads have read the previous item's out of it
        if (seq > 0 && !mbar_wait(bar(O_FREE), (seq - 1) & 1, err, DEVERR_ATTN_MMA)) break;
        for (int j = 0; j < it.n_tiles; ++j, ++g) {
          const int sb = g & 1, vst = g % kKV;  // tile parity / V ring stage
          const uint32_t vph = (g / kKV) & 1;
          TRACE_ONLY(c0 = clock64();)
          if (!mbar_wait(bar(V_FULL + vst), vph, err, DEVERR_ATTN_MMA)) { ok = false; break; }
          TRACE_ONLY(w_v += clock64() - c0; c0 = clock64();)
          if (!mbar_wait(bar(P_FULL), static_cast<uint32_t>(g & 1), err, DEVERR_ATTN_MMA)) { ok = false; break; }  // one phase per tile
          TRACE_ONLY(w_p += clock64() - c0;)
          TL(2, g, true);
          tc_fence_after();
          // 16 keys per step: 8 columns of packed bf16 pairs of P in tensor memory, 2 KB of the V tile
          umma_bf16_ts_pair_x8<128, 256, 384, 512, 640, 768, 896>(tmem_o, tmem_p,
                                                                  vdesc0 + static_cast<uint64_t>(vst * (kHalfBytes >> 4)),
                                                                  idesc_pv, j > 0 ? 1u : 0u);
          umma_commit_pair(bar(V_EMPTY + vst));
          umma_commit_pair(bar(PV_DONE + sb));
          TL(9, g, true);
        }
      }
      TRACE_VALUE(12, true, clock64() - c_begin);
      TRACE_VALUE(4, true, w_v);
      TRACE_VALUE(5, true, w_p);
    }
  }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 224;");
    const int quarter = warp & 3;
    const int wg = (warp - 4) >> 2;     // softmax warpgroup: key tiles j = wg, wg + 2, ...; S buffer wg
    const int r = quarter * 32 + lane;  // query row in this CTA's tile == TMEM lane
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t s_addr = tmem_s0 + lane_addr + wg * 128;
    const uint32_t p_full_leader = map_to_leader(bar(P_FULL)), s_empty_leader = map_to_leader(bar(S_EMPTY + wg));
    float* xch = reinterpret_cast<float*>(gen + kSmemXch);  // [item parity][m | l | mu][128]
    bool ok = true;

    // All 128 d columns of this thread's Q row of an item, global -> tensor memory (by the ONE group that opens the item)
    // An item's Q rows of this CTA, global -> the staging boxes in shared memory (one thread; an item ahead of their use)
    auto fetch_q = [&](const Item& it) {
      const int y = it.pt * 2 * kQT + static_cast<int>(rank) * kQT;
      mbar_expect_tx(bar(QS_FULL), 2 * kQT * 128);
      tma_load_4d(base + kSmemQ, &tmap_q, bar(QS_FULL), 0, y, it.h, it.b);
      tma_load_4d(base + kSmemQ + kQT * 128, &tmap_q, bar(QS_FULL), 64, y, it.h, it.b);
    };
    // ... and from there into tensor memory, each thread its row (by the ONE group that opens the item; n = how many
    // items this pair opened before).  Row r's 16-byte chunk c of a box sits at chunk c ^ (r & 7) of its 128 bytes.
    auto put_q = [&](int n) {
      if (ok) ok = mbar_wait(bar(QS_FULL), n & 1, err, DEVERR_ATTN_SOFTMAX);
      const uint8_t* row = gen + kSmemQ + r * 128;
#pragma unroll
      for (int hb = 0; hb < 2; ++hb) {
        uint32_t qw[32];
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint4 t = *reinterpret_cast<const uint4*>(row + hb * (kQT * 128) + ((c ^ (r & 7)) << 4));
          qw[4 * c] = t.x; qw[4 * c + 1] = t.y; qw[4 * c + 2] = t.z; qw[4 * c + 3] = t.w;
        }
        tmem_st_32x32(tmem_q + lane_addr + hb * 32, qw);
      }
      mbar_arrive(bar(QS_FREE));  // the boxes can take the item after this one
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive_cluster(map_to_leader(bar(Q_READY)));
    };
    // The first item: group 1 brings Q in while group 0, which takes tile 0, has nothing else to do either.
    if (wg == 1 && pair_id < args.n_items) {
      if (r == 0) fetch_q(item_at(pair_id));
      put_q(0);
    }

    // development builds: cycles of thread 128 per phase (wait for S, load + scan, decision, exp, wait for the P buffer)
    TRACE_ONLY(long long w_s = 0, w_s0 = 0, t_ld = 0, t_max = 0, w_pv = 0, t_exp = 0, t_end = 0, t_close = 0, c0; const long long c_begin = clock64();)
    int g0 = 0;  // key tiles of the items before this one: tile j of the item is tile g0 + j of the pair
    uint32_t m_seen0 = 0, m_seen1 = 0;
    Item next_it = item_at(pair_id < args.n_items ? pair_id : 0);
#pragma unroll 1
    for (int item = pair_id, seq = 0; item < args.n_items; item += n_pairs, ++seq) {
      const Item it = next_it;  // worked out during the previous item's last waits: the divisions are off this group's path
      const int n_tiles = it.n_tiles;
      const int q0 = it.pt * 2 * kQT + static_cast<int>(rank) * kQT;   // this CTA's first query row
      const int qi = q0 + r;
      float* m_sh = xch + (seq & 1) * 384;  // running maximum of the item's rows, log2 domain
      float* l_sh = m_sh + 128;             // row sum ...
      float* mu_sh = m_sh + 256;            // ... and the maximum it is relative to, of the group that leaves first
      float m_used = -INFINITY, l = 0.0f;   // the maximum this group's sums are relative to
      const int glast = g0 + n_tiles - 1;
      const bool closer = (glast & 1) == wg;  // this group takes the item's last tile and writes its output
      // The "maximum decided" barriers alternate with the item like the values they guard: the group that opens the
      // next item decides its first tile before the other group has looked at this item's last decision, and one
      // barrier would then be two completions ahead of that wait.  The other group's tiles of the item are j_other,
      // j_other + 2, ...; m_seen counts the completions of its barrier before this item.
      const int m_ready = M_READY + (seq & 1) * 2;
      const int j_other = (wg ^ 1) ^ (g0 & 1);
      const uint32_t m_seen = (seq & 1) ? m_seen1 : m_seen0;
      const bool more = item + n_pairs < args.n_items;
      if (!closer && more && r == 0) {
        // this group brings the next item's Q in, an item from now: fetch it as soon as this item's has left the boxes
        if (ok) ok = mbar_wait(bar(QS_FREE), seq & 1, err, DEVERR_ATTN_SOFTMAX);
        if (ok) fetch_q(item_at(item + n_pairs));
      }
      // this group takes the pair's tiles of parity wg (S buffer wg), whichever items they belong to
#pragma unroll 1
      for (int j = (wg ^ (g0 & 1)); ok && j < n_tiles; j += 2) {
        const int g = g0 + j;
        const uint32_t ph = (g >> 1) & 1;
        TRACE_ONLY(c0 = clock64();)
        if (!mbar_wait(bar(S_FULL + wg), ph, err, DEVERR_ATTN_SOFTMAX)) { ok = false; break; }
        TRACE_ONLY(w_s += clock64() - c0; if (j < 2) w_s0 += clock64() - c0; c0 = clock64();)
        TL(3, g, r == 0);
        tc_fence_after();
        // the S row into registers (raw scores: the scale is folded into the exponent)
        float s[128];
        {
          uint32_t t0[32], t1[32], t2[32], t3[32];  // four loads in flight, one wait
          tmem_ld_32x32(s_addr, t0);
          tmem_ld_32x32(s_addr + 32, t1);
          tmem_ld_32x32(s_addr + 64, t2);
          tmem_ld_32x32(s_addr + 96, t3);
          tmem_wait_ld();
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            s[e] = __uint_as_float(t0[e]);
            s[32 + e] = __uint_as_float(t1[e]);
            s[64 + e] = __uint_as_float(t2[e]);
            s[96 + e] = __uint_as_float(t3[e]);
          }
        }
        tc_fence_before();
        mbar_arrive_cluster(s_empty_leader);  // the buffer can take QK^T of tile g + 2 (once the peer's group is here too)
        const int k0 = j * kKT;
        const bool need_mask = (k0 + kKT > args.Skv) || (args.causal && (k0 + kKT - 1 > q0 + off));
        if (need_mask) {
          const int limit = args.causal ? min(args.Skv - 1, qi + off) : args.Skv - 1;  // last visible key
#pragma unroll
          for (int e = 0; e < 128; ++e)
            if (k0 + e > limit) s[e] = -INFINITY;
        }
        // row maximum: four independent chains of three-input maxima
        float tm[4] = {s[0], s[1], s[2], s[3]};
#pragma unroll
        for (int e = 4; e + 8 <= 128; e += 8) {
          tm[0] = fmax3(tm[0], s[e], s[e + 1]);
          tm[1] = fmax3(tm[1], s[e + 2], s[e + 3]);
          tm[2] = fmax3(tm[2], s[e + 4], s[e + 5]);
          tm[3] = fmax3(tm[3], s[e + 6], s[e + 7]);
        }
        tm[0] = fmax3(tm[0], s[124], s[125]);
        tm[1] = fmax3(tm[1], s[126], s[127]);
        const float tmax = fmaxf(fmax3(tm[0], tm[1], tm[2]), tm[3]) * args.scale_log2;  // log2 domain (scale > 0)
        TRACE_ONLY(t_ld += clock64() - c0; c0 = clock64();)
        TL(4, g, r == 0);
        // ---- the running maximum: tile j's decision follows tile j-1's (made by the other group) ----
        float m;
        if (j == 0) {
          m = tmax;  // key 0 is visible to every row, so m is finite from here on
        } else {
          if (!mbar_wait(bar(m_ready + (wg ^ 1)), (m_seen + ((j - 1 - j_other) >> 1)) & 1, err, DEVERR_ATTN_SOFTMAX)) { ok = false; break; }
          m = m_sh[r];
          const float m_new = fmaxf(m, tmax);
          const bool grow = m_new > m + kRescaleThreshold;
          if (__any_sync(0xffffffffu, grow)) {
            // O must be final for tile j-1 before it is rescaled
            if (!mbar_wait(bar(PV_DONE + ((g - 1) & 1)), ((g - 1) >> 1) & 1, err, DEVERR_ATTN_SOFTMAX)) { ok = false; break; }
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
        mbar_arrive(bar(m_ready + wg));  // tile j + 1 may decide (and rescale O) now
        if (m_used != m) {                // this group's sums follow the maximum (no-op while l == 0)
          l *= fast_exp2(m_used - m);
          m_used = m;
        }
        TRACE_ONLY(t_max += clock64() - c0; c0 = clock64();)
        TL(5, g, r == 0);
        // probabilities as bf16 pairs (the A operand of P V), into registers first: the one P buffer in tensor memory is
        // free only when P V of the previous tile (the other group's) has completed, and that must not hold up the
        // exponentials
        // (two scores per multiply-add and per addition: the packed fp32 forms halve the issue slots next to the exponentials)
        float2 ls[2] = {{0.0f, 0.0f}, {0.0f, 0.0f}};
        const float2 sc2 = {args.scale_log2, args.scale_log2}, neg_m2 = {-m, -m};
        uint32_t pk[64];
#pragma unroll
        for (int e = 0; e < 64; ++e) {
          const float2 x = __ffma2_rn(make_float2(s[2 * e], s[2 * e + 1]), sc2, neg_m2);  // masked scores are -inf -> 0
          const float2 pr = {fast_exp2(x.x), fast_exp2(x.y)};
          ls[e & 1] = __fadd2_rn(ls[e & 1], pr);
          pk[e] = pack_bf16x2(pr.x, pr.y);
        }
        TRACE_ONLY(t_exp += clock64() - c0; c0 = clock64();)
        TL(6, g, r == 0);
        if (g >= 1) {  // the previous tile of the pair -- of this item or of the one before -- has been multiplied
          if (!mbar_wait(bar(PV_DONE + ((g - 1) & 1)), ((g - 1) >> 1) & 1, err, DEVERR_ATTN_SOFTMAX)) { ok = false; break; }
          tc_fence_after();
        }
        TRACE_ONLY(w_pv += clock64() - c0; c0 = clock64();)
        TL(7, g, r == 0);
#pragma unroll
        for (int hc = 0; hc < 2; ++hc) {  // 64 keys = 32 packed columns per store
          uint32_t part[32];
#pragma unroll
          for (int e = 0; e < 32; ++e) part[e] = pk[hc * 32 + e];
          tmem_st_32x32(tmem_p + lane_addr + hc * 32, part);
        }
        tmem_wait_st();
        l += (ls[0].x + ls[0].y) + (ls[1].x + ls[1].y);
        tc_fence_before();
        mbar_arrive_cluster(p_full_leader);
        TL(8, g, r == 0);
      }
      TRACE_ONLY(c0 = clock64();)
      // ---- the item's end.  The group that took the last tile finishes the item (row sums, output); the other group
      // has been free since its own last tile: it hands over its row sum and moves on -- it opens the next item (Q into
      // tensor memory as soon as the last Q K^T of this item is complete) and takes that item's first tile, while the
      // first group is still on this item's last tile and output. ----
      bulk_wait_read();  // this thread's last output rows have left shared memory: whichever group writes there next has
      __syncwarp();      // waited for this point, here or through L_READY
      if (!closer) {
        l_sh[r] = l;
        mu_sh[r] = m_used;  // -inf (and l = 0) if this group had no tile in the item
        mbar_arrive(bar(L_READY + (seq & 1)));
        if (more) {
          // every product with this item's Q: complete when the last S tile is (the other group's buffer)
          if (ok) ok = mbar_wait(bar(S_FULL + (wg ^ 1)), (glast >> 1) & 1, err, DEVERR_ATTN_SOFTMAX);
          put_q(seq + 1);
          next_it = item_at(item + n_pairs);  // (the first products of the next item are on their way meanwhile)
        }
      } else {
        const float m_fin = m_used;  // this group decided the last tile
        if (more) next_it = item_at(item + n_pairs);  // (the last P V is still running)
        if (ok) ok = mbar_wait(bar(L_READY + (seq & 1)), (seq >> 1) & 1, err, DEVERR_ATTN_SOFTMAX);
        l += l_sh[r] * fast_exp2(mu_sh[r] - m_fin);  // 0 * 2^-inf = 0 for a group without tiles
        if (ok) ok = mbar_wait(bar(PV_DONE + (glast & 1)), (glast >> 1) & 1, err, DEVERR_ATTN_SOFTMAX);
        if (ok) {
          tc_fence_after();
          float inv;
          asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(inv) : "f"(l));  // l >= 1 (the row's maximum contributes 2^0); 1 ulp
          const float2 inv2 = {inv, inv};
          const bool valid = qi < args.Sq;
          uint32_t t[4][32];  // the whole row in flight, so that the accumulator is free for the next item at once
#pragma unroll
          for (int c = 0; c < 4; ++c) tmem_ld_32x32(tmem_o + lane_addr + c * 32, t[c]);
          tmem_wait_ld();
          tc_fence_before();
          mbar_arrive_cluster(map_to_leader(bar(O_FREE)));
          // bf16 rows into this warp's boxes (the swizzle the tensor map expects), then one bulk store per box: the
          // rows leave as full lines instead of 16 bytes per thread and row
          uint8_t* orow = gen + kSmemO + quarter * (32 * 256) + lane * 128;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              uint4 o4;
              const float2 a0 = __fmul2_rn(make_float2(__uint_as_float(t[c][v * 8 + 0]), __uint_as_float(t[c][v * 8 + 1])), inv2);
              const float2 a1 = __fmul2_rn(make_float2(__uint_as_float(t[c][v * 8 + 2]), __uint_as_float(t[c][v * 8 + 3])), inv2);
              const float2 a2 = __fmul2_rn(make_float2(__uint_as_float(t[c][v * 8 + 4]), __uint_as_float(t[c][v * 8 + 5])), inv2);
              const float2 a3 = __fmul2_rn(make_float2(__uint_as_float(t[c][v * 8 + 6]), __uint_as_float(t[c][v * 8 + 7])), inv2);
              o4.x = pack_bf16x2(a0.x, a0.y);
              o4.y = pack_bf16x2(a1.x, a1.y);
              o4.z = pack_bf16x2(a2.x, a2.y);
              o4.w = pack_bf16x2(a3.x, a3.y);
              const int ch = (c & 1) * 4 + v;  // chunk of the box's 128-byte row; columns 64.. are the second box
              *reinterpret_cast<uint4*>(orow + (c >> 1) * (32 * 128) + ((ch ^ (lane & 7)) << 4)) = o4;
            }
          }
          fence_proxy_async_smem();
          __syncwarp();
          const int y = q0 + quarter * 32;
          if (lane == 0 && y < args.Sq) {  // rows past the end are clipped by the copy
            const uint32_t src = base + kSmemO + quarter * (32 * 256);
            tma_store_4d(&tmap_o, src, 0, y, it.h, it.b);
            tma_store_4d(&tmap_o, src + 32 * 128, 64, y, it.h, it.b);
            bulk_commit();
          }
          if (valid && args.lse)
            args.lse[(static_cast<long long>(it.b) * args.Hq + it.h) * args.Sq + qi] = 0.6931471805599453f * (m_fin + log2f(l));
        } else {
          mbar_arrive_cluster(map_to_leader(bar(O_FREE)));  // after a failed wait: let the issuer run into its own limit, not hang on this
        }
      }
      TRACE_ONLY(t_end += clock64() - c0; if (closer) t_close += clock64() - c0;)
      TL(closer ? 10 : 11, glast, r == 0);
      if (seq & 1) m_seen1 += (n_tiles - j_other + 1) >> 1; else m_seen0 += (n_tiles - j_other + 1) >> 1;
      g0 += n_tiles;
    }
    bulk_wait_read();  // shared memory must outlive the output stores that read it
    TRACE_VALUE(6, threadIdx.x == 128, clock64() - c_begin);
    TRACE_VALUE(7, threadIdx.x == 128, w_s);
    TRACE_VALUE(8, threadIdx.x == 128, t_ld);
    TRACE_VALUE(9, threadIdx.x == 128, t_max);
    TRACE_VALUE(10, threadIdx.x == 128, w_pv);
    TRACE_VALUE(11, threadIdx.x == 128, t_exp);
    TRACE_VALUE(13, threadIdx.x == 128, t_end);
    TRACE_VALUE(14, threadIdx.x == 128, w_s0);  // ... of which for the group's first tile of an item
    TRACE_VALUE(15, threadIdx.x == 128, t_close);  // ... of which as the group that writes the output
  }

  tc_fence_before();
  __syncthreads();
  pair_sync();  // the peer may still be signalling this CTA's barriers or waiting on a commit from the leader
  TRACE_ONLY(if (threadIdx.x == 0 && blockIdx.x == 0) for (int i = 0; i < 240; ++i) { const long long c = (&tl_sh[0][0])[i]; if (c) trace_put(16 + i / 20, (static_cast<unsigned long long>(196 + i % 20) << 40) | (static_cast<unsigned long long>(c) & ((1ull << 40) - 1)), __LINE__); })
  if (warp == 2) {
    if (*reinterpret_cast<volatile int*>(err) != 0) {
      const uint64_t t0 = global_timer_ns();
      while (global_timer_ns() - t0 < 2000000ull) __nanosleep(1000);
    }
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
  }
}

int make_map(CUtensorMap* m, const bf16* p, int S, int H, int B, long long ss, long long sh, long long sb, int box_rows) {
  const uint64_t dims[4] = {kHD, static_cast<uint64_t>(S), static_cast<uint64_t>(H), static_cast<uint64_t>(B)};
  const uint64_t strides[3] = {static_cast<uint64_t>(ss) * 2, static_cast<uint64_t>(sh) * 2,
                               static_cast<uint64_t>(sb) * 2};
  const uint32_t box[4] = {64, static_cast<uint32_t>(box_rows), 1, 1};
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
  CUtensorMap mk, mv, mq, mo;
  int rc;
  // a dimension of extent 1 still needs a legal (multiple-of-16-byte, non-zero) stride
  auto fix = [](long long st, long long fallback) { return st > 0 ? st : fallback; };
  if ((rc = make_map(&mk, k, s.Skv, s.Hkv, s.B, s.k_ss, fix(s.k_sh, s.k_ss), fix(s.k_sb, s.k_ss), 64))) return rc;
  if ((rc = make_map(&mv, v, s.Skv, s.Hkv, s.B, s.v_ss, fix(s.v_sh, s.v_ss), fix(s.v_sb, s.v_ss), 128))) return rc;
  if ((rc = make_map(&mq, q, s.Sq, s.Hq, s.B, s.q_ss, fix(s.q_sh, s.q_ss), fix(s.q_sb, s.q_ss), kQT))) return rc;
  if ((rc = make_map(&mo, o, s.Sq, s.Hq, s.B, s.o_ss, fix(s.o_sh, s.o_ss), fix(s.o_sb, s.o_ss), 32))) return rc;

  PrefillArgs a{};
  a.lse = lse; a.B = s.B; a.Hq = s.Hq; a.Hkv = s.Hkv; a.Sq = s.Sq; a.Skv = s.Skv;
  a.scale_log2 = s.scale * 1.4426950408889634f;
  a.causal = s.causal;
  a.err = device_error_word();
  if (!a.err) return TEENY_ERR_DRIVER;  // kernels report expired waits through this word: no launch without it

  {
    const int prc = attention_prefill_prepare();
    if (prc) return prc;
  }
  const int pair_tiles = (s.Sq + 2 * kQT - 1) / (2 * kQT);
  const long long items = static_cast<long long>(pair_tiles) * s.Hq * s.B;
  if (items > 0x7fffffffLL) return TEENY_ERR_BAD_ARG;
  a.n_pair_tiles = pair_tiles;
  a.n_items = static_cast<int>(items);
  // One CTA pair per SM pair, each walking its share of the items (TEENY_ATTN_PERSISTENT=0: one pair per item, for A/B
  // timing).
  static const bool persistent = [] { const char* e = getenv("TEENY_ATTN_PERSISTENT"); return !(e && e[0] == '0'); }();
  long long pairs = persistent ? sm_count() / 2 : items;
  if (pairs > items) pairs = items;
  if (pairs < 1) pairs = 1;
  if (pairs > 0x3fffffffLL) return TEENY_ERR_BAD_ARG;
  launch_kernel(attention_prefill_kernel, dim3(static_cast<unsigned>(2 * pairs)), dim3(kThreads), kSmemTotal, stream, 2, mk, mv, mq, mo, a);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace teeny
