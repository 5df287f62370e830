// Qwen3 decoder runner: the host-side executor that strings the kernels of this library into prefill and decode
// steps, with Megatron-style tensor parallelism (one process per GPU, one NCCL all-reduce after each row-parallel
// projection) and CUDA-graph replay of the decode step.
//
// It plays the role of the reference's model executor -- LoadedModel::forward walks the lowered graph and launches
// one kernel per node, capture_graph records the same launches once and CudaGraphModel::run replays them
// (drivers/teeny-cuda/src/model/mod.rs:524, 1245, 1799) -- for the one graph this backend serves: the Qwen3 layer
// sequence recorded in support/teeny-torch/tests/data/qwen3_{1,2,3}.bin.gz.  Like the reference executor it owns no
// weights: the caller passes device pointers (already sharded for this rank) and one workspace it allocated.
//
// Per layer (T tokens, local heads Hq/Hkv, local intermediate I):
//   y = rms_norm(h [+ previous delta])            fused residual add + norm
//   qkv = y Wqkv^T                                tcgen05 GEMM, fused [q | k | v] rows
//   q,k <- head norm + RoPE; k,v -> cache         one kernel
//   a = attention(q, cache)                       tcgen05 flash-attention (prefill) / split-KV decode kernel
//   delta = a Wo^T ; all-reduce                   row-parallel
//   y = rms_norm(h += delta)
//   act = silu(y Wg^T) * (y Wu^T)                 one GEMM, SwiGLU in its epilogue
//   delta = act Wd^T ; all-reduce
// then final norm on the last position of each sequence, vocabulary-parallel LM head, local argmax, all-gather of
// (value, index) candidates and a merge so every rank holds the same greedy token.
#include <dlfcn.h>
#include <nccl.h>

#include <chrono>
#include <cstdlib>
#include <cstring>
#include <new>
#include <thread>
#include <vector>

#include "../../include/teeny_b200.h"
#include "../../include/teeny_qwen3.h"
#include "common.cuh"
#include "kernels.h"
#include <cstdio>

namespace teeny {

namespace {

// ---- NCCL through dlopen: no link-time dependency, and the copy PyTorch already loaded is reused ----
struct NcclApi {
  void* handle = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*GroupStart)() = nullptr;
  ncclResult_t (*GroupEnd)() = nullptr;
  // optional (NCCL >= 2.14): what the guarded set-up needs
  ncclResult_t (*CommInitRankConfig)(ncclComm_t*, int, ncclUniqueId, int, ncclConfig_t*) = nullptr;
  ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t*) = nullptr;
  ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
  ncclResult_t (*Broadcast)(const void*, void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
  bool ok = false;
};
NcclApi g_nccl;

bool load_nccl() {
  if (g_nccl.ok) return true;
  // TEENY_NCCL_LIB names another library with the NCCL entry points (the host-side tests put a stand-in there)
  const char* name = getenv("TEENY_NCCL_LIB");
  if (!g_nccl.handle) g_nccl.handle = dlopen(name && name[0] ? name : "libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
  if (!g_nccl.handle) return false;
  auto sym = [&](const char* n) { return dlsym(g_nccl.handle, n); };
  g_nccl.GetUniqueId = reinterpret_cast<decltype(g_nccl.GetUniqueId)>(sym("ncclGetUniqueId"));
  g_nccl.CommInitRank = reinterpret_cast<decltype(g_nccl.CommInitRank)>(sym("ncclCommInitRank"));
  g_nccl.CommDestroy = reinterpret_cast<decltype(g_nccl.CommDestroy)>(sym("ncclCommDestroy"));
  g_nccl.AllReduce = reinterpret_cast<decltype(g_nccl.AllReduce)>(sym("ncclAllReduce"));
  g_nccl.AllGather = reinterpret_cast<decltype(g_nccl.AllGather)>(sym("ncclAllGather"));
  g_nccl.GroupStart = reinterpret_cast<decltype(g_nccl.GroupStart)>(sym("ncclGroupStart"));
  g_nccl.GroupEnd = reinterpret_cast<decltype(g_nccl.GroupEnd)>(sym("ncclGroupEnd"));
  g_nccl.CommInitRankConfig = reinterpret_cast<decltype(g_nccl.CommInitRankConfig)>(sym("ncclCommInitRankConfig"));
  g_nccl.CommGetAsyncError = reinterpret_cast<decltype(g_nccl.CommGetAsyncError)>(sym("ncclCommGetAsyncError"));
  g_nccl.CommAbort = reinterpret_cast<decltype(g_nccl.CommAbort)>(sym("ncclCommAbort"));
  g_nccl.Broadcast = reinterpret_cast<decltype(g_nccl.Broadcast)>(sym("ncclBroadcast"));
  g_nccl.ok = g_nccl.GetUniqueId && g_nccl.CommInitRank && g_nccl.CommDestroy && g_nccl.AllReduce &&
              g_nccl.AllGather && g_nccl.GroupStart && g_nccl.GroupEnd;
  return g_nccl.ok;
}

// Polls a non-blocking communicator until its pending operation has finished, failed, or `deadline` (steady clock)
// has passed.  Returns ncclSuccess, the error, or ncclInProgress for "still pending at the deadline".
ncclResult_t nccl_wait(ncclComm_t comm, ncclResult_t first, std::chrono::steady_clock::time_point deadline) {
  ncclResult_t state = first;
  while (state == ncclInProgress) {
    if (std::chrono::steady_clock::now() >= deadline) return ncclInProgress;
    std::this_thread::sleep_for(std::chrono::milliseconds(2));
    if (g_nccl.CommGetAsyncError(comm, &state) != ncclSuccess) return ncclInternalError;
  }
  return state;
}

// Communicator set-up that cannot hang on a rank that never arrives.  ncclCommInitRank blocks for ever in that case
// and a blocking communicator under construction cannot be aborted, so the rendezvous is first made with a
// NON-blocking "guard" communicator: init, poll with a host timeout, ncclCommAbort when the timeout expires.  Once the
// guard is up every rank is known to be alive; rank 0 then broadcasts a second unique id over it and all ranks create
// the blocking communicator the runner uses (its collectives are recorded into CUDA graphs, which a non-blocking
// communicator's helper-thread launches do not allow), and the guard is aborted.  Returns 0, or TEENY_ERR_NCCL with
// nothing left behind.
int guarded_comm_init(const ncclUniqueId& id, int rank, int world, long timeout_ms, ncclComm_t* out) {
  const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
  ncclConfig_t config = NCCL_CONFIG_INITIALIZER;
  config.blocking = 0;
  ncclComm_t guard = nullptr;
  ncclResult_t r = g_nccl.CommInitRankConfig(&guard, world, id, rank, &config);
  if (r != ncclSuccess && r != ncclInProgress) return TEENY_ERR_NCCL;
  r = nccl_wait(guard, r, deadline);
  if (r != ncclSuccess) {  // a rank did not arrive in time (or the bootstrap failed): give everything back
    if (guard) g_nccl.CommAbort(guard);
    return TEENY_ERR_NCCL;
  }
  // second id over the guard
  ncclUniqueId id2;
  std::memset(&id2, 0, sizeof(id2));
  int rc = 0;
  void* dbuf = nullptr;
  if (rank == 0 && g_nccl.GetUniqueId(&id2) != ncclSuccess) rc = TEENY_ERR_NCCL;
  if (cudaMalloc(&dbuf, sizeof(id2)) != cudaSuccess) { dbuf = nullptr; rc = TEENY_ERR_NCCL; }
  if (!rc && cudaMemcpy(dbuf, &id2, sizeof(id2), cudaMemcpyHostToDevice) != cudaSuccess) rc = TEENY_ERR_NCCL;
  if (!rc) {
    r = nccl_wait(guard, g_nccl.Broadcast(dbuf, dbuf, sizeof(id2), ncclChar, 0, guard, nullptr), deadline);
    if (r != ncclSuccess) rc = TEENY_ERR_NCCL;
  }
  if (!rc) {
    // the broadcast runs on the legacy default stream; bound the wait for it as well
    cudaError_t q;
    while ((q = cudaStreamQuery(nullptr)) == cudaErrorNotReady) {
      if (std::chrono::steady_clock::now() >= deadline) { rc = TEENY_ERR_NCCL; break; }
      std::this_thread::sleep_for(std::chrono::milliseconds(1));
    }
    if (!rc && q != cudaSuccess) rc = TEENY_ERR_NCCL;
  }
  if (!rc && cudaMemcpy(&id2, dbuf, sizeof(id2), cudaMemcpyDeviceToHost) != cudaSuccess) rc = TEENY_ERR_NCCL;
  if (!rc && g_nccl.CommInitRank(out, world, id2, rank) != ncclSuccess) rc = TEENY_ERR_NCCL;
  g_nccl.CommAbort(guard);
  if (dbuf) cudaFree(dbuf);
  if (rc) cudaGetLastError();
  return rc;
}

// Tensor-parallel context: the NCCL communicator plus, for decode, peer-mapped receive buffers through which the
// row-parallel GEMMs push their partial rows straight into every rank's memory (no collective call on that path).
struct TpContext {
  ncclComm_t comm = nullptr;
  int rank = 0, world = 1;
  bool peer_ok = false;
  size_t rows = 0, cols = 0, slot_elems = 0, data_bytes = 0;
  uint8_t* local = nullptr;    // [2 parities][world][rows][cols] {f32 value, u32 stamp} pairs, then the epoch word
  void* peer[8] = {};          // the same buffer of every rank (own entry = local)
  uint2** recv_tab = nullptr;  // device [2][world]: where this rank writes inside rank q's buffer
  // Two-hop mode (row owners reduce, then broadcast the finished rows): per parity a [rows][cols / 2] array of
  // 16-byte lines behind the epoch word in every rank's buffer; bcast_tab is device [2][world].
  bool two_hop = false;
  size_t bcast_off = 0;
  uint4** bcast_tab = nullptr;
  const uint2* local_recv(int parity) const {
    return reinterpret_cast<const uint2*>(local) + static_cast<size_t>(parity) * world * slot_elems;
  }
  // Counts the decode steps run over this context (by any runner): part of every stamp, so a buffer never sees the
  // same stamp twice.  Local to the rank; the ranks step it in lockstep.
  unsigned* epoch() const { return reinterpret_cast<unsigned*>(local + data_bytes); }
};

// Collective over the communicator: allocate the receive buffer, exchange IPC handles, map the peers.  Leaves
// peer_ok false (on every rank alike) if any rank could not set it up; the runner then all-reduces through NCCL.
// Every local failure (an allocation, a handle, a mapping, a table upload) is folded into the one `ok` byte that the
// ranks exchange, and no rank returns between the collectives, so the ranks cannot end up on different reduction paths
// or in a collective that others skipped.
int tp_enable_peer(TpContext* c, size_t rows, size_t cols, cudaStream_t st) {
  if (c->peer_ok || c->world < 2 || c->world > 8) return 0;
  c->rows = rows; c->cols = cols; c->slot_elems = rows * cols;
  c->data_bytes = 2 * static_cast<size_t>(c->world) * c->slot_elems * sizeof(uint2);
  c->bcast_off = c->data_bytes + 256;
  const size_t bcast_bytes = 2 * c->slot_elems * 8;  // 2 parities x rows x cols / 2 lines of 16 bytes
  const size_t total_bytes = c->bcast_off + bcast_bytes;
  {
    // One hop (every rank gets every partial) costs world x the tensor per rank.  Measured per decode step: 2 ranks
    // 3.25 ms in one hop against 3.53 ms in two; 4 ranks 2.94 ms against 2.89 ms; 8 ranks 3.51 ms against 3.25 ms.  So two
    // hops from 4 ranks on.  TEENY_TP_HOPS=1|2 overrides.
    const char* e = getenv("TEENY_TP_HOPS");
    c->two_hop = e ? (e[0] == '2') : (c->world >= 4);
  }
  cudaIpcMemHandle_t mine;
  std::memset(&mine, 0, sizeof(mine));
  const size_t rec = sizeof(mine) + 8;
  uint8_t* xbuf = nullptr;  // exchange buffer: [world] records of [handle | ok], reused for the later one-byte rounds
  int ok = 1;
  bool nccl_failed = false;
  if (cudaMalloc(&c->local, total_bytes) != cudaSuccess) { c->local = nullptr; ok = 0; }
  if (ok && cudaMemsetAsync(c->local, 0, total_bytes, st) != cudaSuccess) ok = 0;
  if (ok && cudaIpcGetMemHandle(&mine, c->local) != cudaSuccess) ok = 0;
  if (cudaMalloc(&xbuf, rec * c->world) != cudaSuccess) {
    // without the exchange buffer this rank cannot even say "no": the communicator is unusable for set-up
    if (c->local) { cudaFree(c->local); c->local = nullptr; }
    cudaGetLastError();
    return TEENY_ERR_NCCL;
  }
  std::vector<uint8_t> host(rec * c->world, 0);
  // all ranks: ok &= (every rank's ok); one byte per rank through the communicator
  auto agree = [&]() {
    host[0] = static_cast<uint8_t>(ok);
    cudaMemcpyAsync(xbuf + c->rank, host.data(), 1, cudaMemcpyHostToDevice, st);
    if (g_nccl.AllGather(xbuf + c->rank, xbuf, 1, ncclChar, c->comm, st) != ncclSuccess) nccl_failed = true;
    cudaMemcpyAsync(host.data(), xbuf, c->world, cudaMemcpyDeviceToHost, st);
    if (cudaStreamSynchronize(st) != cudaSuccess) nccl_failed = true;
    for (int q = 0; q < c->world; ++q) ok &= host[q];
    if (nccl_failed) ok = 0;
  };
  // first exchange: [handle | ok] records
  std::memcpy(host.data() + rec * c->rank, &mine, sizeof(mine));
  host[rec * c->rank + sizeof(mine)] = static_cast<uint8_t>(ok);
  cudaMemcpyAsync(xbuf + rec * c->rank, host.data() + rec * c->rank, rec, cudaMemcpyHostToDevice, st);
  if (g_nccl.AllGather(xbuf + rec * c->rank, xbuf, rec, ncclChar, c->comm, st) != ncclSuccess) nccl_failed = true;
  cudaMemcpyAsync(host.data(), xbuf, rec * c->world, cudaMemcpyDeviceToHost, st);
  if (cudaStreamSynchronize(st) != cudaSuccess) nccl_failed = true;
  if (nccl_failed) ok = 0;
  for (int q = 0; q < c->world; ++q) ok &= host[rec * q + sizeof(mine)];
  bool mapped[8] = {};
  if (ok) {
    for (int q = 0; q < c->world && ok; ++q) {
      if (q == c->rank) { c->peer[q] = c->local; continue; }
      cudaIpcMemHandle_t h;
      std::memcpy(&h, host.data() + rec * q, sizeof(h));
      if (cudaIpcOpenMemHandle(&c->peer[q], h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
        ok = 0;
        c->peer[q] = nullptr;
        cudaGetLastError();
      } else {
        mapped[q] = true;
      }
    }
  }
  // second exchange: did every rank map every peer?
  if (!nccl_failed) agree();
  if (ok) {
    std::vector<uint2*> rt(2 * c->world);
    std::vector<uint4*> bt(2 * c->world);
    for (int par = 0; par < 2; ++par)
      for (int q = 0; q < c->world; ++q) {
        rt[par * c->world + q] =
            reinterpret_cast<uint2*>(c->peer[q]) + (static_cast<size_t>(par) * c->world + c->rank) * c->slot_elems;
        bt[par * c->world + q] = reinterpret_cast<uint4*>(static_cast<uint8_t*>(c->peer[q]) + c->bcast_off) +
                                 static_cast<size_t>(par) * (c->slot_elems / 2);
      }
    if (cudaMalloc(&c->recv_tab, rt.size() * sizeof(uint2*)) != cudaSuccess) { c->recv_tab = nullptr; ok = 0; }
    if (ok && cudaMemcpy(c->recv_tab, rt.data(), rt.size() * sizeof(uint2*), cudaMemcpyHostToDevice) != cudaSuccess) ok = 0;
    if (ok && cudaMalloc(&c->bcast_tab, bt.size() * sizeof(uint4*)) != cudaSuccess) { c->bcast_tab = nullptr; ok = 0; }
    if (ok && cudaMemcpy(c->bcast_tab, bt.data(), bt.size() * sizeof(uint4*), cudaMemcpyHostToDevice) != cudaSuccess) ok = 0;
  }
  // third exchange: does every rank hold its tables?  Only then do all ranks switch to the peer path together.
  if (!nccl_failed) agree();
  cudaFree(xbuf);
  if (!ok) {
    for (int q = 0; q < c->world; ++q)
      if (mapped[q]) { cudaIpcCloseMemHandle(c->peer[q]); c->peer[q] = nullptr; }
    if (c->recv_tab) { cudaFree(c->recv_tab); c->recv_tab = nullptr; }
    if (c->bcast_tab) { cudaFree(c->bcast_tab); c->bcast_tab = nullptr; }
    if (c->local) { cudaFree(c->local); c->local = nullptr; }
    cudaGetLastError();
    return nccl_failed ? TEENY_ERR_NCCL : 0;  // 0: stay on the NCCL path
  }
  c->peer_ok = true;
  return 0;
}

__global__ void finish_step_kernel(const int* __restrict__ next_ids, int* __restrict__ cur_ids,
                                   int* __restrict__ history, int* __restrict__ state, int B, int max_steps,
                                   unsigned* __restrict__ tp_epoch) {
  pdl_wait();
  // state[0] = position of the next token to append, state[1] = live KV length during the step (= state[0] + 1),
  // state[2] = number of generated tokens so far
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  const int step = state[2];
  if (b < B) {
    const int id = next_ids[b];
    cur_ids[b] = id;
    if (step < max_steps) history[static_cast<size_t>(step) * B + b] = id;
  }
  __syncthreads();  // single block: every thread has read `step`
  if (b == 0) {
    state[0] += 1;
    state[1] += 1;
    state[2] = step + 1;
    if (tp_epoch) *tp_epoch += 1u;  // the pushes of the next step carry new stamps
  }
}

__global__ void set_state_kernel(int* state, int pos, int len, int steps) {
  pdl_wait();
  state[0] = pos;
  state[1] = len;
  state[2] = steps;
}

size_t align_up(size_t v, size_t a = 256) { return (v + a - 1) / a * a; }

}  // namespace

// A projection weight in the form it was given: bf16 [N, K], or FP8 (E4M3) bytes [N, K] with f32 scales
// (teeny_qwen3_set_weight_fp8; kinds as in teeny_linear_w8a16_forward).
struct Weight {
  const bf16* w = nullptr;
  const uint8_t* q = nullptr;
  const float* scale = nullptr;
  int kind = 0, group = 0;
  bool set() const { return w || q; }
};

struct LayerWeights {
  Weight qkv, o, gate_up, down;
  const bf16 *input_ln = nullptr, *post_ln = nullptr, *q_norm = nullptr, *k_norm = nullptr;
};

struct Workspace {
  // offsets into the caller's workspace
  size_t h, y, qkv, attn, delta, act, logits, kcache, vcache, cos, sin, gemm_scratch, attn_scratch, attn_counters, sample_u;
  size_t sample_cand, sample_gather;  // tensor-parallel sampling: this rank's candidate lists, all ranks' lists
  size_t y8, y8_scale;                // the norm kernels' output as two-term FP8 activations (0 bytes when max_batch > 128)
  size_t a8, a8_scale;                // ... and the MLP activation (the down projection's input), split by a kernel of its own
  size_t y8_rows;
  size_t cand_val, cand_idx, gather_val, gather_idx, next_ids, cur_ids, history, state, total;
  size_t gemm_scratch_bytes, attn_scratch_bytes, attn_counter_bytes, cache_layer_elems;
};

}  // namespace teeny

using namespace teeny;

struct teeny_qwen3 {
  teeny_qwen3_config cfg;
  int Hq, Hkv, I, Vl;  // local (per-rank) q heads, kv heads, intermediate, vocab rows
  std::vector<LayerWeights> layers;
  const bf16 *embed = nullptr, *final_norm = nullptr;
  Weight lm_head;
  void* fp8_scratch = nullptr;  // where a large prefill converts one FP8 projection at a time to bf16
  size_t fp8_scratch_bytes = 0;
  const float* inv_freq = nullptr;
  uint8_t* ws = nullptr;
  Workspace off;
  ncclComm_t comm = nullptr;
  TpContext* tp = nullptr;
  int push_round = 0;           // parity of the next peer push within a decode step
  bool pending_gather = false;  // a pushed projection waits to be summed by the next norm
  int pending_parity = 0;
  unsigned pending_round = 0;
  cudaGraphExec_t graph_exec = nullptr;
  cudaStream_t capture_stream = nullptr;
  // tensor-parallel prefill in two half-batches: the all-reduce of one half runs on comm_stream while the other
  // half computes (ev_ready: projection written; ev_done[half]: its all-reduce finished)
  cudaStream_t comm_stream = nullptr;
  cudaEvent_t ev_ready = nullptr, ev_done[2] = {nullptr, nullptr};
  bool overlap_prefill = false;
  // token selection: greedy unless a temperature > 0 was set
  float sample_temperature = 0.0f, sample_top_p = 1.0f;
  int sample_top_k = 1;
  unsigned long long sample_seed = 0;
  int graph_batch = 0;
  unsigned long long graph_kernels = 0;  // kernels recorded in graph_exec (launch accounting)
  int batch = 0;  // batch of the running generation (set by prefill)
  int next_pos = 0;  // host mirror of state[0]: cache position the next decode step appends at (prefill sets it to S)
  bool tables_ready = false;

  template <typename T> T* at(size_t o) const { return reinterpret_cast<T*>(ws + o); }
};

namespace {

bool valid_config(const teeny_qwen3_config& c) {
  if (c.num_layers <= 0 || c.hidden <= 0 || c.num_q_heads <= 0 || c.num_kv_heads <= 0 || c.intermediate <= 0 ||
      c.vocab <= 0 || c.max_batch <= 0 || c.max_len <= 0 || c.max_tokens <= 0 || c.tp_size <= 0 || c.tp_rank < 0 ||
      c.tp_rank >= c.tp_size || c.max_new_tokens < 0)
    return false;
  if (c.head_dim != 128) return false;
  if (c.num_q_heads % c.num_kv_heads || c.num_kv_heads % c.tp_size || c.intermediate % c.tp_size ||
      c.vocab % c.tp_size)
    return false;
  if (c.hidden % 8 || (c.intermediate / c.tp_size) % 64 || (c.vocab / c.tp_size) % 8) return false;
  if (c.max_tokens < c.max_batch) return false;
  return true;
}

Workspace plan(const teeny_qwen3_config& c) {
  Workspace w{};
  const int tp = c.tp_size;
  const size_t Hq = c.num_q_heads / tp, Hkv = c.num_kv_heads / tp, I = c.intermediate / tp, Vl = c.vocab / tp;
  const size_t T = c.max_tokens, D = c.head_dim, H = c.hidden, Bm = c.max_batch;
  size_t o = 0;
  auto take = [&](size_t bytes) { const size_t at = o; o += align_up(bytes); return at; };
  w.h = take(T * H * 2);
  w.y = take(T * H * 2);
  w.qkv = take(T * (Hq + 2 * Hkv) * D * 2);
  w.attn = take(T * Hq * D * 2);
  w.delta = take(T * H * 2);
  w.act = take(T * I * 2);
  w.logits = take(Bm * Vl * 2);
  w.cache_layer_elems = Bm * Hkv * static_cast<size_t>(c.max_len) * D;
  w.kcache = take(w.cache_layer_elems * 2 * c.num_layers);
  w.vcache = take(w.cache_layer_elems * 2 * c.num_layers);
  w.cos = take(static_cast<size_t>(c.max_len) * D * 2);
  w.sin = take(static_cast<size_t>(c.max_len) * D * 2);
  // split-K scratch: the largest need over the decode-shaped GEMMs of a layer and the LM head
  size_t gs = 0;
  const int Bi = c.max_batch;
  const int shapes[5][2] = {{static_cast<int>((Hq + 2 * Hkv) * D), c.hidden},
                            {c.hidden, static_cast<int>(Hq * D)},
                            {static_cast<int>(2 * I), c.hidden},
                            {c.hidden, static_cast<int>(I)},
                            {static_cast<int>(Vl), c.hidden}};
  for (auto& s : shapes) {
    const size_t n = gemm_bf16_scratch_bytes(Bi, s[0], s[1]);
    gs = n > gs ? n : gs;
  }
  w.gemm_scratch_bytes = gs;
  w.gemm_scratch = take(gs);
  w.attn_scratch_bytes = attention_decode_scratch_bytes(c.max_batch, static_cast<int>(Hq), c.head_dim, c.max_len);
  w.attn_scratch = take(w.attn_scratch_bytes);
  w.attn_counter_bytes = Bm * static_cast<size_t>(c.num_kv_heads) * 4;  // arrival counters of the split-sequence merge
  w.attn_counters = take(w.attn_counter_bytes);
  // FP8 weights: a decode step's norm outputs (and the head's) also as two-term FP8, hi rows then lo rows
  w.y8_rows = (tp == 1 && Bm <= 128 && H % 16 == 0) ? Bm : 0;
  w.y8 = take(2 * w.y8_rows * H);
  w.y8_scale = take(w.y8_rows * 4);
  w.a8 = take(I % 16 == 0 ? 2 * w.y8_rows * I : 0);
  w.a8_scale = take(w.y8_rows * 4);
  w.sample_u = take(Bm * 4);
  w.sample_cand = take(tp > 1 ? Bm * 1024 * 8 : 0);
  w.sample_gather = take(tp > 1 ? Bm * 1024 * 8 * tp : 0);
  w.cand_val = take(Bm * 4);
  w.cand_idx = take(Bm * 4);
  w.gather_val = take(Bm * 4 * tp);
  w.gather_idx = take(Bm * 4 * tp);
  w.next_ids = take(Bm * 4);
  w.cur_ids = take(Bm * 4);
  w.history = take(Bm * 4 * static_cast<size_t>(c.max_new_tokens > 0 ? c.max_new_tokens : 1));
  w.state = take(16);
  w.total = o;
  return w;
}

#define TEENY_TRY(expr)                  \
  do {                                   \
    const int rc_ = (expr);              \
    if (rc_ != 0) return rc_;            \
  } while (0)

int all_reduce(teeny_qwen3* m, bf16* buf, size_t count, cudaStream_t st) {
  if (m->cfg.tp_size == 1) return 0;
  if (!m->comm) return TEENY_ERR_NCCL;
  return g_nccl.AllReduce(buf, buf, count, ncclBfloat16, ncclSum, m->comm, st) == ncclSuccess ? 0 : TEENY_ERR_NCCL;
}

// y[T, N] = x[T, K] W^T for one of the model's projection weights, in whichever form it was given.  FP8 weights are
// streamed as bytes while T <= 128 (decode) and converted into the model's FP8 scratch for a larger T (prefill), where
// the bf16 kernels -- the QKV projection's fused epilogue included -- then run on the converted copy.
// x8 true: x has also been written as two-term FP8 activations into the model's y8 buffer (by the norm kernel in front;
// mlp_act: into the a8 buffer, by split_e4m3 behind the gate/up projection) and the weight's scales allow it: the
// conversion-free FP8 x FP8 kernel runs.
int project(teeny_qwen3* m, const bf16* x, int ldx, const Weight& w, bf16* y, int ldy, int T, int N, int K,
            cudaStream_t st, bool swiglu = false, const GemmPush* push = nullptr, const QkvEpilogue* fuse = nullptr,
            bool x8 = false, bool mlp_act = false) {
  void* gs = m->at<void>(m->off.gemm_scratch);
  const bf16* wb = w.w;
  const int w_rows = N;  // rows of W ([N, K]; for swiglu N counts gate and up rows)
  if (w.q && x8 && T <= 128 && w.kind <= 1)
    return gemm_w8a8x2_skinny(m->at<uint8_t>(mlp_act ? m->off.a8 : m->off.y8), K,
                              m->at<float>(mlp_act ? m->off.a8_scale : m->off.y8_scale), w.q, K, w.scale, w.kind, nullptr, y,
                              ldy, T, N, K, st, swiglu, push);
  if (w.q) {
    if (T <= 128) return linear_w8a16(x, ldx, w.q, K, w.scale, w.kind, w.group, nullptr, y, ldy, T, N, K, nullptr, 0, st, swiglu, push);
    const size_t need = static_cast<size_t>(w_rows) * K * sizeof(bf16);
    if (!m->fp8_scratch || m->fp8_scratch_bytes < need || (K & 7)) return TEENY_ERR_SCRATCH;
    TEENY_TRY(dequant_e4m3_bf16(w.q, K, w.scale, w.kind, w.group, static_cast<bf16*>(m->fp8_scratch), K, w_rows, K, st));
    wb = static_cast<const bf16*>(m->fp8_scratch);
  }
  if (fuse) return gemm_bf16_2cta(x, ldx, wb, K, nullptr, y, ldy, T, N, K, st, false, fuse);
  return gemm_bf16(x, ldx, wb, K, false, nullptr, y, ldy, T, N, K, gs, m->off.gemm_scratch_bytes, st, swiglu, push);
}

// Row-parallel projection delta = x W^T followed by the cross-rank sum.  Decode with peer buffers: the GEMM pushes
// its f32 rows into every rank's receive buffer and the sum happens inside the next norm kernel (pending_gather);
// otherwise GEMM to `delta` and, with tp > 1, an NCCL all-reduce.
int row_parallel(teeny_qwen3* m, const bf16* x, int ldx, const Weight& w, bf16* delta, int T, int N, int K, bool decode,
                 cudaStream_t st, bool act8 = false) {
  TpContext* tp = m->tp;
  if (decode && tp && tp->peer_ok && T <= static_cast<int>(tp->rows) && N == static_cast<int>(tp->cols)) {
    const int parity = m->push_round & 1;
    const int owner_rows = tp->two_hop ? (T + tp->world - 1) / tp->world : 0;
    GemmPush push{tp->recv_tab + parity * tp->world, tp->world, tp->epoch(), static_cast<unsigned>(m->push_round),
                  owner_rows};
    TEENY_TRY(project(m, x, ldx, w, delta, N, T, N, K, st, false, &push));
    m->pending_gather = true;
    m->pending_parity = parity;
    m->pending_round = static_cast<unsigned>(m->push_round);
    ++m->push_round;
    return 0;
  }
  TEENY_TRY(project(m, x, ldx, w, delta, N, T, N, K, st, false, nullptr, nullptr, act8, act8));
  return all_reduce(m, delta, static_cast<size_t>(T) * N, st);
}

// Whether the projection behind a norm takes its input as two-term FP8: an FP8 weight with per-tensor or per-channel
// scales, at most 128 rows, one GPU (the gather kernels of the tensor-parallel path write no FP8 copy).
bool wants_x8(const teeny_qwen3* m, const Weight& w, int M) {
  return w.q && w.kind <= 1 && !m->tp && M > 0 && static_cast<size_t>(M) <= m->off.y8_rows;
}

// residual += projection; y = rms_norm(residual) on M rows (row strides ld for delta / residual, H for y).
// split: also write y as two-term FP8 into the model's y8 buffer.
int residual_norm(teeny_qwen3* m, bf16* delta, bf16* h, long long ld, bf16* y, const bf16* w, int M, cudaStream_t st,
                  bool split = false) {
  const teeny_qwen3_config& c = m->cfg;
  if (m->pending_gather) {
    m->pending_gather = false;
    TpContext* tp = m->tp;
    if (tp->two_hop)
      return gather_add_rms_norm_owner_bf16(tp->local_recv(m->pending_parity), tp->slot_elems, tp->world, tp->rank,
                                            (M + tp->world - 1) / tp->world, tp->bcast_tab + m->pending_parity * tp->world,
                                            tp->epoch(), m->pending_round, h, ld, y, c.hidden, w, M, c.hidden, c.eps, st);
    return gather_add_rms_norm_bf16(tp->local_recv(m->pending_parity), tp->slot_elems, tp->world, tp->epoch(),
                                    m->pending_round, h, ld, y, c.hidden, w, M, c.hidden, c.eps, st);
  }
  return add_rms_norm_bf16(delta, ld, h, ld, y, c.hidden, w, M, c.hidden, c.eps, st,
                           split ? m->at<uint8_t>(m->off.y8) : nullptr, c.hidden, split ? m->at<float>(m->off.y8_scale) : nullptr);
}

// TEENY_FP8_DOWN_SPLIT=0 leaves the FP8 down projection on the converting kernel (for A/B timing).
bool down8_enabled() {
  static const bool on = [] { const char* e = getenv("TEENY_FP8_DOWN_SPLIT"); return !(e && e[0] == '0'); }();
  return on;
}

// TEENY_QKV_FUSE=0 keeps head norms / RoPE / cache fill in their own kernel behind the QKV projection (for A/B timing).
bool qkv_fuse_enabled() {
  static const bool on = [] { const char* e = getenv("TEENY_QKV_FUSE"); return !(e && e[0] == '0'); }();
  return on;
}

// The shared layer loop.  T tokens arranged [B, S]; pos0 is the position of the first token of every sequence
// (device value when pos_dev != null).  decode selects the split-KV attention kernel (S == 1).
int run_layers(teeny_qwen3* m, int B, int S, int pos0, const int* pos_dev, const int* len_dev, bool decode,
               cudaStream_t st) {
  const teeny_qwen3_config& c = m->cfg;
  const int T = B * S, H = c.hidden, D = c.head_dim, Hq = m->Hq, Hkv = m->Hkv, I = m->I;
  const int qkv_n = (Hq + 2 * Hkv) * D;
  bf16 *h = m->at<bf16>(m->off.h), *y = m->at<bf16>(m->off.y), *qkv = m->at<bf16>(m->off.qkv);
  bf16 *attn = m->at<bf16>(m->off.attn), *delta = m->at<bf16>(m->off.delta);
  bf16* act = m->at<bf16>(m->off.act);
  const float scale = 1.0f / sqrtf(static_cast<float>(D));
  // (Asking the QKV and gate/up weights into L2 while the norm in front of them waits for the other ranks' partial sums
  // was measured under tensor parallelism: 3.29 ms per decode step against 3.25 ms without, 2 ranks.  Not used.)
  for (int l = 0; l < c.num_layers; ++l) {
    const LayerWeights& w = m->layers[l];
    bf16* kc = m->at<bf16>(m->off.kcache) + static_cast<size_t>(l) * m->off.cache_layer_elems;
    bf16* vc = m->at<bf16>(m->off.vcache) + static_cast<size_t>(l) * m->off.cache_layer_elems;
    const bool qkv8 = wants_x8(m, w.qkv, T), mlp8 = wants_x8(m, w.gate_up, T);
    if (l == 0)
      TEENY_TRY(rms_norm_bf16(h, H, y, H, w.input_ln, nullptr, T, H, c.eps, st, qkv8 ? m->at<uint8_t>(m->off.y8) : nullptr, H,
                              qkv8 ? m->at<float>(m->off.y8_scale) : nullptr));
    else TEENY_TRY(residual_norm(m, delta, h, H, y, w.input_ln, T, st, qkv8));
    // Head norms, RoPE and the cache fill: in a large prefill they run in the epilogue of the QKV projection itself (k
    // and v never pass through the projection buffer); in a small one as one pass over the projection; in decode the
    // attention kernel does them for its own (sequence, kv head) on the way in.
    if (!decode && !pos_dev && qkv_fuse_enabled() && gemm_bf16_uses_2cta(T, qkv_n)) {
      const QkvEpilogue fuse{w.q_norm, w.k_norm, m->at<bf16>(m->off.cos), m->at<bf16>(m->off.sin), kc, vc,
                             S, Hq, Hkv, c.max_len, pos0, c.eps};
      TEENY_TRY(project(m, y, H, w.qkv, qkv, qkv_n, T, qkv_n, H, st, false, nullptr, &fuse));
    } else {
      TEENY_TRY(project(m, y, H, w.qkv, qkv, qkv_n, T, qkv_n, H, st, false, nullptr, nullptr, qkv8));
      if (!decode)
        TEENY_TRY(qk_norm_rope_kv_bf16(qkv, qkv_n, w.q_norm, w.k_norm, m->at<bf16>(m->off.cos), m->at<bf16>(m->off.sin),
                                       kc, vc, T, S, Hq, Hkv, D, c.max_len, pos0, pos_dev, c.eps, st));
    }
    AttnShape a{};
    a.B = B; a.Hq = Hq; a.Hkv = Hkv; a.D = D; a.scale = scale;
    a.q_sb = static_cast<long long>(S) * qkv_n; a.q_sh = D; a.q_ss = qkv_n;
    a.k_sb = static_cast<long long>(Hkv) * c.max_len * D; a.k_sh = static_cast<long long>(c.max_len) * D; a.k_ss = D;
    a.v_sb = a.k_sb; a.v_sh = a.k_sh; a.v_ss = D;
    a.o_sb = static_cast<long long>(S) * Hq * D; a.o_sh = D; a.o_ss = static_cast<long long>(Hq) * D;
    if (decode) {
      a.Sq = 1; a.Skv = c.max_len; a.causal = 0;
      DecodeRope rope{};
      rope.k_new = qkv + static_cast<size_t>(Hq) * D;
      rope.v_new = qkv + static_cast<size_t>(Hq + Hkv) * D;
      rope.new_sb = qkv_n;
      rope.k_cache = kc; rope.v_cache = vc;
      rope.q_w = w.q_norm; rope.k_w = w.k_norm;
      rope.cos_t = m->at<bf16>(m->off.cos); rope.sin_t = m->at<bf16>(m->off.sin);
      rope.pos_dev = pos_dev; rope.pos = pos0; rope.max_len = c.max_len; rope.eps = c.eps;
      // The kernel before this one (the QKV projection) writes only the projection buffer, the one new cache row per
      // sequence is appended by the attention kernel itself, and the length was set a whole step earlier.
      TEENY_TRY(attention_decode_bf16(qkv, kc, vc, attn, a, pos0 + 1, len_dev, m->at<void>(m->off.attn_scratch),
                                      m->off.attn_scratch_bytes, st, 1, &rope, m->at<unsigned>(m->off.attn_counters)));
    } else {
      a.Sq = S; a.Skv = pos0 + S; a.causal = 1;
      TEENY_TRY(attention_prefill_bf16(qkv, kc, vc, attn, nullptr, a, st));
    }
    TEENY_TRY(row_parallel(m, attn, Hq * D, w.o, delta, T, H, Hq * D, decode, st));
    TEENY_TRY(residual_norm(m, delta, h, H, y, w.post_ln, T, st, mlp8));
    TEENY_TRY(project(m, y, H, w.gate_up, act, I, T, 2 * I, H, st, /*swiglu=*/true, nullptr, nullptr, mlp8));
    // (one GPU, FP8 down projection: its input as two-term FP8 costs a small kernel and saves the conversion of 50 M
    // weight bytes next to the tensor core)
    const bool down8 = down8_enabled() && wants_x8(m, w.down, T) && m->off.a8 != m->off.a8_scale;
    if (down8) TEENY_TRY(split_e4m3(act, I, m->at<uint8_t>(m->off.a8), I, m->at<float>(m->off.a8_scale), T, I, st));
    TEENY_TRY(row_parallel(m, act, I, w.down, delta, T, H, I, decode, st, down8));
  }
  return 0;
}

// Tensor-parallel prefill with communication hidden behind compute.  The batch is cut into two halves of whole
// sequences; on the one compute stream the halves alternate block by block (attention block of A, of B, MLP block of
// A, of B, ...), and each row-parallel projection's all-reduce is issued on the communicator's own stream, so it runs
// while the other half's next block computes.  The persistent GEMMs leave comm_sms() SMs to the collective's CTAs for
// the duration (otherwise the collective cannot start until a GEMM ends, or holds back part of the next GEMM's grid).
int comm_sms() {  // TEENY_TP_COMM_SMS overrides (0 = the GEMMs keep every SM)
  static const int n = [] {
    const char* e = getenv("TEENY_TP_COMM_SMS");
    const int v = e ? atoi(e) : 0;
    return v < 0 ? 0 : (v > 64 ? 64 : v);
  }();
  return n;
}

int run_layers_prefill_overlap(teeny_qwen3* m, int B, int S, cudaStream_t st) {
  const teeny_qwen3_config& c = m->cfg;
  const int Bh = B / 2, Th = Bh * S, H = c.hidden, D = c.head_dim, Hq = m->Hq, Hkv = m->Hkv, I = m->I;
  const int qkv_n = (Hq + 2 * Hkv) * D;
  const float scale = 1.0f / sqrtf(static_cast<float>(D));
  cudaStream_t sc = m->comm_stream;
  struct SmLimit {
    explicit SmLimit(int n) { set_sm_limit(n); }
    ~SmLimit() { set_sm_limit(0); }
  } limit(sm_count() - comm_sms());

  auto half_ptrs = [&](int hf, bf16*& h, bf16*& y, bf16*& qkv, bf16*& attn, bf16*& delta, bf16*& act) {
    const size_t r = static_cast<size_t>(hf) * Th;
    h = m->at<bf16>(m->off.h) + r * H;
    y = m->at<bf16>(m->off.y) + r * H;
    qkv = m->at<bf16>(m->off.qkv) + r * qkv_n;
    attn = m->at<bf16>(m->off.attn) + r * Hq * D;
    delta = m->at<bf16>(m->off.delta) + r * H;
    act = m->at<bf16>(m->off.act) + r * I;
  };
  // all-reduce `delta` of one half on the communicator's stream, behind everything issued on st so far
  auto reduce_async = [&](bf16* delta, int hf) -> int {
    if (cudaEventRecord(m->ev_ready, st) != cudaSuccess) return TEENY_ERR_NCCL;
    if (cudaStreamWaitEvent(sc, m->ev_ready, 0) != cudaSuccess) return TEENY_ERR_NCCL;
    TEENY_TRY(all_reduce(m, delta, static_cast<size_t>(Th) * H, sc));
    return cudaEventRecord(m->ev_done[hf], sc) == cudaSuccess ? 0 : TEENY_ERR_NCCL;
  };
  auto wait_reduced = [&](int hf) -> int {
    return cudaStreamWaitEvent(st, m->ev_done[hf], 0) == cudaSuccess ? 0 : TEENY_ERR_NCCL;
  };

  for (int l = 0; l < c.num_layers; ++l) {
    const LayerWeights& w = m->layers[l];
    bf16* kc = m->at<bf16>(m->off.kcache) + static_cast<size_t>(l) * m->off.cache_layer_elems;
    bf16* vc = m->at<bf16>(m->off.vcache) + static_cast<size_t>(l) * m->off.cache_layer_elems;
    const size_t cache_half = static_cast<size_t>(Bh) * Hkv * c.max_len * D;
    for (int hf = 0; hf < 2; ++hf) {  // attention blocks
      bf16 *h, *y, *qkv, *attn, *delta, *act;
      half_ptrs(hf, h, y, qkv, attn, delta, act);
      if (l == 0) {
        TEENY_TRY(rms_norm_bf16(h, H, y, H, w.input_ln, nullptr, Th, H, c.eps, st));
      } else {
        TEENY_TRY(wait_reduced(hf));  // down projection of the layer before
        TEENY_TRY(add_rms_norm_bf16(delta, H, h, H, y, H, w.input_ln, Th, H, c.eps, st));
      }
      if (qkv_fuse_enabled() && gemm_bf16_uses_2cta(Th, qkv_n)) {  // head norms, RoPE and the cache fill in the projection's epilogue
        const QkvEpilogue fuse{w.q_norm, w.k_norm, m->at<bf16>(m->off.cos), m->at<bf16>(m->off.sin),
                               kc + hf * cache_half, vc + hf * cache_half, S, Hq, Hkv, c.max_len, 0, c.eps};
        TEENY_TRY(project(m, y, H, w.qkv, qkv, qkv_n, Th, qkv_n, H, st, false, nullptr, &fuse));
      } else {
        TEENY_TRY(project(m, y, H, w.qkv, qkv, qkv_n, Th, qkv_n, H, st));
        TEENY_TRY(qk_norm_rope_kv_bf16(qkv, qkv_n, w.q_norm, w.k_norm, m->at<bf16>(m->off.cos), m->at<bf16>(m->off.sin),
                                       kc + hf * cache_half, vc + hf * cache_half, Th, S, Hq, Hkv, D, c.max_len, 0, nullptr,
                                       c.eps, st));
      }
      AttnShape a{};
      a.B = Bh; a.Hq = Hq; a.Hkv = Hkv; a.D = D; a.scale = scale;
      a.q_sb = static_cast<long long>(S) * qkv_n; a.q_sh = D; a.q_ss = qkv_n;
      a.k_sb = static_cast<long long>(Hkv) * c.max_len * D; a.k_sh = static_cast<long long>(c.max_len) * D; a.k_ss = D;
      a.v_sb = a.k_sb; a.v_sh = a.k_sh; a.v_ss = D;
      a.o_sb = static_cast<long long>(S) * Hq * D; a.o_sh = D; a.o_ss = static_cast<long long>(Hq) * D;
      a.Sq = S; a.Skv = S; a.causal = 1;
      TEENY_TRY(attention_prefill_bf16(qkv, kc + hf * cache_half, vc + hf * cache_half, attn, nullptr, a, st));
      TEENY_TRY(project(m, attn, Hq * D, w.o, delta, H, Th, H, Hq * D, st));
      TEENY_TRY(reduce_async(delta, hf));
    }
    for (int hf = 0; hf < 2; ++hf) {  // MLP blocks
      bf16 *h, *y, *qkv, *attn, *delta, *act;
      half_ptrs(hf, h, y, qkv, attn, delta, act);
      TEENY_TRY(wait_reduced(hf));  // O projection
      TEENY_TRY(add_rms_norm_bf16(delta, H, h, H, y, H, w.post_ln, Th, H, c.eps, st));
      TEENY_TRY(project(m, y, H, w.gate_up, act, I, Th, 2 * I, H, st, /*swiglu=*/true));
      TEENY_TRY(project(m, act, I, w.down, delta, H, Th, H, I, st));
      TEENY_TRY(reduce_async(delta, hf));
    }
  }
  // the head reads both halves' last down projection
  TEENY_TRY(wait_reduced(0));
  TEENY_TRY(wait_reduced(1));
  return 0;
}

// Final norm on the last token of each sequence, LM head, greedy pick.  Leaves next ids in off.next_ids.
int run_head(teeny_qwen3* m, int B, int S, cudaStream_t st, const int* step_dev = nullptr) {
  const teeny_qwen3_config& c = m->cfg;
  const int H = c.hidden, Vl = m->Vl;
  bf16 *h = m->at<bf16>(m->off.h), *y = m->at<bf16>(m->off.y), *delta = m->at<bf16>(m->off.delta);
  bf16* logits = m->at<bf16>(m->off.logits);
  const size_t last = static_cast<size_t>(S - 1) * H;
  const long long ld = static_cast<long long>(S) * H;
  // residual add + final norm on rows (b, S-1); y rows are packed [B, H]
  const bool head8 = wants_x8(m, m->lm_head, B);
  TEENY_TRY(residual_norm(m, delta + last, h + last, ld, y, m->final_norm, B, st, head8));
  TEENY_TRY(project(m, y, H, m->lm_head, logits, Vl, B, Vl, H, st, false, nullptr, nullptr, head8));
  float* cv = m->at<float>(m->off.cand_val);
  int* ci = m->at<int>(m->off.cand_idx);
  int* next = m->at<int>(m->off.next_ids);
  if (c.tp_size == 1) {
    if (m->sample_temperature > 0.0f) {
      // token t of a generation draws u from (seed, t, row): t = 0 at prefill, the running count in decode
      float* u = m->at<float>(m->off.sample_u);
      TEENY_TRY(sampling_uniform(m->sample_seed, 0, S > 1 || !step_dev ? nullptr : step_dev, u, B, st));
      TEENY_TRY(sample_top_k_top_p_bf16(logits, Vl, B, Vl, m->sample_temperature, m->sample_top_k, m->sample_top_p, u, next,
                                        nullptr, st));
      return 0;
    }
    TEENY_TRY(argmax_bf16(logits, Vl, cv, next, B, Vl, 0, st));
    return 0;
  }
  if (!m->comm) return TEENY_ERR_NCCL;
  if (m->sample_temperature > 0.0f) {
    // every rank: the top-k candidates of its vocabulary shard, all-gathered; then the same merge + pick on every rank
    // (same u, same lists -> same token)
    float* u = m->at<float>(m->off.sample_u);
    unsigned long long* mine = m->at<unsigned long long>(m->off.sample_cand);
    unsigned long long* all = m->at<unsigned long long>(m->off.sample_gather);
    const size_t words = static_cast<size_t>(B) * m->sample_top_k;
    TEENY_TRY(sampling_uniform(m->sample_seed, 0, S > 1 || !step_dev ? nullptr : step_dev, u, B, st));
    TEENY_TRY(sample_candidates_bf16(logits, Vl, B, Vl, m->sample_top_k, c.tp_rank * Vl, mine, st));
    if (g_nccl.AllGather(mine, all, words, ncclUint64, m->comm, st) != ncclSuccess) return TEENY_ERR_NCCL;
    TEENY_TRY(sample_merge(all, c.tp_size, words, B, m->sample_temperature, m->sample_top_k, m->sample_top_p, u, next,
                           nullptr, st));
    return 0;
  }
  TEENY_TRY(argmax_bf16(logits, Vl, cv, ci, B, Vl, c.tp_rank * Vl, st));
  float* gv = m->at<float>(m->off.gather_val);
  int* gi = m->at<int>(m->off.gather_idx);
  // gathered layout [rank][max_batch]; only the first B of each rank's slot are meaningful
  g_nccl.GroupStart();
  ncclResult_t r1 = g_nccl.AllGather(cv, gv, c.max_batch, ncclFloat32, m->comm, st);
  ncclResult_t r2 = g_nccl.AllGather(ci, gi, c.max_batch, ncclInt32, m->comm, st);
  ncclResult_t r3 = g_nccl.GroupEnd();
  if (r1 != ncclSuccess || r2 != ncclSuccess || r3 != ncclSuccess) return TEENY_ERR_NCCL;
  // candidates of part p for row r sit at [p * max_batch + r]: combine with `rows` = max_batch stride
  TEENY_TRY(argmax_combine(gv, gi, next, c.tp_size, c.max_batch, st));
  return 0;
}

// While alive, this thread's launches carry the programmatic-dependent-launch attribute, so each kernel's set-up
// (and the decode GEMMs' first weight tiles) overlaps the tail of the kernel before it.
struct PdlScope {
  PdlScope() { pdl_set_enabled(true); }
  ~PdlScope() { pdl_set_enabled(false); }
};

int decode_body(teeny_qwen3* m, int B, cudaStream_t st) {
  PdlScope pdl;
  m->push_round = 0;  // every step issues an even number of pushes, so the parity sequence repeats
  m->pending_gather = false;
  const teeny_qwen3_config& c = m->cfg;
  int* state = m->at<int>(m->off.state);
  TEENY_TRY(embedding_bf16(m->at<int>(m->off.cur_ids), m->embed, m->at<bf16>(m->off.h), B, c.hidden, c.vocab, st));
  TEENY_TRY(run_layers(m, B, 1, 0, state + 0, state + 1, true, st));
  TEENY_TRY(run_head(m, B, 1, st, state + 2));
  unsigned* tp_epoch = (m->tp && m->tp->peer_ok) ? m->tp->epoch() : nullptr;
  launch_kernel(finish_step_kernel, dim3(1), dim3(1024), 0, st, 1, m->at<int>(m->off.next_ids), m->at<int>(m->off.cur_ids),
                                         m->at<int>(m->off.history), state, B, c.max_new_tokens, tp_epoch);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace

extern "C" {

size_t teeny_qwen3_workspace_bytes(const teeny_qwen3_config* cfg) {
  if (!cfg || !valid_config(*cfg)) return 0;
  return plan(*cfg).total;
}

int teeny_qwen3_create(const teeny_qwen3_config* cfg, void* workspace, size_t workspace_bytes, void* tp_comm,
                       teeny_stream_t stream, teeny_qwen3** out) {
  if (!cfg || !out || !workspace || !valid_config(*cfg)) return TEENY_ERR_BAD_ARG;
  if (cfg->max_batch > 1024) return TEENY_ERR_BAD_ARG;
  if (cfg->tp_size > 1 && !tp_comm) return TEENY_ERR_NCCL;
  if (reinterpret_cast<uintptr_t>(workspace) & 255) return TEENY_ERR_ALIGNMENT;
  const Workspace w = plan(*cfg);
  if (workspace_bytes < w.total) return TEENY_ERR_SCRATCH;
  teeny_qwen3* m = new (std::nothrow) teeny_qwen3();
  if (!m) return TEENY_ERR_BAD_ARG;
  m->cfg = *cfg;
  m->Hq = cfg->num_q_heads / cfg->tp_size;
  m->Hkv = cfg->num_kv_heads / cfg->tp_size;
  m->I = cfg->intermediate / cfg->tp_size;
  m->Vl = cfg->vocab / cfg->tp_size;
  m->layers.resize(cfg->num_layers);
  m->ws = static_cast<uint8_t*>(workspace);
  m->off = w;
  m->tp = static_cast<TpContext*>(tp_comm);
  m->comm = m->tp ? m->tp->comm : nullptr;
  if (m->tp && (m->tp->world != cfg->tp_size || m->tp->rank != cfg->tp_rank)) {
    delete m;
    return TEENY_ERR_BAD_ARG;
  }
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  // function attributes (dynamic shared memory) are set once per device here, outside any stream capture
  int prc = gemm_bf16_prepare();
  if (prc == 0) prc = gemm_bf16_2cta_prepare();
  if (prc == 0) prc = attention_prefill_prepare();
  if (prc == 0) prc = attention_decode_prepare();
  if (prc == 0 && cfg->tp_size > 1) prc = sample_merge_prepare();
  if (prc != 0) {
    delete m;
    return prc;
  }
  // Prefill with the all-reduces on their own stream.  Measured (prefill of 32 x 2048 tokens): 8 GPUs 186 ms against
  // 210 ms in line, so it is the default from 8 ranks on; 2 GPUs 473 ms against 465 ms (only ~40 ms of communication
  // are exposed there and the collective's CTAs slow the GEMMs they share SMs with), so it stays off below 8 (4 GPUs
  // not measured).  Reserving SMs for the collective never paid (TEENY_TP_COMM_SMS, default 0).
  // TEENY_TP_OVERLAP=0|1 overrides.
  const char* ov_env = getenv("TEENY_TP_OVERLAP");
  const bool want_overlap = ov_env ? (ov_env[0] == '1') : (cfg->tp_size >= 8);
  if (m->tp && cfg->tp_size > 1 && want_overlap) {
    bool ok = cudaStreamCreateWithFlags(&m->comm_stream, cudaStreamNonBlocking) == cudaSuccess;
    ok = ok && cudaEventCreateWithFlags(&m->ev_ready, cudaEventDisableTiming) == cudaSuccess;
    ok = ok && cudaEventCreateWithFlags(&m->ev_done[0], cudaEventDisableTiming) == cudaSuccess;
    ok = ok && cudaEventCreateWithFlags(&m->ev_done[1], cudaEventDisableTiming) == cudaSuccess;
    m->overlap_prefill = ok;
  }
  // decode-time peer buffers (collective: every rank creates its runner at the same point)
  const char* peer_env = getenv("TEENY_TP_PEER");  // "0" keeps decode on NCCL all-reduce (for A/B measurements)
  // (two pushes per layer, each with its own round number below 1023)
  if (m->tp && cfg->tp_size > 1 && cfg->max_batch <= 128 && 2 * cfg->num_layers < 1023 && !(peer_env && peer_env[0] == '0')) {
    const int trc = tp_enable_peer(m->tp, cfg->max_batch, cfg->hidden, reinterpret_cast<cudaStream_t>(stream));
    if (trc != 0) {
      delete m;
      return trc;
    }
  }
  // split-K counters must start at zero; generation state too
  cudaError_t e = cudaMemsetAsync(m->ws + w.gemm_scratch, 0, w.gemm_scratch_bytes, st);
  if (e == cudaSuccess) e = cudaMemsetAsync(m->ws + w.state, 0, 16, st);
  if (e == cudaSuccess) e = cudaMemsetAsync(m->ws + w.attn_counters, 0, w.attn_counter_bytes, st);
  if (e != cudaSuccess) {
    delete m;
    return static_cast<int>(e);
  }
  *out = m;
  return 0;
}

void teeny_qwen3_destroy(teeny_qwen3* m) {
  if (!m) return;
  if (m->graph_exec) cudaGraphExecDestroy(m->graph_exec);
  if (m->capture_stream) cudaStreamDestroy(m->capture_stream);
  if (m->comm_stream) cudaStreamDestroy(m->comm_stream);
  if (m->ev_ready) cudaEventDestroy(m->ev_ready);
  for (cudaEvent_t ev : m->ev_done)
    if (ev) cudaEventDestroy(ev);
  delete m;
}

int teeny_qwen3_set_weight(teeny_qwen3* m, int layer, int which, const void* ptr) {
  if (!m || !ptr) return TEENY_ERR_BAD_ARG;
  if (reinterpret_cast<uintptr_t>(ptr) & 15) return TEENY_ERR_ALIGNMENT;
  const bf16* p = static_cast<const bf16*>(ptr);
  if (which >= TEENY_QWEN3_W_EMBED) {
    switch (which) {
      case TEENY_QWEN3_W_EMBED: m->embed = p; return 0;
      case TEENY_QWEN3_W_FINAL_NORM: m->final_norm = p; return 0;
      case TEENY_QWEN3_W_LM_HEAD: m->lm_head = Weight{p}; return 0;
      case TEENY_QWEN3_W_INV_FREQ: m->inv_freq = static_cast<const float*>(ptr); m->tables_ready = false; return 0;
      default: return TEENY_ERR_BAD_ARG;
    }
  }
  if (layer < 0 || layer >= m->cfg.num_layers) return TEENY_ERR_BAD_ARG;
  LayerWeights& w = m->layers[layer];
  switch (which) {
    case TEENY_QWEN3_W_QKV: w.qkv = Weight{p}; break;
    case TEENY_QWEN3_W_O: w.o = Weight{p}; break;
    case TEENY_QWEN3_W_GATE_UP: w.gate_up = Weight{p}; break;
    case TEENY_QWEN3_W_DOWN: w.down = Weight{p}; break;
    case TEENY_QWEN3_W_INPUT_LN: w.input_ln = p; break;
    case TEENY_QWEN3_W_POST_LN: w.post_ln = p; break;
    case TEENY_QWEN3_W_Q_NORM: w.q_norm = p; break;
    case TEENY_QWEN3_W_K_NORM: w.k_norm = p; break;
    default: return TEENY_ERR_BAD_ARG;
  }
  return 0;
}

int teeny_qwen3_set_weight_fp8(teeny_qwen3* m, int layer, int which, const void* bytes, const float* scales,
                               int scale_kind, int group_size) {
  if (!m || !bytes || !scales || scale_kind < 0 || scale_kind > 2) return TEENY_ERR_BAD_ARG;
  if (scale_kind == 2 && (group_size <= 0 || group_size % 64 != 0)) return TEENY_ERR_BAD_ARG;
  if (reinterpret_cast<uintptr_t>(bytes) & 15) return TEENY_ERR_ALIGNMENT;
  Weight v;
  v.q = static_cast<const uint8_t*>(bytes);
  v.scale = scales;
  v.kind = scale_kind;
  v.group = group_size;
  if (which == TEENY_QWEN3_W_LM_HEAD) { m->lm_head = v; return 0; }
  if (layer < 0 || layer >= m->cfg.num_layers) return TEENY_ERR_BAD_ARG;
  LayerWeights& w = m->layers[layer];
  switch (which) {
    case TEENY_QWEN3_W_QKV: w.qkv = v; break;
    case TEENY_QWEN3_W_O: w.o = v; break;
    case TEENY_QWEN3_W_GATE_UP: w.gate_up = v; break;
    case TEENY_QWEN3_W_DOWN: w.down = v; break;
    default: return TEENY_ERR_BAD_ARG;  // norms, the embedding table and inv_freq stay in their own types
  }
  return 0;
}

size_t teeny_qwen3_fp8_scratch_bytes(const teeny_qwen3_config* cfg) {
  if (!cfg || cfg->tp_size <= 0) return 0;
  const size_t H = static_cast<size_t>(cfg->hidden), D = static_cast<size_t>(cfg->head_dim);
  const size_t qkv = (static_cast<size_t>(cfg->num_q_heads) + 2 * static_cast<size_t>(cfg->num_kv_heads)) / cfg->tp_size * D;
  const size_t gate_up = 2 * static_cast<size_t>(cfg->intermediate) / cfg->tp_size;
  const size_t rows = qkv > gate_up ? qkv : gate_up;  // O and down have no more elements than these two
  return (rows > H ? rows : H) * H * sizeof(bf16);
}

int teeny_qwen3_set_fp8_scratch(teeny_qwen3* m, void* scratch, size_t bytes) {
  if (!m || (scratch && (reinterpret_cast<uintptr_t>(scratch) & 15))) return TEENY_ERR_BAD_ARG;
  m->fp8_scratch = scratch;
  m->fp8_scratch_bytes = scratch ? bytes : 0;
  return 0;
}

static int check_ready(teeny_qwen3* m, cudaStream_t st) {
  if (!m->embed || !m->final_norm || !m->lm_head.set() || !m->inv_freq) return TEENY_ERR_BAD_ARG;
  for (const LayerWeights& w : m->layers)
    if (!w.qkv.set() || !w.o.set() || !w.gate_up.set() || !w.down.set() || !w.input_ln || !w.post_ln || !w.q_norm ||
        !w.k_norm)
      return TEENY_ERR_BAD_ARG;
  if (!m->tables_ready) {
    TEENY_TRY(rope_table_bf16(m->inv_freq, m->at<bf16>(m->off.cos), m->at<bf16>(m->off.sin), m->cfg.max_len,
                              m->cfg.head_dim, st));
    m->tables_ready = true;
  }
  return 0;
}

int teeny_qwen3_prefill(teeny_qwen3* m, const int* ids, int B, int S, teeny_stream_t stream) {
  if (!m || !ids || B <= 0 || S <= 0) return TEENY_ERR_BAD_ARG;
  const teeny_qwen3_config& c = m->cfg;
  if (B > c.max_batch || S > c.max_len || static_cast<long long>(B) * S > c.max_tokens) return TEENY_ERR_BAD_ARG;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  TEENY_TRY(check_ready(m, st));
  PdlScope pdl;
  m->batch = B;
  m->next_pos = S;
  // a decode step that failed half-way may have left a push waiting for its norm: a new generation starts clean
  m->pending_gather = false;
  m->push_round = 0;
  int* state = m->at<int>(m->off.state);
  TEENY_TRY(embedding_bf16(ids, m->embed, m->at<bf16>(m->off.h), B * S, c.hidden, c.vocab, st));
  if (m->overlap_prefill && B % 2 == 0 && B * S >= 512)  // small prefills have nothing to hide
    TEENY_TRY(run_layers_prefill_overlap(m, B, S, st));
  else
    TEENY_TRY(run_layers(m, B, S, 0, nullptr, nullptr, false, st));
  TEENY_TRY(run_head(m, B, S, st));
  // generation state: next position S, live length during the next step S + 1, no tokens recorded yet
  launch_kernel(set_state_kernel, dim3(1), dim3(1), 0, st, 1, state, S - 1, S, 0);
  launch_kernel(finish_step_kernel, dim3(1), dim3(1024), 0, st, 1, m->at<int>(m->off.next_ids), m->at<int>(m->off.cur_ids),
                                         m->at<int>(m->off.history), state, B, c.max_new_tokens,
                                         static_cast<unsigned*>(nullptr));
  return static_cast<int>(cudaGetLastError());
}

int teeny_qwen3_decode(teeny_qwen3* m, teeny_stream_t stream) {
  if (!m || m->batch <= 0) return TEENY_ERR_BAD_ARG;
  // A step appends at cache row next_pos.  Past the capacity the append would be skipped while the live length kept
  // growing, and the tokens would be silently wrong: refuse instead.
  if (m->next_pos >= m->cfg.max_len) return TEENY_ERR_BAD_ARG;
  const int rc = decode_body(m, m->batch, reinterpret_cast<cudaStream_t>(stream));
  if (rc == 0) ++m->next_pos;
  return rc;
}

int teeny_qwen3_set_sampling(teeny_qwen3* m, float temperature, int top_k, float top_p, unsigned long long seed) {
  if (!m) return TEENY_ERR_BAD_ARG;
  if (temperature > 0.0f) {
    if (top_k < 1 || top_k > 1024 || !(top_p > 0.0f) || top_p > 1.0f) return TEENY_ERR_BAD_ARG;
    m->sample_temperature = temperature; m->sample_top_k = top_k; m->sample_top_p = top_p; m->sample_seed = seed;
  } else {
    m->sample_temperature = 0.0f;
  }
  if (m->graph_exec) {  // the captured step has the old selection baked in
    cudaGraphExecDestroy(m->graph_exec);
    m->graph_exec = nullptr;
  }
  return TEENY_OK;
}

int teeny_qwen3_capture_decode(teeny_qwen3* m, teeny_stream_t stream) {
  if (!m || m->batch <= 0) return TEENY_ERR_BAD_ARG;
  (void)stream;  // recording needs a non-default stream of its own; the graph is replayed on the caller's stream
  if (m->graph_exec) {
    cudaGraphExecDestroy(m->graph_exec);
    m->graph_exec = nullptr;
  }
  cudaError_t e = cudaSuccess;
  if (!m->capture_stream) e = cudaStreamCreateWithFlags(&m->capture_stream, cudaStreamNonBlocking);
  if (e != cudaSuccess) return static_cast<int>(e);
  cudaStream_t st = m->capture_stream;
  e = cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal);
  if (e != cudaSuccess) return static_cast<int>(e);
  const unsigned long long launches_before = launches_so_far();
  const int rc = decode_body(m, m->batch, st);
  m->graph_kernels = launches_so_far() - launches_before;
  cudaGraph_t graph = nullptr;
  e = cudaStreamEndCapture(st, &graph);
  if (rc != 0) {
    if (graph) cudaGraphDestroy(graph);
    return rc;
  }
  if (e != cudaSuccess) return static_cast<int>(e);
  e = cudaGraphInstantiate(&m->graph_exec, graph, 0);
  cudaGraphDestroy(graph);
  if (e != cudaSuccess) return static_cast<int>(e);
  m->graph_batch = m->batch;
  return 0;
}

int teeny_qwen3_decode_replay(teeny_qwen3* m, teeny_stream_t stream) {
  if (!m || !m->graph_exec || m->graph_batch != m->batch) return TEENY_ERR_BAD_ARG;
  if (m->next_pos >= m->cfg.max_len) return TEENY_ERR_BAD_ARG;  // cache full (see teeny_qwen3_decode)
  const int rc = static_cast<int>(cudaGraphLaunch(m->graph_exec, reinterpret_cast<cudaStream_t>(stream)));
  if (rc == 0) {
    ++m->next_pos;
    count_launches(m->graph_kernels);
  }
  return rc;
}

void* teeny_qwen3_buffer(teeny_qwen3* m, int which) {
  if (!m) return nullptr;
  switch (which) {
    case TEENY_QWEN3_BUF_LOGITS: return m->ws + m->off.logits;
    case TEENY_QWEN3_BUF_NEXT_IDS: return m->ws + m->off.cur_ids;
    case TEENY_QWEN3_BUF_HISTORY: return m->ws + m->off.history;
    case TEENY_QWEN3_BUF_STATE: return m->ws + m->off.state;
    case TEENY_QWEN3_BUF_HIDDEN: return m->ws + m->off.y;
    case TEENY_QWEN3_BUF_K_CACHE: return m->ws + m->off.kcache;
    case TEENY_QWEN3_BUF_V_CACHE: return m->ws + m->off.vcache;
    case TEENY_QWEN3_BUF_RESIDUAL: return m->ws + m->off.h;
    case TEENY_QWEN3_BUF_LAST_DELTA: return m->ws + m->off.delta;
    default: return nullptr;
  }
}

// ---- tensor-parallel plumbing ----
int teeny_tp_unique_id(void* out128) {
  if (!out128) return TEENY_ERR_BAD_ARG;
  if (!load_nccl()) return TEENY_ERR_NCCL;
  static_assert(sizeof(ncclUniqueId) == 128, "ncclUniqueId size");
  ncclUniqueId id;
  if (g_nccl.GetUniqueId(&id) != ncclSuccess) return TEENY_ERR_NCCL;
  std::memcpy(out128, &id, sizeof(id));
  return 0;
}

int teeny_tp_init(const void* id128, int rank, int world, void** comm_out) {
  if (!id128 || !comm_out || world <= 0 || rank < 0 || rank >= world) return TEENY_ERR_BAD_ARG;
  if (!load_nccl()) return TEENY_ERR_NCCL;
  ncclUniqueId id;
  std::memcpy(&id, id128, sizeof(id));
  ncclComm_t comm = nullptr;
  // Only when the caller reserved SMs for the collective (TEENY_TP_COMM_SMS) is NCCL told to stay within them; otherwise
  // NCCL's own choice of CTAs stands (a caller's NCCL_MAX_CTAS always wins).
  if (comm_sms() > 0) {
    char buf[16];
    snprintf(buf, sizeof(buf), "%d", comm_sms());
    setenv("NCCL_MAX_CTAS", buf, 0);
  }
  // TEENY_TP_INIT_TIMEOUT_MS: how long the rendezvous may take before it is abandoned (default 5 minutes; 0 = plain
  // blocking ncclCommInitRank, which waits for ever for a rank that never comes).
  long timeout_ms = 300000;
  if (const char* e = getenv("TEENY_TP_INIT_TIMEOUT_MS")) timeout_ms = atol(e);
  const bool can_guard = g_nccl.CommInitRankConfig && g_nccl.CommGetAsyncError && g_nccl.CommAbort && g_nccl.Broadcast;
  if (timeout_ms > 0 && can_guard) {
    const int rc = guarded_comm_init(id, rank, world, timeout_ms, &comm);
    if (rc != 0) return rc;
  } else if (g_nccl.CommInitRank(&comm, world, id, rank) != ncclSuccess) {
    return TEENY_ERR_NCCL;
  }
  TpContext* c = new (std::nothrow) TpContext();
  if (!c) return TEENY_ERR_BAD_ARG;
  c->comm = comm;
  c->rank = rank;
  c->world = world;
  *comm_out = c;
  return 0;
}

int teeny_tp_destroy(void* ctx) {
  if (!ctx) return 0;
  if (!load_nccl()) return TEENY_ERR_NCCL;
  TpContext* c = static_cast<TpContext*>(ctx);
  for (int q = 0; q < c->world; ++q)
    if (c->peer_ok && q != c->rank && c->peer[q]) cudaIpcCloseMemHandle(c->peer[q]);
  if (c->local) cudaFree(c->local);
  if (c->recv_tab) cudaFree(c->recv_tab);
  if (c->bcast_tab) cudaFree(c->bcast_tab);
  const bool ok = g_nccl.CommDestroy(c->comm) == ncclSuccess;
  delete c;
  return ok ? 0 : TEENY_ERR_NCCL;
}

int teeny_tp_all_reduce_bf16(void* ctx, teeny_bf16* buf, size_t count, teeny_stream_t stream) {
  if (!ctx || !buf) return TEENY_ERR_BAD_ARG;
  if (!load_nccl()) return TEENY_ERR_NCCL;
  return g_nccl.AllReduce(buf, buf, count, ncclBfloat16, ncclSum, static_cast<TpContext*>(ctx)->comm,
                          reinterpret_cast<cudaStream_t>(stream)) == ncclSuccess ? 0 : TEENY_ERR_NCCL;
}

int teeny_tp_peer_enabled(void* ctx) { return ctx && static_cast<TpContext*>(ctx)->peer_ok ? 1 : 0; }

int teeny_tp_gather_add_rms_norm_bf16(const void* recv, size_t slot_elems, int world, const uint32_t* epoch,
                                      uint32_t round, teeny_bf16* residual, teeny_bf16* y, const teeny_bf16* weight,
                                      int M, int N, float eps, unsigned long long wait_limit_ns, teeny_stream_t stream) {
  return gather_add_rms_norm_bf16(static_cast<const uint2*>(recv), slot_elems, world, epoch, round,
                                  reinterpret_cast<bf16*>(residual), N, reinterpret_cast<bf16*>(y), N,
                                  reinterpret_cast<const bf16*>(weight), M, N, eps, reinterpret_cast<cudaStream_t>(stream),
                                  wait_limit_ns);
}

}  // extern "C"
