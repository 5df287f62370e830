/*
 * teeny_qwen3 -- C ABI of the Qwen3 decoder runner and its tensor-parallel plumbing (libteeny_b200.so).
 *
 * The runner is this backend's counterpart of the reference's model executor for one model family:
 *   load / forward / capture / replay  <->  CudaModel::load, LoadedModel::forward, capture_graph, CudaGraphModel::run
 *                                           (drivers/teeny-cuda/src/model/mod.rs:231, 524, 1245, 1799)
 *   weights by name                    <->  LoadedModel::param_info_named / load_param_f32 (model/mod.rs:449, 476)
 * executing the Qwen3 op sequence the reference records in support/teeny-torch/tests/data/qwen3_{1,2,3}.bin.gz
 * (the reference itself runs that graph with PyTorch on the CPU, support/teeny-torch/python/teenygrad/atlas/module.py:42-45).
 * The reference has no multi-GPU code; the teeny_tp_* functions have no counterpart there.
 *
 * All pointers are device pointers owned by the caller unless stated; nothing here allocates device memory.
 * Status codes are those of teeny_b200.h.
 */
#ifndef TEENY_QWEN3_H_
#define TEENY_QWEN3_H_

#include "teeny_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct {
  int num_layers, hidden, num_q_heads, num_kv_heads, head_dim, intermediate, vocab;
  float eps;          /* RMSNorm epsilon (1e-6) */
  int max_batch;      /* sequences per generation */
  int max_len;        /* KV-cache capacity per sequence (prompt + generated) */
  int max_tokens;     /* most tokens in one prefill call (batch * prompt length) */
  int max_new_tokens; /* capacity of the generated-token history */
  int tp_rank, tp_size;
} teeny_qwen3_config;

typedef struct teeny_qwen3 teeny_qwen3;

/* Weight slots.  Per-layer tensors are this rank's shard, fused where the layer fuses them (row-major bf16):
 *   QKV      [(Hq/tp + 2 Hkv/tp) * 128, hidden]   rows: local q heads, then local k heads, then local v heads
 *   O        [hidden, Hq/tp * 128]                 column slice of o_proj (row-parallel)
 *   GATE_UP  [2 * intermediate/tp, hidden]         local gate / up rows interleaved in blocks of 64 channels
 *                                                  (see teeny_linear_swiglu_bf16)
 *   DOWN     [hidden, intermediate/tp]             column slice of down_proj (row-parallel)
 *   INPUT_LN, POST_LN [hidden]; Q_NORM, K_NORM [128]
 * Model-level: EMBED [vocab, hidden] (replicated), FINAL_NORM [hidden], LM_HEAD [vocab/tp, hidden] (row slice; for
 * tied embeddings a slice of EMBED), INV_FREQ f32 [64] (the rotary inv_freq buffer of the model). */
enum {
  TEENY_QWEN3_W_QKV = 0, TEENY_QWEN3_W_O, TEENY_QWEN3_W_GATE_UP, TEENY_QWEN3_W_DOWN, TEENY_QWEN3_W_INPUT_LN,
  TEENY_QWEN3_W_POST_LN, TEENY_QWEN3_W_Q_NORM, TEENY_QWEN3_W_K_NORM,
  TEENY_QWEN3_W_EMBED = 100, TEENY_QWEN3_W_FINAL_NORM, TEENY_QWEN3_W_LM_HEAD, TEENY_QWEN3_W_INV_FREQ
};
enum {
  TEENY_QWEN3_BUF_LOGITS = 0, /* bf16 [batch, vocab/tp]: LM-head output of the last step (this rank's slice) */
  TEENY_QWEN3_BUF_NEXT_IDS,   /* int32 [batch]: token chosen by the last step (input of the next) */
  TEENY_QWEN3_BUF_HISTORY,    /* int32 [max_new_tokens, batch]: every token generated so far */
  TEENY_QWEN3_BUF_STATE,      /* int32 [3]: next position, live KV length of the coming step, tokens generated */
  TEENY_QWEN3_BUF_HIDDEN,     /* bf16 [batch, hidden]: final-norm output of the last step */
  TEENY_QWEN3_BUF_K_CACHE,    /* bf16 [layers, max_batch, Hkv/tp, max_len, 128] */
  TEENY_QWEN3_BUF_V_CACHE,
  /* For layer-level checks (the reference reads intermediate tensors the same way, TensorRef outputs of
   * LoadedModel::forward, drivers/teeny-cuda/src/model/mod.rs:524): after a call, RESIDUAL holds the residual stream
   * before the last layer's MLP output was added and LAST_DELTA that (summed over ranks) output, both bf16
   * [tokens, hidden], so residual + delta is the hidden state the final norm sees.  Rows of each sequence's last
   * position already have the sum in RESIDUAL (the head adds it in place). */
  TEENY_QWEN3_BUF_RESIDUAL,
  TEENY_QWEN3_BUF_LAST_DELTA
};

/* Bytes of workspace (activations, KV cache, RoPE tables, scratch, generation state) for this configuration;
 * 0 if the configuration is not supported (head_dim must be 128; heads, intermediate and vocab divisible by tp). */
size_t teeny_qwen3_workspace_bytes(const teeny_qwen3_config* cfg);
/* Creates the runner over a caller-allocated, 256-byte aligned workspace.  tp_comm: handle from teeny_tp_init when
 * tp_size > 1, else NULL.  Only the small host-side object is allocated here; free it with teeny_qwen3_destroy. */
int teeny_qwen3_create(const teeny_qwen3_config* cfg, void* workspace, size_t workspace_bytes, void* tp_comm,
                       teeny_stream_t stream, teeny_qwen3** out);
void teeny_qwen3_destroy(teeny_qwen3* model);
int teeny_qwen3_set_weight(teeny_qwen3* model, int layer, int which, const void* device_ptr);
/* The same for a projection weight (QKV, O, GATE_UP, DOWN of a layer, or LM_HEAD) given as FP8 E4M3 bytes with f32
 * scales, the "float-quantized" tensors the reference's quantiser writes (utilities/teeny-quant/src/format.rs:215-240);
 * shapes, fusion and row order as for the bf16 slots, scale_kind / group_size as in teeny_linear_w8a16_forward
 * (include/teeny_b200.h), scales of fused or interleaved rows in the same row order.  Decode streams the bytes
 * (teeny_linear_w8a16_forward's M <= 128 path); a prefill of more than 128 tokens converts one projection at a time
 * into the scratch given by teeny_qwen3_set_fp8_scratch (teeny_qwen3_fp8_scratch_bytes for this configuration) and
 * fails with TEENY_ERR_SCRATCH without it.  Norm weights, the embedding table and inv_freq keep their own types. */
int teeny_qwen3_set_weight_fp8(teeny_qwen3* model, int layer, int which, const void* fp8_bytes, const float* scales,
                               int scale_kind, int group_size);
size_t teeny_qwen3_fp8_scratch_bytes(const teeny_qwen3_config* cfg);
int teeny_qwen3_set_fp8_scratch(teeny_qwen3* model, void* scratch, size_t bytes);
/* Prefill: ids int32 [B, S] on the device.  Fills the KV cache, picks the first generated token of every sequence
 * (greedy, lowest index on ties) and records it as history[0]. */
int teeny_qwen3_prefill(teeny_qwen3* model, const int* ids, int B, int S, teeny_stream_t stream);
/* One greedy decode step for the batch of the last prefill: consumes NEXT_IDS, appends to the cache, produces the
 * next token.  teeny_qwen3_decode launches the kernels directly; capture_decode records one step into a CUDA graph
 * (position and length live in device memory, so one graph serves every step) and decode_replay launches it.
 * A generation holds at most max_len cache rows: once prefill length + decode steps reaches max_len, decode and
 * decode_replay return TEENY_ERR_BAD_ARG and launch nothing. */
int teeny_qwen3_decode(teeny_qwen3* model, teeny_stream_t stream);
/* Token selection.  temperature <= 0 (the default): greedy argmax, lowest index on ties.  temperature > 0: the
 * temperature / top-k (1..1024) / top-p sampler of teeny_sample_top_k_top_p_bf16, with u for token t of a generation
 * and batch row r drawn by a stateless hash of (seed, t, r), so a generation is reproducible and replayable on the
 * CPU.  Under tensor parallelism every rank sends the top-k candidates of its vocabulary shard to all ranks and all
 * make the same pick (teeny_sample_candidates_bf16 / teeny_sample_merge).  Drops a captured decode graph: capture
 * again afterwards. */
int teeny_qwen3_set_sampling(teeny_qwen3* model, float temperature, int top_k, float top_p, unsigned long long seed);
int teeny_qwen3_capture_decode(teeny_qwen3* model, teeny_stream_t stream);
int teeny_qwen3_decode_replay(teeny_qwen3* model, teeny_stream_t stream);
/* Device address of one of the runner's buffers inside the workspace (see enum above). */
void* teeny_qwen3_buffer(teeny_qwen3* model, int which);

/* Tensor-parallel plumbing over NCCL (loaded at run time; the process's already-loaded libnccl is reused).
 * Rank 0 calls teeny_tp_unique_id and ships the 128 bytes to the other ranks by any host channel.  teeny_tp_init
 * allocates the small host-side context; teeny_qwen3_create may add a peer-mapped device buffer of
 * 2 * tp_size * max_batch * hidden (value, stamp) pairs to it (the one device allocation this library makes, at
 * set-up). */
int teeny_tp_unique_id(void* out128);
/* Collective over all `world` ranks.  The rendezvous cannot hang on a rank that never arrives: it is made with a
 * non-blocking guard communicator that is polled against a host timeout (TEENY_TP_INIT_TIMEOUT_MS in the environment,
 * default 300000; 0 = plain blocking ncclCommInitRank) and aborted with ncclCommAbort when the timeout expires, in
 * which case TEENY_ERR_NCCL is returned and nothing is left behind.  TEENY_NCCL_LIB names the NCCL library to load
 * (default libnccl.so.2). */
int teeny_tp_init(const void* id128, int rank, int world, void** comm_out);
int teeny_tp_destroy(void* comm);
int teeny_tp_all_reduce_bf16(void* comm, teeny_bf16* buf, size_t count, teeny_stream_t stream);
/* 1 when the context's decode path pushes row-parallel partial sums straight into the peers' memory (set up by
 * teeny_qwen3_create when tp_size > 1 and max_batch <= 128; needs CUDA IPC between the ranks' processes), 0 when it
 * all-reduces through NCCL instead. */
int teeny_tp_peer_enabled(void* comm);
/* The receiving half of the decode-time row-parallel reduction, for hosts that run their own layer loop (the runner
 * uses the same kernel).  recv holds `world` copies of the projection, slot_elems elements apart, each element one
 * 64-bit word {f32 value, 32-bit stamp} that the ranks' GEMM epilogues stored over NVLink; an element has arrived when
 * its stamp equals *epoch * 1024 + round + 1.  The kernel waits per element, sums the copies in rank order in f32,
 * rounds the sum to bf16, adds it into residual [M, N] and writes y = rms_norm(residual) * weight.  No wait is
 * unbounded: after wait_limit_ns nanoseconds without progress (0 = the library's 2 s) the kernel stores 0x301 in the
 * device error word (teeny_device_error) and returns, leaving the context usable.  The reference has no multi-GPU
 * path and no counterpart. */
int teeny_tp_gather_add_rms_norm_bf16(const void* recv, size_t slot_elems, int world, const uint32_t* epoch,
                                      uint32_t round, teeny_bf16* residual, teeny_bf16* y, const teeny_bf16* weight,
                                      int M, int N, float eps, unsigned long long wait_limit_ns, teeny_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* TEENY_QWEN3_H_ */
