"""Qwen3 runner: host wrapper over the C++ executor in libteeny_b200.so (include/teeny_qwen3.h).

Stands where the reference's ``apps/teeny-llm`` wants its Qwen3 path (the reference binary is a placeholder,
``apps/teeny-llm/src/server/main.rs:6-8``); the computation the reference actually runs for Qwen3 is HF
transformers on PyTorch CPU (``support/teeny-torch/python/tests/test_qwen3.py:24-41``), so the interface mirrors
that: HF-named state dict in, greedy ``generate`` out.  torch is used for device memory and streams only.
"""
import ctypes as C
from dataclasses import dataclass

import torch

from . import _lib, tp as tpmod
from ._lib import lib, check, vp, i32, f32, sz

_BF16 = torch.bfloat16


class _Cfg(C.Structure):
    """teeny_qwen3_config"""
    _fields_ = [(n, i32) for n in ("num_layers", "hidden", "num_q_heads", "num_kv_heads", "head_dim",
                                   "intermediate", "vocab")] + [("eps", f32)] + \
               [(n, i32) for n in ("max_batch", "max_len", "max_tokens", "max_new_tokens", "tp_rank", "tp_size")]


SIGNATURES = {
    "teeny_qwen3_workspace_bytes": (sz, [C.POINTER(_Cfg)]),
    "teeny_qwen3_create": (i32, [C.POINTER(_Cfg), vp, sz, vp, vp, C.POINTER(vp)]),
    "teeny_qwen3_destroy": (None, [vp]),
    "teeny_qwen3_set_weight": (i32, [vp, i32, i32, vp]),
    "teeny_qwen3_set_weight_fp8": (i32, [vp, i32, i32, vp, vp, i32, i32]),
    "teeny_qwen3_fp8_scratch_bytes": (sz, [C.POINTER(_Cfg)]),
    "teeny_qwen3_set_fp8_scratch": (i32, [vp, vp, sz]),
    "teeny_qwen3_prefill": (i32, [vp, vp, i32, i32, vp]),
    "teeny_qwen3_decode": (i32, [vp, vp]),
    "teeny_qwen3_set_sampling": (i32, [vp, f32, i32, f32, C.c_ulonglong]),
    "teeny_qwen3_capture_decode": (i32, [vp, vp]),
    "teeny_qwen3_decode_replay": (i32, [vp, vp]),
    "teeny_qwen3_buffer": (vp, [vp, i32]),
    "teeny_tp_unique_id": (i32, [vp]),
    "teeny_tp_init": (i32, [C.c_char_p, i32, i32, C.POINTER(vp)]),
    "teeny_tp_destroy": (i32, [vp]),
    "teeny_tp_all_reduce_bf16": (i32, [vp, vp, sz, vp]),
    "teeny_tp_peer_enabled": (i32, [vp]),
    "teeny_tp_gather_add_rms_norm_bf16": (i32, [vp, sz, i32, vp, C.c_uint32, vp, vp, vp, i32, i32, f32, C.c_ulonglong, vp]),
}
_lib.bind(SIGNATURES)

W_QKV, W_O, W_GATE_UP, W_DOWN, W_INPUT_LN, W_POST_LN, W_Q_NORM, W_K_NORM = range(8)
W_EMBED, W_FINAL_NORM, W_LM_HEAD, W_INV_FREQ = 100, 101, 102, 103
BUF_LOGITS, BUF_NEXT_IDS, BUF_HISTORY, BUF_STATE, BUF_HIDDEN, BUF_K_CACHE, BUF_V_CACHE, BUF_RESIDUAL, BUF_LAST_DELTA = range(9)
_LAYER_SLOTS = {"qkv": W_QKV, "o": W_O, "gate_up": W_GATE_UP, "down": W_DOWN, "input_ln": W_INPUT_LN,
                "post_ln": W_POST_LN, "q_norm": W_Q_NORM, "k_norm": W_K_NORM}


@dataclass
class Qwen3Config:
    num_layers: int
    hidden: int
    num_q_heads: int
    num_kv_heads: int
    head_dim: int
    intermediate: int
    vocab: int
    eps: float = 1e-6
    rope_theta: float = 1e6
    tied: bool = False


QWEN3_0_6B = Qwen3Config(28, 1024, 16, 8, 128, 3072, 151936, tied=True)
QWEN3_8B = Qwen3Config(36, 4096, 32, 8, 128, 12288, 151936, tied=False)


def default_inv_freq(cfg):
    """The model's rotary ``inv_freq`` buffer: 1 / theta^(2i/D), f32 (what HF's default rope init stores)."""
    return 1.0 / (cfg.rope_theta ** (torch.arange(0, cfg.head_dim, 2, dtype=torch.int64).float() / cfg.head_dim))


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def check_generation_fits(prompt_len, max_new_tokens, max_len, history_capacity):
    """Raises unless a generation of ``max_new_tokens`` after a prompt of ``prompt_len`` fits the runner: the first
    token comes out of the prefill, each later one appends one cache row, so rows 0 .. prompt_len + max_new_tokens - 2
    must exist.  (The C side refuses the step that would overflow as well; this fails before any launch.)"""
    if max_new_tokens > history_capacity:
        raise ValueError("max_new_tokens exceeds the runner's history capacity")
    if prompt_len + max_new_tokens - 1 > max_len:
        raise ValueError(f"prompt of {prompt_len} + {max_new_tokens} new tokens needs {prompt_len + max_new_tokens - 1} "
                         f"cache rows; the runner was created with max_len={max_len}")


class Qwen3Runner:
    """Greedy Qwen3 decoding on one GPU (or one tensor-parallel rank)."""

    def __init__(self, cfg, max_batch, max_len, max_tokens=None, max_new_tokens=256, tp_rank=0, tp_size=1,
                 comm=None, device=None):
        self.cfg = cfg
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        tpmod.check_divisible(cfg, tp_size)
        c = _Cfg()
        c.num_layers, c.hidden, c.num_q_heads, c.num_kv_heads = cfg.num_layers, cfg.hidden, cfg.num_q_heads, cfg.num_kv_heads
        c.head_dim, c.intermediate, c.vocab, c.eps = cfg.head_dim, cfg.intermediate, cfg.vocab, cfg.eps
        c.max_batch, c.max_len = max_batch, max_len
        c.max_tokens = max_tokens if max_tokens is not None else max_batch * max_len
        c.max_new_tokens, c.tp_rank, c.tp_size = max_new_tokens, tp_rank, tp_size
        self._c = c
        self.tp_rank, self.tp_size, self.max_batch, self.max_new_tokens = tp_rank, tp_size, max_batch, max_new_tokens
        self.max_len = max_len
        nbytes = lib.teeny_qwen3_workspace_bytes(C.byref(c))
        if nbytes == 0:
            raise ValueError("unsupported Qwen3 configuration for this backend")
        self.workspace = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
        self._h = vp()
        self._comm = comm
        check(lib.teeny_qwen3_create(C.byref(c), C.c_void_p(self.workspace.data_ptr()), nbytes, comm, _stream(),
                                     C.byref(self._h)), "teeny_qwen3_create")
        self._weights = []  # keeps device tensors alive
        self._captured = False
        self.batch = 0

    def __del__(self):
        h = getattr(self, "_h", None)
        if h and lib is not None:  # at interpreter shutdown the module globals may already be gone
            lib.teeny_qwen3_destroy(h)
            self._h = None

    # ---- weights ----
    def _set(self, layer, which, t):
        t = t.to(self.device).contiguous()
        self._weights.append(t)
        check(lib.teeny_qwen3_set_weight(self._h, layer, which, C.c_void_p(t.data_ptr())), "teeny_qwen3_set_weight")

    def load_layer_shards(self, layer, shards):
        for name, slot in _LAYER_SLOTS.items():
            self._set(layer, slot, shards[name].to(_BF16))

    def load_head_shards(self, shards, inv_freq=None):
        self._set(0, W_EMBED, shards["embed"].to(_BF16))
        self._set(0, W_FINAL_NORM, shards["final_norm"].to(_BF16))
        if isinstance(shards["lm_head"], torch.Tensor):
            self._set(0, W_LM_HEAD, shards["lm_head"].to(_BF16))
        else:  # a quant.Fp8Weight
            self._set_fp8(0, W_LM_HEAD, shards["lm_head"])
        inv = default_inv_freq(self.cfg) if inv_freq is None else inv_freq
        self._set(0, W_INV_FREQ, inv.to(torch.float32))

    # ---- FP8 weights (the reference quantiser's float-quantized checkpoints, see quant.py) ----
    def _set_fp8(self, layer, which, w):
        from . import ops
        w = w.to(self.device)
        if ops.fp8_count_nan(w.q):
            raise ValueError("FP8 weight holds NaN encodings (0x7f / 0xff), which the streaming GEMM does not reproduce")
        self._weights += [w.q, w.scale]
        kind = 2 if w.group_size else 1
        check(lib.teeny_qwen3_set_weight_fp8(self._h, layer, which, C.c_void_p(w.q.data_ptr()),
                                             C.c_void_p(w.scale.data_ptr()), kind, w.group_size), "teeny_qwen3_set_weight_fp8")
        if self._c.max_tokens > 128 and getattr(self, "_fp8_scratch", None) is None:
            # a prefill of more than 128 tokens converts one projection at a time into this buffer
            n = lib.teeny_qwen3_fp8_scratch_bytes(C.byref(self._c))
            self._fp8_scratch = torch.empty(n, dtype=torch.uint8, device=self.device)
            check(lib.teeny_qwen3_set_fp8_scratch(self._h, C.c_void_p(self._fp8_scratch.data_ptr()), n),
                  "teeny_qwen3_set_fp8_scratch")

    def load_layer_shards_fp8(self, layer, shards):
        """``shards``: name -> quant.Fp8Weight for the four projections, bf16 tensors for the norms."""
        for name, slot in _LAYER_SLOTS.items():
            t = shards[name]
            if isinstance(t, torch.Tensor):
                self._set(layer, slot, t.to(_BF16))
            else:
                self._set_fp8(layer, slot, t)

    def load_quantized(self, tensors, scheme, inv_freq=None):
        """A checkpoint of the reference's quantiser: ``tensors`` maps HF names to tensors (``*.weight`` quantised next to
        ``*.weight_scale``, norms in a float type), ``scheme`` is quant.parse_quantization_config's.  FP8: projections
        and the LM head stay FP8, the embedding table is converted back to bf16 (on this device) for the lookup.
        Integer schemes: everything is converted back to bf16 on this device."""
        from . import ops, quant
        if isinstance(scheme, quant.IntScheme):  # integer schemes: back to bf16 here, then the ordinary path
            return self.load_state_dict(quant.dequantize_int_state_dict(tensors, scheme, self.device), inv_freq)

        def get(name):
            return quant.Fp8Weight.from_tensors(tensors[name], tensors[name + "_scale"], scheme)

        def norms(i):
            p = f"model.layers.{i}."
            return {"input_ln": tensors[p + "input_layernorm.weight"], "post_ln": tensors[p + "post_attention_layernorm.weight"],
                    "q_norm": tensors[p + "self_attn.q_norm.weight"], "k_norm": tensors[p + "self_attn.k_norm.weight"]}

        for i in range(self.cfg.num_layers):
            shards = quant.shard_layer_fp8(get, self.cfg, i, self.tp_rank, self.tp_size)
            shards.update(norms(i))
            self.load_layer_shards_fp8(i, shards)
        emb_name = "model.embed_tokens.weight"
        if emb_name + "_scale" in tensors:
            e = get(emb_name).to(self.device)
            if ops.fp8_count_nan(e.q):
                raise ValueError("embedding table holds FP8 NaN encodings")
            embed = ops.dequant_fp8(e.q, e.scale, e.strategy, e.group_size)
        else:
            embed = tensors[emb_name].to(_BF16)
        self._set(0, W_EMBED, embed)
        self._set(0, W_FINAL_NORM, tensors["model.norm.weight"].to(_BF16))
        head_name = emb_name if self.cfg.tied else "lm_head.weight"
        vl = self.cfg.vocab // self.tp_size
        if head_name + "_scale" in tensors:
            self._set_fp8(0, W_LM_HEAD, get(head_name).rows(self.tp_rank * vl, (self.tp_rank + 1) * vl))
        else:
            self._set(0, W_LM_HEAD, tensors[head_name][self.tp_rank * vl:(self.tp_rank + 1) * vl].to(_BF16))
        inv = default_inv_freq(self.cfg) if inv_freq is None else inv_freq
        self._set(0, W_INV_FREQ, inv.to(torch.float32))

    def load_state_dict(self, sd, inv_freq=None):
        """HF-named full tensors (``model.layers.{i}.self_attn.q_proj.weight`` ...); sharded for this rank here."""
        for i in range(self.cfg.num_layers):
            self.load_layer_shards(i, tpmod.shard_layer(sd, self.cfg, i, self.tp_rank, self.tp_size))
        self.load_head_shards(tpmod.shard_head(sd, self.cfg, self.tp_rank, self.tp_size), inv_freq)

    # ---- buffers ----
    def _view(self, which, shape, dtype):
        ptr = lib.teeny_qwen3_buffer(self._h, which)
        off = ptr - self.workspace.data_ptr()
        n = int(torch.tensor(shape).prod()) * torch.empty(0, dtype=dtype).element_size()
        return self.workspace[off:off + n].view(dtype).view(*shape)

    def logits(self):
        """bf16 [batch, vocab/tp]: this rank's slice of the last step's LM-head output."""
        return self._view(BUF_LOGITS, (self.batch, self.cfg.vocab // self.tp_size), _BF16)

    def next_ids(self):
        return self._view(BUF_NEXT_IDS, (self.batch,), torch.int32)

    def history(self):
        return self._view(BUF_HISTORY, (self.max_new_tokens, self.batch), torch.int32)

    def state(self):
        return self._view(BUF_STATE, (3,), torch.int32)

    def residual_stream(self, tokens):
        """(residual, last_delta), bf16 [tokens, hidden] each: their sum is the hidden state after the last layer
        (rows of each sequence's last position already hold the sum in ``residual``)."""
        return (self._view(BUF_RESIDUAL, (tokens, self.cfg.hidden), _BF16),
                self._view(BUF_LAST_DELTA, (tokens, self.cfg.hidden), _BF16))

    # ---- execution ----
    def prefill(self, ids):
        """ids: int [B, S] (any device).  Runs the prompt, records the first generated token."""
        ids = ids.to(self.device, dtype=torch.int32).contiguous()
        B, S = ids.shape
        if B != self.batch:
            self._captured = False  # the recorded decode step has the batch baked in; everything else is a fixed address
        self.batch = B
        check(lib.teeny_qwen3_prefill(self._h, C.c_void_p(ids.data_ptr()), B, S, _stream()), "teeny_qwen3_prefill")

    def set_sampling(self, temperature, top_k=50, top_p=1.0, seed=0):
        """Token selection for the following generations: ``temperature <= 0`` is greedy; otherwise temperature /
        top-k / top-p sampling with u for token t and row r a stateless hash of (seed, t, r) (single GPU only)."""
        check(lib.teeny_qwen3_set_sampling(self._h, float(temperature), int(top_k), float(top_p), int(seed)),
              "teeny_qwen3_set_sampling")
        self._captured = False

    def decode_step(self, graph=False):
        if graph:
            if not self._captured:
                check(lib.teeny_qwen3_capture_decode(self._h, _stream()), "teeny_qwen3_capture_decode")
                self._captured = True
            check(lib.teeny_qwen3_decode_replay(self._h, _stream()), "teeny_qwen3_decode_replay")
        else:
            check(lib.teeny_qwen3_decode(self._h, _stream()), "teeny_qwen3_decode")

    def generate(self, prompt_ids, max_new_tokens, use_graph=True):
        """Greedy decode; returns int32 [B, max_new_tokens] on the device (no host sync inside)."""
        check_generation_fits(prompt_ids.shape[1], max_new_tokens, self.max_len, self.max_new_tokens)
        self.prefill(prompt_ids)
        for _ in range(max_new_tokens - 1):
            self.decode_step(graph=use_graph)
        return self.history()[:max_new_tokens].t()


def random_weights_device(cfg, seed, device, std=0.02):
    """Synthetic HF-named weights generated on the GPU (N(0, std) drawn in f32, cast to bf16; norms 1.0), one
    seeded generator per tensor so every tensor-parallel rank draws identical full tensors.  Yields
    (name, tensor) lazily so a caller can shard and drop each one."""
    def nrm(tag, *shape):
        g = torch.Generator(device=device).manual_seed(seed * 1000003 + tag)
        return (torch.randn(*shape, generator=g, dtype=torch.float32, device=device) * std).to(_BF16)

    H, D = cfg.hidden, cfg.head_dim
    yield "model.embed_tokens.weight", nrm(1, cfg.vocab, H)
    for i in range(cfg.num_layers):
        p, t = f"model.layers.{i}.", 100 + i * 16
        yield p + "self_attn.q_proj.weight", nrm(t + 0, cfg.num_q_heads * D, H)
        yield p + "self_attn.k_proj.weight", nrm(t + 1, cfg.num_kv_heads * D, H)
        yield p + "self_attn.v_proj.weight", nrm(t + 2, cfg.num_kv_heads * D, H)
        yield p + "self_attn.o_proj.weight", nrm(t + 3, H, cfg.num_q_heads * D)
        yield p + "mlp.gate_proj.weight", nrm(t + 4, cfg.intermediate, H)
        yield p + "mlp.up_proj.weight", nrm(t + 5, cfg.intermediate, H)
        yield p + "mlp.down_proj.weight", nrm(t + 6, H, cfg.intermediate)
        for n in ("self_attn.q_norm.weight", "self_attn.k_norm.weight"):
            yield p + n, torch.ones(D, dtype=_BF16, device=device)
        for n in ("input_layernorm.weight", "post_attention_layernorm.weight"):
            yield p + n, torch.ones(H, dtype=_BF16, device=device)
    yield "model.norm.weight", torch.ones(H, dtype=_BF16, device=device)
    if not cfg.tied:
        yield "lm_head.weight", nrm(2, cfg.vocab, H)


def load_random_weights(runner, seed, fp8=False):
    """Fill a runner with ``random_weights_device`` tensors, sharding layer by layer (peak extra memory = one layer).
    fp8: the projections and the LM head go in as FP8 E4M3 with one scale per output channel (quant.quantize_fp8 of the
    same random tensors), everything else as bf16."""
    from . import quant
    cfg, dev = runner.cfg, runner.device
    pending, head = {}, {}
    for name, t in random_weights_device(cfg, seed, dev):
        if name.startswith("model.layers."):
            layer = int(name.split(".")[2])
            pending[name] = t
            if len(pending) == 11:
                if fp8:
                    shards = quant.shard_layer_fp8(lambda n: quant.quantize_fp8(pending[n]), cfg, layer, runner.tp_rank,
                                                   runner.tp_size)
                    p = f"model.layers.{layer}."
                    shards.update({"input_ln": pending[p + "input_layernorm.weight"],
                                   "post_ln": pending[p + "post_attention_layernorm.weight"],
                                   "q_norm": pending[p + "self_attn.q_norm.weight"],
                                   "k_norm": pending[p + "self_attn.k_norm.weight"]})
                    runner.load_layer_shards_fp8(layer, shards)
                else:
                    runner.load_layer_shards(layer, tpmod.shard_layer(pending, cfg, layer, runner.tp_rank, runner.tp_size))
                pending = {}
        else:
            head[name] = t
    shards = tpmod.shard_head(head, cfg, runner.tp_rank, runner.tp_size)
    if fp8:
        shards["lm_head"] = quant.quantize_fp8(shards["lm_head"])
    runner.load_head_shards(shards)

