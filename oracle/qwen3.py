"""Qwen3 decoder forward restated op by op in plain PyTorch (CPU) -- TEST INFRASTRUCTURE ONLY.

The reference holds Qwen3 only as data: the traced FX graphs
``support/teeny-torch/tests/data/qwen3_{1,2,3}.bin.gz`` of HF ``transformers``' Qwen3 running on
PyTorch CPU (``support/teeny-torch/python/tests/test_qwen3.py:20-41``; the "teenygrad" backend
executes the traced graph with ``self.gm.forward``, ``python/teenygrad/atlas/module.py:42-45``).
The model arithmetic therefore lives in the third-party package ``transformers`` (version unpinned
by the reference's ``support/teeny-torch/pyproject.toml``; 5.5.0 in this image).  This file restates
the op sequence those fixtures record, with the same cast points:

  * RMSNorm: f32 statistics, ``.to(bf16)``, then ``weight * h`` in bf16;
  * per-head q_norm / k_norm over head_dim, no norm on V;
  * RoPE tables: ``inv_freq @ positions`` in f32, ``cos``/``sin`` in f32, cast to bf16; rotation
    ``q*cos + rotate_half(q)*sin`` in bf16 (each mul/add rounds);
  * KV cache holds post-norm post-RoPE K and raw V; GQA by repeating KV heads;
  * ``scaled_dot_product_attention`` with a boolean causal mask and scale head_dim**-0.5;
  * SwiGLU ``down(silu(gate(x)) * up(x))``; bf16 residual adds;
  * final norm, LM head on the last position, greedy argmax (lowest index on ties).

``tests/test_oracle_qwen3.py`` checks this restatement against ``transformers``' own
``Qwen3ForCausalLM`` built from the same weights (logits and greedy ids).
"""
import math
from dataclasses import dataclass, asdict

import torch
import torch.nn.functional as F


@dataclass
class OracleQwen3Config:
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


QWEN3_0_6B = OracleQwen3Config(28, 1024, 16, 8, 128, 3072, 151936, tied=True)
QWEN3_8B = OracleQwen3Config(36, 4096, 32, 8, 128, 12288, 151936, tied=False)


def make_weights(cfg, seed, std=0.02, generator_device="cpu"):
    """HF-named state dict: N(0, std) drawn in f32 from a seeded generator, cast to bf16; norm weights 1.0."""
    g = torch.Generator(device=generator_device).manual_seed(seed)

    def nrm(*shape):
        return (torch.randn(*shape, generator=g, dtype=torch.float32, device=generator_device) * std).to(torch.bfloat16)

    def ones(n):
        return torch.ones(n, dtype=torch.bfloat16, device=generator_device)

    H, D = cfg.hidden, cfg.head_dim
    sd = {"model.embed_tokens.weight": nrm(cfg.vocab, H)}
    for i in range(cfg.num_layers):
        p = f"model.layers.{i}."
        sd[p + "self_attn.q_proj.weight"] = nrm(cfg.num_q_heads * D, H)
        sd[p + "self_attn.k_proj.weight"] = nrm(cfg.num_kv_heads * D, H)
        sd[p + "self_attn.v_proj.weight"] = nrm(cfg.num_kv_heads * D, H)
        sd[p + "self_attn.o_proj.weight"] = nrm(H, cfg.num_q_heads * D)
        sd[p + "self_attn.q_norm.weight"] = ones(D)
        sd[p + "self_attn.k_norm.weight"] = ones(D)
        sd[p + "mlp.gate_proj.weight"] = nrm(cfg.intermediate, H)
        sd[p + "mlp.up_proj.weight"] = nrm(cfg.intermediate, H)
        sd[p + "mlp.down_proj.weight"] = nrm(H, cfg.intermediate)
        sd[p + "input_layernorm.weight"] = ones(H)
        sd[p + "post_attention_layernorm.weight"] = ones(H)
    sd["model.norm.weight"] = ones(H)
    if not cfg.tied:
        sd["lm_head.weight"] = nrm(cfg.vocab, H)
    return sd


def inv_freq(cfg):
    """``1 / theta ** (arange(0, D, 2) / D)`` in f32, as HF's default rope init computes it."""
    return 1.0 / (cfg.rope_theta ** (torch.arange(0, cfg.head_dim, 2, dtype=torch.int64).float() / cfg.head_dim))


def rope_tables(cfg, positions):
    """positions: int64 [T] -> (cos, sin) bf16 [T, D] (f32 angles, f32 cos/sin, one cast to bf16)."""
    freqs = inv_freq(cfg)[None, :].float() * positions[:, None].float()
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos().to(torch.bfloat16), emb.sin().to(torch.bfloat16)


def _rms(x, w, eps):
    h = x.float()
    h = h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + eps)
    return w * h.to(torch.bfloat16)


def _rotate_half(x):
    d = x.shape[-1] // 2
    return torch.cat((-x[..., d:], x[..., :d]), dim=-1)


class OracleQwen3:
    """Greedy decoder over an HF-named bf16 state dict with a growing KV cache."""

    def __init__(self, cfg, state_dict, f32_twin=False):
        """f32_twin: evaluate the same graph with every projection and the attention computed on operands up-cast to
        f32 and the result rounded to bf16 once -- the same rounding points, another summation order.  The distance
        between the two evaluations is the noise floor a deep bf16 model has between any two correct implementations."""
        self.cfg, self.sd, self.f32_twin = cfg, state_dict, f32_twin
        self.k_cache = [None] * cfg.num_layers
        self.v_cache = [None] * cfg.num_layers
        self.pos = 0

    def reset(self):
        self.k_cache = [None] * self.cfg.num_layers
        self.v_cache = [None] * self.cfg.num_layers
        self.pos = 0

    def _linear(self, x, w):
        if self.f32_twin:
            return F.linear(x.float(), w.float()).to(torch.bfloat16)
        return F.linear(x, w)

    @torch.no_grad()
    def forward(self, ids, return_hidden=False):
        """ids int64 [B, s] appended at the current position -> logits bf16 [B, vocab] of the last position."""
        cfg, sd = self.cfg, self.sd
        B, s = ids.shape
        Hq, Hkv, D = cfg.num_q_heads, cfg.num_kv_heads, cfg.head_dim
        x = F.embedding(ids, sd["model.embed_tokens.weight"])
        positions = torch.arange(self.pos, self.pos + s)
        cos, sin = rope_tables(cfg, positions)
        cos, sin = cos[None, None], sin[None, None]
        L = self.pos + s
        mask = (torch.arange(L)[None, :] <= positions[:, None])[None, None]  # bool [1,1,s,L]
        for i in range(cfg.num_layers):
            p = f"model.layers.{i}."
            y = _rms(x, sd[p + "input_layernorm.weight"], cfg.eps)
            q = self._linear(y, sd[p + "self_attn.q_proj.weight"]).view(B, s, Hq, D)
            k = self._linear(y, sd[p + "self_attn.k_proj.weight"]).view(B, s, Hkv, D)
            v = self._linear(y, sd[p + "self_attn.v_proj.weight"]).view(B, s, Hkv, D).transpose(1, 2)
            q = _rms(q, sd[p + "self_attn.q_norm.weight"], cfg.eps).transpose(1, 2)
            k = _rms(k, sd[p + "self_attn.k_norm.weight"], cfg.eps).transpose(1, 2)
            q = q * cos + _rotate_half(q) * sin
            k = k * cos + _rotate_half(k) * sin
            if self.k_cache[i] is not None:
                k = torch.cat([self.k_cache[i], k], dim=-2)
                v = torch.cat([self.v_cache[i], v], dim=-2)
            self.k_cache[i], self.v_cache[i] = k, v
            g = Hq // Hkv
            ke = k[:, :, None].expand(B, Hkv, g, L, D).reshape(B, Hq, L, D)
            ve = v[:, :, None].expand(B, Hkv, g, L, D).reshape(B, Hq, L, D)
            if self.f32_twin:
                a = F.scaled_dot_product_attention(q.float(), ke.float(), ve.float(), attn_mask=mask, dropout_p=0.0,
                                                   scale=D ** -0.5, is_causal=False).to(torch.bfloat16)
            else:
                a = F.scaled_dot_product_attention(q, ke, ve, attn_mask=mask, dropout_p=0.0,
                                                   scale=D ** -0.5, is_causal=False)
            a = a.transpose(1, 2).reshape(B, s, Hq * D)
            x = x + self._linear(a, sd[p + "self_attn.o_proj.weight"])
            y = _rms(x, sd[p + "post_attention_layernorm.weight"], cfg.eps)
            m = F.silu(self._linear(y, sd[p + "mlp.gate_proj.weight"])) * self._linear(y, sd[p + "mlp.up_proj.weight"])
            x = x + self._linear(m, sd[p + "mlp.down_proj.weight"])
        self.pos = L
        self.last_residual = x  # bf16 [B, s, hidden]: the residual stream after the last layer (layer-level checks)
        h = _rms(x, sd["model.norm.weight"], cfg.eps)
        head = sd["model.embed_tokens.weight"] if cfg.tied else sd["lm_head.weight"]
        logits = self._linear(h[:, -1, :], head)
        return (logits, h) if return_hidden else logits

    @torch.no_grad()
    def generate(self, prompt_ids, steps, return_logits=False):
        """Greedy decode: returns int64 [B, steps] (and the bf16 logits of every step if asked)."""
        self.reset()
        logits = self.forward(prompt_ids)
        out, all_logits = [], []
        for _ in range(steps):
            nxt = torch.argmax(logits.float(), dim=-1)
            out.append(nxt)
            if return_logits:
                all_logits.append(logits)
            if len(out) == steps:
                break
            logits = self.forward(nxt[:, None])
        ids = torch.stack(out, dim=1)
        return (ids, torch.stack(all_logits, dim=1)) if return_logits else ids


def hf_model(cfg, state_dict):
    """The same weights inside ``transformers``' own Qwen3ForCausalLM (CPU, bf16, sdpa attention)."""
    from transformers import Qwen3Config, Qwen3ForCausalLM
    hc = Qwen3Config(vocab_size=cfg.vocab, hidden_size=cfg.hidden, intermediate_size=cfg.intermediate,
                     num_hidden_layers=cfg.num_layers, num_attention_heads=cfg.num_q_heads,
                     num_key_value_heads=cfg.num_kv_heads, head_dim=cfg.head_dim, rms_norm_eps=cfg.eps,
                     rope_theta=cfg.rope_theta, tie_word_embeddings=cfg.tied, max_position_embeddings=40960,
                     attention_bias=False, attn_implementation="sdpa", use_sliding_window=False,
                     layer_types=["full_attention"] * cfg.num_layers)
    if hasattr(hc, "rope_parameters") and isinstance(getattr(hc, "rope_parameters", None), dict):
        hc.rope_parameters["rope_theta"] = cfg.rope_theta
    with torch.device("meta"):
        m = Qwen3ForCausalLM(hc)
    m = m.to_empty(device="cpu").to(torch.bfloat16)
    sd = dict(state_dict)
    if cfg.tied:
        sd["lm_head.weight"] = sd["model.embed_tokens.weight"]
    missing = m.load_state_dict(sd, strict=False)
    assert not [k for k in missing.missing_keys if "inv_freq" not in k], missing
    # rotary inv_freq is a non-persistent buffer: re-create it (to_empty left it uninitialised)
    m.model.rotary_emb.inv_freq = inv_freq(cfg).clone()
    if hasattr(m.model.rotary_emb, "original_inv_freq"):
        m.model.rotary_emb.original_inv_freq = inv_freq(cfg).clone()
    if cfg.tied:
        m.tie_weights()
    return m.eval()
