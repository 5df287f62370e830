"""Tensor-parallel host logic: Megatron-style weight sharding for Qwen3 and NCCL communicator set-up.

Sharding (tp ranks, rank r):
  column-parallel  q_proj (Hq/tp heads), k_proj / v_proj (Hkv/tp heads), gate_proj / up_proj (I/tp rows, interleaved
                   in blocks of 64 channels for the fused SwiGLU GEMM)
  row-parallel     o_proj (columns of the local q heads), down_proj (columns of the local intermediate slice)
  replicated       norms, embedding;  vocabulary-parallel LM head (vocab/tp rows)
A rank's q heads [r*Hq/tp, (r+1)*Hq/tp) use exactly its kv heads [r*Hkv/tp, (r+1)*Hkv/tp), so attention is local.
The pure-tensor functions here run on CPU tensors too (they are covered by gloo world-size-2 tests).
"""
import ctypes as C

import torch


def check_divisible(cfg, tp):
    for name, v in (("num_kv_heads", cfg.num_kv_heads), ("intermediate", cfg.intermediate), ("vocab", cfg.vocab)):
        if v % tp:
            raise ValueError(f"{name}={v} is not divisible by tp={tp}")


def interleave_gate_up(gate, up):
    """[2I, K] weight of the fused SwiGLU GEMM: blocks of 64 gate rows, each followed by the 64 up rows of the same
    channels, so one 128-row weight tile holds both projections of 64 channels."""
    inter, k = gate.shape
    if inter % 64:
        raise ValueError(f"intermediate shard {inter} is not a multiple of 64")
    return torch.stack([gate.reshape(inter // 64, 64, k), up.reshape(inter // 64, 64, k)], dim=1).reshape(2 * inter, k).contiguous()


def shard_layer(sd, cfg, layer, rank, tp):
    """Fused, sharded weights of one layer from an HF-named state dict (full tensors)."""
    check_divisible(cfg, tp)
    p = f"model.layers.{layer}."
    D = cfg.head_dim
    hq, hkv, il = cfg.num_q_heads // tp * D, cfg.num_kv_heads // tp * D, cfg.intermediate // tp
    q = sd[p + "self_attn.q_proj.weight"][rank * hq:(rank + 1) * hq]
    k = sd[p + "self_attn.k_proj.weight"][rank * hkv:(rank + 1) * hkv]
    v = sd[p + "self_attn.v_proj.weight"][rank * hkv:(rank + 1) * hkv]
    gate = sd[p + "mlp.gate_proj.weight"][rank * il:(rank + 1) * il]
    up = sd[p + "mlp.up_proj.weight"][rank * il:(rank + 1) * il]
    return {
        "qkv": torch.cat([q, k, v], dim=0).contiguous(),
        "o": sd[p + "self_attn.o_proj.weight"][:, rank * hq:(rank + 1) * hq].contiguous(),
        "gate_up": interleave_gate_up(gate, up),
        "down": sd[p + "mlp.down_proj.weight"][:, rank * il:(rank + 1) * il].contiguous(),
        "input_ln": sd[p + "input_layernorm.weight"].contiguous(),
        "post_ln": sd[p + "post_attention_layernorm.weight"].contiguous(),
        "q_norm": sd[p + "self_attn.q_norm.weight"].contiguous(),
        "k_norm": sd[p + "self_attn.k_norm.weight"].contiguous(),
    }


def shard_head(sd, cfg, rank, tp):
    check_divisible(cfg, tp)
    vl = cfg.vocab // tp
    head = sd["model.embed_tokens.weight"] if cfg.tied else sd["lm_head.weight"]
    return {
        "embed": sd["model.embed_tokens.weight"].contiguous(),
        "final_norm": sd["model.norm.weight"].contiguous(),
        "lm_head": head[rank * vl:(rank + 1) * vl].contiguous(),
    }


def merge_argmax(vals, idx):
    """Host restatement of the cross-rank greedy pick: vals/idx [parts, rows] -> winning index per row
    (largest value, lowest index on ties).  Used by the CPU tests of the vocabulary-parallel head."""
    best_v, best_i = vals[0].clone(), idx[0].clone()
    for p in range(1, vals.shape[0]):
        take = (vals[p] > best_v) | ((vals[p] == best_v) & (idx[p] < best_i))
        best_v = torch.where(take, vals[p], best_v)
        best_i = torch.where(take, idx[p], best_i)
    return best_i


def init_comm(rank, world, group=None):
    """NCCL communicator for the runner: rank 0 creates the unique id, torch.distributed ships it."""
    import torch.distributed as dist
    from ._lib import check
    from .qwen3 import lib
    buf = (C.c_ubyte * 128)()
    if rank == 0:
        check(lib.teeny_tp_unique_id(buf), "teeny_tp_unique_id")
    backend = dist.get_backend(group)
    t = torch.tensor(list(buf), dtype=torch.uint8, device="cuda" if backend == "nccl" else "cpu")
    dist.broadcast(t, src=0, group=group)
    raw = bytes(t.cpu().tolist())
    comm = C.c_void_p()
    check(lib.teeny_tp_init(raw, rank, world, C.byref(comm)), "teeny_tp_init")
    return comm
