"""Host side of the FP8 weight-only path: reading the checkpoints the reference's quantiser writes and arranging their
tensors the way the runner's fused, sharded weight slots want them.

The file layout is utilities/teeny-quant/src/format.rs:17-35 of the reference (compressed-tensors on plain
safetensors): a quantised ``foo.weight`` keeps its name and shape with dtype F8_E4M3, ``foo.weight_scale`` is a flat F32
vector with one scale per group, and the ``quantization_config`` JSON in the header's ``__metadata__`` names the scheme
(``config_groups.group_0.weights``: type, num_bits, strategy "tensor" | "channel" | "group", axis, group_size,
fp8_variant) and lists the tensors left alone (``ignore``: everything of rank < 2, format.rs:128-132).  Everything of
rank >= 2 is quantised, the embedding table too: it is converted back to bf16 when loaded (a lookup gains nothing from
bytes), the projections and the LM head stay FP8 on the device.
"""
import json
from dataclasses import dataclass

import torch

QUANTIZATION_CONFIG_KEY = "quantization_config"  # format.rs:116


@dataclass
class Fp8Scheme:
    strategy: str          # "tensor" | "channel" | "group"
    group_size: int = 0    # elements of k per scale ("group" only)


@dataclass
class IntScheme:
    """An integer scheme of the quantiser ("int-quantized" = 8 bits as I8, "pack-quantized" = 4 bits, two per byte):
    converted back to bf16 when loaded (teeny_dequant_int_bf16); there is no streaming integer GEMM."""
    bits: int
    symmetric: bool
    strategy: str
    group_size: int = 0
    packed_shapes: dict = None   # name -> logical shape of a nibble-packed tensor (format.rs:86-96)


def parse_quantization_config(metadata):
    """The scheme of a float-quantized checkpoint from its header metadata; raises ValueError for what the kernels do
    not take (integer schemes, E5M2, channel scales along the input axis, group sizes that are not multiples of 64)."""
    if QUANTIZATION_CONFIG_KEY not in metadata:
        raise ValueError("no quantization_config in the file's metadata")
    cfg = json.loads(metadata[QUANTIZATION_CONFIG_KEY])
    if cfg.get("quant_method") != "compressed-tensors" or cfg.get("format") not in (
            "float-quantized", "int-quantized", "pack-quantized"):
        raise ValueError(f"unsupported quantization format {cfg.get('quant_method')!r} / {cfg.get('format')!r}")
    groups = cfg.get("config_groups", {})
    if len(groups) != 1:
        raise ValueError("expected exactly one config group")
    w = next(iter(groups.values()))["weights"]
    if cfg["format"] != "float-quantized":
        bits = {"int-quantized": 8, "pack-quantized": 4}[cfg["format"]]
        if w.get("type") != "int" or w.get("num_bits") != bits:
            raise ValueError(f"{cfg['format']} expects {bits}-bit integer weights, got {w}")
        strategy = w.get("strategy")
        if strategy not in ("tensor", "channel", "group") or (strategy == "channel" and w.get("axis", 0) != 0) or (
                strategy == "group" and (w.get("axis", 1) != 1 or int(w.get("group_size") or 0) <= 0)):
            raise ValueError(f"unsupported integer granularity {w}")
        shapes = {k: tuple(v["logical_shape"]) for k, v in cfg.get("teenygrad_packed_int4", {}).items()}
        return IntScheme(bits, bool(w.get("symmetric", True)), strategy, int(w.get("group_size") or 0), shapes), cfg.get("ignore", [])
    if w.get("type") != "float" or w.get("num_bits") != 8 or w.get("fp8_variant", "e4m3") != "e4m3":
        raise ValueError(f"only FP8 E4M3 weights are supported, got {w}")
    strategy = w.get("strategy")
    if strategy == "tensor":
        return Fp8Scheme("tensor"), cfg.get("ignore", [])
    if strategy == "channel":
        if w.get("axis", 0) != 0:
            raise ValueError("channel scales must run along the output axis (axis 0)")
        return Fp8Scheme("channel"), cfg.get("ignore", [])
    if strategy == "group":
        g = int(w.get("group_size") or 0)
        if w.get("axis", 1) != 1 or g <= 0 or g % 64:
            raise ValueError("group scales must run along the input axis (axis 1) in multiples of 64")
        return Fp8Scheme("group", g), cfg.get("ignore", [])
    raise ValueError(f"unknown strategy {strategy!r}")


@dataclass
class Fp8Weight:
    """An FP8 matrix [N, K] (uint8 bytes) with its scales: [N] ("channel") or [N, ceil(K / group_size)] ("group").  A
    per-tensor scale is widened to per-channel on construction, so that rows of differently scaled tensors can be fused."""
    q: torch.Tensor
    scale: torch.Tensor
    group_size: int = 0

    @property
    def strategy(self):
        return "group" if self.group_size else "channel"

    @staticmethod
    def from_tensors(q, flat_scale, scheme):
        q = q.view(torch.uint8) if q.dtype != torch.uint8 else q
        N, K = q.shape
        s = flat_scale.to(torch.float32).flatten()
        if scheme.strategy == "tensor":
            return Fp8Weight(q, s.expand(N).contiguous())
        if scheme.strategy == "channel":
            if s.numel() != N:
                raise ValueError(f"expected {N} channel scales, got {s.numel()}")
            return Fp8Weight(q, s.contiguous())
        per_row = -(-K // scheme.group_size)
        if s.numel() != N * per_row:
            raise ValueError(f"expected {N * per_row} group scales, got {s.numel()}")
        return Fp8Weight(q, s.view(N, per_row).contiguous(), scheme.group_size)

    def rows(self, a, b):
        return Fp8Weight(self.q[a:b].contiguous(), self.scale[a:b].contiguous(), self.group_size)

    def cols(self, a, b):
        """Columns [a, b) (a row-parallel shard): channel scales stay whole, group scales follow the columns."""
        if not self.group_size:
            return Fp8Weight(self.q[:, a:b].contiguous(), self.scale, 0)
        if a % self.group_size or (b % self.group_size and b != self.q.shape[1]):
            raise ValueError("a column shard must start and end on a scale group")
        g = self.group_size
        return Fp8Weight(self.q[:, a:b].contiguous(), self.scale[:, a // g:-(-b // g)].contiguous(), g)

    @staticmethod
    def cat_rows(parts):
        return Fp8Weight(torch.cat([p.q for p in parts]).contiguous(), torch.cat([p.scale for p in parts]).contiguous(),
                         parts[0].group_size)

    @staticmethod
    def interleave(gate, up):
        """The fused SwiGLU row order (64 gate rows, then the 64 up rows of the same channels), bytes and scales alike."""
        def il(a, b):
            n = a.shape[0]
            if n % 64:
                raise ValueError("intermediate size must be a multiple of 64")
            a2, b2 = a.reshape(n // 64, 64, -1), b.reshape(n // 64, 64, -1)
            return torch.stack([a2, b2], dim=1).reshape(2 * n, -1)
        q = il(gate.q, up.q).contiguous()
        s = il(gate.scale, up.scale)
        return Fp8Weight(q, (s if gate.group_size else s.flatten()).contiguous(), gate.group_size)

    def to(self, device):
        return Fp8Weight(self.q.to(device), self.scale.to(device), self.group_size)

    def dequantize(self):
        """float32 [N, K] on the tensors' device (decode * scale), for checks."""
        w = self.q.view(torch.float8_e4m3fn).float()
        if not self.group_size:
            return w * self.scale[:, None]
        return w * self.scale.repeat_interleave(self.group_size, dim=1)[:, :w.shape[1]]


def dequantize_int_state_dict(tensors, scheme, device):
    """bf16 state dict (on ``device``) of an integer-quantised checkpoint: every ``name`` that has a ``name_scale``
    beside it is converted by the library's kernel, the rest is passed through as bf16."""
    from . import ops
    out = {}
    for name in tensors:
        if name.endswith("_scale") or name.endswith("_zero_point"):
            continue
        t = tensors[name]
        if name + "_scale" not in tensors:
            out[name] = t.to(device).to(torch.bfloat16)
            continue
        shape = scheme.packed_shapes.get(name) if scheme.bits == 4 else tuple(t.shape)
        if shape is None or len(shape) < 2:
            raise ValueError(f"{name}: no logical shape for a packed 4-bit tensor")
        N, K = shape[0], int(torch.tensor(shape[1:]).prod())
        zp = tensors.get(name + "_zero_point") if (name + "_zero_point") in tensors else None
        w = ops.dequant_int(t.to(device), scheme.bits, tensors[name + "_scale"].to(device).float(),
                            None if zp is None else zp.to(device).to(torch.int32), (N, K), scheme.strategy, scheme.group_size)
        out[name] = w.view(*shape)
    return out


def quantize_fp8(w, strategy="channel", group_size=0):
    """FP8 form of a float matrix with PyTorch's cast (round to nearest even; scale = amax / 448 per group, 1 for an
    all-zero group, as utilities/teeny-quant/src/quant/fp8.rs:237-246).  For benchmarks and demos on random weights: it
    differs from the reference's encoder below the smallest normal (results there are kept as subnormals, the reference
    flushes them to zero)."""
    w = w.float()
    N, K = w.shape
    if strategy == "tensor":
        amax = w.abs().amax().expand(N)
    elif strategy == "channel":
        amax = w.abs().amax(dim=1)
    else:
        pad = -K % group_size
        amax = torch.nn.functional.pad(w.abs(), (0, pad)).view(N, -1, group_size).amax(dim=2)
    scale = torch.where(amax == 0, torch.ones_like(amax), amax / 448.0).float()
    full = scale[:, None] if scale.dim() == 1 else scale.repeat_interleave(group_size, dim=1)[:, :K]
    q = (w / full).to(torch.float8_e4m3fn).view(torch.uint8)
    return Fp8Weight(q.contiguous(), scale.contiguous(), group_size if strategy == "group" else 0)


def shard_layer_fp8(get, cfg, layer, rank, tp):
    """Fused, sharded FP8 projections of one layer; ``get(name)`` returns the Fp8Weight of an HF-named tensor."""
    p = f"model.layers.{layer}."
    D = cfg.head_dim
    hq, hkv, il = cfg.num_q_heads // tp * D, cfg.num_kv_heads // tp * D, cfg.intermediate // tp
    q = get(p + "self_attn.q_proj.weight").rows(rank * hq, (rank + 1) * hq)
    k = get(p + "self_attn.k_proj.weight").rows(rank * hkv, (rank + 1) * hkv)
    v = get(p + "self_attn.v_proj.weight").rows(rank * hkv, (rank + 1) * hkv)
    gate = get(p + "mlp.gate_proj.weight").rows(rank * il, (rank + 1) * il)
    up = get(p + "mlp.up_proj.weight").rows(rank * il, (rank + 1) * il)
    return {
        "qkv": Fp8Weight.cat_rows([q, k, v]),
        "o": get(p + "self_attn.o_proj.weight").cols(rank * hq, (rank + 1) * hq),
        "gate_up": Fp8Weight.interleave(gate, up),
        "down": get(p + "mlp.down_proj.weight").cols(rank * il, (rank + 1) * il),
    }


def quantize_state_dict(sd, strategy="channel", group_size=0):
    """What the reference's quantiser does to a checkpoint (format.rs:128-132, 145-246), with ``quantize_fp8``'s
    encoder: every tensor of rank >= 2 becomes FP8 bytes plus ``<name>_scale``; the rest passes through and is listed
    under ``ignore``.  Returns (tensors, metadata) ready for ``safetensors.save_file``."""
    out, ignore = {}, []
    for name, t in sd.items():
        if t.dim() >= 2 and t.is_floating_point():
            w = quantize_fp8(t.reshape(t.shape[0], -1), strategy, group_size)
            scale = w.scale if strategy != "tensor" else w.scale[:1]
            out[name] = w.q.view(torch.float8_e4m3fn).reshape(t.shape)
            out[name + "_scale"] = scale.flatten().contiguous()
        else:
            out[name] = t
            ignore.append(name)
    weights = {"num_bits": 8, "type": "float", "symmetric": True, "strategy": strategy, "fp8_variant": "e4m3"}
    if strategy == "channel":
        weights["axis"] = 0
    if strategy == "group":
        weights["axis"], weights["group_size"] = 1, group_size
    cfg = {"quant_method": "compressed-tensors", "format": "float-quantized",
           "config_groups": {"group_0": {"weights": weights, "targets": ["*"]}}, "ignore": sorted(ignore)}
    return out, {QUANTIZATION_CONFIG_KEY: json.dumps(cfg)}
