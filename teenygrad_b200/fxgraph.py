"""Reader for the traced-graph files of the reference's PyTorch front end, and their lowering onto this backend's
Qwen3 runner.

The reference records a ``torch.fx`` graph as a FlatBuffers ``Graph`` table (schema ``support/teeny-torch/graph.fbs``:
``Graph{nodes:[NodeWrapper], example_inputs}``, node union ``placeholder | call_function | call_method | call_module |
get_attr | output``, argument union ``Value``) compressed with gzip (``support/teeny-torch/tests/data/*.bin.gz``), and
its Rust side turns the nodes into the ``FxGraphLang`` vocabulary (``support/teeny-fxgraph/src/fxgraph/lang.rs:29-83``).
This module reads the same files without a FlatBuffers library (root offset -> vtable -> field offsets), maps each
node's target onto that vocabulary (``op_of``), and ``lower_qwen3`` pattern-matches a Qwen3 trace into the fused
kernel sequence the runner executes, deriving the model configuration from the example inputs on the way.
"""
import gzip
import re
import struct
from dataclasses import dataclass, field

DTYPES = ["float32", "float64", "int32", "int64", "uint8", "int8", "bool", "bfloat16", "float16"]  # enum DType
_NODE_KINDS = [None, "placeholder", "call_function", "call_method", "call_module", "get_attr", "output"]  # union Node
_VALUE_KINDS = [None, "none", "int", "str", "node", "device", "dtype", "ellipsis", "tuple", "list", "slice"]  # union Value


@dataclass(frozen=True)
class NodeRef:
    """An argument that names another node of the graph (``ValNode``)."""
    name: str


@dataclass
class FxNode:
    kind: str
    name: str
    target: str = ""
    args: list = field(default_factory=list)
    kwargs: dict = field(default_factory=dict)
    users: list = field(default_factory=list)


@dataclass
class ExampleTensor:
    dtype: str
    shape: tuple        # ints, or strings for symbolic dimensions
    stride: tuple
    device: str = ""


@dataclass
class FxGraph:
    nodes: list
    example_inputs: list  # ExampleTensor, or a str for a symbolic integer input


class _Buf:
    """Just enough of the FlatBuffers wire format: tables (vtable-indexed fields), strings, vectors, unions."""

    def __init__(self, data):
        self.d = data

    def u8(self, o): return self.d[o]
    def i8(self, o): return struct.unpack_from("<b", self.d, o)[0]
    def u16(self, o): return struct.unpack_from("<H", self.d, o)[0]
    def i32(self, o): return struct.unpack_from("<i", self.d, o)[0]
    def u32(self, o): return struct.unpack_from("<I", self.d, o)[0]

    def indirect(self, o):
        return o + self.u32(o)

    def field(self, table, index):
        """Absolute offset of field `index` inside `table`, or 0 when the field is absent (default value)."""
        vt = table - self.i32(table)
        slot = 4 + 2 * index
        if slot >= self.u16(vt):
            return 0
        off = self.u16(vt + slot)
        return table + off if off else 0

    def string(self, table, index, default=""):
        f = self.field(table, index)
        if not f:
            return default
        s = self.indirect(f)
        n = self.u32(s)
        return self.d[s + 4:s + 4 + n].decode("utf-8")

    def table(self, table, index):
        f = self.field(table, index)
        return self.indirect(f) if f else 0

    def vector(self, table, index):
        """(offset of element 0, length) of a vector field; (0, 0) when absent."""
        f = self.field(table, index)
        if not f:
            return 0, 0
        v = self.indirect(f)
        return v + 4, self.u32(v)

    def table_vector(self, table, index):
        start, n = self.vector(table, index)
        return [self.indirect(start + 4 * i) for i in range(n)]

    def string_vector(self, table, index):
        start, n = self.vector(table, index)
        out = []
        for i in range(n):
            s = self.indirect(start + 4 * i)
            out.append(self.d[s + 4:s + 4 + self.u32(s)].decode("utf-8"))
        return out


def _value(b, wrapper):
    """Decode a ValueWrapper table (fields: value_type u8, value union) into a Python value."""
    if not wrapper:
        return None
    tf = b.field(wrapper, 0)
    kind = _VALUE_KINDS[b.u8(tf)] if tf else None
    t = b.table(wrapper, 1)
    if kind is None or kind == "none":
        return None
    if kind == "int":
        f = b.field(t, 0)
        return b.i32(f) if f else 0
    if kind == "str":
        return b.string(t, 0)
    if kind == "node":
        return NodeRef(b.string(t, 0))
    if kind == "device":
        return ("device", b.string(t, 0))
    if kind == "dtype":
        f = b.field(t, 0)
        return ("dtype", DTYPES[b.i8(f)] if f else DTYPES[0])
    if kind == "ellipsis":
        return Ellipsis
    if kind == "tuple":
        return tuple(_value(b, w) for w in b.table_vector(t, 0))
    if kind == "list":
        return [_value(b, w) for w in b.table_vector(t, 0)]
    if kind == "slice":
        return slice(_value(b, b.table(t, 0)), _value(b, b.table(t, 1)), _value(b, b.table(t, 2)))
    raise ValueError(f"unknown Value kind {kind}")


def _kwargs(b, table, index):
    return {b.string(kv, 0): _value(b, b.table(kv, 1)) for kv in b.table_vector(table, index)}


def parse_graph(data):
    """FlatBuffers bytes of a ``Graph`` -> FxGraph."""
    b = _Buf(data)
    root = b.indirect(0)
    nodes = []
    for w in b.table_vector(root, 0):
        tf = b.field(w, 0)
        kind = _NODE_KINDS[b.u8(tf)] if tf else None
        t = b.table(w, 1)
        if kind is None:
            raise ValueError("node without a type")
        if kind == "placeholder":
            nodes.append(FxNode(kind, b.string(t, 0), b.string(t, 1), users=b.string_vector(t, 2)))
        elif kind in ("call_function", "call_method", "output"):
            nodes.append(FxNode(kind, b.string(t, 0), b.string(t, 1), [_value(b, a) for a in b.table_vector(t, 2)],
                                _kwargs(b, t, 3), b.string_vector(t, 4)))
        else:  # call_module, get_attr: name only
            nodes.append(FxNode(kind, b.string(t, 0)))
    inputs = []
    ex = b.table(root, 1)
    if ex:
        for w in b.table_vector(ex, 0):
            tf = b.field(w, 0)
            which = b.u8(tf) if tf else 0
            t = b.table(w, 1)
            if which == 1:      # SymInt
                inputs.append(b.string(t, 0))
            elif which == 2:    # Tensor
                df = b.field(t, 0)
                shape_t = b.table(t, 2)
                dims = []
                for d in (b.table_vector(shape_t, 0) if shape_t else []):
                    s = b.string(d, 0)
                    dims.append(int(s) if re.fullmatch(r"-?\d+", s) else s)
                start, n = b.vector(t, 3)
                inputs.append(ExampleTensor(DTYPES[b.i8(df)] if df else DTYPES[0], tuple(dims),
                                            tuple(b.u32(start + 4 * i) for i in range(n)), b.string(t, 1)))
            else:
                inputs.append(None)
    return FxGraph(nodes, inputs)


def read_graph(path):
    with gzip.open(path, "rb") as f:
        return parse_graph(f.read())


# ---------------------------------------------------------------------------------------------------------------
# FxGraphLang vocabulary (support/teeny-fxgraph/src/fxgraph/lang.rs:29-83)
# ---------------------------------------------------------------------------------------------------------------
LANG_OPS = ("output", "add", "list", "args", "item", "getitem", "embedding", "arange", "iadd",
            "lazy_load_decompositions", "contiguous", "enter_autocast", "exit_autocast", "silu", "rsqrt", "linear",
            "sym_sum", "vmap_increment_nesting", "vmap_decrement_nesting", "add_batch_dim", "remove_batch_dim",
            "aten.index", "cat", "sdpa", "-", "*", "/", "@", "neg", "to", "new_ones", "le", "and", "float", "expand",
            "transpose", "cos", "sin", "pow", "mean", "view", "unsqueeze", "reshape", "numel")
# torch.fx prints call_function targets as "<built-in function mul>", "<function silu at 0x...>", "<built-in method
# rsqrt of type object at 0x...>", "aten.index"; the word after function / method is what names the operation
_FUNCTION_WORDS = {"mul": "*", "sub": "-", "truediv": "/", "matmul": "@", "scaled_dot_product_attention": "sdpa",
                   "_vmap_increment_nesting": "vmap_increment_nesting", "_vmap_decrement_nesting": "vmap_decrement_nesting",
                   "_add_batch_dim": "add_batch_dim", "_remove_batch_dim": "remove_batch_dim",
                   "_enter_autocast": "enter_autocast", "_exit_autocast": "exit_autocast", "__and__": "and"}
_NO_OPS = {"_log_api_usage_once"}  # the reference drops these too (support/teeny-torch/src/graph/call_function.rs:219-228)


def op_of(node):
    """The FxGraphLang operation a node maps to, "placeholder" / "output" for those kinds, None for nodes the reference
    drops; raises on a target outside the vocabulary."""
    if node.kind in ("placeholder", "output"):
        return node.kind
    t = node.target
    m = re.match(r"<(?:built-in )?(?:function|method) ([^\s>]+)", t)
    word = m.group(1) if m else t
    if word in _NO_OPS:
        return None
    op = _FUNCTION_WORDS.get(word, word)
    if op not in LANG_OPS:
        raise ValueError(f"node {node.name}: target {t!r} is outside the FxGraphLang vocabulary")
    return op


# ---------------------------------------------------------------------------------------------------------------
# Lowering of a Qwen3 trace onto the runner's kernels
# ---------------------------------------------------------------------------------------------------------------
# The kernels one decoder layer costs in the runner (csrc/qwen3_runner.cu, run_layers), in launch order, with the
# traced operations each one covers.  In decode the third and fourth are one launch (the attention kernel norms and
# rotates its own heads and appends to the cache on the way in).
DECODER_LAYER_KERNELS = (
    ("add_rms_norm", "residual add of the previous block (absent in layer 0) + input_layernorm"),
    ("qkv_gemm", "q_proj, k_proj, v_proj as one GEMM over the fused [q; k; v] weight rows"),
    ("head_norm_rope_kv", "q_norm, k_norm over head_dim, rotary embedding of q and k, KV-cache append"),
    ("attention", "GQA expand / reshape + scaled_dot_product_attention under the causal mask"),
    ("o_gemm", "o_proj"),
    ("add_rms_norm", "residual add + post_attention_layernorm"),
    ("gate_up_swiglu_gemm", "gate_proj, up_proj, silu, mul as one GEMM with the activation in its epilogue"),
    ("down_gemm", "down_proj"),
)
HEAD_KERNELS = (("add_rms_norm", "last residual add + final norm"), ("lm_head_gemm", "logits of the kept positions"))


@dataclass
class Kernel:
    """One launch of the plan: the runner kernel, the traced nodes it stands for and what it reads."""
    kind: str
    layer: int                      # -1 for model-level kernels
    nodes: list                     # indices into FxGraph.nodes
    weights: dict = field(default_factory=dict)   # role -> placeholder name
    attrs: dict = field(default_factory=dict)


@dataclass
class Qwen3Plan:
    config: dict                    # num_layers, hidden, num_q_heads, num_kv_heads, head_dim, intermediate, vocab, eps, tied
    kernels: list                   # Kernel, in launch order
    bookkeeping: list               # node indices with no device work: mask construction, scalar reads, layout-only views
    has_kv_cache_inputs: bool       # a decode-step trace (past keys / values come in as inputs)

    def layer_kinds(self, layer):
        return [k.kind for k in self.kernels if k.layer == layer]


class LoweringError(ValueError):
    pass


def hf_name(placeholder):
    """``l_self_modules_model_modules_layers_modules_3_modules_self_attn_modules_q_proj_parameters_weight_`` ->
    ``model.layers.3.self_attn.q_proj.weight`` (the state-dict key the weight loader uses)."""
    s = placeholder
    s = re.sub(r"^l_self_modules_", "", s, flags=re.I)
    s = re.sub(r"_parameters_weight_$", ".weight", s)
    s = re.sub(r"_buffers_inv_freq_$", ".inv_freq", s)
    s = s.replace("_modules_", ".")
    return s


class _Matcher:
    def __init__(self, graph):
        self.g = graph
        self.nodes = graph.nodes
        self.index = {n.name: i for i, n in enumerate(graph.nodes)}
        self.ops = [op_of(n) for n in graph.nodes]
        self.used = {}
        self.example = {}
        ph = [n for n in graph.nodes if n.kind == "placeholder"]
        for n, e in zip(ph, graph.example_inputs):
            self.example[n.name] = e

    def node(self, ref):
        if not isinstance(ref, NodeRef):
            raise LoweringError(f"expected a node argument, got {ref!r}")
        return self.index[ref.name]

    def arg(self, i, k):
        return self.node(self.nodes[i].args[k])

    def expect(self, i, op):
        if self.ops[i] != op:
            raise LoweringError(f"node {i} ({self.nodes[i].name}) is {self.ops[i]!r}, expected {op!r}")
        return i

    def is_placeholder(self, i):
        return self.nodes[i].kind == "placeholder"

    def dtype_of_to(self, i):
        n = self.nodes[i]
        for a in list(n.args[1:]) + list(n.kwargs.values()):
            if isinstance(a, tuple) and len(a) == 2 and a[0] == "dtype":
                return a[1]
        return None

    # ---- patterns; each returns (node indices, attributes) and reads backwards from the pattern's last node ----
    def rms_norm(self, out):
        """weight * (x.float() * rsqrt(mean(x.float()^2, -1) + eps)).to(bf16): returns nodes, input, weight, eps."""
        self.expect(out, "*")
        a, b = self.arg(out, 0), self.arg(out, 1)
        w, cast = (a, b) if self.is_placeholder(a) else (b, a)
        if not self.is_placeholder(w):
            raise LoweringError(f"node {out}: RMSNorm weight multiply without a weight placeholder")
        self.expect(cast, "to")
        if self.dtype_of_to(cast) != "bfloat16":
            raise LoweringError(f"node {cast}: the normalised row must be cast to bfloat16 before the weight multiply")
        scaled = self.expect(self.arg(cast, 0), "*")
        up, rs = self.arg(scaled, 0), self.arg(scaled, 1)
        self.expect(rs, "rsqrt")
        self.expect(up, "to")
        if self.dtype_of_to(up) != "float32":
            raise LoweringError(f"node {up}: RMSNorm statistics must be computed in float32")
        add = self.expect(self.arg(rs, 0), "add")
        mean = self.expect(self.arg(add, 0), "mean")
        eps_item = self.expect(self.arg(add, 1), "item")
        pw = self.expect(self.arg(mean, 0), "pow")
        if self.arg(pw, 0) != up or self.nodes[pw].args[1] != 2 or self.nodes[mean].args[1] != -1:
            raise LoweringError(f"node {out}: not mean(x^2) over the last dimension")
        eps_ph = self.arg(eps_item, 0)
        return ([up, pw, mean, eps_item, add, rs, scaled, cast, out],
                dict(input=self.arg(up, 0), weight=self.nodes[w].name, eps=self.nodes[eps_ph].name))

    def rope(self, out):
        """x * cos + cat(-x[..., 64:], x[..., :64]) * sin on bf16 tensors: returns nodes, x, cos, sin."""
        self.expect(out, "add")
        m1, m2 = self.expect(self.arg(out, 0), "*"), self.expect(self.arg(out, 1), "*")
        x, cos = self.arg(m1, 0), self.arg(m1, 1)
        cat, sin = self.expect(self.arg(m2, 0), "cat"), self.arg(m2, 1)
        parts = self.nodes[cat].args[0]
        neg = self.expect(self.node(parts[0]), "neg")
        x1 = self.expect(self.node(parts[1]), "getitem")
        x2 = self.expect(self.arg(neg, 0), "getitem")
        if self.arg(x1, 0) != x or self.arg(x2, 0) != x:
            raise LoweringError(f"node {out}: rotate_half does not rotate the tensor that is multiplied by cos")
        h1, h2 = self.nodes[x1].args[1][-1], self.nodes[x2].args[1][-1]
        if not (isinstance(h1, slice) and isinstance(h2, slice) and h1.stop == h2.start and h1.start is None and h2.stop is None):
            raise LoweringError(f"node {out}: rotate_half halves are not [..., :d/2] and [..., d/2:]")
        return [m1, x1, x2, neg, cat, m2, out], dict(x=x, cos=cos, sin=sin, half=h1.stop)

    def through(self, i, ops):
        """Walk back through layout-only nodes (given ops), collecting them."""
        seen = []
        while self.ops[i] in ops:
            seen.append(i)
            i = self.arg(i, 0)
        return i, seen


def lower_qwen3(graph):
    """Pattern-match a traced Qwen3 forward (prefill or decode step) into the runner's kernel sequence.

    Raises LoweringError when the trace departs from what the kernels implement (a cast point elsewhere, a different
    rotation, a non-causal mask argument, biases, ...).  Every device-work node ends up in exactly one kernel."""
    m = _Matcher(graph)
    N = m.nodes
    kernels, book = [], []
    linears = [i for i, op in enumerate(m.ops) if op == "linear"]
    sdpas = [i for i, op in enumerate(m.ops) if op == "sdpa"]
    n_layers = len(sdpas)
    if n_layers == 0 or len(linears) != 7 * n_layers + 1:
        raise LoweringError(f"{len(linears)} linear and {len(sdpas)} attention nodes: not a Qwen3 decoder trace")
    for i in linears:
        if N[i].args[2] is not None:
            raise LoweringError(f"node {i}: linear with a bias; the Qwen3 projections have none")
    emb = [i for i, op in enumerate(m.ops) if op == "embedding"]
    if len(emb) != 1:
        raise LoweringError("expected exactly one embedding node")
    emb = emb[0]
    embed_w = N[m.arg(emb, 1)].name
    kernels.append(Kernel("embedding", -1, [emb], dict(table=embed_w)))

    # rotary tables: inv_freq @ positions in float32, cos / sin, * attention_scaling, cast to bfloat16
    mm = [i for i, op in enumerate(m.ops) if op == "@"]
    cos_n = [i for i, op in enumerate(m.ops) if op == "cos"]
    sin_n = [i for i, op in enumerate(m.ops) if op == "sin"]
    if len(mm) != 1 or len(cos_n) != 1 or len(sin_n) != 1:
        raise LoweringError("expected one rotary-table construction (matmul, cos, sin)")
    emb_cat = m.expect(m.arg(cos_n[0], 0), "cat")       # emb = cat(freqs, freqs)
    if m.arg(sin_n[0], 0) != emb_cat:
        raise LoweringError("cos and sin are taken of different angle tensors")
    freqs, seen = m.through(m.node(N[emb_cat].args[0][0]), ("transpose",))
    if freqs != mm[0] or m.node(N[emb_cat].args[0][1]) != seen[0]:
        raise LoweringError("rotary angles are not cat(freqs, freqs) of inv_freq @ positions")
    table_nodes, table_casts = [mm[0], seen[0], emb_cat, cos_n[0], sin_n[0]], {}
    for fn in (cos_n[0], sin_n[0]):
        scaled = [m.index[u] for u in N[fn].users]
        if len(scaled) != 1 or m.ops[scaled[0]] != "*":
            raise LoweringError("cos / sin must be scaled by attention_scaling")
        cast = [m.index[u] for u in N[scaled[0]].users]
        if len(cast) != 1 or m.ops[cast[0]] != "to" or m.dtype_of_to(cast[0]) != "bfloat16":
            raise LoweringError("the rotary tables must be cast to bfloat16 before they are applied")
        table_nodes += [scaled[0], cast[0]]
        table_casts[m.ops[fn]] = cast[0]
    inv_freq = [n.name for n in N if n.kind == "placeholder" and n.name.endswith("inv_freq_")]
    kernels.append(Kernel("rope_table", -1, sorted(table_nodes), dict(inv_freq=inv_freq[0] if inv_freq else ""),
                          dict(table_dtype="bfloat16", angle_dtype="float32")))

    cfg = {}
    residual = emb   # node holding the residual stream entering the next block
    pending_add = None
    for layer in range(n_layers):
        lq, lk, lv, lo, lg, lu, ld = linears[7 * layer:7 * layer + 7]
        sd = sdpas[layer]
        # input norm
        norm_nodes, na = m.rms_norm(m.arg(lq, 0))
        if m.arg(lk, 0) != m.arg(lq, 0) or m.arg(lv, 0) != m.arg(lq, 0):
            raise LoweringError(f"layer {layer}: q, k, v projections do not share one input")
        if na["input"] != residual:
            raise LoweringError(f"layer {layer}: input_layernorm does not read the residual stream")
        kernels.append(Kernel("add_rms_norm", layer, ([pending_add] if pending_add is not None else []) + norm_nodes,
                              dict(weight=na["weight"], eps=na["eps"]),
                              dict(fused_add=pending_add is not None, stats_dtype="float32", cast_before_weight="bfloat16")))
        kernels.append(Kernel("qkv_gemm", layer, [lq, lk, lv],
                              dict(q=N[m.arg(lq, 1)].name, k=N[m.arg(lk, 1)].name, v=N[m.arg(lv, 1)].name)))
        # attention inputs, walking back from the sdpa node
        hn = []
        q_in, seen = m.through(m.arg(sd, 0), ("contiguous",)); hn += seen
        rq_nodes, rq = m.rope(q_in); hn += rq_nodes
        qt, seen = m.through(rq["x"], ("transpose",)); hn += seen
        qn_nodes, qn = m.rms_norm(qt); hn += qn_nodes
        qv, seen = m.through(qn["input"], ("view",)); hn += seen
        if qv != lq:
            raise LoweringError(f"layer {layer}: q_norm does not read q_proj")
        head_dim = N[seen[0]].args[1][-1] if seen else None

        def kv_side(arg_index, roped):
            nodes = []
            x, seen = m.through(m.arg(sd, arg_index), ("contiguous",)); nodes += seen
            attn_nodes = []
            x = m.expect(x, "reshape"); attn_nodes.append(x)
            heads_q = N[x].args[2]
            x = m.expect(m.arg(x, 0), "expand"); attn_nodes.append(x)
            heads_kv, group = N[x].args[2], N[x].args[3]
            x = m.expect(m.arg(x, 0), "getitem"); attn_nodes.append(x)
            x = m.arg(x, 0)
            cache_in = None
            if m.ops[x] == "cat" and N[x].kwargs.get("dim") == -2:   # decode: cat([past, new], dim=-2)
                parts = N[x].args[0]
                cache_in = N[m.node(parts[0])].name
                nodes.append(x)
                x = m.node(parts[1])
            if roped:
                r_nodes, r = m.rope(x); nodes += r_nodes
                t, seen = m.through(r["x"], ("transpose",)); nodes += seen
                n_nodes, n_attr = m.rms_norm(t); nodes += n_nodes
                v0, seen = m.through(n_attr["input"], ("view",)); nodes += seen
                return nodes, attn_nodes, v0, dict(heads_q=heads_q, heads_kv=heads_kv, group=group, cache=cache_in,
                                                   norm=n_attr, rope=r)
            t, seen = m.through(x, ("transpose", "view")); nodes += seen
            return nodes, attn_nodes, t, dict(heads_q=heads_q, heads_kv=heads_kv, group=group, cache=cache_in)

        k_nodes, k_attn, k_src, ka = kv_side(1, True)
        v_nodes, v_attn, v_src, va = kv_side(2, False)
        if k_src != lk or v_src != lv:
            raise LoweringError(f"layer {layer}: key / value paths do not start at k_proj / v_proj")
        if rq["cos"] != ka["rope"]["cos"] or rq["sin"] != ka["rope"]["sin"]:
            raise LoweringError(f"layer {layer}: q and k are rotated with different tables")
        for tab, which in ((rq["cos"], "cos"), (rq["sin"], "sin")):
            src, seen = m.through(tab, ("unsqueeze",))
            if src != table_casts[which]:
                raise LoweringError(f"layer {layer}: rotary {which} is not the bfloat16 table")
            book += [s for s in seen if s not in book]
        kernels.append(Kernel("head_norm_rope_kv", layer, sorted(set(hn + k_nodes + v_nodes)),
                              dict(q_norm=qn["weight"], k_norm=ka["norm"]["weight"]),
                              dict(rotate_half=rq["half"], kv_cache_inputs=(ka["cache"], va["cache"]),
                                   arithmetic_dtype="bfloat16", eps=qn["eps"])))
        # the attention call itself
        kw = N[sd].kwargs
        if kw.get("is_causal") not in (0, False, None) or kw.get("dropout_p") not in (0, 0.0, None):
            raise LoweringError(f"layer {layer}: unexpected attention arguments {kw}")
        mask = kw.get("attn_mask")
        mask_src, seen = m.through(m.node(mask), ("getitem",))
        if N[mask_src].name != "causal_mask":
            raise LoweringError(f"layer {layer}: attention mask is not the causal mask")
        scale_item = m.node(kw["scale"])
        kernels.append(Kernel("attention", layer, sorted(set(k_attn + v_attn + [sd])), {},
                              dict(heads_q=ka["heads_q"], heads_kv=ka["heads_kv"], group=ka["group"], causal=True,
                                   scale=N[m.arg(scale_item, 0)].name)))
        book += seen + [scale_item]
        # output projection: back from o_proj's input to the sdpa node through layout-only nodes
        src, seen = m.through(m.arg(lo, 0), ("contiguous", "reshape", "transpose"))
        if src != sd:
            raise LoweringError(f"layer {layer}: o_proj does not read the attention output")
        book += seen
        kernels.append(Kernel("o_gemm", layer, [lo], dict(o=N[m.arg(lo, 1)].name)))
        # residual add + post-attention norm
        norm_nodes, pa = m.rms_norm(m.arg(lg, 0))
        add1 = m.expect(pa["input"], "add")
        if {m.arg(add1, 0), m.arg(add1, 1)} != {residual, lo}:
            raise LoweringError(f"layer {layer}: first residual add does not add o_proj to the residual stream")
        kernels.append(Kernel("add_rms_norm", layer, [add1] + norm_nodes, dict(weight=pa["weight"], eps=pa["eps"]),
                              dict(fused_add=True, stats_dtype="float32", cast_before_weight="bfloat16")))
        # MLP
        if m.arg(lu, 0) != m.arg(lg, 0):
            raise LoweringError(f"layer {layer}: gate and up projections do not share one input")
        prod = m.expect(m.arg(ld, 0), "*")
        silu = m.expect(m.arg(prod, 0), "silu")
        if m.arg(silu, 0) != lg or m.arg(prod, 1) != lu:
            raise LoweringError(f"layer {layer}: MLP is not down(silu(gate) * up)")
        kernels.append(Kernel("gate_up_swiglu_gemm", layer, [lg, silu, lu, prod],
                              dict(gate=N[m.arg(lg, 1)].name, up=N[m.arg(lu, 1)].name)))
        kernels.append(Kernel("down_gemm", layer, [ld], dict(down=N[m.arg(ld, 1)].name)))
        users = [m.index[u] for u in N[ld].users]
        if len(users) != 1 or m.ops[users[0]] != "add" or {m.arg(users[0], 0), m.arg(users[0], 1)} != {add1, ld}:
            raise LoweringError(f"layer {layer}: second residual add does not add down_proj to the residual stream")
        pending_add, residual = users[0], users[0]
        if layer == 0:
            ex = m.example
            cfg = dict(hidden=ex[embed_w].shape[1], vocab=ex[embed_w].shape[0], head_dim=head_dim,
                       num_q_heads=ex[N[m.arg(lq, 1)].name].shape[0] // head_dim,
                       num_kv_heads=ex[N[m.arg(lk, 1)].name].shape[0] // head_dim,
                       intermediate=ex[N[m.arg(lg, 1)].name].shape[0])
            if (ka["heads_q"], ka["heads_kv"]) != (cfg["num_q_heads"], cfg["num_kv_heads"]):
                raise LoweringError("head counts of the GQA expand disagree with the projection shapes")
    # head: final norm on the kept positions, LM head
    lh = linears[-1]
    x, seen = m.through(m.arg(lh, 0), ("getitem",))
    book += seen + [m.index[a.name] for s in seen for a in _node_refs(N[s].args) if m.ops[m.index[a.name]] == "neg"]
    norm_nodes, fa = m.rms_norm(x)
    if fa["input"] != pending_add:
        raise LoweringError("final norm does not read the last residual add")
    kernels.append(Kernel("add_rms_norm", -1, [pending_add] + norm_nodes, dict(weight=fa["weight"], eps=fa["eps"]),
                          dict(fused_add=True, stats_dtype="float32", cast_before_weight="bfloat16")))
    head_w = N[m.arg(lh, 1)].name
    kernels.append(Kernel("lm_head_gemm", -1, [lh], dict(lm_head=head_w)))
    cfg.update(num_layers=n_layers, tied=(head_w == embed_w))

    # everything else must be host-side bookkeeping: mask construction, scalar reads, layout-only nodes
    used = {}
    for k in kernels:
        for i in k.nodes:
            if i in used:
                raise LoweringError(f"node {i} ({N[i].name}) claimed by {used[i]} and {k.kind}")
            used[i] = k.kind
    free_ops = {"item", "contiguous", "view", "reshape", "transpose", "unsqueeze", "getitem", "expand", "float", "to",
                "arange", "iadd", "lazy_load_decompositions", "vmap_increment_nesting", "vmap_decrement_nesting",
                "add_batch_dim", "remove_batch_dim", "new_ones", "le", "and", "aten.index", "enter_autocast",
                "exit_autocast", "neg", "numel", "sym_sum", "add", None, "placeholder", "output"}
    first_layer_node = min(i for k in kernels if k.layer == 0 for i in k.nodes)
    for i, op in enumerate(m.ops):
        if i in used:
            continue
        if op not in free_ops:
            raise LoweringError(f"node {i} ({N[i].name}, {op}) does device work that no kernel covers")
        if op in ("to", "add", "neg", "float") and i > first_layer_node and i not in book:
            # inside the layers these would be arithmetic or cast points the kernels do not implement
            raise LoweringError(f"node {i} ({N[i].name}, {op}) is an arithmetic / cast node outside every kernel")
        if N[i].kind not in ("placeholder", "output"):
            book.append(i)
    return Qwen3Plan(cfg, kernels, sorted(set(book)), any(k.attrs.get("kv_cache_inputs", (None,))[0] for k in kernels))


def _node_refs(value):
    if isinstance(value, NodeRef):
        yield value
    elif isinstance(value, (list, tuple)):
        for v in value:
            yield from _node_refs(v)
    elif isinstance(value, slice):
        yield from _node_refs((value.start, value.stop, value.step))


def runner_weights(plan):
    """Per-layer and model-level state-dict keys of the plan's weights, in the runner's slots:
    ``{"layers": [{"q": ..., "k": ..., "v": ..., "o": ..., "gate": ..., "up": ..., "down": ..., "input_ln": ...,
    "post_ln": ..., "q_norm": ..., "k_norm": ...}], "embed": ..., "final_norm": ..., "lm_head": ..., "inv_freq": ...}``"""
    layers = [dict() for _ in range(plan.config["num_layers"])]
    out = {"layers": layers}
    for k in plan.kernels:
        w = {role: hf_name(ph) for role, ph in k.weights.items() if ph}
        if k.layer >= 0:
            d = layers[k.layer]
            if k.kind == "add_rms_norm":
                d["post_ln" if "input_ln" in d else "input_ln"] = w["weight"]
            elif k.kind == "head_norm_rope_kv":
                d.update(q_norm=w["q_norm"], k_norm=w["k_norm"])
            else:
                d.update(w)
        elif k.kind == "embedding":
            out["embed"] = w["table"]
        elif k.kind == "rope_table":
            out["inv_freq"] = w.get("inv_freq", "")
        elif k.kind == "add_rms_norm":
            out["final_norm"] = w["weight"]
        elif k.kind == "lm_head_gemm":
            out["lm_head"] = w["lm_head"]
    return out


def runner_config(plan, eps=1e-6, rope_theta=1e6):
    """The plan's model shape as the runner's ``Qwen3Config`` (``teenygrad_b200.qwen3``).  eps and rope_theta are
    scalar inputs of the trace whose values the file does not carry: the caller supplies the model's."""
    from .qwen3 import Qwen3Config
    c = plan.config
    return Qwen3Config(c["num_layers"], c["hidden"], c["num_q_heads"], c["num_kv_heads"], c["head_dim"],
                       c["intermediate"], c["vocab"], eps=eps, rope_theta=rope_theta, tied=c["tied"])


def build_runner(plan, state_dict, max_batch, max_len, eps=1e-6, rope_theta=1e6, **runner_kwargs):
    """A ``Qwen3Runner`` for the traced model: shape from the plan, every weight looked up in ``state_dict`` under the
    key the trace's placeholder names translate to (``runner_weights``)."""
    from . import qwen3
    names = runner_weights(plan)
    sd = {}
    for i, layer in enumerate(names["layers"]):
        p = f"model.layers.{i}."
        for role, key in (("q", "self_attn.q_proj"), ("k", "self_attn.k_proj"), ("v", "self_attn.v_proj"),
                          ("o", "self_attn.o_proj"), ("q_norm", "self_attn.q_norm"), ("k_norm", "self_attn.k_norm"),
                          ("gate", "mlp.gate_proj"), ("up", "mlp.up_proj"), ("down", "mlp.down_proj"),
                          ("input_ln", "input_layernorm"), ("post_ln", "post_attention_layernorm")):
            sd[p + key + ".weight"] = state_dict[layer[role]]
    sd["model.embed_tokens.weight"] = state_dict[names["embed"]]
    sd["model.norm.weight"] = state_dict[names["final_norm"]]
    if not plan.config["tied"]:
        sd["lm_head.weight"] = state_dict[names["lm_head"]]
    r = qwen3.Qwen3Runner(runner_config(plan, eps, rope_theta), max_batch=max_batch, max_len=max_len, **runner_kwargs)
    r.load_state_dict(sd)
    return r


# ---------------------------------------------------------------------------------------------------------------
# JSON form of a graph (fixtures that travel without the binary files)
# ---------------------------------------------------------------------------------------------------------------
def _enc(v):
    if isinstance(v, NodeRef):
        return {"n": v.name}
    if v is Ellipsis:
        return {"e": 1}
    if isinstance(v, slice):
        return {"s": [_enc(v.start), _enc(v.stop), _enc(v.step)]}
    if isinstance(v, tuple):
        if len(v) == 2 and v[0] in ("dtype", "device") and isinstance(v[1], str):
            return {v[0][0:2]: v[1]}          # {"dt": ...} / {"de": ...}
        return {"t": [_enc(x) for x in v]}
    if isinstance(v, list):
        return [_enc(x) for x in v]
    return v


def _dec(v):
    if isinstance(v, dict):
        if "n" in v: return NodeRef(v["n"])
        if "e" in v: return Ellipsis
        if "s" in v: return slice(*[_dec(x) for x in v["s"]])
        if "dt" in v: return ("dtype", v["dt"])
        if "de" in v: return ("device", v["de"])
        if "t" in v: return tuple(_dec(x) for x in v["t"])
        raise ValueError(f"unknown encoded value {v}")
    if isinstance(v, list):
        return [_dec(x) for x in v]
    return v


def graph_to_json(graph):
    return {"nodes": [[n.kind, n.name, n.target, _enc(n.args), {k: _enc(v) for k, v in n.kwargs.items()}, n.users]
                      for n in graph.nodes],
            "example_inputs": [e if (e is None or isinstance(e, str)) else [e.dtype, list(e.shape), list(e.stride), e.device]
                               for e in graph.example_inputs]}


def graph_from_json(obj):
    nodes = [FxNode(k, name, target, _dec(args), {a: _dec(b) for a, b in kwargs.items()}, users)
             for k, name, target, args, kwargs, users in obj["nodes"]]
    inputs = [e if (e is None or isinstance(e, str)) else ExampleTensor(e[0], tuple(e[1]), tuple(e[2]), e[3])
              for e in obj["example_inputs"]]
    return FxGraph(nodes, inputs)
