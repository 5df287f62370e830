"""The traced-graph reader and the lowering of the reference's Qwen3 traces onto the runner's kernel sequence.

Fixtures ``tests/golden/qwen3_fx_{prefill,decode}.json.gz`` are the decoded node lists of the reference's
``support/teeny-torch/tests/data/qwen3_{1,2}.bin.gz`` (written by ``tests/golden/make_fx_golden.py``).
"""
import copy
import gzip
import json
import os
import re
from collections import Counter

import pytest

from teenygrad_b200 import fxgraph as fx

HERE = os.path.dirname(os.path.abspath(__file__))
# a teenygrad checkout named by TEENY_REFERENCE_ROOT, or sitting next to this repository as ``reference``
REF_DATA = os.path.join(os.environ.get("TEENY_REFERENCE_ROOT", os.path.join(os.path.dirname(HERE), os.pardir, "reference")),
                        "support", "teeny-torch", "tests", "data")


def load(which):
    with gzip.open(os.path.join(HERE, "golden", f"qwen3_fx_{which}.json.gz"), "rt") as f:
        return fx.graph_from_json(json.load(f))


@pytest.fixture(scope="module")
def prefill():
    return load("prefill")


@pytest.fixture(scope="module")
def decode():
    return load("decode")


def test_reader_round_trip_on_a_built_graph():
    from fx_builder import encode_graph
    nodes = [
        fx.FxNode("placeholder", "s27", "s27", users=["view"]),
        fx.FxNode("placeholder", "x", "L_x_", users=["lin"]),
        fx.FxNode("placeholder", "w", "L_w_", users=["lin"]),
        fx.FxNode("call_function", "lin", "<built-in function linear>", [fx.NodeRef("x"), fx.NodeRef("w"), None], {}, ["view"]),
        fx.FxNode("call_method", "view", "view", [fx.NodeRef("lin"), (1, fx.NodeRef("s27"), -1, 128)], {}, ["cut"]),
        fx.FxNode("call_function", "cut", "<built-in function getitem>",
                  [fx.NodeRef("view"), (Ellipsis, slice(None, 64, None))], {}, ["cast"]),
        fx.FxNode("call_method", "cast", "to", [fx.NodeRef("cut")], {"dtype": ("dtype", "bfloat16"), "device": ("device", "cpu")},
                  ["cat"]),
        fx.FxNode("call_function", "cat", "<built-in method cat of type object at 0x7c>", [[fx.NodeRef("cast"), fx.NodeRef("cast")]],
                  {"dim": -2}, ["output"]),
        fx.FxNode("output", "output", "", [], {}, []),
    ]
    inputs = ["s27", fx.ExampleTensor("bfloat16", (1, "s27", 1024), (18432, 1024, 1), "cpu"),
              fx.ExampleTensor("float32", (), (), "cpu")]
    g = fx.parse_graph(encode_graph(fx.FxGraph(nodes, inputs)))
    assert g.nodes == nodes
    assert g.example_inputs == inputs
    assert [fx.op_of(n) for n in g.nodes] == ["placeholder", "placeholder", "placeholder", "linear", "view", "getitem", "to",
                                              "cat", "output"]
    assert fx.graph_from_json(json.loads(json.dumps(fx.graph_to_json(g)))).nodes == nodes


@pytest.mark.skipif(not os.path.isdir(REF_DATA), reason="reference checkout not present")
@pytest.mark.parametrize("src,which", [("qwen3_1.bin.gz", "prefill"), ("qwen3_2.bin.gz", "decode")])
def test_fixture_equals_the_reference_file(src, which):
    g = fx.read_graph(os.path.join(REF_DATA, src))
    for n in g.nodes:
        n.target = re.sub(r" at 0x[0-9a-f]+", "", n.target)
    want = load(which)
    assert g.nodes == want.nodes and g.example_inputs == want.example_inputs


def test_trace_vocabulary_and_op_counts(prefill, decode):
    """Every node maps into FxGraphLang (support/teeny-fxgraph/src/fxgraph/lang.rs:29-83); the counts are those of a
    28-layer Qwen3: 7 projections per layer + LM head, 4 norms per layer + final, one SDPA and one SiLU per layer."""
    for g, cats in ((prefill, 57), (decode, 113)):
        c = Counter(fx.op_of(n) for n in g.nodes)
        assert set(k for k in c if k) <= set(fx.LANG_OPS) | {"placeholder", "output"}
        assert (c["linear"], c["rsqrt"], c["silu"], c["sdpa"], c["neg"], c["embedding"], c["@"]) == (197, 113, 28, 28, 57, 1, 1)
        assert c["cat"] == cats  # decode adds the key / value cache concatenations: 2 per layer


@pytest.mark.parametrize("which", ["prefill", "decode"])
def test_lowering_gives_the_runner_kernel_sequence(which, prefill, decode):
    g = prefill if which == "prefill" else decode
    plan = fx.lower_qwen3(g)
    assert plan.config == dict(num_layers=28, hidden=1024, num_q_heads=16, num_kv_heads=8, head_dim=128,
                               intermediate=3072, vocab=151936, tied=True)   # BASELINE config 4's model
    want = [k for k, _ in fx.DECODER_LAYER_KERNELS]
    for layer in range(28):
        assert plan.layer_kinds(layer) == want, layer
    assert [k.kind for k in plan.kernels if k.layer < 0] == ["embedding", "rope_table"] + [k for k, _ in fx.HEAD_KERNELS]
    assert plan.has_kv_cache_inputs == (which == "decode")
    # cast points the kernels implement (and the lowering insists on)
    norms = [k for k in plan.kernels if k.kind == "add_rms_norm"]
    assert len(norms) == 2 * 28 + 1
    assert all(k.attrs["stats_dtype"] == "float32" and k.attrs["cast_before_weight"] == "bfloat16" for k in norms)
    assert [k.attrs["fused_add"] for k in norms[:3]] == [False, True, True]
    rope = [k for k in plan.kernels if k.kind == "rope_table"][0]
    assert rope.attrs == dict(table_dtype="bfloat16", angle_dtype="float32")
    heads = [k for k in plan.kernels if k.kind == "head_norm_rope_kv"]
    assert all(k.attrs["rotate_half"] == 64 and k.attrs["arithmetic_dtype"] == "bfloat16" for k in heads)
    assert all((k.attrs["kv_cache_inputs"][0] is not None) == (which == "decode") for k in heads)
    attn = [k for k in plan.kernels if k.kind == "attention"]
    assert all(k.attrs["causal"] and (k.attrs["heads_q"], k.attrs["heads_kv"], k.attrs["group"]) == (16, 8, 2) for k in attn)
    # every node is either inside exactly one kernel or host-side bookkeeping
    covered = [i for k in plan.kernels for i in k.nodes]
    assert len(covered) == len(set(covered))
    n_compute = sum(1 for n in g.nodes if n.kind in ("call_function", "call_method"))
    assert len(set(covered) | set(plan.bookkeeping)) >= n_compute - 1  # the one dropped node: _log_api_usage_once
    heavy = {"linear", "sdpa", "silu", "rsqrt", "pow", "mean", "embedding", "@", "cos", "sin", "cat", "*"}
    assert all(fx.op_of(g.nodes[i]) not in heavy for i in plan.bookkeeping)


def test_weight_names_are_the_checkpoint_keys(prefill):
    names = fx.runner_weights(fx.lower_qwen3(prefill))
    assert names["embed"] == names["lm_head"] == "model.embed_tokens.weight"
    assert names["final_norm"] == "model.norm.weight" and names["inv_freq"] == "model.rotary_emb.inv_freq"
    assert names["layers"][27] == {
        "input_ln": "model.layers.27.input_layernorm.weight", "q": "model.layers.27.self_attn.q_proj.weight",
        "k": "model.layers.27.self_attn.k_proj.weight", "v": "model.layers.27.self_attn.v_proj.weight",
        "q_norm": "model.layers.27.self_attn.q_norm.weight", "k_norm": "model.layers.27.self_attn.k_norm.weight",
        "o": "model.layers.27.self_attn.o_proj.weight", "post_ln": "model.layers.27.post_attention_layernorm.weight",
        "gate": "model.layers.27.mlp.gate_proj.weight", "up": "model.layers.27.mlp.up_proj.weight",
        "down": "model.layers.27.mlp.down_proj.weight"}


def _mutated(graph, name, **changes):
    g = copy.deepcopy(graph)
    n = next(n for n in g.nodes if n.name == name)
    for k, v in changes.items():
        setattr(n, k, v)
    return g


def test_lowering_refuses_traces_the_kernels_do_not_implement(prefill):
    # the normalised row cast to float16 instead of bfloat16 before the weight multiply (node to_7 of layer 0)
    with pytest.raises(fx.LoweringError, match="bfloat16"):
        fx.lower_qwen3(_mutated(prefill, "to_7", args=[fx.NodeRef("hidden_states_1"), ("dtype", "float16")]))
    # statistics in bfloat16
    with pytest.raises(fx.LoweringError, match="float32"):
        fx.lower_qwen3(_mutated(prefill, "hidden_states", args=[fx.NodeRef("inputs_embeds"), ("dtype", "bfloat16")]))
    # rotary tables left in float32
    with pytest.raises(fx.LoweringError, match="rotary"):
        fx.lower_qwen3(_mutated(prefill, "cos_2", kwargs={"dtype": ("dtype", "float32")}))
    # a projection with a bias
    with pytest.raises(fx.LoweringError, match="bias"):
        fx.lower_qwen3(_mutated(prefill, "linear_1", args=[fx.NodeRef("hidden_states_2"), fx.NodeRef(
            "l_self_modules_model_modules_layers_modules_0_modules_self_attn_modules_k_proj_parameters_weight_"),
            fx.NodeRef("hidden_states_2")]))
    # the "other" rotation convention (interleaved halves swapped)
    with pytest.raises(fx.LoweringError, match="rotate_half"):
        fx.lower_qwen3(_mutated(prefill, "x1", args=[fx.NodeRef("query_states"), (Ellipsis, slice(None, 32, None))]))
    # an op outside the vocabulary
    with pytest.raises(ValueError, match="vocabulary"):
        fx.lower_qwen3(_mutated(prefill, "silu", target="<function gelu>"))
