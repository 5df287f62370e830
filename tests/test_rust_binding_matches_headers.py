"""The Rust sources under integration/ (what a teenygrad maintainer adds to drivers/teeny-cuda and
kernels/teeny-kernels) against include/*.h: no Rust toolchain exists where this library is built, so both sides are
parsed and compared -- function names, arity and argument types of the ``extern "C"`` block, ``#[repr(C)]`` struct
fields, constants, the argument extraction of every ``launch_direct`` arm and the visit sequence of every
``RuntimeOp::pack_args`` against the C declaration of the entry point it names."""
import os
import re
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "integration"))

import cabi  # noqa: E402

B200_RS = os.path.join(ROOT, "integration", "teeny-cuda", "src", "b200.rs")
OPS_RS = os.path.join(ROOT, "integration", "teeny-kernels", "src", "b200_ops.rs")


def test_extern_block_matches_the_headers():
    functions, structs, enums = cabi.parse_headers()
    assert len(functions) >= 50
    rust_fns, rust_structs, rust_consts = cabi.parse_rust_extern(open(B200_RS).read())
    assert sorted(rust_fns) == sorted(name for name, _, _ in functions)
    for name, ret, args in functions:
        r_args, r_ret = rust_fns[name]
        assert r_args == [cabi.TYPES[t] for t, _ in args], name
        assert r_ret == (None if ret == "void" else cabi.TYPES[ret]), name
    for cname, fields in structs.items():
        assert rust_structs[cabi.STRUCT_NAMES[cname]] == [(cabi.rust_arg_name(f), cabi.TYPES[t]) for t, f in fields], cname
    assert rust_consts == enums


def test_generated_block_is_current():
    text = open(B200_RS).read()
    a, b = text.index(cabi.BEGIN), text.index(cabi.END) + len(cabi.END)
    assert text[a:b] == cabi.render_rust(*cabi.parse_headers()), "run python integration/cabi.py"


_KIND = {"p": "ptr", "i": "int", "l": "long long", "f": "float"}


def _c_kind(ctype):
    if ctype.endswith("*"):
        return "ptr"
    return {"int": "int", "long long": "long long", "float": "float", "size_t": "size_t",
            "teeny_stream_t": "stream", "unsigned long long": "unsigned long long"}[ctype]


def test_launch_direct_arms_follow_the_declarations():
    functions = {name: args for name, _, args in cabi.parse_headers()[0]}
    text = open(B200_RS).read()
    body = text[text.index("pub fn launch_direct"):]
    arms = re.findall(r'"(\w+)" => (\w+)\((.*?)\),\n', body)
    assert len(arms) >= 20
    for entry, called, arglist in arms:
        assert entry == called, f"arm {entry} calls {called}"
        want = [_c_kind(t) for t, _ in functions[entry]]
        got = []
        for tok in (a.strip() for a in arglist.replace("(a, ", "(a;").split(",")):
            m = re.match(r"([pilf])\(a;(\d+)\)(\.cast\(\))?$", tok)
            if m:
                assert int(m.group(2)) == len([g for g in got if g in _KIND.values()]), (entry, tok)  # positions in order
                got.append(_KIND[m.group(1)])
            elif tok == "null":
                got.append("ptr")
            elif tok == "0":
                got.append("size_t")
            elif tok == "stream":
                got.append("stream")
            else:
                raise AssertionError(f"{entry}: unexpected argument expression {tok!r}")
        assert got == want, entry


def test_pack_args_visit_the_entry_points_arguments_in_order():
    functions = {name: args for name, _, args in cabi.parse_headers()[0]}
    text = open(OPS_RS).read()
    packs = re.findall(r"// entry point: (\w+)\n\s*fn (\w+)\(.*?\{\n(.*?)\n    \}\n", text, flags=re.S)
    assert sorted(e for e, _, _ in packs) == sorted(["linear_forward_entry_point_bf16", "teeny_add_rms_norm_bf16",
                                                     "teeny_linear_swiglu_bf16", "teeny_qk_norm_rope_kv_bf16",
                                                     "teeny_flash_attn_fwd_bf16"])
    visit_kind = {"visit_ptr": "ptr", "visit_i32": "int", "visit_i64": "long long", "visit_f32": "float"}
    for entry, _, body in packs:
        visits = re.findall(r"visitor\.(visit_\w+)\(.*?\); // (\w+)", body)
        decl = [(t, n) for t, n in functions[entry] if _c_kind(t) not in ("stream", "size_t") and n != "global_scratch"]
        assert [visit_kind[v] for v, _ in visits] == [_c_kind(t) for t, _ in decl], entry
        assert [n for _, n in visits] == [n for _, n in decl], entry   # the trailing comments name the C parameters
    # every entry point an op lowers to has a direct-call arm
    arms = set(re.findall(r'"(\w+)" => ', open(B200_RS).read()))
    lowered = set(re.findall(r'lowered\("\w+", "(\w+)"', text)) | set(re.findall(r'"(teeny_\w+)"', text))
    assert lowered <= arms, lowered - arms
