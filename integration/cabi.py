"""Parses the C declarations of include/*.h and renders them as a Rust ``extern "C"`` block.

    python integration/cabi.py            # rewrites the generated block inside integration/teeny-cuda/src/b200.rs

The Rust sources under ``integration/`` are what a teenygrad maintainer drops into ``drivers/teeny-cuda`` and
``kernels/teeny-kernels`` to bind this library (no Rust toolchain is needed to keep them honest: the tests parse both
sides and fail on any drift in names, arity, argument types, struct fields or enum values).
"""
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADERS = ("teeny_b200.h", "teeny_qwen3.h")
RUST_FILE = os.path.join(ROOT, "integration", "teeny-cuda", "src", "b200.rs")
BEGIN, END = "// ---- generated from include/*.h: begin ----", "// ---- generated from include/*.h: end ----"

# C type (whitespace-normalised) -> Rust type
TYPES = {
    "void": "()", "int": "c_int", "float": "f32", "size_t": "usize", "long long": "c_longlong",
    "unsigned long long": "c_ulonglong", "teeny_stream_t": "CUstream", "uint32_t": "u32", "const uint32_t*": "*const u32",
    "unsigned*": "*mut c_uint", "unsigned long long*": "*mut c_ulonglong", "const unsigned long long*": "*const c_ulonglong",
    "const float*": "*const f32", "float*": "*mut f32", "const int*": "*const c_int", "int*": "*mut c_int",
    "const teeny_bf16*": "*const u16", "teeny_bf16*": "*mut u16", "const void*": "*const c_void", "void*": "*mut c_void",
    "void**": "*mut *mut c_void", "const char*": "*const c_char",
    "const teeny_attn_shape*": "*const TeenyAttnShape", "const teeny_qwen3_config*": "*const TeenyQwen3Config",
    "teeny_qwen3*": "*mut TeenyQwen3", "teeny_qwen3**": "*mut *mut TeenyQwen3",
}
STRUCT_NAMES = {"teeny_attn_shape": "TeenyAttnShape", "teeny_qwen3_config": "TeenyQwen3Config"}


def _strip_comments(text):
    return re.sub(r"/\*.*?\*/", " ", text, flags=re.S)


def _norm_type(t):
    t = re.sub(r"\s+", " ", t.strip())
    t = re.sub(r"\s*\*\s*", "*", t)
    return t


def parse_headers(include_dir=None):
    """-> (functions, structs, enums): functions = [(name, ret_ctype, [(ctype, argname), ...])] in declaration order,
    structs = {c_name: [(ctype, field), ...]}, enums = {NAME: value}."""
    include_dir = include_dir or os.path.join(ROOT, "include")
    functions, structs, enums = [], {}, {}
    for h in HEADERS:
        text = _strip_comments(open(os.path.join(include_dir, h)).read())
        text = re.sub(r"^\s*#.*$", "", text, flags=re.M)
        for m in re.finditer(r"typedef\s+struct\s*\{(.*?)\}\s*(\w+)\s*;", text, flags=re.S):
            fields = []
            for decl in m.group(1).split(";"):
                decl = decl.strip()
                if not decl:
                    continue
                ctype, names = re.match(r"((?:unsigned\s+)?(?:long\s+long|\w+))\s+(.*)", decl, flags=re.S).groups()
                fields += [(_norm_type(ctype), n.strip()) for n in names.split(",")]
            structs[m.group(2)] = fields
        for m in re.finditer(r"enum\s*\{(.*?)\}\s*;", text, flags=re.S):
            value = -1
            for item in m.group(1).split(","):
                item = item.strip()
                if not item:
                    continue
                if "=" in item:
                    name, v = (s.strip() for s in item.split("="))
                    value = int(v, 0)
                else:
                    name, value = item, value + 1
                enums[name] = value
        body = re.sub(r"typedef[^;{]*(\{.*?\})?[^;]*;", " ", text, flags=re.S)
        body = re.sub(r"enum\s*\{.*?\}\s*;", " ", body, flags=re.S)
        body = re.sub(r'extern\s+"C"\s*\{', " ", body)
        for m in re.finditer(r"([\w\s\*]+?)\b(\w+)\s*\(([^;{()]*)\)\s*;", body):
            ret, name, args = _norm_type(m.group(1)), m.group(2), m.group(3).strip()
            parsed = []
            if args and args != "void":
                for a in args.split(","):
                    am = re.match(r"(.*?)(\w+)$", a.strip(), flags=re.S)
                    parsed.append((_norm_type(am.group(1)), am.group(2)))
            functions.append((name, ret, parsed))
    return functions, structs, enums


_RUST_KEYWORDS = {"type", "ref", "fn", "in", "loop", "match", "mod", "move", "use", "where", "box"}


def rust_arg_name(name):
    s = re.sub(r"(?<=[a-z0-9])(?=[A-Z])", "_", name).lower()
    return s + "_" if s in _RUST_KEYWORDS else s


def render_rust(functions, structs, enums):
    out = [BEGIN]
    for cname, fields in structs.items():
        out.append("#[repr(C)]\n#[derive(Clone, Copy, Debug, Default)]\npub struct %s {" % STRUCT_NAMES[cname])
        for ctype, f in fields:
            out.append(f"    pub {rust_arg_name(f)}: {TYPES[ctype]},")
        out.append("}")
    out.append("/// Opaque runner handle (`teeny_qwen3`).\n#[repr(C)]\npub struct TeenyQwen3 {\n    _private: [u8; 0],\n}")
    for name, value in enums.items():
        out.append(f"pub const {name}: c_int = {value};")
    out.append('#[link(name = "teeny_b200")]\nextern "C" {')
    for name, ret, args in functions:
        rendered = ", ".join(f"{rust_arg_name(a)}: {TYPES[t]}" for t, a in args)
        tail = "" if ret == "void" else f" -> {TYPES[ret]}"
        out.append(f"    pub fn {name}({rendered}){tail};")
    out.append("}")
    out.append(END)
    return "\n".join(out)


def parse_rust_extern(text):
    """-> (functions, structs, consts) as found in a Rust source: functions = {name: ([rust types], ret or None)}."""
    block = re.search(r'extern\s+"C"\s*\{(.*?)\n\}', text, flags=re.S).group(1)
    functions = {}
    for m in re.finditer(r"pub fn (\w+)\((.*?)\)(?:\s*->\s*([^;]+))?;", block, flags=re.S):
        args = [a.split(":", 1)[1].strip() for a in m.group(2).split(",") if a.strip()]
        functions[m.group(1)] = (args, m.group(3).strip() if m.group(3) else None)
    structs = {}
    for m in re.finditer(r"#\[repr\(C\)\][^{]*?pub struct (\w+) \{(.*?)\}", text, flags=re.S):
        structs[m.group(1)] = [(f.split(":")[0].replace("pub", "").strip(), f.split(":")[1].strip())
                               for f in m.group(2).split(",") if ":" in f]
    consts = {m.group(1): int(m.group(2)) for m in re.finditer(r"pub const (\w+): c_int = (-?\d+);", text)}
    return functions, structs, consts


def main():
    text = open(RUST_FILE).read()
    a, b = text.index(BEGIN), text.index(END) + len(END)
    new = text[:a] + render_rust(*parse_headers()) + text[b:]  # rendered in full before the file is touched
    open(RUST_FILE, "w").write(new)


if __name__ == "__main__":
    main()
