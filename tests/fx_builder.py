"""A minimal FlatBuffers writer for the traced-graph schema (test helper): lets the reader in
``teenygrad_b200.fxgraph`` be exercised on graphs built in the test, without the FlatBuffers package.

Objects are laid out front to back: a table is written with zeroed offset fields, its children are appended behind it
and the offsets patched (an unsigned offset must point forward; the signed vtable offset may point either way).
"""
import struct

from teenygrad_b200 import fxgraph as fx


class Builder:
    def __init__(self):
        self.b = bytearray(4)  # root offset, patched at the end
        self.todo = []

    def _align(self, n=4):
        while len(self.b) % n:
            self.b.append(0)

    def string(self, s):
        self._align()
        at = len(self.b)
        raw = s.encode()
        self.b += struct.pack("<I", len(raw)) + raw + b"\0"
        return at

    def table(self, fields):
        """fields: list of None | ("u8", v) | ("i8", v) | ("i32", v) | ("ref", callable that writes the child and
        returns its position).  Returns the table position."""
        self._align()
        sizes = {"u8": 1, "i8": 1, "i32": 4, "ref": 4}
        vt_at = len(self.b)
        offs, cur = [], 4
        for f in fields:
            if f is None:
                offs.append(0)
                continue
            sz = sizes[f[0]]
            cur = (cur + sz - 1) // sz * sz
            offs.append(cur)
            cur += sz
        tsize = (cur + 3) // 4 * 4
        self.b += struct.pack("<HH", 4 + 2 * len(fields), tsize) + b"".join(struct.pack("<H", o) for o in offs)
        self._align()
        t_at = len(self.b)
        self.b += bytearray(tsize)
        struct.pack_into("<i", self.b, t_at, t_at - vt_at)
        for f, o in zip(fields, offs):
            if f is None:
                continue
            if f[0] == "u8":
                self.b[t_at + o] = f[1]
            elif f[0] == "i8":
                struct.pack_into("<b", self.b, t_at + o, f[1])
            elif f[0] == "i32":
                struct.pack_into("<i", self.b, t_at + o, f[1])
            else:
                child = f[1]()
                struct.pack_into("<I", self.b, t_at + o, child - (t_at + o))
        return t_at

    def vector(self, writers):
        """A vector of offsets to children (tables or strings)."""
        self._align()
        at = len(self.b)
        self.b += struct.pack("<I", len(writers)) + bytearray(4 * len(writers))
        for i, w in enumerate(writers):
            slot = at + 4 + 4 * i
            child = w()
            struct.pack_into("<I", self.b, slot, child - slot)
        return at

    def u32_vector(self, values):
        self._align()
        at = len(self.b)
        self.b += struct.pack("<I", len(values)) + b"".join(struct.pack("<I", v) for v in values)
        return at

    def finish(self, root):
        struct.pack_into("<I", self.b, 0, root)
        return bytes(self.b)


def _value(b, v):
    """Writes a ValueWrapper for a Python value (the inverse of the reader's decoding)."""
    kinds = fx._VALUE_KINDS

    def wrap(kind, inner_fields):
        return b.table([("u8", kinds.index(kind)), ("ref", lambda: b.table(inner_fields))])

    if v is None:
        return wrap("none", [])
    if isinstance(v, fx.NodeRef):
        return wrap("node", [("ref", lambda: b.string(v.name))])
    if v is Ellipsis:
        return wrap("ellipsis", [])
    if isinstance(v, bool) or isinstance(v, int):
        return wrap("int", [("i32", int(v))])
    if isinstance(v, str):
        return wrap("str", [("ref", lambda: b.string(v))])
    if isinstance(v, slice):
        return wrap("slice", [("ref", lambda: _value(b, v.start)), ("ref", lambda: _value(b, v.stop)),
                              ("ref", lambda: _value(b, v.step))])
    if isinstance(v, tuple) and len(v) == 2 and v[0] == "dtype":
        return wrap("dtype", [("i8", fx.DTYPES.index(v[1]))])
    if isinstance(v, tuple) and len(v) == 2 and v[0] == "device":
        return wrap("device", [("ref", lambda: b.string(v[1]))])
    if isinstance(v, (tuple, list)):
        kind = "tuple" if isinstance(v, tuple) else "list"
        return wrap(kind, [("ref", lambda: b.vector([(lambda x=x: _value(b, x)) for x in v]))])
    raise TypeError(v)


def encode_graph(graph):
    """FxGraph -> FlatBuffers bytes of a ``Graph`` table."""
    b = Builder()

    def node_writer(n):
        def call_like():
            return b.table([("ref", lambda: b.string(n.name)), ("ref", lambda: b.string(n.target)),
                            ("ref", lambda: b.vector([(lambda a=a: _value(b, a)) for a in n.args])),
                            ("ref", lambda: b.vector([(lambda k=k, v=v: b.table([("ref", lambda: b.string(k)),
                                                                                  ("ref", lambda: _value(b, v))]))
                                                      for k, v in n.kwargs.items()])),
                            ("ref", lambda: b.vector([(lambda u=u: b.string(u)) for u in n.users]))])

        def placeholder():
            return b.table([("ref", lambda: b.string(n.name)), ("ref", lambda: b.string(n.target)),
                            ("ref", lambda: b.vector([(lambda u=u: b.string(u)) for u in n.users]))])

        inner = placeholder if n.kind == "placeholder" else call_like
        return lambda: b.table([("u8", fx._NODE_KINDS.index(n.kind)), ("ref", inner)])

    def input_writer(e):
        if isinstance(e, str):
            return lambda: b.table([("u8", 1), ("ref", lambda: b.table([("ref", lambda: b.string(e))]))])

        def tensor():
            return b.table([("i8", fx.DTYPES.index(e.dtype)), ("ref", lambda: b.string(e.device)),
                            ("ref", lambda: b.table([("ref", lambda: b.vector(
                                [(lambda d=d: b.table([("ref", lambda: b.string(str(d)))])) for d in e.shape]))])),
                            ("ref", lambda: b.u32_vector(list(e.stride)))])
        return lambda: b.table([("u8", 2), ("ref", tensor)])

    root = b.table([("ref", lambda: b.vector([node_writer(n) for n in graph.nodes])),
                    ("ref", lambda: b.table([("ref", lambda: b.vector([input_writer(e) for e in graph.example_inputs]))]))])
    return b.finish(root)
