"""Writes tests/golden/qwen3_fx_{prefill,decode}.json.gz from the reference's traced Qwen3 graphs.

    python tests/golden/make_fx_golden.py /path/to/teenygrad

Reads ``support/teeny-torch/tests/data/qwen3_1.bin.gz`` (prefill trace) and ``qwen3_2.bin.gz`` (decode-step trace) with
``teenygrad_b200.fxgraph.read_graph`` and stores the decoded node lists as JSON, so the lowering tests run where the
reference checkout is absent.  Memory addresses inside function reprs ("at 0x...") are dropped: they carry nothing.
"""
import gzip
import json
import os
import re
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from teenygrad_b200 import fxgraph  # noqa: E402


def normalised(graph):
    for n in graph.nodes:
        n.target = re.sub(r" at 0x[0-9a-f]+", "", n.target)
    return graph


def main(ref_root):
    data = os.path.join(ref_root, "support", "teeny-torch", "tests", "data")
    for src, dst in (("qwen3_1.bin.gz", "qwen3_fx_prefill.json.gz"), ("qwen3_2.bin.gz", "qwen3_fx_decode.json.gz")):
        g = normalised(fxgraph.read_graph(os.path.join(data, src)))
        blob = json.dumps(fxgraph.graph_to_json(g), separators=(",", ":")).encode()
        with gzip.GzipFile(os.path.join(HERE, dst), "wb", mtime=0) as f:
            f.write(blob)
        print(dst, len(g.nodes), "nodes", os.path.getsize(os.path.join(HERE, dst)), "bytes")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    main(sys.argv[1])
