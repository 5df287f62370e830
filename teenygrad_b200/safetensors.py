"""Reading (memory-mapped) and writing the safetensors format, and Qwen3 checkpoints laid out the Hugging Face way.

The reference reads weights the same way: ``SafeTensors::from_pretrained`` maps the file and hands out tensor views
(utilities/teeny-data/src/safetensors/mod.rs:28-46); parameters are then matched by name and uploaded
(drivers/teeny-cuda/src/model/mod.rs:449-476).  A file is an 8-byte little-endian header length, a JSON header
``{name: {"dtype", "shape", "data_offsets": [begin, end]}, "__metadata__": {...}}`` and the raw little-endian tensor bytes.

``SafeTensors`` is a read-only mapping name -> torch tensor over one file, several shard files or a checkpoint
directory (``model.safetensors`` or ``model.safetensors.index.json`` + shards).  Tensors are views of the mapping, so
``Qwen3Runner.load_state_dict(SafeTensors(path))`` touches only the rows its tensor-parallel rank keeps of the
column-parallel weights, one layer at a time.
"""
import json
import os
import struct
from collections.abc import Mapping

import numpy as np
import torch

# safetensors dtype -> (numpy dtype of the mapped bytes, torch dtype of the view)
_DTYPES = {
    "BF16": (np.uint16, torch.bfloat16), "F16": (np.float16, torch.float16), "F32": (np.float32, torch.float32),
    "F64": (np.float64, torch.float64), "I64": (np.int64, torch.int64), "I32": (np.int32, torch.int32),
    "I16": (np.int16, torch.int16), "I8": (np.int8, torch.int8), "U8": (np.uint8, torch.uint8),
    "BOOL": (np.uint8, torch.bool),
    # the two FP8 encodings of the format (what the reference's quantiser writes its float-quantized weights as)
    "F8_E4M3": (np.uint8, torch.float8_e4m3fn), "F8_E5M2": (np.uint8, torch.float8_e5m2),
}
_NAMES = {v[1]: k for k, v in _DTYPES.items()}


def read_header(path):
    """(header dict without ``__metadata__``, metadata dict, offset of the data section)."""
    with open(path, "rb") as f:
        raw = f.read(8)
        if len(raw) != 8:
            raise ValueError(f"{path}: not a safetensors file (shorter than its length field)")
        (n,) = struct.unpack("<Q", raw)
        size = os.path.getsize(path)
        if n > size - 8 or n > (100 << 20):
            raise ValueError(f"{path}: header length {n} does not fit the file")
        header = json.loads(f.read(n).decode("utf-8"))
    meta = header.pop("__metadata__", {}) or {}
    for name, info in header.items():
        b, e = info["data_offsets"]
        if info["dtype"] not in _DTYPES:
            raise ValueError(f"{path}: tensor {name} has unsupported dtype {info['dtype']}")
        count = int(np.prod(info["shape"], dtype=np.int64)) if info["shape"] else 1
        if not (0 <= b <= e <= size - 8 - n) or e - b != count * np.dtype(_DTYPES[info["dtype"]][0]).itemsize:
            raise ValueError(f"{path}: tensor {name} has inconsistent offsets {b}..{e} for shape {info['shape']}")
    return header, meta, 8 + n


class SafeTensors(Mapping):
    """Read-only ``name -> tensor`` over memory-mapped safetensors files."""

    def __init__(self, *sources):
        paths = []
        for src in sources:
            src = os.fspath(src)
            if os.path.isdir(src):
                index = os.path.join(src, "model.safetensors.index.json")
                if os.path.exists(index):
                    with open(index) as f:
                        shards = sorted(set(json.load(f)["weight_map"].values()))
                    paths += [os.path.join(src, s) for s in shards]
                else:
                    paths.append(os.path.join(src, "model.safetensors"))
            else:
                paths.append(src)
        if not paths:
            raise ValueError("no safetensors file given")
        self._where = {}  # name -> (file number, info)
        self._maps, self._data0, self.metadata = [], [], {}
        for i, path in enumerate(paths):
            header, meta, data0 = read_header(path)
            self.metadata.update(meta)
            # copy-on-write mapping: pages stay shared with the file unless somebody writes into a view
            self._maps.append(np.memmap(path, dtype=np.uint8, mode="c"))
            self._data0.append(data0)
            for name, info in header.items():
                if name in self._where:
                    raise ValueError(f"tensor {name} appears in more than one file")
                self._where[name] = (i, info)

    def __len__(self):
        return len(self._where)

    def __iter__(self):
        return iter(self._where)

    def __getitem__(self, name):
        i, info = self._where[name]
        np_dtype, torch_dtype = _DTYPES[info["dtype"]]
        b, e = info["data_offsets"]
        raw = self._maps[i][self._data0[i] + b:self._data0[i] + e]
        t = torch.from_numpy(raw.view(np_dtype) if e > b else np.empty(0, dtype=np_dtype))
        if torch_dtype in (torch.bfloat16, torch.bool, torch.float8_e4m3fn, torch.float8_e5m2):
            t = t.view(torch_dtype)
        return t.view(*info["shape"]) if info["shape"] else t.view(())


def save_file(tensors, path, metadata=None):
    """Writes ``tensors`` (name -> CPU torch tensor) as one safetensors file, names in sorted order, 8-byte aligned."""
    header, blobs, offset = {}, [], 0
    for name in sorted(tensors):
        t = tensors[name].detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise ValueError(f"{name}: dtype {t.dtype} has no safetensors name")
        raw = t.view(torch.uint16).numpy().tobytes() if t.dtype == torch.bfloat16 else (
            t.view(torch.uint8).numpy().tobytes() if t.dtype in (torch.bool, torch.float8_e4m3fn, torch.float8_e5m2)
            else t.numpy().tobytes())
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + len(raw)]}
        blobs.append(raw)
        offset += len(raw)
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    js = json.dumps(header, separators=(",", ":")).encode("utf-8")
    js += b" " * (-len(js) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(js)))
        f.write(js)
        for raw in blobs:
            f.write(raw)


def save_sharded(tensors, directory, max_shard_bytes):
    """Writes a Hugging Face style sharded checkpoint: ``model-0000i-of-0000n.safetensors`` + the index file."""
    os.makedirs(directory, exist_ok=True)
    groups, cur, cur_bytes = [], {}, 0
    for name in sorted(tensors):
        nbytes = tensors[name].numel() * tensors[name].element_size()
        if cur and cur_bytes + nbytes > max_shard_bytes:
            groups.append(cur)
            cur, cur_bytes = {}, 0
        cur[name] = tensors[name]
        cur_bytes += nbytes
    if cur:
        groups.append(cur)
    weight_map, total = {}, 0
    for i, g in enumerate(groups):
        fname = f"model-{i + 1:05d}-of-{len(groups):05d}.safetensors"
        save_file(g, os.path.join(directory, fname), {"format": "pt"})
        for name, t in g.items():
            weight_map[name] = fname
            total += t.numel() * t.element_size()
    with open(os.path.join(directory, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {"total_size": total}, "weight_map": weight_map}, f, indent=1)
    return [os.path.join(directory, n) for n in sorted(set(weight_map.values()))]
