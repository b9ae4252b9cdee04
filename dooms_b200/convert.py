"""GGUF conversions for the decoder. fuse_qkv: the attention q / k / v projections of every layer as one `blk.N.attn_qkv.weight` (rows q, then k, then
v) and, where the model has them, their biases as one `blk.N.attn_qkv.bias`: the file layout the loader reads when it is there
(src/pipeline/native_llama.cpp:75-88; the reference's converter is tools/convert/fuse_qkv_gguf.py, which stops at models with biases). Block formats
are fused as bytes: rows are whole blocks, so stacking rows is concatenating their bytes.

    python -m dooms_b200.convert fuse-qkv IN.gguf OUT.gguf
"""
from __future__ import annotations

import argparse
import re

import numpy as np

from . import _lib as L
from .gguf_io import GgufWriter

_GGML_TO_DTYPE = {v: k for k, v in L.GGML_TYPE_ID.items()}


def _metadata(reader) -> dict:
    """The file's metadata as the writer takes it (scalars, strings, integer arrays); the format's own bookkeeping keys are left to the writer."""
    out = {}
    for key, field in reader.fields.items():
        if key.startswith("GGUF.") or key == "general.alignment":
            continue
        value = field.contents()
        if isinstance(value, (np.integer,)):
            value = int(value)
        elif isinstance(value, (np.floating,)):
            value = float(value)
        elif isinstance(value, (np.bool_,)):
            value = bool(value)
        elif isinstance(value, (list, tuple)):
            value = [int(v) for v in value]
        out[key] = value
    return out


def fuse_qkv(src: str, dst: str) -> int:
    """Writes dst as src with fused attention projections (and biases); returns the number of layers fused. Layers whose q, k and v differ in type, or
    that are fused already, are copied as they are."""
    from gguf import GGUFReader
    r = GGUFReader(str(src))
    by_name = {t.name: t for t in r.tensors}

    def entry(name, tensors):
        first = tensors[0]
        dtype = _GGML_TO_DTYPE[int(first.tensor_type)]
        shape = [int(d) for d in reversed(first.shape)]            # outermost first
        shape[0] = sum(int(t.shape[-1]) for t in tensors) if len(shape) > 1 else sum(int(t.shape[0]) for t in tensors)
        return (name, dtype, shape, lambda: np.concatenate([np.ascontiguousarray(t.data).view(np.uint8).reshape(-1) for t in tensors]))

    out, fused, skip = [], 0, set()
    for t in r.tensors:
        if t.name in skip:
            continue
        m = re.fullmatch(r"(blk\.\d+)\.attn_q\.(weight|bias)", t.name)
        if m:
            parts = [by_name.get(f"{m.group(1)}.attn_{x}.{m.group(2)}") for x in "qkv"]
            weights = [by_name.get(f"{m.group(1)}.attn_{x}.weight") for x in "qkv"]
            fusable = all(w is not None for w in weights) and len({int(w.tensor_type) for w in weights}) == 1      # biases follow their matrices
            if fusable and all(p is not None for p in parts) and len({int(p.tensor_type) for p in parts}) == 1:
                out.append(entry(f"{m.group(1)}.attn_qkv.{m.group(2)}", parts))
                skip.update(p.name for p in parts)
                fused += m.group(2) == "weight"
                continue
        out.append(entry(t.name, [t]))
    GgufWriter().write(dst, _metadata(r), out)
    return fused


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="what", required=True)
    f = sub.add_parser("fuse-qkv")
    f.add_argument("src")
    f.add_argument("dst")
    a = ap.parse_args(argv)
    print(f"fused q / k / v of {fuse_qkv(a.src, a.dst)} layers: {a.src} -> {a.dst}")


if __name__ == "__main__":
    main()
