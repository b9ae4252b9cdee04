"""Generates the committed golden vectors of tests/golden (run from the repository root: python tests/golden/make_golden.py).

Two independent sources pin the CPU checker (oracle/oracle.c):
  dequant_<type>.npz   random block bytes and their values as gguf-py's `dequantize` computes them (the GGUF project's own numpy implementation of ggml's
                       dequantize_row_*), plus the block sizes.
  decoder_<name>.npz   logits of a tiny seeded model after the reference test's 11-token prompt and its greedy continuation, from the plain numpy
                       float64 decoder in this file: the Llama definition written out as in the reference's test `Reference` class
                       (tests/unit/test_metal_llama_decoder.cpp:110-192), weights dequantized by gguf-py. It shares no code with oracle.c.
The model files themselves are not stored: they are regenerated from (spec, seed) by dooms_b200.synth, whose bytes are pinned by the sha256 recorded here.
"""
from __future__ import annotations

import hashlib
import sys
import tempfile
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

from gguf import GGMLQuantizationType as T  # noqa: E402
from gguf import GGUFReader, quants  # noqa: E402

from dooms_b200 import _lib as L  # noqa: E402
from dooms_b200 import synth  # noqa: E402

HERE = Path(__file__).resolve().parent
GG = {L.F32: T.F32, L.F16: T.F16, L.Q4_0: T.Q4_0, L.Q5_0: T.Q5_0, L.Q8_0: T.Q8_0, L.Q4_K: T.Q4_K, L.Q6_K: T.Q6_K}
K_PROMPT = [3, 17, 42, 8, 8, 21, 0, 49, 12, 30, 5]


def random_blocks(dtype: int, nb: int, seed: int) -> np.ndarray:
    g = np.random.default_rng(seed)
    b = g.integers(0, 256, (nb, L.BLOCK_BYTES[dtype]), dtype=np.uint8)
    for off in {L.Q4_0: [0], L.Q5_0: [0], L.Q8_0: [0], L.Q4_K: [0, 2], L.Q6_K: [208]}[dtype]:
        scale = (g.standard_normal(nb) * 0.01).astype(np.float16)
        b[:, off:off + 2] = scale.view(np.uint8).reshape(nb, 2)
    # edge blocks: all-zero quants, all-ones quants, zero scale, negative scale, the largest finite scale
    b[0, :] = 0
    b[1, :] = 0xFF
    for off in {L.Q4_0: [0], L.Q5_0: [0], L.Q8_0: [0], L.Q4_K: [0, 2], L.Q6_K: [208]}[dtype]:
        b[1, off:off + 2] = np.array([1.0], dtype=np.float16).view(np.uint8)
        b[2, off:off + 2] = np.array([0.0], dtype=np.float16).view(np.uint8)
        b[3, off:off + 2] = np.array([-0.25], dtype=np.float16).view(np.uint8)
        b[4, off:off + 2] = np.array([65504.0], dtype=np.float16).view(np.uint8)
    return b


class NumpyDecoder:
    """float64 llama / qwen2 decoder, one position at a time."""

    def __init__(self, path: str):
        r = GGUFReader(path)

        def scalar(key):
            f = r.fields[key]
            return f.parts[f.data[0]][0]
        arch = bytes(r.fields["general.architecture"].parts[r.fields["general.architecture"].data[0]]).decode()
        p = arch + "."
        self.neox = arch == "qwen2"
        self.n_layer = int(scalar(p + "block_count"))
        self.E = int(scalar(p + "embedding_length"))
        self.nh = int(scalar(p + "attention.head_count"))
        self.nkv = int(scalar(p + "attention.head_count_kv"))
        self.hd = self.E // self.nh
        self.base = float(scalar(p + "rope.freq_base"))
        self.eps = float(np.float32(scalar(p + "attention.layer_norm_rms_epsilon")))
        self.t = {}
        for t in r.tensors:
            shape = [int(d) for d in reversed(t.shape)]
            self.t[t.name] = quants.dequantize(t.data, t.tensor_type).astype(np.float64).reshape(shape)
        if "output.weight" not in self.t:
            self.t["output.weight"] = self.t["token_embd.weight"]
        self.k = [[] for _ in range(self.n_layer)]
        self.v = [[] for _ in range(self.n_layer)]

    def rms(self, x, g):
        return x / np.sqrt((x * x).mean() + self.eps) * g

    def rope(self, v, pos):
        hd = self.hd
        i = np.arange(hd // 2)
        th = pos * np.power(self.base, -2.0 * i / hd)
        i0, i1 = (i, i + hd // 2) if self.neox else (2 * i, 2 * i + 1)
        a, b = v[i0].copy(), v[i1].copy()
        v[i0] = a * np.cos(th) - b * np.sin(th)
        v[i1] = a * np.sin(th) + b * np.cos(th)

    def step(self, x):
        t, hd, nh, nkv = self.t, self.hd, self.nh, self.nkv
        Q, KV = nh * hd, nkv * hd
        pos = len(self.k[0])
        for l in range(self.n_layer):
            b = f"blk.{l}."
            xn = self.rms(x, t[b + "attn_norm.weight"])
            q, k, v = t[b + "attn_q.weight"] @ xn, t[b + "attn_k.weight"] @ xn, t[b + "attn_v.weight"] @ xn
            if b + "attn_q.bias" in t:
                q, k, v = q + t[b + "attn_q.bias"], k + t[b + "attn_k.bias"], v + t[b + "attn_v.bias"]
            for h in range(nh):
                self.rope(q[h * hd:(h + 1) * hd], pos)
            for h in range(nkv):
                self.rope(k[h * hd:(h + 1) * hd], pos)
            self.k[l].append(k.astype(np.float32).astype(np.float16).astype(np.float64))     # the cache is f16
            self.v[l].append(v.astype(np.float32).astype(np.float16).astype(np.float64))
            K, V = np.stack(self.k[l]), np.stack(self.v[l])
            att = np.empty(Q)
            for h in range(nh):
                kv = h // (nh // nkv)
                s = K[:, kv * hd:(kv + 1) * hd] @ q[h * hd:(h + 1) * hd] / np.sqrt(float(hd))
                pr = np.exp(s - s.max())
                att[h * hd:(h + 1) * hd] = (pr / pr.sum()) @ V[:, kv * hd:(kv + 1) * hd]
            x = x + t[b + "attn_output.weight"] @ att
            fn = self.rms(x, t[b + "ffn_norm.weight"])
            g, u = t[b + "ffn_gate.weight"] @ fn, t[b + "ffn_up.weight"] @ fn
            x = x + t[b + "ffn_down.weight"] @ (g / (1 + np.exp(-g)) * u)
        return t["output.weight"] @ self.rms(x, t["output_norm.weight"])

    def token(self, tok):
        return self.step(self.t["token_embd.weight"][tok].copy())


def main():
    for dt in (L.Q4_0, L.Q5_0, L.Q8_0, L.Q4_K, L.Q6_K):
        blocks = random_blocks(dt, 12, 100 + dt)
        with np.errstate(over="ignore", invalid="ignore"):
            values = quants.dequantize(blocks, GG[dt]).astype(np.float32)
        np.savez_compressed(HERE / f"dequant_{L.DTYPE_NAMES[dt]}.npz", blocks=blocks, values=values, block_elems=L.BLOCK_ELEMS[dt], block_bytes=L.BLOCK_BYTES[dt])

    from helpers import QUANT_PLANS, tiny_f16
    cases = {"llama_f16": (tiny_f16(), 1), "qwen_f16": (tiny_f16(qwen=True), 4), "mix": (synth.tiny_spec(QUANT_PLANS["Q4_K_M-like mix"]), 11),
             "q4_0": (synth.tiny_spec(QUANT_PLANS["q4_0"]), 11), "q4_K": (synth.tiny_spec(QUANT_PLANS["q4_K"]), 11)}
    for name, (spec, seed) in cases.items():
        with tempfile.TemporaryDirectory() as d:
            path = str(Path(d) / "m.gguf")
            synth.write_model(spec, path, seed)
            sha = hashlib.sha256(open(path, "rb").read()).hexdigest()
            dec = NumpyDecoder(path)
            for tok in K_PROMPT:
                logits = dec.token(tok)
            prompt_logits = logits.copy()
            greedy = []
            tok = int(np.argmax(logits))
            for _ in range(8):
                greedy.append(tok)
                logits = dec.token(tok)
                tok = int(np.argmax(logits))
        np.savez_compressed(HERE / f"decoder_{name}.npz", prompt=np.array(K_PROMPT, dtype=np.int32), logits=prompt_logits, greedy=np.array(greedy, dtype=np.int32),
                            seed=seed, sha256=sha)
        print(name, sha[:12], greedy)


if __name__ == "__main__":
    main()
