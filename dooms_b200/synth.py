"""Synthetic llama / qwen2 GGUF models: the benchmark configurations' shapes and quantization plans with seeded random weights.

Stands in for the public checkpoints the reference benchmarks (none of their weights are used): matrices are drawn N(0, 0.02) and quantized per tensor
plan, norm gains U(0.7, 1.3), q/k/v biases N(0, 0.02), as the reference's tests draw theirs (tests/unit/test_metal_llama_decoder.cpp:41-53). Each tensor
has its own seed (base seed, tensor index), so a tensor's bytes do not depend on which others were generated. Small models draw from numpy's PCG64; with
device="cuda" the draws come from torch's CUDA generator instead (fast enough for 8B / 32B shapes; a different but equally seeded stream).
"""
from __future__ import annotations

import dataclasses
from pathlib import Path
from typing import Callable

import numpy as np
import torch

from . import _lib as L
from .gguf_io import GgufWriter
from .quantize import quantize


@dataclasses.dataclass
class ModelSpec:
    name: str
    arch: str                # "llama" or "qwen2"
    n_layer: int
    n_embd: int
    n_head: int
    n_head_kv: int
    n_ff: int
    n_vocab: int
    rope_base: float
    rms_eps: float
    context_length: int
    tied: bool
    bias: bool
    plan: Callable[[str, int], int]      # (tensor kind, layer) -> dtype; kinds: token_embd, output, attn_q, attn_k, attn_v, attn_output, ffn_gate, ffn_up, ffn_down
    random_blocks: bool = False          # quantized matrices as random block bytes with power-of-two scales (every value exact in f16), see random_blocks()
    weight_std: float = 0.02
    embd_std: float = 0.02
    bias_std: float = 0.02

    @property
    def head_dim(self) -> int:
        return self.n_embd // self.n_head

    def matrices(self):
        """(gguf name, kind, layer, rows, cols) of every weight matrix, in file order."""
        E, F, V = self.n_embd, self.n_ff, self.n_vocab
        Q, KV = self.n_head * self.head_dim, self.n_head_kv * self.head_dim
        out = [("token_embd.weight", "token_embd", -1, V, E)]
        if not self.tied:
            out.append(("output.weight", "output", -1, V, E))
        for l in range(self.n_layer):
            b = f"blk.{l}."
            out += [(b + "attn_q.weight", "attn_q", l, Q, E), (b + "attn_k.weight", "attn_k", l, KV, E), (b + "attn_v.weight", "attn_v", l, KV, E),
                    (b + "attn_output.weight", "attn_output", l, E, Q), (b + "ffn_gate.weight", "ffn_gate", l, F, E), (b + "ffn_up.weight", "ffn_up", l, F, E),
                    (b + "ffn_down.weight", "ffn_down", l, E, F)]
        return out

    def matrix_bytes(self) -> int:
        """Bytes of weight matrices a decode step reads: every layer matrix plus the output matrix (the tied table when there is no separate one)."""
        total = 0
        for name, kind, l, rows, cols in self.matrices():
            if kind == "token_embd" and not self.tied:
                continue
            dt = self.plan(kind, l)
            total += rows * cols // L.BLOCK_ELEMS[dt] * L.BLOCK_BYTES[dt]
        return total


def pure(dtype: int):
    return lambda kind, layer: dtype


def q4_k_m_small(kind: str, layer: int) -> int:
    """The Q4_K_M-style mix on rows of 896 elements, which are not whole 256-element super-blocks: llama-quantize's fallback types there, as the reference
    describes them (metal_llama_decoder.mm:83 "Q4_K_M files mix q5_0 and q8_0 there"; test plan at tests/unit/test_metal_llama_decoder.cpp:390)."""
    even = layer % 2 == 0
    return {"token_embd": L.Q8_0, "output": L.Q8_0, "attn_q": L.Q5_0, "attn_k": L.Q5_0, "attn_v": L.Q8_0 if even else L.Q5_0, "attn_output": L.Q5_0,
            "ffn_gate": L.Q5_0, "ffn_up": L.Q5_0, "ffn_down": L.Q6_K if even else L.Q4_K}[kind]


def q4_k_m_large(kind: str, layer: int) -> int:
    """Q4_K everywhere; Q6_K for the output / token table and for attn_v and ffn_down in even layers."""
    if kind in ("token_embd", "output"):
        return L.Q6_K
    if kind in ("attn_v", "ffn_down") and layer % 2 == 0:
        return L.Q6_K
    return L.Q4_K


def config_spec(index: int) -> ModelSpec:
    """The benchmark configurations 0-3 (4 reuses the model of 0)."""
    if index in (0, 4):
        return ModelSpec("qwen2.5-0.5b-arch-q4_0", "qwen2", 24, 896, 14, 2, 4864, 151936, 1e6, 1e-6, 32768, True, True, pure(L.Q4_0))
    if index == 1:
        return ModelSpec("qwen2.5-0.5b-arch-q4_k_m", "qwen2", 24, 896, 14, 2, 4864, 151936, 1e6, 1e-6, 32768, True, True, q4_k_m_small)
    if index == 2:
        return ModelSpec("llama-3-8b-arch-q4_0", "llama", 32, 4096, 32, 8, 14336, 128256, 5e5, 1e-5, 8192, False, False, pure(L.Q4_0))
    if index == 3:
        return ModelSpec("qwen2.5-32b-arch-q4_k_m", "qwen2", 64, 5120, 40, 8, 27648, 152064, 1e6, 1e-6, 32768, False, True, q4_k_m_large)
    raise ValueError(index)


def tiny_spec(dtype_plan, arch: str = "qwen2", n_embd: int = 256, n_head: int = 4, n_head_kv: int = 2, n_ff: int = 2304, n_vocab: int = 50, n_layer: int = 2,
              context_length: int = 1024, tied: bool = False, random_blocks: bool = False) -> ModelSpec:
    """The shape of the reference's quantized test model (tests/unit/test_metal_llama_decoder.cpp:279-285): E 256, 4 / 2 heads of 64, F 2304, V 50."""
    return ModelSpec("tiny", arch, n_layer, n_embd, n_head, n_head_kv, n_ff, n_vocab, 10000.0, 1e-5, context_length, tied, arch == "qwen2", dtype_plan,
                     random_blocks=random_blocks, weight_std=0.15, embd_std=1.0, bias_std=0.3)


def random_blocks(dtype: int, rows: int, cols: int, seed: int) -> np.ndarray:
    """Random block bytes with power-of-two scales sized for weights of std ~0.14, so that every dequantized value is exact in f16: the reference test's
    random_quant (tests/unit/test_metal_llama_decoder.cpp:226-254). With such weights a half-rounded operand tile loses nothing on the weight side."""
    g = np.random.Generator(np.random.PCG64(seed))
    nb = rows * cols // L.BLOCK_ELEMS[dtype]
    b = g.integers(0, 256, (nb, L.BLOCK_BYTES[dtype]), dtype=np.uint8)

    def put_half(off, value):
        b[:, off:off + 2] = np.array([value], dtype=np.float16).view(np.uint8)
    if dtype == L.Q4_0:
        put_half(0, 1 / 32)
    elif dtype == L.Q5_0:
        put_half(0, 1 / 64)
    elif dtype == L.Q8_0:
        put_half(0, 1 / 512)
    elif dtype == L.Q4_K:
        put_half(0, 1 / 1024)
        put_half(2, 1 / 1024)
    elif dtype == L.Q6_K:
        b[:, 192:208] = g.integers(-63, 64, (nb, 16)).astype(np.int8).view(np.uint8)      # |scale| <= 63: |scale * q| < 2048, exact in f16
        put_half(208, 1 / 4096)
    else:
        raise ValueError(dtype)
    return b.reshape(rows, -1)


_CHAT_FAMILIES = {
    # family: (control tokens, end-of-turn token, a Jinja template of that family: this library looks only for the family's markers in it)
    "chatml": (["<|im_start|>", "<|im_end|>"], "<|im_end|>",
               "{% for message in messages %}{{'<|im_start|>' + message['role'] + '\n' + message['content'] + '<|im_end|>' + '\n'}}{% endfor %}"
               "{% if add_generation_prompt %}{{ '<|im_start|>assistant\n' }}{% endif %}"),
    "llama3": (["<|start_header_id|>", "<|end_header_id|>", "<|eot_id|>"], "<|eot_id|>",
               "{% for message in messages %}{{ '<|start_header_id|>' + message['role'] + '<|end_header_id|>\n\n' + message['content'] | trim + '<|eot_id|>' }}{% endfor %}"
               "{% if add_generation_prompt %}{{ '<|start_header_id|>assistant<|end_header_id|>\n\n' }}{% endif %}"),
    "smolvlm": (["<|im_start|>", "<end_of_utterance>"], "<end_of_utterance>",
                "<|im_start|>{% for message in messages %}{{ message['role'] | capitalize + ': ' + message['content'] + '<end_of_utterance>\n' }}{% endfor %}"
                "{% if add_generation_prompt %}{{ 'Assistant:' }}{% endif %}"),
    "other": ([], None, "{% for message in messages %}{{ '[TURN] ' + message['content'] }}{% endfor %}"),
}


def byte_level_vocab(n_vocab: int, chat: str | None = None) -> dict:
    """Tokenizer metadata of a small byte-level BPE vocabulary with n_vocab (>= 270) entries: the 256 byte tokens in the byte alphabet of such
    vocabularies, a few merges of common English pairs, filler tokens, and an end-of-text token as the last id. chat ("chatml", "llama3", "smolvlm", "other"): with
    that family's control tokens in the ids just below the last one, its end-of-turn token as tokenizer.ggml.eot_token_id and a tokenizer.chat_template."""
    printable = [b for b in range(256) if 0x21 <= b <= 0x7E or 0xA1 <= b <= 0xAC or 0xAE <= b <= 0xFF]
    to_cp, nxt = {}, 256
    for b in range(256):
        if b in printable:
            to_cp[b] = b
        else:
            to_cp[b] = nxt
            nxt += 1
    sym = lambda text: "".join(chr(to_cp[b]) for b in text.encode())
    tokens = [chr(to_cp[b]) for b in range(256)]
    merges = []
    for left, right in (("h", "e"), ("l", "l"), ("he", "ll"), ("hell", "o"), (" ", "w"), ("o", "r"), (" w", "or"), (" wor", "l"), (" worl", "d"), ("t", "h"), (" ", "th"),
                        ("S", "T"), ("O", "P")):
        merges.append(f"{sym(left)} {sym(right)}")
        tokens.append(sym(left) + sym(right))
    assert n_vocab >= len(tokens) + 1
    while len(tokens) < n_vocab - 1:
        tokens.append(f"<filler_{len(tokens)}>")
    tokens.append("<|endoftext|>")
    types = [1] * (n_vocab - 1) + [3]
    md = {"tokenizer.ggml.model": "gpt2", "tokenizer.ggml.tokens": tokens, "tokenizer.ggml.merges": merges, "tokenizer.ggml.token_type": types,
          "tokenizer.ggml.eos_token_id": n_vocab - 1, "tokenizer.ggml.bos_token_id": n_vocab - 1, "tokenizer.ggml.add_bos_token": False}
    if chat is not None:
        control, end_of_turn, template = _CHAT_FAMILIES[chat]
        for i, name in enumerate(control):
            at = n_vocab - 1 - len(control) + i
            tokens[at], types[at] = name, 3
            if name == end_of_turn:
                md["tokenizer.ggml.eot_token_id"] = at
        md["tokenizer.chat_template"] = template
    return md


def sentencepiece_vocab(n_vocab: int) -> dict:
    """Tokenizer metadata of a small sentencepiece-style vocabulary with n_vocab (>= 300) entries: <unk>, <s>, </s>, the 256 byte tokens <0xHH>, single
    characters, a few pieces of common English with scores (longer pieces score higher, as trained vocabularies have it), filler tokens."""
    sp = "\u2581"
    tokens, scores, types = ["<unk>", "<s>", "</s>"], [0.0, 0.0, 0.0], [2, 3, 3]
    for b in range(256):
        tokens.append(f"<0x{b:02X}>"); scores.append(0.0); types.append(6)
    for ch in [sp] + list("abcdefghijklmnopqrstuvwxyz,.!"):
        tokens.append(ch); scores.append(-10.0); types.append(1)
    for piece, score in ((sp + "h", -6.0), ("he", -5.5), ("ll", -5.0), (sp + "he", -4.5), ("llo", -4.0), (sp + "hello", -1.0), ("hell", -3.8), (sp + "w", -6.0), ("or", -5.0),
                         ("ld", -5.2), (sp + "wor", -3.0), (sp + "world", -1.5), (sp + "t", -6.1), ("th", -4.9), (sp + "th", -3.5), (sp + "the", -2.0)):
        tokens.append(piece); scores.append(score); types.append(1)
    assert n_vocab >= len(tokens)
    while len(tokens) < n_vocab:
        tokens.append(f"<filler_{len(tokens)}>"); scores.append(-100.0); types.append(1)
    return {"tokenizer.ggml.model": "llama", "tokenizer.ggml.tokens": tokens, "tokenizer.ggml.scores": scores, "tokenizer.ggml.token_type": types,
            "tokenizer.ggml.bos_token_id": 1, "tokenizer.ggml.eos_token_id": 2, "tokenizer.ggml.add_bos_token": True}


def _normal(shape, std: float, seed: int, device: str) -> torch.Tensor:
    if device == "cpu":
        g = np.random.Generator(np.random.PCG64(seed))
        return torch.from_numpy(g.standard_normal(shape, dtype=np.float32) * np.float32(std))
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    return torch.randn(shape, generator=gen, device=device, dtype=torch.float32) * std


def write_model(spec: ModelSpec, path: str | Path, seed: int, device: str = "cpu", vocab=False) -> dict:
    """Writes the model as a GGUF file; returns {"matrix_bytes": ...}. vocab: True with the tokenizer metadata of byte_level_vocab(n_vocab),
    "sentencepiece" with that of sentencepiece_vocab(n_vocab), "chatml" / "llama3" / "smolvlm" / "other" with byte_level_vocab(n_vocab, chat=...)."""
    md = {
        "general.architecture": spec.arch,
        "general.name": spec.name,
        f"{spec.arch}.block_count": spec.n_layer,
        f"{spec.arch}.embedding_length": spec.n_embd,
        f"{spec.arch}.attention.head_count": spec.n_head,
        f"{spec.arch}.attention.head_count_kv": spec.n_head_kv,
        f"{spec.arch}.feed_forward_length": spec.n_ff,
        f"{spec.arch}.context_length": spec.context_length,
        f"{spec.arch}.rope.freq_base": float(spec.rope_base),
        f"{spec.arch}.attention.layer_norm_rms_epsilon": float(spec.rms_eps),
    }
    if vocab:
        md.update(sentencepiece_vocab(spec.n_vocab) if vocab == "sentencepiece" else byte_level_vocab(spec.n_vocab, chat=vocab if isinstance(vocab, str) else None))
    tensors = []
    counter = [0]

    def next_seed() -> int:
        counter[0] += 1
        return seed * 1_000_003 + counter[0]

    def matrix(kind, layer, rows, cols):
        s = next_seed()
        dt = spec.plan(kind, layer)
        std = spec.embd_std if kind == "token_embd" else spec.weight_std

        def produce():
            if spec.random_blocks and dt != L.F16:
                return random_blocks(dt, rows, cols, s)
            out = []
            step = max(1, (1 << 26) // cols)          # 64M elements at a time
            for r0 in range(0, rows, step):
                r1 = min(rows, r0 + step)
                out.append(quantize(dt, _normal((r1 - r0, cols), std, s * 131 + r0, device)).cpu().numpy())
            return np.concatenate(out, axis=0)
        return dt, produce

    def vector(n, kind):
        s = next_seed()

        def produce():
            g = np.random.Generator(np.random.PCG64(s))
            if kind == "norm":
                return g.uniform(0.7, 1.3, n).astype(np.float32)
            return (g.standard_normal(n, dtype=np.float32) * np.float32(spec.bias_std)).astype(np.float32)
        return produce

    E = spec.n_embd
    Q, KV = spec.n_head * spec.head_dim, spec.n_head_kv * spec.head_dim
    for name, kind, layer, rows, cols in spec.matrices():
        if kind == "attn_q":
            tensors.append((f"blk.{layer}.attn_norm.weight", L.F32, [E], vector(E, "norm")))
        if kind == "ffn_gate":
            tensors.append((f"blk.{layer}.ffn_norm.weight", L.F32, [E], vector(E, "norm")))
        dt, produce = matrix(kind, layer, rows, cols)
        tensors.append((name, dt, [rows, cols], produce))
        if spec.bias and kind in ("attn_q", "attn_k", "attn_v"):
            tensors.append((name.replace(".weight", ".bias"), L.F32, [rows], vector(rows, "bias")))
        if kind == "token_embd":
            tensors.append(("output_norm.weight", L.F32, [E], vector(E, "norm")))
    GgufWriter().write(path, md, tensors)
    return {"matrix_bytes": spec.matrix_bytes()}


def prompt_tokens(n: int, n_vocab: int, seed: int) -> np.ndarray:
    """n seeded uniform token ids in [0, n_vocab)."""
    g = np.random.Generator(np.random.PCG64(seed))
    return g.integers(0, n_vocab, n, dtype=np.int32)
