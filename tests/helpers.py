"""Shared pieces of the parity tests: model files, error measures, the oracle's greedy continuation."""
from __future__ import annotations

import numpy as np

from dooms_b200 import _lib as L
from dooms_b200 import synth
from oracle import binding as ob

K_PROMPT = [3, 17, 42, 8, 8, 21, 0, 49, 12, 30, 5]     # the reference's kPrompt, tests/unit/test_metal_llama_decoder.cpp:202

F16, Q40, Q50, Q80, Q4K, Q6K = L.F16, L.Q4_0, L.Q5_0, L.Q8_0, L.Q4_K, L.Q6_K


def rel_l2(a: np.ndarray, b: np.ndarray) -> float:
    """sqrt(sum (a-b)^2 / sum b^2), the reference tests' measure (test_metal_llama_decoder.cpp:196-200)."""
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return float(np.sqrt(((a - b) ** 2).sum() / (b ** 2).sum()))


def plan_of(embd, output, q, k, v, wo, gate, down0, down1):
    """A per-tensor type plan in the order of the reference's QuantPlan (test_metal_llama_decoder.cpp:256)."""
    def plan(kind, layer):
        return {"token_embd": embd, "output": output, "attn_q": q, "attn_k": k, "attn_v": v, "attn_output": wo, "ffn_gate": gate, "ffn_up": gate,
                "ffn_down": down0 if layer == 0 else down1}[kind]
    return plan


QUANT_PLANS = {
    "q4_0": plan_of(*[Q40] * 9), "q5_0": plan_of(*[Q50] * 9), "q8_0": plan_of(*[Q80] * 9), "q4_K": plan_of(*[Q4K] * 9), "q6_K": plan_of(*[Q6K] * 9),
    "Q4_K_M-like mix": plan_of(Q80, Q6K, Q50, Q50, Q80, Q50, Q50, Q4K, Q6K),     # test_metal_llama_decoder.cpp:390
}


def tiny_f16(qwen: bool = False, head_dim: int = 16, context_length: int = 1024) -> synth.ModelSpec:
    """make_tiny of the reference's test (test_metal_llama_decoder.cpp:57-82): 2 layers, E 64, 4 / 2 heads, F 96 (2208 for the qwen block), V 50, f16."""
    s = synth.tiny_spec(synth.pure(F16), arch="qwen2" if qwen else "llama", n_embd=4 * head_dim, n_head=4, n_head_kv=2, n_ff=2208 if qwen else 96, n_vocab=50,
                        context_length=context_length)
    return s      # a GGUF file fixes head_dim = E / n_head, so wider heads widen E with them


def write(model_dir, name: str, spec: synth.ModelSpec, seed: int) -> str:
    path = str(model_dir / f"{name}.gguf")
    synth.write_model(spec, path, seed)
    return path


def oracle_greedy(o: ob.OracleDecoder, logits: np.ndarray, n: int) -> list[int]:
    """n tokens of free-running greedy generation, the oracle feeding back its own argmax (test_metal_llama_decoder.cpp:340-346)."""
    out = []
    t = ob.argmax(logits)
    for _ in range(n):
        out.append(t)
        t = ob.argmax(o.eval_tokens([t]))
    return out


def collect(dec, n: int, depth: int) -> list[int]:
    got: list[int] = []
    dec.generate(n, depth, lambda tok: got.append(tok) or True)
    return got
