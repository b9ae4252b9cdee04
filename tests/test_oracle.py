"""Pins the CPU checker (oracle/oracle.c) before anything trusts it: committed golden vectors made by independent implementations (tests/golden/
make_golden.py), hand-worked block patterns, gguf-py's dequantize, and the reference's own argmax and block tables where its sources were compiled."""
import hashlib
from pathlib import Path

import numpy as np
import pytest

from dooms_b200 import _lib as L
from dooms_b200 import synth
from dooms_b200.quantize import quantize
from oracle import binding as ob

from helpers import K_PROMPT, QUANT_PLANS, oracle_greedy, rel_l2, tiny_f16, write

GOLDEN = Path(__file__).resolve().parent / "golden"
QUANT = [L.Q4_0, L.Q5_0, L.Q8_0, L.Q4_K, L.Q6_K]


@pytest.mark.parametrize("dtype", QUANT)
def test_dequantize_matches_the_golden_vectors(dtype):
    g = np.load(GOLDEN / f"dequant_{L.DTYPE_NAMES[dtype]}.npz")
    blocks, want = g["blocks"], g["values"]
    assert int(g["block_elems"]) == L.BLOCK_ELEMS[dtype] and int(g["block_bytes"]) == L.BLOCK_BYTES[dtype]
    got = ob.dequantize(dtype, blocks, blocks.shape[0] * L.BLOCK_ELEMS[dtype]).reshape(want.shape)
    same = (got.view(np.uint32) == want.view(np.uint32)) | (np.isnan(got) & np.isnan(want))
    assert same.all()


def test_dequantize_hand_worked_blocks():
    """Values worked out from the formulas (src/backend/metal/llama_kernels.h:1014-1018, 1046-1050, 1076-1079)."""
    half = lambda v: list(np.array([v], dtype=np.float16).view(np.uint8))
    # q4_0: d = 0.5, qs[0] = 0x1F -> element 0 = (15 - 8) * 0.5, element 16 = (1 - 8) * 0.5; the rest 0x88 -> 0
    b = np.array(half(0.5) + [0x1F] + [0x88] * 15, dtype=np.uint8)
    v = ob.dequantize(L.Q4_0, b, 32)
    assert v[0] == 3.5 and v[16] == -3.5 and np.all(v[1:16] == 0) and np.all(v[17:] == 0)
    # q5_0: d = 2, qh bit 0 and bit 16 set, qs[0] = 0x00 -> element 0 = (16 - 16) * 2 = 0, element 16 = 0; element 1 = (0 - 16) * 2
    b = np.array(half(2.0) + [0x01, 0x00, 0x01, 0x00] + [0x00] * 16, dtype=np.uint8)
    v = ob.dequantize(L.Q5_0, b, 32)
    assert v[0] == 0 and v[16] == 0 and v[1] == -32 and v[17] == -32
    # q8_0: d = 0.25, q = -128 and 127
    b = np.array(half(0.25) + [0x80, 0x7F] + [0] * 30, dtype=np.uint8)
    v = ob.dequantize(L.Q8_0, b, 32)
    assert v[0] == -32 and v[1] == 31.75 and np.all(v[2:] == 0)
    # q4_K: d = 1, dmin = 0.5; sub-block 0 scale 3 min 2, sub-block 5 scale 63 min 63 (6-bit values split over two bytes)
    scales = [0] * 12
    scales[0], scales[4] = 3, 2
    scales[1] |= (63 >> 4) << 6          # high 2 bits of sub-block 5's scale
    scales[5] |= (63 >> 4) << 6          # high 2 bits of its min
    scales[9] = (63 & 15) | ((63 & 15) << 4)
    qs = [0] * 128
    qs[0] = 0x07                          # sub-block 0 element 0 = 7
    qs[64 + 3] = 0x90                     # sub-block 5 (high nibbles of bytes 64..95) element 3 = 9
    b = np.array(half(1.0) + half(0.5) + scales + qs, dtype=np.uint8)
    v = ob.dequantize(L.Q4_K, b, 256)
    assert v[0] == 1 * 3 * 7 - 0.5 * 2 and v[1] == -1.0 and v[5 * 32 + 3] == 63 * 9 - 0.5 * 63 and v[5 * 32] == -31.5
    # q6_K: d = 0.5, scale of sub-block 0 = -3, element 0 = 0b110101 = 53 -> 0.5 * -3 * (53 - 32)
    ql, qh, sc = [0] * 128, [0] * 64, [0] * 16
    ql[0], qh[0], sc[0] = 0x05, 0x03, 0xFD
    b = np.array(ql + qh + sc + half(0.5), dtype=np.uint8)
    v = ob.dequantize(L.Q6_K, b, 256)
    assert v[0] == 0.5 * -3 * 21 and v[1] == 0.5 * -3 * -32 and v[16] == 0


@pytest.mark.parametrize("dtype", QUANT)
def test_dequantize_matches_gguf_py_on_quantized_normal_weights(dtype):
    gguf = pytest.importorskip("gguf")
    x = np.random.default_rng(dtype).standard_normal((4, 1024)).astype(np.float32) * 0.02
    import torch
    blocks = quantize(dtype, torch.from_numpy(x)).numpy()
    gt = {L.Q4_0: gguf.GGMLQuantizationType.Q4_0, L.Q5_0: gguf.GGMLQuantizationType.Q5_0, L.Q8_0: gguf.GGMLQuantizationType.Q8_0,
          L.Q4_K: gguf.GGMLQuantizationType.Q4_K, L.Q6_K: gguf.GGMLQuantizationType.Q6_K}[dtype]
    want = gguf.quants.dequantize(blocks, gt).astype(np.float32)
    got = np.stack([ob.dequantize(dtype, blocks[r], 1024) for r in range(4)])
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    assert np.abs(got - x).max() < 0.02 * 0.6          # and the quantizers are sane: error well under one standard deviation
    if dtype in (L.Q4_0, L.Q5_0, L.Q8_0):               # these follow ggml's reference quantizers bit for bit
        assert np.array_equal(gguf.quants.quantize(x, gt), blocks)


def test_argmax_rules():
    """tests/unit/test_argmax.cpp:23-74: first index on ties, NaN never wins, all-NaN gives 0."""
    assert ob.argmax(np.array([1, 3, 3, 2], dtype=np.float32)) == 1
    assert ob.argmax(np.array([np.nan, 1, 2], dtype=np.float32)) == 2
    assert ob.argmax(np.array([2, np.nan, 1], dtype=np.float32)) == 0
    assert ob.argmax(np.array([np.nan, np.nan], dtype=np.float32)) == 0
    v = np.random.default_rng(0).standard_normal(151936).astype(np.float32)
    assert ob.argmax(v) == int(np.argmax(v))
    ref = ob.reference_reader()
    if ref is not None:          # the reference's own host argmax, compiled from its sources
        for case in (v, np.array([1, 3, 3, 2], dtype=np.float32), np.array([np.nan, 1, 2], dtype=np.float32), np.array([np.nan, np.nan], dtype=np.float32)):
            assert ref.ref_argmax_f32(case.ctypes.data, case.size) == ob.argmax(case)


def test_block_tables_match_the_reference():
    """Quant sizing (tests/unit/test_gguf.cpp:401-416; src/core/dtype.cpp:19-29)."""
    want = {"q4_0": (32, 18), "q5_0": (32, 22), "q8_0": (32, 34), "q4_k": (256, 144), "q6_k": (256, 210), "f16": (1, 2), "f32": (1, 4)}
    lib = L.lib()
    for dt, name in enumerate(L.DTYPE_NAMES):
        if name in want:
            assert (lib.dooms_dtype_block_elems(dt), lib.dooms_dtype_block_bytes(dt)) == want[name] == (L.BLOCK_ELEMS[dt], L.BLOCK_BYTES[dt])
            assert lib.dooms_dtype_name(dt).decode() == name
    ref = ob.reference_reader()
    if ref is not None:
        for name, (e, b) in want.items():
            assert (ref.ref_block_elems(name.encode()), ref.ref_block_bytes(name.encode())) == (e, b)


@pytest.mark.parametrize("name", ["llama_f16", "qwen_f16", "mix", "q4_0", "q4_K"])
def test_decoder_matches_the_golden_logits(model_dir, name):
    g = np.load(GOLDEN / f"decoder_{name}.npz")
    spec = {"llama_f16": tiny_f16(), "qwen_f16": tiny_f16(qwen=True), "mix": synth.tiny_spec(QUANT_PLANS["Q4_K_M-like mix"]),
            "q4_0": synth.tiny_spec(QUANT_PLANS["q4_0"]), "q4_K": synth.tiny_spec(QUANT_PLANS["q4_K"])}[name]
    path = write(model_dir, "golden_" + name, spec, int(g["seed"]))
    assert hashlib.sha256(open(path, "rb").read()).hexdigest() == str(g["sha256"])      # the generator still writes the same bytes
    o = ob.OracleDecoder(path, 64)
    logits = o.eval_tokens(g["prompt"])
    assert rel_l2(logits, g["logits"]) < 1e-12
    assert oracle_greedy(o, logits, 8) == list(g["greedy"])
    # one token per call and all at once are the same computation
    o2 = ob.OracleDecoder(path, 64)
    for t in g["prompt"]:
        last = o2.eval_tokens([int(t)])
    assert np.array_equal(last, logits)
    # the f32 variant used as the timed CPU baseline stays close to the checker
    fast = ob.OracleDecoder(path, 64, fast=True)
    assert rel_l2(fast.eval_tokens(g["prompt"]), logits) < 5e-4          # f32 sums; a key or value landing on the other side of an f16 rounding boundary costs ~1e-4


def test_operand_rounding_variant_stays_within_the_batched_tolerance(model_dir):
    """The checker's variant that rounds the prefill operands to f16 like the reference's tiles (llama_kernels.h:186-199) sits within the reference's 3e-3."""
    path = write(model_dir, "golden_mix", synth.tiny_spec(QUANT_PLANS["Q4_K_M-like mix"]), 11)
    exact = ob.OracleDecoder(path, 64).eval_tokens(K_PROMPT)
    rounded = ob.OracleDecoder(path, 64, round_operands=True).eval_tokens(K_PROMPT)
    err = rel_l2(rounded, exact)
    assert 0 < err < 3e-3


def test_oracle_refuses_overflow_and_bad_tokens(model_dir):
    path = write(model_dir, "golden_q4_0", synth.tiny_spec(QUANT_PLANS["q4_0"]), 11)
    o = ob.OracleDecoder(path, 8)
    with pytest.raises(ValueError):
        o.eval_tokens([1] * 9)
    with pytest.raises(ValueError):
        o.eval_tokens([50])
    o.eval_tokens([1] * 8)
    assert o.position() == 8


# ---- the reference's own CPU decoder class, compiled from the reference's test file (oracle/_ref/libref_decoder.so) ----
REFERENCE_CASES = {
    # make_tiny's variants (tests/unit/test_metal_llama_decoder.cpp:57-82): llama and qwen2 blocks, head_dim 16 and 64
    "llama_f16": lambda: tiny_f16(), "qwen_f16": lambda: tiny_f16(qwen=True), "llama_f16_hd64": lambda: tiny_f16(head_dim=64), "qwen_f16_hd64": lambda: tiny_f16(qwen=True, head_dim=64),
    # random blocks with power-of-two scales, every value exact in f16 (random_quant, :226-254), each format alone and the Q4_K_M-like plan (:390)
    **{name: (lambda plan=plan: synth.tiny_spec(plan, random_blocks=True)) for name, plan in QUANT_PLANS.items()},
}


@pytest.mark.parametrize("name", sorted(REFERENCE_CASES))
def test_checker_matches_the_reference_class(model_dir, name):
    """oracle.c against `Reference` (tests/unit/test_metal_llama_decoder.cpp:110-192) itself, built from the reference's source: the prompt's logits position by
    position and eight free-running greedy tokens, as the reference's own tests drive it (:322-350). Both compute in double; they differ only in the order
    of the sums."""
    if ob.reference_decoder_lib() is None:
        pytest.skip("oracle/_ref/libref_decoder.so is not built (the reference's sources are needed to build it)")
    path = write(model_dir, "refclass_" + name.replace(" ", "_"), REFERENCE_CASES[name](), 23)
    ref = ob.ReferenceDecoder(path)
    assert ref.exact, "the model's weights are not exactly representable in f16: Reference would see other weights than the checker"
    o = ob.OracleDecoder(path, 64)
    for t in K_PROMPT:
        want = ref.eval_tokens([t])
        got = o.eval_tokens([t])
        assert rel_l2(got, want) < 1e-12
    tok_ref, tok_o = [], []
    for _ in range(8):
        t = int(np.argmax(want))          # the reference test's argmax (std::max_element: first maximum)
        assert ob.argmax(got) == t
        tok_ref.append(t)
        want, got = ref.eval_tokens([t]), o.eval_tokens([t])
        assert rel_l2(got, want) < 1e-12
    # the whole prompt in one call is the same computation in the checker
    o2 = ob.OracleDecoder(path, 64)
    ref.reset()
    assert rel_l2(o2.eval_tokens(K_PROMPT), ref.eval_tokens(K_PROMPT)) < 1e-12
    # embeddings: Reference::embedding and the checker's row lookup agree exactly
    assert np.array_equal(ref.embedding(7), o.embedding(7).astype(np.float64))


@pytest.mark.parametrize("name,round_operands", [("llama_f16", False), ("qwen_f16", False), ("Q4_K_M-like mix", False), ("Q4_K_M-like mix", True), ("q4_0", True)])
def test_streaming_checker_matches_the_checker(model_dir, name, round_operands):
    """The layer-at-a-time restatement used at the configurations' real sizes (oracle/streaming.py) against oracle.c: a prompt in one call, single
    positions after it, with and without the prefill tiles' operand rounding. Both run in double; only the order of the sums differs."""
    from oracle.streaming import StreamingOracle
    spec = {"llama_f16": tiny_f16(), "qwen_f16": tiny_f16(qwen=True)}.get(name) or synth.tiny_spec(QUANT_PLANS[name])
    path = write(model_dir, "stream_" + name.replace(" ", "_"), spec, 31)
    prompt = [(i * 13 + 5) % 50 for i in range(45)]          # the reference's long-prompt recipe (test_metal_llama_decoder.cpp:440)
    o = ob.OracleDecoder(path, 64, round_operands=round_operands)
    s = StreamingOracle(path, 64, round_operands=round_operands)
    want, got = o.eval_tokens(prompt), s.eval_tokens(prompt)
    # a sum that lands on the other side of an f16 rounding boundary moves one operand by an ulp: far below every tolerance in use, but not 1e-12
    assert rel_l2(got, want) < (1e-5 if round_operands else 1e-11)
    for t in (7, 7, 31):
        want, got = o.eval_tokens([t]), s.eval_tokens([t])
        assert rel_l2(got, want) < (1e-5 if round_operands else 1e-11)
        assert ob.argmax(got) == ob.argmax(want)
