"""Files with fused attention projections (`blk.N.attn_qkv.weight`, the reference's tools/convert/fuse_qkv_gguf.py layout, here also with fused biases): the
converter keeps every other tensor and all metadata, both GGUF readers agree on the result, the checker computes the same logits from either file, and
on the GPU the decoder gives the same bits from the fused file as from the file it was made from."""
import numpy as np
import pytest

from dooms_b200 import CudaLlamaDecoder, convert, synth
from dooms_b200 import _lib as L
from dooms_b200.gguf_io import GgufFile
from oracle import binding as ob

from helpers import K_PROMPT, QUANT_PLANS, collect, oracle_greedy, rel_l2, tiny_f16, write

CASES = {"llama_q4_0": lambda: synth.tiny_spec(QUANT_PLANS["q4_0"], arch="llama"), "qwen_q4_K_biases": lambda: synth.tiny_spec(QUANT_PLANS["q4_K"]),
         "qwen_f16_biases": lambda: tiny_f16(qwen=True), "mix_not_fusable": lambda: synth.tiny_spec(QUANT_PLANS["Q4_K_M-like mix"])}


def pair(model_dir, name):
    src = write(model_dir, "fuse_src_" + name, CASES[name](), 17)
    dst = str(model_dir / f"fuse_dst_{name}.gguf")
    return src, dst, convert.fuse_qkv(src, dst)


@pytest.mark.parametrize("name", sorted(CASES))
def test_converter_fuses_what_can_be_fused(model_dir, name):
    src, dst, n = pair(model_dir, name)
    a, b = GgufFile(src), GgufFile(dst)
    ta, tb = {t["name"]: t for t in a.tensors()}, {t["name"]: t for t in b.tensors()}
    if name == "mix_not_fusable":          # q / k are q5_0 and v q8_0 there: nothing to fuse, the file is copied
        assert n == 0 and set(ta) == set(tb)
    else:
        assert n == 2 and "blk.0.attn_qkv.weight" in tb and "blk.0.attn_q.weight" not in tb
        q, k, v = (ta[f"blk.1.attn_{x}.weight"] for x in "qkv")
        f = tb["blk.1.attn_qkv.weight"]
        assert f["shape"] == [q["shape"][0] + k["shape"][0] + v["shape"][0], q["shape"][1]] and f["dtype"] == q["dtype"]
        assert np.array_equal(b.tensor_bytes("blk.1.attn_qkv.weight"), np.concatenate([a.tensor_bytes(f"blk.1.attn_{x}.weight") for x in "qkv"]))
        assert ("blk.0.attn_qkv.bias" in tb) == ("blk.0.attn_q.bias" in ta)
    for key in ("general.architecture",):
        assert a.get_string(key) == b.get_string(key)
    arch = a.get_string("general.architecture")
    for key in ("block_count", "embedding_length", "attention.head_count", "attention.head_count_kv", "feed_forward_length", "context_length"):
        assert a.get_uint(f"{arch}.{key}") == b.get_uint(f"{arch}.{key}")
    assert a.get_float(f"{arch}.rope.freq_base") == b.get_float(f"{arch}.rope.freq_base")
    ref = ob.reference_reader()
    if ref is not None:                    # the reference's own reader takes the converted file as well
        code, parsed = ob.reference_parse(open(dst, "rb").read())
        assert code == 0 and len(parsed["tensors"]) == len(tb)
    # the checker computes the same logits from either layout
    want = ob.OracleDecoder(src, 64).eval_tokens(K_PROMPT)
    got = ob.OracleDecoder(dst, 64).eval_tokens(K_PROMPT)
    assert np.array_equal(want, got)


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["llama_q4_0", "qwen_q4_K_biases", "qwen_f16_biases"])
def test_decoder_runs_fused_files_bit_for_bit_like_their_sources(model_dir, name):
    src, dst, _ = pair(model_dir, name)
    o = ob.OracleDecoder(dst, 128)
    want = o.eval_tokens(K_PROMPT)
    results = []
    for path in (src, dst):
        dec = CudaLlamaDecoder.load(path, 128, 64)
        dec.eval_tokens(K_PROMPT)
        one_call = dec.logits()
        dec.reset()
        for t in K_PROMPT:
            dec.eval_tokens([t])
        single = dec.logits()
        tokens = collect(dec, 10, 2)
        results.append((one_call, single, tokens))
        dec.close()
    assert np.array_equal(results[0][0], results[1][0]) and np.array_equal(results[0][1], results[1][1]) and results[0][2] == results[1][2]
    assert rel_l2(results[1][1], want) < 1e-4
    assert results[1][2] == oracle_greedy(o, want, 10)
