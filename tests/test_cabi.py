"""The C ABI library loads without a GPU and exports exactly what include/dooms_cuda.h declares; argument checks that need no device."""
import ctypes as C
import re
from pathlib import Path

import numpy as np
import pytest

from dooms_b200 import _lib as L
from dooms_b200.decoder import CudaLlamaDecoder, LlamaDecoderConfig, weight_ref

HEADER = Path(__file__).resolve().parent.parent / "include" / "dooms_cuda.h"


def declared_symbols():
    text = HEADER.read_text()
    return sorted(set(re.findall(r"DOOMS_CUDA_API[^;(]*?\b(dooms_\w+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound():
    handle = C.CDLL(str(L.LIB_PATH))
    names = declared_symbols()
    assert len(names) >= 40
    for name in names:
        assert hasattr(handle, name), name
        assert name in L.SIGNATURES, f"{name} has no ctypes signature"
    assert sorted(L.SIGNATURES) == names


def test_struct_layouts_match_the_header_sizes():
    assert C.sizeof(L.WeightRef) == 32 and C.sizeof(L.LayerWeights) == 14 * 32
    assert C.sizeof(L.LlamaConfig) == 8 + 14 * 4
    assert C.sizeof(L.KernelTime) == 24 and C.sizeof(L.GgufTensor) == 72


def test_code_names_are_the_reference_names():
    lib = L.lib()
    assert [lib.dooms_cuda_code_name(i).decode() for i in range(8)] == L.CODE_NAMES


def tiny_weights(n_layer=2, E=64, nh=4, nkv=2, hd=16, F=96, V=50):
    keep = []

    def mat(rows, cols):
        a = np.zeros((rows, cols), dtype=np.float16)
        keep.append(a)
        return weight_ref(a, L.F16, rows, cols)

    def vec(n):
        a = np.ones(n, dtype=np.float32)
        keep.append(a)
        return weight_ref(a, L.F32, 1, n)
    Q, KV = nh * hd, nkv * hd
    layers = [{"attn_norm": vec(E), "attn_q": mat(Q, E), "attn_k": mat(KV, E), "attn_v": mat(KV, E), "attn_output": mat(E, Q), "ffn_norm": vec(E),
               "ffn_gate": mat(F, E), "ffn_up": mat(F, E), "ffn_down": mat(E, F)} for _ in range(n_layer)]
    cfg = LlamaDecoderConfig(n_layer, E, nh, nkv, hd, F, V, 10000.0, False, 1e-5, 32, 8)
    return cfg, mat(V, E), vec(E), mat(V, E), layers, keep


def create_code(cfg, embd, norm, out, layers):
    try:
        CudaLlamaDecoder.create(cfg, embd, norm, out, layers).close()
        return L.OK
    except L.DoomsError as e:
        return e.code


def test_create_validates_before_touching_a_device():
    """The shape and dtype checks of create (metal_llama_decoder.mm:426-494; tests/unit/test_metal_llama_decoder.cpp:594-608) need no GPU."""
    cfg, embd, norm, out, layers, keep = tiny_weights()
    layers[1]["ffn_up"].rows = 95
    assert create_code(cfg, embd, norm, out, layers) == L.INVALID_ARGUMENT
    cfg, embd, norm, out, layers, keep = tiny_weights()
    layers[0]["ffn_down"].dtype = L.F32
    assert create_code(cfg, embd, norm, out, layers) == L.UNSUPPORTED
    cfg, embd, norm, out, layers, keep = tiny_weights()
    assert create_code(cfg, embd, norm, out, layers[:1]) == L.INVALID_ARGUMENT
    cfg, embd, norm, out, layers, keep = tiny_weights()
    cfg.n_head_kv = 3
    assert create_code(cfg, embd, norm, out, layers) == L.INVALID_ARGUMENT
    cfg, embd, norm, out, layers, keep = tiny_weights()
    cfg.head_dim = 24
    assert create_code(cfg, embd, norm, out, layers) == L.UNSUPPORTED
    cfg, embd, norm, out, layers, keep = tiny_weights()
    cfg.prefill_tile = 3
    assert create_code(cfg, embd, norm, out, layers) == L.INVALID_ARGUMENT
    cfg, embd, norm, out, layers, keep = tiny_weights()
    layers[0]["ffn_up"].dtype = L.Q8_0          # gate and up of different types (and 64-wide rows are whole q8_0 blocks)
    assert create_code(cfg, embd, norm, out, layers) == L.UNSUPPORTED
    cfg, embd, norm, out, layers, keep = tiny_weights()
    bias = np.zeros(64, dtype=np.float32)
    layers[0]["attn_q_bias"] = weight_ref(bias, L.F32, 1, 64)          # a bias for q but not k / v
    assert create_code(cfg, embd, norm, out, layers) == L.INVALID_ARGUMENT
    cfg, embd, norm, out, layers, keep = tiny_weights()
    layers[0]["attn_q"].dtype = L.Q4_K          # 64-wide rows are not whole 256-element blocks
    assert create_code(cfg, embd, norm, out, layers) == L.INVALID_ARGUMENT
    # a valid model: without a GPU the only thing left to fail is the device
    cfg, embd, norm, out, layers, keep = tiny_weights()
    if L.lib().dooms_cuda_device_count() == 0:
        assert create_code(cfg, embd, norm, out, layers) == L.UNSUPPORTED


def test_struct_size_zero_is_rejected():
    lib = L.lib()
    cfg = L.LlamaConfig()
    w = L.LlamaWeights()
    w.struct_size = C.sizeof(L.LlamaWeights)
    h = C.c_void_p()
    assert lib.dooms_cuda_llama_create(C.byref(cfg), C.byref(w), None, C.byref(h)) == L.INVALID_ARGUMENT
    assert b"struct_size" in lib.dooms_cuda_last_error()
    assert lib.dooms_cuda_llama_create(None, C.byref(w), None, C.byref(h)) == L.INVALID_ARGUMENT


@pytest.mark.skipif(L.lib().dooms_cuda_device_count() > 0, reason="only meaningful without a GPU")
def test_compute_entry_points_fail_loudly_without_a_device():
    lib = L.lib()
    x = np.zeros(64, dtype=np.float32)
    code = lib.dooms_cuda_rms_norm(x.ctypes.data, x.ctypes.data, x.ctypes.data, 1, 64, 1e-5, None)
    assert code in (L.UNSUPPORTED, L.INTERNAL) and code != L.OK
