"""TEST INFRASTRUCTURE - Python binding of the CPU checker (oracle/oracle.c) and of the reference's own GGUF reader (oracle/_ref).

Only tests, the smoke test and the benchmark's CPU-baseline leg import this. The model file is read with gguf-py (the file format's own package), not with
the product's reader, so the checker shares no parsing code with what it checks.
"""
from __future__ import annotations

import ctypes as C
import json
import subprocess
from pathlib import Path

import numpy as np

from dooms_b200 import _lib as L

HERE = Path(__file__).resolve().parent
ORACLE_SO = HERE / "_build" / "liboracle.so"
REF_SO = HERE / "_ref" / "libref_gguf.so"

_GGML_TO_DTYPE = {v: k for k, v in L.GGML_TYPE_ID.items()}


REF_DECODER_SO = HERE / "_ref" / "libref_decoder.so"


def reference_checkout() -> str:
    """Where the reference's sources lie: $DOOMS_REFERENCE_DIR, else a `reference` directory beside this repository; "" when neither exists."""
    import os
    for cand in (os.environ.get("DOOMS_REFERENCE_DIR"), str(HERE.parent.parent / "reference")):
        if cand and (Path(cand) / "src" / "format").is_dir():
            return cand
    return ""


def build(ref_root: str | None = None) -> None:
    """Builds the checker; with the reference's sources at hand also oracle/_ref (the reference's own reader and its own CPU decoder class)."""
    ref_root = reference_checkout() if ref_root is None else ref_root
    subprocess.run(["make", "-C", str(HERE), "all", f"REF={ref_root}"], check=True, capture_output=True)


_oracle = None


def oracle() -> C.CDLL:
    global _oracle
    if _oracle is None:
        if not ORACLE_SO.exists():
            build()
        o = C.CDLL(str(ORACLE_SO))
        o.oracle_dequantize.argtypes = [C.c_int32, C.c_void_p, C.c_int64, C.c_void_p]
        o.oracle_round_to_half.restype = C.c_float
        o.oracle_round_to_half.argtypes = [C.c_float]
        o.oracle_argmax_f32.restype = C.c_int32
        o.oracle_argmax_f32.argtypes = [C.c_void_p, C.c_int64]
        o.oracle_argmax_f64.restype = C.c_int32
        o.oracle_argmax_f64.argtypes = [C.c_void_p, C.c_int64]
        o.oracle_create.restype = C.c_void_p
        o.oracle_create.argtypes = [C.POINTER(L.LlamaConfig), C.POINTER(L.LlamaWeights)]
        o.oracle_destroy.argtypes = [C.c_void_p]
        o.oracle_reset.argtypes = [C.c_void_p]
        o.oracle_position.restype = C.c_int32
        o.oracle_position.argtypes = [C.c_void_p]
        o.oracle_set_fast.argtypes = [C.c_void_p, C.c_int32]
        o.oracle_set_round_operands.argtypes = [C.c_void_p, C.c_int32]
        o.oracle_set_threads.restype = C.c_int32
        o.oracle_set_threads.argtypes = [C.c_int32]
        o.oracle_eval_embeddings.restype = C.c_int32
        o.oracle_eval_embeddings.argtypes = [C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p]
        o.oracle_eval_tokens.restype = C.c_int32
        o.oracle_eval_tokens.argtypes = [C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p]
        o.oracle_embedding.argtypes = [C.c_void_p, C.c_int32, C.c_void_p]
        _oracle = o
    return _oracle


def set_threads(n: int) -> int:
    """Threads the checker's parallel loops use from now on (0: leave as is); returns the count in effect. torch.distributed.run exports
    OMP_NUM_THREADS=1 to its workers, which would otherwise leave the timed CPU baseline on one core."""
    return int(oracle().oracle_set_threads(int(n)))


def dequantize(dtype: int, blocks: np.ndarray, n: int) -> np.ndarray:
    """n elements of one row of `dtype` blocks -> float32, by the reference's block formulas."""
    blocks = np.ascontiguousarray(blocks).view(np.uint8)
    out = np.empty(n, dtype=np.float32)
    oracle().oracle_dequantize(dtype, blocks.ctypes.data, n, out.ctypes.data)
    return out


def argmax(v: np.ndarray) -> int:
    v = np.ascontiguousarray(v)
    if v.dtype == np.float32:
        return oracle().oracle_argmax_f32(v.ctypes.data, v.size)
    v = v.astype(np.float64)
    return oracle().oracle_argmax_f64(v.ctypes.data, v.size)


def model_structs(path: str, n_ctx: int, n_batch: int = 512):
    """(LlamaConfig, LlamaWeights, keepalive) for a llama / qwen2 GGUF file, tensors pointing into gguf-py's memory map. The mapping from metadata and tensor
    names is the reference loader's (src/pipeline/native_llama.cpp:18-99)."""
    from gguf import GGUFReader
    r = GGUFReader(str(path))
    fields = r.fields

    def scalar(key):
        f = fields[key]
        return f.parts[f.data[0]][0]

    arch = bytes(fields["general.architecture"].parts[fields["general.architecture"].data[0]]).decode()
    p = arch + "."
    c = L.LlamaConfig()
    c.struct_size = C.sizeof(L.LlamaConfig)
    c.n_layer = int(scalar(p + "block_count"))
    c.n_embd = int(scalar(p + "embedding_length"))
    c.n_head = int(scalar(p + "attention.head_count"))
    c.n_head_kv = int(scalar(p + "attention.head_count_kv"))
    c.n_ff = int(scalar(p + "feed_forward_length"))
    c.head_dim = c.n_embd // c.n_head
    c.rope_base = float(scalar(p + "rope.freq_base"))
    c.rms_eps = float(scalar(p + "attention.layer_norm_rms_epsilon"))
    c.rope_neox = 1 if arch == "qwen2" else 0
    c.n_ctx, c.n_batch, c.spin_wait, c.prefill_tile = n_ctx, n_batch, 1, 0
    tensors = {t.name: t for t in r.tensors}

    def ref(name):
        w = L.WeightRef()
        t = tensors.get(name)
        if t is None:
            return w
        w.data = t.data.ctypes.data
        w.dtype = _GGML_TO_DTYPE[int(t.tensor_type)]
        shape = [int(d) for d in reversed(t.shape)]          # gguf-py lists the fastest dimension first
        w.rows, w.cols = (1, shape[0]) if len(shape) == 1 else (shape[0], shape[1])
        return w

    w = L.LlamaWeights()
    w.struct_size = C.sizeof(L.LlamaWeights)
    w.token_embd = ref("token_embd.weight")
    w.output_norm = ref("output_norm.weight")
    w.output = ref("output.weight")
    if not w.output.data:
        w.output = w.token_embd
    c.n_vocab = w.token_embd.rows
    layers = (L.LayerWeights * c.n_layer)()
    for l in range(c.n_layer):
        b = f"blk.{l}."
        for field, name in (("attn_norm", "attn_norm.weight"), ("attn_q", "attn_q.weight"), ("attn_k", "attn_k.weight"), ("attn_v", "attn_v.weight"),
                            ("attn_qkv", "attn_qkv.weight"), ("attn_q_bias", "attn_q.bias"), ("attn_k_bias", "attn_k.bias"), ("attn_v_bias", "attn_v.bias"),
                            ("attn_qkv_bias", "attn_qkv.bias"), ("attn_output", "attn_output.weight"), ("ffn_norm", "ffn_norm.weight"),
                            ("ffn_gate", "ffn_gate.weight"), ("ffn_up", "ffn_up.weight"), ("ffn_down", "ffn_down.weight")):
            setattr(layers[l], field, ref(b + name))
    w.layers = C.cast(layers, C.POINTER(L.LayerWeights))
    w.n_layers = c.n_layer
    return c, w, (r, layers)


class OracleDecoder:
    """The CPU restatement of the decoder over a GGUF file: eval_tokens / eval_embeddings return the last position's logits as float64."""

    def __init__(self, path: str, n_ctx: int, fast: bool = False, round_operands: bool = False):
        self.cfg, self.weights, self._keep = model_structs(path, n_ctx)
        self._h = oracle().oracle_create(C.byref(self.cfg), C.byref(self.weights))
        oracle().oracle_set_fast(self._h, int(fast))
        oracle().oracle_set_round_operands(self._h, int(round_operands))

    def close(self):
        if self._h:
            oracle().oracle_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def reset(self):
        oracle().oracle_reset(self._h)

    def set_round_operands(self, mode: int) -> None:
        """0: exact; 1: calls of several positions round the projections' operands to f16 like the prefill tiles; 2: every call does, the output projection
        included (a decode step that runs several sequences as the rows of one chunk)."""
        oracle().oracle_set_round_operands(self._h, int(mode))

    def position(self) -> int:
        return oracle().oracle_position(self._h)

    def eval_tokens(self, tokens) -> np.ndarray:
        a = np.ascontiguousarray(np.asarray(tokens, dtype=np.int32))
        out = np.empty(self.cfg.n_vocab, dtype=np.float64)
        rc = oracle().oracle_eval_tokens(self._h, a.ctypes.data, a.size, out.ctypes.data)
        if rc != 0:
            raise ValueError(f"oracle_eval_tokens: {rc}")
        return out

    def eval_embeddings(self, emb: np.ndarray) -> np.ndarray:
        a = np.ascontiguousarray(emb, dtype=np.float32)
        out = np.empty(self.cfg.n_vocab, dtype=np.float64)
        rc = oracle().oracle_eval_embeddings(self._h, a.ctypes.data, a.shape[0], out.ctypes.data)
        if rc != 0:
            raise ValueError(f"oracle_eval_embeddings: {rc}")
        return out

    def embedding(self, token: int) -> np.ndarray:
        out = np.empty(self.cfg.n_embd, dtype=np.float32)
        oracle().oracle_embedding(self._h, token, out.ctypes.data)
        return out


# ---- the reference's own CPU decoder class (oracle/_ref/libref_decoder.so), when it was built ----
_ref_decoder = None


def reference_decoder_lib():
    global _ref_decoder
    if _ref_decoder is None and REF_DECODER_SO.exists():
        r = C.CDLL(str(REF_DECODER_SO))
        r.ref_decoder_new.restype = C.c_void_p
        r.ref_decoder_new.argtypes = [C.c_int32] * 7 + [C.c_float, C.c_int32, C.c_float, C.c_void_p, C.c_void_p, C.c_void_p]
        r.ref_decoder_add_layer.argtypes = [C.c_void_p] * 9
        for name in ("ref_decoder_seal", "ref_decoder_reset", "ref_decoder_free"):
            getattr(r, name).argtypes = [C.c_void_p]
        r.ref_decoder_step.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
        r.ref_decoder_embedding.argtypes = [C.c_void_p, C.c_int32, C.c_void_p]
        _ref_decoder = r
    return _ref_decoder


class ReferenceDecoder:
    """The reference test's own `Reference` class (tests/unit/test_metal_llama_decoder.cpp:110-192, compiled from the reference's file) over a GGUF model.
    The class takes f16 matrices: quantized tensors are handed over as the f16 values of their dequantization (by this checker's block formulas, which are
    pinned against gguf-py), exactly what the reference's quantized tests do with ggml's to_float (:226-254); `exact` says whether that conversion lost
    nothing (true for f16 files and for blocks with power-of-two scales)."""

    def __init__(self, path: str):
        lib = reference_decoder_lib()
        if lib is None:
            raise RuntimeError("oracle/_ref/libref_decoder.so is not built (needs the reference's sources: make -C oracle ref REF=...)")
        self._lib = lib
        cfg, w, keep = model_structs(path, 8)
        self.cfg = cfg
        self.exact = True
        self._keep = []

        def matrix(ref) -> np.ndarray:
            n = ref.rows * ref.cols
            nbytes = n // L.BLOCK_ELEMS[ref.dtype] * L.BLOCK_BYTES[ref.dtype]
            raw = np.ctypeslib.as_array(C.cast(ref.data, C.POINTER(C.c_uint8)), shape=(nbytes,))
            f32 = dequantize(ref.dtype, raw, n)
            f16 = f32.astype(np.float16)
            if not np.array_equal(f16.astype(np.float32), f32):
                self.exact = False
            self._keep.append(f16)
            return f16

        def vector(ref) -> np.ndarray:
            raw = np.ctypeslib.as_array(C.cast(ref.data, C.POINTER(C.c_uint8)), shape=(ref.cols * (4 if ref.dtype == L.F32 else 2),))
            v = np.ascontiguousarray(dequantize(ref.dtype, raw, ref.cols), dtype=np.float32)
            self._keep.append(v)
            return v

        embd, out, on = matrix(w.token_embd), matrix(w.output), vector(w.output_norm)
        self._h = lib.ref_decoder_new(cfg.n_layer, cfg.n_embd, cfg.n_head, cfg.n_head_kv, cfg.head_dim, cfg.n_ff, cfg.n_vocab, cfg.rope_base, cfg.rope_neox, cfg.rms_eps,
                                      embd.ctypes.data, out.ctypes.data, on.ctypes.data)
        for l in range(cfg.n_layer):
            lw = w.layers[l]
            qkv = matrix(lw.attn_qkv) if lw.attn_qkv.data else np.concatenate([matrix(lw.attn_q), matrix(lw.attn_k), matrix(lw.attn_v)])
            bias = None
            if lw.attn_qkv_bias.data:
                bias = vector(lw.attn_qkv_bias)
            elif lw.attn_q_bias.data:
                bias = np.concatenate([vector(lw.attn_q_bias), vector(lw.attn_k_bias), vector(lw.attn_v_bias)])
            self._keep += [qkv, bias]
            an, fn = vector(lw.attn_norm), vector(lw.ffn_norm)
            wo, gate, up, down = matrix(lw.attn_output), matrix(lw.ffn_gate), matrix(lw.ffn_up), matrix(lw.ffn_down)
            lib.ref_decoder_add_layer(self._h, an.ctypes.data, fn.ctypes.data, bias.ctypes.data if bias is not None else None, qkv.ctypes.data, wo.ctypes.data,
                                      gate.ctypes.data, up.ctypes.data, down.ctypes.data)
        lib.ref_decoder_seal(self._h)
        del keep

    def close(self):
        if self._h:
            self._lib.ref_decoder_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def reset(self):
        self._lib.ref_decoder_reset(self._h)

    def embedding(self, token: int) -> np.ndarray:
        out = np.empty(self.cfg.n_embd, dtype=np.float64)
        self._lib.ref_decoder_embedding(self._h, int(token), out.ctypes.data)
        return out

    def step(self, x: np.ndarray) -> np.ndarray:
        """One position given as n_embd input values; the logits (Reference::step)."""
        x = np.ascontiguousarray(x, dtype=np.float64)
        out = np.empty(self.cfg.n_vocab, dtype=np.float64)
        self._lib.ref_decoder_step(self._h, x.ctypes.data, out.ctypes.data)
        return out

    def eval_tokens(self, tokens) -> np.ndarray:
        out = None
        for t in tokens:
            out = self.step(self.embedding(int(t)))
        return out


# ---- the reference's own GGUF reader (oracle/_ref), when it was built ----
_ref = None


def reference_reader():
    """The library built from the reference's sources, or None when it is not there (it cannot be rebuilt without the reference checkout)."""
    global _ref
    if _ref is None and REF_SO.exists():
        r = C.CDLL(str(REF_SO))
        r.ref_gguf_parse.restype = C.c_int
        r.ref_gguf_parse.argtypes = [C.c_void_p, C.c_size_t, C.c_char_p, C.c_size_t]
        r.ref_gguf_open.restype = C.c_int
        r.ref_gguf_open.argtypes = [C.c_char_p, C.c_char_p, C.c_size_t]
        r.ref_argmax_f32.restype = C.c_int64
        r.ref_argmax_f32.argtypes = [C.c_void_p, C.c_size_t]
        r.ref_block_elems.restype = C.c_int64
        r.ref_block_elems.argtypes = [C.c_char_p]
        r.ref_block_bytes.restype = C.c_int64
        r.ref_block_bytes.argtypes = [C.c_char_p]
        _ref = r
    return _ref


def reference_parse(data: bytes):
    """(code, parsed dict or error message) from the reference's GgufFile::parse on these bytes."""
    r = reference_reader()
    buf = C.create_string_buffer(1 << 22)
    src = C.create_string_buffer(data, len(data)) if data else None
    code = r.ref_gguf_parse(src, len(data), buf, len(buf))
    text = buf.value.decode("utf-8", "replace")
    return code, (json.loads(text) if code == 0 else text)
