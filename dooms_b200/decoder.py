"""Python face of the CUDA decoder: the method set of the reference's MetalLlamaDecoder (src/backend/metal/metal_llama_decoder.h:63-106) and of
load_native_llama (src/pipeline/native_llama.h:22), over the C ABI. Errors come back as DoomsError with the reference's code names."""
from __future__ import annotations

import ctypes as C
import dataclasses
from typing import Callable, Sequence

import numpy as np

from . import _lib as L
from ._lib import DoomsError  # noqa: F401  (re-exported)


@dataclasses.dataclass
class LlamaDecoderConfig:
    n_layer: int = 0
    n_embd: int = 0
    n_head: int = 0
    n_head_kv: int = 0
    head_dim: int = 0
    n_ff: int = 0
    n_vocab: int = 0
    rope_base: float = 0.0
    rope_neox: bool = False
    rms_eps: float = 0.0
    n_ctx: int = 0
    n_batch: int = 0
    spin_wait: bool = True
    prefill_tile: int = 0

    def to_c(self) -> L.LlamaConfig:
        c = L.LlamaConfig()
        c.struct_size = C.sizeof(L.LlamaConfig)
        for f in dataclasses.fields(self):
            setattr(c, f.name, int(getattr(self, f.name)) if f.type in ("bool", "int") else getattr(self, f.name))
        return c

    @staticmethod
    def from_c(c: L.LlamaConfig) -> "LlamaDecoderConfig":
        return LlamaDecoderConfig(c.n_layer, c.n_embd, c.n_head, c.n_head_kv, c.head_dim, c.n_ff, c.n_vocab, c.rope_base, bool(c.rope_neox), c.rms_eps,
                                  c.n_ctx, c.n_batch, bool(c.spin_wait), c.prefill_tile)


def weight_ref(array: np.ndarray | None, dtype: int = L.F32, rows: int = 0, cols: int = 0) -> L.WeightRef:
    """A WeightRef over a numpy array's memory (the caller keeps the array alive until create() returns)."""
    r = L.WeightRef()
    if array is None:
        return r
    r.data = array.ctypes.data
    r.dtype = dtype
    r.rows = rows
    r.cols = cols
    return r


LAYER_FIELDS = [n for n, _ in L.LayerWeights._fields_]


def cuda_options(device: int = 0, tp_rank: int = 0, tp_size: int = 1, nccl_unique_id: bytes | None = None, operand_bf16: bool = False,
                 use_graphs: bool = True, max_sequences: int = 1):
    o = L.CudaOptions()
    o.struct_size = C.sizeof(L.CudaOptions)
    o.device, o.tp_rank, o.tp_size = device, tp_rank, tp_size
    keep = None
    if nccl_unique_id is not None:
        keep = C.create_string_buffer(nccl_unique_id, 128)
        o.nccl_unique_id = C.cast(keep, C.c_void_p)
    path = L.nccl_library_path()
    o.nccl_library = path.encode() if path else None
    o.operand_bf16 = int(operand_bf16)
    o.use_graphs = int(use_graphs)
    o.max_sequences = int(max_sequences)
    return o, keep


def nccl_unique_id() -> bytes:
    buf = C.create_string_buffer(128)
    path = L.nccl_library_path()
    L.check(L.lib().dooms_cuda_nccl_unique_id(path.encode() if path else None, buf))
    return buf.raw


class CudaLlamaDecoder:
    def __init__(self, handle: C.c_void_p):
        self._h = handle

    # ---- construction ----
    @staticmethod
    def load(path: str, n_ctx: int = 2048, n_batch: int = 512, spin_wait: bool = True, prefill_tile: int = 0, **cuda) -> "CudaLlamaDecoder":
        """load_native_llama: GGUF metadata -> config, tensors -> weights, then create."""
        o = L.NativeOptions(C.sizeof(L.NativeOptions), n_ctx, n_batch, int(spin_wait), prefill_tile)
        co, keep = cuda_options(**cuda)
        h = C.c_void_p()
        L.check(L.lib().dooms_cuda_llama_load(str(path).encode(), C.byref(o), C.byref(co), C.byref(h)))
        del keep
        return CudaLlamaDecoder(h)

    @staticmethod
    def create(config: LlamaDecoderConfig, token_embd: L.WeightRef, output_norm: L.WeightRef, output: L.WeightRef, layers: Sequence[dict],
               **cuda) -> "CudaLlamaDecoder":
        """create(config, weights): layers is a list of {field name of LlamaLayerWeights: WeightRef}."""
        arr = (L.LayerWeights * max(1, len(layers)))()
        for i, lw in enumerate(layers):
            for name, ref in lw.items():
                setattr(arr[i], name, ref)
        w = L.LlamaWeights()
        w.struct_size = C.sizeof(L.LlamaWeights)
        w.token_embd, w.output_norm, w.output = token_embd, output_norm, output
        w.layers = C.cast(arr, C.POINTER(L.LayerWeights))
        w.n_layers = len(layers)
        c = config.to_c()
        co, keep = cuda_options(**cuda)
        h = C.c_void_p()
        L.check(L.lib().dooms_cuda_llama_create(C.byref(c), C.byref(w), C.byref(co), C.byref(h)))
        del keep
        return CudaLlamaDecoder(h)

    def close(self):
        if self._h:
            L.lib().dooms_cuda_llama_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ---- the reference's method set ----
    def config(self) -> LlamaDecoderConfig:
        c = L.LlamaConfig()
        L.check(L.lib().dooms_cuda_llama_config(self._h, C.byref(c)))
        return LlamaDecoderConfig.from_c(c)

    def position(self) -> int:
        return L.lib().dooms_cuda_llama_position(self._h)

    def reset(self) -> None:
        L.check(L.lib().dooms_cuda_llama_reset(self._h))

    def eval_tokens(self, tokens: Sequence[int]) -> None:
        a = np.ascontiguousarray(np.asarray(tokens, dtype=np.int32))
        L.check(L.lib().dooms_cuda_llama_eval_tokens(self._h, a.ctypes.data_as(C.POINTER(C.c_int32)), a.size))

    def eval_embeddings(self, embeddings: np.ndarray | None, n: int | None = None) -> None:
        if embeddings is None:
            L.check(L.lib().dooms_cuda_llama_eval_embeddings(self._h, None, n or 0))
            return
        a = np.ascontiguousarray(embeddings, dtype=np.float32)
        L.check(L.lib().dooms_cuda_llama_eval_embeddings(self._h, a.ctypes.data_as(C.POINTER(C.c_float)), a.shape[0] if n is None else n))

    def embed_tokens(self, tokens: Sequence[int]) -> np.ndarray:
        """The tokens' rows of the embedding table as float32 [n][n_embd]."""
        a = np.ascontiguousarray(np.asarray(tokens, dtype=np.int32))
        out = np.empty((a.size, self.config().n_embd), dtype=np.float32)
        L.check(L.lib().dooms_cuda_llama_embed_tokens(self._h, a.ctypes.data, a.size, out.ctypes.data))
        return out

    def pending_token(self) -> int:
        v = C.c_int32()
        L.check(L.lib().dooms_cuda_llama_pending_token(self._h, C.byref(v)))
        return v.value

    def logits(self) -> np.ndarray:
        n = self.config().n_vocab
        out = np.empty(n, dtype=np.float32)
        L.check(L.lib().dooms_cuda_llama_logits(self._h, out.ctypes.data_as(C.POINTER(C.c_float)), n))
        return out

    def generate(self, max_tokens: int, depth: int, on_token: Callable[[int], bool]) -> None:
        err = []

        def cb(tok, _user):
            try:
                return 1 if on_token(tok) else 0
            except BaseException as e:   # never unwind through C
                err.append(e)
                return 0
        L.check(L.lib().dooms_cuda_llama_generate(self._h, max_tokens, depth, L.TOKEN_CALLBACK(cb), None))
        if err:
            raise err[0]

    # ---- several sequences on one decoder (include/dooms_cuda.h: dooms_cuda_llama_select_sequence / _decode_batch) ----
    def max_sequences(self) -> int:
        return L.lib().dooms_cuda_llama_max_sequences(self._h)

    def max_batch_rows(self) -> int:
        return L.lib().dooms_cuda_llama_max_batch_rows(self._h)

    def select_sequence(self, slot: int) -> None:
        L.check(L.lib().dooms_cuda_llama_select_sequence(self._h, slot))

    def decode_batch(self, slots: Sequence[int], steps: int = 1) -> np.ndarray:
        """`steps` greedy steps for the listed KV-cache slots at once (-1: an idle row); the tokens as int32 [steps][len(slots)]."""
        a = np.ascontiguousarray(np.asarray(slots, dtype=np.int32))
        out = np.empty((steps, a.size), dtype=np.int32)
        L.check(L.lib().dooms_cuda_llama_decode_batch(self._h, a.ctypes.data, a.size, steps, out.ctypes.data))
        return out

    def profile_pass(self, rows: int = 1) -> list[dict]:
        arr = (L.KernelTime * 32)()
        n = C.c_int32()
        L.check(L.lib().dooms_cuda_llama_profile_pass(self._h, rows, arr, 32, C.byref(n)))
        return [{"kind": arr[i].kind.decode(), "dispatches": arr[i].dispatches, "gpu_ms": arr[i].gpu_ms} for i in range(n.value)]

    def timings(self) -> dict:
        t = L.Timings()
        t.struct_size = C.sizeof(L.Timings)
        L.check(L.lib().dooms_cuda_llama_timings(self._h, C.byref(t)))
        return {n: getattr(t, n) for n, _ in L.Timings._fields_ if n != "struct_size"}
