"""ctypes binding of the C ABI in include/dooms_cuda.h. The library is the product: if it is missing this module raises, there is no fallback."""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "lib" / "libdooms_cuda.so"

OK, INVALID_ARGUMENT, NOT_FOUND, DATA_LOSS, UNSUPPORTED, RESOURCE_EXHAUSTED, IO_ERROR, INTERNAL = range(8)
CODE_NAMES = ["Ok", "InvalidArgument", "NotFound", "DataLoss", "Unsupported", "ResourceExhausted", "IoError", "Internal"]

F32, F16, BF16, I32, Q4_0, Q5_0, Q8_0, Q4_K, Q6_K = range(9)
DTYPE_NAMES = ["f32", "f16", "bf16", "i32", "q4_0", "q5_0", "q8_0", "q4_k", "q6_k"]
BLOCK_ELEMS = [1, 1, 1, 1, 32, 32, 32, 256, 256]
BLOCK_BYTES = [4, 2, 2, 4, 18, 22, 34, 144, 210]
GGML_TYPE_ID = {F32: 0, F16: 1, Q4_0: 2, Q5_0: 6, Q8_0: 8, Q4_K: 12, Q6_K: 14, I32: 26, BF16: 30}


class DoomsError(RuntimeError):
    """A non-OK dooms_code from the library; .code is the numeric code, .code_name the reference's name for it."""

    def __init__(self, code: int, message: str):
        super().__init__(f"{CODE_NAMES[code] if 0 <= code < 8 else code}: {message}")
        self.code = code
        self.code_name = CODE_NAMES[code] if 0 <= code < 8 else str(code)
        self.message = message


class WeightRef(C.Structure):
    _fields_ = [("data", C.c_void_p), ("dtype", C.c_int32), ("rows", C.c_int64), ("cols", C.c_int64)]


class LlamaConfig(C.Structure):
    _fields_ = [("struct_size", C.c_size_t), ("n_layer", C.c_int32), ("n_embd", C.c_int32), ("n_head", C.c_int32), ("n_head_kv", C.c_int32),
                ("head_dim", C.c_int32), ("n_ff", C.c_int32), ("n_vocab", C.c_int32), ("rope_base", C.c_float), ("rope_neox", C.c_int32),
                ("rms_eps", C.c_float), ("n_ctx", C.c_int32), ("n_batch", C.c_int32), ("spin_wait", C.c_int32), ("prefill_tile", C.c_int32)]


class LayerWeights(C.Structure):
    _fields_ = [(n, WeightRef) for n in ("attn_norm", "attn_q", "attn_k", "attn_v", "attn_qkv", "attn_q_bias", "attn_k_bias", "attn_v_bias",
                                         "attn_qkv_bias", "attn_output", "ffn_norm", "ffn_gate", "ffn_up", "ffn_down")]


class LlamaWeights(C.Structure):
    _fields_ = [("struct_size", C.c_size_t), ("token_embd", WeightRef), ("output_norm", WeightRef), ("output", WeightRef),
                ("layers", C.POINTER(LayerWeights)), ("n_layers", C.c_int32)]


class CudaOptions(C.Structure):
    _fields_ = [("struct_size", C.c_size_t), ("device", C.c_int32), ("tp_rank", C.c_int32), ("tp_size", C.c_int32), ("nccl_unique_id", C.c_void_p),
                ("nccl_library", C.c_char_p), ("operand_bf16", C.c_int32), ("use_graphs", C.c_int32), ("max_sequences", C.c_int32)]


class NativeOptions(C.Structure):
    _fields_ = [("struct_size", C.c_size_t), ("n_ctx", C.c_int32), ("n_batch", C.c_int32), ("spin_wait", C.c_int32), ("prefill_tile", C.c_int32)]


class KernelTime(C.Structure):
    _fields_ = [("kind", C.c_char_p), ("dispatches", C.c_int32), ("gpu_ms", C.c_double)]


class Timings(C.Structure):
    _fields_ = [("struct_size", C.c_size_t), ("last_eval_ms", C.c_double), ("last_generate_ms", C.c_double), ("last_eval_launches", C.c_int64),
                ("last_generate_launches", C.c_int64), ("weight_bytes", C.c_int64), ("kv_bytes", C.c_int64), ("last_batch_ms", C.c_double),
                ("last_batch_launches", C.c_int64), ("tp_peer_allreduce", C.c_int64), ("tp_symmetric_window", C.c_int64)]


class LlmOptions(C.Structure):
    _fields_ = [("struct_size", C.c_size_t), ("n_ctx", C.c_int32), ("n_batch", C.c_int32), ("queue_depth", C.c_int32), ("device", C.c_int32)]


class Sampling(C.Structure):
    _fields_ = [("struct_size", C.c_size_t), ("temperature", C.c_float), ("top_k", C.c_int32), ("top_p", C.c_float), ("repeat_penalty", C.c_float), ("seed", C.c_uint32)]


class ChatMessage(C.Structure):
    _fields_ = [("role", C.c_char_p), ("content", C.c_char_p)]


class GenerationInfo(C.Structure):
    _fields_ = [("struct_size", C.c_size_t), ("prompt_tokens", C.c_int32), ("completion_tokens", C.c_int32), ("finish_reason", C.c_int32),
                ("prefill_ms", C.c_double), ("first_token_ms", C.c_double), ("decode_ms", C.c_double)]


TEXT_CALLBACK = C.CFUNCTYPE(C.c_int32, C.c_char_p, C.c_void_p)
FINISH_NONE, FINISH_STOP, FINISH_LENGTH, FINISH_CANCELLED = 0, 1, 2, 3


class GgufTensor(C.Structure):
    _fields_ = [("name", C.c_char_p), ("dtype", C.c_int32), ("rank", C.c_int32), ("shape", C.c_int64 * 4), ("offset", C.c_uint64),
                ("nbytes", C.c_uint64), ("data", C.c_void_p)]


class TpShare(C.Structure):
    _fields_ = [("struct_size", C.c_size_t)] + [(n, C.c_int64) for n in ("q_row0", "q_rows", "kv_row0", "kv_rows", "ff_row0", "ff_rows", "vocab_row0", "vocab_rows",
                                                                      "attn_col0", "attn_cols")]


TOKEN_CALLBACK = C.CFUNCTYPE(C.c_int32, C.c_int32, C.c_void_p)

# name -> (restype, argtypes); every symbol include/dooms_cuda.h declares
SIGNATURES = {
    "dooms_cuda_last_error": (C.c_char_p, []),
    "dooms_cuda_code_name": (C.c_char_p, [C.c_int32]),
    "dooms_cuda_device_count": (C.c_int32, []),
    "dooms_dtype_block_elems": (C.c_int64, [C.c_int32]),
    "dooms_dtype_block_bytes": (C.c_int64, [C.c_int32]),
    "dooms_dtype_bytes": (C.c_int32, [C.c_int32, C.c_int64, C.POINTER(C.c_uint64)]),
    "dooms_dtype_name": (C.c_char_p, [C.c_int32]),
    "dooms_gguf_open": (C.c_int32, [C.c_char_p, C.POINTER(C.c_void_p)]),
    "dooms_gguf_parse": (C.c_int32, [C.c_void_p, C.c_size_t, C.POINTER(C.c_void_p)]),
    "dooms_gguf_close": (None, [C.c_void_p]),
    "dooms_gguf_version": (C.c_uint32, [C.c_void_p]),
    "dooms_gguf_alignment": (C.c_uint64, [C.c_void_p]),
    "dooms_gguf_tensor_count": (C.c_int64, [C.c_void_p]),
    "dooms_gguf_tensor_at": (C.c_int32, [C.c_void_p, C.c_int64, C.POINTER(GgufTensor)]),
    "dooms_gguf_find_tensor": (C.c_int32, [C.c_void_p, C.c_char_p, C.POINTER(GgufTensor)]),
    "dooms_gguf_get_string": (C.c_int32, [C.c_void_p, C.c_char_p, C.POINTER(C.c_char_p)]),
    "dooms_gguf_get_uint": (C.c_int32, [C.c_void_p, C.c_char_p, C.POINTER(C.c_uint64)]),
    "dooms_gguf_get_int": (C.c_int32, [C.c_void_p, C.c_char_p, C.POINTER(C.c_int64)]),
    "dooms_gguf_get_float": (C.c_int32, [C.c_void_p, C.c_char_p, C.POINTER(C.c_double)]),
    "dooms_gguf_get_bool": (C.c_int32, [C.c_void_p, C.c_char_p, C.POINTER(C.c_int32)]),
    "dooms_cuda_llama_create": (C.c_int32, [C.POINTER(LlamaConfig), C.POINTER(LlamaWeights), C.POINTER(CudaOptions), C.POINTER(C.c_void_p)]),
    "dooms_cuda_llama_load": (C.c_int32, [C.c_char_p, C.POINTER(NativeOptions), C.POINTER(CudaOptions), C.POINTER(C.c_void_p)]),
    "dooms_cuda_llama_destroy": (None, [C.c_void_p]),
    "dooms_cuda_llama_config": (C.c_int32, [C.c_void_p, C.POINTER(LlamaConfig)]),
    "dooms_cuda_llama_position": (C.c_int32, [C.c_void_p]),
    "dooms_cuda_llama_reset": (C.c_int32, [C.c_void_p]),
    "dooms_cuda_llama_eval_tokens": (C.c_int32, [C.c_void_p, C.POINTER(C.c_int32), C.c_int32]),
    "dooms_cuda_llama_eval_embeddings": (C.c_int32, [C.c_void_p, C.POINTER(C.c_float), C.c_int32]),
    "dooms_cuda_llama_pending_token": (C.c_int32, [C.c_void_p, C.POINTER(C.c_int32)]),
    "dooms_cuda_llama_logits": (C.c_int32, [C.c_void_p, C.POINTER(C.c_float), C.c_int64]),
    "dooms_cuda_llama_generate": (C.c_int32, [C.c_void_p, C.c_int32, C.c_int32, TOKEN_CALLBACK, C.c_void_p]),
    "dooms_cuda_llama_profile_pass": (C.c_int32, [C.c_void_p, C.c_int32, C.POINTER(KernelTime), C.c_int32, C.POINTER(C.c_int32)]),
    "dooms_cuda_llama_timings": (C.c_int32, [C.c_void_p, C.POINTER(Timings)]),
    "dooms_cuda_llm_open": (C.c_int32, [C.c_char_p, C.POINTER(LlmOptions), C.POINTER(C.c_void_p)]),
    "dooms_cuda_llm_close": (None, [C.c_void_p]),
    "dooms_cuda_llm_context_size": (C.c_int32, [C.c_void_p]),
    "dooms_cuda_llm_generate": (C.c_int32, [C.c_void_p, C.c_char_p, C.c_int32, C.POINTER(Sampling), C.POINTER(C.c_char_p), C.c_int32, C.c_void_p, C.c_size_t, C.POINTER(C.c_size_t)]),
    "dooms_cuda_llm_generate_stream": (C.c_int32, [C.c_void_p, C.c_char_p, C.c_int32, C.POINTER(Sampling), C.POINTER(C.c_char_p), C.c_int32, TEXT_CALLBACK, C.c_void_p]),
    "dooms_cuda_llm_generate_tokens": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.POINTER(Sampling), C.POINTER(C.c_char_p), C.c_int32, C.c_void_p, C.c_size_t,
                                                   C.POINTER(C.c_size_t), C.c_void_p, C.c_int32, C.POINTER(C.c_int32)]),
    "dooms_cuda_llm_generate_from_embeddings": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.c_int32, C.c_void_p, C.c_int32, C.c_int32, TEXT_CALLBACK, C.c_void_p,
                                                            C.c_void_p, C.c_size_t, C.POINTER(C.c_size_t)]),
    "dooms_cuda_llama_embed_tokens": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p]),
    "dooms_cuda_llm_last_generation": (C.c_int32, [C.c_void_p, C.POINTER(GenerationInfo)]),
    "dooms_cuda_llm_count_tokens": (C.c_int32, [C.c_void_p, C.c_char_p, C.c_int32, C.POINTER(C.c_int32)]),
    "dooms_cuda_vocab_open": (C.c_int32, [C.c_char_p, C.POINTER(C.c_void_p)]),
    "dooms_cuda_vocab_close": (None, [C.c_void_p]),
    "dooms_cuda_vocab_size": (C.c_int32, [C.c_void_p]),
    "dooms_cuda_vocab_is_end_of_generation": (C.c_int32, [C.c_void_p, C.c_int32]),
    "dooms_cuda_vocab_piece": (C.c_int32, [C.c_void_p, C.c_int32, C.c_void_p, C.c_int32, C.POINTER(C.c_int32)]),
    "dooms_cuda_vocab_tokenize": (C.c_int32, [C.c_void_p, C.c_char_p, C.c_int32, C.c_void_p, C.c_int32, C.POINTER(C.c_int32)]),
    "dooms_cuda_vocab_tokenize_special": (C.c_int32, [C.c_void_p, C.c_char_p, C.c_int32, C.c_int32, C.c_void_p, C.c_int32, C.POINTER(C.c_int32)]),
    "dooms_cuda_vocab_apply_chat_template": (C.c_int32, [C.c_void_p, C.POINTER(ChatMessage), C.c_int32, C.c_int32, C.c_void_p, C.c_size_t, C.POINTER(C.c_size_t)]),
    "dooms_cuda_llm_chat": (C.c_int32, [C.c_void_p, C.POINTER(ChatMessage), C.c_int32, C.c_int32, C.POINTER(Sampling), C.POINTER(C.c_char_p), C.c_int32, C.c_void_p, C.c_size_t,
                                        C.POINTER(C.c_size_t)]),
    "dooms_cuda_llm_chat_stream": (C.c_int32, [C.c_void_p, C.POINTER(ChatMessage), C.c_int32, C.c_int32, C.POINTER(Sampling), C.POINTER(C.c_char_p), C.c_int32, TEXT_CALLBACK,
                                               C.c_void_p]),
    "dooms_cuda_llm_count_chat_tokens": (C.c_int32, [C.c_void_p, C.POINTER(ChatMessage), C.c_int32, C.POINTER(C.c_int32)]),
    "dooms_cuda_text_stream": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int32, C.POINTER(C.c_char_p), C.c_int32, TEXT_CALLBACK, C.c_void_p, C.c_void_p, C.c_size_t,
                                           C.POINTER(C.c_size_t), C.POINTER(C.c_int32), C.POINTER(C.c_int32)]),
    "dooms_cuda_sample": (C.c_int32, [C.c_void_p, C.c_int32, C.POINTER(Sampling), C.c_int32, C.c_void_p]),
    "dooms_cuda_llama_max_sequences": (C.c_int32, [C.c_void_p]),
    "dooms_cuda_llama_max_batch_rows": (C.c_int32, [C.c_void_p]),
    "dooms_cuda_llama_select_sequence": (C.c_int32, [C.c_void_p, C.c_int32]),
    "dooms_cuda_llama_decode_batch": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p]),
    "dooms_cuda_dequantize": (C.c_int32, [C.c_int32, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p]),
    "dooms_cuda_matvec": (C.c_int32, [C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_uint32, C.c_void_p]),
    "dooms_cuda_gate_up": (C.c_int32, [C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p]),
    "dooms_cuda_matmul": (C.c_int32, [C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int64, C.c_int64, C.c_uint32, C.c_void_p]),
    "dooms_cuda_split_input_bytes": (C.c_int64, [C.c_int64]),
    "dooms_cuda_split_input": (C.c_int32, [C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p]),
    "dooms_cuda_matvec_split": (C.c_int32, [C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_uint32, C.c_void_p]),
    "dooms_cuda_kernel_status": (C.c_int32, [C.c_void_p, C.POINTER(C.c_int32)]),
    "dooms_cuda_rms_norm": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_float, C.c_void_p]),
    "dooms_cuda_argmax": (C.c_int32, [C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p]),
    "dooms_cuda_argmax_noalloc": (C.c_int32, [C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p]),
    "dooms_cuda_attention_scratch_bytes": (C.c_int64, [C.c_int32, C.c_int32, C.c_int32]),
    "dooms_cuda_attention_decode": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_void_p]),
    "dooms_cuda_tp_share": (C.c_int32, [C.POINTER(LlamaConfig), C.c_int32, C.c_int32, C.POINTER(TpShare)]),
    "dooms_cuda_tp_share_blocks": (C.c_int32, [C.POINTER(LlamaConfig), C.c_int32, C.c_int32, C.c_int64, C.c_int64, C.POINTER(TpShare)]),
    "dooms_cuda_nccl_unique_id": (C.c_int32, [C.c_char_p, C.c_void_p]),
}

_lib = None


def lib() -> C.CDLL:
    """The loaded library with typed entry points. Raises if it was not built (python -m dooms_b200.build)."""
    global _lib
    if _lib is None:
        path = os.environ.get("DOOMS_CUDA_LIB", str(LIB_PATH))
        if not os.path.exists(path):
            raise RuntimeError(f"{path} is missing: build it with `python -m dooms_b200.build`; there is no CPU fallback")
        handle = C.CDLL(path)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)   # AttributeError if the symbol is not exported
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(code: int) -> None:
    if code != OK:
        raise DoomsError(code, lib().dooms_cuda_last_error().decode("utf-8", "replace"))


def nccl_library_path() -> str | None:
    """libnccl.so.2 of the nvidia-nccl wheel torch itself loads, if present."""
    try:
        import nvidia.nccl  # type: ignore
        p = Path(nvidia.nccl.__path__[0]) / "lib" / "libnccl.so.2"
        return str(p) if p.exists() else None
    except Exception:
        return None
