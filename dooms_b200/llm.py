"""The text-model surface over the C ABI (include/dooms_cuda.h: dooms_cuda_llm_*, dooms_cuda_vocab_*, dooms_cuda_text_stream, dooms_cuda_sample): the
reference's `Llm` (src/pipeline/llm_pipeline.h) for the CUDA decoder. Vocabulary, text assembly and sampler run on the host and need no GPU.
Text crosses the boundary as UTF-8 bytes; a model may emit bytes that are no valid UTF-8 (a random-weight model does), so they are carried through Python
strings with the surrogateescape error handler: what comes back encodes to exactly the bytes the library produced."""
from __future__ import annotations

import ctypes as C
from typing import Callable, Sequence

import numpy as np

from . import _lib as L


def _sampling(temperature=0.0, top_k=40, top_p=0.95, repeat_penalty=1.0, seed=0):
    s = L.Sampling()
    s.struct_size = C.sizeof(L.Sampling)
    s.temperature, s.top_k, s.top_p, s.repeat_penalty, s.seed = temperature, top_k, top_p, repeat_penalty, seed
    return s


def _stops(stop: Sequence[str] | None):
    stop = list(stop or [])
    arr = (C.c_char_p * max(1, len(stop)))(*[s.encode("utf-8", "surrogateescape") for s in stop])
    return arr, len(stop)


def _text(call) -> str:
    """Runs call(buffer, capacity, needed) with a buffer that grows once to the size the library asks for."""
    needed = C.c_size_t()
    buf = C.create_string_buffer(4096)
    code = call(buf, len(buf), C.byref(needed))
    if code == L.RESOURCE_EXHAUSTED and needed.value > len(buf):
        buf = C.create_string_buffer(needed.value)
        code = call(buf, len(buf), C.byref(needed))
    L.check(code)
    return buf.value.decode("utf-8", "surrogateescape")


def _messages(messages):
    """[(role, content), ...] or [{"role": ..., "content": ...}, ...] as an array of dooms_cuda_chat_message."""
    pairs = [(m["role"], m["content"]) if isinstance(m, dict) else tuple(m) for m in messages]
    arr = (L.ChatMessage * max(1, len(pairs)))()
    for i, (role, content) in enumerate(pairs):
        arr[i].role, arr[i].content = role.encode("utf-8", "surrogateescape"), content.encode("utf-8", "surrogateescape")
    return arr, len(pairs)


def sample(logits: np.ndarray, draws: int = 1, **sampling) -> list[int]:
    """`draws` tokens from one row of logits (dooms_cuda_sample); keyword arguments as dooms_cuda_sampling, none: greedy."""
    v = np.ascontiguousarray(logits, dtype=np.float32)
    out = np.empty(draws, dtype=np.int32)
    s = _sampling(**sampling) if sampling else None
    L.check(L.lib().dooms_cuda_sample(v.ctypes.data, v.size, C.byref(s) if s else None, draws, out.ctypes.data))
    return [int(t) for t in out]


class Vocab:
    def __init__(self, path: str):
        self._h = C.c_void_p()
        L.check(L.lib().dooms_cuda_vocab_open(str(path).encode(), C.byref(self._h)))

    def close(self):
        if self._h:
            L.lib().dooms_cuda_vocab_close(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __len__(self) -> int:
        return L.lib().dooms_cuda_vocab_size(self._h)

    def piece(self, token: int) -> bytes:
        n = C.c_int32()
        buf = C.create_string_buffer(256)
        L.check(L.lib().dooms_cuda_vocab_piece(self._h, token, buf, 256, C.byref(n)))
        return buf.raw[:n.value]

    def is_end_of_generation(self, token: int) -> bool:
        return bool(L.lib().dooms_cuda_vocab_is_end_of_generation(self._h, token))

    def tokenize(self, text: str, add_special: bool = True, parse_special: bool = False) -> list[int]:
        n = C.c_int32()
        out = np.empty(4 * len(text.encode()) + 8, dtype=np.int32)
        L.check(L.lib().dooms_cuda_vocab_tokenize_special(self._h, text.encode(), int(add_special), int(parse_special), out.ctypes.data, out.size, C.byref(n)))
        return [int(t) for t in out[:n.value]]

    def apply_chat_template(self, messages, add_generation_prompt: bool = True) -> str:
        """The conversation in the format of the file's chat template; Unsupported without one or with one of an unknown family."""
        arr, n = _messages(messages)
        return _text(lambda buf, cap, needed: L.lib().dooms_cuda_vocab_apply_chat_template(self._h, arr, n, int(add_generation_prompt), buf, cap, needed))

    def stream(self, tokens: Sequence[int], stop: Sequence[str] | None = None, on_text: Callable[[str], bool] | None = None):
        """The text assembly over `tokens`: (text, tokens consumed, finish reason). on_text receives each piece and returns False to cancel."""
        a = np.ascontiguousarray(np.asarray(tokens, dtype=np.int32))
        arr, n_stop = _stops(stop)
        cb = L.TEXT_CALLBACK(lambda piece, _u: 0 if (on_text is None or on_text(piece.decode("utf-8", "surrogateescape")) is not False) else 1)
        consumed, reason = C.c_int32(), C.c_int32()
        text = _text(lambda buf, cap, needed: L.lib().dooms_cuda_text_stream(self._h, a.ctypes.data, a.size, arr, n_stop, cb, None, buf, cap, needed, C.byref(consumed),
                                                                            C.byref(reason)))
        return text, consumed.value, reason.value


class Llm:
    def __init__(self, path: str, n_ctx: int = 4096, n_batch: int = 512, queue_depth: int = 4, device: int = 0):
        o = L.LlmOptions()
        o.struct_size = C.sizeof(L.LlmOptions)
        o.n_ctx, o.n_batch, o.queue_depth, o.device = n_ctx, n_batch, queue_depth, device
        self._h = C.c_void_p()
        L.check(L.lib().dooms_cuda_llm_open(str(path).encode(), C.byref(o), C.byref(self._h)))

    def close(self):
        if self._h:
            L.lib().dooms_cuda_llm_close(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def context_size(self) -> int:
        return L.lib().dooms_cuda_llm_context_size(self._h)

    def count_tokens(self, text: str, add_special: bool = True) -> int:
        n = C.c_int32()
        L.check(L.lib().dooms_cuda_llm_count_tokens(self._h, text.encode(), int(add_special), C.byref(n)))
        return n.value

    def generate(self, prompt: str, max_new_tokens: int = 128, stop: Sequence[str] | None = None, on_text: Callable[[str], bool] | None = None, **sampling) -> str:
        arr, n_stop = _stops(stop)
        s = _sampling(**sampling) if sampling else None
        sp = C.byref(s) if s else None
        if on_text is None:
            return _text(lambda buf, cap, needed: L.lib().dooms_cuda_llm_generate(self._h, prompt.encode("utf-8", "surrogateescape"), max_new_tokens, sp, arr, n_stop, buf, cap, needed))
        pieces: list[str] = []

        def cb(piece, _u):
            text = piece.decode("utf-8", "surrogateescape")
            pieces.append(text)
            return 0 if on_text(text) is not False else 1
        L.check(L.lib().dooms_cuda_llm_generate_stream(self._h, prompt.encode("utf-8", "surrogateescape"), max_new_tokens, sp, arr, n_stop, L.TEXT_CALLBACK(cb), None))
        return "".join(pieces)

    def count_chat_tokens(self, messages) -> int:
        arr, n_messages = _messages(messages)
        n = C.c_int32()
        L.check(L.lib().dooms_cuda_llm_count_chat_tokens(self._h, arr, n_messages, C.byref(n)))
        return n.value

    def chat(self, messages, max_new_tokens: int = 128, stop: Sequence[str] | None = None, on_text: Callable[[str], bool] | None = None, **sampling) -> str:
        """The assistant's answer to a conversation ([(role, content), ...]) formatted with the file's chat template."""
        msgs, n_messages = _messages(messages)
        arr, n_stop = _stops(stop)
        s = _sampling(**sampling) if sampling else None
        sp = C.byref(s) if s else None
        if on_text is None:
            return _text(lambda buf, cap, needed: L.lib().dooms_cuda_llm_chat(self._h, msgs, n_messages, max_new_tokens, sp, arr, n_stop, buf, cap, needed))
        pieces: list[str] = []

        def cb(piece, _u):
            text = piece.decode("utf-8", "surrogateescape")
            pieces.append(text)
            return 0 if on_text(text) is not False else 1
        L.check(L.lib().dooms_cuda_llm_chat_stream(self._h, msgs, n_messages, max_new_tokens, sp, arr, n_stop, L.TEXT_CALLBACK(cb), None))
        return "".join(pieces)

    def generate_tokens(self, prompt: Sequence[int], max_new_tokens: int = 128, stop: Sequence[str] | None = None, **sampling):
        """(text, generated token ids) from a prompt given as token ids."""
        a = np.ascontiguousarray(np.asarray(prompt, dtype=np.int32))
        arr, n_stop = _stops(stop)
        s = _sampling(**sampling) if sampling else None
        toks = np.empty(max(1, max_new_tokens), dtype=np.int32)
        n = C.c_int32()
        text = _text(lambda buf, cap, needed: L.lib().dooms_cuda_llm_generate_tokens(self._h, a.ctypes.data, a.size, max_new_tokens, C.byref(s) if s else None, arr, n_stop, buf, cap,
                                                                                    needed, toks.ctypes.data, toks.size, C.byref(n)))
        return text, [int(t) for t in toks[:n.value]]

    def generate_from_embeddings(self, before: Sequence[int], image: np.ndarray | None, after: Sequence[int], max_new_tokens: int = 128,
                                 on_text: Callable[[str], bool] | None = None) -> str:
        """The text side of a vision-language pipeline: token rows, the image's embedding rows ([rows][n_embd] floats) and more token rows as one sequence."""
        b = np.ascontiguousarray(np.asarray(before, dtype=np.int32))
        a = np.ascontiguousarray(np.asarray(after, dtype=np.int32))
        img = np.ascontiguousarray(image, dtype=np.float32) if image is not None else np.zeros((0, 1), dtype=np.float32)
        cb = L.TEXT_CALLBACK(lambda piece, _u: 0 if (on_text is None or on_text(piece.decode("utf-8", "surrogateescape")) is not False) else 1)
        return _text(lambda buf, cap, needed: L.lib().dooms_cuda_llm_generate_from_embeddings(self._h, b.ctypes.data, b.size, img.ctypes.data, img.shape[0], a.ctypes.data, a.size,
                                                                                             max_new_tokens, cb, None, buf, cap, needed))

    def last_generation(self) -> dict:
        info = L.GenerationInfo()
        info.struct_size = C.sizeof(L.GenerationInfo)
        L.check(L.lib().dooms_cuda_llm_last_generation(self._h, C.byref(info)))
        return {n: getattr(info, n) for n, _ in L.GenerationInfo._fields_ if n != "struct_size"}
