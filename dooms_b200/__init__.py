"""dooms_b200: a CUDA (sm_100a) backend for the llama / qwen2 GGUF decoder of dooms.cpp, behind a C ABI (include/dooms_cuda.h)."""
from ._lib import DoomsError, lib  # noqa: F401
from .decoder import CudaLlamaDecoder, LlamaDecoderConfig  # noqa: F401
