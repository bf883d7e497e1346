from . import llama, marutar  # noqa: F401  (register LlamaForCausalLM and Marutar)
from .model import DecoderModel, cache_needs, expected_tensors

__all__ = ["DecoderModel", "cache_needs", "expected_tensors"]
