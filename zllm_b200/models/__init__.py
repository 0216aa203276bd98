from .decoder import DecoderModel, Runtime, expected_tensors, optional_tensors, required_tensors
from . import llama, sepirax  # noqa: F401  (register LlamaForCausalLM and Sepirax)

__all__ = ["DecoderModel", "Runtime", "expected_tensors", "optional_tensors", "required_tensors"]
