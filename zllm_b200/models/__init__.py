from .decoder import DecoderModel, Runtime, expected_tensors, optional_tensors, required_tensors
from . import llama, sepirax, vasonex  # noqa: F401  (register LlamaForCausalLM, Sepirax and Vasonex)

__all__ = ["DecoderModel", "Runtime", "expected_tensors", "optional_tensors", "required_tensors"]
