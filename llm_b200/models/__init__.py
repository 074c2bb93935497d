from . import fopivik, llama, norusun, tevudra  # noqa: F401  (register Fopivik, LlamaForCausalLM, Norusun, Tevudra)
from .spec import LayerSpec, ModelSpec, PartSpec

__all__ = ["LayerSpec", "ModelSpec", "PartSpec"]
