from . import fopivik, llama, norusun, potipel, tevudra  # noqa: F401  (register Fopivik, LlamaForCausalLM, Norusun, Potipel, Tevudra)
from .spec import LayerSpec, ModelSpec, PartSpec

__all__ = ["LayerSpec", "ModelSpec", "PartSpec"]
