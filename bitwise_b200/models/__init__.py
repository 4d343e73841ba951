from .decoder import DecoderModel, LayerRun, sequential_schedule
from . import llama  # noqa: F401  (registers LlamaForCausalLM)

__all__ = ["DecoderModel", "LayerRun", "sequential_schedule"]
