from .model import LayerCall, Model
from . import llama  # registers LlamaForCausalLM
from . import zukotar  # registers Zukotar

__all__ = ["LayerCall", "Model", "llama", "zukotar"]
