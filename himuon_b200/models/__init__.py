"""Model definitions: offline architecture table and the decoder-only causal LM."""

from .config import MODEL_CONFIGS, DecoderConfig, get_config
from .decoder import CausalLM, CausalLMOutput

__all__ = ["MODEL_CONFIGS", "DecoderConfig", "get_config", "CausalLM", "CausalLMOutput"]
