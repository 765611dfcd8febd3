"""Model / tokenizer construction and the parameter-count helpers.

Same entry points as ``src/himuon/model.py:4-44``.  The reference resolves the architecture and
tokenizer through the HF Hub and instantiates ``AutoModelForCausalLM.from_config`` (random
weights); here the architecture comes from the in-tree table and the model is this package's own
decoder.  The HF tokenizer is used when it is available in the local HF cache, otherwise a
byte-level stand-in.
"""

from __future__ import annotations

from .models import CausalLM, get_config
from .utils.tokenizer import ByteTokenizer

_HUB_PREFIX = {"llama": "meta-llama", "qwen": "Qwen"}


def get_model_and_tokenizer(model_name: str):
    lower = model_name.lower()
    if not (lower.startswith("llama") or lower.startswith("qwen") or lower.startswith("tiny")):
        raise ValueError(f"Model {model_name} not supported")
    cfg = get_config(model_name)
    model = CausalLM(cfg)
    tokenizer = None
    for key, org in _HUB_PREFIX.items():
        if lower.startswith(key):
            try:  # only succeeds when the tokenizer files are already cached locally
                from transformers import AutoTokenizer

                tokenizer = AutoTokenizer.from_pretrained(f"{org}/{model_name}", local_files_only=True)
            except Exception:
                tokenizer = None
    if tokenizer is None:
        tokenizer = ByteTokenizer(cfg.vocab_size, cfg.eos_token_id)
    return model, tokenizer


def count_model_parameters(model):
    n = sum(p.numel() for p in model.parameters() if p.requires_grad)
    if n < 1e5:
        return n, f"{n:.0f} trainable parameters"
    if n < 1e8:
        return n, f"{n / 1e6:.2f}M trainable parameters"
    return n, f"{n / 1e9:.2f}B trainable parameters"


def count_num_training_tokens(model, chinchilla_factor: float = 1.0) -> int:
    """Chinchilla budget: ``20 * chinchilla_factor * n_params`` tokens."""
    n, _ = count_model_parameters(model)
    return int(20 * chinchilla_factor * n)
