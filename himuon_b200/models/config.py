"""Offline architecture table for the decoder families the framework trains.

The reference resolves configs through the HF Hub (``src/himuon/model.py:7-20``);
no network exists here, so the published architecture hyper-parameters of each
supported checkpoint name are kept in-tree.  ``to_hf_dict`` emits a ``config.json``
that ``transformers`` can load.
"""

from __future__ import annotations

from dataclasses import asdict, dataclass, field


@dataclass
class DecoderConfig:
    model_type: str = "qwen3"            # "qwen3" (QK-norm) or "llama"
    vocab_size: int = 151936
    hidden_size: int = 1024
    intermediate_size: int = 3072
    num_hidden_layers: int = 28
    num_attention_heads: int = 16
    num_key_value_heads: int = 8
    head_dim: int = 128
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1_000_000.0
    tie_word_embeddings: bool = True
    max_position_embeddings: int = 40960
    initializer_range: float = 0.02
    bos_token_id: int = 151643
    eos_token_id: int = 151645
    extra: dict = field(default_factory=dict)

    @property
    def qk_norm(self) -> bool:
        return self.model_type == "qwen3"

    def to_hf_dict(self) -> dict:
        d = asdict(self)
        d.pop("extra")
        d.update(self.extra)
        d["architectures"] = ["Qwen3ForCausalLM" if self.model_type == "qwen3" else "LlamaForCausalLM"]
        d["hidden_act"] = "silu"
        d["attention_bias"] = False
        d["attention_dropout"] = 0.0
        d["torch_dtype"] = "bfloat16"
        d["use_cache"] = False
        if self.model_type == "llama":
            d["mlp_bias"] = False
        return d


def _qwen3(h, inter, layers, heads, kv, tie, **kw):
    return DecoderConfig("qwen3", 151936, h, inter, layers, heads, kv, 128, 1e-6, 1_000_000.0, tie, 40960, **kw)


def _llama3(h, inter, layers, heads, kv, tie, vocab=128256, head_dim=None, theta=500000.0, **kw):
    return DecoderConfig("llama", vocab, h, inter, layers, heads, kv, head_dim or h // heads, 1e-5, theta, tie,
                         131072, bos_token_id=128000, eos_token_id=128001, **kw)


MODEL_CONFIGS: dict[str, DecoderConfig] = {
    "Qwen3-0.6B": _qwen3(1024, 3072, 28, 16, 8, True),
    "Qwen3-1.7B": _qwen3(2048, 6144, 28, 16, 8, True),
    "Qwen3-4B": _qwen3(2560, 9728, 36, 32, 8, True),
    "Qwen3-8B": _qwen3(4096, 12288, 36, 32, 8, False),
    "Llama-3.2-1B": _llama3(2048, 8192, 16, 32, 8, True),
    "Llama-3.2-3B": _llama3(3072, 8192, 28, 24, 8, True),
    "Llama-3.1-8B": _llama3(4096, 14336, 32, 32, 8, False),
    "Llama-3-8B": _llama3(4096, 14336, 32, 32, 8, False),
    # 220M-parameter Llama used by the reference's tile-shape quality experiment
    # (microbench/experiments/exp_tile_shape_quality.py:88-98): hidden 640, 12 layers.
    "llama_220m": _llama3(640, 1728, 12, 10, 10, False, head_dim=64, theta=10000.0),
    # Tiny CPU configuration used by the fp32 single-process regression run.
    "tiny-llama": DecoderConfig("llama", 1024, 128, 352, 2, 4, 2, 32, 1e-5, 10000.0, False, 2048,
                                bos_token_id=0, eos_token_id=1),
    "tiny-qwen3": DecoderConfig("qwen3", 1024, 128, 352, 2, 4, 2, 32, 1e-6, 10000.0, True, 2048,
                                bos_token_id=0, eos_token_id=1),
}


def get_config(name: str) -> DecoderConfig:
    """Case-insensitive lookup of an architecture by checkpoint name."""
    for key, cfg in MODEL_CONFIGS.items():
        if key.lower() == name.lower():
            return cfg
    raise ValueError(f"Model {name} not supported (known: {sorted(MODEL_CONFIGS)})")
