"""Bank layout shared by the Qwen3 and Llama-3 decoder families."""

from __future__ import annotations

import torch.nn as nn

from .bank import BankSpec, ParamBank
from .wrap import get_layers, rewire_linear

_ROLES = {
    "q": "self_attn.q_proj", "k": "self_attn.k_proj", "v": "self_attn.v_proj", "o": "self_attn.o_proj",
    "gate": "mlp.gate_proj", "up": "mlp.up_proj", "down": "mlp.down_proj",
}


def _module(layer, dotted):
    for part in dotted.split("."):
        layer = getattr(layer, part)
    return layer


class DecoderBankScheme:
    """Five banks: ``q_bank``, ``kv_bank`` (k, v interleaved at ``2i``, ``2i+1``), ``o_bank``,
    ``gate_up_bank`` (gate, up interleaved) and ``down_bank``; the layer axis is padded up to a
    multiple of the world size.  Embeddings, lm_head and norms stay ordinary parameters."""

    BANK_NAMES = ("q_bank", "kv_bank", "o_bank", "gate_up_bank", "down_bank")

    def collect(self, model: nn.Module, world_size: int) -> list[BankSpec]:
        layers = get_layers(model)
        L = len(layers)
        names = {r: [f"model.layers.{i}.{path}.weight" for i in range(L)] for r, path in _ROLES.items()}
        shapes = {r: tuple(_module(layers[0], path).weight.shape) for r, path in _ROLES.items()}
        assert shapes["k"] == shapes["v"], f"k/v shape mismatch: {shapes['k']} vs {shapes['v']}"
        assert shapes["gate"] == shapes["up"], f"gate/up shape mismatch: {shapes['gate']} vs {shapes['up']}"

        def interleave(a, b):
            return [n for pair in zip(a, b, strict=True) for n in pair]

        def pad(n):
            return -(-n // world_size) * world_size

        return [
            BankSpec("q_bank", shapes["q"], names["q"], pad(L)),
            BankSpec("kv_bank", shapes["k"], interleave(names["k"], names["v"]), pad(2 * L)),
            BankSpec("o_bank", shapes["o"], names["o"], pad(L)),
            BankSpec("gate_up_bank", shapes["gate"], interleave(names["gate"], names["up"]), pad(2 * L)),
            BankSpec("down_bank", shapes["down"], names["down"], pad(L)),
        ]

    def install(self, model: nn.Module, banks: list[ParamBank]) -> nn.Module:
        by_name = {b.spec.name: b for b in banks}
        for b in banks:
            setattr(model, b.spec.name, b.parameter)   # on the outer *ForCausalLM module
        for i, layer in enumerate(get_layers(model)):
            a, m = layer.self_attn, layer.mlp
            rewire_linear(a.q_proj, model, "q_bank", by_name["q_bank"], i)
            rewire_linear(a.k_proj, model, "kv_bank", by_name["kv_bank"], 2 * i)
            rewire_linear(a.v_proj, model, "kv_bank", by_name["kv_bank"], 2 * i + 1)
            rewire_linear(a.o_proj, model, "o_bank", by_name["o_bank"], i)
            rewire_linear(m.gate_proj, model, "gate_up_bank", by_name["gate_up_bank"], 2 * i)
            rewire_linear(m.up_proj, model, "gate_up_bank", by_name["gate_up_bank"], 2 * i + 1)
            rewire_linear(m.down_proj, model, "down_bank", by_name["down_bank"], i)
        return model
