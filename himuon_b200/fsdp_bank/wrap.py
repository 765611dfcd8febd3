"""Building banks from a model and undoing them for checkpoints.

Contracts (pinned upstream by ``tests/unit/test_fsdp_bank.py`` against
``src/himuon/fsdp_bank/wrap.py:19-175``): banks are zero-initialised ``(n_padded, H, W)``
Parameters on the model's device / dtype; ``rewire_linear`` copies the weight into its slot,
removes the Linear's own ``weight`` Parameter, records ``_bank_name`` / ``_bank_idx`` and routes the
forward through the bank attribute of the root model (looked up on every call, so a sharding
engine may replace it); ``unbank_state_dict`` restores the ``model.layers.{i}.*`` keys and drops
pad slots.
"""

from __future__ import annotations

import torch
import torch.nn as nn

from .. import ops
from .bank import ParamBank
from .scheme import BankScheme


def get_layers(model: nn.Module):
    """Decoder layers of a ``*ForCausalLM`` model (``model.model.layers``)."""
    return model.model.layers


def wrap_with_banks(model: nn.Module, scheme: BankScheme, world_size: int) -> tuple[nn.Module, list[ParamBank]]:
    specs = scheme.collect(model, world_size)
    first = next(model.parameters())
    banks = []
    for spec in specs:
        H, W = spec.matrix_shape
        param = nn.Parameter(torch.zeros(spec.n_padded, H, W, device=first.device, dtype=first.dtype))
        banks.append(ParamBank(spec=spec, parameter=param,
                               name_to_idx={n: i for i, n in enumerate(spec.source_param_names)}))
    scheme.install(model, banks)
    return model, banks


def release_pre_shard_refs(banks: list[ParamBank]) -> None:
    """Drop the un-sharded Parameters captured at wrap time once a sharding engine has replaced them."""
    for b in banks:
        b.parameter = None


def unbank_state_dict(banked_state_dict: dict, banks: list[ParamBank]) -> dict:
    names = {b.spec.name for b in banks}
    out = {k: v for k, v in banked_state_dict.items() if k not in names}
    for b in banks:
        if b.spec.name not in banked_state_dict:
            raise KeyError(f"bank {b.spec.name!r} missing from state_dict (keys: {sorted(banked_state_dict)[:5]}...)")
        tensor = banked_state_dict[b.spec.name]
        for idx, hf_name in enumerate(b.spec.source_param_names):
            out[hf_name] = tensor[idx].clone()
    return out


def rewire_linear(linear: nn.Linear, root_model: nn.Module, bank_name: str, bank: ParamBank, layer_idx: int) -> None:
    assert isinstance(linear, nn.Linear), f"expected nn.Linear, got {type(linear)}"
    expected = bank.spec.matrix_shape
    assert tuple(linear.weight.shape) == expected, (
        f"shape mismatch for {bank.spec.name}[{layer_idx}]: linear.weight={tuple(linear.weight.shape)} vs bank={expected}")
    with torch.no_grad():
        bank.parameter.data[layer_idx].copy_(linear.weight.data)
    del linear._parameters["weight"]
    linear._bank_name = bank_name
    linear._bank_idx = layer_idx
    # plain attribute, not a registered submodule: a reference cycle through the module tree is not wanted
    object.__setattr__(linear, "_bank_root", root_model)

    def forward(x, _linear=linear):
        root = _linear._bank_root
        engine = getattr(root, "_bank_engine", None)
        if engine is not None:
            return engine.linear(x, _linear._bank_name, _linear._bank_idx, _linear.bias)
        w = getattr(root, _linear._bank_name)[_linear._bank_idx]
        y = ops.linear(x, w)
        return y if _linear.bias is None else y + _linear.bias

    linear.forward = forward
