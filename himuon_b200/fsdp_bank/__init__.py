"""Parameter banks: per-layer projections of one shape stacked to ``(num_layers, H, W)`` and sharded on
the layer axis, so every rank owns whole matrices and the optimizer needs no collective
(``src/himuon/fsdp_bank/__init__.py:25-34``)."""

from .bank import BankSpec, ParamBank
from .llama3_scheme import Llama3BankScheme
from .qwen3_scheme import Qwen3BankScheme
from .scheme import BankScheme
from .wrap import get_layers, release_pre_shard_refs, rewire_linear, unbank_state_dict, wrap_with_banks

__all__ = [
    "BankSpec", "ParamBank", "BankScheme", "Qwen3BankScheme", "Llama3BankScheme",
    "wrap_with_banks", "release_pre_shard_refs", "unbank_state_dict", "rewire_linear", "get_layers",
]
