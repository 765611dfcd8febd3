"""Bank scheme for Qwen3 decoders (``src/himuon/fsdp_bank/qwen3_scheme.py:26-122``)."""

from ._decoder_scheme import DecoderBankScheme


class Qwen3BankScheme(DecoderBankScheme):
    pass
