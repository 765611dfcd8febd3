"""Bank scheme for Llama-3 decoders: Llama-3.1-8B, Llama-3.2-3B, Llama-3.2-1B
(``src/himuon/fsdp_bank/llama3_scheme.py:35-119``)."""

from ._decoder_scheme import DecoderBankScheme


class Llama3BankScheme(DecoderBankScheme):
    pass
