"""himuon_b200: a Blackwell-native (sm_100a) training framework around the HiMuon optimizer.

Sub-packages: ``optimizers`` / ``optim`` (HiMuon, Muon, MuonFsdp, AdamW, SOAP + factory),
``fsdp_bank`` (parameter banks), ``models`` (decoder LMs), ``ops`` (kernels + autograd),
``parallel`` (symmetric memory, fused collectives, DDP and bank-sharded engines), ``utils``.
"""

__version__ = "0.1.0"
