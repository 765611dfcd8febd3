"""Microbenchmarks and small-scale experiments around the HiMuon optimizer (kernel timing, optimizer-step
timing, Newton-Schulz quality, associative-memory probes).  Counterpart of the reference's ``microbench/``."""
