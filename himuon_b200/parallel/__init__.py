"""Multi-GPU execution: symmetric (peer-mapped) memory, fused collectives over NVLink, the
data-parallel engine and the bank-sharded engine."""
