"""One module per experiment; each exposes ``run(...) -> dict`` and ``plot(data, out_dir)``."""
