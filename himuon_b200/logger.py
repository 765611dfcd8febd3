"""Run loggers (file/stderr via loguru, optional Weights & Biases).

The metric line format ``Step: … LR: … Training loss: …, Tokens: …[, Eval loss: …]``
is the one the reference prints (``src/himuon/logger.py:23-27``) and that its FSDP
smoke test parses (``tests/integration/test_himuon_fsdp_smoke.py:48``).
"""

from __future__ import annotations

import os

try:  # optional extra, exactly as upstream
    import wandb
except ImportError:  # pragma: no cover
    wandb = None


def format_metrics(metrics: dict) -> str:
    msg = (
        f"Step: {metrics['step']} LR: {metrics['lr']:.6f} "
        f"Training loss: {metrics['loss']:.4f}, Tokens: {metrics['tokens']:,}"
    )
    if "eval_loss" in metrics:
        msg += f", Eval loss: {metrics['eval_loss']:.4f}"
    return msg


class LoguruLogger:
    """Logs to stderr and ``logs/<run_name>.log``."""

    def __init__(self, run_name: str | None):
        from loguru import logger

        self.logger = logger
        if run_name is not None and not os.path.exists(f"logs/{run_name}.log"):
            self.add(f"logs/{run_name}.log")

    def add(self, *args, **kwargs):
        self.logger.add(*args, **kwargs)

    def info(self, msg):
        self.logger.info(msg)

    def log_metrics(self, metrics: dict, verbose: bool = True):
        self.logger.info(format_metrics(metrics))

    def log_optimizer_source(self, optimizer):
        pass


class WandbLogger:
    """Logs metrics to the W&B project ``himuon``."""

    def __init__(self, config, run_name: str):
        if wandb is None:
            raise ImportError("wandb is not installed.")
        wandb.init(project="himuon", config=config, name=run_name)

    def add(self, *args, **kwargs):
        pass

    def info(self, msg):
        wandb.termlog(str(msg))

    def log_metrics(self, metrics: dict, verbose: bool = True):
        wandb.log(metrics)
        if verbose:
            wandb.termlog(format_metrics(metrics))

    def log_optimizer_source(self, optimizer):
        import inspect

        wandb.save(inspect.getfile(type(optimizer)), policy="now")
