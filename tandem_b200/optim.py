"""Alias of tandem_b200.parallel.optim under the reference's module name (tandem/optim.py)."""

from .parallel.optim import ShardedAdamW  # noqa: F401
