"""Alias of tandem_b200.parallel.zero under the reference's module name (tandem/zero.py)."""

from .parallel.zero import FSDP, FlatLayout, ZeRO, split_sizes  # noqa: F401
