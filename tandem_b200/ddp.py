"""Alias of tandem_b200.parallel.ddp under the reference's module name (tandem/ddp.py)."""

from .parallel.ddp import DDP, Bucket, BucketAdamW  # noqa: F401
