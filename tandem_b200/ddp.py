"""Alias of tandem_b200.parallel.ddp under the reference's module name (tandem/ddp.py)."""

from .parallel.ddp import DDP, BucketAdamW, GradArena, ShardedBucketAdamW, Span  # noqa: F401

Bucket = Span  # the name the reference uses for the unit of gradient exchange (tandem/ddp.py:22)
