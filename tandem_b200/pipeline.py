"""Alias of tandem_b200.parallel.pipeline under the reference's module name (tandem/pipeline.py)."""

from .parallel.pipeline import Pipeline, plan, split_units  # noqa: F401
