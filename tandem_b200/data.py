"""Alias of tandem_b200.utils.data under the reference's module name (tandem/data.py)."""

from .utils.data import Text, synthetic, uniform_tokens  # noqa: F401
