"""Alias of tandem_b200.utils.profile under the reference's module name (tandem/profile.py)."""

from .utils.profile import Timeline, chrome_trace, summarize  # noqa: F401
