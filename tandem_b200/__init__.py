"""tandem_b200: a single-machine distributed-training runtime for 8xB200
(NVLink 5 / NVSwitch) with the capabilities and public API of tandem
(reference: tandem/__init__.py:1-6 exports CommError, Group, Work, launch)."""

from .comm import CommError, Group, Work, launch

__all__ = ["CommError", "Group", "Work", "launch"]
__version__ = "0.1.0"
