"""Alias of tandem_b200.models.gpt under the reference's module name (tandem/model.py)."""

from .models.gpt import GPT, Attention, Block, Config, Embed, Head, count_params, loss_fn  # noqa: F401
