from fairscale_b200.models.transformer_lm import TransformerLM  # noqa: F401
