"""The language model of the benchmark scripts under the path the reference's scripts import it from
(benchmarks/models/transformer_lm.py there); the implementation lives in the package."""

from fairscale_b200.models.transformer_lm import *  # noqa: F401,F403
from fairscale_b200.models.transformer_lm import TransformerDecoderLayer, TransformerLM  # noqa: F401
