"""Model families used by the benchmarks and examples: decoder-only transformers
in the three configurations the baselines name (70M, 110M, 1.3B)."""
from .decoder import Decoder, DecoderConfig, PRESETS, build_decoder  # noqa: F401
