"""Parts a model is put together from: norms, position encodings, mixers, feed-forwards, blocks."""

from .registry import CATEGORIES, build_part, part_class, register_part
from . import norm, rope, attention, biased_attention, latent_attention, wkv, mlp, block, streams, diff_attention, gla, moe, conv, talking_attention, key_value_attention, mlstm, pair  # noqa: F401  (each registers its kind)

__all__ = ["CATEGORIES", "build_part", "part_class", "register_part"]
