"""How a part names the tensors it needs."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class WeightSpec:
    """One tensor a part reads from the checkpoint.

    shape     the exact shape it must have; a dimension given as -1 may have any size (a size that no key of the
              configuration gives: the part reads it from the tensor when it loads it).
    init      how the random-weights mode fills it: "normal" (N(0, std)), "gain"
              (1 + N(0, gain_std)), "small" (N(0, gain_std): offsets of gains from one, biases), or
              ("uniform", lo, hi).
    fallback  full name of another tensor that stands in when this one is absent
              (a tied output head reads the embedding table).
    integer   the tensor is an integer table (kept as int32).
    full_precision  the part computes with this tensor in 32-bit whatever the model's precision (norm
              gains): a loader that converts tensors to the model's precision leaves it as stored.
    """
    shape: tuple[int, ...]
    init: str | tuple = "normal"
    fallback: str | None = None
    integer: bool = False
    full_precision: bool = False
