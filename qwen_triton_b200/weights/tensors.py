"""What a model expects of its checkpoint: tensor names, shapes and roles."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class TensorSpec:
    """One checkpoint tensor a part needs.

    ``role`` decides the precision it is kept in and how random weights are drawn:

    * ``matrix``  a projection or embedding table; kept in the compute dtype
      (bfloat16 or float32); random: N(0, ``init_std``).
    * ``vector``  a small per-channel tensor such as a norm weight; kept in
      float32, which holds bfloat16 and 32-bit files alike without loss;
      random: ``init_mean`` + N(0, ``init_std``).
    * ``table``   an integer table; kept as int32; random: zeros.
    """

    shape: tuple[int, ...]
    role: str = "matrix"
    init_std: float = 0.02
    init_mean: float = 0.0
    optional: bool = False   # e.g. lm_head.weight of a tied model: read if present, never required
