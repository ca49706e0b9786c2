"""What a part asks of a checkpoint: one ``TensorSpec`` per tensor."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Tuple


@dataclass(frozen=True)
class TensorSpec:
    """``name``: the tensor's name in the checkpoint.  ``shape``: what the
    configuration implies; a size of None is one the configuration does not
    give and the checkpoint's tensor decides.  ``kind``: ``matrix`` (operand of a matrix product
    or a lookup table of activations: kept in the compute dtype), ``vector``
    (norm weights, biases: a tensor stored in 32-bit stays so) or ``table``
    (integers: kept as int32).  ``optional``: absence is not an error.
    ``init``: how the random-weights mode draws it: ``normal`` N(0, 0.02),
    ``norm`` 1 + N(0, 0.1), ``norm_zero`` N(0, 0.1), ``conv`` N(0, 0.5), ``unit``
    N(0, 1 / fan-in) (products that keep their input's scale), ``bias`` N(0, 0.02),
    ``lane_read`` 1 / n + N(0, 0.1), ``lane_mix`` the unit matrix + N(0, 0.1), ``half`` 0.5 + N(0, 0.1),
    ``sink`` N(0, 0.5), ``unit_interval`` sigmoid(N(0, 1)), ``unit_rows`` N(0, 1),
    ``decay_bias`` 2 + N(0, 1), ``zeros``."""

    name: str
    shape: Tuple[int, ...]
    kind: str = "matrix"
    optional: bool = False
    init: str = "normal"
