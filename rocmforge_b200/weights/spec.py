"""What a part says about each tensor it wants from the weight file."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple


@dataclass(frozen=True)
class ParamSpec:
    """One named tensor.

    kind     "matrix": operand of a matrix product, kept in the compute dtype.
             "vector": norm weight or bias; a vector stored in 32-bit stays 32-bit,
             one stored in bfloat16 stays bfloat16 (all 32-bit on the float32 path).
             "int_table": integer table, kept as int32.
    init     how the random-weights mode fills it: "normal" (mean 0, ``std``), "ones", "zeros".
    tied_to  full name of another tensor that stands in when this one is absent.
    """
    shape: Tuple[int, ...]
    kind: str = "matrix"
    init: str = "normal"
    std: float = 0.02
    tied_to: Optional[str] = None
