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
    init     how the random-weights mode fills it: "normal" (``mean``, ``std``), "ones", "zeros".
    tied_to  full name of another tensor that stands in when this one is absent.
    optional a tensor that a folder may hold or not (one that the model does not use: a file that has it is not at
             fault, and the random-weights mode does not make it).
    """
    shape: Tuple[int, ...]
    kind: str = "matrix"
    init: str = "normal"
    std: float = 0.02
    mean: float = 0.0
    tied_to: Optional[str] = None
    optional: bool = False
