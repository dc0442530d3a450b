"""What a part says about one of its tensors: shape, how a random model fills
it, and whether it holds numbers or an integer table."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Tuple


@dataclass(frozen=True)
class ParamSpec:
    shape: Tuple[int, ...]
    # "matrix"/"table": N(0, 0.02); "norm": 1 + N(0, 0.05); "zeros"; "int_table": uniform ints
    init: str = "matrix"
    kind: str = "float"            # "float" follows the dtype rule of the loader; "int" is kept as int32
    std: float = 0.02
    # a tensor that may be absent from the file; the part then gets `fallback` (another
    # global tensor name) or nothing
    optional: bool = False
    fallback: str = ""
