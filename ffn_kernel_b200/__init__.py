"""B200 (sm_100a) implementation of the routed MaskedLinear / MaskedFFN operators.

Import surface of the reference package (``ffn_kernel/__init__.py:1``):
``from ffn_kernel_b200 import MaskedLinear, MaskedFFN``.
"""
from .ops import MaskedFFN, MaskedLinear  # noqa: F401
from .modules import GraphedMaskedFFN, MaskedFFNModule, MaskedLinearModule, TensorParallelMaskedFFN  # noqa: F401
from .route import Route, check_status, route  # noqa: F401

__all__ = ["MaskedLinear", "MaskedFFN", "MaskedLinearModule", "MaskedFFNModule", "TensorParallelMaskedFFN", "GraphedMaskedFFN",
           "route", "Route", "check_status"]
