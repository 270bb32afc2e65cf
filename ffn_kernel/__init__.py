"""Import-compatible alias: ``from ffn_kernel import MaskedLinear, MaskedFFN`` resolves to the
B200 implementation in ``ffn_kernel_b200`` (the reference package's surface, ``ffn_kernel/__init__.py:1``)."""
from ffn_kernel_b200.ops import *  # noqa: F401,F403
from ffn_kernel_b200.ops import MaskedFFN, MaskedLinear  # noqa: F401
