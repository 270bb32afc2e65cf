"""``ffn_kernel.ops``: the operator API under the reference's module path (``ffn_kernel/ops.py:9-38``).
The classes are the B200 implementation in ``ffn_kernel_b200.ops`` (same objects, not copies)."""
from ffn_kernel_b200.ops import MaskedFFN, MaskedLinear  # noqa: F401

from .ffn import _bf16_ffn_forward  # noqa: F401  (what ffn_kernel/ops.py:6 imports)
from .linear import _bf16_linear_backward, _bf16_linear_forward  # noqa: F401  (ffn_kernel/ops.py:5)

__all__ = ["MaskedLinear", "MaskedFFN"]
