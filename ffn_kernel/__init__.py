"""Drop-in package name of the reference (``ffn_kernel/__init__.py:1``: ``from .ops import *``).

``ffn_kernel.ops``, ``ffn_kernel.linear`` and ``ffn_kernel.ffn`` are the modules the reference's own
code imports from (``ffn_kernel/ops.py:5-6``, ``test_linear.py:6``, ``test_ffn.py:6``); each one
re-exports the B200 implementation that lives in ``ffn_kernel_b200`` under the reference's names."""
from .ops import *  # noqa: F401,F403
from .ops import MaskedFFN, MaskedLinear  # noqa: F401
