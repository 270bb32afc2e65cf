"""``ffn_kernel.linear``: the MaskedLinear host launchers under the reference's module path
(``ffn_kernel/linear.py:418-452`` ``_bf16_linear_forward``, ``ffn_kernel/linear.py:455-496``
``_bf16_linear_backward``).  Same names, arguments and results; the work is done by the sm_100a
kernels of ``ffn_kernel_b200`` (no Triton kernels and no JSON tile tables exist here)."""
from ffn_kernel_b200.linear import (_bf16_linear_backward, _bf16_linear_forward,  # noqa: F401
                                    _bf16_linear_train_forward)

__all__ = ["_bf16_linear_forward", "_bf16_linear_backward", "_bf16_linear_train_forward"]
