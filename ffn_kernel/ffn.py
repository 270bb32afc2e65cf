"""``ffn_kernel.ffn``: the MaskedFFN host launchers under the reference's module path
(``ffn_kernel/ffn.py:527-560`` ``_bf16_ffn_forward``: the SwiGLU intermediate in token order).
``_bf16_ffn_fused_forward`` is the whole ``MaskedFFN.forward`` (``ffn_kernel/ops.py:28-32``);
the training forward and the backward are what the reference left unfinished
(``ffn_kernel/ffn.py:116-524``)."""
from ffn_kernel_b200.ffn import (_bf16_ffn_backward, _bf16_ffn_forward, _bf16_ffn_fused_forward,  # noqa: F401
                                 _bf16_ffn_train_forward)

__all__ = ["_bf16_ffn_forward", "_bf16_ffn_fused_forward", "_bf16_ffn_train_forward", "_bf16_ffn_backward"]
