"""The import surface of the reference package, module by module: what ``ffn_kernel/ops.py:5-6``,
``test_linear.py:6``, ``test_ffn.py:6`` and ``ffn_kernel/__init__.py:1`` import must resolve here,
and to the B200 implementation (no second copy of the operators)."""
import inspect


def test_reference_import_statements_resolve():
    from ffn_kernel import MaskedFFN, MaskedLinear                                   # test_ffn.py:6, test_linear.py:6
    from ffn_kernel.ops import MaskedFFN as F2, MaskedLinear as L2                   # ffn_kernel/__init__.py:1
    from ffn_kernel.linear import _bf16_linear_backward, _bf16_linear_forward       # ffn_kernel/ops.py:5
    from ffn_kernel.ffn import _bf16_ffn_forward                                    # ffn_kernel/ops.py:6
    import ffn_kernel_b200
    assert MaskedFFN is F2 is ffn_kernel_b200.MaskedFFN
    assert MaskedLinear is L2 is ffn_kernel_b200.MaskedLinear
    for fn in (_bf16_linear_forward, _bf16_linear_backward, _bf16_ffn_forward):
        assert callable(fn)


def test_launcher_signatures_keep_the_reference_arguments():
    from ffn_kernel.ffn import _bf16_ffn_forward
    from ffn_kernel.linear import _bf16_linear_backward, _bf16_linear_forward
    # ffn_kernel/linear.py:418, :455 and ffn_kernel/ffn.py:527: leading positional parameters
    assert list(inspect.signature(_bf16_linear_forward).parameters)[:4] == ["a", "b1", "b2", "mask"]
    assert list(inspect.signature(_bf16_linear_backward).parameters)[:5] == ["gd", "a", "b1", "b2", "mask"]
    assert list(inspect.signature(_bf16_ffn_forward).parameters)[:6] == ["x", "w1", "w3", "u1", "u3", "mask"]


def test_operator_signatures():
    from ffn_kernel.ops import MaskedFFN, MaskedLinear
    assert list(inspect.signature(MaskedLinear.forward).parameters) == ["ctx", "a", "b1", "b2", "mask"]
    assert list(inspect.signature(MaskedFFN.forward).parameters) == ["ctx", "a", "w1", "w2", "w3", "u1", "u2", "u3",
                                                                      "mask"]
