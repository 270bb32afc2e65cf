"""Generate the golden vectors in this directory from the reference's own modules.

Run once in a container that has the reference checkout (it is not needed at
test time):

    python tests/golden/make_golden.py /path/to/reference

The reference's PyTorch modules live in its benchmark scripts
(``test_linear.py:41-49`` ``Torch``; ``test_ffn.py:32-47`` ``Torch``), which
import two packages that are not installed here (``profiler``, ``IPython``);
both are stubbed so that the scripts import on CPU.  The modules are evaluated
in float32 on bf16-rounded inputs (the parity reference, stored as float32) and
in bfloat16 (the reference's own arithmetic, stored as raw bf16 bits in uint16); the MaskedLinear gradients come from autograd
through the same module with an upstream gradient, as ``test_linear.py:94-97``
does with ``.sum().backward()``.
"""
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _import_reference(ref_root):
    for name in ("profiler", "IPython"):
        stub = types.ModuleType(name)
        stub.WallTime = object
        stub.embed = lambda *a, **k: None
        sys.modules.setdefault(name, stub)
    # the scripts import the Triton package at module scope; only the Torch classes are used
    sys.path.insert(0, ref_root)
    import test_ffn
    import test_linear
    return test_linear.Torch, test_ffn.Torch


def _bf16(shape, std, gen):
    return (torch.randn(shape, generator=gen) * std).to(torch.bfloat16)


def _u16(t):
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def _mask(B, S, gen):
    # interleaved spans and isolated tokens, unlike the reference's single span
    m = torch.zeros(B * S, dtype=torch.bool)
    pos = 0
    while pos < B * S:
        pos += int(torch.randint(1, 40, (1,), generator=gen))
        n = int(torch.randint(1, 70, (1,), generator=gen))
        m[pos:pos + n] = True
        pos += n
    return m.view(B, S)


def linear_case(TorchLinear, name, B, S, K, N, seed):
    gen = torch.Generator().manual_seed(seed)
    x, wv, wt, g = _bf16((B, S, K), 1.0, gen), _bf16((N, K), 0.02, gen), _bf16((N, K), 0.02, gen), \
        _bf16((B, S, N), 1.0, gen)
    mask = _mask(B, S, gen)
    out = {}
    for tag, dt in (("f32", torch.float32), ("bf16", torch.bfloat16)):
        mod = TorchLinear(K, N).to(dt)
        with torch.no_grad():
            mod.linear_v.weight.copy_(wv.to(dt))
            mod.linear_t.weight.copy_(wt.to(dt))
        xi = x.to(dt).requires_grad_(True)
        y = mod(xi, mask)
        y.backward(g.to(dt))
        pack = (lambda t: t.detach().float().numpy()) if dt == torch.float32 else (lambda t: _u16(t.detach()))
        out[f"y_{tag}"] = pack(y)
        out[f"dx_{tag}"] = pack(xi.grad)
        out[f"dwv_{tag}"] = pack(mod.linear_v.weight.grad)   # [N,K] storage order
        out[f"dwt_{tag}"] = pack(mod.linear_t.weight.grad)
    np.savez_compressed(os.path.join(HERE, name + ".npz"), x=_u16(x), wv=_u16(wv), wt=_u16(wt), g=_u16(g),
                        mask=mask.numpy(), **out)


def ffn_case(TorchFFN, name, B, S, d, h, seed, with_grads=False):
    gen = torch.Generator().manual_seed(seed)
    x = _bf16((B, S, d), 1.0, gen)
    names = ("w1", "w2", "w3", "u1", "u2", "u3")
    shapes = ((h, d), (d, h), (h, d), (h, d), (d, h), (h, d))
    ws = {n: _bf16(s, 0.02, gen) for n, s in zip(names, shapes)}
    mask = _mask(B, S, gen)
    out = {}
    for tag, dt in (("f32", torch.float32), ("bf16", torch.bfloat16)):
        mod = TorchFFN(d, h).to(dt)
        with torch.no_grad():
            for n in names:
                getattr(mod, n).weight.copy_(ws[n].to(dt))
        y = mod(x.to(dt), mask)
        out[f"y_{tag}"] = y.float().numpy() if dt == torch.float32 else _u16(y)
    if with_grads:
        # The reference module's forward is wrapped in torch.no_grad(); the undecorated function
        # (``__wrapped__``) is the same expression and lets autograd produce the FFN gradients the
        # reference itself never implemented (ffn_kernel/ops.py:34-38).  float32, [out, in] storage order.
        g = _bf16((B, S, d), 1.0, gen)
        mod = TorchFFN(d, h).float()
        with torch.no_grad():
            for n in names:
                getattr(mod, n).weight.copy_(ws[n].float())
        xi = x.float().requires_grad_(True)
        y = TorchFFN.forward.__wrapped__(mod, xi, mask)
        y.backward(g.float())
        out["g"] = _u16(g)
        out["dx_f32"] = xi.grad.numpy()
        for n in names:
            out[f"d{n}_f32"] = getattr(mod, n).weight.grad.numpy()
    np.savez_compressed(os.path.join(HERE, name + ".npz"), x=_u16(x), mask=mask.numpy(),
                        **{n: _u16(w) for n, w in ws.items()}, **out)


if __name__ == "__main__":
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py /path/to/reference-checkout")
    ref = sys.argv[1]
    TorchLinear, TorchFFN = _import_reference(ref)
    linear_case(TorchLinear, "linear_b2_s192_k64_n96", 2, 192, 64, 96, seed=1)
    linear_case(TorchLinear, "linear_b1_s200_k128_n192", 1, 200, 128, 192, seed=2)
    ffn_case(TorchFFN, "ffn_b2_s160_d64_h160", 2, 160, 64, 160, seed=3, with_grads=True)
    ffn_case(TorchFFN, "ffn_b1_s257_d128_h256", 1, 257, 128, 256, seed=4)
    print("golden vectors written to", HERE)
