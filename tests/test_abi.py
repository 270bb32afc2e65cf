"""The C-ABI library: it loads, exports every function include/ffnk.h declares, the ctypes
binding covers the same set, and argument checks reject bad calls before any launch."""
import ctypes
import os
import re

import pytest

from conftest import ROOT


def declared_functions():
    text = open(os.path.join(ROOT, "include", "ffnk.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ffnk_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = declared_functions()
    for must in ("ffnk_route", "ffnk_linear_fwd", "ffnk_linear_bwd", "ffnk_ffn_gateup", "ffnk_ffn_down",
                 "ffnk_ffn_decode", "ffnk_read_status"):
        assert must in names


def test_library_exports_every_declared_symbol(libffnk):
    raw = ctypes.CDLL(libffnk._name)
    for name in declared_functions():
        assert hasattr(raw, name), f"{name} is declared in include/ffnk.h but not exported"


def test_ctypes_binding_covers_the_header():
    from ffn_kernel_b200 import _lib
    assert sorted(_lib.SIGNATURES) == declared_functions()


def test_pure_host_functions(libffnk):
    L = libffnk
    assert L.ffnk_version() >= 100
    assert L.ffnk_route_capacity(0) == 0
    assert L.ffnk_route_capacity(1) == 128
    assert L.ffnk_route_capacity(128) == 128
    assert L.ffnk_route_capacity(129) == 256
    assert L.ffnk_route_workspace_bytes(1) >= 8
    assert L.ffnk_decode_max_tokens() >= 1
    assert L.ffnk_status_string(0) == b"ok"
    assert b"null" in L.ffnk_status_string(-1)


def test_decode_table_entry(libffnk):
    # up to 80 tokens at small FFNs, about 57 at d=1024/h=2816, a single token at wide FFNs (the GEMM path with
    # its split-K down projection is ahead there); never beyond the kernel's capacity; monotone in M
    L = libffnk
    assert L.ffnk_decode_max_tokens() == 80 and L.ffnk_decode_capacity() == 127
    for d, h, lo, hi in ((1024, 2816, 50, 64), (4096, 11008, 1, 1), (2048, 8192, 1, 1), (256, 520, 80, 80),
                         (512, 1024, 80, 80)):
        takes = [bool(L.ffnk_ffn_takes_decode(M, d, h)) for M in range(0, 130)]
        limit = max(M for M, t in enumerate(takes) if t)
        assert lo <= limit <= hi, (d, h, limit)
        assert not takes[0] and all(takes[1:limit + 1]) and not any(takes[limit + 1:])


def test_tune_override_names(libffnk):
    L = libffnk
    for name in (b"pair", b"narrow", b"permute", b"epi_warps", b"group_m", b"wgrad_pair", b"max_run_rows",
                 b"copy_threshold", b"verbose", b"route_resident", b"ksplit", b"early_start"):
        assert L.ffnk_tune_override(name, -1) == 0
    assert L.ffnk_tune_override(b"no_such_entry", 1) < 0
    assert L.ffnk_tune_override(None, 1) < 0


def test_argument_errors_are_reported_before_any_launch(libffnk):
    L = libffnk
    # null pointers
    assert L.ffnk_linear_fwd(None, 8, None, None, 1, 8, None, None, None, 8, None, 16, 8, 8, None, None) == -1
    assert L.ffnk_ffn_down(None, 8, None, None, 1, 8, None, None, None, 8, 16, 8, 8, None, None) == -1
    assert L.ffnk_route(None, 16, None, None, None, None, None) == -1
    # sizes: not a multiple of 8 / negative
    fake = ctypes.c_void_p(0x1000)
    assert L.ffnk_linear_fwd(fake, 8, fake, fake, 1, 8, fake, fake, fake, 8, None, 16, 12, 8, fake, None) == -2
    assert L.ffnk_linear_fwd(fake, 8, fake, fake, 1, 8, fake, fake, fake, 8, None, -1, 8, 8, fake, None) == -2
    # misaligned leading dimension
    assert L.ffnk_linear_fwd(fake, 9, fake, fake, 1, 8, fake, fake, fake, 8, None, 16, 8, 8, fake, None) == -3
    # decode: too many tokens, wrong weight layout
    n = L.ffnk_decode_capacity()
    assert 1 <= L.ffnk_decode_max_tokens() <= n
    args = [fake, 8, fake, fake, fake, fake, fake, fake, 1, 8, 1, 8, fake, fake, fake, 8]
    assert L.ffnk_ffn_decode(*args, n + 1, 8, 8, fake, None) == -2
    args[8], args[9] = 8, 1
    assert L.ffnk_ffn_decode(*args, 1, 8, 8, fake, None) == -4
    # empty problems succeed without touching the device
    assert L.ffnk_linear_fwd(None, 8, None, None, 1, 8, None, None, None, 8, None, 0, 8, 8, None, None) == 0


def test_python_wrappers_refuse_cpu_tensors():
    import torch
    from ffn_kernel_b200 import MaskedFFN, MaskedLinear, route
    x = torch.zeros(16, 8, dtype=torch.bfloat16)
    w = torch.zeros(8, 8, dtype=torch.bfloat16)
    m = torch.zeros(16, dtype=torch.bool)
    with pytest.raises(RuntimeError, match="CUDA"):
        MaskedLinear.apply(x, w, w, m)
    with pytest.raises(RuntimeError, match="CUDA"):
        MaskedFFN.apply(x, w, w, w, w, w, w, m)
    with pytest.raises(RuntimeError, match="CUDA"):
        route(m)


def test_reference_import_surface():
    import ffn_kernel
    import ffn_kernel_b200
    assert ffn_kernel.MaskedLinear is ffn_kernel_b200.MaskedLinear
    assert ffn_kernel.MaskedFFN is ffn_kernel_b200.MaskedFFN


def test_header_is_valid_c99_and_cxx():
    # the boundary is a C ABI: the header must compile as C (no C++-isms) and as C++ (extern "C" guards)
    import shutil
    import subprocess
    header = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "include", "ffnk.h")
    for compiler, flags in (("gcc", ["-std=c99", "-x", "c"]), ("g++", ["-std=c++17", "-x", "c++"])):
        exe = shutil.which(compiler)
        if exe is None:
            pytest.skip(f"{compiler} not installed")
        res = subprocess.run([exe, *flags, "-Wall", "-Werror", "-pedantic", "-fsyntax-only", header],
                             capture_output=True, text=True)
        assert res.returncode == 0, res.stderr
