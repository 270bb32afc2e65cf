"""ctypes binding of libffnk.so, the C-ABI library that holds every CUDA kernel.

There is no fallback: if the library is missing or a call is rejected, an exception
is raised.  Nothing in this package computes on the CPU or through another library.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_int, c_int32, c_int64, c_void_p, POINTER

_HERE = os.path.dirname(os.path.abspath(__file__))
# FFNK_LIB points at another build of the same library (A/B runs of kernel variants)
LIB_PATH = os.environ.get("FFNK_LIB") or os.path.join(_HERE, "lib", "libffnk.so")

_I32P = POINTER(c_int32)

# name -> (restype, argtypes); mirrors include/ffnk.h declaration by declaration
SIGNATURES = {
    "ffnk_version": (c_int, []),
    "ffnk_route_capacity": (c_int64, [c_int64]),
    "ffnk_route_workspace_bytes": (c_int64, [c_int64]),
    "ffnk_route": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "ffnk_route_noalloc": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p]),
    "ffnk_linear_fwd": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_int64, c_void_p, c_void_p,
                                c_void_p, c_int64, c_void_p, c_int64, c_int64, c_int64, c_void_p, c_void_p]),
    "ffnk_linear_bwd": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_int64,
                                c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p,
                                c_int64, c_int64, c_int64, c_void_p, c_void_p]),
    "ffnk_linear_bwd_parts": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_int64,
                                      c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p,
                                      c_int64, c_int64, c_int64, c_int, c_void_p, c_void_p]),
    "ffnk_route_permute_max_tokens": (c_int64, []),
    "ffnk_route_permute_rows": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_void_p,
                                        c_int64, c_void_p]),
    "ffnk_permute_rows": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                                  c_void_p]),
    "ffnk_ffn_gateup": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64,
                                c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int64, c_int64, c_int64,
                                c_void_p, c_void_p]),
    "ffnk_ffn_down": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_int64, c_void_p, c_void_p,
                              c_void_p, c_int64, c_int64, c_int64, c_int64, c_void_p, c_void_p]),
    "ffnk_ffn_down_to_peers": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_int64, c_void_p, c_void_p,
                                       POINTER(c_void_p), c_int, c_int, c_int64, c_int64, c_int64, c_int64, c_int64,
                                       c_void_p, c_void_p]),
    "ffnk_sum_row_blocks": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p, c_int64, c_void_p]),
    "ffnk_peer_barrier": (c_int, [POINTER(c_void_p), c_int, c_int, c_int32, c_int64, c_void_p, c_void_p]),
    "ffnk_sum_row_blocks_to_peers": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_int64, POINTER(c_void_p),
                                             c_int, c_int64, c_int64, c_int, c_void_p]),
    "ffnk_decode_max_tokens": (c_int, []),
    "ffnk_decode_capacity": (c_int, []),
    "ffnk_ffn_takes_decode": (c_int, [c_int64, c_int64, c_int64]),
    "ffnk_ffn_decode": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                c_int64, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_int64,
                                c_int64, c_int64, c_int64, c_void_p, c_void_p]),
    "ffnk_ffn_workspace_bytes": (c_int64, [c_int64, c_int64, c_int64]),
    "ffnk_ffn_permute_first": (c_int, [c_int64, c_int64, c_int64]),
    "ffnk_ffn_forward": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                 c_int64, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_int64, c_void_p, c_int64,
                                 c_int64, c_int64, c_int64, c_int, c_void_p, c_void_p]),
    "ffnk_ffn_forward_train": (c_int, [c_void_p, c_int64] + [c_void_p] * 6 + [c_int64] * 4 + [c_void_p] * 9
                               + [c_int64] * 4 + [c_void_p, c_void_p]),
    "ffnk_ffn_backward": (c_int, [c_void_p, c_int64] + [c_void_p] * 10 + [c_int64] * 4 + [c_void_p] * 6 + [c_int64]
                          + [c_void_p] * 6 + [c_int64] * 3 + [c_void_p, c_void_p]),
    "ffnk_read_status": (c_int, [c_void_p, c_int, c_void_p]),
    "ffnk_selftest_bounded_wait": (c_int, [c_void_p, c_int64, c_void_p]),
    "ffnk_set_sm_margin": (c_int, [c_int]),
    "ffnk_debug_profile_buffer": (c_int, [c_void_p]),
    "ffnk_tune_override": (c_int, [c_char_p, c_int]),
    "ffnk_status_string": (c_char_p, [c_int]),
}

_lib = None


class FfnkError(RuntimeError):
    """A call into libffnk.so was rejected or reported a device-side error."""

    def __init__(self, where: str, code: int):
        self.code = code
        msg = lib().ffnk_status_string(code).decode() if _lib is not None else "?"
        super().__init__(f"{where}: {msg} (code {code})")


def lib() -> ctypes.CDLL:
    """The loaded library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: the CUDA kernels have not been built. "
                "Run `python -m ffn_kernel_b200.build` (needs nvcc); there is no CPU or Triton fallback.")
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)      # AttributeError if the library lacks a declared symbol
            fn.restype, fn.argtypes = res, args
        _lib = handle
        _apply_env_overrides(handle)
    return _lib


# Tile-table overrides for measurements (`python -m ffn_kernel_b200.tune`, the forced-variant test runs):
# FFNK_PAIR, FFNK_NARROW, FFNK_PERMUTE, FFNK_EPI_WARPS, FFNK_GROUP_M, FFNK_WGRAD_PAIR, FFNK_MAX_RUN_ROWS,
# FFNK_COPY_THRESHOLD, FFNK_VERBOSE, FFNK_ROUTE_RESIDENT, FFNK_KSPLIT, FFNK_EARLY_START are read HERE, once, and handed to the library through
# ffnk_tune_override; the library itself never looks at the environment.
_ENV_OVERRIDES = ("pair", "narrow", "permute", "epi_warps", "group_m", "wgrad_pair", "max_run_rows",
                  "copy_threshold", "verbose", "route_resident", "ksplit", "early_start")


def _apply_env_overrides(handle) -> None:
    for name in _ENV_OVERRIDES:
        raw = os.environ.get("FFNK_" + name.upper())
        if raw is None or raw == "":
            continue
        try:
            value = int(raw)
        except ValueError:
            raise RuntimeError(f"FFNK_{name.upper()}={raw!r} is not an integer") from None
        check(f"ffnk_tune_override({name})", handle.ffnk_tune_override(name.encode(), value))


def check(where: str, code: int) -> None:
    if code != 0:
        raise FfnkError(where, code)
