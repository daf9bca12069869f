"""ctypes binding of ``libgrain_b200.so`` (declared in ``include/grain_gemm_b200.h``).

Mirrors the reference's native bridges (``src/grain_gemm/kernels/cuda.py:59-125`` and
``src/grain_gemm/kernels/moe_gather.py:29-107`` there): the library is loaded once, only
when its manifest matches the sources beside it, every call goes to torch's current
stream, and a non-zero status becomes a ``RuntimeError`` with the decoded text.  There
is no fallback: a missing or stale library is an error.
"""

from __future__ import annotations

import ctypes
from functools import lru_cache

import torch

from . import build as _build

_VOID = ctypes.c_void_p
_INT = ctypes.c_int
_LL = ctypes.c_longlong
_SIZE = ctypes.c_size_t

OUT_DTYPE = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}
VARIANTS = {
    "auto": 0, "simt": 1, "tc_n256": 2, "tc_n128": 3, "tc_n64": 4,
    "tc_pair_n256": 5, "tc_pair_n128": 6, "tc_splitk": 7, "gemv": 8,
}
VARIANT_NAMES = {value: key for key, value in VARIANTS.items()}

# name -> (restype, argtypes); the order is the order of the C declaration.
_SIGNATURES = {
    "gg_abi_version": (_INT, []),
    "gg_error_string": (ctypes.c_char_p, [_INT]),
    "grain_cuda_error_string": (ctypes.c_char_p, [_INT]),
    "gg_int8_gemm": (_INT, [_VOID] * 5 + [_INT] * 3 + [_LL] * 9 + [_INT] * 3 + [_VOID]),
    "gg_int8_gemm_workspace_bytes": (_SIZE, [_INT] * 4),
    "gg_int8_gemm_ws": (_INT, [_VOID] * 5 + [_INT] * 3 + [_LL] * 9 + [_INT] * 3 + [_VOID, _SIZE, _VOID]),
    "gg_int8_gemm_select": (_INT, [_VOID] * 3 + [_INT] * 3 + [_LL] * 5 + [_INT] * 2),
    "gg_int8_gemm_partials": (_INT, [_VOID] * 6 + [_INT] * 3 + [_LL] * 8 + [_INT, _VOID]),
    "grain_cute_g256": (_INT, [_VOID] * 5 + [_INT] * 4 + [_VOID]),
    "gg_moe_route_workspace_bytes": (_SIZE, [_INT] * 3),
    "gg_moe_route": (_INT, [_VOID, _INT, _VOID, _INT, _INT, _INT] + [_VOID] * 7 + [_SIZE, _VOID]),
    "gg_moe_route_noalloc": (_INT, [_VOID, _INT, _VOID, _INT, _INT, _INT] + [_VOID] * 6 + [_VOID]),
    "gg_moe_route_noalloc_capacity_bytes": (_SIZE, []),
    "gg_moe_tile_capacity": (_INT, [_INT] * 3),
    "gg_moe_tiles": (_INT, [_VOID, _INT, _INT, _INT, _VOID, _VOID, _VOID]),
    "gg_moe_topk": (_INT, [_VOID, _INT, _INT, _INT, _INT, _VOID, _VOID, _INT, _VOID]),
    "gg_moe_route_topk": (_INT, [_VOID, _INT, _VOID, _INT, _INT, _INT, _VOID, _VOID, _INT] + [_VOID] * 7),
    "gg_quantize_rows": (_INT, [_VOID, _INT, _LL, _INT, _INT, _VOID, _VOID, _VOID]),
    "gg_moe_silu_table": (_INT, [_VOID, _INT, _VOID]),
    "gg_moe_gate_up_scratch_bytes": (_SIZE, [_INT] * 5),
    "gg_moe_gate_up": (_INT, [_VOID] * 8 + [_INT, _INT] + [_VOID] * 3 + [_INT] * 8 + [_VOID]),
    "gg_moe_down": (_INT, [_VOID] * 7 + [_INT, _INT, _VOID, _VOID] + [_INT] * 5 + [_VOID]),
    "gg_ep_plan": (_INT, [_VOID, _INT, _VOID] + [_INT] * 5 + [_VOID] * 4),
    "gg_ep_dispatch": (_INT, [_VOID, _VOID, _VOID, _INT, _VOID, _VOID] + [_INT] * 8 + [_VOID] * 6),
    "gg_ep_row_mask": (_INT, [_VOID, _INT, _INT, _INT, _VOID, _VOID]),
    "gg_ep_row_destination": (_INT, [_VOID, _VOID] + [_INT] * 6 + [_VOID] * 5),
    "gg_peer_alloc": (_INT, [_SIZE, ctypes.POINTER(_VOID)]),
    "gg_peer_free": (_INT, [_VOID]),
    "gg_peer_export": (_INT, [_VOID, _VOID]),
    "gg_peer_import": (_INT, [_VOID, ctypes.POINTER(_VOID)]),
    "gg_peer_release": (_INT, [_VOID]),
    "gg_moe_combine": (_INT, [_VOID] * 4 + [_INT] * 4 + [_VOID]),
    "gg_device_status": (_INT, [ctypes.POINTER(_INT), _VOID]),
    "gg_selftest_wait_timeout": (_INT, [_LL, _VOID, _VOID]),
    "gg_report_to_host": (_INT, [_VOID, _INT, _VOID, _VOID]),
}

EXPORTS = tuple(_SIGNATURES)


@lru_cache(maxsize=1)
def library():
    """Load the library; raise ``RuntimeError`` when it is absent or stale."""
    if not _build.LIBRARY.is_file():
        raise RuntimeError(
            f"{_build.LIBRARY.name} is not built; run `python -m grain_gemm_b200.build`")
    if not _build.is_current():
        raise RuntimeError(
            f"{_build.LIBRARY.name} does not match the sources beside it; "
            "rebuild with `python -m grain_gemm_b200.build`")
    lib = ctypes.CDLL(str(_build.LIBRARY))
    for name, (restype, argtypes) in _SIGNATURES.items():
        function = getattr(lib, name)
        function.restype = restype
        function.argtypes = argtypes
    if lib.gg_abi_version() != _build.ABI_VERSION:
        raise RuntimeError("libgrain_b200.so reports a different ABI version than this package")
    return lib


def is_available():
    try:
        library()
    except (OSError, RuntimeError, AttributeError):
        return False
    return True


def check(status, what):
    if status:
        text = library().gg_error_string(status).decode()
        raise RuntimeError(f"{what} failed: {text} (status {status})")


def stream_pointer(device):
    return _VOID(torch.cuda.current_stream(device).cuda_stream)


def pointer(tensor):
    return _VOID(tensor.data_ptr()) if tensor is not None else _VOID(0)


def device_status(device=None):
    """Read and clear the device status word (synchronises the current stream)."""
    value = _INT(0)
    check(library().gg_device_status(ctypes.byref(value), stream_pointer(device)), "gg_device_status")
    return value.value
