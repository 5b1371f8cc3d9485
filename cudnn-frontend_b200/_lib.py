"""ctypes binding of libb200moe.so (declarations mirror include/b200moe.h).

There is no fallback: if the library is missing the import of any operator fails loudly.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, c_char_p, c_float, c_int32, c_int64, c_void_p

from . import _build

E_NULL, E_SHAPE, E_ALIGN, E_UNSUPPORTED, E_WORKSPACE, E_DEVICE = -1, -2, -3, -4, -5, -6
DTYPE_BF16, DTYPE_E4M3, DTYPE_F16, DTYPE_F32, DTYPE_E5M2, DTYPE_E2M1 = 0, 1, 2, 3, 4, 5
ACT_SWIGLU, ACT_GEGLU = 0, 1
ABI_VERSION = 7  # b200moe_abi_version() of the header these declarations mirror
FLAG_DISCRETE_COL_SFD = 1
FLAG_TILE_SINGLE = 2
FLAG_TILE_PAIR = 4
FLAG_DYNAMIC_SCHED = 8
FLAG_B_NMAJOR = 16
FLAG_OFFSETS_HAVE_PREV = 32
FLAG_TEST_SKIP_B_LOADS = 64
FLAG_ACCUMULATE = 128
WORKSPACE_DISCRETE, WORKSPACE_DYNAMIC_SCHED = 1, 2
NOALLOC_MAX_EXPERTS = 256


class GemmArgs(Structure):
    _fields_ = [
        ("a", c_void_p),
        ("sfa", c_void_p),
        ("b", c_void_p),
        ("sfb", c_void_p),
        ("b_ptrs", c_void_p),
        ("sfb_ptrs", c_void_p),
        ("padded_offsets", c_void_p),
        ("alpha", c_void_p),
        ("prob", c_void_p),
        ("norm_const", c_void_p),
        ("c", c_void_p),
        ("d", c_void_p),
        ("d_col", c_void_p),
        ("amax", c_void_p),
        ("sfd_row", c_void_p),
        ("sfd_col", c_void_p),
        ("workspace", c_void_p),
        ("workspace_bytes", c_int64),
        ("m_rows", c_int64),
        ("n", c_int64),
        ("k", c_int64),
        ("num_experts", c_int32),
        ("d_dtype", c_int32),
        ("flags", c_int32),
        ("sm_margin", c_int32),
        ("d_row_map", c_void_p),
        ("d_peer_ptrs", c_void_p),
        ("d_peer_slots", c_int64),
        ("bias", c_void_p),
        ("bias_dtype", c_int32),
        ("act_func", c_int32),
        ("ab_dtype", c_int32),
        ("c_dtype", c_int32),
        ("wait_limit_ms", c_int32),
        ("sched_light_m_tiles", c_int32),
        ("l2_stream_m_tiles", c_int32),
        ("sf_vec_size", c_int32),
        ("sf_dtype", c_int32),
        ("beta", c_void_p),
        ("dprob", c_void_p),
    ]


_SIGNATURES = {
    "b200moe_fc1_swiglu": (ctypes.c_int, [POINTER(GemmArgs), c_void_p]),
    "b200moe_fc2_quant": (ctypes.c_int, [POINTER(GemmArgs), c_void_p]),
    "b200moe_dswiglu": (ctypes.c_int, [POINTER(GemmArgs), c_void_p]),
    "b200moe_wgrad": (ctypes.c_int, [POINTER(GemmArgs), c_void_p]),
    "b200moe_fc1_swiglu_discrete_noalloc": (ctypes.c_int, [POINTER(GemmArgs), c_void_p]),
    "b200moe_workspace_bytes": (c_int64, [c_int32, c_int32]),
    "b200moe_quantize_mxfp8": (ctypes.c_int, [c_void_p, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_void_p]),
    "b200moe_route": (
        ctypes.c_int,
        [c_void_p, c_int64, c_int32, c_int32, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
    ),
    "b200moe_route_scratch_bytes": (c_int64, [c_int64, c_int32]),
    "b200moe_zero_pad_rows": (ctypes.c_int, [c_void_p, c_void_p, c_void_p, c_int32, c_int64, c_void_p, c_void_p]),
    "b200moe_scatter_rows": (
        ctypes.c_int,
        [c_void_p, c_void_p, c_int64, c_int32, c_int64, c_void_p, c_void_p, c_void_p, c_void_p],
    ),
    "b200moe_dispatch_quantize": (
        ctypes.c_int,
        [c_void_p, c_void_p, c_void_p, c_int64, c_int32, c_int64, c_void_p, c_void_p, c_void_p, c_void_p],
    ),
    "b200moe_place_quantized_rows": (
        ctypes.c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_void_p],
    ),
    "b200moe_dispatch_quantize_peer": (
        ctypes.c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int32, c_int64, c_int32, c_int32, c_int32, c_int64,
         c_int64, c_void_p, c_void_p, c_void_p],
    ),  # fmt: skip
    "b200moe_dispatch_quantize_peer_chunk": (
        ctypes.c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int32, c_int64, c_int32, c_int32, c_int32, c_int64,
         c_int64, c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_int32, c_void_p],
    ),  # fmt: skip
    "b200moe_copy_segments": (ctypes.c_int, [c_int32, POINTER(c_int64), POINTER(c_int64), POINTER(c_int64), c_void_p]),
    "b200moe_dispatch_record_pitch": (ctypes.c_int, [c_int64]),
    "b200moe_unpack_dispatch_records": (ctypes.c_int, [c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_void_p]),
    "b200moe_peer_alloc": (ctypes.c_int, [c_int64, POINTER(c_void_p), c_void_p]),
    "b200moe_peer_open": (ctypes.c_int, [c_void_p, POINTER(c_void_p)]),
    "b200moe_peer_close": (ctypes.c_int, [c_void_p]),
    "b200moe_peer_free": (ctypes.c_int, [c_void_p]),
    "b200moe_gather_rows": (ctypes.c_int, [c_void_p, c_void_p, c_int64, c_int64, c_void_p, c_void_p]),
    "b200moe_combine_rows": (ctypes.c_int, [c_void_p, c_void_p, c_int64, c_int32, c_int64, c_void_p, c_void_p]),
    "b200moe_last_error": (c_char_p, []),
    "b200moe_device_status": (ctypes.c_int, [ctypes.c_int]),
    "b200moe_abi_version": (ctypes.c_int, []),
}

EXPORTED_SYMBOLS = tuple(_SIGNATURES)

_lib = None


def load() -> ctypes.CDLL:
    """Load (building first when nvcc is present and the library is stale) and type the library."""
    global _lib
    if _lib is not None:
        return _lib
    override = os.environ.get("B200MOE_LIBRARY")  # load a prebuilt library from another path
    path = override or _build.LIB_PATH
    if not override and _build.is_stale():
        try:
            _build.build()
        except RuntimeError:
            if not os.path.exists(path):
                raise
    if not os.path.exists(path):
        raise RuntimeError(f"{path} is missing: build it with `python -m cudnn_frontend_b200._build` (needs nvcc)")
    lib = ctypes.CDLL(path)
    lib.b200moe_abi_version.restype = ctypes.c_int
    if lib.b200moe_abi_version() != ABI_VERSION:
        raise RuntimeError(f"{path} has ABI version {lib.b200moe_abi_version()}, this package needs {ABI_VERSION}: rebuild the library")
    for name, (restype, argtypes) in _SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def last_error() -> str:
    return load().b200moe_last_error().decode()


def check(rc: int) -> None:
    """Map a C-ABI status to the exception type the reference raises for that class of error."""
    if rc == 0:
        return
    msg = last_error() or f"libb200moe error {rc}"
    if rc == E_UNSUPPORTED:
        raise NotImplementedError(msg)
    if rc < 0 and rc != E_DEVICE:
        raise ValueError(msg)
    raise RuntimeError(msg)
