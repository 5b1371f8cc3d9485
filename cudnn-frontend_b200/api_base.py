"""Check / compile / execute protocol shared by the operator classes.

Mirrors the contract of the reference's ``APIBase`` (python/cudnn/api_base.py:333-1020):
construct with *sample* tensors, ``check_support()`` validates shapes, strides, dtypes and
configuration and raises ``ValueError`` / ``NotImplementedError`` / ``RuntimeError`` for the
same classes of problems, ``compile()`` prepares launch state, ``execute()`` launches on
the caller's stream and allocates nothing.  ``TupleDict`` is the wrappers' return type
(python/cudnn/api_base.py:1023-1052).
"""

from __future__ import annotations

import logging
import threading
from dataclasses import dataclass
from typing import Iterable, Optional, Sequence, Tuple, Union

import torch


def ceil_div(a: int, b: int) -> int:
    return (a + b - 1) // b


def is_power_of_2(n: int) -> bool:
    return n > 0 and (n & (n - 1)) == 0


_warned = set()
_warned_lock = threading.Lock()


def warn_experimental_api_once(logger: logging.Logger, api_name: str) -> None:
    """One "experimental API" warning per class per process (python/cudnn/api_base.py:35-45)."""
    with _warned_lock:
        if api_name in _warned:
            return
        _warned.add(api_name)
    logger.warning("%s is an experimental API", api_name)


def _reset_experimental_api_warning_registry() -> None:
    with _warned_lock:
        _warned.clear()


@dataclass(frozen=True)
class TensorSpec:
    """What validation needs to know about a tensor, without holding its storage."""

    name: str
    dtype: torch.dtype
    shape: Tuple[int, ...]
    stride: Tuple[int, ...]
    device: torch.device

    @staticmethod
    def of(t: Optional[torch.Tensor], name: str) -> Optional["TensorSpec"]:
        if t is None:
            return None
        if not isinstance(t, torch.Tensor):
            raise TypeError(f"{name} must be a torch.Tensor, got {type(t).__name__}")
        return TensorSpec(name, t.dtype, tuple(t.shape), tuple(t.stride()), t.device)

    def logical(self) -> "TensorSpec":
        """Shape and strides in elements.  ``float4_e2m1fn_x2`` packs two elements per byte along its
        contiguous dimension: that extent doubles and every other stride doubles, as the reference's
        ``_tensor_shape`` / ``_tensor_stride`` do (python/cudnn/api_base.py:650-713)."""
        if self.dtype != torch.float4_e2m1fn_x2 or 1 not in self.stride:
            return self
        inner = self.stride.index(1)
        shape = tuple(d * 2 if i == inner else d for i, d in enumerate(self.shape))
        stride = tuple(st if i == inner else st * 2 for i, st in enumerate(self.stride))
        return TensorSpec(self.name, self.dtype, shape, stride, self.device)


class TupleDict(dict):
    """A dict whose iteration yields values in insertion order (so it unpacks like a tuple)
    and that also accepts integer positions as keys."""

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self._order = list(super().keys())

    def __iter__(self):
        return (dict.__getitem__(self, k) for k in self._order)

    def __getitem__(self, key):
        if isinstance(key, int):
            if not 0 <= key < len(self._order):
                raise IndexError(f"index {key} out of range for TupleDict with {len(self._order)} items")
            return dict.__getitem__(self, self._order[key])
        return dict.__getitem__(self, key)


_FP8 = (torch.float8_e4m3fn, torch.float8_e5m2)
_FP4 = (torch.float4_e2m1fn_x2, torch.uint8)  # the reference reads uint8 operands as raw packed FP4


def as_packed_fp4(t):
    """A ``uint8`` A / B operand is raw packed FP4 (two E2M1 values per byte), as in the reference
    (``interpret_uint8_as_fp4x2``, python/cudnn/api_base.py:602-609): seen as ``float4_e2m1fn_x2`` from here on.
    Anything else passes through."""
    if isinstance(t, torch.Tensor) and t.dtype == torch.uint8:
        return t.view(torch.float4_e2m1fn_x2)
    return t


def packed_fp4_dtype(dtype):
    """The dtype counterpart of :func:`as_packed_fp4` (for ``b_dtype`` of the discrete-weight forms)."""
    return torch.float4_e2m1fn_x2 if dtype == torch.uint8 else dtype


class OperatorBase:
    """Common state machine and validators of the operator classes."""

    def __init__(self):
        self._logger = logging.getLogger(f"{__name__}.{type(self).__name__}")
        self._is_supported = False
        self._is_compiled = False
        warn_experimental_api_once(self._logger, type(self).__name__)

    # -- validators (same exception types as the reference's) ---------------------------------
    @staticmethod
    def _value_error_if(cond: bool, msg: str) -> None:
        if cond:
            raise ValueError(msg)

    @staticmethod
    def _not_implemented_error_if(cond: bool, msg: str) -> None:
        if cond:
            raise NotImplementedError(msg)

    @staticmethod
    def _is_fp8(dtype) -> bool:
        return dtype in _FP8

    @staticmethod
    def _is_fp4x2(dtype) -> bool:
        return dtype in _FP4

    def _check_shape(self, spec: Optional[TensorSpec], shape: Sequence[int], label: str) -> None:
        if spec is None:
            return
        self._value_error_if(tuple(spec.shape) != tuple(shape), f"{label} must have shape {tuple(shape)}, got {tuple(spec.shape)}")

    def _check_stride(self, spec: Optional[TensorSpec], stride: Sequence[int], msg: str) -> None:
        """Strides must match on every dimension whose extent is larger than one."""
        if spec is None:
            return
        ok = all(sz <= 1 or st == want for sz, st, want in zip(spec.shape, spec.stride, stride))
        self._value_error_if(not ok, f"{spec.name}: {msg} (expected strides {tuple(stride)}, got {spec.stride})")

    def _check_dtype(self, spec_or_dtype, allowed: Union[torch.dtype, Iterable[torch.dtype]], label: str, extra: str = ""):
        if spec_or_dtype is None:
            return None
        dtype = spec_or_dtype.dtype if isinstance(spec_or_dtype, TensorSpec) else spec_or_dtype
        allowed = (allowed,) if isinstance(allowed, torch.dtype) else tuple(allowed)
        self._value_error_if(dtype not in allowed, f"{label} dtype must be one of {allowed}, got {dtype}. {extra}".strip())
        return dtype

    @staticmethod
    def _require_sm100() -> None:
        if not torch.cuda.is_available():
            raise RuntimeError("CUDA is not available")
        major, minor = torch.cuda.get_device_capability(torch.cuda.current_device())
        if major * 10 + minor < 100:
            raise RuntimeError(f"requires SM100+ compute capability, found SM{major * 10 + minor}")

    def _ensure_compiled(self) -> None:
        if not self._is_compiled:
            raise RuntimeError(f"{type(self).__name__}: call check_support() and compile() before execute()")

    # -- protocol -----------------------------------------------------------------------------
    def check_support(self) -> bool:  # pragma: no cover - abstract
        raise NotImplementedError

    def compile(self) -> None:  # pragma: no cover - abstract
        raise NotImplementedError

    def execute(self, *args, **kwargs) -> None:  # pragma: no cover - abstract
        raise NotImplementedError

    def __call__(self, *args, **kwargs):
        return self.execute(*args, **kwargs)


def check_tile_and_cluster(op: OperatorBase, mma_tiler_mn, cluster_shape_mn, m_aligned: int, *, only_n256: bool) -> None:
    """The reference's tile / cluster / alignment rules
    (python/cudnn/grouped_gemm/grouped_gemm_swiglu/api.py:354-403).  The kernels here always run
    128 x 256 CTA tiles, so the two parameters are accepted as hints after validation; groups may
    be padded to any multiple of 128 rows (the reference insists on exactly 256)."""
    use_2cta = mma_tiler_mn[0] == 256
    op._value_error_if(not use_2cta and mma_tiler_mn[0] not in (64, 128), f"MMA tiler M must be 64 or 128 when use_2cta_instrs=False, got {mma_tiler_mn[0]}")
    op._value_error_if(mma_tiler_mn[1] not in ((256,) if only_n256 else (128, 256)), f"MMA tiler N must be {'256' if only_n256 else '128 or 256'}, got {mma_tiler_mn[1]}")
    cm, cn = cluster_shape_mn
    op._value_error_if(cm % (2 if use_2cta else 1) != 0, f"cluster_shape_mn[0] must be divisible by 2 when use_2cta_instrs=True, got {cm}")
    op._value_error_if(
        not (cm > 0 and cn > 0 and cm <= 4 and cn <= 4 and cm * cn <= 16 and is_power_of_2(cm) and is_power_of_2(cn)),
        f"Invalid cluster shape: expected powers of 2 with product <= 16, got {cm},{cn}",
    )
    cluster_tiler_m = (cm // (2 if use_2cta else 1)) * mma_tiler_mn[0]
    op._value_error_if(cluster_tiler_m not in (128, 256), f"Invalid cluster tiler shape: expected cluster_tiler_m in {{128, 256}}, got {cluster_tiler_m}")
    op._value_error_if(m_aligned <= 0 or m_aligned % 128 != 0, f"m_aligned must be a positive multiple of 128, got {m_aligned}")


def pick_tile_mode(mma_tiler_mn, m_aligned: int):
    """Tile mode of the launch from the caller's tiler and group alignment: a 128-row tiler maps to
    single-CTA tiles; groups padded to a multiple of 256 rows waste nothing in 256-row CTA-pair
    tiles, whatever their size; otherwise the library decides from the average group size."""
    if mma_tiler_mn[0] <= 128:
        return "single"
    if m_aligned % 256 == 0:
        return "pair"
    return None
