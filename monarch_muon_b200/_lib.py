"""ctypes binding of libmonarch_muon_b200.so (the C ABI in include/monarch_muon_b200.h).

There is no fallback: if the library is missing it is built with nvcc, and if
that fails, or no CUDA device is present when a kernel is requested, the call
raises.  Nothing here computes on the CPU.
"""
from __future__ import annotations

import ctypes as C
import os
import threading

import torch

from . import build as _build

BF16, F32 = 0, 1
STATE_FP8_ABSMAX, STATE_FP8_EXPAND, STATE_BF16, STATE_F32 = 0, 1, 2, 3
DIV_IEEE, DIV_FULL, DIV_IEEE_STRICT = 0, 1, 2
# Default arithmetic of the FP8 quantisers: the GPU instructions the reference's Triton kernels compile to
# (div.full.f32, sqrt.approx.ftz.f32, library powf).  With it the absmax codec reproduces the reference's
# kernel bit for bit on the same GPU; DIV_IEEE reproduces the CPU oracle bit for bit instead.
DIV_DEFAULT = DIV_FULL
DIV_NAMES = {"full": DIV_FULL, "ieee": DIV_IEEE, "ieee_strict": DIV_IEEE_STRICT}
NS_TCGEN05, NS_SIMT, NS_TCGEN05_MULTI = 0, 1, 2
STATUS_NAMES = {0x101: "TMA producer waited too long for a free stage", 0x102: "MMA issuer waited too long for operands",
                0x103: "MMA issuer waited too long for a drained accumulator",
                0x104: "epilogue waited too long for an accumulator", 0x105: "a role waited too long for its next tile",
                0x106: "tile scheduler waited too long for a slot", 0x1F0: "wait probe expired (expected)"}
STATUS_WAIT_PROBE = 0x1F0
GEMM_K, GEMM_MN, GEMM_SYM = 0, 1, 2


class MomentumSeg(C.Structure):
    _fields_ = [("grad", C.c_void_p), ("state", C.c_void_p), ("scale", C.c_void_p), ("expand", C.c_void_p),
                ("sqrt_minmax", C.c_void_p), ("m_bf16", C.c_void_p), ("numel", C.c_int64),
                ("block_elems", C.c_int64), ("first_block", C.c_int64)]


class UpdateSeg(C.Structure):
    _fields_ = [("weight", C.c_void_p), ("ortho", C.c_void_p), ("numel", C.c_int64)]


class GradSeg(C.Structure):
    _fields_ = [("grad", C.c_void_p), ("numel", C.c_int64), ("dtype", C.c_int32), ("pad_", C.c_int32)]


class AdamWSeg(C.Structure):
    _fields_ = [("param", C.c_void_p), ("grad", C.c_void_p), ("exp_avg", C.c_void_p), ("exp_avg_sq", C.c_void_p),
                ("numel", C.c_int64), ("step", C.c_int32), ("pad_", C.c_int32)]


class AdamWFp8Seg(C.Structure):
    _fields_ = [("param", C.c_void_p), ("grad", C.c_void_p),
                ("exp_avg", C.c_void_p), ("scale_exp_avg", C.c_void_p), ("expand_exp_avg", C.c_void_p),
                ("sqrt_minmax_exp_avg", C.c_void_p),
                ("exp_avg_sq", C.c_void_p), ("scale_exp_avg_sq", C.c_void_p), ("expand_exp_avg_sq", C.c_void_p),
                ("sqrt_minmax_exp_avg_sq", C.c_void_p),
                ("numel", C.c_int64), ("step", C.c_int32), ("pad_", C.c_int32)]


class MasterUpdateSeg(C.Structure):
    _fields_ = [("master", C.c_void_p), ("shadow", C.c_void_p), ("ortho", C.c_void_p), ("numel", C.c_int64)]


class MasterAdamWSeg(C.Structure):
    _fields_ = [("master", C.c_void_p), ("shadow", C.c_void_p), ("grad", C.c_void_p), ("exp_avg", C.c_void_p),
                ("exp_avg_sq", C.c_void_p), ("numel", C.c_int64), ("step", C.c_int32), ("pad_", C.c_int32)]


# every symbol include/monarch_muon_b200.h declares: name -> (restype, argtypes)
_vp, _i, _i64, _f, _d = C.c_void_p, C.c_int, C.c_int64, C.c_float, C.c_double
SYMBOLS = {
    "mmb_version": (_i, []),
    "mmb_last_error": (C.c_char_p, []),
    "mmb_launch_count": (_i64, []),
    "mmb_set_sm_limit": (_i, [_i]),
    "mmb_set_gemm_schedule": (_i, [_i]),
    "mmb_set_gemm_dependent_launch": (_i, [_i]),
    "mmb_set_stream_ctas_per_sm": (_i, [_i]),
    "mmb_momentum_scratch_floats": (_i64, [C.POINTER(MomentumSeg), _i]),
    "mmb_momentum_step": (_i, [C.POINTER(MomentumSeg), _i, _i, _i, _i, _f, _f, _i, _vp, _vp, _i64, _vp]),
    "mmb_momentum_static_max_floats": (_i64, []),
    "mmb_momentum_step_static": (_i, [C.POINTER(MomentumSeg), _i, _i, _i, _i, _f, _f, _i, _vp, _vp]),
    "mmb_fp8_quantize": (_i, [_vp, _vp, _vp, _vp, _vp, _i64, _i, _i, _i, _i, _vp]),
    "mmb_fp8_dequantize": (_i, [_vp, _vp, _vp, _vp, _vp, _i64, _i, _i, _vp]),
    "mmb_ns_workspace_bytes": (_i64, [_i, _i, _i]),
    "mmb_newton_schulz": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp, _i64, _i, _vp, _vp]),
    "mmb_newton_schulz_update": (_i, [_vp, _vp, _i, _i, _i, _vp, _i, _f, _vp, _i64, _i, _vp, _vp]),
    "mmb_wait_probe": (_i, [_i64, _vp, _vp]),
    "mmb_gemm_occupancy": (_i, [_i, C.POINTER(C.c_int)]),
    "mmb_gemm_bf16": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _f, _f, _vp, _i, _i, _vp, _vp]),
    "mmb_muon_update": (_i, [C.POINTER(UpdateSeg), _i, _i, _f, _vp]),
    "mmb_adamw_step": (_i, [C.POINTER(AdamWSeg), _i, _i, _d, _d, _d, _d, _d, _vp]),
    "mmb_adamw_fp8_step": (_i, [C.POINTER(AdamWFp8Seg), _i, _i, _i, _i, _d, _d, _d, _d, _d, _i, _vp]),
    "mmb_muon_update_master": (_i, [C.POINTER(MasterUpdateSeg), _i, _f, _vp]),
    "mmb_adamw_master_step": (_i, [C.POINTER(MasterAdamWSeg), _i, _i, _d, _d, _d, _d, _d, _vp]),
    "mmb_grad_norm_scratch_floats": (_i64, []),
    "mmb_grad_norm_clip": (_i, [C.POINTER(GradSeg), _i, _f, _vp, _vp, _i64, _vp]),
    "mmb_set_device_grad_scale": (_i, [_vp]),
    "mmb_multimem_reduce_bf16": (_i, [_vp, _vp, _i64, _i, _vp]),
    "mmb_multimem_broadcast": (_i, [_vp, _vp, _i64, _i, _vp]),
    "mmb_peer_reduce_bf16": (_i, [C.POINTER(_vp), _i, _vp, _i64, _i, _vp]),
    "mmb_peer_broadcast": (_i, [_vp, C.POINTER(_vp), _i, _i64, _i, _vp]),
    "mmb_device_status_create": (_i, [C.POINTER(_vp)]),
    "mmb_device_status_destroy": (_i, [_vp]),
    "mmb_device_status_read": (_i, [_vp, C.POINTER(C.c_int32), _i, _vp]),
}

_lock = threading.Lock()
_lib = None


def load():
    """Load (building first if needed) the shared library; raises on failure."""
    global _lib
    with _lock:
        if _lib is None:
            path = os.environ.get("MMB_LIBRARY")          # a prebuilt library elsewhere (must export the same ABI)
            if not path:
                path = _build.LIB_PATH
                if not os.path.exists(path) or os.environ.get("MMB_REBUILD") == "1":
                    path = _build.build()
            lib = C.CDLL(path)
            for name, (res, args) in SYMBOLS.items():
                fn = getattr(lib, name)          # AttributeError if the symbol is missing
                fn.restype = res
                fn.argtypes = args
            _lib = lib
    return _lib


def check(rc: int, what: str = "") -> None:
    if rc != 0:
        msg = load().mmb_last_error().decode("utf-8", "replace")
        raise RuntimeError(f"libmonarch_muon_b200 {what} failed ({rc}): {msg}")


def require_cuda(*tensors) -> None:
    if not torch.cuda.is_available():
        raise RuntimeError("monarch_muon_b200 needs a CUDA device (B200, sm_100a); there is no CPU path")
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("monarch_muon_b200: tensor is not on a CUDA device; there is no CPU path")


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.bfloat16:
        return BF16
    if dt == torch.float32:
        return F32
    raise TypeError(f"monarch_muon_b200 supports bfloat16 and float32 tensors, got {dt}")


def ptr(t) -> int:
    return 0 if t is None else t.data_ptr()


_status_words: dict = {}


def status_word(device: torch.device) -> int:
    """Per-device status word that kernels write when a bounded wait expires."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _status_words:
        out = C.c_void_p()
        with torch.cuda.device(idx):
            check(load().mmb_device_status_create(C.byref(out)), "device_status_create")
        _status_words[idx] = out.value
    return _status_words[idx]


def read_status(device: torch.device, reset: bool = True) -> int:
    """Synchronise the current stream and return the device status word (0 = fine)."""
    host = C.c_int32(0)
    idx = device.index if device.index is not None else torch.cuda.current_device()
    with torch.cuda.device(idx):
        check(load().mmb_device_status_read(status_word(device), C.byref(host), int(reset), stream_ptr()),
              "device_status_read")
    return host.value


def launch_count() -> int:
    """Kernels launched by the library in this process so far."""
    return int(load().mmb_launch_count())


def set_stream_ctas_per_sm(n: int) -> None:
    """Cap the grids of the bandwidth-bound kernels at n CTAs per SM (0 = default)."""
    check(load().mmb_set_stream_ctas_per_sm(int(n)), "set_stream_ctas_per_sm")


def set_gemm_schedule(dynamic: bool) -> None:
    """Newton-Schulz GEMM tiles: drawn from a counter (True) or fixed round-robin (False, default)."""
    check(load().mmb_set_gemm_schedule(1 if dynamic else 0), "set_gemm_schedule")


def set_gemm_dependent_launch(on: bool) -> None:
    """Newton-Schulz GEMMs launched with programmatic stream serialisation (True, default) or plainly."""
    check(load().mmb_set_gemm_dependent_launch(1 if on else 0), "set_gemm_dependent_launch")


def set_sm_limit(n: int) -> None:
    """Size kernel grids for at most n SMs (0 = all)."""
    load().mmb_set_sm_limit(int(n))


class launch_options:
    """Context manager around the library's per-thread launch options: they are set on entry and always
    put back to their defaults on exit, also when the body raises.

        with _lib.launch_options(sm_limit=140, dynamic_schedule=True):
            ...launch kernels...
    """

    def __init__(self, *, sm_limit: int = 0, dynamic_schedule: bool = False, stream_ctas_per_sm: int = 0,
                 dependent_launch: bool = True):
        self.sm_limit, self.dynamic, self.ctas = int(sm_limit), bool(dynamic_schedule), int(stream_ctas_per_sm)
        self.dependent = bool(dependent_launch)

    def __enter__(self):
        if self.sm_limit:
            set_sm_limit(self.sm_limit)
        if self.dynamic:
            set_gemm_schedule(True)
        if self.ctas:
            set_stream_ctas_per_sm(self.ctas)
        if not self.dependent:
            set_gemm_dependent_launch(False)
        return self

    def __exit__(self, *exc):
        if self.sm_limit:
            set_sm_limit(0)
        if self.dynamic:
            set_gemm_schedule(False)
        if self.ctas:
            set_stream_ctas_per_sm(0)
        if not self.dependent:
            set_gemm_dependent_launch(True)
        return False
