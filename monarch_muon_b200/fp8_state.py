"""FP8 (E4M3, groups of 128) optimizer-state codecs and the fused momentum step.

Host-side mirror of the reference's codec entry points
(pretrain/src/models/monarch/coat_state_muon.py:94-114 `dequantize`,
`quantize_`) plus the fused heavy-ball step that replaces
dequantise -> momentum update -> quantise.  Two codecs:

  "absmax"  one fp32 scale per group: scale = (absmax + 1e-20)/448
            (pretrain/third_party/coat/optimizer/triton_kernels.py:34-36,51-63)
  "expand"  COAT dynamic-range expansion: scale, expand, sqrt_minmax per group
            (coat_state_muon.py:22-91)
"""
from __future__ import annotations

import ctypes as C
from typing import Sequence

import torch

from . import _lib

GROUP_SIZE = 128
FP8 = {"E4M3": torch.float8_e4m3fn}
# state name -> signed (coat_state_muon.py:19)
STATES = {"momentum_buffer": True, "exp_avg": True, "exp_avg_sq": False}
_FORMAT = {"absmax": _lib.STATE_FP8_ABSMAX, "expand": _lib.STATE_FP8_EXPAND}


def groups_of(numel: int) -> int:
    return -(-numel // GROUP_SIZE)


def quantize_(state: dict, name: str, value: torch.Tensor, signed: bool = True, dtype=torch.float8_e4m3fn,
              expand_min: int = 16, codec: str = "expand", div_mode: int = _lib.DIV_DEFAULT) -> None:
    """Store fp32 `value` as state[name] (E4M3 codes, value's shape) plus the
    per-group side arrays state['scale_'+name] (and 'expand_', 'sqrt_minmax_'
    for the expansion codec), allocating them on first use."""
    _lib.require_cuda(value)
    if dtype != torch.float8_e4m3fn:
        raise TypeError("only E4M3 optimizer states are supported")
    value = value.contiguous().to(torch.float32)
    n = value.numel()
    if state.get(name) is None or state[name].dtype != dtype or state[name].shape != value.shape:
        state[name] = torch.empty(value.shape, device=value.device, dtype=dtype)
        keys = ("scale",) if codec == "absmax" else ("scale", "expand", "sqrt_minmax")
        for key in keys:
            state[f"{key}_{name}"] = torch.empty(groups_of(n), device=value.device, dtype=torch.float32)
    lib = _lib.load()
    with torch.cuda.device(value.device):
        _lib.check(lib.mmb_fp8_quantize(value.data_ptr(), state[name].data_ptr(), state[f"scale_{name}"].data_ptr(),
                                        _lib.ptr(state.get(f"expand_{name}")),
                                        _lib.ptr(state.get(f"sqrt_minmax_{name}")), n, _FORMAT[codec], int(signed),
                                        div_mode, expand_min, _lib.stream_ptr()), "fp8_quantize")


def dequantize(state: dict, name: str, signed: bool = True, codec: str | None = None) -> torch.Tensor:
    """fp32 tensor decoded from state[name] and its side arrays."""
    data = state[name]
    _lib.require_cuda(data)
    if codec is None:
        codec = "expand" if f"expand_{name}" in state else "absmax"
    out = torch.empty(data.shape, device=data.device, dtype=torch.float32)
    lib = _lib.load()
    with torch.cuda.device(data.device):
        _lib.check(lib.mmb_fp8_dequantize(data.data_ptr(), state[f"scale_{name}"].data_ptr(),
                                          _lib.ptr(state.get(f"expand_{name}")),
                                          _lib.ptr(state.get(f"sqrt_minmax_{name}")), out.data_ptr(), data.numel(),
                                          _FORMAT[codec], int(signed), _lib.stream_ptr()), "fp8_dequantize")
    return out


class MomentumPlan:
    """A reusable segment table for mmb_momentum_step.

    Each entry describes one parameter tensor: its state storage, where its
    bf16 momentum goes, and its block geometry.  Gradient pointers are filled
    in per step (autograd may hand out fresh gradient tensors every step).
    """

    def __init__(self, device: torch.device):
        self.device = device
        self.entries: list[dict] = []
        self.total_blocks = 0

    def add(self, *, state: torch.Tensor, m_bf16: torch.Tensor | None, numel: int, block_elems: int,
            scale=None, expand=None, sqrt_minmax=None) -> int:
        first = self.total_blocks
        nblocks = numel // block_elems if block_elems > 0 and numel % block_elems == 0 else 1
        self.entries.append(dict(state=state, m_bf16=m_bf16, numel=numel, block_elems=block_elems, scale=scale,
                                 expand=expand, sqrt_minmax=sqrt_minmax, first_block=first))
        self.total_blocks += nblocks
        return first

    def table(self, grads: Sequence[torch.Tensor], which: Sequence[int] | None = None):
        idx = range(len(self.entries)) if which is None else which
        segs = (_lib.MomentumSeg * len(grads))()
        for k, (i, g) in enumerate(zip(idx, grads)):
            e = self.entries[i]
            s = segs[k]
            s.grad = g.data_ptr()
            s.state = e["state"].data_ptr()
            s.scale = _lib.ptr(e["scale"])
            s.expand = _lib.ptr(e["expand"])
            s.sqrt_minmax = _lib.ptr(e["sqrt_minmax"])
            s.m_bf16 = _lib.ptr(e["m_bf16"])
            s.numel = e["numel"]
            s.block_elems = e["block_elems"]
            s.first_block = e["first_block"]
        return segs


def momentum_step(segs, nseg: int, *, grad_dtype: torch.dtype, state_format: int, beta: float,
                  grad_scale: float = 1.0, div_mode: int = _lib.DIV_DEFAULT, expand_min: int = 16,
                  block_sumsq: torch.Tensor | None = None, scratch: torch.Tensor | None = None) -> None:
    """Launch the fused momentum kernel over a prepared segment table."""
    lib = _lib.load()
    _lib.check(lib.mmb_momentum_step(segs, nseg, _lib.dtype_code(grad_dtype), state_format, div_mode, beta,
                                     grad_scale, expand_min, _lib.ptr(block_sumsq), _lib.ptr(scratch),
                                     0 if scratch is None else scratch.numel(), _lib.stream_ptr()), "momentum_step")


def scratch_floats(segs, nseg: int) -> int:
    return int(_lib.load().mmb_momentum_scratch_floats(segs, nseg))


def fp8_momentum_flat(codes: torch.Tensor, scales: torch.Tensor, grad: torch.Tensor, beta: float, *,
                      m_bf16: torch.Tensor | None = None, block_elems: int | None = None,
                      block_sumsq: torch.Tensor | None = None, grad_scale: float = 1.0,
                      div_mode: int = _lib.DIV_DEFAULT, expand: torch.Tensor | None = None,
                      sqrt_minmax: torch.Tensor | None = None, expand_min: int = 16) -> None:
    """One FP8-state heavy-ball step on a flat buffer, in place:
    codes (uint8/E4M3 [n]), scales (fp32 [ceil(n/128)]), grad (bf16/fp32 [n]).
    With `expand` and `sqrt_minmax` (fp32, one per group) the state is in the
    range-expansion format, else in the absmax format."""
    _lib.require_cuda(codes, scales, grad)
    if (expand is None) != (sqrt_minmax is None):
        raise ValueError("expand and sqrt_minmax go together")
    n = codes.numel()
    seg = (_lib.MomentumSeg * 1)()
    seg[0].grad = grad.data_ptr()
    seg[0].state = codes.data_ptr()
    seg[0].scale = scales.data_ptr()
    seg[0].expand = _lib.ptr(expand)
    seg[0].sqrt_minmax = _lib.ptr(sqrt_minmax)
    seg[0].m_bf16 = _lib.ptr(m_bf16)
    seg[0].numel = n
    seg[0].block_elems = block_elems if block_elems else n
    seg[0].first_block = 0
    scratch = None
    if block_sumsq is not None:
        scratch = torch.empty(scratch_floats(seg, 1), dtype=torch.float32, device=codes.device)
    with torch.cuda.device(codes.device):
        momentum_step(seg, 1, grad_dtype=grad.dtype,
                      state_format=_lib.STATE_FP8_ABSMAX if expand is None else _lib.STATE_FP8_EXPAND, beta=beta,
                      grad_scale=grad_scale, div_mode=div_mode, expand_min=expand_min, block_sumsq=block_sumsq,
                      scratch=scratch)
