"""Batched Newton-Schulz and the GEMM family it is built from (CUDA only).

`newton_schulz_batched` mirrors the reference function of the same role,
_newton_schulz_batched (pretrain/src/models/monarch/monarch_muon.py:36-50; the
bf16 path of membench/src/models/monarch/monarch_muon.py:161-166): input a
(batch, rows, cols) stack, output the same shape, Frobenius normalisation with
eps on the norm, five quintic iterations, tall blocks handled without a
transpose in memory.  Arithmetic is bf16 operands with fp32 accumulation on
the tcgen05 tensor cores.
"""
from __future__ import annotations

import torch

from . import _lib

_workspaces: dict = {}


def _buffer(tag: str, nbytes: int, device: torch.device) -> torch.Tensor:
    """Grow-only scratch, one buffer per (device, stream, tag), 1 KiB aligned (the caching allocator's
    512-byte granularity plus an explicit offset).  Work that shares a buffer is ordered by its stream;
    another stream gets a buffer of its own."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    key = (index, torch.cuda.current_stream(device).cuda_stream, tag)
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes + 1024:
        _workspaces.pop(key, None)
        buf = torch.empty(nbytes + 1024, dtype=torch.uint8, device=device)
        _workspaces[key] = buf
    off = (-buf.data_ptr()) % 1024
    return buf[off:off + nbytes]


def _workspace(nbytes: int, device: torch.device) -> torch.Tensor:
    """Newton-Schulz workspace (A, P and two X buffers)."""
    return _buffer("ns", nbytes, device)


def scratch_bf16(tag: str, numel: int, device: torch.device) -> torch.Tensor:
    """A bf16 scratch array of `numel` elements from the same pool (the Newton-Schulz input of one slice
    when the optimizer state is not itself a bf16 array)."""
    return _buffer(tag, 2 * numel, device).view(torch.bfloat16)


def release_workspaces() -> None:
    _workspaces.clear()


def newton_schulz_batched(stack: torch.Tensor, *, out: torch.Tensor | None = None,
                          block_sumsq: torch.Tensor | None = None, backend: int = _lib.NS_TCGEN05,
                          max_batch: int | None = None) -> torch.Tensor:
    """Orthogonalise every (rows, cols) block of a bf16 CUDA stack.

    out          optional destination (may be `stack` itself)
    block_sumsq  optional fp32 [batch] sums of squares (otherwise computed)
    max_batch    process the stack in slices of at most this many blocks to
                 bound the workspace (default: whole stack)
    """
    _lib.require_cuda(stack)
    if stack.dim() != 3:
        raise ValueError("newton_schulz_batched expects (batch, rows, cols)")
    if stack.dtype != torch.bfloat16:
        raise TypeError("newton_schulz_batched computes in bfloat16; cast the stack first")
    if not stack.is_contiguous():
        raise ValueError("newton_schulz_batched expects a contiguous stack")
    if out is None:
        out = torch.empty_like(stack)
    elif out.shape != stack.shape or out.dtype != stack.dtype or not out.is_contiguous():
        raise ValueError("out must match the stack")
    batch, rows, cols = stack.shape
    if batch == 0:
        return out
    lib = _lib.load()
    step = batch if not max_batch else min(batch, max_batch)
    status = _lib.status_word(stack.device)
    with torch.cuda.device(stack.device):
        ws = _workspace(lib.mmb_ns_workspace_bytes(step, rows, cols), stack.device)
        for b0 in range(0, batch, step):
            nb = min(step, batch - b0)
            ss = None if block_sumsq is None else block_sumsq[b0:b0 + nb]
            _lib.check(lib.mmb_newton_schulz(stack[b0:b0 + nb].data_ptr(), out[b0:b0 + nb].data_ptr(), _lib.ptr(ss),
                                             nb, rows, cols, ws.data_ptr(), ws.numel(), backend, status,
                                             _lib.stream_ptr()), "newton_schulz")
    return out


def gemm_bf16(a: torch.Tensor, b: torch.Tensor, *, a_mode: int = _lib.GEMM_K, b_mode: int = _lib.GEMM_K,
              sym_out: bool = False, alpha: float = 1.0, diag: float = 0.0, inv_norm: torch.Tensor | None = None,
              sigma_pow: int = 0, backend: int = _lib.NS_TCGEN05, out: torch.Tensor | None = None) -> torch.Tensor:
    """D[b] = sigma_b * alpha * opA[b] @ opB[b]^T + diag * I on bf16 stacks.

    a is (batch, M, K) in GEMM_K mode, (batch, K, M) in GEMM_MN mode, and a
    symmetric (batch, M, M) matrix in GEMM_SYM mode, of which only the 256x256
    blocks on or above the block diagonal are read; b likewise with N.
    With sym_out only those blocks of D are written (the rest of `out` is left
    untouched).
    """
    _lib.require_cuda(a, b)
    batch = a.shape[0]
    M, K = (a.shape[2], a.shape[1]) if a_mode == _lib.GEMM_MN else (a.shape[1], a.shape[2])
    N, Kb = (b.shape[2], b.shape[1]) if b_mode == _lib.GEMM_MN else (b.shape[1], b.shape[2])
    if K != Kb or b.shape[0] != batch:
        raise ValueError("operand shapes do not agree")
    for t in (a, b):
        if t.dtype != torch.bfloat16 or not t.is_contiguous():
            raise TypeError("gemm_bf16 expects contiguous bfloat16 tensors")
    d = out if out is not None else torch.empty(batch, M, N, dtype=torch.bfloat16, device=a.device)
    lib = _lib.load()
    with torch.cuda.device(a.device):
        _lib.check(lib.mmb_gemm_bf16(a.data_ptr(), b.data_ptr(), d.data_ptr(), batch, M, N, K, a_mode, b_mode,
                                     int(sym_out), alpha, diag, _lib.ptr(inv_norm), sigma_pow, backend,
                                     _lib.status_word(a.device), _lib.stream_ptr()), "gemm_bf16")
    return d


def newton_schulz_update(stack: torch.Tensor, weight_ptrs: torch.Tensor, weight_dtype: torch.dtype, alpha: float, *,
                         block_sumsq: torch.Tensor | None = None, backend: int = _lib.NS_TCGEN05) -> None:
    """W[b] <- W[b] + alpha * NS(stack)[b] in one call (mmb_newton_schulz_update): the counterpart of
    _newton_schulz_batched followed by `param.data.add_(ortho, alpha=)` (monarch_muon.py:36-50, 160-165).
    `weight_ptrs` is an int64 CUDA tensor with one device address per block: that block's rows x cols
    weights, row-major, 16-byte aligned.  `stack` is only read."""
    _lib.require_cuda(stack, weight_ptrs)
    if stack.dim() != 3 or stack.dtype != torch.bfloat16 or not stack.is_contiguous():
        raise ValueError("newton_schulz_update expects a contiguous bfloat16 (batch, rows, cols) stack")
    batch, rows, cols = stack.shape
    if weight_ptrs.dtype != torch.int64 or weight_ptrs.numel() != batch or not weight_ptrs.is_contiguous():
        raise ValueError("weight_ptrs must be a contiguous int64 tensor with one address per block")
    if batch == 0:
        return
    lib = _lib.load()
    with torch.cuda.device(stack.device):
        ws = _workspace(lib.mmb_ns_workspace_bytes(batch, rows, cols), stack.device)
        _lib.check(lib.mmb_newton_schulz_update(stack.data_ptr(), _lib.ptr(block_sumsq), batch, rows, cols,
                                                weight_ptrs.data_ptr(), _lib.dtype_code(weight_dtype), float(alpha),
                                                ws.data_ptr(), ws.numel(), backend, _lib.status_word(stack.device),
                                                _lib.stream_ptr()), "newton_schulz_update")
