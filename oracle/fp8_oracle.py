"""CPU restatement of the FP8 optimizer-state codecs (test infrastructure).

Two codecs, both E4M3 ("fn": no infinities, max 448) in groups of 128
contiguous elements, groups restarting at each tensor, tail group masked:

absmax      one fp32 scale per group.
            dequantise  m = float(code) * scale
                        (pretrain/third_party/coat/optimizer/triton_kernels.py:34-36)
            quantise    scale' = (absmax + 1e-20) / 448 ; code' = RTNE(m / scale')
                        (triton_kernels.py:51-63)
expansion   COAT dynamic-range expansion, three fp32 side values per group
            (pretrain/src/models/monarch/coat_state_muon.py:22-43 dequantise,
            :46-91 quantise).  PARITY UNPINNED ON THE CPU: the reference kernel
            cannot be executed without a GPU (the Triton interpreter has no
            libdevice.pow), so no reference output pins this restatement.  It is
            not the arbiter of the CUDA expansion codec: that is the reference's
            own kernel, JIT-compiled and run on the GPU from the staged copy
            under oracle/_ref/ (tests/test_gpu_reference.py).

Divisions are IEEE round-to-nearest here.  The reference's Triton build
lowers `/` to the GPU's approximate full-range division, whose last-bit
behaviour is hardware defined and cannot be restated on a CPU; the CUDA
kernels offer both: their default issues the GPU instruction and is
bit-compared with the reference's kernels on the GPU, their IEEE mode is
bit-compared with this file.
"""
from __future__ import annotations

import numpy as np
import torch

GROUP = 128
E4M3_MAX = 448.0
ABSMAX_EPS = 1e-20        # triton_kernels.py:24
EXPAND_EPS = 1e-30        # coat_state_muon.py:25,49
E4M3 = torch.float8_e4m3fn


# ------------------------------------------------------------------ E4M3 cast
def e4m3_encode_numpy(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even, saturating fp32 -> E4M3 byte codes, written from
    the format definition (bias 7, 3 mantissa bits, subnormals at 2^-9 steps,
    0x7F/0xFF = NaN, max finite 448) and independent of torch's cast."""
    x = np.asarray(x, dtype=np.float32)
    sign = (np.signbit(x)).astype(np.uint8) << 7
    a = np.abs(x).astype(np.float64)
    out = np.zeros(x.shape, dtype=np.uint8)
    nan = np.isnan(a)
    a = np.minimum(np.where(nan, 0.0, a), 1e30)
    # exponent of the value, clamped to the subnormal exponent (-6)
    with np.errstate(divide="ignore"):
        e = np.floor(np.log2(np.where(a > 0, a, 1.0))).astype(np.int64)
    e = np.clip(e, -6, 8)
    step = np.ldexp(1.0, e - 3)                 # spacing of representable values
    q = np.rint(a / step)                        # numpy rint = ties to even
    val = q * step
    val = np.minimum(val, E4M3_MAX)              # saturate (satfinite)
    # re-derive fields from the rounded value
    with np.errstate(divide="ignore"):
        e2 = np.floor(np.log2(np.where(val > 0, val, 1.0))).astype(np.int64)
    normal = val >= 2.0 ** -6
    mant_n = np.rint(val / np.ldexp(1.0, e2 - 3)).astype(np.int64) - 8
    code_n = ((e2 + 7) << 3) | mant_n
    code_s = np.rint(val / 2.0 ** -9).astype(np.int64)
    out = np.where(normal, code_n, code_s).astype(np.uint8)
    out = np.where(nan, 0x7F, out).astype(np.uint8)
    return (out | sign).astype(np.uint8)


def e4m3_decode_numpy(codes: np.ndarray) -> np.ndarray:
    c = np.asarray(codes, dtype=np.uint8).astype(np.int64)
    s = np.where(c & 0x80, -1.0, 1.0)
    e = (c >> 3) & 0xF
    m = c & 0x7
    val = np.where(e == 0, m * 2.0 ** -9, (8 + m) * np.ldexp(1.0, e - 10))
    val = np.where((c & 0x7F) == 0x7F, np.nan, val)
    return (s * val).astype(np.float32)


def _cast_e4m3(q: torch.Tensor) -> torch.Tensor:
    """fp32 -> E4M3 codes (uint8 view).  torch's cast is RTNE; values in
    (448, 464) round to 448 as the saturating GPU cast does, and finite inputs
    here never exceed 448*(1+ulp)."""
    return q.to(E4M3).view(torch.uint8)


def _groups(numel: int) -> int:
    return -(-numel // GROUP)


def _padded(flat: torch.Tensor) -> torch.Tensor:
    pad = (-flat.numel()) % GROUP
    if pad:
        flat = torch.cat([flat, flat.new_zeros(pad)])
    return flat.view(-1, GROUP)


# --------------------------------------------------------------- absmax codec
def absmax_dequant(codes_u8: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    """triton_kernels.py:34-36: m = float(code) * scale, fp32, flat."""
    n = codes_u8.numel()
    vals = _padded(codes_u8.reshape(-1)).view(E4M3).to(torch.float32)
    return (vals * scales.to(torch.float32)[:, None]).reshape(-1)[:n]


def absmax_quant(m: torch.Tensor):
    """triton_kernels.py:51-63.  m: flat fp32.  Returns (codes uint8, scales fp32)."""
    n = m.numel()
    rows = _padded(m.reshape(-1).to(torch.float32))
    absmax = rows.abs().amax(dim=1)                         # masked tail reads 0
    scales = (absmax + ABSMAX_EPS) / E4M3_MAX
    codes = _cast_e4m3(rows / scales[:, None]).reshape(-1)[:n]
    return codes.contiguous(), scales


def absmax_momentum_step(codes_u8, scales, grad, beta: float, grad_scale: float = 1.0):
    """One heavy-ball step on absmax-coded momentum.

    dequantise (fp32) -> m = beta*m (one rounding) -> m = m + g (second
    rounding; the gradient is promoted to fp32 first, as torch's add_ of a
    bf16 tensor into an fp32 buffer does; monarch_muon.py:148) -> requantise.
    Returns (codes, scales, m_fp32, m_bf16); m_bf16 = RN_bf16(m) is what
    Newton-Schulz consumes (membench twin :161-163).
    """
    m = absmax_dequant(codes_u8, scales)
    m = m * torch.tensor(beta, dtype=torch.float32)
    g = grad.reshape(-1)
    if grad_scale != 1.0:
        # a scaled gradient is what grad.mul_(scale) leaves behind (clip_grad_norm_, DDP averaging):
        # computed in fp32, rounded to the gradient's own dtype
        g = (g.to(torch.float32) * torch.tensor(grad_scale, dtype=torch.float32)).to(grad.dtype)
    g = g.to(torch.float32)
    m = m + g
    new_codes, new_scales = absmax_quant(m)
    return new_codes, new_scales, m, m.to(torch.bfloat16)


# ------------------------------------------------------------ expansion codec
def expand_quant(value: torch.Tensor, signed: bool = True, expand_min: int = 16):
    """coat_state_muon.py:46-91, fp32 throughout.
    Returns (codes uint8, scale, expand, sqrt_minmax), the last three per group."""
    n = value.numel()
    rows = _padded(value.reshape(-1).to(torch.float32))
    idx = torch.arange(rows.numel()).view_as(rows)
    mask = idx < n
    f32 = torch.float32
    eps = torch.tensor(EXPAND_EPS, dtype=f32)
    abs_m = rows.abs()
    valid = mask & (abs_m > 0)
    absmax = torch.where(mask, abs_m, torch.zeros((), dtype=f32)).amax(dim=1)
    big = torch.tensor(3.4028235e38, dtype=f32)
    absmin = torch.where(valid, abs_m, big).amin(dim=1)
    nonzero = valid.sum(dim=1)
    absmax = torch.maximum(absmax, eps)
    absmin = torch.where(nonzero > 0, torch.maximum(absmin, eps), eps)
    one_eps = torch.tensor(1.0, dtype=f32) + eps            # == 1 in fp32
    ratio = torch.maximum(absmax / absmin, one_eps)
    ratio_upper = torch.tensor(E4M3_MAX * E4M3_MAX / 2.0, dtype=f32)
    log_ratio = torch.log2(ratio)
    safe_log = torch.where(log_ratio > eps, log_ratio, torch.ones((), dtype=f32))
    raw_expand = torch.floor((torch.log2(ratio_upper) / safe_log) * expand_min) / expand_min
    min_expand = torch.tensor(1.0 / expand_min, dtype=f32)
    expand = torch.where(ratio <= one_eps, torch.ones((), dtype=f32),
                         torch.maximum(raw_expand, min_expand))
    sqrt_mm = torch.maximum(torch.sqrt(absmax) * torch.sqrt(absmin), eps)
    base = torch.maximum(abs_m / sqrt_mm[:, None], eps)
    powed = torch.pow(base, expand[:, None])
    if signed:
        sgn = torch.where(rows >= 0, 1.0, -1.0).to(f32)
        normalized = torch.where(valid, sgn * powed, torch.zeros((), dtype=f32))
    else:
        normalized = torch.where(valid, powed, torch.zeros((), dtype=f32))
    scale_base = torch.maximum(absmax / sqrt_mm, eps)
    scale = torch.maximum(torch.pow(scale_base, expand) / E4M3_MAX, eps)
    codes = _cast_e4m3(normalized / scale[:, None]).reshape(-1)[:n]
    return codes.contiguous(), scale, expand, sqrt_mm


def expand_dequant(codes_u8, scale, expand, sqrt_mm, signed: bool = True):
    """coat_state_muon.py:22-43."""
    n = codes_u8.numel()
    f32 = torch.float32
    eps = torch.tensor(EXPAND_EPS, dtype=f32)
    raw = _padded(codes_u8.reshape(-1)).view(E4M3).to(f32)
    ex = torch.maximum(expand.to(f32), eps)[:, None]
    sq = torch.maximum(sqrt_mm.to(f32), eps)[:, None]
    scaled = raw * scale.to(f32)[:, None]
    if signed:
        absolute = scaled.abs()
        sgn = torch.where(scaled >= 0, 1.0, -1.0).to(f32)
        power = torch.pow(torch.maximum(absolute, eps), 1.0 / ex)
        out = torch.where(absolute > 0, sgn * power * sq, torch.zeros((), dtype=f32))
    else:
        scaled = torch.clamp_min(scaled, 0.0)
        power = torch.pow(torch.maximum(scaled, eps), 1.0 / ex)
        out = torch.where(scaled > 0, power * sq, torch.zeros((), dtype=f32))
    return out.reshape(-1)[:n]


def expand_momentum_step(codes_u8, scale, expand, sqrt_mm, grad, beta: float, expand_min: int = 16):
    """One heavy-ball step on range-expansion-coded momentum: what
    CoatStateMonarchMuon.step does to a momentum buffer (coat_state_muon.py:126-139
    around monarch_muon.py:148): dequantise to fp32, m = beta*m, m = m + g,
    quantise again.  Returns (codes, scale, expand, sqrt_minmax, m_fp32)."""
    m = expand_dequant(codes_u8, scale, expand, sqrt_mm, signed=True)
    m = m * torch.tensor(beta, dtype=torch.float32)
    m = m + grad.reshape(-1).to(torch.float32)
    c, s, e, q = expand_quant(m, signed=True, expand_min=expand_min)
    return c, s, e, q, m


def adamw_fp8_step(p, grad, m_state, v_state, step: int, *, lr, betas, weight_decay, eps, codec: str = "expand",
                   expand_min: int = 16):
    """One AdamW step with both moments held in FP8: what CoatStateMonarchMuon.step does to an AdamW
    parameter (coat_state_muon.py:126-139): dequantise exp_avg (signed) and exp_avg_sq (unsigned) to fp32,
    run the reference's AdamW (monarch_muon.py:186-201: decay first, eps after sqrt(v)/sqrt(bc2)) with
    those fp32 moments, quantise them again.  `p` is updated in place in its own dtype; `m_state` and
    `v_state` are tuples (codes, scale[, expand, sqrt_minmax]).  Returns (m_state', v_state', m_fp32, v_fp32)."""
    import math
    beta1, beta2 = betas
    if codec == "expand":
        m = expand_dequant(*m_state, signed=True).view(p.shape)
        v = expand_dequant(*v_state, signed=False).view(p.shape)
    else:
        m = absmax_dequant(*m_state).view(p.shape)
        v = absmax_dequant(*v_state).view(p.shape)
    g32 = grad.to(torch.float32)
    if weight_decay > 0:
        p.mul_(1.0 - lr * weight_decay)
    m.mul_(beta1).add_(g32, alpha=1.0 - beta1)
    v.mul_(beta2).addcmul_(g32, g32, value=1.0 - beta2)
    bc1 = 1.0 - beta1 ** step
    bc2 = 1.0 - beta2 ** step
    denom = (v.sqrt() / math.sqrt(bc2)).add_(eps)
    p.copy_(p.to(torch.float32).addcdiv_(m, denom, value=-(lr / bc1)))
    if codec == "expand":
        return (expand_quant(m, signed=True, expand_min=expand_min), expand_quant(v, signed=False, expand_min=expand_min),
                m, v)
    return absmax_quant(m), absmax_quant(v), m, v
