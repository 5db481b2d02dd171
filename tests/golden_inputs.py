"""Seeded inputs shared by tests/golden/make_golden.py and the parity tests.

Everything is drawn on the CPU generator so the same bits come out wherever
the same torch build runs; `checksum` guards against generator drift.
"""
from __future__ import annotations

import torch

# (tag, dtype, shapes): stacks fed to Newton-Schulz
NS_CASES = (
    ("f32", torch.float32, ((2, 64, 64), (2, 96, 64), (2, 64, 96), (1, 40, 24))),
    ("bf16", torch.bfloat16, ((2, 128, 128), (1, 344, 128), (1, 128, 344))),
)

OPT_STEPS = 3
# case -> (dtype, muon shapes, adamw shapes, hyper-parameters)
OPT_CASES = {
    "fp32": (torch.float32,
             ((2, 64, 64), (2, 96, 64), (2, 64, 96), (2, 64, 64)),
             ((128, 32), (32,)),
             dict(lr=0.02, adamw_lr=3e-4, momentum=0.95, betas=(0.9, 0.95), weight_decay=0.1, eps=1e-8)),
    "bf16": (torch.bfloat16,
             ((2, 128, 128), (1, 344, 128), (1, 128, 344), (1, 128, 128)),
             ((256, 64), (64,)),
             dict(lr=0.02, adamw_lr=3e-4, momentum=0.95, betas=(0.9, 0.95), weight_decay=0.1, eps=1e-8)),
}


def _gen(*key) -> torch.Generator:
    seed = 0x5EED
    for k in key:
        seed = (seed * 1000003 + (hash(k) if not isinstance(k, str) else sum(map(ord, k)))) % (2 ** 31 - 1)
    return torch.Generator().manual_seed(seed)


def checksum(t: torch.Tensor) -> int:
    """Order-sensitive integer digest of a tensor's bits."""
    if t.dtype == torch.bfloat16:
        v = t.contiguous().view(torch.int16).to(torch.int64) & 0xFFFF
    elif t.dtype == torch.float32:
        v = t.contiguous().view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    else:
        v = t.contiguous().view(torch.uint8).to(torch.int64)
    v = v.reshape(-1)
    w = (torch.arange(v.numel(), dtype=torch.int64) % 8191) + 1
    return int(((v * w) % 2147483647).sum().item() % 2147483647)


def ns_input(tag: str, index: int, shape, dtype) -> torch.Tensor:
    return torch.randn(shape, generator=_gen("ns", tag, index), dtype=torch.float32).to(dtype)


def opt_params(case: str):
    dtype, muon_shapes, adamw_shapes, _ = OPT_CASES[case]
    muon = [torch.nn.Parameter((0.02 * torch.randn(s, generator=_gen("p", case, "m", i))).to(dtype))
            for i, s in enumerate(muon_shapes)]
    adamw = [torch.nn.Parameter((0.02 * torch.randn(s, generator=_gen("p", case, "a", i))).to(dtype))
             for i, s in enumerate(adamw_shapes)]
    return muon, adamw


def opt_grads(case: str, step: int):
    """Gradients of one step.  The last Muon tensor has no gradient on step 0
    (the reference skips parameters whose grad is None and creates their state
    lazily), which exercises that path."""
    dtype, muon_shapes, adamw_shapes, _ = OPT_CASES[case]
    mg = [(1e-3 * torch.randn(s, generator=_gen("g", case, "m", i, step))).to(dtype)
          for i, s in enumerate(muon_shapes)]
    ag = [(1e-3 * torch.randn(s, generator=_gen("g", case, "a", i, step))).to(dtype)
          for i, s in enumerate(adamw_shapes)]
    if step == 0:
        mg[-1] = None
    return mg, ag


def coat_input() -> torch.Tensor:
    """Values spread over seven decades, length not a multiple of 128, with a
    zero run, like the reference's codec test (test_coat_state_muon.py:27-28)."""
    n = 128 * 40 + 5
    g = torch.randn(n, generator=_gen("coat")) * torch.logspace(-6, 1, n)
    g[128 * 3:128 * 4] = 0.0          # an all-zero group
    g[128 * 5 + 7] = 0.0
    return g


# fine-tuning optimizer (fp32 master weights, bf16 parameters): a Monarch factor, two dense matrices
# (one taller than wide) under Muon; an embedding-like matrix and a norm vector under AdamW
SFT_STEPS = 3
SFT_MUON_SHAPES = ((2, 128, 128), (96, 64), (64, 160))
SFT_ADAMW_SHAPES = ((256, 64), (64,))
SFT_HYPER = dict(muon_lr=1e-3, adamw_lr=3e-5, momentum=0.95, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)


def sft_params():
    muon = [torch.nn.Parameter((0.02 * torch.randn(s, generator=_gen("sft", "m", i))).bfloat16())
            for i, s in enumerate(SFT_MUON_SHAPES)]
    adamw = [torch.nn.Parameter((0.02 * torch.randn(s, generator=_gen("sft", "a", i))).bfloat16())
             for i, s in enumerate(SFT_ADAMW_SHAPES)]
    return muon, adamw


def sft_grads(step: int):
    mg = [(1e-2 * torch.randn(s, generator=_gen("sftg", "m", i, step))).bfloat16() for i, s in enumerate(SFT_MUON_SHAPES)]
    ag = [(1e-2 * torch.randn(s, generator=_gen("sftg", "a", i, step))).bfloat16() for i, s in enumerate(SFT_ADAMW_SHAPES)]
    if step == 0:
        mg[-1] = None          # skipped on the first step: state is created lazily on the second
    return mg, ag
