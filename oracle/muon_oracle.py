"""CPU restatement of the Monarch-Muon step (test infrastructure, never shipped).

Every function names the reference lines it follows.  Paths are relative to
the reference project root.  Two twins exist upstream:

* pretrain/src/models/monarch/monarch_muon.py   - state and Newton-Schulz in
  the parameter dtype (fp32 in the pretraining recipe);
* membench/src/models/monarch/monarch_muon.py   - same API, the merged
  momentum is cast to bf16 before Newton-Schulz (lines 161-166).

`ns_dtype=None` follows the first, `ns_dtype=torch.bfloat16` the second.
"""
from __future__ import annotations

import math
from collections import OrderedDict

import torch

NS_COEFFS = (3.4445, -4.7750, 2.0315)   # monarch_muon.py:47
NS_STEPS = 5                            # monarch_muon.py:45
NS_EPS = 1e-7                           # monarch_muon.py:39


def newton_schulz(stack: torch.Tensor) -> torch.Tensor:
    """Quintic Newton-Schulz on a (batch, rows, cols) stack.

    Follows monarch_muon.py:36-50: per-matrix Frobenius normalisation with
    eps added to the norm, transpose when rows > cols, five times
    X <- a X + b (X X^T) X + c (X X^T)^2 X, every intermediate rounded to the
    tensor dtype because each is its own torch op.
    """
    a, b, c = NS_COEFFS
    fro = stack.norm(p="fro", dim=(-2, -1), keepdim=True)
    x = stack / (fro + NS_EPS)
    tall = x.shape[-2] > x.shape[-1]
    if tall:
        x = x.transpose(-2, -1)
    for _ in range(NS_STEPS):
        gram = x @ x.transpose(-2, -1)
        # upstream writes `3.4445*B - 4.7750*BBt @ B + 2.0315*(BBt@BBt) @ B`,
        # i.e. the scalar multiplies the Gram matrices before the product.
        x = a * x + (b * gram) @ x + (c * (gram @ gram)) @ x
    if tall:
        x = x.transpose(-2, -1)
    return x


def heavy_ball_(buf: torch.Tensor, grad: torch.Tensor, beta: float) -> torch.Tensor:
    """buf <- beta*buf, then buf <- buf + grad (two roundings).  monarch_muon.py:147-148.
    The scalar enters the multiply in fp32 (torch's op-math type for bf16)."""
    buf.mul_(beta)
    buf.add_(grad)
    return buf


def muon_group_step(params, grads, bufs, *, lr: float, beta: float, ns_dtype=None,
                    foreach_cpu: bool = False):
    """One Muon step over 3-D Monarch factors.  monarch_muon.py:139-165
    (membench twin :139-170 when ns_dtype is bfloat16).

    params/grads/bufs are parallel lists; params and bufs are updated in place.
    Returns the per-shape orthogonalised stacks (for tests).

    foreach_cpu=True issues the momentum as torch._foreach_mul_/_foreach_add_
    like the membench twin (:150-151).  On a CPU those round the Python scalar
    to the tensor dtype first (beta 0.95 becomes bf16 0.94921875), whereas the
    same calls on a GPU - and the plain mul_/add_ used otherwise - multiply by
    fp32 0.95.  The flag exists only to reproduce the twin's CPU output bit for
    bit in the golden tests; GPU parity uses the fp32-scalar form.
    """
    if foreach_cpu:
        torch._foreach_mul_(bufs, beta)
        torch._foreach_add_(bufs, grads)
    else:
        for buf, grad in zip(bufs, grads):
            heavy_ball_(buf, grad, beta)
    by_shape: "OrderedDict[tuple, list]" = OrderedDict()
    for p, buf in zip(params, bufs):
        by_shape.setdefault((buf.dtype, buf.shape[1], buf.shape[2]), []).append((p, buf))
    out = {}
    for (_, rows, cols), items in by_shape.items():
        stack = torch.cat([buf for _, buf in items], dim=0)
        if ns_dtype is not None and stack.dtype != ns_dtype:
            stack = stack.to(ns_dtype)
        ortho = newton_schulz(stack)
        if ortho.dtype != items[0][1].dtype:
            ortho = ortho.to(items[0][1].dtype)
        scale = (rows / cols) ** 0.5
        at = 0
        for p, buf in items:
            nb = buf.shape[0]
            p.add_(ortho[at:at + nb], alpha=-lr * scale)
            at += nb
        out[(rows, cols)] = ortho
    return out


def adamw_tensor_step(p, grad, exp_avg, exp_avg_sq, step: int, *, lr, betas, weight_decay, eps):
    """Decoupled AdamW on one tensor.  monarch_muon.py:186-201.

    Order matters for parity: weight decay multiplies the parameter first,
    eps is added after sqrt(v) is divided by sqrt(bias_correction2).
    `step` is the already-incremented step count.
    """
    beta1, beta2 = betas
    if weight_decay > 0:
        p.mul_(1.0 - lr * weight_decay)
    exp_avg.mul_(beta1).add_(grad, alpha=1.0 - beta1)
    exp_avg_sq.mul_(beta2).addcmul_(grad, grad, value=1.0 - beta2)
    bc1 = 1.0 - beta1 ** step
    bc2 = 1.0 - beta2 ** step
    denom = (exp_avg_sq.sqrt() / math.sqrt(bc2)).add_(eps)
    p.addcdiv_(exp_avg, denom, value=-(lr / bc1))


def adamw_group_step_foreach_cpu(ps, grads, exp_avgs, exp_avg_sqs, step: int, *, lr, betas,
                                 weight_decay, eps):
    """The membench twin's AdamW (membench/.../monarch_muon.py:191-208) issued
    with the same torch._foreach_* calls, to reproduce its CPU output exactly
    (see muon_group_step about scalar rounding on CPU).  One step count serves
    the whole group."""
    beta1, beta2 = betas
    if weight_decay > 0:
        torch._foreach_mul_(ps, 1.0 - lr * weight_decay)
    torch._foreach_mul_(exp_avgs, beta1)
    torch._foreach_add_(exp_avgs, grads, alpha=1.0 - beta1)
    torch._foreach_mul_(exp_avg_sqs, beta2)
    torch._foreach_addcmul_(exp_avg_sqs, grads, grads, value=1.0 - beta2)
    bc1 = 1.0 - beta1 ** step
    bc2 = 1.0 - beta2 ** step
    denom = torch._foreach_sqrt(exp_avg_sqs)
    torch._foreach_div_(denom, math.sqrt(bc2))
    torch._foreach_add_(denom, eps)
    torch._foreach_addcdiv_(ps, exp_avgs, denom, value=-lr / bc1)


class OracleMonarchMuon:
    """Minimal stateful driver around the functions above.

    Mirrors the reference optimizer's observable behaviour
    (monarch_muon.py:78-127): two groups, one shared lr unless overridden per
    group, parameters without a gradient are skipped, state created lazily.
    It is deliberately not a torch.optim.Optimizer - it only has to produce
    numbers to compare with.
    """

    def __init__(self, muon_params, adamw_params, *, lr=5e-3, momentum=0.95,
                 adamw_betas=(0.9, 0.95), adamw_weight_decay=0.1, adamw_eps=1e-8,
                 ns_dtype=None, foreach_cpu: bool = False):
        self.foreach_cpu = foreach_cpu
        self.muon = list(muon_params)
        self.adamw = list(adamw_params)
        self.lr = {"muon": lr, "adamw": lr}
        self.momentum = momentum
        self.betas = adamw_betas
        self.wd = adamw_weight_decay
        self.eps = adamw_eps
        self.ns_dtype = ns_dtype
        self.state: dict = {}

    @torch.no_grad()
    def step(self, muon_grads, adamw_grads):
        """Gradients are passed explicitly (None = skip that parameter)."""
        live = [(p, g) for p, g in zip(self.muon, muon_grads) if g is not None]
        if live:
            ps = [p for p, _ in live]
            gs = [g for _, g in live]
            bufs = []
            for p in ps:
                st = self.state.setdefault(id(p), {})
                if "momentum_buffer" not in st:
                    st["momentum_buffer"] = torch.zeros_like(p)
                bufs.append(st["momentum_buffer"])
            muon_group_step(ps, gs, bufs, lr=self.lr["muon"], beta=self.momentum,
                            ns_dtype=self.ns_dtype, foreach_cpu=self.foreach_cpu)
        live = [(p, g) for p, g in zip(self.adamw, adamw_grads) if g is not None]
        for p, g in live:
            st = self.state.setdefault(id(p), {})
            if not st:
                st["step"] = 0
                st["exp_avg"] = torch.zeros_like(p)
                st["exp_avg_sq"] = torch.zeros_like(p)
            st["step"] += 1
        if self.foreach_cpu and live:
            sts = [self.state[id(p)] for p, _ in live]
            adamw_group_step_foreach_cpu(
                [p for p, _ in live], [g for _, g in live], [s["exp_avg"] for s in sts],
                [s["exp_avg_sq"] for s in sts], sts[0]["step"], lr=self.lr["adamw"],
                betas=self.betas, weight_decay=self.wd, eps=self.eps)
            return
        for p, g in live:
            st = self.state[id(p)]
            adamw_tensor_step(p, g, st["exp_avg"], st["exp_avg_sq"], st["step"],
                              lr=self.lr["adamw"], betas=self.betas,
                              weight_decay=self.wd, eps=self.eps)


# --------------------------------------------------------------------------
# Shape book-keeping shared by tests and the benchmark's CPU leg.
# --------------------------------------------------------------------------

def monarch_factor_shapes(in_features: int, out_features: int, nblocks: int):
    """Shapes of the two block-diagonal factors of one Monarch linear layer.
    pretrain/src/models/monarch/monarch_linear.py:73-83."""
    in_blk = -(-in_features // nblocks)
    out_blk = -(-out_features // nblocks)
    if in_blk * nblocks < out_blk * nblocks:
        return (nblocks, in_blk, in_blk), (nblocks, out_blk, in_blk)
    return (nblocks, out_blk, in_blk), (nblocks, out_blk, out_blk)


def llama_monarch_muon_shapes(d_model: int, n_layers: int, intermediate: int, nblocks: int):
    """Every Muon tensor of a LLaMA-style decoder whose q,k,v,o,gate,up,down
    linears are Monarch layers (lm_head excluded, monarch_linear.py:105)."""
    shapes = []
    for _ in range(n_layers):
        for _ in range(4):                                   # q, k, v, o
            shapes += list(monarch_factor_shapes(d_model, d_model, nblocks))
        for _ in range(2):                                   # gate, up
            shapes += list(monarch_factor_shapes(d_model, intermediate, nblocks))
        shapes += list(monarch_factor_shapes(intermediate, d_model, nblocks))  # down
    return shapes


def ns_flops(rows: int, cols: int) -> float:
    """Algorithmic FLOPs of five quintic iterations on one block:
    Gram 2m^2n + square 2m^3 + apply 2m^2n per iteration, m = min, n = max."""
    m, n = min(rows, cols), max(rows, cols)
    return NS_STEPS * (4.0 * m * m * n + 2.0 * m ** 3)
