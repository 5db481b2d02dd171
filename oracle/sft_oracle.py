"""CPU restatement of the reference's fine-tuning optimizer (test infrastructure, never shipped).

Follows finetune/sft_optimizer.py of the reference: fp32 master weights, fp32
momentum, bf16 (or any dtype) model parameters refreshed from the master after
every step; per group either Muon (heavy ball, five Newton-Schulz steps in
bf16, sqrt(rows/cols) scaling) or AdamW.  The reference calls
torch.optim._functional.adamw for the latter; its single-tensor arithmetic
(torch/optim/adam.py of the pinned torch >= 2.8: decoupled decay, lerp_ for the
first moment, eps after sqrt(v)/sqrt(bc2)) is written out below.
"""
from __future__ import annotations

import torch

from . import muon_oracle


def orthogonalize(momentum: torch.Tensor) -> torch.Tensor:
    """finetune/sft_optimizer.py:5-14: the same quintic iteration as
    monarch_muon.py:36-50 on a bf16 copy of the momentum, over the last two
    dimensions."""
    return muon_oracle.newton_schulz(momentum.to(torch.bfloat16))


def adamw_master_(master, grad, exp_avg, exp_avg_sq, step: int, *, lr, betas, weight_decay, eps):
    """One torch.optim.AdamW update of an fp32 tensor (sft_optimizer.py:51-55)."""
    beta1, beta2 = betas
    master.mul_(1 - lr * weight_decay)
    exp_avg.lerp_(grad, 1 - beta1)
    exp_avg_sq.mul_(beta2).addcmul_(grad, grad, value=1 - beta2)
    bc1 = 1 - beta1 ** step
    bc2 = 1 - beta2 ** step
    step_size = lr / bc1
    denom = (exp_avg_sq.sqrt() / (bc2 ** 0.5)).add_(eps)
    master.addcdiv_(exp_avg, denom, value=-step_size)


class OracleSFT:
    """groups: list of dicts {"params": [tensors], "algorithm": "muon"|"adamw", "lr": ..} with the
    reference's defaults for what is missing (sft_optimizer.py:18-21)."""

    def __init__(self, groups, lr=3e-5, momentum=0.95, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1):
        self.groups = []
        for g in groups:
            d = dict(lr=lr, momentum=momentum, betas=betas, eps=eps, weight_decay=weight_decay, algorithm="adamw")
            d.update(g)
            self.groups.append(d)
        self.state: dict = {}

    @torch.no_grad()
    def step(self, grads):
        """grads: one list per group, parallel to its params (None = skipped)."""
        for group, gs in zip(self.groups, grads):
            for p, g in zip(group["params"], gs):
                if g is None:
                    continue
                st = self.state.setdefault(id(p), {})
                if not st:                                            # sft_optimizer.py:36-42
                    st["master"] = p.detach().float().clone()
                    st["momentum"] = torch.zeros_like(st["master"])
                    st["step"] = 0
                    if group["algorithm"] == "adamw":
                        st["variance"] = torch.zeros_like(st["master"])
                        st["adam_step"] = 0
                master, buf = st["master"], st["momentum"]
                grad = g.float()
                if group["algorithm"] == "muon":                      # :45-49
                    st["step"] += 1
                    buf.mul_(group["momentum"]).add_(grad)
                    update = orthogonalize(buf).float()
                    scale = (p.shape[-2] / p.shape[-1]) ** 0.5
                    master.add_(update, alpha=-group["lr"] * scale)
                else:                                                 # :50-55
                    st["adam_step"] += 1
                    adamw_master_(master, grad, buf, st["variance"], st["adam_step"], lr=group["lr"],
                                  betas=group["betas"], weight_decay=group["weight_decay"], eps=group["eps"])
                p.copy_(master)                                       # :56
