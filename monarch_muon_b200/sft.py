"""Fine-tuning optimizer with fp32 master weights (drop-in for the reference's SFTOptimizer).

Reference: finetune/sft_optimizer.py:17-71.  Every parameter keeps an fp32
`master` copy and an fp32 `momentum`; a step updates the master and refreshes
the (bf16) parameter from it.  Param groups choose `algorithm`: "muon"
(heavy ball, five Newton-Schulz steps in bf16 over the last two dimensions,
sqrt(rows/cols) scaling; any parameter with ndim >= 2, 3-D Monarch factors
block by block) or "adamw" (torch.optim.AdamW arithmetic on the master).

Same kernels as MonarchMuonOptimizer underneath: the fused momentum kernel
(fp32 state, gradient read in its own dtype, bf16 copy + block norms out), the
tcgen05 Newton-Schulz, and one-pass master updates that also write the bf16
parameter (`mmb_muon_update_master`, `mmb_adamw_master_step`).
"""
from __future__ import annotations

from collections import OrderedDict

import torch

from . import _lib, fp8_state
from .newton_schulz import newton_schulz_batched

NS_SLICE_BLOCKS = 256          # Newton-Schulz workspace is sized for at most this many blocks at once


class SFTOptimizer(torch.optim.Optimizer):
    """SFTOptimizer(params, lr=3e-5, momentum=0.95, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)

    `params` is an iterable of tensors or of group dicts with an "algorithm"
    key ("adamw" when absent), as in the reference.  State per parameter:
    master, momentum (the AdamW first moment in AdamW groups), step, and for
    AdamW variance and adam_step - the reference's names."""

    def __init__(self, params, lr=3e-5, momentum=0.95, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1):
        super().__init__(params, dict(lr=lr, momentum=momentum, betas=betas, eps=eps, weight_decay=weight_decay,
                                      algorithm="adamw"))
        self._arenas: dict = {}
        self._adam_steps: dict = {}      # host copies of state["adam_step"], so that a step needs no device read

    # ------------------------------------------------------------------ state
    def _state_for(self, p, group):
        state = self.state[p]
        if not state:                                             # sft_optimizer.py:36-42
            state["master"] = p.detach().float().clone(memory_format=torch.contiguous_format)
            state["momentum"] = torch.zeros_like(state["master"])
            state["step"] = 0
            if group["algorithm"] == "adamw":
                state["variance"] = torch.zeros_like(state["master"])
                state["adam_step"] = torch.tensor(0.0, device=p.device)
                self._adam_steps[p] = 0
        return state

    @staticmethod
    def _shadow_ptr(p):
        """The bf16 parameter is written by the kernel; other dtypes are refreshed with copy_."""
        return p.data.data_ptr() if (p.dtype == torch.bfloat16 and p.data.is_contiguous()) else None

    # ------------------------------------------------------------------- step
    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            live = [p for p in group["params"] if p.grad is not None]
            if not live:
                continue
            _lib.require_cuda(*live)
            with torch.cuda.device(live[0].device):
                if group["algorithm"] == "muon":
                    self._muon(group, live)
                else:
                    self._adamw(group, live)
        return loss

    def _arena(self, key, blocks: int, rows: int, cols: int, device):
        a = self._arenas.get(key)
        if a is None or a[0].shape[0] < blocks:
            a = (torch.empty((blocks, rows, cols), dtype=torch.bfloat16, device=device),
                 torch.empty(blocks, dtype=torch.float32, device=device))
            self._arenas[key] = a
        return a

    def _muon(self, group, live) -> None:
        lib = _lib.load()
        by_shape: "OrderedDict[tuple, list]" = OrderedDict()
        for p in live:
            if p.dim() < 2:
                raise ValueError("Muon parameters need at least two dimensions")
            by_shape.setdefault((p.device, p.grad.dtype, p.shape[-2], p.shape[-1]), []).append(p)
        for (dev, gdtype, rows, cols), ps in by_shape.items():
            block = rows * cols
            counts = [p.numel() // block for p in ps]
            total = sum(counts)
            stack, sumsq = self._arena((dev, rows, cols), total, rows, cols, dev)
            norms_fused = block % fp8_state.GROUP_SIZE == 0       # block sums come out of the momentum kernel
            segs = (_lib.MomentumSeg * len(ps))()
            upd = (_lib.MasterUpdateSeg * len(ps))()
            at = 0
            keep = []        # contiguous copies of strided gradients must outlive the launch that reads them
            for k, (p, nb) in enumerate(zip(ps, counts)):
                st = self._state_for(p, group)
                st["step"] += 1
                g = p.grad
                if not g.is_contiguous():
                    g = g.contiguous()
                    keep.append(g)
                segs[k].grad = g.data_ptr()
                segs[k].state = st["momentum"].data_ptr()
                segs[k].m_bf16 = stack[at:].data_ptr()
                segs[k].numel = p.numel()
                segs[k].block_elems = block if norms_fused else p.numel()
                segs[k].first_block = at
                upd[k].master = st["master"].data_ptr()
                upd[k].shadow = self._shadow_ptr(p)
                upd[k].ortho = stack[at:].data_ptr()
                upd[k].numel = p.numel()
                at += nb
            scratch = None
            if norms_fused:
                scratch = torch.empty(fp8_state.scratch_floats(segs, len(ps)), dtype=torch.float32, device=dev)
            # momentum <- beta*momentum + grad (fp32, two roundings); bf16 copy into the stack
            fp8_state.momentum_step(segs, len(ps), grad_dtype=gdtype, state_format=_lib.STATE_F32,
                                    beta=group["momentum"], block_sumsq=sumsq if norms_fused else None,
                                    scratch=scratch)
            backend = _lib.NS_TCGEN05 if (rows % 8 == 0 and cols % 8 == 0) else _lib.NS_SIMT
            newton_schulz_batched(stack[:total], out=stack[:total], block_sumsq=sumsq[:total] if norms_fused else None,
                                  backend=backend, max_batch=NS_SLICE_BLOCKS)
            alpha = -group["lr"] * (rows / cols) ** 0.5
            _lib.check(lib.mmb_muon_update_master(upd, len(ps), alpha, _lib.stream_ptr()), "muon_update_master")
            for p in ps:
                if self._shadow_ptr(p) is None:
                    p.copy_(self.state[p]["master"])

    def _adamw(self, group, live) -> None:
        lib = _lib.load()
        beta1, beta2 = group["betas"]
        by_dtype: "OrderedDict[tuple, list]" = OrderedDict()
        for p in live:
            by_dtype.setdefault((p.device, p.grad.dtype), []).append(p)
        for (dev, gdtype), ps in by_dtype.items():
            segs = (_lib.MasterAdamWSeg * len(ps))()
            keep = []
            for k, p in enumerate(ps):
                st = self._state_for(p, group)
                if p not in self._adam_steps:                     # state came from load_state_dict
                    self._adam_steps[p] = int(st["adam_step"].item())
                self._adam_steps[p] += 1
                st["adam_step"] += 1
                g = p.grad if p.grad.is_contiguous() else p.grad.contiguous()
                keep.append(g)
                segs[k].master = st["master"].data_ptr()
                segs[k].shadow = self._shadow_ptr(p)
                segs[k].grad = g.data_ptr()
                segs[k].exp_avg = st["momentum"].data_ptr()
                segs[k].exp_avg_sq = st["variance"].data_ptr()
                segs[k].numel = p.numel()
                segs[k].step = self._adam_steps[p]
            _lib.check(lib.mmb_adamw_master_step(segs, len(ps), _lib.dtype_code(gdtype), group["lr"], beta1, beta2,
                                                 group["weight_decay"], group["eps"], _lib.stream_ptr()),
                       "adamw_master_step")
            for p in ps:
                if self._shadow_ptr(p) is None:
                    p.copy_(self.state[p]["master"])

    def load_state_dict(self, state_dict):
        """torch casts floating state to the parameter dtype on load; masters and moments stay fp32."""
        saved = {pid: {k: v for k, v in entry.items() if torch.is_tensor(v) and v.is_floating_point()}
                 for pid, entry in state_dict["state"].items()}
        super().load_state_dict(state_dict)
        ids = [i for g in state_dict["param_groups"] for i in g["params"]]
        params = [p for g in self.param_groups for p in g["params"]]
        for pid, p in zip(ids, params):
            for k, v in saved.get(pid, {}).items():
                self.state[p][k] = v.to(device=p.device, dtype=torch.float32).clone()
        self._adam_steps.clear()


_NOT_MUON = ("embed_tokens", "lm_head")     # token embedding and output head stay with AdamW


def parameter_groups(model, optimizer: str, lr: float, config: dict):
    """Param groups for SFTOptimizer, with the reference's rule for who gets which algorithm
    (finetune/sft_optimizer.py:62-71).

    A parameter is stepped by Muon when it is a matrix or a stack of matrices (two or more dimensions) and
    is neither the token embedding nor the output head; all others are stepped by AdamW at the learning
    rate `config["muon_adamw_lr"]`.  Muon groups carry no weight decay.  Asking for "adamw" puts every
    parameter, in the same order (Muon candidates first), into a single AdamW group at `lr`."""
    named = list(model.named_parameters())
    is_muon = {id(p): p.ndim >= 2 and not any(tag in name for tag in _NOT_MUON) for name, p in named}
    muon_side = [p for _, p in named if is_muon[id(p)]]
    adamw_side = [p for _, p in named if not is_muon[id(p)]]
    if optimizer == "adamw":
        return [dict(params=muon_side + adamw_side, algorithm="adamw", lr=lr)]
    return [dict(params=muon_side, algorithm="muon", lr=lr, weight_decay=0.0),
            dict(params=adamw_side, algorithm="adamw", lr=config["muon_adamw_lr"])]
