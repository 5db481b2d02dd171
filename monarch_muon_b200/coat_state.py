"""Monarch-Muon with FP8 optimizer states (drop-in for CoatStateMonarchMuon).

Reference: pretrain/src/models/monarch/coat_state_muon.py:117-151.  The
reference dequantises every state tensor to fp32, runs the unchanged step and
quantises back.  Here the Muon momentum never leaves FP8 between steps: the
fused momentum kernel decodes, updates and re-encodes in one pass.  The
embedded AdamW's two moments (a small share of the state) follow the
reference's scheme: decode, step, encode, with the stand-alone codec kernels.
"""
from __future__ import annotations

import torch

from . import fp8_state
from .optimizer import MonarchMuonOptimizer


class CoatStateMonarchMuon(MonarchMuonOptimizer):
    """`qargs` is the reference's QuantizationConfig (or any object with the
    same optimizer fields: qgroup_size, first/second_order_expansion,
    first/second_order_bit, expand_min).  `codec="absmax"` selects the plain
    per-group absmax format instead of COAT's range expansion."""

    def __init__(self, *args, qargs=None, codec: str = "expand", **kwargs):
        expand_min = 16
        if qargs is not None:
            assert qargs.qgroup_size == fp8_state.GROUP_SIZE, "optimizer states use groups of 128"
            if codec == "expand":
                assert qargs.first_order_expansion in ("expand", "true") and \
                    qargs.second_order_expansion in ("expand", "true")
            if qargs.first_order_bit != "E4M3" or qargs.second_order_bit != "E4M3":
                raise NotImplementedError("only E4M3 optimizer states are implemented")
            expand_min = qargs.expand_min
        if codec not in ("expand", "absmax"):
            raise ValueError("codec must be 'expand' or 'absmax'")
        self.codec = codec
        kwargs.setdefault("state_format", "fp8_expand" if codec == "expand" else "fp8_absmax")
        kwargs.setdefault("expand_min", expand_min)
        super().__init__(*args, **kwargs)

    def _adamw_step(self, group, lr: float) -> None:
        live = [p for p in group["params"] if p.grad is not None]
        packed = []
        for p in live:
            st = self.state[p]
            for name in ("exp_avg", "exp_avg_sq"):
                if name in st and st[name].dtype == torch.float8_e4m3fn:
                    st[name] = fp8_state.dequantize(st, name, fp8_state.STATES[name], codec=self.codec).to(p.dtype)
            packed.append(st)
        super()._adamw_step(group, lr)
        for st in packed:
            for name in ("exp_avg", "exp_avg_sq"):
                value = st.pop(name)
                fp8_state.quantize_(st, name, value.float(), fp8_state.STATES[name], torch.float8_e4m3fn,
                                    self.expand_min, codec=self.codec, div_mode=self.fp8_div)

    def load_state_dict(self, state_dict):
        # keep FP8 payloads and fp32 side arrays of the AdamW moments out of torch's dtype cast
        saved = {}
        for pid, entry in state_dict["state"].items():
            for k, v in entry.items():
                if torch.is_tensor(v) and (k in ("exp_avg", "exp_avg_sq") or k.endswith(("_exp_avg", "_exp_avg_sq"))):
                    saved.setdefault(pid, {})[k] = v
        super().load_state_dict(state_dict)
        saved_ids = [i for g in state_dict["param_groups"] for i in g["params"]]
        params = [p for g in self.param_groups for p in g["params"]]
        by_id = dict(zip(saved_ids, params))
        for pid, entry in saved.items():
            p = by_id[pid]
            for k, v in entry.items():
                self.state[p][k] = v.to(p.device).clone()
