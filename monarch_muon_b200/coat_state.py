"""Monarch-Muon with FP8 optimizer states (drop-in for CoatStateMonarchMuon).

Reference: pretrain/src/models/monarch/coat_state_muon.py:117-151.  The
reference dequantises every state tensor to fp32, runs the unchanged step and
quantises back.  Here no state leaves FP8 between steps: the fused momentum
kernel and the fused FP8 AdamW kernel decode, update and re-encode a group of
128 elements in registers, one pass each.
"""
from __future__ import annotations

import torch

from . import _lib, fp8_state
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

    def _adamw_new_state(self, p, state) -> None:
        """Both moments start as all-zero codes (they decode to 0 whatever the side arrays hold)."""
        n = p.numel()
        groups = fp8_state.groups_of(n)
        state["step"] = 0
        keys = ("scale",) if self.codec == "absmax" else ("scale", "expand", "sqrt_minmax")
        for name in ("exp_avg", "exp_avg_sq"):
            state[name] = torch.zeros(p.shape, dtype=torch.uint8, device=p.device).view(torch.float8_e4m3fn)
            for key in keys:
                state[f"{key}_{name}"] = torch.ones(groups, dtype=torch.float32, device=p.device)

    def _adamw_step(self, group, lr: float) -> None:
        """One fused pass per parameter dtype: decode both moments, AdamW in fp32, encode them again."""
        beta1, beta2 = group["betas"]
        by_dtype = self._adamw_collect(group)
        if not by_dtype:
            return
        lib = _lib.load()
        fmt = _lib.STATE_FP8_EXPAND if self.codec == "expand" else _lib.STATE_FP8_ABSMAX
        self._mark("begin")
        for dtype, items in by_dtype.items():
            segs = (_lib.AdamWFp8Seg * len(items))()
            for k, (p, g, st) in enumerate(items):
                if st["exp_avg"].dtype != torch.float8_e4m3fn:      # state restored from a non-FP8 checkpoint
                    for name in ("exp_avg", "exp_avg_sq"):
                        value = st.pop(name)
                        fp8_state.quantize_(st, name, value.float(), fp8_state.STATES[name], torch.float8_e4m3fn,
                                            self.expand_min, codec=self.codec, div_mode=self.fp8_div)
                s = segs[k]
                s.param, s.grad = p.data.data_ptr(), g.data_ptr()
                s.exp_avg, s.exp_avg_sq = st["exp_avg"].data_ptr(), st["exp_avg_sq"].data_ptr()
                s.scale_exp_avg, s.scale_exp_avg_sq = st["scale_exp_avg"].data_ptr(), st["scale_exp_avg_sq"].data_ptr()
                s.expand_exp_avg = _lib.ptr(st.get("expand_exp_avg"))
                s.sqrt_minmax_exp_avg = _lib.ptr(st.get("sqrt_minmax_exp_avg"))
                s.expand_exp_avg_sq = _lib.ptr(st.get("expand_exp_avg_sq"))
                s.sqrt_minmax_exp_avg_sq = _lib.ptr(st.get("sqrt_minmax_exp_avg_sq"))
                s.numel = p.numel()
                s.step = st["step"]
            with torch.cuda.device(items[0][0].device):
                _lib.check(lib.mmb_adamw_fp8_step(segs, len(items), _lib.dtype_code(dtype), fmt, self.fp8_div, lr,
                                                  beta1, beta2, group["weight_decay"], group["eps"],
                                                  self.expand_min, _lib.stream_ptr()), "adamw_fp8_step")
        self._mark("adamw")

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
