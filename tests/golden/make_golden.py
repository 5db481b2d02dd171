"""Regenerate tests/golden/*.npz by RUNNING THE REFERENCE'S OWN PYTHON on CPU.

Run in a container that has the reference checkout:

    python tests/golden/make_golden.py /path/to/reference

The reference modules are loaded by file path (both optimizer twins are called
models.monarch.monarch_muon upstream, so they get distinct module names here).
Nothing from the reference is copied: only its numerical outputs on seeded
inputs are stored.  Inputs are regenerated from the seeds by
tests/golden_inputs.py, which this script shares with the tests; a checksum of
every input is stored so that a drift of the CPU random generator is detected
instead of showing up as a parity failure.

Vectors written
---------------
ns.npz         _newton_schulz_batched (pretrain twin) on fp32 and bf16 stacks
opt_fp32.npz   3 steps of the pretrain twin's MonarchMuonOptimizer, fp32
opt_bf16.npz   3 steps of the membench twin (bf16 params/state, bf16 NS)
coat_absmax.npz  COAT's plain FP8 AdamW kernel (third_party/coat/optimizer/
               triton_kernels.py:6-63) under TRITON_INTERPRET=1, used as a
               quantiser (beta=0 -> m=g) and as dequantise-halve-requantise
               (g=0, beta=0.5).  The interpreter's fp8 cast drops the carry
               when rounding reaches the next power of two, so its codes are a
               pin only away from those carries; its scales are exact.
sft.npz        3 steps of finetune/sft_optimizer.py's SFTOptimizer (fp32 master
               weights, bf16 parameters; a Muon group and an AdamW group)
"""
from __future__ import annotations

import importlib.util
import os
import sys

os.environ.setdefault("TRITON_INTERPRET", "1")

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import golden_inputs as gi  # noqa: E402


def _load(name, path):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _np(t: torch.Tensor) -> np.ndarray:
    if t.dtype == torch.bfloat16:
        return t.contiguous().view(torch.int16).numpy().view(np.uint16)
    if t.dtype == torch.float8_e4m3fn:
        return t.contiguous().view(torch.uint8).numpy()
    return t.contiguous().numpy()


def make_ns(ref_pre, out):
    data = {}
    for tag, dtype, shapes in gi.NS_CASES:
        for i, shape in enumerate(shapes):
            x = gi.ns_input(tag, i, shape, dtype)
            y = ref_pre._newton_schulz_batched(x)
            data[f"{tag}_{i}_checksum"] = np.array(gi.checksum(x))
            data[f"{tag}_{i}_out"] = _np(y.contiguous())
    np.savez_compressed(out, **data)


def run_opt(ref_mod, case, out):
    dtype, muon_shapes, adamw_shapes, hyper = gi.OPT_CASES[case]
    muon, adamw = gi.opt_params(case)
    opt = ref_mod.MonarchMuonOptimizer(muon, adamw, lr=hyper["lr"], momentum=hyper["momentum"],
                                       adamw_betas=hyper["betas"],
                                       adamw_weight_decay=hyper["weight_decay"],
                                       adamw_eps=hyper["eps"])
    opt.param_groups[1]["lr"] = hyper["adamw_lr"]
    data = {"checksum_params": np.array(sum(gi.checksum(p.data) for p in muon + adamw))}
    for step in range(gi.OPT_STEPS):
        mg, ag = gi.opt_grads(case, step)
        for p, g in zip(muon, mg):
            p.grad = g
        for p, g in zip(adamw, ag):
            p.grad = g
        data[f"checksum_grads_{step}"] = np.array(sum(gi.checksum(g) for g in mg + ag if g is not None))
        opt.step()
        opt.zero_grad(set_to_none=True)
        for i, p in enumerate(muon):
            data[f"s{step}_muon_{i}"] = _np(p.data.clone())
    for i, p in enumerate(muon):
        st = opt.state[p]
        if "momentum_buffer" in st:
            data[f"final_mom_{i}"] = _np(st["momentum_buffer"])
    for i, p in enumerate(adamw):
        data[f"final_adamw_{i}"] = _np(p.data)
        st = opt.state[p]
        if "exp_avg" in st:
            data[f"final_exp_avg_{i}"] = _np(st["exp_avg"])
            data[f"final_exp_avg_sq_{i}"] = _np(st["exp_avg_sq"])
            data[f"final_step_{i}"] = np.array(st["step"])
    np.savez_compressed(out, **data)


def make_coat(ref_root, out):
    import triton
    tk = _load("ref_coat_kernels", os.path.join(
        ref_root, "pretrain/third_party/coat/optimizer/triton_kernels.py"))
    g = gi.coat_input()
    n = g.numel()
    groups = triton.cdiv(n, 128)
    p = torch.zeros(n)
    m8 = torch.zeros(n, dtype=torch.float8_e4m3fn)
    v8 = torch.zeros(n, dtype=torch.float8_e4m3fn)
    sm = torch.zeros(groups)
    sv = torch.zeros(groups)
    args = dict(GROUP_SIZE=128)
    # beta1 = beta2 = 0: m = g, v = g*g, stored by the kernel's quantiser
    tk.triton_fp8_adamw_kernel[(groups,)](p, g, m8, sm, v8, sv, 0.0, 0.0, 0.0, 1.0, 1e-8, 0.0,
                                          448.0, 448.0, n, **args)
    data = {"checksum": np.array(gi.checksum(g)), "q1_codes": _np(m8.clone()), "q1_scales": sm.clone().numpy()}
    # g = 0, beta = 0.5: dequantise, halve exactly, requantise
    z = torch.zeros(n)
    tk.triton_fp8_adamw_kernel[(groups,)](p, z, m8, sm, v8, sv, 0.5, 0.5, 0.0, 1.0, 1e-8, 0.0,
                                          448.0, 448.0, n, **args)
    data["q2_codes"] = _np(m8.clone())
    data["q2_scales"] = sm.clone().numpy()
    np.savez_compressed(out, **data)


def make_sft(ref_root, out):
    sft = _load("ref_sft_optimizer", os.path.join(ref_root, "finetune/sft_optimizer.py"))
    h = gi.SFT_HYPER
    muon, adamw = gi.sft_params()
    opt = sft.SFTOptimizer([{"params": muon, "algorithm": "muon", "lr": h["muon_lr"], "weight_decay": 0.0},
                            {"params": adamw, "algorithm": "adamw", "lr": h["adamw_lr"]}],
                           momentum=h["momentum"], betas=h["betas"], eps=h["eps"], weight_decay=h["weight_decay"])
    data = {"checksum_params": np.array(sum(gi.checksum(p.data) for p in muon + adamw))}
    for step in range(gi.SFT_STEPS):
        mg, ag = gi.sft_grads(step)
        for p, g in zip(muon + adamw, mg + ag):
            p.grad = g
        opt.step()
        for i, p in enumerate(muon + adamw):
            data[f"s{step}_p{i}"] = _np(p.data.clone())
    for i, p in enumerate(muon + adamw):
        st = opt.state[p]
        data[f"final_master_{i}"] = _np(st["master"])
        data[f"final_momentum_{i}"] = _np(st["momentum"])
        if "variance" in st:
            data[f"final_variance_{i}"] = _np(st["variance"])
    np.savez_compressed(out, **data)


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py /path/to/reference-checkout")
    ref_root = sys.argv[1]
    pre = _load("ref_pretrain_monarch_muon",
                os.path.join(ref_root, "pretrain/src/models/monarch/monarch_muon.py"))
    mem = _load("ref_membench_monarch_muon",
                os.path.join(ref_root, "membench/src/models/monarch/monarch_muon.py"))
    make_ns(pre, os.path.join(HERE, "ns.npz"))
    run_opt(pre, "fp32", os.path.join(HERE, "opt_fp32.npz"))
    run_opt(mem, "bf16", os.path.join(HERE, "opt_bf16.npz"))
    make_coat(ref_root, os.path.join(HERE, "coat_absmax.npz"))
    make_sft(ref_root, os.path.join(HERE, "sft.npz"))
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)))


if __name__ == "__main__":
    main()
