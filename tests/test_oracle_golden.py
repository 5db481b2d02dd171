"""The CPU oracle against vectors produced by the reference's own Python.

tests/golden/*.npz were written by tests/golden/make_golden.py, which imports
and runs the reference on CPU.  These tests pin oracle/ to those outputs:
bit-exact for everything torch computes deterministically (Newton-Schulz,
momentum, update, AdamW - same ops in the same order), and for the FP8 absmax
codec bit-exact scales plus codes equal wherever the Triton interpreter's
emulated fp8 cast is itself correct.
"""
import os

import numpy as np
import pytest
import torch

import golden_inputs as gi
from oracle import fp8_oracle, muon_oracle

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _t(arr: np.ndarray, dtype) -> torch.Tensor:
    if dtype == torch.bfloat16:
        return torch.from_numpy(arr.view(np.int16).copy()).view(torch.bfloat16)
    return torch.from_numpy(arr.copy())


@pytest.mark.parametrize("tag,dtype,shapes", gi.NS_CASES, ids=[c[0] for c in gi.NS_CASES])
def test_newton_schulz_bit_exact(tag, dtype, shapes):
    gold = np.load(os.path.join(GOLD, "ns.npz"))
    for i, shape in enumerate(shapes):
        x = gi.ns_input(tag, i, shape, dtype)
        assert gi.checksum(x) == int(gold[f"{tag}_{i}_checksum"]), "CPU generator drifted"
        want = _t(gold[f"{tag}_{i}_out"], dtype)
        got = muon_oracle.newton_schulz(x)
        assert got.shape == want.shape
        assert torch.equal(got.contiguous(), want), (tag, shape)


@pytest.mark.parametrize("case", ["fp32", "bf16"])
def test_optimizer_three_steps_bit_exact(case):
    gold = np.load(os.path.join(GOLD, f"opt_{case}.npz"))
    dtype, _, _, hyper = gi.OPT_CASES[case]
    muon, adamw = gi.opt_params(case)
    muon = [p.data for p in muon]
    adamw = [p.data for p in adamw]
    opt = muon_oracle.OracleMonarchMuon(
        muon, adamw, lr=hyper["lr"], momentum=hyper["momentum"], adamw_betas=hyper["betas"],
        adamw_weight_decay=hyper["weight_decay"], adamw_eps=hyper["eps"],
        ns_dtype=torch.bfloat16 if case == "bf16" else None,
        # the bf16 vectors come from the membench twin run on CPU, whose
        # torch._foreach_* calls round Python scalars to bf16 there
        foreach_cpu=(case == "bf16"))
    opt.lr["adamw"] = hyper["adamw_lr"]
    for step in range(gi.OPT_STEPS):
        mg, ag = gi.opt_grads(case, step)
        opt.step(mg, ag)
        for i, p in enumerate(muon):
            assert torch.equal(p, _t(gold[f"s{step}_muon_{i}"], dtype)), (step, i)
    for i, p in enumerate(muon):
        assert torch.equal(opt.state[id(p)]["momentum_buffer"], _t(gold[f"final_mom_{i}"], dtype))
    for i, p in enumerate(adamw):
        assert torch.equal(p, _t(gold[f"final_adamw_{i}"], dtype))
        st = opt.state[id(p)]
        assert st["step"] == int(gold[f"final_step_{i}"])
        assert torch.equal(st["exp_avg"], _t(gold[f"final_exp_avg_{i}"], dtype))
        assert torch.equal(st["exp_avg_sq"], _t(gold[f"final_exp_avg_sq_{i}"], dtype))


def test_absmax_codec_against_reference_kernel():
    gold = np.load(os.path.join(GOLD, "coat_absmax.npz"))
    g = gi.coat_input()
    assert gi.checksum(g) == int(gold["checksum"])
    codes, scales = fp8_oracle.absmax_quant(g)
    assert np.array_equal(scales.numpy().view(np.uint32), gold["q1_scales"].view(np.uint32))
    _codes_match_up_to_interpreter_carry(codes.numpy(), gold["q1_codes"])
    # dequantise -> halve -> requantise (the reference kernel's second step)
    m = fp8_oracle.absmax_dequant(codes, scales) * 0.5
    # feed the interpreter's own first-step codes so step 2 is compared on equal inputs
    m_ref_in = fp8_oracle.absmax_dequant(torch.from_numpy(gold["q1_codes"].copy()),
                                         torch.from_numpy(gold["q1_scales"].copy())) * 0.5
    c2, s2 = fp8_oracle.absmax_quant(m_ref_in)
    assert np.array_equal(s2.numpy().view(np.uint32), gold["q2_scales"].view(np.uint32))
    _codes_match_up_to_interpreter_carry(c2.numpy(), gold["q2_codes"])
    assert m.shape == g.shape


def _codes_match_up_to_interpreter_carry(ours: np.ndarray, ref: np.ndarray):
    """The interpreter's fp8 cast loses the carry when RTNE rounds a value up
    to the next power of two (it returns half the correct value).  Everywhere
    else the codes must be identical; at the carries ours must be the power of
    two and the interpreter's exactly half of it."""
    diff = ours != ref
    assert diff.mean() < 0.05
    a = fp8_oracle.e4m3_decode_numpy(ours[diff])
    b = fp8_oracle.e4m3_decode_numpy(ref[diff])
    assert np.all((ours[diff] & 0x07) == 0), "mismatch away from a mantissa carry"
    assert np.array_equal(a, 2.0 * b)


def test_e4m3_cast_two_implementations_agree():
    x = (torch.randn(200000, generator=torch.Generator().manual_seed(1))
         * torch.logspace(-12, 2.6, 200000)).clamp(-463, 463)
    x[:8] = torch.tensor([0.0, -0.0, 448.0, 449.0, 463.9, 2.0 ** -9, 2.0 ** -10, 1.5 * 2.0 ** -9])
    want = x.to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(fp8_oracle.e4m3_encode_numpy(x.numpy()), want)
    allc = np.arange(256, dtype=np.uint8)
    assert np.array_equal(fp8_oracle.e4m3_decode_numpy(allc),
                          torch.from_numpy(allc).view(torch.float8_e4m3fn).float().numpy(), equal_nan=True)


def test_expansion_codec_round_trip_and_edges():
    g = gi.coat_input()
    for signed, v in ((True, g), (False, g * g)):
        codes, scale, expand, sq = fp8_oracle.expand_quant(v, signed=signed)
        back = fp8_oracle.expand_dequant(codes, scale, expand, sq, signed=signed)
        nz = v != 0
        rel = ((back - v).abs()[nz] / v.abs()[nz])
        # E4M3 after range compression (expand < 1): coarse but bounded
        assert rel.max() < 0.6 and rel.mean() < 0.05
        assert torch.all(back[~nz] == 0)
        # all-zero group: expand 1, sqrt_minmax = eps, scale = 1/448 (coat_state_muon.py:56-71)
        assert expand[3] == 1.0 and scale[3] == pytest.approx(1.0 / 448.0)
        # expand is a multiple of 1/16 and at least 1/16
        assert torch.all(expand * 16 == torch.floor(expand * 16)) and expand.min() >= 1.0 / 16


def test_shape_book_keeping_matches_reference_counts():
    shapes = muon_oracle.llama_monarch_muon_shapes(4096, 32, 11008, 4)
    assert len(shapes) == 448
    assert sum(s[0] * s[1] * s[2] for s in shapes) == 2_558_525_440
    blocks = {}
    for nb, r, c in shapes:
        blocks[(r, c)] = blocks.get((r, c), 0) + nb
    assert blocks == {(1024, 1024): 1408, (2752, 1024): 256, (1024, 2752): 128}
    flops = sum(nb * muon_oracle.ns_flops(r, c) for nb, r, c in shapes)
    assert abs(flops / 1e12 - 71.640) < 0.01
    small = muon_oracle.llama_monarch_muon_shapes(256, 4, 688, 2)
    assert sum(s[0] * s[1] * s[2] for s in small) == 2_498_560


def test_sft_optimizer_three_steps_bit_exact():
    """oracle/sft_oracle.py against the reference's SFTOptimizer (fp32 master weights, bf16 parameters,
    Muon on a Monarch factor and on 2-D matrices, AdamW on the rest)."""
    from oracle import sft_oracle
    gold = np.load(os.path.join(GOLD, "sft.npz"))
    h = gi.SFT_HYPER
    muon, adamw = gi.sft_params()
    assert sum(gi.checksum(p.data) for p in muon + adamw) == int(gold["checksum_params"]), "CPU generator drifted"
    muon = [p.data for p in muon]
    adamw = [p.data for p in adamw]
    opt = sft_oracle.OracleSFT([{"params": muon, "algorithm": "muon", "lr": h["muon_lr"], "weight_decay": 0.0},
                                {"params": adamw, "algorithm": "adamw", "lr": h["adamw_lr"]}],
                               momentum=h["momentum"], betas=h["betas"], eps=h["eps"], weight_decay=h["weight_decay"])
    for step in range(gi.SFT_STEPS):
        mg, ag = gi.sft_grads(step)
        opt.step([mg, ag])
        for i, p in enumerate(muon + adamw):
            assert torch.equal(p, _t(gold[f"s{step}_p{i}"], torch.bfloat16)), (step, i)
    for i, p in enumerate(muon + adamw):
        st = opt.state[id(p)]
        assert torch.equal(st["master"], _t(gold[f"final_master_{i}"], torch.float32)), i
        assert torch.equal(st["momentum"], _t(gold[f"final_momentum_{i}"], torch.float32)), i
        if "variance" in st:
            assert torch.equal(st["variance"], _t(gold[f"final_variance_{i}"], torch.float32)), i
