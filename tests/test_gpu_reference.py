"""The CUDA path against THE REFERENCE ITSELF, run on the same GPU.

oracle/_ref/ holds the reference project's own files, unmodified (staged by
oracle/make_ref.py; a manifest of hashes is verified below).  Here its Triton
FP8 kernels are JIT-compiled on the GPU and its optimizer classes run as they
are, and this library's kernels are held against their outputs:

  absmax codec      COAT's plain kernel, pretrain/third_party/coat/optimizer/
                    triton_kernels.py:6-63              -> bit-exact
  expansion codec   quantize_/dequantize, pretrain/src/models/monarch/
                    coat_state_muon.py:22-114           -> expand_ and sqrt_minmax_
                    bit-exact; scale_ to a few ulp and codes to a few per million,
                    because the two sides get `pow` from different compilers
                    (see test_expansion_codec_against_the_reference_kernels)
  optimizer step    membench/src/models/monarch/monarch_muon.py (bf16) and
                    pretrain/.../coat_state_muon.py:117-151 (FP8 state), same seeded
                    inputs                              -> momentum bit-exact (bf16),
                    weights within the Newton-Schulz tolerance

The reference's own pin of its codec (pretrain/tests/test_coat_state_muon.py:25-51)
is run first, as it is, to show that the arbiter works on this GPU.
"""
import json
import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

E4M3 = torch.float8_e4m3fn


@pytest.fixture(scope="module")
def ref():
    from oracle import make_ref, ref_loader
    assert ref_loader.available(), "oracle/_ref/ is missing: run `python oracle/make_ref.py <reference checkout>`"
    assert make_ref.verify(), "a staged reference file no longer has its recorded hash"
    return ref_loader.pretrain()


@pytest.fixture(scope="module")
def mm():
    from monarch_muon_b200 import _lib, fp8_state
    return {"lib": _lib, "fp8": fp8_state}


def bits(t):
    if t.dtype == E4M3:
        return t.contiguous().view(torch.uint8).reshape(-1)
    if t.dtype == torch.bfloat16:
        return t.contiguous().view(torch.int16).reshape(-1)
    return t.contiguous().view(torch.int32).reshape(-1)


def mismatches(a, b) -> int:
    return int((bits(a) != bits(b)).sum().item())


def same_values(a, b) -> bool:
    """Equality the way the reference's own test states it (rtol=0, atol=0 on the float values: a
    negative and a positive zero code are the same value)."""
    return bool(torch.equal(a.float(), b.float()))


def cases():
    """The reference's own test tensor (pretrain/tests/test_coat_state_muon.py:27-28: (1000, 129), values
    over seven decades, numel not a multiple of 128, seed 23) and one 4-block Monarch factor of N(0, 1e-3)."""
    torch.manual_seed(23)
    p = torch.zeros(1000, 129, device="cuda")
    g = torch.randn_like(p) * torch.logspace(-6, 1, p.numel(), device="cuda").view_as(p)
    yield "1000x129_seven_decades", g
    gen = torch.Generator(device="cuda").manual_seed(5)
    yield "factor_4x1024x1024", torch.empty(4, 1024, 1024, device="cuda").normal_(0, 1e-3, generator=gen)


def coat_kernel_as_quantiser(ref, value, expansion: str):
    """COAT's fused FP8 AdamW kernel with lr 0, betas 0, weight decay 0: exp_avg becomes `value` and
    exp_avg_sq its square, each stored by the kernel's own quantiser (the trick of the reference's test)."""
    p = torch.zeros_like(value)
    p.grad = value.clone()
    q = ref.qconfig.QuantizationConfig(first_order_expansion=expansion, second_order_expansion=expansion)
    opt = ref.triton_fp8_adamw.TritonCoatAdamW([p], lr=0.0, betas=(0.0, 0.0), weight_decay=0.0, qargs=q)
    opt.step()
    return opt, p


def test_reference_own_codec_pin_passes_here(ref):
    """pretrain/tests/test_coat_state_muon.py::test_codec_is_the_coat_adamw_kernel, loaded from the staged
    copy and run unmodified."""
    import importlib
    import unittest
    mod = importlib.import_module("test_coat_state_muon")
    suite = unittest.TestSuite([mod.CoatStateMuonTests("test_codec_is_the_coat_adamw_kernel")])
    result = unittest.TextTestRunner(stream=open(os.devnull, "w")).run(suite)
    assert result.wasSuccessful(), result.failures + result.errors


@pytest.mark.parametrize("case", ["1000x129_seven_decades", "factor_4x1024x1024"])
def test_absmax_codec_is_bit_exact_with_the_reference_kernel(ref, mm, case):
    """FP8 codes and scales of the absmax codec, default arithmetic (MMB_DIV_FULL), against COAT's plain
    kernel on the GPU: quantise (signed first moment, unsigned second), then the second step of the
    reference's own test - dequantise, halve, requantise."""
    g = dict(cases())[case]
    opt, p = coat_kernel_as_quantiser(ref, g, "false")
    up = opt.state[p]
    for name, value, signed in (("exp_avg", g, True), ("exp_avg_sq", g * g, False)):
        ours = {}
        mm["fp8"].quantize_(ours, name, value, signed, E4M3, 16, codec="absmax")
        assert mismatches(ours[f"scale_{name}"], up[f"scale_{name}"]) == 0, name
        assert mismatches(ours[name], up[name]) == 0, name
    before = {}
    for name in ("exp_avg", "exp_avg_sq"):
        dec = mm["fp8"].dequantize({name: up[name].clone(), f"scale_{name}": up[f"scale_{name}"].clone()}, name, True,
                                   codec="absmax")
        want = up[name].float() * up[f"scale_{name}"].repeat_interleave(128)[: g.numel()].view_as(g)
        assert mismatches(dec, want) == 0                      # triton_kernels.py:34-36: float(code) * scale
        before[name] = dec
    for grp in opt.param_groups:
        grp["betas"] = (0.5, 0.5)
    p.grad.zero_()
    opt.step()
    for name in ("exp_avg", "exp_avg_sq"):
        ours = {}
        mm["fp8"].quantize_(ours, name, before[name] * 0.5, True, E4M3, 16, codec="absmax")
        assert mismatches(ours[f"scale_{name}"], up[f"scale_{name}"]) == 0, name
        # the kernel adds (1 - beta) * 0 = +0 to every element, which turns a negative zero into a positive
        # one: values are compared like the reference's own test compares them
        assert same_values(ours[name], up[name]), name


@pytest.mark.parametrize("gdtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("case", ["1000x129_seven_decades", "factor_4x1024x1024"])
def test_fused_absmax_momentum_is_bit_exact_with_the_reference_kernels(ref, mm, case, gdtype):
    """Three heavy-ball steps of the fused kernel on FP8 absmax state against the same steps assembled from
    the reference's pieces: float(code) * scale (triton_kernels.py:34-36), buf.mul_(beta).add_(grad)
    (monarch_muon.py:148), COAT's kernel as the quantiser (triton_kernels.py:51-63).  Codes, scales and
    the bf16 momentum must agree in every bit."""
    g = dict(cases())[case]
    opt, p = coat_kernel_as_quantiser(ref, g, "false")
    codes_ref, scale_ref = opt.state[p]["exp_avg"].clone(), opt.state[p]["scale_exp_avg"].clone()
    codes = codes_ref.clone().view(torch.uint8).reshape(-1)
    scale = scale_ref.clone()
    m16 = torch.empty(g.numel(), dtype=torch.bfloat16, device="cuda")
    gen = torch.Generator(device="cuda").manual_seed(11)
    for step in range(3):
        grad = (torch.empty_like(g).normal_(0, 1, generator=gen) * g.abs().mean()).to(gdtype)
        buf = codes_ref.float() * scale_ref.repeat_interleave(128)[: g.numel()].view_as(g)
        buf.mul_(0.95).add_(grad)
        o2, p2 = coat_kernel_as_quantiser(ref, buf, "false")
        codes_ref, scale_ref = o2.state[p2]["exp_avg"], o2.state[p2]["scale_exp_avg"]
        mm["fp8"].fp8_momentum_flat(codes, scale, grad.reshape(-1), 0.95, m_bf16=m16)
        assert mismatches(scale, scale_ref) == 0, step
        assert mismatches(codes.view(E4M3), codes_ref) == 0, step
        assert mismatches(m16, buf.bfloat16()) == 0, step


# Measured on a B200 (this test prints the table with `pytest -s`): with the default arithmetic the
# expansion codec's expand_ and sqrt_minmax_ equal the reference's in every bit; scale_ differs by one ulp
# (three at most) in about a third of the groups and the dequantised values by up to 5 ulp in about a third of the elements,
# because `pow` is the only operation the two sides do not share: Triton hands libdevice's powf body to its
# own LLVM, nvcc to NVVM, and the two compile it to different instruction sequences (the same kernel built
# from Triton's bundled libdevice, with and without -ftz / -fmad, gives nvcc's bits, not Triton's; log2
# agrees on every input).  Codes then differ where normalized / scale falls within that ulp of a rounding
# boundary: 0 to 3 elements in 4.2 million.  The bounds below are those measurements with some headroom,
# not tolerances chosen in advance.
EXPAND_CODES_PER_MILLION = 3.0
EXPAND_SCALE_ULP = 4      # measured: up to 3
EXPAND_DEQUANT_ULP = 8    # measured: up to 5


@pytest.mark.parametrize("case", ["1000x129_seven_decades", "factor_4x1024x1024"])
def test_expansion_codec_against_the_reference_kernels(ref, mm, case):
    g = dict(cases())[case]
    csm = ref.coat_state_muon
    lib = mm["lib"]
    report = {}
    for name, value, signed in (("exp_avg", g, True), ("exp_avg_sq", g * g, False)):
        want = {}
        csm.quantize_(want, name, value, signed, E4M3, 16)
        keys = (name, f"scale_{name}", f"expand_{name}", f"sqrt_minmax_{name}")
        for mode_name, mode in (("full", lib.DIV_FULL), ("ieee", lib.DIV_IEEE), ("ieee_strict", lib.DIV_IEEE_STRICT)):
            ours = {}
            mm["fp8"].quantize_(ours, name, value, signed, E4M3, 16, codec="expand", div_mode=mode)
            report[f"{name}/{mode_name}"] = {k: mismatches(ours[k], want[k]) for k in keys}
        ours = {}
        mm["fp8"].quantize_(ours, name, value, signed, E4M3, 16, codec="expand")          # default = full
        assert mismatches(ours[f"expand_{name}"], want[f"expand_{name}"]) == 0
        assert mismatches(ours[f"sqrt_minmax_{name}"], want[f"sqrt_minmax_{name}"]) == 0
        ulp = (bits(ours[f"scale_{name}"]) - bits(want[f"scale_{name}"])).abs().max()
        assert int(ulp) <= EXPAND_SCALE_ULP
        per_million = mismatches(ours[name], want[name]) / g.numel() * 1e6
        assert per_million <= max(EXPAND_CODES_PER_MILLION, 1e6 / g.numel()), per_million
        # dequantise the REFERENCE's state with both
        dec_ref = csm.dequantize(want, name, signed)
        dec = mm["fp8"].dequantize(want, name, signed, codec="expand")
        d = (bits(dec) - bits(dec_ref)).abs()
        report[f"{name}/dequantize"] = {"elements_differing": int((d != 0).sum()), "max_ulp": int(d.max())}
        assert int(d.max()) <= EXPAND_DEQUANT_ULP
        assert torch.equal(dec == 0, dec_ref == 0)
    print("\nexpansion codec vs reference kernels,", case, g.numel(), "elements:", json.dumps(report, indent=1))


def test_fused_expansion_momentum_against_the_reference_sequence(ref, mm):
    """CoatStateMonarchMuon's momentum path as the reference runs it - dequantize -> mul_(beta).add_(grad) ->
    quantize_ (coat_state_muon.py:126-139 around monarch_muon.py:148) - against the fused kernel, one step
    from the reference's own state.  expand_ must agree in all but a few groups per ten thousand (a last-bit
    difference of a decoded value moves the floor() by 1/16), codes in all but one element in ten thousand,
    the bf16 momentum in all but one in ten thousand."""
    g = dict(cases())["factor_4x1024x1024"]
    csm = ref.coat_state_muon
    lib = mm["lib"]
    st = {}
    csm.quantize_(st, "momentum_buffer", g, True, E4M3, 16)
    gen = torch.Generator(device="cuda").manual_seed(11)
    grad = torch.empty_like(g).normal_(0, 1e-3, generator=gen)
    buf = csm.dequantize(st, "momentum_buffer", True)
    buf.mul_(0.95).add_(grad)
    want = {}
    csm.quantize_(want, "momentum_buffer", buf, True, E4M3, 16)
    report = {}
    for mode_name, mode in (("full", lib.DIV_FULL), ("ieee", lib.DIV_IEEE)):
        c = st["momentum_buffer"].clone().view(torch.uint8).reshape(-1)
        s, e, q = (st[f"{k}_momentum_buffer"].clone() for k in ("scale", "expand", "sqrt_minmax"))
        m16 = torch.empty(g.numel(), dtype=torch.bfloat16, device="cuda")
        mm["fp8"].fp8_momentum_flat(c, s, grad.reshape(-1), 0.95, m_bf16=m16, div_mode=mode, expand=e, sqrt_minmax=q)
        n, ng = g.numel(), s.numel()
        report[mode_name] = {"codes_per_million": mismatches(c.view(E4M3), want["momentum_buffer"]) / n * 1e6,
                             "expand_groups": mismatches(e, want["expand_momentum_buffer"]),
                             "scale_groups": mismatches(s, want["scale_momentum_buffer"]),
                             "sqrt_minmax_groups": mismatches(q, want["sqrt_minmax_momentum_buffer"]),
                             "bf16_m_per_million": mismatches(m16, buf.bfloat16()) / n * 1e6, "groups": ng}
        assert report[mode_name]["codes_per_million"] <= 100.0
        assert report[mode_name]["expand_groups"] <= max(3, ng // 3000)
        assert report[mode_name]["bf16_m_per_million"] <= 100.0
    print("\nfused expansion momentum vs reference sequence:", json.dumps(report, indent=1))


# ---------------------------------------------------------------- whole optimizer steps
def _small_model_params(dtype, seed=3):
    gen = torch.Generator().manual_seed(seed)
    shapes = [(2, 128, 128), (2, 344, 128), (2, 128, 344), (4, 256, 256)]
    muon = [(0.02 * torch.randn(s, generator=gen)).to(dtype) for s in shapes]
    adamw = [(0.02 * torch.randn(1000, 64, generator=gen)).to(dtype), torch.ones(64, dtype=dtype)]
    grads = [[(1e-3 * torch.randn(t.shape, generator=gen)).to(dtype) for t in muon + adamw] for _ in range(3)]
    return muon, adamw, grads


def relf(a, b):
    return float((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-30))


def test_bf16_step_against_the_reference_class_on_the_gpu(mm):
    """Three steps of membench/src/models/monarch/monarch_muon.py's MonarchMuonOptimizer (the reference's
    bf16 path, run on the GPU from the staged copy) against this library's class on identical seeded
    inputs: momentum buffers bit-exact, AdamW state and weights within the stated tolerances."""
    from monarch_muon_b200 import MonarchMuonOptimizer
    from oracle import ref_loader
    twin = ref_loader.membench_twin()
    muon, adamw, grads = _small_model_params(torch.bfloat16)
    a_m = [torch.nn.Parameter(t.clone().cuda()) for t in muon]
    a_a = [torch.nn.Parameter(t.clone().cuda()) for t in adamw]
    b_m = [torch.nn.Parameter(t.clone().cuda()) for t in muon]
    b_a = [torch.nn.Parameter(t.clone().cuda()) for t in adamw]
    kw = dict(lr=0.02, momentum=0.95, adamw_betas=(0.9, 0.95), adamw_weight_decay=0.1, adamw_eps=1e-8)
    theirs = twin.MonarchMuonOptimizer(a_m, a_a, **kw)
    ours = MonarchMuonOptimizer(b_m, b_a, **kw)
    theirs.param_groups[1]["lr"] = ours.param_groups[1]["lr"] = 3e-4      # the class has one lr for both groups
    w0 = [p.data.clone() for p in b_m]
    for gs in grads:
        for p, g in zip(a_m + a_a, gs):
            p.grad = g.clone().cuda()
        for p, g in zip(b_m + b_a, gs):
            p.grad = g.clone().cuda()
        theirs.step()
        ours.step()
        for pa, pb in zip(a_m, b_m):
            assert mismatches(theirs.state[pa]["momentum_buffer"], ours.state[pb]["momentum_buffer"]) == 0
    for pa, pb, w in zip(a_m, b_m, w0):
        assert relf(pb.data, pa.data) < 1e-2                       # weights
        assert relf(pb.data - w, pa.data - w) < 1.2e-1             # three steps' increment, bf16 storage
    for pa, pb in zip(a_a, b_a):
        # AdamW: the kernel issues the instructions torch's CUDA kernels issue, so everything is equal bit for bit
        assert mismatches(pb.data, pa.data) == 0
        assert mismatches(ours.state[pb]["exp_avg"], theirs.state[pa]["exp_avg"]) == 0
        assert mismatches(ours.state[pb]["exp_avg_sq"], theirs.state[pa]["exp_avg_sq"]) == 0


@pytest.mark.parametrize("twin_name", ["pretrain", "membench"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_adamw_is_bit_exact_with_the_reference_classes_on_the_gpu(twin_name, dtype):
    """The AdamW group of both reference twins (pretrain/src/models/monarch/monarch_muon.py:171-201, separate
    torch ops per tensor; membench/src/models/monarch/monarch_muon.py:176-208, torch._foreach ops), run on the
    GPU, against `adamw_kernel`: parameters and both moments equal bit for bit after each of five steps, with
    weight decay, a ragged tensor and a short vector.  What that takes: hyper-parameters as doubles (1 - beta
    formed like Python forms it), `addcmul_` as fma(value, g*g, v), and the division by sqrt(1 - beta2^t) as a
    multiplication by its reciprocal formed in double - what torch's CUDA kernels do."""
    from monarch_muon_b200 import MonarchMuonOptimizer
    from oracle import ref_loader
    twin = ref_loader.pretrain_twin() if twin_name == "pretrain" else ref_loader.membench_twin()
    gen = torch.Generator().manual_seed(77)
    shapes = [(1000, 64), (64,), (333, 77), (128 * 40,)]
    w = [(0.05 * torch.randn(s, generator=gen)).to(dtype) for s in shapes]
    a = [torch.nn.Parameter(t.clone().cuda()) for t in w]
    b = [torch.nn.Parameter(t.clone().cuda()) for t in w]
    kw = dict(lr=3e-4, momentum=0.95, adamw_betas=(0.9, 0.95), adamw_weight_decay=0.1, adamw_eps=1e-8)
    theirs = twin.MonarchMuonOptimizer([], a, **kw)
    ours = MonarchMuonOptimizer([], b, **kw)
    for step in range(5):
        for pa, pb, sh in zip(a, b, shapes):
            n = int(torch.Size(sh).numel())
            g = (1e-2 * torch.randn(sh, generator=gen) * torch.logspace(-3, 0, n).view(sh)).to(dtype)
            pa.grad = g.clone().cuda()
            pb.grad = g.clone().cuda()
        theirs.step()
        ours.step()
        for pa, pb in zip(a, b):
            assert mismatches(pb.data, pa.data) == 0, (step, tuple(pa.shape))
            assert mismatches(ours.state[pb]["exp_avg"], theirs.state[pa]["exp_avg"]) == 0, (step, tuple(pa.shape))
            assert mismatches(ours.state[pb]["exp_avg_sq"], theirs.state[pa]["exp_avg_sq"]) == 0, (step, tuple(pa.shape))


def test_fp8_state_step_against_the_reference_class_on_the_gpu(ref):
    """CoatStateMonarchMuon, the reference's (pretrain/src/models/monarch/coat_state_muon.py:117-151, fp32
    parameters as in the pretraining recipe) against this library's, three steps on identical inputs: state
    dtypes and keys equal; after the first step (m = g on both sides) expand_/sqrt_minmax_ of the momentum
    bit-exact and codes equal to a few per million; weights within the Newton-Schulz tolerance."""
    from monarch_muon_b200 import CoatStateMonarchMuon
    muon, adamw, grads = _small_model_params(torch.float32)
    a_m = [torch.nn.Parameter(t.clone().cuda()) for t in muon]
    a_a = [torch.nn.Parameter(t.clone().cuda()) for t in adamw]
    b_m = [torch.nn.Parameter(t.clone().cuda()) for t in muon]
    b_a = [torch.nn.Parameter(t.clone().cuda()) for t in adamw]
    q = ref.qconfig.QuantizationConfig()
    kw = dict(lr=0.02, momentum=0.95, adamw_betas=(0.9, 0.95), adamw_weight_decay=0.1, adamw_eps=1e-8)
    theirs = ref.coat_state_muon.CoatStateMonarchMuon(a_m, a_a, qargs=q, **kw)
    ours = CoatStateMonarchMuon(b_m, b_a, qargs=q, **kw)
    theirs.param_groups[1]["lr"] = ours.param_groups[1]["lr"] = 3e-4      # the class has one lr for both groups
    w0 = [p.data.clone() for p in b_m]
    for step, gs in enumerate(grads):
        for p, g in zip(a_m + a_a, gs):
            p.grad = g.clone().cuda()
        for p, g in zip(b_m + b_a, gs):
            p.grad = g.clone().cuda()
        theirs.step()
        ours.step()
        for pa, pb in zip(a_m + a_a, b_m + b_a):
            sa, sb = theirs.state[pa], ours.state[pb]
            assert set(k for k in sa if torch.is_tensor(sa[k])) == set(k for k in sb if torch.is_tensor(sb[k]))
            for k, v in sa.items():
                if torch.is_tensor(v):
                    assert sb[k].dtype == v.dtype and sb[k].shape == v.shape, k
        if step == 0:
            for pa, pb in zip(a_m, b_m):
                sa, sb = theirs.state[pa], ours.state[pb]
                assert mismatches(sa["expand_momentum_buffer"], sb["expand_momentum_buffer"]) == 0
                assert mismatches(sa["sqrt_minmax_momentum_buffer"], sb["sqrt_minmax_momentum_buffer"]) == 0
                assert mismatches(sa["momentum_buffer"], sb["momentum_buffer"]) <= max(1, pa.numel() // 100000)
            for pa, pb in zip(a_a, b_a):
                # AdamW moments after the first step (zero state on both sides): the values that are encoded are
                # equal bit for bit (see test_adamw_is_bit_exact_...), so codes, expand_ and sqrt_minmax_ are too;
                # scale_ goes through `pow`, which the two sides get from different compilers
                sa, sb = theirs.state[pa], ours.state[pb]
                for name in ("exp_avg", "exp_avg_sq"):
                    assert mismatches(sa[name], sb[name]) <= max(1, pa.numel() // 100000), name
                    assert mismatches(sa[f"expand_{name}"], sb[f"expand_{name}"]) == 0, name
                    assert mismatches(sa[f"sqrt_minmax_{name}"], sb[f"sqrt_minmax_{name}"]) == 0, name
                    assert float((sa[f"scale_{name}"] / sb[f"scale_{name}"] - 1).abs().max()) < 1e-6, name
    for pa, pb, w in zip(a_m, b_m, w0):
        # the reference orthogonalises in fp32/TF32 here (fp32 parameters), this library in bf16
        assert relf(pb.data - w, pa.data - w) < 5e-2
    for pa, pb in zip(a_a, b_a):
        # both sides keep the moments as E4M3 between steps; the fused kernel contracts to FMA where the
        # reference runs separate torch ops, so a few moment codes differ and with them m / sqrt(v)
        print("adamw relF", relf(pb.data, pa.data))
        assert relf(pb.data, pa.data) < 1e-3
