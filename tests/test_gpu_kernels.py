"""GPU parity of the individual kernels, through the C ABI, against the CPU oracle."""
import numpy as np
import pytest
import torch

import golden_inputs as gi

pytestmark = pytest.mark.gpu


def relf(a, b):
    a = a.float().cpu()
    b = b.float().cpu()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


@pytest.fixture(scope="module")
def mm():
    from monarch_muon_b200 import _lib, fp8_state, newton_schulz
    _lib.load()
    return dict(lib=_lib, fp8=fp8_state, ns=newton_schulz)


# ------------------------------------------------------------------ GEMM family
GEMM_CASES = [
    # batch, M, N, K
    (3, 128, 128, 128),
    (2, 256, 512, 192),
    (2, 1024, 1024, 1024),
    (2, 344, 128, 128),      # ragged M (not a multiple of 128)
    (2, 128, 344, 128),      # ragged N
    (2, 128, 128, 344),      # ragged K (not a multiple of 64)
    (1, 1024, 2752, 1024),
    (1, 2752, 1024, 1024),
    (2, 64, 64, 256),        # the 64-wide tile variant
]


def _backend(mm, name):
    return mm["lib"].NS_TCGEN05 if name == "tcgen05" else mm["lib"].NS_SIMT


def _check(got, want):
    # fp32 accumulation of exact bf16 products; only the final bf16 rounding differs
    assert relf(got, want) < 4e-3, relf(got, want)
    assert torch.allclose(got.float().cpu(), want, rtol=1.6e-2, atol=1e-2 * float(want.abs().max()))


@pytest.mark.parametrize("backend", ["tcgen05", "simt"])
@pytest.mark.parametrize("a_k,b_k", [(True, True), (True, False), (False, True), (False, False)])
@pytest.mark.parametrize("shape", GEMM_CASES, ids=lambda s: "x".join(map(str, s)))
def test_gemm_family(mm, shape, a_k, b_k, backend):
    batch, M, N, K = shape
    if backend == "simt" and M * N * K > 256 * 512 * 192:
        pytest.skip("the CUDA-core cross-check kernel is only exercised on small shapes")
    g = torch.Generator().manual_seed(hash(shape) % 1000 + 2 * a_k + b_k)
    a = torch.randn(batch, M, K, generator=g).bfloat16()
    b = torch.randn(batch, N, K, generator=g).bfloat16()
    inv = torch.rand(batch, generator=g) * 0.1 + 0.01
    alpha, diag = 2.0315, -1.175
    want = (inv.view(-1, 1, 1) ** 2) * alpha * (a.float() @ b.float().transpose(1, 2))
    idx = torch.arange(min(M, N))
    want[:, idx, idx] += diag
    a_dev = (a if a_k else a.transpose(1, 2).contiguous()).cuda()
    b_dev = (b if b_k else b.transpose(1, 2).contiguous()).cuda()
    L = mm["lib"]
    got = mm["ns"].gemm_bf16(a_dev, b_dev, a_mode=L.GEMM_K if a_k else L.GEMM_MN,
                             b_mode=L.GEMM_K if b_k else L.GEMM_MN, alpha=alpha, diag=diag,
                             inv_norm=inv.cuda(), sigma_pow=2, backend=_backend(mm, backend))
    assert L.read_status(got.device) == 0
    _check(got, want)


def _poison_lower_blocks(s):
    """NaN in every 256x256 block strictly below the block diagonal: a symmetric
    operand must never be read there."""
    out = s.clone()
    m = s.shape[-1]
    r = torch.arange(m) // 256
    below = r.view(-1, 1) > r.view(1, -1)
    out[:, below] = float("nan")
    return out, below


@pytest.mark.parametrize("backend", ["tcgen05", "simt"])
@pytest.mark.parametrize("m,n", [(1024, 1024), (512, 1280), (344, 128), (1024, 2752), (128, 128)])
def test_gemm_symmetric_operands(mm, m, n, backend):
    if backend == "simt" and m * n > 512 * 1280:
        pytest.skip("cross-check kernel only on small shapes")
    L = mm["lib"]
    g = torch.Generator().manual_seed(m + n)
    h = torch.randn(2, m, m, generator=g).bfloat16()
    sym = (h.float() + h.float().transpose(1, 2)).bfloat16()      # exactly symmetric in bf16
    x = torch.randn(2, m, n, generator=g).bfloat16()              # stored [K=m][N=n] -> MN-major B
    y = torch.randn(2, n, m, generator=g).bfloat16()              # stored [M=n][K=m] -> K-major A
    poisoned, below = _poison_lower_blocks(sym)
    be = _backend(mm, backend)
    # A symmetric:  D = S X
    got = mm["ns"].gemm_bf16(poisoned.cuda(), x.cuda(), a_mode=L.GEMM_SYM, b_mode=L.GEMM_MN, backend=be)
    _check(got, sym.float() @ x.float())
    # B symmetric:  D = Y S
    got = mm["ns"].gemm_bf16(y.cuda(), poisoned.cuda(), a_mode=L.GEMM_K, b_mode=L.GEMM_SYM, backend=be)
    _check(got, y.float() @ sym.float())
    # both symmetric, symmetric output: only blocks on or above the block diagonal are written
    out = torch.full((2, m, m), 7.0, dtype=torch.bfloat16, device="cuda")
    mm["ns"].gemm_bf16(poisoned.cuda(), poisoned.cuda(), a_mode=L.GEMM_SYM, b_mode=L.GEMM_SYM, sym_out=True,
                       alpha=0.5, diag=0.25, backend=be, out=out)
    want = 0.5 * (sym.float() @ sym.float()) + 0.25 * torch.eye(m)
    got = out.float().cpu()
    assert torch.all(got[:, below] == 7.0)                         # untouched
    keep = ~below
    assert relf(got[:, keep], want[:, keep]) < 4e-3
    assert L.read_status(out.device) == 0


# ------------------------------------------------------------------ Newton-Schulz
NS_SHAPES = [(3, 128, 128), (2, 344, 128), (2, 128, 344), (2, 256, 256), (2, 256, 512), (2, 1024, 1024), (1, 2752, 1024),
             (1, 1024, 2752),
             # the 2-block variant of the model: m = 2048 runs 8 x 8 pair tiles, 36 of 64 of them for symmetric products
             (1, 2048, 2048), (1, 5504, 2048), (1, 2048, 5504)]

# Tolerances, relative Frobenius norm per stack.  The reference's own bf16 path
# differs from its fp32 path by e_ref (about 2.4e-2 on N(0,1) blocks, more on
# ill-conditioned ones) because the quintic amplifies the rounding of small
# singular values.  This kernel rounds in fewer places, so it must be at least
# as close to the fp32 oracle as the reference's bf16 path is (15 % slack for
# different rounding points), and - two independent perturbations of that size
# adding in quadrature - within 1.5 e_ref of the bf16 oracle.
NS_SLACK_VS_BF16_ORACLE = 1.5
NS_SLACK_VS_FP32 = 1.15


@pytest.mark.parametrize("backend", ["tcgen05", "simt"])
@pytest.mark.parametrize("shape", NS_SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_newton_schulz_against_oracle(mm, shape, backend):
    from oracle import muon_oracle
    if backend == "simt" and shape[1] * shape[2] > 256 * 512:
        pytest.skip("cross-check kernel only on small shapes")
    g = torch.Generator().manual_seed(sum(shape))
    x = torch.randn(shape, generator=g).bfloat16()
    ref32 = muon_oracle.newton_schulz(x.float())
    ref16 = muon_oracle.newton_schulz(x)
    be = mm["lib"].NS_TCGEN05 if backend == "tcgen05" else mm["lib"].NS_SIMT
    got = mm["ns"].newton_schulz_batched(x.cuda(), backend=be)
    assert mm["lib"].read_status(got.device) == 0
    assert torch.isfinite(got).all()
    e_ref = relf(ref16, ref32)
    e_got32 = relf(got, ref32)
    e_got16 = relf(got, ref16)
    print(f"NS {shape} {backend}: ours-vs-fp32 {e_got32:.3e}  ref-bf16-vs-fp32 {e_ref:.3e}  ours-vs-bf16 {e_got16:.3e}")
    assert e_got32 <= max(NS_SLACK_VS_FP32 * e_ref, 1e-2)
    assert e_got16 <= max(NS_SLACK_VS_BF16_ORACLE * e_ref, 1.5e-2)
    # scale invariance of the normalised iteration: NS(7x) == NS(x) up to bf16 noise
    got7 = mm["ns"].newton_schulz_batched((x * 7).cuda(), backend=be)
    assert relf(got7, got) < 3e-2


@pytest.mark.parametrize("wdtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("backend", ["tcgen05", "simt"])
@pytest.mark.parametrize("shape", [(3, 128, 128), (2, 344, 128), (2, 128, 344), (5, 256, 512), (2, 64, 64),
                                   (3, 1024, 1024), (2, 2752, 1024), (2, 1024, 2752)],
                         ids=lambda s: "x".join(map(str, s)))
def test_newton_schulz_with_fused_update_equals_two_kernels(mm, shape, backend, wdtype):
    """mmb_newton_schulz_update (the update applied in the epilogue of the last GEMM) must leave exactly
    the weights that mmb_newton_schulz followed by mmb_muon_update leaves: same bf16 rounding of the
    orthogonalised block, same fused multiply-add, same rounding to the weights' type - for bf16 and fp32
    weights, wide, tall, ragged and small blocks, blocks scattered over separate tensors, and with the
    dynamic tile schedule."""
    L = mm["lib"]
    if backend == "simt" and shape[1] * shape[2] > 256 * 512:
        pytest.skip("cross-check kernel only on small shapes")
    be = L.NS_TCGEN05 if backend == "tcgen05" else L.NS_SIMT
    batch, rows, cols = shape
    g = torch.Generator().manual_seed(sum(shape) + 1)
    x = torch.randn(shape, generator=g).bfloat16().cuda()
    # blocks of two "parameters" that are not adjacent in memory
    n0 = batch // 2 + 1
    wa = (0.02 * torch.randn(n0, rows, cols, generator=g)).to(wdtype).cuda()
    wb = (0.02 * torch.randn(batch - n0, rows, cols, generator=g)).to(wdtype).cuda()
    alpha = -0.02 * (rows / cols) ** 0.5
    want = torch.cat([wa, wb]).clone()
    ortho = mm["ns"].newton_schulz_batched(x, backend=be)
    seg = (L.UpdateSeg * 1)()
    seg[0].weight, seg[0].ortho, seg[0].numel = want.data_ptr(), ortho.data_ptr(), want.numel()
    L.check(L.load().mmb_muon_update(seg, 1, L.dtype_code(wdtype), alpha, L.stream_ptr()))
    esz = wa.element_size()
    ptrs = [wa.data_ptr() + k * rows * cols * esz for k in range(n0)] + \
           [wb.data_ptr() + k * rows * cols * esz for k in range(batch - n0)]
    table = torch.tensor(ptrs, dtype=torch.int64).cuda()
    x_before = x.clone()
    for dynamic in ((False, True) if backend == "tcgen05" else (False,)):
        a2, b2 = wa.clone(), wb.clone()
        ptrs2 = [a2.data_ptr() + k * rows * cols * esz for k in range(n0)] + \
                [b2.data_ptr() + k * rows * cols * esz for k in range(batch - n0)]
        table2 = torch.tensor(ptrs2, dtype=torch.int64).cuda()
        with L.launch_options(dynamic_schedule=dynamic):
            mm["ns"].newton_schulz_update(x, table2, wdtype, alpha, backend=be)
        assert L.read_status(x.device) == 0
        got = torch.cat([a2, b2])
        assert torch.equal(got, want), (dynamic, float((got.float() - want.float()).abs().max()))
    assert torch.equal(x, x_before)                      # the input stack is only read
    del table


def test_dependent_launch_does_not_change_the_result(mm):
    """The GEMMs of one Newton-Schulz call follow one another with programmatic stream serialisation by
    default (a kernel's CTAs set up while the previous kernel drains, then wait for it); launched plainly
    they must give the same bits."""
    L = mm["lib"]
    g = torch.Generator().manual_seed(77)
    x = torch.randn(6, 512, 1376, generator=g).to(torch.bfloat16).cuda()
    be = L.NS_TCGEN05_MULTI
    a = mm["ns"].newton_schulz_batched(x, backend=be).clone()
    with L.launch_options(dependent_launch=False):
        b = mm["ns"].newton_schulz_batched(x, backend=be).clone()
    with L.launch_options(dependent_launch=False, dynamic_schedule=True):
        c = mm["ns"].newton_schulz_batched(x, backend=be).clone()
    with L.launch_options(dynamic_schedule=True):
        d = mm["ns"].newton_schulz_batched(x, backend=be).clone()
    assert L.read_status(x.device) == 0
    assert torch.equal(a, b) and torch.equal(a, c) and torch.equal(a, d)


def test_bounded_wait_expires_and_reports(mm):
    """A wait that nothing answers: one warp runs the GEMM's own bounded wait, with a limit of about a
    millisecond, on a barrier no one arrives at.  The kernel must return, the status word must hold the
    probe's code, and the device must go on working (a normal GEMM afterwards, status 0)."""
    L = mm["lib"]
    dev = torch.device("cuda", torch.cuda.current_device())
    assert L.read_status(dev) == 0
    L.check(L.load().mmb_wait_probe(2_000_000, L.status_word(dev), L.stream_ptr()), "wait_probe")
    assert L.read_status(dev, reset=False) == L.STATUS_WAIT_PROBE      # first writer wins, stays until reset
    assert L.read_status(dev) == L.STATUS_WAIT_PROBE
    assert L.read_status(dev) == 0
    a = torch.randn(2, 256, 256, generator=torch.Generator().manual_seed(1)).bfloat16().cuda()
    got = mm["ns"].gemm_bf16(a, a)
    _check(got, a.float().cpu() @ a.float().cpu().transpose(1, 2))
    assert L.read_status(dev) == 0
    assert L.load().mmb_wait_probe(0, L.status_word(dev), L.stream_ptr()) != 0   # limits outside 1..2e9 are refused


def test_newton_schulz_in_place_and_sliced(mm):
    x = torch.randn(5, 256, 128, generator=torch.Generator().manual_seed(3)).bfloat16().cuda()
    a = mm["ns"].newton_schulz_batched(x)
    b = mm["ns"].newton_schulz_batched(x, max_batch=2)
    assert torch.equal(a, b)                       # batch slicing does not change any block
    y = x.clone()
    mm["ns"].newton_schulz_batched(y, out=y)
    assert torch.equal(a, y)                       # in place
    z = mm["ns"].newton_schulz_batched(x)
    assert torch.equal(a, z)                       # run-to-run bit reproducibility


def test_dynamic_tile_schedule_gives_the_same_bits(mm):
    """Newton-Schulz with tiles drawn from a counter instead of the fixed round-robin: every tile is
    computed exactly once by the same code, so the output is bit-identical; the counters rearm
    themselves, so repeated calls and several shapes in a row work."""
    lib = mm["lib"]
    gen = torch.Generator(device="cuda").manual_seed(12)
    stacks = [torch.empty(s, dtype=torch.bfloat16, device="cuda").normal_(0, 1, generator=gen)
              for s in ((40, 1024, 1024), (3, 2752, 1024), (5, 1024, 2752), (2, 512, 256))]
    ns = mm["ns"].newton_schulz_batched
    want = [ns(x) for x in stacks]
    lib.set_gemm_schedule(True)
    try:
        for rep in range(3):
            for x, w in zip(stacks, want):
                assert torch.equal(ns(x), w), (rep, tuple(x.shape))
        assert lib.read_status(torch.device("cuda", torch.cuda.current_device())) == 0
    finally:
        lib.set_gemm_schedule(False)


# ------------------------------------------------------------------ FP8 momentum
@pytest.mark.parametrize("n,block", [(128 * 40 + 5, None), (4 * 128 * 128, 128 * 128), (2 * 344 * 128, 344 * 128),
                                     (1 << 22, 1 << 20), (17, None)])
@pytest.mark.parametrize("gdtype", [torch.bfloat16, torch.float32])
def test_fp8_absmax_momentum_bit_exact(mm, n, block, gdtype):
    from oracle import fp8_oracle
    gen = torch.Generator().manual_seed(n % 997)
    m0 = torch.randn(n, generator=gen) * 1e-3
    if block is None:
        m0 = m0 * torch.logspace(-4, 2, n)         # wide dynamic range, exercises the tail group
    codes, scales = fp8_oracle.absmax_quant(m0)
    d_codes, d_scales = codes.cuda(), scales.cuda()
    d_m = torch.empty(n, dtype=torch.bfloat16, device="cuda")
    nblk = n // block if block else 1
    for step in range(3):
        g = (torch.randn(n, generator=gen) * 1e-3).to(gdtype)
        codes, scales, m32, m16 = fp8_oracle.absmax_momentum_step(codes, scales, g, 0.95)
        d_ss = torch.zeros(nblk, device="cuda")
        mm["fp8"].fp8_momentum_flat(d_codes, d_scales, g.cuda(), 0.95, m_bf16=d_m, block_elems=block,
                                    block_sumsq=d_ss, div_mode=mm["lib"].DIV_IEEE)
        assert torch.equal(d_codes.cpu(), codes), f"codes differ at step {step}"
        assert np.array_equal(d_scales.cpu().numpy().view(np.uint32), scales.numpy().view(np.uint32))
        assert torch.equal(d_m.cpu(), m16)
        want_ss = m32.double().pow(2).view(nblk, -1).sum(1)
        assert torch.allclose(d_ss.cpu().double(), want_ss, rtol=1e-5)


def test_fp8_momentum_grad_scale_and_full_div(mm):
    from oracle import fp8_oracle
    n = 128 * 64
    gen = torch.Generator().manual_seed(5)
    codes, scales = fp8_oracle.absmax_quant(torch.randn(n, generator=gen) * 1e-3)
    g = (torch.randn(n, generator=gen) * 1e-3).bfloat16()
    want = fp8_oracle.absmax_momentum_step(codes, scales, g, 0.95, grad_scale=0.125)
    dc, ds = codes.cuda(), scales.cuda()
    mm["fp8"].fp8_momentum_flat(dc, ds, g.cuda(), 0.95, grad_scale=0.125, div_mode=mm["lib"].DIV_IEEE)
    assert torch.equal(dc.cpu(), want[0]) and torch.equal(ds.cpu(), want[1])
    # approximate-division mode (what the reference's Triton build emits): scales within 2 ulp,
    # codes equal except where the quotient sits on a rounding boundary
    dc2, ds2 = codes.cuda(), scales.cuda()
    mm["fp8"].fp8_momentum_flat(dc2, ds2, g.cuda(), 0.95, grad_scale=0.125, div_mode=mm["lib"].DIV_FULL)
    ulp = (ds2.cpu().view(torch.int32) - want[1].view(torch.int32)).abs().max()
    assert ulp <= 2
    assert (dc2.cpu() != want[0]).float().mean() < 1e-3


@pytest.mark.parametrize("n", [128 * 4096, 128 * 333 + 77])
def test_fp8_expand_momentum_against_oracle(mm, n):
    """Fused momentum in the range-expansion format.  pow/log2 come from different libraries on the two
    sides (libm in the oracle, libdevice or the special-function unit on the GPU), so group parameters
    agree to rounding noise and codes almost everywhere, as for the stand-alone codec.  The default
    arithmetic (exact quotients + hardware pow for exponents <= 4) is held against the strict one
    (compiler division + library powf): expand equal in all but a few groups, group parameters equal to
    rounding noise in all but a few, at most 1 code in 2000 different."""
    from oracle import fp8_oracle
    lib = mm["lib"]
    gen = torch.Generator().manual_seed(31 + n % 7)
    v = torch.randn(n, generator=gen) * 1e-3 * torch.logspace(-2, 1, n)
    v[::97] = 0.0                                           # zeros are skipped by absmin and decode to 0
    v[128 * 5:128 * 6] = 0.0                                # an all-zero group
    v[128 * 9:128 * 10] = 3e-4                              # a constant group: ratio 1 -> expand 1
    codes, scale, expand, sq = fp8_oracle.expand_quant(v)
    g = (torch.randn(n, generator=gen) * 1e-3).bfloat16()
    want = fp8_oracle.expand_momentum_step(codes, scale, expand, sq, g, 0.95)
    got = {}
    for name, mode in (("default", lib.DIV_IEEE), ("strict", lib.DIV_IEEE_STRICT), ("full", lib.DIV_FULL)):
        d = [t.cuda() for t in (codes, scale, expand, sq)]
        m16 = torch.empty(n, dtype=torch.bfloat16, device="cuda")
        ss = torch.zeros(1, device="cuda")
        mm["fp8"].fp8_momentum_flat(d[0], d[1], g.cuda(), 0.95, m_bf16=m16, block_sumsq=ss, div_mode=mode,
                                    expand=d[2], sqrt_minmax=d[3])
        got[name] = [t.cpu() for t in d] + [m16.cpu(), ss.cpu()]
    for name, (c, s, e, q, m16, ss) in got.items():
        # expand comes out of a floor(): last-bit differences in the decoded state move it by 1/16 in a
        # few groups, and the scale with it; everything else is compared where expand agrees
        same = e == want[2]
        assert same.float().mean() > 0.95, name
        # a group's smallest element is often what beta*m + g nearly cancels to, which magnifies last-bit
        # differences of the decoded m: the group parameters agree to 1e-5 in most groups (94 % measured
        # with the hardware pow, 99 % with the library's) and to a fraction of a percent in the rest; they
        # are stored with the codes, so a group stays consistent with itself either way
        for ours, ref in ((s[same], want[1][same]), (q, want[3])):
            rel = (ours - ref).abs() / ref
            assert (rel > 1e-5).float().mean() < 0.15 and rel.max() < 1e-2, name
        assert (c != want[0]).float().mean() < 1e-3, name
        # the decoded old state enters m: bf16 copies agree except for last-bit flips
        assert relf(m16.float(), want[4]) < 5e-3, name
        assert torch.allclose(ss.double(), want[4].double().pow(2).sum().view(1), rtol=1e-4), name
        assert torch.all(m16.float()[want[4] == 0] == 0), name
    dc, ds, de, dq, dm, _ = got["default"]
    sc, ss_, se, sq_, sm, _ = got["strict"]
    same = de == se
    assert same.float().mean() > 0.999
    for ours, ref in ((dq, sq_), (ds[same], ss_[same])):
        rel = (ours - ref).abs() / ref
        assert (rel > 1e-5).float().mean() < 0.15 and rel.max() < 1e-2
    assert (dc != sc).float().mean() < 5e-4
    assert (dm != sm).float().mean() < 2e-3


@pytest.mark.parametrize("codec", ["absmax", "expand"])
@pytest.mark.parametrize("signed", [True, False])
def test_standalone_codecs(mm, codec, signed):
    from oracle import fp8_oracle
    g = gi.coat_input()
    v = g if signed else g * g
    st = {}
    mm["fp8"].quantize_(st, "exp_avg", v.cuda(), signed=signed, codec=codec, div_mode=mm["lib"].DIV_IEEE)
    back = mm["fp8"].dequantize(st, "exp_avg", signed=signed)
    if codec == "absmax":
        codes, scales = fp8_oracle.absmax_quant(v)
        assert torch.equal(st["exp_avg"].view(torch.uint8).cpu(), codes)
        assert torch.equal(st["scale_exp_avg"].cpu(), scales)
        assert torch.equal(back.cpu(), fp8_oracle.absmax_dequant(codes, scales))
    else:
        codes, scale, expand, sq = fp8_oracle.expand_quant(v, signed=signed)
        # pow/log2 differ in the last bits between libm and the GPU's libdevice:
        # the per-group parameters agree to fp32 rounding noise, the codes almost everywhere
        assert torch.allclose(st["scale_exp_avg"].cpu(), scale, rtol=1e-5)
        assert torch.allclose(st["sqrt_minmax_exp_avg"].cpu(), sq, rtol=1e-6)
        same_expand = st["expand_exp_avg"].cpu() == expand
        assert same_expand.float().mean() > 0.95
        mism = (st["exp_avg"].view(torch.uint8).cpu() != codes).float().mean()
        assert mism < 0.05
        want = fp8_oracle.expand_dequant(codes, scale, expand, sq, signed=signed)
        nz = v != 0
        assert relf(back.cpu()[nz], v[nz]) < 0.08 and relf(want[nz], v[nz]) < 0.08
        assert torch.all(back.cpu()[~nz] == 0)


def test_fast_exact_quotient_equals_compiler_division_on_many_elements(mm):
    """MMB_DIV_IEEE forms m/s with a reciprocal and one correction step; it must give the bits of the
    compiler's IEEE division (MMB_DIV_IEEE_STRICT) - here on 2^28 elements over a wide range of group
    scales, including groups whose scale has an all-ones mantissa, infinities and zeros."""
    n = 1 << 28
    gen = torch.Generator(device="cuda").manual_seed(77)
    g = torch.empty(n, device="cuda").normal_(0, 1, generator=gen)
    g *= torch.pow(10.0, torch.empty(n // 128, device="cuda").uniform_(-12, 4, generator=gen)).repeat_interleave(128)
    g[:128] = 0.0
    # a group whose new scale (absmax + 1e-20)/448 has an all-ones mantissa (the correction step's one
    # exception): search the neighbourhood of 448 * 1.9999999 for such an absmax
    import numpy as np
    top = np.array([0x3FFFFFFF], dtype=np.uint32).view(np.float32)[0]
    near = (np.array([np.float32(top * np.float32(448.0))]).view(np.uint32)[0]
            + np.arange(-2000, 2000)).astype(np.uint32).view(np.float32)
    sc = ((near + np.float32(1e-20)) / np.float32(448.0)).astype(np.float32)
    hit = near[(sc.view(np.uint32) & 0x7FFFFF) == 0x7FFFFF]
    assert hit.size > 0
    g[128:256] *= 1e-3
    g[128] = float(hit[0])
    g[256] = float("inf")                      # fp32 gradients keep these exact values
    out = []
    for mode in (mm["lib"].DIV_IEEE, mm["lib"].DIV_IEEE_STRICT):
        codes = torch.zeros(n, dtype=torch.uint8, device="cuda")
        scales = torch.zeros(n // 128, device="cuda")
        for _ in range(2):
            mm["fp8"].fp8_momentum_flat(codes, scales, g, 0.95, div_mode=mode)
        out.append((codes, scales))
    assert torch.equal(out[0][0], out[1][0])
    assert torch.equal(out[0][1].view(torch.int32), out[1][1].view(torch.int32))


def test_reciprocal_quotient_equals_the_division_instruction_on_many_elements(mm):
    """In its default arithmetic the fused kernel forms m / s as m * rcp.approx(s) with one reciprocal per
    group; the stand-alone quantiser issues div.full.f32 per element, the instruction the reference's Triton
    kernels compile `/` to.  Both must give the same codes and scales: 2^27 elements, group scales over
    sixteen decades, zero groups, a group with an infinite element."""
    n = 1 << 27
    gen = torch.Generator(device="cuda").manual_seed(78)
    g = torch.empty(n, device="cuda").normal_(0, 1, generator=gen)
    g *= torch.pow(10.0, torch.empty(n // 128, device="cuda").uniform_(-12, 4, generator=gen)).repeat_interleave(128)
    g[:128] = 0.0
    g[256] = float("inf")
    L = mm["lib"]
    codes = torch.zeros(n, dtype=torch.uint8, device="cuda")
    scales = torch.zeros(n // 128, device="cuda")
    state = torch.zeros(n, device="cuda")
    for step in range(2):
        mm["fp8"].fp8_momentum_flat(codes, scales, g, 0.95, div_mode=L.DIV_FULL)
        state.mul_(0.95).add_(g)                     # heavy ball on the decoded state, two roundings
        want = {}
        mm["fp8"].quantize_(want, "m", state, True, codec="absmax", div_mode=L.DIV_FULL)
        assert torch.equal(scales.view(torch.int32), want["scale_m"].view(torch.int32)), step
        assert torch.equal(codes, want["m"].view(torch.uint8)), step
        state = mm["fp8"].dequantize(want, "m", True, codec="absmax")


ONCHIP_SHAPES = [(3, 128, 128), (2, 344, 128), (2, 128, 344), (300, 128, 128), (5, 96, 200), (4, 128, 384),
                 (3, 384, 128), (7, 200, 72),
                 # two row blocks: 128 < rows <= 256, rows <= cols <= 256
                 (2, 256, 256), (3, 192, 256), (5, 136, 200), (160, 256, 256), (2, 200, 200)]


@pytest.mark.parametrize("shape", ONCHIP_SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_onchip_newton_schulz_matches_the_multi_launch_path_and_the_oracle(mm, shape):
    """Blocks whose short side is at most 128 (and long side at most 384), and wide or square blocks of up to
    256 x 256, run all five iterations in one launch with X, Ah and Pp resident in shared and tensor memory.  Same operands, same roundings as the
    fifteen-launch path: the results must agree to bf16 rounding noise (the order of the K = 16 partial
    products inside an accumulator may differ) and meet the same bounds against the CPU oracle; one launch
    instead of seventeen; repeated calls and more blocks than SMs give identical bits; the fused weight
    update equals the two-kernel form bit for bit."""
    from oracle import muon_oracle
    L = mm["lib"]
    g = torch.Generator().manual_seed(sum(shape) + 3)
    x = torch.randn(shape, generator=g).bfloat16()
    xd = x.cuda()
    n0 = L.launch_count()
    got = mm["ns"].newton_schulz_batched(xd, backend=L.NS_TCGEN05)
    launches = L.launch_count() - n0
    assert L.read_status(xd.device) == 0
    assert launches == 3, launches                       # block norms, their reciprocals, the on-chip kernel
    multi = mm["ns"].newton_schulz_batched(xd, backend=L.NS_TCGEN05_MULTI)
    assert L.read_status(xd.device) == 0
    assert torch.isfinite(got).all()
    assert relf(got, multi) < 4e-3, relf(got, multi)
    if shape[0] <= 8:
        ref32 = muon_oracle.newton_schulz(x.float())
        ref16 = muon_oracle.newton_schulz(x)
        e_ref = relf(ref16, ref32)
        assert relf(got, ref32) <= max(NS_SLACK_VS_FP32 * e_ref, 1e-2)
        assert relf(got, ref16) <= max(NS_SLACK_VS_BF16_ORACLE * e_ref, 1.5e-2)
    again = mm["ns"].newton_schulz_batched(xd, backend=L.NS_TCGEN05)
    assert torch.equal(got, again)
    # fused update on scattered blocks == result stored, then the update kernel
    batch, rows, cols = shape
    for wdtype in (torch.bfloat16, torch.float32):
        w = (0.02 * torch.randn(shape, generator=g)).to(wdtype).cuda()
        want = w.clone()
        alpha = -0.02 * (rows / cols) ** 0.5
        seg = (L.UpdateSeg * 1)()
        seg[0].weight, seg[0].ortho, seg[0].numel = want.data_ptr(), got.data_ptr(), want.numel()
        L.check(L.load().mmb_muon_update(seg, 1, L.dtype_code(wdtype), alpha, L.stream_ptr()))
        ptrs = torch.tensor([w.data_ptr() + k * rows * cols * w.element_size() for k in range(batch)], dtype=torch.int64).cuda()
        mm["ns"].newton_schulz_update(xd, ptrs, wdtype, alpha, backend=L.NS_TCGEN05)
        assert L.read_status(xd.device) == 0
        assert torch.equal(w, want), wdtype


# ------------------------------------------------ transfer kernels of the sharded step, on one GPU
@pytest.mark.parametrize("world", [1, 2, 3, 4, 8, 16])
def test_peer_reduce_sums_the_copies_in_rank_order(mm, world):
    """mmb_peer_reduce_bf16 over `world` buffers (here all on one GPU; between GPUs the addresses are peer
    mappings): dst = bf16(fp32 sum of the copies in the order given), bit for bit, for sizes with and
    without a remainder for the unrolled loop."""
    L = mm["lib"]
    C = L.C
    g = torch.Generator().manual_seed(100 + world)
    for n in (8 * 1000, 8 * (128 * 148 * 8 * 2 + 37)):
        copies = [torch.randn(n, generator=g).to(torch.bfloat16).cuda() for _ in range(world)]
        want = torch.zeros(n, dtype=torch.float32, device="cuda")
        for c in copies:
            want += c.float()                                 # fp32 accumulation in rank order
        want = want.to(torch.bfloat16)
        got = torch.empty(n, dtype=torch.bfloat16, device="cuda")
        ptrs = (C.c_void_p * world)(*[c.data_ptr() for c in copies])
        L.check(L.load().mmb_peer_reduce_bf16(ptrs, world, got.data_ptr(), n * 2, 148, L.stream_ptr()), "peer_reduce")
        torch.cuda.synchronize()
        assert torch.equal(got, want)


@pytest.mark.parametrize("count", [0, 1, 3, 7])
def test_peer_broadcast_writes_every_copy(mm, count):
    L = mm["lib"]
    C = L.C
    n = 8 * (128 * 148 * 8 + 11)
    src = torch.randn(n, generator=torch.Generator().manual_seed(7)).to(torch.bfloat16).cuda()
    dsts = [torch.zeros(n, dtype=torch.bfloat16, device="cuda") for _ in range(count)]
    ptrs = (C.c_void_p * max(1, count))(*[d.data_ptr() for d in dsts])
    L.check(L.load().mmb_peer_broadcast(src.data_ptr(), ptrs, count, n * 2, 148, L.stream_ptr()), "peer_broadcast")
    torch.cuda.synchronize()
    assert all(torch.equal(d, src) for d in dsts)


def test_transfer_kernels_refuse_bad_arguments(mm):
    L = mm["lib"]
    C = L.C
    lib = L.load()
    a = torch.zeros(64, dtype=torch.bfloat16, device="cuda")
    b = torch.zeros(64, dtype=torch.bfloat16, device="cuda")
    one = (C.c_void_p * 1)(a.data_ptr())
    assert lib.mmb_peer_reduce_bf16(one, 17, b.data_ptr(), 128, 1, None) == -1          # too many copies
    assert lib.mmb_peer_reduce_bf16(one, 1, b.data_ptr(), 100, 1, None) == -1           # not a multiple of 16 bytes
    assert lib.mmb_peer_reduce_bf16(one, 1, b.data_ptr() + 2, 96, 1, None) == -1        # misaligned
    assert lib.mmb_peer_broadcast(a.data_ptr(), one, 1, 128, 1, None) == -1             # destination is the source
    assert lib.mmb_peer_broadcast(a.data_ptr(), one, 0, 128, 1, None) == 0              # nothing to do
    assert lib.mmb_multimem_reduce_bf16(None, b.data_ptr(), 128, 1, None) == -1
