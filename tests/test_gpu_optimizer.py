"""The optimizer step through the public API on a GPU, against the CPU oracle."""
import copy
import io

import numpy as np
import pytest
import torch

import golden_inputs as gi

pytestmark = pytest.mark.gpu


def relf(a, b):
    a = a.float().cpu()
    b = b.float().cpu()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


def _oracle(case, ns_bf16=True):
    from oracle import muon_oracle
    dtype, _, _, hyper = gi.OPT_CASES[case]
    muon, adamw = gi.opt_params(case)
    muon = [p.data for p in muon]
    adamw = [p.data for p in adamw]
    opt = muon_oracle.OracleMonarchMuon(muon, adamw, lr=hyper["lr"], momentum=hyper["momentum"],
                                        adamw_betas=hyper["betas"], adamw_weight_decay=hyper["weight_decay"],
                                        adamw_eps=hyper["eps"], ns_dtype=torch.bfloat16 if ns_bf16 else None)
    opt.lr["adamw"] = hyper["adamw_lr"]
    return opt, muon, adamw


def _ours(case, **kw):
    from monarch_muon_b200 import MonarchMuonOptimizer
    dtype, _, _, hyper = gi.OPT_CASES[case]
    muon, adamw = gi.opt_params(case)
    muon = [torch.nn.Parameter(p.data.cuda()) for p in muon]
    adamw = [torch.nn.Parameter(p.data.cuda()) for p in adamw]
    cls = kw.pop("cls", MonarchMuonOptimizer)
    opt = cls(muon, adamw, lr=hyper["lr"], momentum=hyper["momentum"], adamw_betas=hyper["betas"],
              adamw_weight_decay=hyper["weight_decay"], adamw_eps=hyper["eps"], **kw)
    opt.param_groups[1]["lr"] = hyper["adamw_lr"]
    return opt, muon, adamw


def _feed(muon, adamw, mg, ag):
    for p, g in zip(muon, mg):
        p.grad = None if g is None else g.cuda()
    for p, g in zip(adamw, ag):
        p.grad = None if g is None else g.cuda()


# Tolerances (relative Frobenius norm):
#  - weight *increments* after each step vs the bf16-Newton-Schulz oracle: the
#    Newton-Schulz tolerance (5e-2) for fp32 weights; bf16 weights add their own
#    storage rounding (one bf16 ulp of |W| ~ 2e-2 is ~7% of one step's increment).
#  - weights themselves: 1e-2 (the test blocks are only 64-128 wide, so three
#    steps of lr 0.02 move the weights by a third of their norm; 5e-2 of that).
TOL_DELTA = {"fp32": 5e-2, "bf16": 1.2e-1}
TOL_W = 1e-2


@pytest.mark.parametrize("case", ["fp32", "bf16"])
def test_three_steps_match_oracle(case):
    from monarch_muon_b200 import _lib
    ref, rmuon, radamw = _oracle(case)
    w0 = [p.clone() for p in rmuon]
    opt, muon, adamw = _ours(case)
    for step in range(gi.OPT_STEPS):
        mg, ag = gi.opt_grads(case, step)
        ref.step(mg, ag)
        _feed(muon, adamw, mg, ag)
        opt.step()
        opt.zero_grad(set_to_none=True)
        if step == 0:
            assert len(opt.state[muon[-1]]) == 0           # no gradient yet -> no state yet
        for i, (p, r) in enumerate(zip(muon, rmuon)):
            assert relf(p.data, r) < TOL_W, (step, i)
            if mg[i] is not None or step > 0:
                assert relf(p.data.float().cpu() - w0[i].float(), r.float() - w0[i].float()) < TOL_DELTA[case], (step, i)
    assert _lib.read_status(muon[0].device) == 0
    # momentum: same two roundings in the same type -> identical bits
    for p, r in zip(muon, rmuon):
        assert torch.equal(opt.state[p]["momentum_buffer"].cpu(), ref.state[id(r)]["momentum_buffer"])
    # AdamW: same op order; fused-multiply-add vs separate multiply/add can move the last bit
    for p, r in zip(adamw, radamw):
        st, rst = opt.state[p], ref.state[id(r)]
        assert st["step"] == rst["step"] == gi.OPT_STEPS
        tol = 1e-6 if case == "fp32" else 4e-3
        assert relf(p.data, r) < tol
        assert relf(st["exp_avg"], rst["exp_avg"]) < tol
        assert relf(st["exp_avg_sq"], rst["exp_avg_sq"]) < tol


def test_fp32_weights_close_to_fp32_newton_schulz_oracle():
    """Against the pretrain twin's fp32 Newton-Schulz the bf16 tensor-core path
    must be no further than the reference's own bf16 path is."""
    ref32, r32, _ = _oracle("fp32", ns_bf16=False)
    ref16, r16, _ = _oracle("fp32", ns_bf16=True)
    w0 = [p.clone() for p in r32]
    opt, muon, adamw = _ours("fp32")
    mg, ag = gi.opt_grads("fp32", 1)
    ref32.step(mg, ag)
    ref16.step(mg, ag)
    _feed(muon, adamw, mg, ag)
    opt.step()
    for p, a, b, w in zip(muon, r32, r16, w0):
        e_ref = relf(b - w, a - w)
        e_got = relf(p.data.cpu() - w, a - w)
        assert e_got <= max(1.15 * e_ref, 1e-2), (e_got, e_ref)


@pytest.mark.parametrize("case", ["fp32", "bf16"])
def test_fp8_absmax_state_is_bit_exact(case):
    from oracle import fp8_oracle, muon_oracle
    from monarch_muon_b200 import CoatStateMonarchMuon
    opt, muon, adamw = _ours(case, cls=CoatStateMonarchMuon, codec="absmax", fp8_div="ieee")     # the CPU oracle divides IEEE
    _, _, _, hyper = gi.OPT_CASES[case]
    # oracle chain per tensor: codes/scales start at zero (state created as zeros)
    chain = [None] * len(muon)
    w_ref = [p.data.clone().cpu() for p in muon]
    for step in range(gi.OPT_STEPS):
        mg, ag = gi.opt_grads(case, step)
        _feed(muon, adamw, mg, ag)
        opt.step()
        opt.zero_grad(set_to_none=True)
        for i, g in enumerate(mg):
            if g is None:
                continue
            n = g.numel()
            if chain[i] is None:
                chain[i] = (torch.zeros(n, dtype=torch.uint8), torch.zeros(-(-n // 128)))
            codes, scales, m32, m16 = fp8_oracle.absmax_momentum_step(chain[i][0], chain[i][1], g, hyper["momentum"])
            chain[i] = (codes, scales)
            st = opt.state[muon[i]]
            assert st["momentum_buffer"].dtype == torch.float8_e4m3fn
            assert st["momentum_buffer"].shape == muon[i].shape
            assert torch.equal(st["momentum_buffer"].view(torch.uint8).cpu().reshape(-1), codes), (step, i)
            assert np.array_equal(st["scale_momentum_buffer"].cpu().numpy().view(np.uint32),
                                  scales.numpy().view(np.uint32)), (step, i)
            # weights: oracle Newton-Schulz on the same bf16 momentum
            o = muon_oracle.newton_schulz(m16.view(g.shape))
            scale = (g.shape[1] / g.shape[2]) ** 0.5
            w_ref[i] = (w_ref[i].float() - hyper["lr"] * scale * o.float()).to(w_ref[i].dtype)
            assert relf(muon[i].data, w_ref[i]) < TOL_W
    for p in adamw:                                   # AdamW moments are stored as E4M3 too
        st = opt.state[p]
        assert st["exp_avg"].dtype == torch.float8_e4m3fn and st["exp_avg_sq"].dtype == torch.float8_e4m3fn
        assert st["scale_exp_avg"].dtype == torch.float32


def test_fp8_expand_state_tracks_fp32_state():
    from monarch_muon_b200 import CoatStateMonarchMuon

    class Q:  # the optimizer fields of the reference's QuantizationConfig
        qgroup_size = 128
        first_order_expansion = second_order_expansion = "true"
        first_order_bit = second_order_bit = "E4M3"
        expand_min = 16

    opt8, m8, a8 = _ours("fp32", cls=CoatStateMonarchMuon, qargs=Q())
    opt, m, a = _ours("fp32")
    w0 = [p.data.clone() for p in m]
    for step in range(gi.OPT_STEPS):
        mg, ag = gi.opt_grads("fp32", step)
        _feed(m8, a8, mg, ag)
        _feed(m, a, mg, ag)
        opt8.step()
        opt.step()
    for p8, p, w in zip(m8, m, w0):
        st = opt8.state[p8]
        assert st["momentum_buffer"].dtype == torch.float8_e4m3fn
        for key in ("scale", "expand", "sqrt_minmax"):
            assert st[f"{key}_momentum_buffer"].dtype == torch.float32
        # FP8 momentum is a perturbation of a few percent; the orthogonalised update stays close
        assert relf(p8.data - w, p.data - w) < 0.25
    for p8, p in zip(a8, a):
        assert relf(p8.data, p.data) < 1e-3


@pytest.mark.parametrize("fmt", ["param", "fp8_absmax", "fp8_expand"])
def test_state_dict_round_trip(fmt):
    from monarch_muon_b200 import MonarchMuonOptimizer
    opt, muon, adamw = _ours("bf16", state_format=fmt)
    for step in range(2):
        _feed(muon, adamw, *gi.opt_grads("bf16", step + 1))
        opt.step()
    buf = io.BytesIO()
    torch.save(opt.state_dict(), buf)
    buf.seek(0)
    opt2, muon2, adamw2 = _ours("bf16", state_format=fmt)
    for a, b in zip(muon + adamw, muon2 + adamw2):
        b.data.copy_(a.data)
    opt2.load_state_dict(torch.load(buf, weights_only=False))
    sd1, sd2 = opt.state_dict(), opt2.state_dict()
    for key, entry in sd1["state"].items():
        for name, v in entry.items():
            w = sd2["state"][key][name]
            if torch.is_tensor(v):
                assert v.dtype == w.dtype, name
                assert torch.equal(v.view(torch.uint8) if v.dtype == torch.float8_e4m3fn else v,
                                   w.view(torch.uint8) if w.dtype == torch.float8_e4m3fn else w), name
            else:
                assert v == w
    g = gi.opt_grads("bf16", 2)
    _feed(muon, adamw, *g)
    _feed(muon2, adamw2, *g)
    opt.step()
    opt2.step()
    for a, b in zip(muon + adamw, muon2 + adamw2):
        assert torch.equal(a.data, b.data)


def test_optimizer_protocol_hooks_scheduler_and_errors():
    from monarch_muon_b200 import MonarchMuonOptimizer
    opt, muon, adamw = _ours("bf16")
    assert [g["update_type"] for g in opt.param_groups] == ["muon", "adamw"]
    assert "momentum" in opt.param_groups[0] and "betas" in opt.param_groups[1]
    calls = []
    opt.register_step_post_hook(lambda o, a, k: calls.append(1))
    sched = torch.optim.lr_scheduler.LambdaLR(opt, lambda it: 0.5 ** it)
    _feed(muon, adamw, *gi.opt_grads("bf16", 1))
    before = [p.data.clone() for p in muon]
    loss = opt.step(lambda: torch.tensor(3.0))
    assert float(loss) == 3.0 and calls == [1]
    sched.step()
    assert opt.param_groups[0]["lr"] == pytest.approx(0.01)
    d1 = [(p.data - b).float().norm() for p, b in zip(muon, before)]
    before = [p.data.clone() for p in muon]
    opt.step()                                           # same grads, half the lr, momentum grown
    d2 = [(p.data - b).float().norm() for p, b in zip(muon, before)]
    for a, b in zip(d1, d2):
        assert 0.35 < float(b / a) < 0.65                # orthogonalised update scales with lr only
    repr(opt)
    cpu = [torch.nn.Parameter(torch.zeros(2, 8, 8))]
    cpu[0].grad = torch.zeros(2, 8, 8)
    with pytest.raises(RuntimeError):
        MonarchMuonOptimizer(cpu, []).step()
    with pytest.raises(ValueError):
        bad = torch.nn.Parameter(torch.zeros(2, 2, 8, 8, device="cuda"))
        bad.grad = torch.zeros_like(bad)
        MonarchMuonOptimizer([bad], []).step()


def test_many_tensors_span_several_launch_tables():
    """More tensors than one kernel-parameter table holds (96 momentum / 128 update segments)."""
    from monarch_muon_b200 import MonarchMuonOptimizer
    from oracle import muon_oracle
    gen = torch.Generator().manual_seed(11)
    shapes = [(1, 64, 64)] * 150 + [(2, 64, 128)] * 60
    ws = [(0.02 * torch.randn(s, generator=gen)).bfloat16() for s in shapes]
    gs = [(1e-3 * torch.randn(s, generator=gen)).bfloat16() for s in shapes]
    aw = [(0.02 * torch.randn(33, generator=gen)).bfloat16() for _ in range(140)]
    ag = [(1e-3 * torch.randn(33, generator=gen)).bfloat16() for _ in range(140)]
    ref = muon_oracle.OracleMonarchMuon([w.clone() for w in ws], [w.clone() for w in aw], lr=0.02,
                                        ns_dtype=torch.bfloat16)
    ref.step(gs, ag)
    muon = [torch.nn.Parameter(w.cuda()) for w in ws]
    adamw = [torch.nn.Parameter(w.cuda()) for w in aw]
    opt = MonarchMuonOptimizer(muon, adamw, lr=0.02)
    _feed(muon, adamw, gs, ag)
    opt.step()
    for p, r in zip(muon, ref.muon):
        assert relf(p.data, r) < TOL_W
        assert torch.equal(opt.state[p]["momentum_buffer"].cpu(), ref.state[id(r)]["momentum_buffer"])
    for p, r in zip(adamw, ref.adamw):
        assert relf(p.data, r) < 4e-3


def test_step_fed_from_host_memory_equals_step_on_device_gradients():
    opt_a, muon_a, adamw_a = _ours("bf16", state_format="fp8_absmax", ns_max_batch=2)
    opt_b, muon_b, adamw_b = _ours("bf16", state_format="fp8_absmax", ns_max_batch=2)
    for step in range(gi.OPT_STEPS):
        mg, ag = gi.opt_grads("bf16", step)
        _feed(muon_a, adamw_a, mg, ag)
        opt_a.step()
        host = [None if g is None else g.pin_memory() for g in mg + ag]
        opt_b.step(host_grads=host)
        opt_a.zero_grad(set_to_none=True)
    torch.cuda.synchronize()
    for a, b in zip(muon_a + adamw_a, muon_b + adamw_b):
        assert torch.equal(a.data, b.data)
    for a, b in zip(muon_a, muon_b):
        assert torch.equal(opt_a.state[a]["momentum_buffer"].view(torch.uint8),
                           opt_b.state[b]["momentum_buffer"].view(torch.uint8))


def test_dense_2d_matrices_take_the_muon_update_as_single_blocks():
    """The reference's fine-tuning optimizer applies the same Newton-Schulz update to plain 2-D weight
    matrices (finetune/sft_optimizer.py:40-50); here a 2-D Muon parameter is one block."""
    from monarch_muon_b200 import MonarchMuonOptimizer
    from oracle import muon_oracle
    gen = torch.Generator().manual_seed(21)
    w2 = (0.02 * torch.randn(256, 384, generator=gen)).bfloat16()
    w3 = (0.02 * torch.randn(2, 256, 384, generator=gen)).bfloat16()
    g2 = (1e-3 * torch.randn(256, 384, generator=gen)).bfloat16()
    g3 = (1e-3 * torch.randn(2, 256, 384, generator=gen)).bfloat16()
    p2, p3 = torch.nn.Parameter(w2.cuda()), torch.nn.Parameter(w3.cuda())
    opt = MonarchMuonOptimizer([p2, p3], [], lr=0.02)
    p2.grad, p3.grad = g2.cuda(), g3.cuda()
    opt.step()
    assert opt.state[p2]["momentum_buffer"].shape == p2.shape
    o2 = muon_oracle.newton_schulz(g2[None])[0]
    want = w2.float() - 0.02 * (256 / 384) ** 0.5 * o2.float()
    assert relf(p2.data, want) < TOL_W
    o3 = muon_oracle.newton_schulz(g3)
    assert relf(p3.data, w3.float() - 0.02 * (256 / 384) ** 0.5 * o3.float()) < TOL_W


@pytest.mark.parametrize("case", ["fp32", "bf16"])
def test_fused_gradient_clipping_matches_clip_then_step(case):
    """clip_grad_norm_ + step() must equal torch.nn.utils.clip_grad_norm_ followed by the oracle's step."""
    from oracle import muon_oracle
    ref, rmuon, radamw = _oracle(case)
    opt, muon, adamw = _ours(case)
    max_norm = 0.05                                   # the seeded gradients have a global norm of about 0.3
    for step in range(2):
        mg, ag = gi.opt_grads(case, step + 1)
        _feed(muon, adamw, mg, ag)
        cpu_params = [torch.nn.Parameter(t.clone()) for t in mg + ag]
        for q, g in zip(cpu_params, mg + ag):
            q.grad = g.clone()
        want_norm = torch.nn.utils.clip_grad_norm_(cpu_params, max_norm)
        clipped = [q.grad for q in cpu_params]
        ref.step(clipped[:len(mg)], clipped[len(mg):])
        got_norm = opt.clip_grad_norm_(max_norm)
        opt.step()
        assert float(got_norm) == pytest.approx(float(want_norm), rel=4e-3 if case == "bf16" else 1e-5)
        assert float(want_norm) > max_norm            # the clip is active
    # with bf16 gradients torch keeps the total norm and the coefficient in bf16 (up to 0.4 % off the
    # fp32 value used here), which carries straight into the momentum
    tol = 1e-6 if case == "fp32" else 1e-2
    for p, r in zip(muon, rmuon):
        assert relf(p.data, r) < TOL_W
        assert relf(opt.state[p]["momentum_buffer"], ref.state[id(r)]["momentum_buffer"]) < tol
    for p, r in zip(adamw, radamw):
        assert relf(p.data, r) < tol
    # without a new clip_grad_norm_ call the next step is unscaled again
    mg, ag = gi.opt_grads(case, 2)
    _feed(muon, adamw, mg, ag)
    before = [opt.state[p]["momentum_buffer"].float().clone() for p in muon]
    opt.step()
    for p, b, g in zip(muon, before, mg):
        want = (b.cpu() * 0.95).to(p.dtype).float() + g.float() if case == "bf16" else b.cpu() * 0.95 + g.float()
        assert relf(opt.state[p]["momentum_buffer"], want.to(p.dtype)) < 1e-6


def test_edge_cases_zero_nan_and_empty_groups():
    from monarch_muon_b200 import MonarchMuonOptimizer, _lib, newton_schulz_batched
    from oracle import muon_oracle
    # Newton-Schulz: an all-zero block stays zero (0 / (0 + 1e-7)), a block with a NaN/Inf poisons only itself
    x = torch.randn(4, 256, 384, generator=torch.Generator().manual_seed(8)).bfloat16()
    x[1].zero_()
    x[2, 5, 7] = float("nan")
    x[3, 0, 0] = float("inf")
    out = newton_schulz_batched(x.cuda()).cpu()
    ref = muon_oracle.newton_schulz(x)
    assert relf(out[0], ref[0]) < 5e-2
    assert torch.all(out[1] == 0) and torch.all(ref[1] == 0)
    assert torch.isnan(out[2]).all() and torch.isnan(ref[2]).all()
    assert not torch.isfinite(out[3]).any()
    assert _lib.read_status(torch.device("cuda", 0)) == 0           # non-finite data is not a device error
    # the optimizer accepts an empty Muon group, an empty AdamW group, and a step with no gradients at all
    w = torch.nn.Parameter(torch.ones(2, 64, 64, device="cuda"))
    v = torch.nn.Parameter(torch.ones(10, device="cuda"))
    only_adamw = MonarchMuonOptimizer([], [v], lr=1e-2)
    v.grad = torch.ones_like(v)
    only_adamw.step()
    assert float(v.data[0]) < 1.0
    only_muon = MonarchMuonOptimizer([w], [], lr=1e-2)
    only_muon.step()                                                # no gradient anywhere: nothing happens
    assert torch.all(w.data == 1.0) and len(only_muon.state) == 0
    w.grad = torch.zeros_like(w)                                    # zero gradient: zero momentum, zero update
    only_muon.step()
    assert torch.all(w.data == 1.0) and torch.all(only_muon.state[w]["momentum_buffer"] == 0)
    # FP8 state with an Inf gradient: the group saturates/poisons without faulting, the rest is unaffected
    p = torch.nn.Parameter(torch.zeros(1, 128, 128, device="cuda", dtype=torch.bfloat16))
    opt = MonarchMuonOptimizer([p], [], lr=1e-2, state_format="fp8_absmax")
    g = torch.full((1, 128, 128), 1e-3, dtype=torch.bfloat16)
    g[0, 3, 0] = float("inf")
    p.grad = g.cuda()
    opt.step()
    torch.cuda.synchronize()
    codes = opt.state[p]["momentum_buffer"].view(torch.uint8).cpu().reshape(-1, 128)
    assert torch.all(codes[0] == codes[0, 0]) and int(codes[0, 0]) != 0x7F      # untouched group: all equal finite codes
    assert _lib.read_status(torch.device("cuda", 0)) == 0


@pytest.mark.parametrize("codec", ["expand", "absmax"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_fused_fp8_adamw_against_oracle(codec, dtype):
    """CoatStateMonarchMuon's AdamW group: both moments stay E4M3 between steps and one kernel decodes,
    steps and re-encodes them.  Against the oracle's dequantise -> AdamW with fp32 moments -> quantise
    (the reference's sequence), three steps, a tensor with a ragged tail and a short vector."""
    from monarch_muon_b200 import CoatStateMonarchMuon
    from oracle import fp8_oracle
    gen = torch.Generator().manual_seed(41)
    shapes = [(300, 77), (64,), (128 * 40,)]
    w = [(0.05 * torch.randn(s, generator=gen)).to(dtype) for s in shapes]
    ours = [torch.nn.Parameter(t.clone().cuda()) for t in w]
    ref = [t.clone() for t in w]
    hyper = dict(lr=3e-3, betas=(0.9, 0.95), weight_decay=0.1, eps=1e-8)
    opt = CoatStateMonarchMuon([], ours, lr=hyper["lr"], adamw_betas=hyper["betas"],
                               adamw_weight_decay=hyper["weight_decay"], adamw_eps=hyper["eps"], codec=codec, fp8_div="ieee")
    nside = 3 if codec == "expand" else 1
    zero_state = lambda n: (torch.zeros(n, dtype=torch.uint8),) + tuple(torch.ones(-(-n // 128)) for _ in range(nside))
    states = [(zero_state(t.numel()), zero_state(t.numel())) for t in w]
    for step in range(1, 4):
        grads = [(1e-2 * torch.randn(s, generator=gen) * torch.logspace(-2, 0, int(torch.Size(s).numel())).view(s)).to(dtype)
                 for s in shapes]
        for p, g in zip(ours, grads):
            p.grad = g.cuda()
        opt.step()
        for i, (p, r, g) in enumerate(zip(ours, ref, grads)):
            ms, vs, m32, v32 = fp8_oracle.adamw_fp8_step(r, g, states[i][0], states[i][1], step, codec=codec, **hyper)
            st = opt.state[p]
            assert st["exp_avg"].dtype == torch.float8_e4m3fn and st["exp_avg_sq"].dtype == torch.float8_e4m3fn
            assert st["step"] == step
            assert relf(p.data.float(), r.float()) < (1e-6 if dtype == torch.float32 else 4e-3), (step, i)
            for name, want, signed in (("exp_avg", ms, True), ("exp_avg_sq", vs, False)):
                codes = st[name].view(torch.uint8).cpu().view(-1)
                if codec == "absmax" and step == 1:
                    # from exact zeros both sides do the same fp32 arithmetic: scales to the last bit or two
                    # (FMA vs separate multiply-add), codes equal except on rounding boundaries
                    assert torch.allclose(st[f"scale_{name}"].cpu(), want[1], rtol=1e-6)
                assert (codes != want[0]).float().mean() < 2e-2, (step, i, name)
                back = fp8_oracle.expand_dequant(codes, *[st[f"{k}_{name}"].cpu() for k in ("scale", "expand", "sqrt_minmax")],
                                                 signed=signed) if codec == "expand" else \
                    fp8_oracle.absmax_dequant(codes, st[f"scale_{name}"].cpu())
                exact = m32 if name == "exp_avg" else v32
                assert relf(back, exact.view(-1)) < 0.08, (step, i, name)          # FP8 resolution
            # carry OUR state into the oracle's next step so that single-step arithmetic is compared,
            # not the drift of two FP8 trajectories
            pick = lambda name: (st[name].view(torch.uint8).cpu().view(-1),) + tuple(
                st[f"{k}_{name}"].cpu() for k in (("scale", "expand", "sqrt_minmax") if codec == "expand" else ("scale",)))
            states[i] = (pick("exp_avg"), pick("exp_avg_sq"))
            r.copy_(p.data.cpu())


@pytest.mark.parametrize("fmt", ["fp8_absmax", "param"])
def test_two_stream_overlap_gives_the_same_bits(fmt):
    """overlap=True issues the same kernels on the same data from two streams (momentum of the next slice,
    update of the previous one and AdamW beside Newton-Schulz, tiles drawn dynamically): weights and state
    after three steps are bit-identical to the one-stream step, also with gradient clipping fused."""
    from monarch_muon_b200 import MonarchMuonOptimizer
    a, am, aa = _ours("bf16", state_format=fmt, ns_max_batch=2, overlap=True)     # several slices per shape
    b, bm, ba = _ours("bf16", state_format=fmt, ns_max_batch=2)
    for step in range(gi.OPT_STEPS):
        mg, ag = gi.opt_grads("bf16", step)
        _feed(am, aa, mg, ag)
        _feed(bm, ba, mg, ag)
        if step == 1:
            a.clip_grad_norm_(0.05)
            b.clip_grad_norm_(0.05)
        a.step()
        b.step()
    torch.cuda.synchronize()
    for p, q in zip(am + aa, bm + ba):
        assert torch.equal(p.data, q.data)
        for k, v in a.state[p].items():
            if torch.is_tensor(v):
                assert torch.equal(v.view(torch.uint8) if v.dtype == torch.float8_e4m3fn else v,
                                   b.state[q][k].view(torch.uint8) if v.dtype == torch.float8_e4m3fn else b.state[q][k]), k


@pytest.mark.parametrize("case", ["bf16", "fp32"])
@pytest.mark.parametrize("fmt", ["fp8_absmax", "param"])
def test_fused_update_gives_the_same_bits_as_the_update_kernel(fmt, case):
    """The weight update applied in the epilogue of the last Newton-Schulz GEMM (default) against Newton-Schulz
    to memory followed by the update kernel: identical weights and state after three steps, bf16 and fp32
    parameters, slices cut into several Newton-Schulz sub-slices."""
    a, am, aa = _ours(case, state_format=fmt, ns_max_batch=2)
    b, bm, ba = _ours(case, state_format=fmt, ns_max_batch=2, fuse_update=False)
    for step in range(gi.OPT_STEPS):
        mg, ag = gi.opt_grads(case, step)
        _feed(am, aa, mg, ag)
        _feed(bm, ba, mg, ag)
        a.step()
        b.step()
    torch.cuda.synchronize()
    for p, q in zip(am + aa, bm + ba):
        assert torch.equal(p.data, q.data)
        for k, v in a.state[p].items():
            if torch.is_tensor(v):
                w = b.state[q][k]
                assert torch.equal(v.view(torch.uint8) if v.dtype == torch.float8_e4m3fn else v,
                                   w.view(torch.uint8) if w.dtype == torch.float8_e4m3fn else w), k
