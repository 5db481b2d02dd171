"""The fine-tuning optimizer (fp32 master weights, bf16 parameters) on the GPU against the oracle's
restatement of the reference's SFTOptimizer and against the vectors the reference itself produced."""
import io
import os

import numpy as np
import pytest
import torch

import golden_inputs as gi

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def relf(a, b):
    a, b = a.double().cpu(), b.double().cpu()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


def _bf16(arr):
    return torch.from_numpy(arr.view(np.int16).copy()).view(torch.bfloat16)


def _setup():
    from monarch_muon_b200.sft import SFTOptimizer
    h = gi.SFT_HYPER
    muon, adamw = gi.sft_params()
    muon = [torch.nn.Parameter(p.data.cuda()) for p in muon]
    adamw = [torch.nn.Parameter(p.data.cuda()) for p in adamw]
    opt = SFTOptimizer([{"params": muon, "algorithm": "muon", "lr": h["muon_lr"], "weight_decay": 0.0},
                        {"params": adamw, "algorithm": "adamw", "lr": h["adamw_lr"]}],
                       momentum=h["momentum"], betas=h["betas"], eps=h["eps"], weight_decay=h["weight_decay"])
    return opt, muon, adamw


def _oracle():
    from oracle import sft_oracle
    h = gi.SFT_HYPER
    muon, adamw = gi.sft_params()
    muon = [p.data for p in muon]
    adamw = [p.data for p in adamw]
    ref = sft_oracle.OracleSFT([{"params": muon, "algorithm": "muon", "lr": h["muon_lr"], "weight_decay": 0.0},
                                {"params": adamw, "algorithm": "adamw", "lr": h["adamw_lr"]}],
                               momentum=h["momentum"], betas=h["betas"], eps=h["eps"], weight_decay=h["weight_decay"])
    return ref, muon, adamw


def test_three_steps_against_oracle_and_reference_vectors():
    opt, muon, adamw = _setup()
    ref, rmuon, radamw = _oracle()
    gold = np.load(os.path.join(GOLD, "sft.npz"))
    start = [p.data.clone() for p in muon + adamw]
    for step in range(gi.SFT_STEPS):
        mg, ag = gi.sft_grads(step)
        for p, g in zip(muon + adamw, mg + ag):
            p.grad = None if g is None else g.cuda()
        opt.step()
        ref.step([mg, ag])
        for i, (p, r) in enumerate(zip(muon + adamw, rmuon + radamw)):
            st, rst = opt.state.get(p, {}), ref.state.get(id(r), {})
            if not rst:
                assert not st and torch.equal(p.data.cpu(), r), (step, i)     # skipped: untouched
                continue
            is_muon = i < len(muon)
            # momentum: same two fp32 roundings on both sides -> bit-exact; AdamW moments to fp32 noise
            if is_muon:
                assert torch.equal(st["momentum"].cpu(), rst["momentum"]), (step, i)
                assert st["step"] == rst["step"]
                # masters differ through Newton-Schulz only: compare the accumulated update
                d_ours = st["master"].cpu() - start[i].float().cpu()
                d_ref = rst["master"] - start[i].float().cpu()
                assert relf(d_ours, d_ref) < 5e-2, (step, i)      # fp32-accumulated iteration vs bf16-rounded one
                assert relf(st["master"], rst["master"]) < 1e-3
            else:
                assert relf(st["momentum"], rst["momentum"]) < 1e-6
                assert relf(st["variance"], rst["variance"]) < 1e-6
                assert relf(st["master"], rst["master"]) < 1e-6
                assert float(st["adam_step"]) == rst["adam_step"]
                # the bf16 parameter is the rounded master: equal to the reference's except where the
                # master sits within fp32 noise of a bf16 rounding boundary
                want = _bf16(gold[f"s{step}_p{i}"])
                assert (p.data.cpu() != want).float().mean() < 2e-3, (step, i)
            assert torch.equal(p.data, st["master"].bfloat16()), (step, i)     # parameter == bf16(master)
            assert st["master"].dtype == torch.float32 and st["momentum"].dtype == torch.float32


def test_adamw_matches_torch_adamw_on_the_master():
    """The reference's own check (finetune/test_sft.py:13-26): SFT AdamW == torch.optim.AdamW on an fp32
    copy, parameter compared after rounding to bf16."""
    from monarch_muon_b200.sft import SFTOptimizer
    gen = torch.Generator().manual_seed(7)
    p = torch.nn.Parameter(torch.randn(8, 12, generator=gen).bfloat16().cuda())
    reference = torch.nn.Parameter(p.detach().float().clone())
    actual = SFTOptimizer([p], lr=3e-5)
    expected = torch.optim.AdamW([reference], lr=3e-5, betas=(0.9, 0.95), weight_decay=0.1)
    for _ in range(5):
        g = torch.randn(8, 12, generator=gen).bfloat16().cuda()
        p.grad, reference.grad = g, g.float()
        actual.step()
        expected.step()
        assert relf(actual.state[p]["master"], reference.data) < 1e-6
        assert (p.data != reference.data.bfloat16()).float().mean() <= 1 / 96
    assert actual.state[p]["master"].dtype == torch.float32


def test_small_updates_accumulate_in_master():
    """finetune/test_sft.py:28-34: thirty steps too small for bf16 still move the parameter."""
    from monarch_muon_b200.sft import SFTOptimizer
    p = torch.nn.Parameter(torch.ones(4, 4, dtype=torch.bfloat16, device="cuda"))
    opt = SFTOptimizer([p], lr=1e-4, weight_decay=0)
    for _ in range(30):
        p.grad = torch.ones_like(p)
        opt.step()
    assert float(p.detach().min()) < 1.0


def test_odd_shapes_fp32_parameters_and_state_dict():
    """A matrix whose sides are not multiples of 8 (cross-check Newton-Schulz kernel, norms computed
    from the stack), an fp32 parameter (refreshed with copy_), and a state_dict round trip that keeps
    masters and moments fp32."""
    from monarch_muon_b200.sft import SFTOptimizer
    from oracle import sft_oracle
    gen = torch.Generator().manual_seed(3)
    shapes = [(10, 12), (3, 16, 24)]
    w = [(0.05 * torch.randn(s, generator=gen)) for s in shapes]
    a = 0.05 * torch.randn(40, generator=gen)
    ours_m = [torch.nn.Parameter(w[0].bfloat16().cuda()), torch.nn.Parameter(w[1].clone().cuda())]   # bf16, fp32
    ours_a = [torch.nn.Parameter(a.bfloat16().cuda())]
    ref_m = [w[0].bfloat16(), w[1].clone()]
    ref_a = [a.bfloat16()]
    mk = lambda m, aa: [{"params": m, "algorithm": "muon", "lr": 2e-3, "weight_decay": 0.0},
                        {"params": aa, "algorithm": "adamw", "lr": 1e-4}]
    opt = SFTOptimizer(mk(ours_m, ours_a))
    ref = sft_oracle.OracleSFT(mk(ref_m, ref_a))
    for step in range(2):
        gm = [(1e-2 * torch.randn(s, generator=gen)) for s in shapes]
        ga = 1e-2 * torch.randn(40, generator=gen)
        gm = [gm[0].bfloat16(), gm[1]]
        for p, g in zip(ours_m + ours_a, gm + [ga.bfloat16()]):
            p.grad = g.cuda()
        opt.step()
        ref.step([gm, [ga.bfloat16()]])
    for p, r in zip(ours_m, ref_m):
        assert relf(p.data.float(), r.float()) < 2e-3
    assert relf(ours_a[0].data.float(), ref_a[0].float()) < 1e-3
    buf = io.BytesIO()
    torch.save(opt.state_dict(), buf)
    buf.seek(0)
    opt2 = SFTOptimizer(mk([torch.nn.Parameter(p.data.clone()) for p in ours_m],
                           [torch.nn.Parameter(p.data.clone()) for p in ours_a]))
    opt2.load_state_dict(torch.load(buf, weights_only=False))
    for p, q in zip(ours_m + ours_a, [x for g in opt2.param_groups for x in g["params"]]):
        for k, v in opt.state[p].items():
            if torch.is_tensor(v):
                assert opt2.state[q][k].dtype == v.dtype and torch.equal(opt2.state[q][k], v), k
    # both continue identically
    for o, params in ((opt, ours_m + ours_a), (opt2, [x for g in opt2.param_groups for x in g["params"]])):
        gen2 = torch.Generator().manual_seed(11)
        for p in params:
            p.grad = (1e-2 * torch.randn(p.shape, generator=gen2)).to(p.dtype).cuda()
        o.step()
    for p, q in zip(ours_m + ours_a, [x for g in opt2.param_groups for x in g["params"]]):
        assert torch.equal(p.data, q.data)


def test_parameter_groups_split():
    from monarch_muon_b200.sft import parameter_groups

    class Tiny(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.embed_tokens = torch.nn.Embedding(16, 8)
            self.proj = torch.nn.Linear(8, 8)
            self.norm = torch.nn.LayerNorm(8)
            self.lm_head = torch.nn.Linear(8, 16, bias=False)

    m = Tiny()
    groups = parameter_groups(m, "muon", 1e-3, {"muon_adamw_lr": 3e-5})
    assert [g["algorithm"] for g in groups] == ["muon", "adamw"]
    assert len(groups[0]["params"]) == 1 and groups[0]["params"][0] is m.proj.weight and groups[0]["weight_decay"] == 0.0
    assert groups[1]["lr"] == 3e-5 and len(groups[1]["params"]) == 5
    only = parameter_groups(m, "adamw", 1e-3, {})
    assert len(only) == 1 and len(only[0]["params"]) == 6


def test_strided_gradients_are_read_through_a_copy_that_outlives_the_launch():
    """A gradient that is not contiguous (here: the transpose of a contiguous tensor) is stepped through a
    contiguous copy; the copy must stay alive until the kernels that read it have been launched.  Several
    such parameters in one group, so that a freed copy would be handed to the next one: the result must
    equal the step on contiguous gradients bit for bit."""
    from monarch_muon_b200.sft import SFTOptimizer
    gen = torch.Generator().manual_seed(31)
    shapes = [(128, 256), (256, 128), (128, 256), (2, 128, 256)]
    ws = [torch.randn(s, generator=gen).bfloat16() for s in shapes]
    gs = [torch.randn(s, generator=gen).bfloat16() for s in shapes]
    results = []
    for strided in (False, True):
        params = [torch.nn.Parameter(w.clone().cuda()) for w in ws]
        opt = SFTOptimizer([{"params": params, "algorithm": "muon"}], lr=1e-2)
        for step in range(2):
            for p, g in zip(params, gs):
                g = g.cuda()
                if strided:
                    g = g.transpose(-1, -2).contiguous().transpose(-1, -2)      # same values, strided layout
                    assert not g.is_contiguous()
                p.grad = g
            opt.step()
        torch.cuda.synchronize()
        results.append([p.data.clone() for p in params])
    for a, b in zip(*results):
        assert torch.equal(a, b)


def test_adamw_groups_are_bit_exact_with_the_reference_class_on_the_gpu():
    """The reference's SFTOptimizer (finetune/sft_optimizer.py:17-59, staged unmodified) run on the GPU, where its
    AdamW branch calls torch.optim's fused kernel, against this library's class: master weights, both moments
    and the bf16 parameters equal bit for bit after each of six steps, then again from a late step count (the
    bias corrections are float powers of the float betas there)."""
    from oracle import ref_loader
    if not ref_loader.available():
        pytest.skip("oracle/_ref/ not staged (python oracle/make_ref.py <reference checkout>)")
    from monarch_muon_b200.sft import SFTOptimizer
    ref = ref_loader.sft()
    gen = torch.Generator().manual_seed(5)
    shapes = [(1000, 64), (64,), (333, 77)]
    w = [(0.05 * torch.randn(s, generator=gen)).bfloat16() for s in shapes]
    a = [torch.nn.Parameter(t.clone().cuda()) for t in w]
    b = [torch.nn.Parameter(t.clone().cuda()) for t in w]
    theirs = ref.SFTOptimizer([{"params": a, "algorithm": "adamw"}], lr=3e-5)
    ours = SFTOptimizer([{"params": b, "algorithm": "adamw"}], lr=3e-5)

    def bits(t):
        return t.contiguous().view(torch.int32 if t.dtype == torch.float32 else torch.int16).reshape(-1)

    def one_step(tag):
        for pa, pb, sh in zip(a, b, shapes):
            g = (1e-2 * torch.randn(sh, generator=gen)).bfloat16()
            pa.grad, pb.grad = g.clone().cuda(), g.clone().cuda()
        theirs.step()
        ours.step()
        for pa, pb in zip(a, b):
            sa, sb = theirs.state[pa], ours.state[pb]
            for name in ("master", "momentum", "variance"):
                assert torch.equal(bits(sa[name]), bits(sb[name])), (tag, name, tuple(pa.shape))
            assert torch.equal(bits(pa.data), bits(pb.data)), (tag, tuple(pa.shape))

    for step in range(6):
        one_step(step)
    for pa, pb in zip(a, b):                                  # jump both sides to a late step
        theirs.state[pa]["adam_step"].fill_(997.0)
        ours.state[pb]["adam_step"].fill_(997.0)
    ours._adam_steps.clear()                                  # host copies of the step counts are re-read from the state
    for step in range(3):
        one_step(997 + step)
