"""Config 1: a 4-layer LLaMA-style model with 2-block Monarch linears, fp32,
one forward/backward per step on random tokens and three optimizer steps
(Muon lr 0.02, momentum 0.95; AdamW lr 3e-4, betas 0.9/0.95, wd 0.1), ours on
the GPU against the CPU oracle fed the same gradients."""
import copy

import pytest
import torch

pytestmark = pytest.mark.gpu


def relf(a, b):
    a, b = a.float().cpu(), b.float().cpu()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


def test_three_training_steps_of_a_monarch_llama():
    from monarch_muon_b200 import MonarchMuonOptimizer, _lib
    from oracle import muon_oracle
    from plumbing_model import TinyMonarchLlama, split_params

    model = TinyMonarchLlama()
    twin = copy.deepcopy(model)                      # the oracle's copy stays on the CPU
    model.cuda()
    muon, adamw = split_params(model)
    tmuon, tadamw = split_params(twin)
    shapes = {}
    for p in muon:
        shapes[tuple(p.shape)] = shapes.get(tuple(p.shape), 0) + 1
    assert shapes == {(2, 128, 128): 44, (2, 344, 128): 8, (2, 128, 344): 4}
    assert sum(p.numel() for p in muon) == 2_498_560 and len(adamw) == 11
    assert sum(p.numel() for p in adamw) == 25_733_888

    opt = MonarchMuonOptimizer(muon, adamw, lr=0.02, momentum=0.95, adamw_betas=(0.9, 0.95),
                               adamw_weight_decay=0.1, adamw_eps=1e-8)
    opt.param_groups[1]["lr"] = 3e-4                 # the reference has one lr default; per-group lr is set after
    tm_data, ta_data = [p.data for p in tmuon], [p.data for p in tadamw]
    ref = muon_oracle.OracleMonarchMuon(tm_data, ta_data, lr=0.02, momentum=0.95,
                                        adamw_betas=(0.9, 0.95), adamw_weight_decay=0.1, adamw_eps=1e-8,
                                        ns_dtype=torch.bfloat16)
    ref.lr["adamw"] = 3e-4
    # second oracle: the pretraining twin's fp32 Newton-Schulz, the yardstick for the tolerance
    twin32 = copy.deepcopy(twin)
    t32m, t32a = split_params(twin32)
    t32_data = [p.data for p in t32m]
    ref32 = muon_oracle.OracleMonarchMuon(t32_data, [p.data for p in t32a], lr=0.02, momentum=0.95,
                                          adamw_betas=(0.9, 0.95), adamw_weight_decay=0.1, adamw_eps=1e-8)
    ref32.lr["adamw"] = 3e-4
    gen = torch.Generator().manual_seed(17)
    losses = []
    for step in range(3):
        tokens = torch.randint(0, 50257, (4, 129), generator=gen)
        x, y = tokens[:, :-1].cuda(), tokens[:, 1:].cuda()
        loss = model(x, y)
        loss.backward()
        losses.append(loss.item())
        grads_m = [p.grad.detach().cpu().clone() for p in muon]
        grads_a = [p.grad.detach().cpu().clone() for p in adamw]
        before = [p.data.clone().cpu() for p in muon]
        before16 = [r.clone() for r in tm_data]
        before32 = [r.clone() for r in t32_data]
        opt.step()
        opt.zero_grad(set_to_none=True)
        ref.step(grads_m, grads_a)
        ref32.step(grads_m, [g.clone() for g in grads_a])
        # The momentum is identical in all three, so each step's increment is -lr*scale*NS(m) of the same m.
        # Real gradients are ill-conditioned, which makes bf16 Newton-Schulz deviate more than on Gaussian
        # blocks; the bar is relative to the reference's own bf16-vs-fp32 gap e_ref, per tensor:
        # ours-vs-fp32 <= 1.15 e_ref and ours-vs-bf16 <= 1.5 e_ref.
        worst = 0.0
        for p, b, r16, b16, r32, b32 in zip(muon, before, tm_data, before16, t32_data, before32):
            d_ours, d16, d32 = p.data.cpu() - b, r16 - b16, r32 - b32
            e_ref = relf(d16, d32)
            assert relf(d_ours, d32) <= max(1.15 * e_ref, 1.5e-2), (relf(d_ours, d32), e_ref)
            assert relf(d_ours, d16) <= max(1.5 * e_ref, 1.5e-2), (relf(d_ours, d16), e_ref)
            worst = max(worst, e_ref)
            assert relf(p.data, r16) < 2e-2
        print(f"step {step}: loss {losses[-1]:.4f}, worst reference bf16-vs-fp32 increment gap {worst:.3e}")
        for p, r in zip(adamw, ta_data):
            assert relf(p.data, r) < 1e-5
    assert _lib.read_status(torch.device("cuda", 0)) == 0
    assert abs(losses[0] - 10.89) < 0.15             # ln(50257) = 10.82 for an untrained model
    assert all(torch.isfinite(p.data).all() for p in muon + adamw)
    # fp32 parameters keep fp32 momentum, exactly the oracle's (same two roundings)
    for p, r in zip(muon, tm_data):
        assert opt.state[p]["momentum_buffer"].dtype == torch.float32
        assert torch.equal(opt.state[p]["momentum_buffer"].cpu(), ref.state[id(r)]["momentum_buffer"])


def test_arms_learn_and_fp8_states_track_the_plain_arm():
    """Mirror of the reference's integration test (pretrain/tests/test_coat_state_muon.py:53-99): 15 steps on
    one fixed random batch; every arm's loss must be finite and fall by at least 0.3, the FP8-state arms
    must end within 3 % of the plain arm, their states must be E4M3, and a state_dict round trip must
    reproduce them bit for bit."""
    import io
    from monarch_muon_b200 import CoatStateMonarchMuon, MonarchMuonOptimizer
    from plumbing_model import TinyMonarchLlama, split_params

    class Q:  # optimizer fields of the reference's QuantizationConfig
        qgroup_size = 128
        first_order_expansion = second_order_expansion = "true"
        first_order_bit = second_order_bit = "E4M3"
        expand_min = 16

    tokens = torch.randint(0, 50257, (4, 129), generator=torch.Generator().manual_seed(3)).cuda()
    x, y = tokens[:, :-1], tokens[:, 1:]

    def build(arm):
        model = TinyMonarchLlama(seed=1).cuda()
        muon, adamw = split_params(model)
        kw = dict(lr=5e-3, momentum=0.95, adamw_betas=(0.9, 0.95), adamw_weight_decay=0.1, adamw_eps=1e-8)
        if arm == "plain":
            opt = MonarchMuonOptimizer(muon, adamw, **kw)
        elif arm == "fp8_expand":
            opt = CoatStateMonarchMuon(muon, adamw, qargs=Q(), **kw)
        else:
            opt = CoatStateMonarchMuon(muon, adamw, codec="absmax", **kw)
        return model, opt

    final = {}
    for arm in ("plain", "fp8_expand", "fp8_absmax"):
        model, opt = build(arm)
        losses = []
        for _ in range(15):
            loss = model(x, y)
            loss.backward()
            losses.append(loss.item())
            opt.step()
            opt.zero_grad(set_to_none=True)
        assert all(map(lambda v: v == v and abs(v) < 1e9, losses)), losses
        assert losses[-1] < losses[0] - 0.3, (arm, losses)
        # this small model memorises the batch within 15 steps (loss -> 0.02), so the arms are compared on
        # the whole loss curve rather than on the noisy tail
        final[arm] = sum(losses) / len(losses)
        if arm != "plain":
            assert abs(final[arm] - final["plain"]) / final["plain"] < 0.03, (arm, final)
            states = list(opt.state.values())
            assert all(s["momentum_buffer"].dtype == torch.float8_e4m3fn for s in states if "momentum_buffer" in s)
            assert all(s["exp_avg"].dtype == torch.float8_e4m3fn and s["exp_avg_sq"].dtype == torch.float8_e4m3fn
                       for s in states if "exp_avg" in s)
            assert any("momentum_buffer" in s for s in states) and any("exp_avg" in s for s in states)
            buf = io.BytesIO()
            torch.save(opt.state_dict(), buf)
            buf.seek(0)
            saved = opt.state_dict()
            _, restored = build(arm)
            restored.load_state_dict(torch.load(buf, weights_only=False))
            back = restored.state_dict()
            for key, entry in back["state"].items():
                for name, value in entry.items():
                    if torch.is_tensor(value):
                        ref_v = saved["state"][key][name]
                        assert value.dtype == ref_v.dtype, name
                        a = value.view(torch.uint8) if value.dtype == torch.float8_e4m3fn else value
                        b = ref_v.view(torch.uint8) if ref_v.dtype == torch.float8_e4m3fn else ref_v
                        assert torch.equal(a, b), name
        del model, opt
        torch.cuda.empty_cache()
