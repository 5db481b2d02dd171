"""The full 6.89B-reference step (448 Muon tensors, 2.56e9 elements, FP8 momentum)
checked through properties that do not need an oracle at that size."""
import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


@pytest.mark.skipif(not torch.cuda.is_available() or
                    torch.cuda.get_device_properties(0).total_memory < 80e9, reason="needs ~35 GB of HBM")
def test_full_model_step_properties():
    import bench
    from monarch_muon_b200 import MonarchMuonOptimizer, _lib, fp8_state
    dev = torch.device("cuda", 0)
    muon, adamw = bench.build_workload(dev, 4)
    assert sum(p.numel() for p in muon) == 2_558_525_440
    probe = [muon[0], muon[9], muon[12]]                       # one tensor of each block shape
    assert {tuple(p.shape[1:]) for p in probe} == {(1024, 1024), (2752, 1024), (1024, 2752)}
    before = [p.data.clone() for p in probe]
    lr = 0.02
    opt = MonarchMuonOptimizer(muon, adamw, lr=lr, state_format="fp8_absmax", fp8_div="ieee")   # the CPU oracle divides IEEE
    torch.cuda.synchronize()
    held_before = torch.cuda.memory_allocated(dev)
    opt.step()
    torch.cuda.synchronize()
    assert _lib.read_status(dev) == 0
    # Memory.  Persistent optimizer state of the Muon tensors is one byte per element plus one fp32 scale per
    # 128 (the reference's bf16 momentum is two bytes per element); everything else the step allocates -
    # the bf16 stack of one slice, the Newton-Schulz workspace, the AdamW moments - stays under 7 GB.
    n_muon = sum(p.numel() for p in muon)
    muon_state = sum(v.numel() * v.element_size() for p in muon for v in opt.state[p].values() if torch.is_tensor(v))
    assert muon_state == n_muon + 4 * (n_muon // 128)
    adamw_state = sum(v.numel() * v.element_size() for p in adamw for v in opt.state[p].values() if torch.is_tensor(v))
    scratch = torch.cuda.memory_allocated(dev) - held_before - muon_state - adamw_state
    assert scratch < 5.6e9, scratch               # 1.5 GB stack + 3.9 GB workspace (256 tall blocks) + block sums
    # Probe blocks against the CPU oracle: first block of one tensor per shape.  First step from zero state:
    # m = g exactly, so the oracle needs only the gradient.
    from oracle import fp8_oracle, muon_oracle
    for p, w0 in zip(probe, before):
        g0 = p.grad[0].cpu()
        n = g0.numel()
        codes, scales, _, m16 = fp8_oracle.absmax_momentum_step(torch.zeros(n, dtype=torch.uint8),
                                                                torch.zeros(n // 128), g0.reshape(-1), 0.95)
        st = opt.state[p]
        assert torch.equal(st["momentum_buffer"][0].view(torch.uint8).cpu().reshape(-1), codes)
        o = muon_oracle.newton_schulz(m16.view(1, *g0.shape))[0]
        base = w0[0].float().cpu()
        want = (base - lr * (g0.shape[0] / g0.shape[1]) ** 0.5 * o.float()).bfloat16().float()    # stored as bf16, like ours
        got = p.data[0].float().cpu()
        # one step's increment, both sides rounded to bf16 weights: Newton-Schulz differences of 1-2 % flip the
        # rounding of a few percent of the elements by one bf16 step of |W|
        rel_step = float(((got - base) - (want - base)).norm() / (want - base).norm())
        assert rel_step < 1.2e-1, rel_step
        assert float((got - want).norm() / want.norm()) < 1e-2
    # a second step from the same gradients moves every probed block again by about the same amount
    mid = [p.data.clone() for p in probe]
    opt.step()
    torch.cuda.synchronize()
    for p, w0, w1 in zip(probe, before, mid):
        d1 = (w1.float() - w0.float()).norm()
        d2 = (p.data.float() - w1.float()).norm()
        assert 0.8 < float(d2 / d1) < 1.25
    assert _lib.read_status(dev) == 0
