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
    opt = MonarchMuonOptimizer(muon, adamw, lr=lr, state_format="fp8_absmax")
    opt.step()
    torch.cuda.synchronize()
    assert _lib.read_status(dev) == 0
    for p, w0 in zip(probe, before):
        nb, r, c = p.shape
        delta = (p.data.float() - w0.float()) / (-lr * (r / c) ** 0.5)      # = Newton-Schulz output (+ bf16 weight rounding)
        assert torch.isfinite(delta).all()
        # the quintic maps every singular value of a full-rank block into about [0.68, 1.13]
        # (bf16 storage of the weights adds some noise), so ||O||_F^2 / min(r, c) is about 1
        energy = delta.pow(2).sum(dim=(1, 2)) / min(r, c)
        assert float(energy.min()) > 0.45 and float(energy.max()) < 1.4, energy
        # and the output is near-orthogonal: O O^T (or O^T O) close to a multiple of the identity
        o = delta[0] if r <= c else delta[0].t()
        gram = o @ o.t()
        off = gram - torch.diag(torch.diag(gram))
        assert float(off.norm() / gram.norm()) < 0.35
        # FP8 state decodes to the gradient (first step: m = g) within E4M3's relative step of 2^-4
        st = opt.state[p]
        m = fp8_state.dequantize(st, "momentum_buffer", True, codec="absmax")
        g = p.grad.float()
        assert float((m - g).norm() / g.norm()) < 0.04
    # a second step from the same gradients moves every probed block again by about the same amount
    mid = [p.data.clone() for p in probe]
    opt.step()
    torch.cuda.synchronize()
    for p, w0, w1 in zip(probe, before, mid):
        d1 = (w1.float() - w0.float()).norm()
        d2 = (p.data.float() - w1.float()).norm()
        assert 0.8 < float(d2 / d1) < 1.25
    assert _lib.read_status(dev) == 0
