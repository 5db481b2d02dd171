"""The product has no CPU path: on a machine without a GPU (or with CPU tensors) every optimizer refuses
to step with a clear error instead of computing something else."""
import pytest
import torch


def _params():
    m = [torch.nn.Parameter(torch.zeros(2, 16, 16))]
    a = [torch.nn.Parameter(torch.zeros(8))]
    for p in m + a:
        p.grad = torch.ones_like(p)
    return m, a


def test_monarch_muon_refuses_cpu_tensors():
    from monarch_muon_b200 import MonarchMuonOptimizer
    m, a = _params()
    with pytest.raises(RuntimeError, match="CUDA"):
        MonarchMuonOptimizer(m, a).step()


def test_sft_optimizer_refuses_cpu_tensors():
    from monarch_muon_b200 import SFTOptimizer
    m, a = _params()
    opt = SFTOptimizer([{"params": m, "algorithm": "muon"}, {"params": a, "algorithm": "adamw"}])
    with pytest.raises(RuntimeError, match="CUDA"):
        opt.step()
    assert not opt.state[m[0]] and not opt.state[a[0]]          # nothing was touched


def test_kernel_wrappers_refuse_cpu_tensors():
    from monarch_muon_b200 import newton_schulz_batched, quantize_
    with pytest.raises(RuntimeError, match="CUDA"):
        newton_schulz_batched(torch.zeros(1, 8, 8, dtype=torch.bfloat16))
    with pytest.raises(RuntimeError, match="CUDA"):
        quantize_({}, "m", torch.zeros(128))
