"""monarch_muon_b200 - the Monarch-Muon optimizer step on NVIDIA B200 (sm_100a).

Public surface (mirrors the reference's `models.monarch` names):

    MonarchMuonOptimizer   torch.optim.Optimizer with Muon + AdamW groups
    CoatStateMonarchMuon   the same with FP8 (E4M3) optimizer states
    newton_schulz_batched  batched quintic Newton-Schulz on bf16 stacks
    quantize_, dequantize  FP8 state codecs

All arithmetic runs in libmonarch_muon_b200.so (CUDA, C ABI declared in
include/monarch_muon_b200.h).  There is no CPU implementation: importing works
anywhere, computing needs a CUDA device.
"""
from .optimizer import MonarchMuonOptimizer  # noqa: F401
from .coat_state import CoatStateMonarchMuon  # noqa: F401
from .newton_schulz import newton_schulz_batched, gemm_bf16  # noqa: F401
from .fp8_state import quantize_, dequantize  # noqa: F401
from .sft import SFTOptimizer  # noqa: F401

__all__ = ["MonarchMuonOptimizer", "CoatStateMonarchMuon", "SFTOptimizer", "newton_schulz_batched", "gemm_bf16",
           "quantize_", "dequantize"]
