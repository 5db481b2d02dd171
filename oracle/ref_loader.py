"""Import the reference project's own modules from the staged copy in oracle/_ref/.

TEST INFRASTRUCTURE ONLY (see oracle/make_ref.py).  The staged files are the
reference's, unmodified; this module only arranges sys.path and module names so
that they can be imported side by side:

  pretrain()   the pretraining tree: models.monarch.{monarch_muon,coat_state_muon},
               third_party.coat.optimizer.{triton_kernels,triton_fp8_adamw},
               third_party.coat.utils._fp8_quantization_config, optim.base, ...
               (imported under their upstream names; pretrain/src and pretrain/ go
               on sys.path exactly as pretrain/src/main.py:12-17 and
               pretrain/tests/conftest.py arrange it)
  membench_twin()  membench/src/models/monarch/monarch_muon.py loaded by file path
               under a distinct module name (upstream both twins are called
               models.monarch.monarch_muon)
  sft()        finetune/sft_optimizer.py by file path
"""
from __future__ import annotations

import importlib
import importlib.util
import os
import sys
import types

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.join(HERE, "_ref")


def available() -> bool:
    return os.path.exists(os.path.join(ROOT, "MANIFEST.json"))


def require() -> None:
    if not available():
        raise FileNotFoundError("oracle/_ref/ is missing: run `python oracle/make_ref.py <reference checkout>`")


def _by_path(name: str, rel: str):
    mod = sys.modules.get(name)
    if mod is not None:
        return mod
    spec = importlib.util.spec_from_file_location(name, os.path.join(ROOT, rel))
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def pretrain() -> types.SimpleNamespace:
    """The pretraining tree's modules on the FP8-state path.  Importing models.monarch pulls in the
    reference's Triton riffle kernels, so this needs Triton (and a GPU to run anything)."""
    require()
    for p in (os.path.join(ROOT, "pretrain", "tests"), os.path.join(ROOT, "pretrain"),
              os.path.join(ROOT, "pretrain", "src")):
        if p not in sys.path:
            sys.path.insert(0, p)
    # The staged TritonCoatAdamW.step() calls torch.optim.Optimizer._cuda_graph_capture_health_check, which
    # newer torch releases renamed; give the base class the old name back (the reference file stays as it is).
    import torch
    base = torch.optim.Optimizer
    if not hasattr(base, "_cuda_graph_capture_health_check") and hasattr(base, "_accelerator_graph_capture_health_check"):
        base._cuda_graph_capture_health_check = base._accelerator_graph_capture_health_check
    ns = types.SimpleNamespace()
    ns.monarch_muon = importlib.import_module("models.monarch.monarch_muon")
    ns.coat_state_muon = importlib.import_module("models.monarch.coat_state_muon")
    ns.triton_kernels = importlib.import_module("third_party.coat.optimizer.triton_kernels")
    ns.triton_fp8_adamw = importlib.import_module("third_party.coat.optimizer.triton_fp8_adamw")
    ns.qconfig = importlib.import_module("third_party.coat.utils._fp8_quantization_config")
    return ns


def pretrain_twin():
    """pretrain/src/models/monarch/monarch_muon.py alone (pure torch, no Triton import)."""
    require()
    return _by_path("_ref_pretrain_monarch_muon", "pretrain/src/models/monarch/monarch_muon.py")


def membench_twin():
    """membench/src/models/monarch/monarch_muon.py alone (pure torch): the bf16 reference step."""
    require()
    return _by_path("_ref_membench_monarch_muon", "membench/src/models/monarch/monarch_muon.py")


def sft():
    require()
    return _by_path("_ref_sft_optimizer", "finetune/sft_optimizer.py")
