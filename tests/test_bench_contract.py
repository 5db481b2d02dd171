"""bench.py's bookkeeping, checked without a GPU: the workload is the 6.89B-reference model's optimizer
step, and the reference arm prints a line with the agreed keys."""
import json
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def test_workload_counts_match_the_model():
    import bench
    flops, muon_elems, adamw_elems = bench.workload_counts(4)
    assert muon_elems == 2_558_525_440                       # 1408 + 256 + 128 blocks of the 4-block model
    assert adamw_elems == 2 * 50257 * 4096 + 65 * 4096       # embeddings, output head, 65 norm vectors
    assert abs(flops / 1e12 - 71.640) < 0.01                 # 1408 x 32.212 + 384 x 68.451 GFLOP
    flops2, muon2, _ = bench.workload_counts(2)
    assert muon2 == 2 * muon_elems and abs(flops2 / 1e12 - 286.6) < 0.1


def test_reference_arm_line(monkeypatch, capsys):
    import bench
    monkeypatch.setattr(bench, "cpu_reference_step_ms", lambda nb, steps, warmup, threads=None: (1234.5, "sample", 7, "reference"))
    monkeypatch.setattr(sys, "argv", ["bench.py", "--impl", "reference", "--steps", "2", "--warmup", "1"])
    assert bench.main() == 0
    line = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["unit"] == "ms" and line["higher_is_better"] is False
    assert line["metric"] == bench.METRIC and line["value"] == 1234.5
    assert line["cpu_baseline"] == {"value": 1234.5, "unit": "ms", "cores": 7, "kind": "reference", "sample": "sample"}
    assert line["e2e"] == {"value": 1234.5, "unit": "ms", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert line["config"]["workload"].startswith("full optimizer step")


def test_reference_arm_is_silent_on_other_ranks(monkeypatch, capsys):
    import bench
    monkeypatch.setenv("RANK", "1")
    monkeypatch.setenv("WORLD_SIZE", "2")
    monkeypatch.setattr(sys, "argv", ["bench.py", "--impl", "reference", "--gpus", "2"])
    assert bench.main() == 0
    assert capsys.readouterr().out.strip() == ""


def test_product_arm_needs_a_gpu(monkeypatch):
    import torch
    import bench
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    monkeypatch.setattr(sys, "argv", ["bench.py", "--steps", "1"])
    with pytest.raises(SystemExit, match="CUDA"):
        bench.main()


def test_cpu_reference_arm_runs_the_staged_reference_class(monkeypatch):
    """With oracle/_ref/ staged, the CPU arm steps the reference's own MonarchMuonOptimizer (kind
    "reference"); here on a tiny stand-in model so that the test takes a second."""
    import bench
    from monarch_muon_b200 import shapes as S
    from oracle import ref_loader
    if not ref_loader.available():
        pytest.skip("oracle/_ref/ not staged (python oracle/make_ref.py <reference checkout>)")
    monkeypatch.setitem(S.MODEL_689B, "d_model", 256)
    monkeypatch.setitem(S.MODEL_689B, "n_layers", 24)
    monkeypatch.setitem(S.MODEL_689B, "intermediate", 688)
    monkeypatch.setitem(S.MODEL_689B, "vocab", 4096)
    ms, desc, threads, kind = bench.cpu_reference_step_ms(4, 1, 0, threads=2)
    assert kind == "reference" and ms > 0 and "reference's own" in desc
