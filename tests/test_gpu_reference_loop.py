"""The reference's own training program, unmodified, stepping with this library's optimizer.

pretrain/src/main.py builds the model, the parameter groups, the optimizer and the LR scheduler
(main.py:88-203) and hands them to pretrain/src/optim/base.py:train(), whose iteration is
clip_grad_norm_ -> opt.step() -> scheduler.step() -> opt.zero_grad(set_to_none=True) (base.py:121-125), with
checkpoints through opt.state_dict()/load_state_dict() (optim/utils.py:103-132).  The staged copy of those
files (oracle/_ref/) runs here as it is.  Two things are substituted from outside, without touching a file:

  * the data readers (main.get_data_readers): the FineWeb-Edu shards are not on this machine, so a reader
    with the same interface serves seeded random token batches;
  * the optimizer class that main.py imports at `from models.monarch import MonarchMuonOptimizer`
    (main.py:154) / `from models.monarch.coat_state_muon import CoatStateMonarchMuon` (:151): the one-line
    swap a maintainer makes to adopt this library.

Each arm runs 6 iterations, stops (--stop-after), and is started again on the same experiment directory:
main.py finds ckpts/latest/main.pt, restores model, optimizer and scheduler through the reference's
load_checkpoint and continues to iteration 10.  The same two runs with the reference's own optimizer give
the loss curve to compare with.
"""
import argparse
import importlib.util
import json
import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


class _Reader:
    """Stand-in for the reference's FineWeb readers (data/fineweb.py:72-104): sample_batch(), set_step(),
    num_batches().  A small fixed pool of seeded token sequences, so that a few iterations already lower
    the loss."""

    def __init__(self, vocab, batch, seq, seed, pool=4):
        gen = torch.Generator().manual_seed(seed)
        self.tokens = torch.randint(0, vocab, (pool, batch, seq + 1), generator=gen)
        self.step = 0

    def set_step(self, step):
        self.step = step

    def num_batches(self):
        return self.tokens.shape[0]

    def sample_batch(self):
        t = self.tokens[self.step % self.tokens.shape[0]]
        self.step += 1
        return t[:, :-1].contiguous(), t[:, 1:].contiguous()


def _load_main():
    from oracle import ref_loader
    ref_loader.pretrain()                                   # sys.path as pretrain/src/main.py:12-17 sets it
    path = os.path.join(ref_loader.ROOT, "pretrain", "src", "main.py")
    spec = importlib.util.spec_from_file_location("_ref_pretrain_main", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _run(main_mod, exp_dir, name, extra):
    from config.base import parse_args
    argv = ["--experiment-name", name, "--results-base-folder", str(exp_dir), "--wandb-group", "n1",
            "--opt", "monarch_muon", "--monarch-nblocks", "2", "--device", "cuda:0",
            "--n-layer", "2", "--n-embd", "256", "--n-head", "4", "--multiple-of", "16",
            "--sequence-length", "64", "--vocab-size", "512", "--batch-size", "4", "--acc-steps", "2",
            "--iterations", "10", "--warmup-steps", "2", "--lr", "0.02", "--grad-clip", "1.0",
            "--eval-interval", "3", "--eval-batches", "2", "--log-interval", "1", "--latest-ckpt-interval", "2",
            "--seed", "0"] + extra
    args = parse_args(argparse.ArgumentParser(allow_abbrev=False), argv, None)
    main_mod.get_data_readers = lambda a: {"train": _Reader(a.vocab_size, a.batch_size, a.sequence_length, 1),
                                           "val": _Reader(a.vocab_size, a.eval_batch_size, a.sequence_length, 2)}
    main_mod.main(args)
    with open(os.path.join(str(exp_dir), "n1", name, "summary.json")) as f:
        return json.load(f)


@pytest.mark.parametrize("fp8_states", [False, True])
def test_reference_training_loop_with_this_optimizer(tmp_path, fp8_states, capsys):
    from oracle import ref_loader
    assert ref_loader.available(), "oracle/_ref/ is missing: run `python oracle/make_ref.py <reference checkout>`"
    main_mod = _load_main()
    import models.monarch as ref_monarch
    import models.monarch.coat_state_muon as ref_coat
    import monarch_muon_b200 as ours
    from monarch_muon_b200 import _lib
    extra = ["--fp8-optim"] if fp8_states else []
    curves = {}
    tf32 = (torch.backends.cuda.matmul.allow_tf32, torch.backends.cudnn.allow_tf32)    # main.py:52-53 switches them on
    for arm in ("reference", "ours"):
        saved = (ref_monarch.MonarchMuonOptimizer, ref_coat.CoatStateMonarchMuon)
        if arm == "ours":
            ref_monarch.MonarchMuonOptimizer = ours.MonarchMuonOptimizer
            ref_coat.CoatStateMonarchMuon = ours.CoatStateMonarchMuon
        launches0 = _lib.launch_count()
        try:
            first = _run(main_mod, tmp_path, arm, extra + ["--stop-after", "6"])     # iterations 0..5, checkpoints at 2, 4, 6
            ckpt = torch.load(os.path.join(str(tmp_path), "n1", arm, "ckpts", "latest", "main.pt"),
                              map_location="cpu", weights_only=False)
            second = _run(main_mod, tmp_path, arm, extra)                            # resumes at 6, runs to 10
        finally:
            ref_monarch.MonarchMuonOptimizer, ref_coat.CoatStateMonarchMuon = saved
            torch.backends.cuda.matmul.allow_tf32, torch.backends.cudnn.allow_tf32 = tf32
        assert ckpt["itr"] == 6
        if arm == "ours":
            assert _lib.launch_count() > launches0, "this library's kernels did not run"
            # the checkpoint holds reference-shaped optimizer state
            state = ckpt["optimizer"]["state"]
            muon_entries = [e for e in state.values() if "momentum_buffer" in e]
            adam_entries = [e for e in state.values() if "exp_avg" in e]
            assert muon_entries and adam_entries
            want = torch.float8_e4m3fn if fp8_states else torch.float32
            assert all(e["momentum_buffer"].dtype == want for e in muon_entries)
            if fp8_states:
                assert all(e["scale_momentum_buffer"].dtype == torch.float32 and "expand_momentum_buffer" in e
                           and "sqrt_minmax_momentum_buffer" in e for e in muon_entries)
                assert all(e["exp_avg"].dtype == want and e["exp_avg_sq"].dtype == want for e in adam_entries)
        curves[arm] = first["train_loss"] + second["train_loss"]
        assert len(first["train_loss"]) == 6 and len(second["train_loss"]) == 4
        assert all(torch.isfinite(torch.tensor(curves[arm])))
    ref_curve, our_curve = curves["reference"], curves["ours"]
    assert abs(our_curve[0] - ref_curve[0]) < 1e-3                   # same seed, same model, before any step
    assert our_curve[-1] < our_curve[0] - 0.3                        # it learns (the reference's own bar, test_coat_state_muon.py:86)
    assert abs(our_curve[-1] - ref_curve[-1]) / ref_curve[-1] < 0.03  # and like the reference's optimizer does (:88)
    with capsys.disabled():
        print("\nreference loop, fp8 states" if fp8_states else "\nreference loop", json.dumps(curves))
