"""Host logic of the sharded step on CPU ranks (gloo, world size 2 and 3).

The ownership plan, arena layout, collectives and per-chunk pipeline are
exercised with the CUDA kernels replaced by the CPU oracle (injected through
`local_factory`); the sharded result must equal a serial oracle step on the
averaged gradient.
"""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from monarch_muon_b200 import partition, shapes


def test_plan_full_model_is_balanced():
    m = shapes.MODEL_689B
    ms = shapes.llama_monarch_muon_shapes(m["d_model"], m["n_layers"], m["intermediate"], 4)
    an = [a * (b if len(s) > 1 else 1) for s in shapes.llama_adamw_shapes(m["d_model"], m["n_layers"], m["vocab"])
          for a, b in [(s[0], s[1] if len(s) > 1 else 1)]]
    for world in (1, 2, 4, 8):
        plan = partition.make_plan(ms, an, world, n_chunks=4)
        fl = partition.flops_per_rank(plan, ms, shapes.ns_flops)
        assert max(fl) == pytest.approx(min(fl))                       # equal Newton-Schulz work per rank
        assert abs(sum(fl) / 1e12 - 71.640) < 0.01
        # every tensor sits inside its owner's shard, no overlaps, 128-element aligned
        spans = []
        for t in plan.muon:
            ch = plan.chunks[t.chunk]
            lo = ch.offset + t.rank * ch.shard_elems
            assert lo <= t.offset and t.offset + t.numel <= lo + ch.shard_elems and t.offset % 128 == 0
            spans.append((t.offset, t.offset + t.numel))
        spans.sort()
        assert all(a[1] <= b[0] for a, b in zip(spans, spans[1:]))
        muon_elems = sum(t.numel for t in plan.muon)
        assert muon_elems == 2_558_525_440
        assert plan.total_elems - muon_elems - sum(an) < 0.001 * plan.total_elems   # padding is negligible
        covered = sum(l for r in range(world) for _, _, l, _ in plan.adamw_slices(r))
        assert covered == sum(an)


def test_plan_uneven_counts_are_padded_not_lost():
    ms = [(2, 64, 64)] * 5 + [(1, 96, 64)] * 3
    plan = partition.make_plan(ms, [1000, 17], world=3, n_chunks=2)
    assert sorted(t.index for t in plan.muon) == list(range(8))
    for r in range(3):
        for _, start, length, off in plan.adamw_slices(r):
            assert length > 0 and start >= 0
    assert sum(l for r in range(3) for _, _, l, _ in plan.adamw_slices(r)) == 1017


class _OracleLocal:
    """What MonarchMuonOptimizer is to the sharded step, computed by the CPU oracle."""

    def __init__(self, muon, adamw, *, lr, momentum, adamw_betas, adamw_weight_decay, adamw_eps):
        from oracle import muon_oracle
        self.muon, self.adamw = list(muon), list(adamw)
        self.opt = muon_oracle.OracleMonarchMuon([p.data for p in self.muon], [p.data for p in self.adamw], lr=lr,
                                                 momentum=momentum, adamw_betas=adamw_betas,
                                                 adamw_weight_decay=adamw_weight_decay, adamw_eps=adamw_eps)
        self.param_groups = [{"update_type": "muon", "lr": lr, "momentum": momentum},
                             {"update_type": "adamw", "lr": lr, "betas": adamw_betas,
                              "weight_decay": adamw_weight_decay, "eps": adamw_eps}]
        self.grad_scale = 1.0

    def step(self):
        self.opt.lr["muon"] = self.param_groups[0]["lr"]
        self.opt.lr["adamw"] = self.param_groups[1]["lr"]
        self.opt.step([p.grad * self.grad_scale for p in self.muon], [p.grad for p in self.adamw])


def _make(seed_w=5):
    gen = torch.Generator().manual_seed(seed_w)
    ms = [(2, 32, 32)] * 5 + [(1, 48, 32)] * 4 + [(2, 32, 48)] * 3
    asz = [(300, 8), (8,), (77,)]
    muon = [torch.nn.Parameter(0.02 * torch.randn(s, generator=gen)) for s in ms]
    adamw = [torch.nn.Parameter(0.02 * torch.randn(s, generator=gen)) for s in asz]
    return muon, adamw


def _grads(rank, step, params):
    gen = torch.Generator().manual_seed(1000 * step + rank)
    return [1e-3 * torch.randn(p.shape, generator=gen) for p in params]


def _worker(rank, world, port, steps, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from monarch_muon_b200.sharded import ShardedMonarchMuon
        muon, adamw = _make()
        opt = ShardedMonarchMuon(muon, adamw, lr=0.02, n_chunks=2, local_factory=_OracleLocal)
        opt.param_groups[1]["lr"] = 3e-4
        for step in range(steps):
            for p, g in zip(muon + adamw, _grads(rank, step, muon + adamw)):
                p.grad.copy_(g)                                  # gradients are arena views
            opt.step()
        if rank == 0:
            torch.save([p.data.clone() for p in muon + adamw], out)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_sharded_step_equals_serial_on_averaged_gradient(world, tmp_path):
    from oracle import muon_oracle
    steps = 2
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    out = str(tmp_path / "sharded.pt")
    mp.spawn(_worker, args=(world, port, steps, out), nprocs=world, join=True)
    got = torch.load(out)
    muon, adamw = _make()
    ref = muon_oracle.OracleMonarchMuon([p.data for p in muon], [p.data for p in adamw], lr=0.02)
    ref.lr["adamw"] = 3e-4
    for step in range(steps):
        per_rank = [_grads(r, step, muon + adamw) for r in range(world)]
        avg = [sum(gs) / world for gs in zip(*per_rank)]
        ref.step(avg[:len(muon)], avg[len(muon):])
    for g, p in zip(got, muon + adamw):
        # same arithmetic, only the order of the gradient sum differs (all-reduce vs python sum)
        assert torch.allclose(g, p.data, rtol=2e-4, atol=2e-6)
