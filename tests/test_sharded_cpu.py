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


def test_plan_deals_remainders_by_load():
    """Counts that do not divide by the world size: no rank gets more than one tensor of a shape above
    another, and the extras of the light shape go to the ranks that did not get an extra heavy one."""
    ms = [(1, 64, 128)] * 5 + [(1, 64, 64)] * 5          # 5 heavy + 5 light tensors on 4 ranks, one chunk
    plan = partition.make_plan(ms, [], world=4, n_chunks=1)
    per_rank = {r: [t.index for t in plan.muon if t.rank == r] for r in range(4)}
    heavy = {r: sum(1 for i in v if i < 5) for r, v in per_rank.items()}
    light = {r: sum(1 for i in v if i >= 5) for r, v in per_rank.items()}
    assert sorted(heavy.values()) == [1, 1, 1, 2] and sorted(light.values()) == [1, 1, 1, 2]
    assert all(heavy[r] + light[r] <= 3 for r in range(4))
    assert not any(heavy[r] == 2 and light[r] == 2 for r in range(4))     # the two extras sit on different ranks
    fl = partition.flops_per_rank(plan, ms, shapes.ns_flops)
    both_extras_on_one_rank = 2 * shapes.ns_flops(64, 128) + 2 * shapes.ns_flops(64, 64)
    assert max(fl) < both_extras_on_one_rank               # what dealing every shape "first ranks first" would give


class _MomentumLocal(torch.optim.Optimizer):
    """A minimal torch optimizer with per-parameter state, standing in for MonarchMuonOptimizer where only
    the bookkeeping of ShardedMonarchMuon (state gathering, ownership) is under test."""

    def __init__(self, muon, adamw, *, lr, momentum, adamw_betas, adamw_weight_decay, adamw_eps):
        super().__init__([{"params": list(muon), "update_type": "muon", "momentum": momentum},
                          {"params": list(adamw), "update_type": "adamw", "betas": adamw_betas,
                           "weight_decay": adamw_weight_decay, "eps": adamw_eps}], dict(lr=lr))
        self.grad_scale = 1.0

    @torch.no_grad()
    def step(self):
        for g in self.param_groups:
            for p in g["params"]:
                st = self.state[p]
                if g["update_type"] == "muon":
                    buf = st.setdefault("momentum_buffer", torch.zeros_like(p))
                    buf.mul_(g["momentum"]).add_(p.grad * self.grad_scale)
                    p.add_(buf, alpha=-g["lr"])
                else:
                    st["step"] = st.get("step", 0) + 1
                    m = st.setdefault("exp_avg", torch.zeros_like(p))
                    v = st.setdefault("exp_avg_sq", torch.zeros_like(p))
                    m.mul_(0.9).add_(p.grad, alpha=0.1)
                    v.mul_(0.95).addcmul_(p.grad, p.grad, value=0.05)
                    p.add_(m / (v.sqrt() + 1e-8), alpha=-g["lr"])


def _state_worker(rank, world, port, path, mode):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from monarch_muon_b200.sharded import ShardedMonarchMuon
        muon, adamw = _make()
        # comm="auto": on CPU ranks (gloo) there is no symmetric memory, so the choice must fall back to the
        # torch.distributed collectives; an explicit "p2p" must be refused
        opt = ShardedMonarchMuon(muon, adamw, lr=0.02, n_chunks=2, local_factory=_MomentumLocal, comm="auto")
        assert opt.comm == "nccl"
        try:
            ShardedMonarchMuon(muon, adamw, lr=0.02, n_chunks=2, local_factory=_MomentumLocal, comm="p2p")
            raise AssertionError("comm='p2p' accepted on gloo ranks")
        except RuntimeError as exc:
            assert "p2p" in str(exc)
        if mode == "save":
            for step in range(2):
                if step == 1:
                    for p in muon + adamw:                        # what model.zero_grad() does by default
                        p.grad = None
                    for p, g in zip(muon + adamw, _grads(rank, step, muon + adamw)):
                        p.grad = g.clone()                        # fresh tensors outside the arena
                else:
                    for p, g in zip(muon + adamw, _grads(rank, step, muon + adamw)):
                        p.grad.copy_(g)
                opt.step()
            sd = opt.state_dict()                                 # collective
            if rank == 0:
                torch.save({"sd": sd, "weights": [p.data.clone() for p in muon + adamw]}, path)
        else:
            blob = torch.load(path, weights_only=False)
            for p, w in zip(muon + adamw, blob["weights"]):
                p.data.copy_(w)
            opt.load_state_dict(blob["sd"])
            for p, g in zip(muon + adamw, _grads(0, 7, muon + adamw)):     # same gradient on every rank
                p.grad.copy_(g)
            opt.step()
            again = opt.state_dict()
            if rank == 0:
                torch.save({"sd": again, "weights": [p.data.clone() for p in muon + adamw]}, path + f".w{world}")
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_state_dict_is_reference_shaped_and_reshards(tmp_path):
    """state_dict() gathers the sharded state into the reference's shape (one entry per parameter, Muon
    first; AdamW tensors cut across ranks reassembled), independent of the world size; a checkpoint saved
    on 2 ranks resumes on 3 ranks and on 2 ranks with identical results.  The second saved step feeds
    gradients the way a training loop does after model.zero_grad(): fresh tensors, not the arena views."""
    path = str(tmp_path / "ckpt.pt")
    mp.spawn(_state_worker, args=(2, _free_port(), path, "save"), nprocs=2, join=True)
    blob = torch.load(path, weights_only=False)
    muon, adamw = _make()
    sd = blob["sd"]
    assert sorted(sd["state"].keys()) == list(range(len(muon) + len(adamw)))
    assert [g["update_type"] for g in sd["param_groups"]] == ["muon", "adamw"]
    assert sd["param_groups"][0]["params"] == list(range(len(muon)))
    for i, p in enumerate(muon):
        assert sd["state"][i]["momentum_buffer"].shape == p.shape
    for j, p in enumerate(adamw):
        e = sd["state"][len(muon) + j]
        assert e["exp_avg"].shape == p.shape and e["exp_avg_sq"].shape == p.shape and e["step"] == 2
    for world in (2, 3):
        mp.spawn(_state_worker, args=(world, _free_port(), path, "load"), nprocs=world, join=True)
    a = torch.load(path + ".w2", weights_only=False)
    b = torch.load(path + ".w3", weights_only=False)
    for x, y in zip(a["weights"], b["weights"]):
        assert torch.allclose(x, y, rtol=1e-6, atol=1e-8)
    for k, ea in a["sd"]["state"].items():
        for name, v in ea.items():
            w = b["sd"]["state"][k][name]
            assert torch.allclose(v, w, rtol=1e-6, atol=1e-9) if torch.is_tensor(v) else v == w


def _fault_worker(rank, world, port, mode):
    import datetime
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    from monarch_muon_b200.sharded import ShardedMonarchMuon
    muon, adamw = _make()
    if mode == "mismatched_plan" and rank == 1:
        muon = muon[:-1]                                           # one rank passes a different parameter list
    opt = ShardedMonarchMuon(muon, adamw, lr=0.02, n_chunks=2, local_factory=_MomentumLocal)
    if mode == "rank_raises" and rank == 1:
        raise RuntimeError("rank 1 fails before the collective")   # e.g. a data-loader error before step()
    opt.step()


@pytest.mark.parametrize("mode", ["mismatched_plan", "rank_raises"])
def test_host_side_faults_raise_instead_of_hanging(mode):
    """Failures made on the host, none on a device.  (1) Ranks that built different ownership plans: the
    constructor's digest exchange raises ValueError on every rank.  (2) A rank that raises before the step's
    first collective: the other rank's collective ends with an error (connection closed by the dead peer, or
    the group's 8-second timeout) instead of waiting forever.  Either way the launcher sees a failed job
    within seconds."""
    import time
    t0 = time.time()
    with pytest.raises(Exception) as info:
        mp.spawn(_fault_worker, args=(2, _free_port(), mode), nprocs=2, join=True)
    assert time.time() - t0 < 60
    text = str(info.value)
    if mode == "mismatched_plan":
        assert "different ownership plans" in text
    else:
        assert "rank 1 fails" in text or "timed out" in text.lower() or "closed" in text.lower() or "exit" in text.lower()
