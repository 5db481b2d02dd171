"""Owner-computes data-parallel Monarch-Muon step over torch.distributed.

The reference trains with DDP: gradients are all-reduced and every rank then
runs the whole optimizer step redundantly (pretrain/src/distributed/ddp.py:42-52).
Here each rank steps only the tensors it owns:

    reduce-scatter(gradients)  ->  local momentum / Newton-Schulz / update /
    AdamW on the owned shard   ->  all-gather(updated weights)

over NCCL (NVLink / NVSwitch).  The wire volume equals the all-reduce it
replaces; optimizer state and optimizer compute shrink by the world size.
Nothing in the step reads another GPU's memory from a kernel: remote data lands
in local HBM through NCCL first.

Weights and gradients live in two flat arenas laid out by `partition.make_plan`
(chunk-major, then rank-major).  Parameters are re-pointed at views of the
weight arena and given gradient views of the gradient arena, so backward
accumulates straight into the buffer that is reduce-scattered.  Chunks are
pipelined: all reduce-scatters are queued up front on one communicator, each
chunk's local step waits only for its own reduce-scatter, and its all-gather is
queued on a second communicator as soon as its kernels are enqueued.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import partition


class _Done:
    """Stand-in for a finished collective."""

    def wait(self):
        return True


class ShardedMonarchMuon:
    """Sharded Muon + AdamW step.

    muon_params / adamw_params : lists of parameters, identical on every rank
        (all of one floating dtype and on one device).
    process_group : group for the collectives (default: the world group).  A
        second group over the same ranks is created for the all-gathers so they
        can run beside the reduce-scatters.
    average : divide the reduced gradient by the world size (DDP semantics).
    local_factory(muon_params, adamw_params, **hyper) : builds the optimizer
        that steps the owned views; defaults to MonarchMuonOptimizer (CUDA).
    comm_sms : SMs kept free of this library's kernels during the step, for the
        collectives' kernels.
    dynamic_schedule : let the Newton-Schulz GEMMs draw their tiles from a counter
        during the step, so that SMs taken by a collective's kernels cost those
        SMs' share of the work instead of stalling a whole launch.
    """

    def __init__(self, muon_params, adamw_params, *, process_group=None, lr: float = 5e-3, momentum: float = 0.95,
                 adamw_betas=(0.9, 0.95), adamw_weight_decay: float = 0.1, adamw_eps: float = 1e-8,
                 n_chunks: int = 4, average: bool = True, local_factory=None, second_group: bool = True,
                 comm_sms: int = 0, dynamic_schedule: bool = True, **local_kwargs):
        if not dist.is_initialized():
            raise RuntimeError("ShardedMonarchMuon needs an initialised torch.distributed process group")
        self.group = process_group
        self.world = dist.get_world_size(process_group)
        self.rank = dist.get_rank(process_group)
        self.backend = dist.get_backend(process_group)
        self.ag_group = dist.new_group(ranks=list(range(dist.get_world_size())), backend=self.backend) \
            if (second_group and process_group is None) else process_group
        self.muon_params = list(muon_params)
        self.adamw_params = list(adamw_params)
        allp = self.muon_params + self.adamw_params
        if not allp:
            raise ValueError("no parameters")
        self.dtype, self.device = allp[0].dtype, allp[0].device
        for p in allp:
            if p.dtype != self.dtype or p.device != self.device:
                raise ValueError("all parameters must share one dtype and device")
        for p in self.muon_params:
            if p.dim() != 3:
                raise ValueError("Muon parameters must be 3-D (nblocks, rows, cols)")
        self.plan = partition.make_plan([tuple(p.shape) for p in self.muon_params],
                                        [p.numel() for p in self.adamw_params], self.world, n_chunks)
        self.average = average
        # SMs left free during the step so that NCCL's kernels can run beside the persistent GEMMs
        # (which otherwise occupy every SM and serialise with them)
        self.comm_sms = comm_sms
        self.dynamic_schedule = dynamic_schedule
        n = self.plan.total_elems
        self.w_arena = torch.zeros(n, dtype=self.dtype, device=self.device)
        self.g_arena = torch.zeros(n, dtype=self.dtype, device=self.device)
        # reduced gradients of the owned shards, chunk after chunk (the gradient arena itself is left
        # untouched by the reduce-scatter, so it can keep accumulating or be reused)
        self.own_offset = []
        at = 0
        for ch in self.plan.chunks:
            self.own_offset.append(at)
            at += ch.shard_elems
        self.g_own = torch.zeros(at, dtype=self.dtype, device=self.device)
        # re-point parameters and gradients at the arenas
        with torch.no_grad():
            for p, place in zip(self.muon_params, self.plan.muon):
                self._rebind(p, place.offset)
            for p, (_, off, _) in zip(self.adamw_params, self.plan.adamw):
                self._rebind(p, off)
        # local optimizers, one per chunk, over views of the owned shard
        if local_factory is None:
            from .optimizer import MonarchMuonOptimizer
            local_factory = MonarchMuonOptimizer
        hyper = dict(lr=lr, momentum=momentum, adamw_betas=adamw_betas, adamw_weight_decay=adamw_weight_decay,
                     adamw_eps=adamw_eps, **local_kwargs)
        self.param_groups = [
            {"update_type": "muon", "lr": lr, "momentum": momentum, "params": self.muon_params},
            {"update_type": "adamw", "lr": lr, "betas": adamw_betas, "weight_decay": adamw_weight_decay,
             "eps": adamw_eps, "params": self.adamw_params},
        ]
        self.local = []
        for k, ch in enumerate(self.plan.chunks):
            if ch.kind == "muon":
                owned = []
                for t in self.plan.owned_muon(self.rank, k):
                    shape = self.muon_params[t.index].shape
                    owned.append(self._proxy(k, t.offset, t.numel, shape))
                self.local.append(local_factory(owned, [], **hyper) if owned else None)
            else:
                owned = [self._proxy(k, off, length, (length,))
                         for _, _, length, off in self.plan.adamw_slices(self.rank)]
                self.local.append(local_factory([], owned, **hyper) if owned else None)

    # ----------------------------------------------------------------- layout
    def _rebind(self, p, offset: int) -> None:
        view = self.w_arena[offset:offset + p.numel()].view(p.shape)
        view.copy_(p.data)
        p.data = view
        p.grad = self.g_arena[offset:offset + p.numel()].view(p.shape)

    def _proxy(self, k: int, offset: int, numel: int, shape):
        """A parameter object over an owned slice: weights in the weight arena, gradient in g_own."""
        ch = self.plan.chunks[k]
        local = self.own_offset[k] + (offset - (ch.offset + self.rank * ch.shard_elems))
        q = torch.nn.Parameter(self.w_arena[offset:offset + numel].view(shape), requires_grad=False)
        q.grad = self.g_own[local:local + numel].view(shape)
        return q

    def chunk_views(self, k: int):
        """(gradient chunk arena, reduced-gradient shard, weight chunk arena, owned weight shard)."""
        ch = self.plan.chunks[k]
        n = self.world * ch.shard_elems
        lo = ch.offset + self.rank * ch.shard_elems
        return (self.g_arena[ch.offset:ch.offset + n], self.g_own[self.own_offset[k]:self.own_offset[k] + ch.shard_elems],
                self.w_arena[ch.offset:ch.offset + n], self.w_arena[lo:lo + ch.shard_elems])

    # ------------------------------------------------------------ collectives
    def _reduce_scatter(self, whole, mine):
        if self.backend == "nccl":
            return dist.reduce_scatter_tensor(mine, whole, op=dist.ReduceOp.SUM, group=self.group, async_op=True)
        # CPU ranks (gloo has no reduce-scatter): all-reduce a copy, keep this rank's shard
        tmp = whole.clone()
        dist.all_reduce(tmp, op=dist.ReduceOp.SUM, group=self.group)
        n = mine.numel()
        mine.copy_(tmp[self.rank * n:(self.rank + 1) * n])
        return _Done()

    def _all_gather(self, whole, mine):
        if self.backend == "nccl":
            return dist.all_gather_into_tensor(whole, mine, group=self.ag_group, async_op=True)
        keep = mine.clone()
        whole.zero_()
        mine.copy_(keep)
        return dist.all_reduce(whole, op=dist.ReduceOp.SUM, group=self.ag_group, async_op=True)

    # ------------------------------------------------------------------- step
    def _check_gradients_in_arena(self) -> None:
        """Every parameter's .grad must still be the arena view installed at construction: the
        reduce-scatter sends the arena, not whatever tensor autograd may have put there instead.
        `model.zero_grad()` (set_to_none=True by default) and `p.grad = None` break that; a fresh
        gradient found here is copied into the arena and the view is put back."""
        for params, places in ((self.muon_params, [(pl.offset,) for pl in self.plan.muon]),
                               (self.adamw_params, [(off,) for _, off, _ in self.plan.adamw])):
            for p, (offset,) in zip(params, places):
                view = self.g_arena[offset:offset + p.numel()].view(p.shape)
                g = p.grad
                if g is None:
                    view.zero_()                       # no gradient this step: contributes nothing to the sum
                    p.grad = view
                elif g.data_ptr() != view.data_ptr() or not g.is_contiguous():
                    if g.shape != p.shape:
                        raise ValueError("gradient shape differs from its parameter")
                    view.copy_(g)
                    p.grad = view

    @torch.no_grad()
    def step(self):
        self._check_gradients_in_arena()
        nccl = self.backend == "nccl"
        if nccl:
            from . import _lib
            total = torch.cuda.get_device_properties(self.device).multi_processor_count
            options = _lib.launch_options(sm_limit=max(2, total - self.comm_sms) if self.comm_sms > 0 else 0,
                                          dynamic_schedule=self.dynamic_schedule)
        else:
            import contextlib
            options = contextlib.nullcontext()
        with options:                                  # launch options are put back even if a local step raises
            self._step_chunks()

    def _step_chunks(self):
        nchunks = len(self.plan.chunks)
        rs = []
        for k in range(nchunks):
            g_whole, g_mine, _, _ = self.chunk_views(k)
            rs.append(self._reduce_scatter(g_whole, g_mine))
        ag = []
        scale = 1.0 / self.world if self.average else 1.0
        for k in range(nchunks):
            rs[k].wait()
            opt = self.local[k]
            ch = self.plan.chunks[k]
            if opt is not None:
                group = self.param_groups[0 if ch.kind == "muon" else 1]
                for g in opt.param_groups:
                    if g["update_type"] == group["update_type"]:
                        for key, val in group.items():
                            if key not in ("params", "update_type"):
                                g[key] = val
                if ch.kind == "muon":
                    opt.grad_scale = scale
                elif scale != 1.0:
                    self.chunk_views(k)[1].mul_(scale)      # AdamW has no fused gradient scale
                opt.step()
            _, _, w_whole, w_mine = self.chunk_views(k)
            ag.append(self._all_gather(w_whole, w_mine))
        for w in ag:
            w.wait()

    def zero_grad(self, set_to_none: bool = False):
        """Gradients are arena views and stay allocated; they are zeroed in place (set_to_none is
        accepted for signature compatibility and ignored).  Prefer this to model.zero_grad(): gradients
        that were replaced or dropped are found by step() and copied back into the arena, at the cost
        of that copy."""
        self.g_arena.zero_()
        for p, pl in zip(self.muon_params, self.plan.muon):
            if p.grad is None or p.grad.data_ptr() != self.g_arena[pl.offset:].data_ptr():
                p.grad = self.g_arena[pl.offset:pl.offset + p.numel()].view(p.shape)
        for p, (_, off, _) in zip(self.adamw_params, self.plan.adamw):
            if p.grad is None or p.grad.data_ptr() != self.g_arena[off:].data_ptr():
                p.grad = self.g_arena[off:off + p.numel()].view(p.shape)

    def state_dict(self):
        """Per-rank shard: the local optimizers' state, in chunk order."""
        return {"rank": self.rank, "world": self.world,
                "chunks": [None if o is None else o.state_dict() for o in self.local]}

    def load_state_dict(self, sd):
        if sd["world"] != self.world or sd["rank"] != self.rank:
            raise ValueError("sharded state was saved for another rank/world size")
        for o, s in zip(self.local, sd["chunks"]):
            if o is not None and s is not None:
                o.load_state_dict(s)
