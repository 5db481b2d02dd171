"""Owner-computes data-parallel Monarch-Muon step over torch.distributed.

The reference trains with DDP: gradients are all-reduced and every rank then
runs the whole optimizer step redundantly (pretrain/src/distributed/ddp.py:42-52).
Here each rank steps only the tensors it owns:

    reduce-scatter(gradients)  ->  local momentum / Newton-Schulz + update /
    AdamW on the owned shard   ->  all-gather(updated weights)

The wire volume equals the all-reduce it replaces; optimizer state and optimizer
compute shrink by the world size.

Weights and gradients live in two flat arenas laid out by `partition.make_plan`
(chunk-major, then rank-major).  Parameters are re-pointed at views of the
weight arena and given gradient views of the gradient arena, so backward
accumulates straight into the buffer that is reduced.  Chunks are pipelined.

Three transports (`comm=`):

  "nccl"      NCCL reduce-scatter / all-gather through torch.distributed: all
              reduce-scatters are queued up front on one communicator, each
              chunk's local step waits only for its own, and its all-gather is
              queued on a second communicator as soon as its kernels are
              enqueued.  Remote data lands in local HBM through NCCL; no kernel
              of this library touches another GPU's memory.
  "multimem"  this library's own kernels over NVSwitch multicast
              (csrc/multimem.cu): the arenas are symmetric memory, a rank reduces
              its shard of a chunk with multimem.ld_reduce (the sum is formed
              inside the switch) on one side stream and broadcasts its updated
              shard with multimem.st on another, while the GEMMs of the chunk in
              between run on the caller's stream.  The reduce loads the links
              outbound and the broadcast inbound, so the two overlap at full
              rate, which two ring collectives cannot.  Ranks are ordered against
              each other by one tiny NCCL all-reduce before the first reduce of a
              step and one after the last broadcast; the kernels themselves never
              wait on a peer.  Pays from four GPUs on (with two, a ring moves
              fewer bytes per link).
  "p2p"       the same pipeline with plain peer loads and stores (symmetric
              memory's per-rank pointers, no multicast object): a rank sums its
              shard from every rank's gradient arena in rank order and writes its
              updated shard into every rank's weight arena.  Ring-equal bytes per
              link, one hop, and - like the multicast kernels - CTAs small enough
              to share an SM with a GEMM CTA.
  "auto"      what measured fastest on B200s: "p2p" for two ranks (where the arenas
              can be mapped as symmetric memory), "nccl" otherwise.
"""
from __future__ import annotations

import contextlib
import hashlib

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
    comm : "nccl", "multimem" or "auto" (see the module text).
    comm_sms : SMs kept free of this library's compute kernels during the step,
        for the communication kernels (default 0: NCCL's kernels take SMs from the
        GEMMs as they come, the multicast kernels are small enough to share an SM
        with a GEMM CTA).
    comm_ctas : CTAs of each multicast or peer kernel (default: one per SM).
    chunk_edge : size of the first and the last Muon chunk relative to the inner ones
        (their transfers are the ones no computation hides).
    dynamic_schedule : let the Newton-Schulz GEMMs draw their tiles from a counter
        during the step, so that SMs taken by a communication kernel cost those
        SMs' share of the work instead of stalling a whole launch.
    """

    def __init__(self, muon_params, adamw_params, *, process_group=None, lr: float = 5e-3, momentum: float = 0.95,
                 adamw_betas=(0.9, 0.95), adamw_weight_decay: float = 0.1, adamw_eps: float = 1e-8,
                 n_chunks: int = 4, average: bool = True, local_factory=None, second_group: bool = True,
                 comm: str = "nccl", comm_sms: int | None = None, comm_ctas: int | None = None,
                 dynamic_schedule: bool = True, chunk_edge: float = 0.5, **local_kwargs):
        if not dist.is_initialized():
            raise RuntimeError("ShardedMonarchMuon needs an initialised torch.distributed process group")
        if comm not in ("nccl", "multimem", "p2p", "auto"):
            raise ValueError("comm must be 'nccl', 'multimem', 'p2p' or 'auto'")
        self.group = process_group
        self.world = dist.get_world_size(process_group)
        self.rank = dist.get_rank(process_group)
        self.backend = dist.get_backend(process_group)
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
                                        [p.numel() for p in self.adamw_params], self.world, n_chunks, edge=chunk_edge)
        self._check_same_plan_everywhere()
        self.ag_group = dist.new_group(ranks=list(range(dist.get_world_size())), backend=self.backend) \
            if (second_group and process_group is None) else process_group
        self.average = average
        self.dynamic_schedule = dynamic_schedule
        self.comm_ctas = int(comm_ctas) if comm_ctas is not None else (
            torch.cuda.get_device_properties(self.device).multi_processor_count if self.device.type == "cuda" else 1)
        n = self.plan.total_elems
        # ---- arenas: symmetric memory when this library's multicast kernels move the data
        self.comm = "nccl"
        self._mc_g = self._mc_w = 0
        self._peer_g = self._peer_w = None             # per-rank base addresses of the arenas (symmetric memory)
        want_mc = comm == "multimem"
        want_p2p = comm == "p2p" or (comm == "auto" and self.world == 2)
        if (want_mc or want_p2p) and self.backend == "nccl" and self.dtype == torch.bfloat16:
            arenas = self._symmetric_arenas(n, need_multicast=want_mc)
            if arenas is not None:
                self.w_arena, self.g_arena, self._mc_w, self._mc_g, self._peer_w, self._peer_g = arenas
                self.comm = "multimem" if want_mc else "p2p"
            elif comm in ("multimem", "p2p"):
                raise RuntimeError(f"comm='{comm}': the arenas could not be mapped as symmetric memory"
                                   + (" with NVSwitch multicast" if want_mc else "") + " on this group")
        elif comm == "p2p":
            raise RuntimeError("comm='p2p' needs the NCCL backend and bf16 parameters")
        if self.comm == "nccl":
            self.w_arena = torch.zeros(n, dtype=self.dtype, device=self.device)
            self.g_arena = torch.zeros(n, dtype=self.dtype, device=self.device)
        # SMs left free during the step so that communication kernels can run beside the persistent GEMMs
        # (which otherwise occupy every SM and serialise with them)
        self.comm_sms = 0 if comm_sms is None else int(comm_sms)
        # reduced gradients of the owned shards, chunk after chunk (the gradient arena itself is left
        # untouched by the reduction, so it can keep accumulating or be reused)
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
        self._owned = []            # per chunk: [(kind, index in the caller's list, start inside the tensor, proxy)]
        for k, ch in enumerate(self.plan.chunks):
            if ch.kind == "muon":
                owned = []
                for t in self.plan.owned_muon(self.rank, k):
                    shape = self.muon_params[t.index].shape
                    owned.append(("muon", t.index, 0, self._proxy(k, t.offset, t.numel, shape)))
                self.local.append(local_factory([q for *_, q in owned], [], **hyper) if owned else None)
            else:
                owned = [("adamw", idx, start, self._proxy(k, off, length, (length,)))
                         for idx, start, length, off in self.plan.adamw_slices(self.rank)]
                self.local.append(local_factory([], [q for *_, q in owned], **hyper) if owned else None)
            self._owned.append(owned)
        self._streams = None
        self._flag = None

    # ----------------------------------------------------------------- checks
    def _check_same_plan_everywhere(self) -> None:
        """Every rank must have built the same ownership plan (same parameter lists, chunking and world
        size): a rank with another table would reduce and gather other byte ranges.  Compared through one
        all-gather of a digest; a mismatch raises on every rank instead of corrupting or hanging later."""
        text = repr((self.world, [(c.offset, c.shard_elems, c.kind) for c in self.plan.chunks],
                     [(t.index, t.chunk, t.rank, t.offset, t.numel) for t in self.plan.muon], self.plan.adamw,
                     str(self.dtype)))
        digest = hashlib.sha256(text.encode()).digest()[:8]
        mine = torch.tensor(list(digest), dtype=torch.uint8)
        if self.backend == "nccl":
            mine = mine.to(self.device)
        gathered = [torch.empty_like(mine) for _ in range(self.world)]
        dist.all_gather(gathered, mine, group=self.group)
        if any(not torch.equal(g, mine) for g in gathered):
            raise ValueError("ShardedMonarchMuon: the ranks built different ownership plans (different parameter "
                             "lists, chunk counts or dtypes); every rank must pass the same parameters in the same order")

    def _symmetric_arenas(self, n: int, need_multicast: bool = True):
        """Weight and gradient arenas in symmetric memory with their multicast addresses and per-rank
        addresses, or None when the group cannot provide them (no peer access or, where asked for, no
        NVSwitch multicast; allocation refused).  All ranks decide together."""
        ok, out = 1, None
        try:
            import torch.distributed._symmetric_memory as symm_mem
            group = self.group if self.group is not None else dist.group.WORLD
            w = symm_mem.empty(n, dtype=self.dtype, device=self.device)
            g = symm_mem.empty(n, dtype=self.dtype, device=self.device)
            hw = symm_mem.rendezvous(w, group)
            hg = symm_mem.rendezvous(g, group)
            mw, mg = int(hw.multicast_ptr or 0), int(hg.multicast_ptr or 0)
            pw, pg = [int(a) for a in hw.buffer_ptrs], [int(a) for a in hg.buffer_ptrs]
            if (need_multicast and (not mw or not mg)) or len(pw) != self.world or not all(pw) or not all(pg):
                ok = 0
            else:
                w.zero_()
                g.zero_()
                out = (w, g, mw, mg, pw, pg)
                self._symm_handles = (hw, hg)        # keep the mappings alive
        except Exception:                            # no symmetric memory in this build / on this fabric
            ok = 0
        flag = torch.tensor([ok], device=self.device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group)
        return out if int(flag.item()) == 1 else None

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

    def _fence(self):
        """Order this rank's stream against every other rank's: a one-element NCCL all-reduce.  Work queued
        before it on any rank has finished before work queued after it on any rank starts."""
        if self._flag is None:
            self._flag = torch.zeros(1, dtype=torch.float32, device=self.device)
        dist.all_reduce(self._flag, group=self.group)

    # ------------------------------------------------------------------- step
    def _check_gradients_in_arena(self) -> None:
        """Every parameter's .grad must still be the arena view installed at construction: the
        reduction reads the arena, not whatever tensor autograd may have put there instead.
        `model.zero_grad()` (set_to_none=True by default) and `p.grad = None` break that; a fresh
        gradient found here is copied into the arena and the view is put back."""
        for params, offsets in ((self.muon_params, [pl.offset for pl in self.plan.muon]),
                                (self.adamw_params, [off for _, off, _ in self.plan.adamw])):
            for p, offset in zip(params, offsets):
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
    def step(self, host_grad_arena: torch.Tensor | None = None):
        """One sharded step.  `host_grad_arena` (extension): this rank's gradients as one pinned host tensor
        with the arena's layout and dtype; it is copied into the gradient arena chunk by chunk on a copy
        stream, each chunk's reduction starting as soon as its own copy has landed, so the host-to-device
        transfer of later chunks runs under the reduction and compute of earlier ones."""
        self._copied = None
        if host_grad_arena is not None:
            if host_grad_arena.shape != self.g_arena.shape or host_grad_arena.dtype != self.g_arena.dtype:
                raise ValueError("host_grad_arena must have the gradient arena's shape and dtype")
            self._enqueue_host_copies(host_grad_arena)
        else:
            self._check_gradients_in_arena()
        if self.backend == "nccl":
            from . import _lib
            total = torch.cuda.get_device_properties(self.device).multi_processor_count
            options = _lib.launch_options(sm_limit=max(2, total - self.comm_sms) if self.comm_sms > 0 else 0,
                                          dynamic_schedule=self.dynamic_schedule)
        else:
            options = contextlib.nullcontext()
        with options:                                  # launch options are put back even if a local step raises
            if self.comm in ("multimem", "p2p"):
                self._step_chunks_own_kernels()
            else:
                self._step_chunks()

    def _enqueue_host_copies(self, host) -> None:
        main = torch.cuda.current_stream(self.device)
        if getattr(self, "_copy_stream", None) is None:
            self._copy_stream = torch.cuda.Stream(device=self.device)
            self._issue_stream = torch.cuda.Stream(device=self.device)
        cs = self._copy_stream
        cs.wait_stream(main)                           # last step's readers of the arena are done
        self._copied = []
        with torch.cuda.stream(cs):
            for ch in self.plan.chunks:
                lo, hi = ch.offset, ch.offset + self.world * ch.shard_elems
                self.g_arena[lo:hi].copy_(host[lo:hi], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(cs)
                self._copied.append(ev)

    def _local_step(self, k: int) -> None:
        opt = self.local[k]
        if opt is None:
            return
        ch = self.plan.chunks[k]
        scale = 1.0 / self.world if self.average else 1.0
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

    def _step_chunks(self):
        nchunks = len(self.plan.chunks)
        rs = []
        for k in range(nchunks):
            g_whole, g_mine, _, _ = self.chunk_views(k)
            if self._copied is not None:
                # the collective is issued from a stream that waits for this chunk's copy only, so the
                # caller's stream (and the local steps queued on it) does not wait for later copies
                with torch.cuda.stream(self._issue_stream):
                    self._issue_stream.wait_event(self._copied[k])
                    rs.append(self._reduce_scatter(g_whole, g_mine))
            else:
                rs.append(self._reduce_scatter(g_whole, g_mine))
        ag = []
        for k in range(nchunks):
            rs[k].wait()
            self._local_step(k)
            _, _, w_whole, w_mine = self.chunk_views(k)
            ag.append(self._all_gather(w_whole, w_mine))
        for w in ag:
            w.wait()

    def _launch_reduce(self, lib, k: int, stream) -> None:
        """This rank's share of chunk k's reduce-scatter: g_own[chunk k] = sum over ranks of the shard."""
        from . import _lib
        ch = self.plan.chunks[k]
        esz = self.g_arena.element_size()
        lo = (ch.offset + self.rank * ch.shard_elems) * esz
        dst = self.g_own[self.own_offset[k]:].data_ptr()
        if self.comm == "multimem":
            _lib.check(lib.mmb_multimem_reduce_bf16(self._mc_g + lo, dst, ch.shard_elems * esz, self.comm_ctas, stream),
                       "multimem_reduce_bf16")
        else:
            copies = (_lib.C.c_void_p * self.world)(*[base + lo for base in self._peer_g])
            _lib.check(lib.mmb_peer_reduce_bf16(copies, self.world, dst, ch.shard_elems * esz, self.comm_ctas, stream),
                       "peer_reduce_bf16")

    def _launch_broadcast(self, lib, k: int, stream) -> None:
        """This rank's share of chunk k's all-gather: its updated shard goes into every rank's weight arena."""
        from . import _lib
        ch = self.plan.chunks[k]
        esz = self.w_arena.element_size()
        lo = ch.offset + self.rank * ch.shard_elems
        src = self.w_arena[lo:].data_ptr()
        if self.comm == "multimem":
            _lib.check(lib.mmb_multimem_broadcast(src, self._mc_w + lo * esz, ch.shard_elems * esz, self.comm_ctas, stream),
                       "multimem_broadcast")
        else:
            others = [base + lo * esz for r, base in enumerate(self._peer_w) if r != self.rank]
            copies = (_lib.C.c_void_p * max(1, len(others)))(*others)
            _lib.check(lib.mmb_peer_broadcast(src, copies, len(others), ch.shard_elems * esz, self.comm_ctas, stream),
                       "peer_broadcast")

    def _step_chunks_own_kernels(self):
        """The chunk pipeline over this library's own transfer kernels (multicast or peer loads/stores): all
        reductions are queued on one side stream, each chunk's local step waits for its own reduction on the
        caller's stream, and its broadcast goes to a second side stream; reductions and broadcasts overlap
        each other and the GEMMs."""
        from . import _lib
        lib = _lib.load()
        main = torch.cuda.current_stream(self.device)
        if self._streams is None:
            # High priority: the transfer kernels' CTAs are small and meant to sit beside the GEMM CTAs, but the
            # GEMMs are launched ahead of time (programmatic serialisation) and a pending GEMM grid that cannot
            # be placed yet would otherwise hold up the placement of a transfer kernel queued behind it.
            self._streams = (torch.cuda.Stream(device=self.device, priority=-1),
                             torch.cuda.Stream(device=self.device, priority=-1))
        s_red, s_bc = self._streams
        esz = self.g_arena.element_size()
        nchunks = len(self.plan.chunks)
        self._fence()                                  # every rank's gradients are in its arena
        s_red.wait_stream(main)
        s_bc.wait_stream(main)
        reduced = []
        with torch.cuda.stream(s_red):
            for k in range(nchunks):
                ch = self.plan.chunks[k]
                if self._copied is not None:
                    # gradients arriving from the host: a chunk may be reduced once every rank's copy of that
                    # chunk has landed - one more fence per chunk, on the reduction stream
                    s_red.wait_event(self._copied[k])
                    self._fence()
                self._launch_reduce(lib, k, s_red.cuda_stream)
                ev = torch.cuda.Event()
                ev.record(s_red)
                reduced.append(ev)
        for k in range(nchunks):
            ch = self.plan.chunks[k]
            main.wait_event(reduced[k])
            self._local_step(k)
            done = torch.cuda.Event()
            done.record(main)
            with torch.cuda.stream(s_bc):
                s_bc.wait_event(done)
                self._launch_broadcast(lib, k, s_bc.cuda_stream)
        main.wait_stream(s_bc)
        main.wait_stream(s_red)
        self._fence()                                  # every rank's broadcasts have landed everywhere

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

    # ----------------------------------------------------------- checkpoints
    def _local_entries(self):
        """This rank's optimizer state, keyed like the reference's state_dict: for a Muon tensor
        ("muon", index) -> its state; for the slice of an AdamW tensor ("adamw", index, start) -> the
        slice's state.  Tensors are moved to the CPU."""
        out = {}
        for owned, opt in zip(self._owned, self.local):
            if opt is None:
                continue
            for kind, idx, start, proxy in owned:
                st = opt.state.get(proxy)
                if not st:
                    continue
                entry = {k: (v.detach().cpu() if torch.is_tensor(v) else v) for k, v in st.items()}
                out[(kind, idx) if kind == "muon" else (kind, idx, start)] = entry
        return out

    def state_dict(self):
        """The optimizer state in the reference's shape: {"state": {parameter index: {...}}, "param_groups":
        [...]} with Muon parameters first (indices as in MonarchMuonOptimizer(muon_params, adamw_params)),
        identical on every rank and independent of the world size it was saved on, so that the reference's
        save_checkpoint / load_checkpoint (pretrain/src/optim/utils.py:103-132) round-trip it and a run can
        resume on another number of GPUs.  Collective: every rank must call it.  Moments of an AdamW tensor
        that is cut across ranks are reassembled (element-wise state; `step` is taken from its first slice)."""
        for opt in self.local:
            if opt is not None and hasattr(opt, "check_device_status"):
                opt.check_device_status()
        gathered = [None] * self.world
        dist.all_gather_object(gathered, self._local_entries(), group=self.group)
        nm = len(self.muon_params)
        state = {}
        pieces = {}
        for entries in gathered:
            for key, entry in entries.items():
                if key[0] == "muon":
                    state[key[1]] = entry
                else:
                    pieces.setdefault(key[1], []).append((key[2], entry))
        for idx, parts in pieces.items():
            parts.sort(key=lambda t: t[0])
            p = self.adamw_params[idx]
            merged = {}
            for name, v in parts[0][1].items():
                if torch.is_tensor(v) and v.dim() > 0:
                    if any(v2[name].dtype == torch.float8_e4m3fn for _, v2 in parts):
                        raise NotImplementedError("FP8 AdamW moments of a tensor cut across ranks are not merged")
                    merged[name] = torch.cat([e[name].reshape(-1) for _, e in parts]).view(p.shape)
                else:
                    merged[name] = v
            state[nm + idx] = merged
        groups = []
        at = 0
        for g in self.param_groups:
            d = {k: v for k, v in g.items() if k != "params"}
            d["params"] = list(range(at, at + len(g["params"])))
            at += len(g["params"])
            groups.append(d)
        return {"state": state, "param_groups": groups}

    def load_state_dict(self, sd):
        """Restore a state dict written by state_dict() - on any world size - or by the reference's
        optimizer: every rank takes the entries of the tensors (and AdamW slices) it owns."""
        nm = len(self.muon_params)
        for g, saved in zip(self.param_groups, sd["param_groups"]):
            for k, v in saved.items():
                if k != "params":
                    g[k] = v
        for owned, opt in zip(self._owned, self.local):
            if opt is None:
                continue
            local_state = {}
            params = [q for *_, q in owned]
            for i, (kind, idx, start, proxy) in enumerate(owned):
                entry = sd["state"].get(idx if kind == "muon" else nm + idx)
                if entry is None:
                    continue
                if kind == "muon":
                    local_state[i] = dict(entry)
                else:
                    n = proxy.numel()
                    local_state[i] = {k: (v.reshape(-1)[start:start + n].clone() if torch.is_tensor(v) and v.dim() > 0 else v)
                                      for k, v in entry.items()}
            base = opt.state_dict()["param_groups"]
            # the local optimizer numbers its parameters 0.. in the order of `owned`
            opt.load_state_dict({"state": local_state, "param_groups": base})
