"""MonarchMuonOptimizer for B200: the reference optimizer's API over CUDA kernels.

Drop-in for the reference class of the same name
(pretrain/src/models/monarch/monarch_muon.py:57-201; bf16 twin in
membench/src/models/monarch/monarch_muon.py): same constructor, same two
param groups (`update_type` "muon" for the 3-D Monarch factors, "adamw" for
everything else), `group["lr"]` read at call time so LR schedulers work,
parameters without a gradient skipped, state created lazily on the first
step, standard `state_dict` / `load_state_dict` / step hooks.

What differs is where the arithmetic runs.  Muon tensors of one block shape are
worked through in slices (runs of consecutive tensors); per slice:

  1. one fused momentum kernel (heavy ball + optional FP8 state codec + bf16
     copy for Newton-Schulz + per-block sums of squares);
  2. per <= `ns_max_batch` blocks, 15 tcgen05 GEMM launches (5 x Gram / Poly /
     Apply) on that bf16 stack - the reference's torch.cat is gone because the
     blocks of a slice already lie back to back - the last of which applies
     W <- W - lr*sqrt(rows/cols)*O in its epilogue, so the orthogonalised blocks
     are never written to memory and no separate update kernel runs.

AdamW is one launch per <= 128 tensors.

Memory.  The persistent Muon state is what the format says and nothing more:
E4M3 codes (1 byte per element) plus per-group side arrays, or the
parameter-dtype buffer like the reference.  The bf16 stack that feeds
Newton-Schulz is scratch for one slice (at most `momentum_slice_elems`
elements, 1.48 GB by default) drawn from a pool shared by all optimizers of a
device and stream; with bf16 parameters in the reference's own format the
state is itself that stack and no scratch is needed.

There is no CPU path: tensors must live on a CUDA device.
"""
from __future__ import annotations

from collections import OrderedDict

import torch

from . import _lib, fp8_state
from .newton_schulz import newton_schulz_batched, newton_schulz_update, scratch_bf16

_STATE_FORMATS = ("param", "fp8_absmax", "fp8_expand")


class _ShapeGroup:
    """All Muon tensors of one (dtype, rows, cols), their arena slices and tables."""

    def __init__(self, dtype, rows, cols):
        self.dtype, self.rows, self.cols = dtype, rows, cols
        self.params: list = []
        self.block_start: list[int] = []      # first block of each tensor inside the group's state arrays
        self.nblocks = 0
        self.bf16_state = None                # bf16 [nblocks, rows, cols] when the state is itself the NS input
        self.first_block_global = 0           # index of the group's first block in block_sumsq


class MonarchMuonOptimizer(torch.optim.Optimizer):
    """Muon (batched Newton-Schulz on 3-D Monarch factors) + AdamW in one optimizer.

    Parameters (reference signature, monarch_muon.py:78-90)
    ----------
    muon_params, adamw_params : iterables of parameters
    lr, momentum, adamw_betas, adamw_weight_decay, adamw_eps : as upstream

    Extra keyword-only knobs (defaults reproduce the reference's behaviour)
    ----------
    state_format : "param" keeps `momentum_buffer` in the parameter dtype like
        the reference; "fp8_absmax" / "fp8_expand" store it as E4M3 codes with
        per-128-group side arrays (absmax scale, or COAT range expansion).
    fp8_div : arithmetic of the FP8 quantiser (MMB_DIV_* in the header).  "full" (default) uses the GPU
        instructions the reference's Triton kernels compile to, so FP8 absmax codes and scales equal the
        reference kernel's bit for bit on the same GPU; "ieee" uses IEEE division and equals the CPU
        oracle bit for bit (and, for the range-expansion format, forms powers on the special-function
        unit: faster, about one code in 10^4 differs); "ieee_strict" is "ieee" through the compiler's
        division and the library powf everywhere.
    ns_backend : "tcgen05" (tensor cores) or "simt" (cross-check kernel).
    ns_max_batch : slice Newton-Schulz into at most this many blocks per call
        to bound its workspace.
    fuse_update : (on by default) apply the weight update in the epilogue of the last Newton-Schulz GEMM.
        Off: Newton-Schulz writes the orthogonalised slice to a second scratch stack and a separate kernel
        updates the weights (same bits either way; kept for measurement).
    momentum_slice_elems : elements of one momentum launch, i.e. of the bf16
        scratch stack between the momentum kernel and Newton-Schulz (default
        704 Mi elements = 1.48 GB; never fewer than `ns_max_batch` blocks).  Gradients fed from host memory are always
        pipelined in slices of `ns_max_batch` blocks.
    overlap : (off by default) run the bandwidth-bound kernels (momentum of the next slice, weight
        update of the previous one, AdamW) on a second stream beside the
        tensor-bound Newton-Schulz of the current slice.  Same kernels on the
        same data, so results do not change.  Not used when gradients are fed
        from host memory (that path pipelines the copies instead).  Measured on a
        power-capped B200: 59.7 ms against 60.6 ms per step.
    """

    def __init__(self, muon_params, adamw_params, *, lr: float = 5e-3, momentum: float = 0.95,
                 adamw_betas: tuple[float, float] = (0.9, 0.95), adamw_weight_decay: float = 0.1,
                 adamw_eps: float = 1e-8, state_format: str = "param", fp8_div: str = "full",
                 ns_backend: str = "tcgen05", ns_max_batch: int | None = 256, expand_min: int = 16,
                 overlap: bool = False, momentum_slice_elems: int = 704 << 20, fuse_update: bool = True):
        if state_format not in _STATE_FORMATS:
            raise ValueError(f"state_format must be one of {_STATE_FORMATS}")
        muon_params = list(muon_params)
        adamw_params = list(adamw_params)
        defaults = dict(lr=lr)
        param_groups = [
            {"params": muon_params, "update_type": "muon", "momentum": momentum},
            {"params": adamw_params, "update_type": "adamw", "betas": adamw_betas,
             "weight_decay": adamw_weight_decay, "eps": adamw_eps},
        ]
        super().__init__(param_groups, defaults)
        self.state_format = state_format
        self.fp8_div = _lib.DIV_NAMES[fp8_div]
        self.ns_backend = {"tcgen05": _lib.NS_TCGEN05, "simt": _lib.NS_SIMT}[ns_backend]
        self.ns_max_batch = ns_max_batch
        self.momentum_slice_elems = int(momentum_slice_elems)
        self.fuse_update = bool(fuse_update)
        self.expand_min = expand_min
        self.grad_scale = 1.0            # multiplies Muon gradients inside the momentum kernel
        self._plans: dict = {}           # id(group) -> plan
        self._marks = None               # list of (phase, begin event, end event) while phase timing is on
        self._open: dict = {}            # stream -> event that opened the current span
        self._clip_scratch = self._clip_out = None
        self._clip_pending = False       # clip_grad_norm_ was called: the next step scales gradients on the device
        self._host = None                # {id(param): host gradient} during a step fed from host memory
        self._copy_streams: dict = {}
        self.overlap = overlap
        self._side_streams: dict = {}
        self._deferred: list = []        # AdamW groups to be stepped beside Newton-Schulz in this step
        _lib.load()                      # fail now, not at the first step, if the library is missing

    # ------------------------------------------------------------------ public
    @torch.no_grad()
    def step(self, closure=None, *, host_grads=None):
        """One optimizer step.

        host_grads (extension): a sequence parallel to all parameters (Muon group
        first, then AdamW, `None` entries allowed) or a dict {parameter: tensor}
        of gradients in (pinned) host memory.  They are copied to the device
        slice by slice on a side stream while earlier slices are already being
        stepped, instead of being staged in full before the step starts.
        """
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        self._host = self._host_map(host_grads)
        if self._clip_pending:
            _lib.load().mmb_set_device_grad_scale(self._clip_out[1:].data_ptr())
        try:
            groups = list(self.param_groups)
            overlapping = self.overlap and self._host is None
            if overlapping:
                # AdamW groups are stepped on the side stream while the first slice is in Newton-Schulz
                muon = [g for g in groups if g["update_type"] == "muon" and any(p.grad is not None for p in g["params"])]
                if muon:
                    self._deferred = [g for g in groups if g["update_type"] != "muon"]
                    groups = [g for g in groups if g["update_type"] == "muon"]
            for group in groups:
                lr = group["lr"]
                if group["update_type"] == "muon":
                    self._muon_step(group, lr, overlapping)
                else:
                    self._adamw_step(group, lr)
            for group in self._deferred:              # no Muon slice picked them up
                self._adamw_step(group, group["lr"])
            self._deferred = []
        finally:
            self._deferred = []
            if self._clip_pending:
                _lib.load().mmb_set_device_grad_scale(None)
                self._clip_pending = False
            if self._host is not None:
                for plan in self._plans.values():          # events belong to this step only
                    if plan is not None:
                        for sls in plan["slices"].values():
                            for sl in sls:
                                sl["event"] = None
            self._host = None
        return loss

    def _host_map(self, host_grads):
        if host_grads is None:
            return None
        if isinstance(host_grads, dict):
            return {id(p): g for p, g in host_grads.items() if g is not None}
        params = [p for g in self.param_groups for p in g["params"]]
        host_grads = list(host_grads)
        if len(host_grads) != len(params):
            raise ValueError("host_grads must have one entry per parameter")
        return {id(p): g for p, g in zip(params, host_grads) if g is not None}

    # Phase timing: CUDA events on the current stream at phase boundaries.
    def enable_phase_timing(self, on: bool = True) -> None:
        self._marks = [] if on else None
        self._open = {}

    def _mark(self, phase: str) -> None:
        """"begin" opens a span on the current stream, any other name closes it under that name.  Spans
        of different streams may overlap in time; each is the device time of its own phase."""
        if self._marks is not None:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            key = torch.cuda.current_stream().cuda_stream
            if phase == "begin":
                self._open[key] = ev
            else:
                e0 = self._open.get(key)
                if e0 is not None:
                    self._marks.append((phase, e0, ev))
                self._open[key] = ev                     # consecutive phases share a boundary

    def check_device_status(self) -> None:
        """Raise if a kernel of this library reported an expired bounded wait since the last check (the
        Newton-Schulz GEMMs give up a hand-off that never comes, store a code and return; their output is
        then incomplete).  Synchronises the current stream of every device that holds Muon parameters.
        Called by state_dict() and phase_times_ms(), i.e. where the caller synchronises anyway."""
        for plan in self._plans.values():
            if plan is None:
                continue
            code = _lib.read_status(plan["device"])
            if code != 0:
                what = _lib.STATUS_NAMES.get(code, "unknown code")
                raise RuntimeError(f"monarch_muon_b200: a kernel gave up a bounded wait (status {code:#x}: {what}); "
                                   "the weights written by that step are incomplete")

    def state_dict(self):
        self.check_device_status()
        return super().state_dict()

    def phase_times_ms(self) -> dict:
        """Milliseconds per phase accumulated since phase timing was enabled
        (call after a synchronise); clears the recorded events."""
        self.check_device_status()
        out: dict = {}
        for name, e0, e1 in (self._marks or []):
            out[name] = out.get(name, 0.0) + e0.elapsed_time(e1)
        if self._marks is not None:
            self._marks = []
            self._open = {}
        return out

    @torch.no_grad()
    def clip_grad_norm_(self, max_norm: float) -> torch.Tensor:
        """Global-norm gradient clipping fused into the next step().

        Counterpart of torch.nn.utils.clip_grad_norm_(params, max_norm) as the reference's loop calls it
        right before step() (pretrain/src/optim/base.py:121-123), without its host synchronisation and
        without rewriting the gradients: one kernel pass computes the norm of all current gradients and
        the clip coefficient min(1, max_norm / (norm + 1e-6)) on the device, and the next step() multiplies
        every gradient by it as it is read.  Returns the total norm as a 0-dim device tensor."""
        grads = [p.grad for g in self.param_groups for p in g["params"] if p.grad is not None]
        if not grads:
            return torch.zeros((), device="cuda")
        _lib.require_cuda(*grads)
        dev = grads[0].device
        lib = _lib.load()
        segs = (_lib.GradSeg * len(grads))()
        keep = []
        for k, g in enumerate(sorted(grads, key=lambda t: str(t.dtype))):    # one table run per dtype
            if not g.is_contiguous():
                g = g.contiguous()
                keep.append(g)
            segs[k].grad = g.data_ptr()
            segs[k].numel = g.numel()
            segs[k].dtype = _lib.dtype_code(g.dtype)
        with torch.cuda.device(dev):
            need = int(lib.mmb_grad_norm_scratch_floats())
            if self._clip_scratch is None or self._clip_scratch.numel() < need or self._clip_scratch.device != dev:
                self._clip_scratch = torch.empty(need, dtype=torch.float32, device=dev)
                self._clip_out = torch.empty(2, dtype=torch.float32, device=dev)
            _lib.check(lib.mmb_grad_norm_clip(segs, len(grads), float(max_norm), self._clip_out.data_ptr(),
                                              self._clip_scratch.data_ptr(), need, _lib.stream_ptr()), "grad_norm_clip")
        self._clip_pending = True
        return self._clip_out[0]

    def block_sumsq(self, group_index: int = 0):
        """fp32 sums of squares of bf16(momentum) per block from the last step (device tensor)."""
        plan = self._plans.get(id(self.param_groups[group_index]))
        return None if plan is None else plan["block_sumsq"]

    # ------------------------------------------------------------ Muon: plan
    def _fp8(self) -> bool:
        return self.state_format != "param"

    def _build_plan(self, group):
        params = group["params"]
        if not params:
            return None
        dev = params[0].device
        shapes: "OrderedDict[tuple, _ShapeGroup]" = OrderedDict()
        for p in params:
            _lib.require_cuda(p)
            if p.dim() not in (2, 3):
                raise ValueError("Muon parameters must be 3-D (nblocks, rows, cols) Monarch factors "
                                 "or 2-D matrices (treated as one block)")
            if p.device != dev:
                raise ValueError("all Muon parameters must live on one device")
            _lib.dtype_code(p.dtype)
            nb, rows, cols = self._blocks_of(p)
            key = (p.dtype, rows, cols)
            sg = shapes.get(key)
            if sg is None:
                sg = shapes[key] = _ShapeGroup(*key)
            sg.params.append(p)
            sg.block_start.append(sg.nblocks)
            sg.nblocks += nb
        plan = {"device": dev, "shapes": shapes, "params": list(params), "entry": {}}
        total_blocks = 0
        for sg in shapes.values():
            sg.first_block_global = total_blocks
            total_blocks += sg.nblocks
            sg.fp32_state = None
            sg.codes = sg.scale = sg.expand = sg.sqrt_mm = None
            if self.state_format == "param" and sg.dtype == torch.bfloat16:
                # the reference's own format with bf16 parameters: the state is the Newton-Schulz input
                sg.bf16_state = torch.zeros(sg.nblocks, sg.rows, sg.cols, dtype=torch.bfloat16, device=dev)
            elif self.state_format == "param":
                sg.fp32_state = torch.zeros(sg.nblocks, sg.rows, sg.cols, dtype=torch.float32, device=dev)
            else:
                sg.codes = torch.zeros(sg.nblocks, sg.rows, sg.cols, dtype=torch.uint8, device=dev)
                ngroups = sum(fp8_state.groups_of(p.numel()) for p in sg.params)
                sg.scale = torch.zeros(ngroups, dtype=torch.float32, device=dev)
                if self.state_format == "fp8_expand":
                    sg.expand = torch.ones(ngroups, dtype=torch.float32, device=dev)
                    sg.sqrt_mm = torch.ones(ngroups, dtype=torch.float32, device=dev)
            g_at = 0
            for p, b0 in zip(sg.params, sg.block_start):
                nb = self._blocks_of(p)[0]
                ng = fp8_state.groups_of(p.numel())
                views = {}
                if self._fp8():
                    state_t = sg.codes[b0:b0 + nb].view(p.shape)
                    views["momentum_buffer"] = state_t.view(torch.float8_e4m3fn)
                    views["scale_momentum_buffer"] = sg.scale[g_at:g_at + ng]
                    if sg.expand is not None:
                        views["expand_momentum_buffer"] = sg.expand[g_at:g_at + ng]
                        views["sqrt_minmax_momentum_buffer"] = sg.sqrt_mm[g_at:g_at + ng]
                elif sg.fp32_state is not None:
                    state_t = sg.fp32_state[b0:b0 + nb].view(p.shape)
                    views["momentum_buffer"] = state_t
                else:
                    state_t = sg.bf16_state[b0:b0 + nb].view(p.shape)
                    views["momentum_buffer"] = state_t
                plan["entry"][id(p)] = (state_t, sg, b0, views)
                g_at += ng
        plan["block_sumsq"] = torch.zeros(total_blocks, dtype=torch.float32, device=dev)
        plan["scratch"] = None
        plan["slices"] = {}
        return plan

    @staticmethod
    def _blocks_of(p):
        """(nblocks, rows, cols) of a Muon parameter; a 2-D matrix is one block (the reference's
        fine-tuning optimizer applies the same update to dense matrices, finetune/sft_optimizer.py:40-50)."""
        return (p.shape[0], p.shape[1], p.shape[2]) if p.dim() == 3 else (1, p.shape[0], p.shape[1])

    def _plan_for(self, group):
        plan = self._plans.get(id(group))
        if plan is None or len(plan["params"]) != len(group["params"]) or \
                any(a is not b for a, b in zip(plan["params"], group["params"])):
            plan = self._build_plan(group)
            self._plans[id(group)] = plan
        return plan

    def _state_code(self, sg) -> int:
        if self.state_format == "fp8_absmax":
            return _lib.STATE_FP8_ABSMAX
        if self.state_format == "fp8_expand":
            return _lib.STATE_FP8_EXPAND
        return _lib.STATE_BF16 if sg.dtype == torch.bfloat16 else _lib.STATE_F32

    # ------------------------------------------------------------ Muon: step
    def _slices_for(self, plan, live, host_fed: bool):
        """Cut the live tensors into slices: runs of consecutive tensors of one block shape.  A slice is
        the unit of one momentum launch (and of host-to-device pipelining); its blocks go through
        Newton-Schulz in sub-slices of at most `ns_max_batch` blocks.  Cached per set of live tensors."""
        key = (tuple(id(p) for p in live), host_fed)
        cached = plan["slices"].get(key)
        if cached is not None:
            return cached
        live_ids = set(key[0])
        ns_cap = self.ns_max_batch or (1 << 30)
        slices = []
        for sg in plan["shapes"].values():
            blk = sg.rows * sg.cols
            # host-fed gradients: small slices, so that the first copy is short and the last compute is too
            cap = ns_cap if host_fed else max(ns_cap, self.momentum_slice_elems // blk)
            cur = None
            for p, b0 in zip(sg.params, sg.block_start):
                if id(p) not in live_ids:
                    cur = None
                    continue
                nb = self._blocks_of(p)[0]
                if cur is None or cur["b1"] - cur["b0"] + nb > cap:
                    cur = {"sg": sg, "items": [], "b0": b0, "b1": b0, "tables": {}, "event": None, "sub": None,
                           "index": len(slices)}
                    slices.append(cur)
                cur["items"].append((p, b0))
                cur["b1"] = b0 + nb
        plan["slices"][key] = slices
        return slices

    def _muon_step(self, group, lr: float, overlapping: bool = False) -> None:
        host = self._host
        # fed from the host, only the parameters named there step (a device buffer left over from an
        # earlier step is not a gradient of this one)
        live = [p for p in group["params"] if (id(p) in host if host is not None else p.grad is not None)]
        if not live:
            return
        plan = self._plan_for(group)
        dev = plan["device"]
        with torch.cuda.device(dev):
            slices = self._slices_for(plan, live, host is not None)
            if overlapping and host is None:
                self._muon_slices_overlapped(group, lr, plan, slices)
                return
            self._mark("begin")
            if host is not None:
                self._enqueue_host_copies(slices, host, dev)
            for sl in slices:
                if sl["event"] is not None:
                    torch.cuda.current_stream().wait_event(sl["event"])
                stack = self._slice_momentum(group, plan, sl, "m0")
                self._mark("momentum")
                self._slice_newton_schulz_update(plan, sl, stack, lr)
                self._mark("newton_schulz")

    def _muon_slices_overlapped(self, group, lr: float, plan, slices) -> None:
        """Two streams: Newton-Schulz (with its fused update) of slice k on the caller's stream; momentum
        of slice k+1 and (once) the AdamW groups on a side stream.  Newton-Schulz is tensor bound and the
        others are bandwidth bound, so they share the chip: the side-stream kernels are launched as one
        small CTA per SM (128 threads, at most 64 registers, no shared memory), which fits on an SM beside
        a GEMM CTA, so the GEMMs keep every SM.  The side stream has high priority: the GEMMs are launched
        ahead of time (programmatic serialisation), and a pending GEMM grid that cannot be placed yet would
        otherwise hold up the placement of a kernel queued behind it.  The first slice's momentum has
        nothing to hide behind and runs with full grids.  The bf16 stacks of consecutive slices alternate
        between two scratch buffers."""
        dev = plan["device"]
        main = torch.cuda.current_stream()
        side = self._side_streams.get(dev)
        if side is None:
            side = self._side_streams[dev] = torch.cuda.Stream(device=dev, priority=-1)
        shared = _lib.launch_options(stream_ctas_per_sm=1)
        with _lib.launch_options(dynamic_schedule=True):   # pairs that share their SMs draw fewer tiles
            side.wait_stream(main)                      # gradients and last step's weights are ready
            n = len(slices)
            mom_done = [torch.cuda.Event() for _ in range(n)]
            ns_done = [torch.cuda.Event() for _ in range(n)]
            stacks = [None] * n
            # the scratch pool is keyed by stream: draw both buffers on the caller's stream
            tags = ("m0", "m1")
            for k, sl in enumerate(slices):
                stacks[k] = self._slice_stack(plan, sl, tags[k & 1])
            with torch.cuda.stream(side):
                self._mark("begin")
                self._slice_momentum(group, plan, slices[0], tags[0], stack=stacks[0])
                self._mark("momentum")
                mom_done[0].record(side)
            for k, sl in enumerate(slices):
                with torch.cuda.stream(side), shared:
                    if k + 1 < n:
                        if k >= 1:
                            side.wait_event(ns_done[k - 1])    # the buffer of slice k+1 was slice k-1's
                        self._mark("begin")
                        self._slice_momentum(group, plan, slices[k + 1], tags[(k + 1) & 1], stack=stacks[k + 1])
                        self._mark("momentum")
                        mom_done[k + 1].record(side)
                    if k == 0:
                        deferred, self._deferred = self._deferred, []
                        for g in deferred:
                            self._adamw_step(g, g["lr"])
                main.wait_event(mom_done[k])
                self._mark("begin")
                self._slice_newton_schulz_update(plan, sl, stacks[k], lr)
                self._mark("newton_schulz")
                ns_done[k].record(main)
            main.wait_stream(side)

    def _slice_stack(self, plan, sl, tag: str):
        """The bf16 (blocks, rows, cols) stack Newton-Schulz reads for this slice: the state itself when
        that is a bf16 array, else scratch that the momentum kernel fills."""
        sg = sl["sg"]
        if sg.bf16_state is not None:
            return sg.bf16_state[sl["b0"]:sl["b1"]]
        nb = sl["b1"] - sl["b0"]
        flat = scratch_bf16(tag, nb * sg.rows * sg.cols, plan["device"])
        return flat.view(nb, sg.rows, sg.cols)

    def _slice_momentum(self, group, plan, sl, tag: str, stack=None):
        """Momentum (+codec, +bf16 copy, +block norms) of one slice; tables are cached, only gradient
        and scratch pointers change.  State is registered lazily, like _get_momentum_buffer
        (monarch_muon.py:133-137).  Returns the slice's bf16 stack."""
        sg = sl["sg"]
        dev = plan["device"]
        if stack is None:
            stack = self._slice_stack(plan, sl, tag)
        blk = sg.rows * sg.cols
        buckets: "OrderedDict[tuple, list]" = OrderedDict()
        keep = []
        for p, pb0 in sl["items"]:
            st = self.state[p]
            state_t, _, _, views = plan["entry"][id(p)]
            if "momentum_buffer" not in st:
                st.update(views)
            g = p.grad
            if g.shape != p.shape:
                raise ValueError("gradient shape differs from its parameter")
            if not g.is_contiguous():
                g = g.contiguous()
                keep.append(g)
            buckets.setdefault(g.dtype, []).append((p, pb0, state_t, views, g))
        scode = self._state_code(sg)
        for gdtype, items in buckets.items():
            cached = sl["tables"].get(gdtype)
            if cached is None or cached[2] != len(items):
                segs = (_lib.MomentumSeg * len(items))()
                for k, (p, pb0, state_t, views, g) in enumerate(items):
                    sgm = segs[k]
                    sgm.state = state_t.data_ptr()
                    sgm.scale = _lib.ptr(views.get("scale_momentum_buffer"))
                    sgm.expand = _lib.ptr(views.get("expand_momentum_buffer"))
                    sgm.sqrt_minmax = _lib.ptr(views.get("sqrt_minmax_momentum_buffer"))
                    sgm.numel = p.numel()
                    sgm.block_elems = blk
                    sgm.first_block = sg.first_block_global + pb0
                cached = sl["tables"][gdtype] = (segs, None, len(items))
            segs = cached[0]
            for k, (p, pb0, state_t, views, g) in enumerate(items):
                segs[k].grad = g.data_ptr()
                segs[k].m_bf16 = stack[pb0 - sl["b0"]:].data_ptr()       # scratch may move between steps
            need = cached[1]
            if need is None:
                need = fp8_state.scratch_floats(segs, len(items))
                sl["tables"][gdtype] = (segs, need, len(items))
            if plan["scratch"] is None or plan["scratch"].numel() < need:
                plan["scratch"] = torch.empty(need, dtype=torch.float32, device=dev)
            fp8_state.momentum_step(segs, len(items), grad_dtype=gdtype, state_format=scode,
                                    beta=group["momentum"], grad_scale=self.grad_scale,
                                    div_mode=self.fp8_div, expand_min=self.expand_min,
                                    block_sumsq=plan["block_sumsq"], scratch=plan["scratch"])
        return stack

    def _slice_subslices(self, sl):
        """Newton-Schulz sub-slices of a slice: (first block, last block) inside the slice and the device
        table of weight addresses, one per block.  The table is rebuilt when a parameter's storage moved."""
        sg = sl["sg"]
        bases = tuple(p.data.data_ptr() for p, _ in sl["items"])
        sub = sl["sub"]
        if sub is not None and sub["bases"] == bases:
            return sub["parts"]
        esz = 2 if sg.dtype == torch.bfloat16 else 4
        blk_bytes = sg.rows * sg.cols * esz
        ptrs = []
        for (p, _), base in zip(sl["items"], bases):
            if not p.data.is_contiguous():
                raise ValueError("Muon parameters must be contiguous")
            if base % 16 or blk_bytes % 16:
                raise ValueError("Muon parameters must be 16-byte aligned")
            ptrs += [base + k * blk_bytes for k in range(self._blocks_of(p)[0])]
        table = torch.tensor(ptrs, dtype=torch.int64).to(sg.params[0].device, non_blocking=False)
        cap = self.ns_max_batch or len(ptrs)
        parts = [(a, min(a + cap, len(ptrs)), table[a:min(a + cap, len(ptrs))]) for a in range(0, len(ptrs), cap)]
        sl["sub"] = {"bases": bases, "parts": parts}
        return parts

    def _slice_newton_schulz_update(self, plan, sl, stack, lr: float) -> None:
        """W <- W - lr*sqrt(rows/cols)*NS(momentum) for the tensors of one slice, the update fused into
        the last GEMM's epilogue (monarch_muon.py:157-165)."""
        sg = sl["sg"]
        alpha = -lr * (sg.rows / sg.cols) ** 0.5
        first = sg.first_block_global + sl["b0"]
        if self.fuse_update:
            for a, b, table in self._slice_subslices(sl):
                newton_schulz_update(stack[a:b], table, sg.dtype, alpha,
                                     block_sumsq=plan["block_sumsq"][first + a:first + b], backend=self.ns_backend)
            return
        nb = sl["b1"] - sl["b0"]
        ortho = scratch_bf16("ortho", nb * sg.rows * sg.cols, plan["device"]).view(nb, sg.rows, sg.cols)
        cap = self.ns_max_batch or nb
        for a in range(0, nb, cap):
            b = min(a + cap, nb)
            newton_schulz_batched(stack[a:b], out=ortho[a:b], block_sumsq=plan["block_sumsq"][first + a:first + b],
                                  backend=self.ns_backend)
        self._mark("newton_schulz")
        segs = (_lib.UpdateSeg * len(sl["items"]))()
        for k, (p, pb0) in enumerate(sl["items"]):
            if not p.data.is_contiguous():
                raise ValueError("Muon parameters must be contiguous")
            segs[k].weight = p.data.data_ptr()
            segs[k].ortho = ortho[pb0 - sl["b0"]:].data_ptr()
            segs[k].numel = p.numel()
        _lib.check(_lib.load().mmb_muon_update(segs, len(sl["items"]), _lib.dtype_code(sg.dtype), alpha,
                                               _lib.stream_ptr()), "muon_update")
        self._mark("update")

    # ------------------------------------------------- gradients from the host
    def _copy_stream(self, dev):
        st = self._copy_streams.get(dev)
        if st is None:
            st = self._copy_streams[dev] = torch.cuda.Stream(device=dev)
        return st

    def _device_grad(self, p, h):
        if h.shape != p.shape:
            raise ValueError("host gradient shape differs from its parameter")
        if p.grad is None or p.grad.dtype != h.dtype or not p.grad.is_contiguous():
            p.grad = torch.empty(p.shape, dtype=h.dtype, device=p.device)
        return p.grad

    def _enqueue_host_copies(self, slices, host, dev):
        """Queue every slice's host-to-device gradient copies on a side stream, one event per slice, so
        the copy of slice i+1 runs while slice i is being computed."""
        cs = self._copy_stream(dev)
        cs.wait_stream(torch.cuda.current_stream())     # last step's kernels are done with the buffers
        with torch.cuda.stream(cs):
            for sl in slices:
                for p, _ in sl["items"]:
                    h = host.get(id(p))
                    if h is not None:
                        self._device_grad(p, h).copy_(h, non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(cs)
                sl["event"] = ev

    # ----------------------------------------------------------------- AdamW
    def _adamw_new_state(self, p, state) -> None:
        """Lazy state of one AdamW parameter (monarch_muon.py:181-185)."""
        state["step"] = 0
        state["exp_avg"] = torch.zeros_like(p, memory_format=torch.contiguous_format)
        state["exp_avg_sq"] = torch.zeros_like(p, memory_format=torch.contiguous_format)

    def _adamw_collect(self, group):
        """Parameters of the AdamW group that step now, by dtype: (parameter, gradient, state) with the
        state created and its step count already incremented; host-fed gradients are copied in first."""
        by_dtype: "OrderedDict[torch.dtype, list]" = OrderedDict()
        host = self._host
        if host is not None:
            fed = [p for p in group["params"] if id(p) in host]
            if fed:
                dev = fed[0].device
                _lib.require_cuda(fed[0])
                with torch.cuda.device(dev):
                    cs = self._copy_stream(dev)
                    with torch.cuda.stream(cs):
                        for p in fed:
                            self._device_grad(p, host[id(p)]).copy_(host[id(p)], non_blocking=True)
                    torch.cuda.current_stream().wait_stream(cs)
        for p in group["params"]:
            if p.grad is None or (host is not None and id(p) not in host):
                continue
            _lib.require_cuda(p)
            state = self.state[p]
            if len(state) == 0:
                self._adamw_new_state(p, state)
            state["step"] += 1
            g = p.grad
            if g.dtype != p.dtype:
                g = g.to(p.dtype)
            if not g.is_contiguous():
                g = g.contiguous()
            if not p.data.is_contiguous():
                raise ValueError("AdamW parameters must be contiguous")
            by_dtype.setdefault(p.dtype, []).append((p, g, state))
        return by_dtype

    def _adamw_step(self, group, lr: float) -> None:
        beta1, beta2 = group["betas"]
        by_dtype = self._adamw_collect(group)
        if not by_dtype:
            return
        lib = _lib.load()
        self._mark("begin")
        for dtype, items in by_dtype.items():
            segs = (_lib.AdamWSeg * len(items))()
            for k, (p, g, state) in enumerate(items):
                segs[k].param = p.data.data_ptr()
                segs[k].grad = g.data_ptr()
                segs[k].exp_avg = state["exp_avg"].data_ptr()
                segs[k].exp_avg_sq = state["exp_avg_sq"].data_ptr()
                segs[k].numel = p.numel()
                segs[k].step = state["step"]
            with torch.cuda.device(items[0][0].device):
                _lib.check(lib.mmb_adamw_step(segs, len(items), _lib.dtype_code(dtype), lr, beta1, beta2,
                                              group["weight_decay"], group["eps"], _lib.stream_ptr()), "adamw_step")
        self._mark("adamw")

    # ----------------------------------------------------------- checkpoints
    _MANAGED = ("momentum_buffer", "scale_momentum_buffer", "expand_momentum_buffer",
                "sqrt_minmax_momentum_buffer")

    def load_state_dict(self, state_dict):
        """Restore a reference-shaped state dict.  torch casts floating state to
        the parameter dtype, which would squash fp32 scale arrays and FP8 codes
        (coat_state_muon.py:141-151 works around the same thing), so the Muon
        state is taken out first and copied into the arenas afterwards."""
        saved_ids = [i for g in state_dict["param_groups"] for i in g["params"]]
        params = [p for g in self.param_groups for p in g["params"]]
        if len(saved_ids) != len(params):
            raise ValueError("loaded state dict has a different number of parameters")
        stripped_state = {}
        managed = {}
        for pid, entry in state_dict["state"].items():
            keep = {k: v for k, v in entry.items() if k not in self._MANAGED}
            mine = {k: v for k, v in entry.items() if k in self._MANAGED}
            if keep:
                stripped_state[pid] = keep
            if mine:
                managed[pid] = mine
        super().load_state_dict({"state": stripped_state, "param_groups": state_dict["param_groups"]})
        by_id = dict(zip(saved_ids, params))
        muon_group = self.param_groups[0]
        plan = self._plan_for(muon_group) if muon_group["params"] else None
        for pid, mine in managed.items():
            p = by_id[pid]
            _, _, _, views = plan["entry"][id(p)]
            buf = mine.get("momentum_buffer")
            if self._fp8() and buf is not None and buf.dtype != torch.float8_e4m3fn:
                # a checkpoint written with plain (bf16/fp32) momentum, loaded into FP8 state: quantise it
                tmp = {}
                fp8_state.quantize_(tmp, "momentum_buffer", buf.to(p.device, torch.float32), True, torch.float8_e4m3fn,
                                    self.expand_min, codec="expand" if self.state_format == "fp8_expand" else "absmax",
                                    div_mode=self.fp8_div)
                mine = tmp
            for k, v in mine.items():
                if k not in views:
                    raise ValueError(f"state '{k}' does not fit state_format={self.state_format}")
                dst = views[k]
                src = v.to(dst.device)
                if dst.dtype == torch.float8_e4m3fn:
                    src = src.to(torch.float8_e4m3fn) if src.dtype != torch.float8_e4m3fn else src
                    dst.view(torch.uint8).copy_(src.view(torch.uint8).reshape(dst.shape))
                else:
                    dst.copy_(src.to(dst.dtype).reshape(dst.shape))
            self.state[p].update(views)
