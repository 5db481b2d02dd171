#!/usr/bin/env python
"""Benchmark of the Monarch-Muon optimizer step on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--nblocks 4]

Workload (N = 1): the full optimizer step at the 6.89B-dense-reference size
with 4-block Monarch factors: 448 Muon tensors (1408 blocks 1024x1024, 256
blocks 2752x1024, 128 blocks 1024x2752 = 2,558,525,440 elements) with FP8
(E4M3 absmax) momentum state, batched Newton-Schulz and the weight update, plus
the AdamW group (embedding, LM head, 65 norm vectors; vocab 50257).  Weights
N(0, 0.02) and gradients N(0, 1e-3) are seeded synthetic bf16 tensors - there is
no dataset on this path.

One JSON line is printed by rank 0.  `value` is device-timed milliseconds per
step with gradients already in HBM; `e2e` repeats the measurement through the
public `optimizer.step()` with every gradient copied from pinned host memory
inside the timed region and the per-block momentum norms read back.

The default line also carries, each with its own clock sample: the two isolated
kernels of the metric (`isolated_ns`: 128 + 64 + 64 blocks; `isolated_fp8_*`:
1.6e9 and 2,558,525,440 elements), the reference's own GPU step on the same
workload (`reference_gpu`), the 2-block model's step (`nblocks2_step`), and
`peak_memory_gb` / `optimizer_state_gb`.

`--impl reference` times the reference's own optimizer class (the staged copy
under oracle/_ref/; the oracle's restatement if that copy is absent) on all
host threads, on a bounded sample of blocks scaled to the full step by block and
element counts; `--reference-device cuda` runs that class on the GPU instead.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from monarch_muon_b200 import shapes as S  # noqa: E402

METRIC = "monarch_muon_opt_step_ms_6.89B_ref_nb4"
H100_PUBLISHED_MS = 304.4      # README.md:16 of the reference, one H100, bf16 state


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=p["hbm_gbs"], bf16_tflops=p["bf16_tflops"],
                    bf16_tflops_sustained=p.get("bf16_tflops_sustained", p["bf16_tflops"]), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


# ----------------------------------------------------------------- clock sampler
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.rows: list[list[str]] = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def stop(self, t_begin: float = 0.0, t_end: float = float("inf")) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons, watts = [], None, set(), []
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for ts, r in self.rows:
            if len(r) < 8 or ts < t_begin or ts > t_end + 0.15:
                continue
            try:
                sm.append(float(r[0]))
                smax = float(r[1])
                watts.append(float(r[2]))
            except ValueError:
                continue
            for name, v in zip(names, r[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": smax, "samples": len(sm),
                "power_w": statistics.median(watts) if watts else None, "reasons": sorted(reasons)}


# ------------------------------------------------------------------ the workload
def build_workload(device, nblocks: int, seed: int = 1234):
    """Parameters and gradients of the 6.89B-reference model's optimizer step."""
    gen = torch.Generator(device=device).manual_seed(seed)
    m = S.MODEL_689B
    muon_shapes = S.llama_monarch_muon_shapes(m["d_model"], m["n_layers"], m["intermediate"], nblocks)
    adamw_shapes = S.llama_adamw_shapes(m["d_model"], m["n_layers"], m["vocab"])
    muon, adamw = [], []
    for s in muon_shapes:
        w = torch.empty(s, dtype=torch.bfloat16, device=device).normal_(0.0, 0.02, generator=gen)
        muon.append(torch.nn.Parameter(w))
    for s in adamw_shapes:
        w = torch.empty(s, dtype=torch.bfloat16, device=device).normal_(0.0, 0.02, generator=gen)
        adamw.append(torch.nn.Parameter(w))
    for p in muon + adamw:
        p.grad = torch.empty_like(p).normal_(0.0, 1e-3, generator=gen)
    return muon, adamw


def workload_counts(nblocks: int):
    m = S.MODEL_689B
    shp = S.llama_monarch_muon_shapes(m["d_model"], m["n_layers"], m["intermediate"], nblocks)
    flops = sum(s[0] * S.ns_flops(s[1], s[2]) for s in shp)
    muon_elems = sum(s[0] * s[1] * s[2] for s in shp)
    adamw_elems = sum(int(torch.Size(s).numel()) for s in S.llama_adamw_shapes(m["d_model"], m["n_layers"], m["vocab"]))
    return flops, muon_elems, adamw_elems


# ------------------------------------------------------------------ CPU baseline
def _reference_twin():
    """The reference's own bf16 optimizer class (membench/src/models/monarch/monarch_muon.py, unmodified,
    from the staged copy under oracle/_ref/), or None when that copy is absent."""
    try:
        from oracle import ref_loader
        if ref_loader.available():
            return ref_loader.membench_twin().MonarchMuonOptimizer
    except Exception:                                          # a broken staging must not take the bench down
        pass
    return None


def cpu_reference_step_ms(nblocks: int, steps: int, warmup: int, threads: int | None = None):
    """The reference step (bf16 twin: bf16 state, bf16 Newton-Schulz) on the host cores, on a sample of
    blocks of every shape and a slice of the AdamW group, each part scaled linearly to the full step
    (blocks are independent, AdamW is element-wise).  Runs the reference's own class when oracle/_ref/
    holds it (kind "reference"), else the oracle's restatement of it (kind "port").
    Returns (ms per full step, description of the sample, threads, kind)."""
    threads = threads or os.cpu_count() or 1
    torch.set_num_threads(threads)
    m = S.MODEL_689B
    shp = S.llama_monarch_muon_shapes(m["d_model"], m["n_layers"], m["intermediate"], nblocks)
    full: dict = {}
    for nb, r, c in shp:
        full[(r, c)] = full.get((r, c), 0) + nb
    # the same fraction of every block shape (96 of the 1408 square blocks at nblocks=4)
    frac = 96.0 / max(full.values())
    sample = {k: max(1, int(round(v * frac))) for k, v in full.items()}
    gen = torch.Generator().manual_seed(7)
    _, _, adamw_elems = workload_counts(nblocks)
    a_n = 1 << 23
    twin = _reference_twin()
    kw = dict(lr=0.02, momentum=0.95, adamw_betas=(0.9, 0.95), adamw_weight_decay=0.1, adamw_eps=1e-8)
    parts = []                                                 # (callable, scale to the full step)
    if twin is not None:
        kind = "reference"
        for (r, c), nb in sample.items():
            # tensors of `nblocks` blocks each, like the model's factors
            ps = [torch.nn.Parameter((0.02 * torch.randn(nblocks, r, c, generator=gen)).bfloat16())
                  for _ in range(max(1, nb // nblocks))]
            for p in ps:
                p.grad = (1e-3 * torch.randn(p.shape, generator=gen)).bfloat16()
            sample[(r, c)] = len(ps) * nblocks
            opt = twin(ps, [], **kw)
            parts.append((opt.step, full[(r, c)] / sample[(r, c)]))
        ap = torch.nn.Parameter((0.02 * torch.randn(a_n, generator=gen)).bfloat16())
        ap.grad = (1e-3 * torch.randn(a_n, generator=gen)).bfloat16()
        aopt = twin([], [ap], **kw)
        parts.append((aopt.step, adamw_elems / a_n))
    else:
        kind = "port"
        from oracle import muon_oracle
        for (r, c), nb in sample.items():
            w = (0.02 * torch.randn(nb, r, c, generator=gen)).bfloat16()
            g = (1e-3 * torch.randn(nb, r, c, generator=gen)).bfloat16()
            buf = torch.zeros_like(w)
            parts.append((lambda w=w, g=g, buf=buf: muon_oracle.muon_group_step([w], [g], [buf], lr=0.02, beta=0.95,
                                                                                ns_dtype=torch.bfloat16),
                          full[(r, c)] / nb))
        ap = (0.02 * torch.randn(a_n, generator=gen)).bfloat16()
        ag = (1e-3 * torch.randn(a_n, generator=gen)).bfloat16()
        am, av = torch.zeros_like(ap), torch.zeros_like(ap)
        count = [0]

        def adamw_part():
            count[0] += 1
            muon_oracle.adamw_tensor_step(ap, ag, am, av, count[0], lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1, eps=1e-8)
        parts.append((adamw_part, adamw_elems / a_n))

    def one_pass() -> float:
        total = 0.0
        for fn, scale in parts:
            t0 = time.perf_counter()
            fn()
            total += (time.perf_counter() - t0) * scale
        return total * 1e3

    with torch.no_grad():
        for _ in range(warmup):
            one_pass()
        times = [one_pass() for _ in range(steps)]
    desc = (("the reference's own MonarchMuonOptimizer (membench twin, bf16) " if kind == "reference"
             else "restatement of the reference's bf16 step (momentum, cat, Newton-Schulz, update) ")
            + "on " + ", ".join(f"{nb} of {full[k]} blocks {k[0]}x{k[1]}" for k, nb in sample.items())
            + f"; AdamW on {a_n} of {adamw_elems} elements; each part scaled linearly to the full count; "
            + f"median of {len(times)} passes")
    return statistics.median(times), desc, threads, kind


def gpu_reference_step_ms(dev, nblocks: int, steps: int, warmup: int):
    """The reference's own GPU step: membench/src/models/monarch/monarch_muon.py's MonarchMuonOptimizer,
    unmodified (staged under oracle/_ref/), on the full workload with bf16 parameters, gradients and state,
    timed with CUDA events per step on a side stream as the reference's harness does
    (membench/scripts/monarch_benchmark/benchmark_train_step.py:297-310, 382-397).  Falls back to the
    oracle's torch-op restatement when the staged copy is absent.  Returns a dict."""
    torch.backends.cuda.matmul.allow_tf32 = True     # as the reference's harness sets it (:346)
    muon, adamw = build_workload(dev, nblocks)
    twin = _reference_twin()
    kw = dict(lr=0.02, momentum=0.95, adamw_betas=(0.9, 0.95), adamw_weight_decay=0.1, adamw_eps=1e-8)
    if twin is not None:
        opt = twin(muon, adamw, **kw)
        step, kind = opt.step, "reference"
    else:
        from oracle import muon_oracle
        ref = muon_oracle.OracleMonarchMuon([p.data for p in muon], [p.data for p in adamw], ns_dtype=torch.bfloat16,
                                            foreach_cpu=True, **kw)
        mg, ag = [p.grad for p in muon], [p.grad for p in adamw]
        step, kind = (lambda: ref.step(mg, ag)), "port"
    torch.cuda.reset_peak_memory_stats(dev)
    sampler = ClockSampler(dev.index or 0)
    sampler.start()
    side = torch.cuda.Stream(device=dev)
    side.wait_stream(torch.cuda.current_stream())
    times = []
    with torch.cuda.stream(side):
        for _ in range(max(3, warmup)):
            step()
        torch.cuda.synchronize()
        t_begin = time.time()
        for _ in range(steps):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            step()
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
        t_end = time.time()
    out = {"value": statistics.median(times), "unit": "ms", "kind": kind, "steps": steps,
           "min": min(times), "max": max(times), "state": "bf16 momentum and AdamW moments (the reference's format)",
           "peak_memory_gb": torch.cuda.max_memory_allocated(dev) / 1e9, "clocks": sampler.stop(t_begin, t_end)}
    del muon, adamw
    torch.cuda.empty_cache()
    return out


def gpu_reference_step(args, config) -> int:
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    r = gpu_reference_step_ms(dev, args.nblocks, args.steps, args.warmup)
    ms = r["value"]
    line = {"impl": "reference", "reference_device": "cuda", "metric": METRIC, "value": ms, "unit": "ms", "n_gpus": 1,
            "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms, "higher_is_better": False,
            "scaling": "strong", "vs_baseline": ms / H100_PUBLISHED_MS, "dtype": "bf16", "data": "synthetic",
            "config": dict(config, workload=config["workload"].replace("FP8 E4M3 absmax momentum state",
                                                                       "bf16 momentum state (the reference's)")),
            "note": ("the reference's own MonarchMuonOptimizer (membench twin) on the GPU" if r["kind"] == "reference" else
                     "torch-op restatement of the reference's bf16 step on the GPU") + ", full workload, gradients resident, "
                    "median of per-step CUDA-event times",
            "reference_kind": r["kind"], "peak_memory_gb": r["peak_memory_gb"], "clocks": r["clocks"], "gpu_launches": 0}
    print(json.dumps(line))
    return 0


# ------------------------------------------------------------------------- main
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--nblocks", type=int, default=4, choices=[2, 4])
    ap.add_argument("--case", default="step", choices=["step", "ns", "fp8", "gemm", "adamw", "guest"],
                    help="step: the full optimizer step (headline); ns: isolated batched Newton-Schulz on the "
                         "128+64+64 block set; fp8: isolated FP8 momentum kernel on a flat buffer; gemm: the library's "
                         "batched GEMM beside cuBLAS (torch.bmm) on the Newton-Schulz shapes, each run back to "
                         "back for seconds so that the power cap is in force; adamw: the AdamW kernel alone on a flat bf16 "
                         "tensor of --fp8-elems elements (FP8 moments with --state-format coat)")
    ap.add_argument("--ns-blocks", type=int, default=128, help="square blocks in --case ns (tall/wide get half each)")
    ap.add_argument("--ns-update", type=int, default=0, choices=[0, 1],
                    help="--case ns: apply the weight update in the last GEMM's epilogue (as the optimizer step does)")
    ap.add_argument("--fp8-elems", type=int, default=1_600_000_000)
    ap.add_argument("--comm-sms", type=int, default=-1,
                    help="SMs left to the communication kernels during the sharded step (-1: the transport's default)")
    ap.add_argument("--comm-ctas", type=int, default=-1,
                    help="CTAs of each multicast kernel in the sharded step (-1: one per SM)")
    ap.add_argument("--comm", default="auto", choices=["nccl", "multimem", "p2p", "auto"],
                    help="transport of the sharded step: NCCL collectives, this library's NVSwitch multicast kernels, "
                         "its peer load/store kernels, or auto (peer kernels on two GPUs, NCCL on more: what measured "
                         "fastest)")
    ap.add_argument("--chunks", type=int, default=4, help="pipeline chunks of the sharded (multi-GPU) step")
    ap.add_argument("--chunk-edge", type=float, default=0.5,
                    help="size of the first and last Muon chunk of the sharded step relative to the inner ones")
    ap.add_argument("--dynamic-schedule", type=int, default=None, choices=[0, 1],
                    help="Newton-Schulz GEMM tiles drawn from a counter (1) or fixed round-robin (0); default: 1 in "
                         "the sharded (multi-GPU) step, 0 on one GPU")
    ap.add_argument("--state-format", default="fp8_absmax", choices=["fp8_absmax", "fp8_expand", "param", "coat"],
                    help="momentum state: FP8 absmax (headline), COAT range expansion, or the parameter dtype")
    ap.add_argument("--ns-max-batch", type=int, default=256, help="blocks per Newton-Schulz slice")
    ap.add_argument("--reference-device", default="cpu", choices=["cpu", "cuda"],
                    help="--impl reference only: cpu (default; the reference's CPU step on host cores) or cuda (the "
                         "same torch-op restatement run on the GPU, i.e. what the reference's own step costs on this box)")
    ap.add_argument("--overlap", type=int, default=0, choices=[0, 1],
                    help="run momentum / update / AdamW on a second stream beside Newton-Schulz (1) or everything on "
                         "one stream (0, the optimizer's default)")
    ap.add_argument("--fp8-div", default="full", choices=["full", "ieee", "ieee_strict"],
                    help="arithmetic of the FP8 quantiser: full (default; the reference kernels' GPU instructions, "
                         "bit-exact with them for the absmax codec), ieee (bit-exact with the CPU oracle)")
    ap.add_argument("--fused-update", type=int, default=1, choices=[0, 1],
                    help="weight update in the last Newton-Schulz GEMM's epilogue (1, default) or as its own kernel (0)")
    ap.add_argument("--dependent-launch", type=int, default=1, choices=[0, 1],
                    help="Newton-Schulz GEMMs launched with programmatic stream serialisation (1, the default) or plainly")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-subrecords", action="store_true",
                    help="leave out the extra measurements of the default line (isolated kernels, the reference's "
                         "GPU step, the 2-block model)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    config = {"workload": f"full optimizer step, 6.89B-dense-reference LLaMA, Monarch nblocks={args.nblocks}, "
                          "FP8 E4M3 absmax momentum state, bf16 weights/grads, AdamW group vocab 50257",
              "cache": "inputs_larger_than_l2 (5.9 GB of gradients and 5.9 GB of weights per step)"}

    if args.impl == "reference":
        if rank != 0:
            return 0
        if args.reference_device == "cuda":
            return gpu_reference_step(args, config)
        ms, desc, threads, kind = cpu_reference_step_ms(args.nblocks, max(1, args.steps), max(0, args.warmup))
        line = {"impl": "reference", "metric": METRIC, "value": ms, "unit": "ms", "n_gpus": args.gpus,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": False,
                "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": config,
                "cpu_baseline": {"value": ms, "unit": "ms", "cores": threads, "kind": kind, "sample": desc},
                "e2e": {"value": ms, "unit": "ms", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "gpu_launches": 0}
        print(json.dumps(line))
        return 0

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU path for the product")
    if world > 1:
        from bench_sharded import run_sharded   # multi-GPU path lives beside this file
        return run_sharded(args, rank, world, local_rank, config, METRIC)

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    from monarch_muon_b200 import MonarchMuonOptimizer, _lib
    if args.dynamic_schedule:
        _lib.set_gemm_schedule(True)
    if not args.dependent_launch:
        _lib.set_gemm_dependent_launch(False)
    if args.case == "gemm":
        return run_gemm_comparison(args, dev)
    if args.case == "adamw":
        return run_adamw_isolated(args, dev)
    if args.case == "guest":
        return run_guest_probe(args, dev)
    if args.case != "step":
        return run_isolated(args, dev)

    muon, adamw = build_workload(dev, args.nblocks)
    if args.state_format == "coat":
        from monarch_muon_b200 import CoatStateMonarchMuon
        opt = CoatStateMonarchMuon(muon, adamw, lr=0.02, momentum=0.95, adamw_betas=(0.9, 0.95),
                                   adamw_weight_decay=0.1, adamw_eps=1e-8, ns_max_batch=args.ns_max_batch,
                                   overlap=bool(args.overlap), fp8_div=args.fp8_div, fuse_update=bool(args.fused_update))
    else:
        opt = MonarchMuonOptimizer(muon, adamw, lr=0.02, momentum=0.95, adamw_betas=(0.9, 0.95),
                                   adamw_weight_decay=0.1, adamw_eps=1e-8, state_format=args.state_format,
                                   ns_max_batch=args.ns_max_batch, overlap=bool(args.overlap), fp8_div=args.fp8_div,
                                   fuse_update=bool(args.fused_update))
    if args.state_format != "fp8_absmax":
        config["workload"] = config["workload"].replace("FP8 E4M3 absmax momentum state",
                                                        f"momentum state format {args.state_format}")
    flops, muon_elems, adamw_elems = workload_counts(args.nblocks)
    pk = peaks()

    sampler = ClockSampler(local_rank)
    sampler.start()
    for _ in range(max(3, args.warmup)):
        opt.step()
    torch.cuda.synchronize()
    assert _lib.read_status(dev) == 0, "a kernel reported an expired wait"

    opt.enable_phase_timing(True)
    l0 = _lib.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    t_begin = time.time()
    e0.record()
    for _ in range(args.steps):
        opt.step()
    e1.record()
    torch.cuda.synchronize()
    t_end = time.time()
    launches = _lib.launch_count() - l0
    clocks = sampler.stop(t_begin, t_end)
    ms = e0.elapsed_time(e1) / args.steps
    phases_timed = {k: v / args.steps for k, v in opt.phase_times_ms().items()}
    # Phase times that the rooflines use come from steps with everything on one stream: with the two-stream
    # overlap the bandwidth-bound kernels deliberately run on one CTA per SM beside the GEMMs, so their own
    # duration says nothing about the kernels.
    phases = phases_timed
    if opt.overlap:
        opt.overlap = False
        opt.step()
        torch.cuda.synchronize()
        opt.phase_times_ms()
        serial_steps = 3
        for _ in range(serial_steps):
            opt.step()
        torch.cuda.synchronize()
        phases = {k: v / serial_steps for k, v in opt.phase_times_ms().items()}
        opt.overlap = True
    opt.enable_phase_timing(False)
    status = _lib.read_status(dev)

    ns_ms = phases.get("newton_schulz", float("nan"))
    ach_tf = flops / (ns_ms * 1e-3) / 1e12
    roofline = {"kernel": "gemm_kernel (tcgen05 Newton-Schulz GEMMs, 15 launches per block-shape slice)",
                "bound": "tensor", "achieved": ach_tf, "peak": pk["bf16_tflops_sustained"], "unit": "TFLOP/s",
                "frac": ach_tf / pk["bf16_tflops_sustained"], "peak_kind": f"{pk['source']}, sustained bf16 GEMM",
                "achieved_note": "algorithmic FLOPs (5*(4m^2n+2m^3) per block) over the CUDA-event time of all "
                                 "Newton-Schulz launches of the step; symmetric tiles that are skipped count as done",
                "traffic": None,
                "traffic_note": "not measured in this run (DRAM counters need a profiler pass); an ncu capture of a "
                                "32-block launch read at or below the algorithmic operand and result bytes"}
    mom_ms = phases.get("momentum", float("nan"))
    mom_gbs = muon_elems * S.FP8_ABSMAX_BYTES_PER_ELEM / (mom_ms * 1e-3) / 1e9
    roofline_fp8 = {"kernel": "momentum_kernel (FP8 absmax heavy-ball)", "bound": "hbm", "achieved": mom_gbs,
                    "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": mom_gbs / pk["hbm_gbs"],
                    "peak_kind": f"{pk['source']}, copy bandwidth", "traffic": 0.98 * muon_elems * S.FP8_ABSMAX_BYTES_PER_ELEM,
                    "traffic_note": "0.98 x algorithmic bytes: the ratio an ncu capture of a 4e8-element launch "
                                    "measured, scaled by element count (traffic grows in proportion)"}

    peak_memory_gb = torch.cuda.max_memory_allocated(dev) / 1e9     # parameters, gradients, state and scratch
    state_bytes = sum(v.numel() * v.element_size() for st in opt.state.values() for v in st.values() if torch.is_tensor(v))
    e2e = None
    if not args.no_e2e:
        e2e = run_e2e(opt, muon, adamw, args.steps, dev)
    cpu = None
    if not args.no_cpu_baseline:
        cms, desc, threads, kind = cpu_reference_step_ms(args.nblocks, 3, 1)
        cpu = {"value": cms, "unit": "ms", "cores": threads, "kind": kind, "sample": desc}

    # Further measurements of the same metric family, each with its own clock sample, so that every figure
    # quoted for this library can be read off one line.
    sub = {}
    if not args.no_subrecords and args.state_format == "fp8_absmax" and args.nblocks == 4:
        del opt, muon, adamw
        from monarch_muon_b200.newton_schulz import release_workspaces
        release_workspaces()
        torch.cuda.empty_cache()
        sub["isolated_ns"] = measure_isolated_ns(dev, 4, 128, 10, 3)
        sub["small_block_ns"] = measure_small_block_ns(dev, 20, 5)
        sub["small_block_ns_256"] = measure_small_block_ns(dev, 20, 5, sets=[(128, 256, 256)])
        sub["isolated_fp8_1.6e9"] = measure_isolated_fp8(dev, 1_600_000_000, "fp8_absmax", args.fp8_div, 20, 3)
        sub["isolated_fp8_2558525440"] = measure_isolated_fp8(dev, 2_558_525_440, "fp8_absmax", args.fp8_div, 20, 3)
        release_workspaces()
        torch.cuda.empty_cache()
        sub["reference_gpu"] = gpu_reference_step_ms(dev, 4, 8, 3)
        sub["reference_gpu"]["speedup_device_timed"] = sub["reference_gpu"]["value"] / ms
        sub["nblocks2_step"] = measure_nblocks2_step(dev, 5, 3)

    line = {"metric": METRIC, "value": ms, "unit": "ms", "n_gpus": 1, "steps": args.steps, "warmup": max(3, args.warmup),
            "ms_per_step": ms, "higher_is_better": False, "scaling": "strong",
            "vs_baseline": ms / H100_PUBLISHED_MS, "dtype": "bf16", "data": "synthetic", "config": config,
            "phases_ms": phases, "phases_note": "per-phase device time with everything on one stream (sum = the step "
            "without overlap)" if args.overlap else "per-phase device time", "phases_overlapped_ms": phases_timed if args.overlap else None,
            "roofline": roofline, "roofline_fp8_state": roofline_fp8,
            "ns_algorithmic_tflop_per_step": flops / 1e12, "cpu_baseline": cpu, "e2e": e2e,
            "gpu_launches": launches, "clocks": clocks, "device_status": status,
            "peak_memory_gb": peak_memory_gb, "optimizer_state_gb": state_bytes / 1e9,
            "baseline_note": "vs_baseline divides by the reference's published 304.4 ms on one H100 (bf16 state)"}
    line.update(sub)
    print(json.dumps(line))
    return 0


def measure_nblocks2_step(dev, steps: int, warmup: int) -> dict:
    """The same optimizer step on the 2-block variant of the model (704 + 128 + 64 blocks of 2048x2048,
    5504x2048, 2048x5504: twice the Monarch elements, four times the Newton-Schulz FLOPs)."""
    from monarch_muon_b200 import MonarchMuonOptimizer, _lib
    from monarch_muon_b200.newton_schulz import release_workspaces
    muon, adamw = build_workload(dev, 2)
    opt = MonarchMuonOptimizer(muon, adamw, lr=0.02, momentum=0.95, adamw_betas=(0.9, 0.95), adamw_weight_decay=0.1,
                               adamw_eps=1e-8, state_format="fp8_absmax")
    flops, muon_elems, _ = workload_counts(2)
    for _ in range(max(2, warmup)):
        opt.step()
    torch.cuda.synchronize()
    opt.enable_phase_timing(True)
    sampler = ClockSampler(dev.index or 0)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    tb = time.time()
    e0.record()
    for _ in range(steps):
        opt.step()
    e1.record()
    torch.cuda.synchronize()
    te = time.time()
    ms = e0.elapsed_time(e1) / steps
    phases = {k: v / steps for k, v in opt.phase_times_ms().items()}
    ns_ms = phases.get("newton_schulz", float("nan"))
    out = {"value": ms, "unit": "ms", "steps": steps, "phases_ms": phases, "monarch_elements": muon_elems,
           "ns_algorithmic_tflop_per_step": flops / 1e12, "ns_tflops": flops / (ns_ms * 1e-3) / 1e12,
           "device_status": _lib.read_status(dev), "clocks": sampler.stop(tb, te)}
    del opt, muon, adamw
    release_workspaces()
    torch.cuda.empty_cache()
    return out


def _timed(fn, steps: int, warmup: int, sampler=None):
    for _ in range(max(3, warmup)):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_begin = time.time()
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps, t_begin, time.time()


def run_adamw_isolated(args, dev):
    """The AdamW kernel alone: one flat bf16 parameter of --fp8-elems elements stepped through the optimizer
    (no Muon group), with plain bf16 moments or, with --state-format coat, both moments in the range-expansion
    FP8 format.  Algorithmic bytes per element: 14 (p, g, m, v in; p, m, v out) or 10 + 48/128."""
    from monarch_muon_b200 import CoatStateMonarchMuon, MonarchMuonOptimizer, _lib
    n = args.fp8_elems // 128 * 128
    gen = torch.Generator(device=dev).manual_seed(5)
    p = torch.nn.Parameter(torch.empty(n, dtype=torch.bfloat16, device=dev).normal_(0, 0.02, generator=gen))
    p.grad = torch.empty(n, dtype=torch.bfloat16, device=dev).normal_(0, 1e-3, generator=gen)
    coat = args.state_format == "coat"
    opt = (CoatStateMonarchMuon if coat else MonarchMuonOptimizer)([], [p], lr=3e-4, adamw_betas=(0.9, 0.95),
                                                                  adamw_weight_decay=0.1, adamw_eps=1e-8)
    pk = peaks()
    l0 = _lib.launch_count()
    sampler = ClockSampler(dev.index)
    sampler.start()
    ms, tb, te = _timed(opt.step, args.steps, args.warmup)
    per_elem = 10 + 48 / 128 if coat else 14
    ach = n * per_elem / (ms * 1e-3) / 1e9
    line = {"metric": "adamw_gbs", "value": ach, "unit": "GB/s", "higher_is_better": True, "ms_per_step": ms,
            "config": {"workload": f"isolated AdamW kernel, flat bf16 tensor of {n} elements, "
                                   + ("E4M3 range-expansion moments" if coat else "bf16 moments"),
                       "cache": "inputs_larger_than_l2"},
            "roofline": {"bound": "hbm", "achieved": ach, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": ach / pk["hbm_gbs"],
                         "peak_kind": f"{pk['source']}, copy bandwidth", "traffic": None},
            "n_gpus": 1, "steps": args.steps, "warmup": max(3, args.warmup), "dtype": "bf16", "data": "synthetic",
            "scaling": "strong", "vs_baseline": None, "gpu_launches": _lib.launch_count() - l0,
            "clocks": sampler.stop(tb, te), "device_status": _lib.read_status(dev)}
    print(json.dumps(line))
    return 0


def run_guest_probe(args, dev):
    """Do the small transfer kernels share SMs with the Newton-Schulz GEMMs?  Newton-Schulz on 128 blocks of
    1024 x 1024 (four calls, ~11 ms) is timed alone, and again while this library's peer-store kernel
    (mmb_peer_broadcast, here onto buffers of the same GPU: a copy of 512 MB per launch) runs on a second,
    high-priority stream with one CTA per SM, with one per two SMs, and with two per SM.  CTAs of 128 threads
    without shared memory fit beside a GEMM CTA once per SM; a second one per SM does not, and the GEMM
    launches then wait for SMs."""
    import ctypes as C
    from monarch_muon_b200 import _lib, newton_schulz_batched
    lib = _lib.load()
    gen = torch.Generator(device=dev).manual_seed(11)
    x = torch.empty(128, 1024, 1024, dtype=torch.bfloat16, device=dev).normal_(0, 1, generator=gen)
    nbytes = 512 << 20
    src = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    dst = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    side = torch.cuda.Stream(device=dev, priority=-1)
    reps = 4

    def ns():
        for _ in range(reps):
            newton_schulz_batched(x, backend=_lib.NS_TCGEN05_MULTI)

    for _ in range(2):
        ns()
    torch.cuda.synchronize()

    def timed(ctas, copies):
        torch.cuda.synchronize()
        e0, e1, s0, s1 = (torch.cuda.Event(enable_timing=True) for _ in range(4))
        if ctas:
            ptr = (C.c_void_p * 1)(dst.data_ptr())
            with torch.cuda.stream(side):
                s0.record(side)
                for _ in range(copies):
                    _lib.check(lib.mmb_peer_broadcast(src.data_ptr(), ptr, 1, nbytes, ctas, side.cuda_stream), "peer_broadcast")
                s1.record(side)
            time.sleep(0.002)                         # the copy is under way before the first GEMM is queued
        e0.record()
        ns()
        e1.record()
        torch.cuda.synchronize()
        out = {"newton_schulz_ms": e0.elapsed_time(e1)}
        if ctas:
            ms = s0.elapsed_time(s1)
            out.update(guest_ctas=ctas, guest_ms=ms, guest_gbs=2.0 * nbytes * copies / ms / 1e6)
        return out

    rows = {"alone": timed(0, 0), "alone_again": timed(0, 0)}
    for name, ctas, copies in (("one_guest_per_sm", sms, 40), ("one_guest_per_two_sms", sms // 2, 24),
                               ("two_guests_per_sm", 2 * sms, 40)):
        rows[name] = timed(ctas, copies)
    line = {"metric": "newton_schulz_ms_beside_guest_kernel", "unit": "ms", "n_gpus": 1, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"{reps} x Newton-Schulz on 128 blocks of 1024x1024 beside mmb_peer_broadcast copying "
                                   "512 MB per launch on a high-priority stream"},
            "rows": rows, "device_status": _lib.read_status(dev)}
    print(json.dumps(line))
    return 0


def run_gemm_comparison(args, dev):
    """Sustained throughput of mmb_gemm_bf16 and of cuBLAS (torch.bmm) on the GEMM shapes of one
    Newton-Schulz iteration at the 4-block model (Gram K=1024 and K=2752, Apply N=2752) and on a large
    square GEMM, each run back to back for ~3 s with clocks and power sampled: the yardstick for what a
    library GEMM reaches on these shapes under the power cap.  Last line: the symmetric Gram as the step
    runs it (only block-upper tiles computed), in algorithmic FLOPs."""
    from monarch_muon_b200 import gemm_bf16
    gen = torch.Generator(device=dev).manual_seed(3)

    def sustained(fn, flops, secs=3.0):
        for _ in range(5):
            fn()
        torch.cuda.synchronize()
        sampler = ClockSampler(dev.index)
        sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0, n = time.time(), 0
        e0.record()
        while time.time() - t0 < secs:
            for _ in range(20):
                fn()
            n += 20
            torch.cuda.synchronize()
        e1.record()
        torch.cuda.synchronize()
        clocks = sampler.stop(t0 + 1.0, time.time())
        ms = e0.elapsed_time(e1) / n
        return {"us": ms * 1e3, "tflops": flops / ms / 1e9, "sm_mhz": clocks["sm_mhz"], "power_w": clocks.get("power_w"),
                "reasons": clocks["reasons"]}

    rows = []
    for (b, M, N, K) in [(256, 1024, 1024, 1024), (128, 1024, 1024, 2752), (128, 1024, 2752, 1024), (8, 8192, 8192, 8192)]:
        a = torch.empty(b, M, K, dtype=torch.bfloat16, device=dev).normal_(0, 1, generator=gen)
        bb = torch.empty(b, N, K, dtype=torch.bfloat16, device=dev).normal_(0, 1, generator=gen)
        out = torch.empty(b, M, N, dtype=torch.bfloat16, device=dev)
        bt = bb.transpose(1, 2)
        fl = 2.0 * b * M * N * K
        rows.append({"shape": f"{b}x{M}x{N}x{K}", "cublas": sustained(lambda: torch.bmm(a, bt, out=out), fl),
                     "ours": sustained(lambda: gemm_bf16(a, bb, out=out), fl)})
        del a, bb, out, bt
    x = torch.empty(256, 1024, 1024, dtype=torch.bfloat16, device=dev).normal_(0, 1, generator=gen)
    out = torch.empty(256, 1024, 1024, dtype=torch.bfloat16, device=dev)
    rows.append({"shape": "256x1024x1024x1024 Gram, block-upper tiles only, algorithmic FLOPs",
                 "ours": sustained(lambda: gemm_bf16(x, x, sym_out=True, out=out), 2.0 * 256 * 1024 ** 3)})
    print(json.dumps({"metric": "sustained_batched_gemm_tflops", "unit": "TFLOP/s", "n_gpus": 1, "dtype": "bf16",
                      "data": "synthetic", "rows": rows}))
    return 0


def measure_isolated_ns(dev, nblocks: int, ns_blocks: int, steps: int, warmup: int, with_update: bool = False) -> dict:
    """Batched Newton-Schulz alone on N(0,1) bf16 blocks: `ns_blocks` square blocks and half as many of the
    tall and of the wide shape (128 + 64 + 64 at the 4-block shapes is the metric's isolated case).  With
    `with_update` the weight update rides in the last GEMM's epilogue, as in the optimizer step."""
    from monarch_muon_b200 import newton_schulz_batched
    from monarch_muon_b200.newton_schulz import newton_schulz_update
    pk = peaks()
    gen = torch.Generator(device=dev).manual_seed(99)
    r = 1024 * 4 // nblocks
    t = 2752 * 4 // nblocks
    sets = [(ns_blocks, r, r), (max(1, ns_blocks // 2), t, r), (max(1, ns_blocks // 2), r, t)]
    xs = [torch.empty(s, dtype=torch.bfloat16, device=dev).normal_(0, 1, generator=gen) for s in sets]
    outs = [torch.empty_like(x) for x in xs]
    flops = sum(s[0] * S.ns_flops(s[1], s[2]) for s in sets)

    tables = [torch.tensor([o.data_ptr() + k * s[1] * s[2] * 2 for k in range(s[0])], dtype=torch.int64).to(dev)
              for o, s in zip(outs, sets)]

    def fn():
        for x, o, t in zip(xs, outs, tables):
            if with_update:                       # `outs` play the weights
                for a in range(0, x.shape[0], 256):
                    newton_schulz_update(x[a:a + 256], t[a:a + 256], torch.bfloat16, -0.02)
            else:
                newton_schulz_batched(x, out=o, max_batch=256)
    sampler = ClockSampler(dev.index or 0)
    sampler.start()
    ms, tb, te = _timed(fn, steps, warmup)
    ach = flops / (ms * 1e-3) / 1e12
    return {"value": ach, "unit": "TFLOP/s", "ms": ms, "steps": steps,
            "workload": "isolated batched Newton-Schulz, bf16, N(0,1) blocks: " + ", ".join(f"{s[0]}x{s[1]}x{s[2]}" for s in sets),
            "roofline": {"bound": "tensor", "achieved": ach, "peak": pk["bf16_tflops"], "unit": "TFLOP/s",
                         "frac": ach / pk["bf16_tflops"], "peak_kind": f"{pk['source']}, burst bf16 GEMM", "traffic": None},
            "clocks": sampler.stop(tb, te)}


def measure_small_block_ns(dev, steps: int, warmup: int, sets=None) -> dict:
    """Newton-Schulz on the block set of the small plumbing model (d_model 256, 4 layers, 2-block Monarch:
    88 blocks of 128x128, 16 of 344x128, 8 of 128x344), or on `sets` (e.g. the 256 x 256 attention blocks of
    a 1024-wide, 4-block model), where every block fits one SM: the one-launch on-chip kernel beside the
    fifteen-launch path on the same inputs."""
    from monarch_muon_b200 import _lib, newton_schulz_batched
    gen = torch.Generator(device=dev).manual_seed(7)
    sets = sets or [(88, 128, 128), (16, 344, 128), (8, 128, 344)]
    xs = [torch.empty(s, dtype=torch.bfloat16, device=dev).normal_(0, 1, generator=gen) for s in sets]
    outs = [torch.empty_like(x) for x in xs]
    res = {"workload": "Newton-Schulz on " + ", ".join(f"{s[0]}x{s[1]}x{s[2]}" for s in sets) + " bf16 blocks"}
    for name, backend in (("one_launch_on_chip", _lib.NS_TCGEN05), ("fifteen_launches", _lib.NS_TCGEN05_MULTI)):
        def fn():
            for x, o in zip(xs, outs):
                newton_schulz_batched(x, out=o, backend=backend)
        l0 = _lib.launch_count()
        fn()
        per_call = _lib.launch_count() - l0
        ms, _, _ = _timed(fn, steps, warmup)
        res[name] = {"us": ms * 1e3, "kernel_launches": per_call}
    res["speedup"] = res["fifteen_launches"]["us"] / res["one_launch_on_chip"]["us"]
    return res


def measure_isolated_fp8(dev, n: int, state_format: str, div: str, steps: int, warmup: int) -> dict:
    """The FP8 momentum kernel alone on a flat buffer of n elements (bf16 gradients N(0,1e-3), state
    quantised once from N(0,1e-3)), writing codes, scales and the bf16 momentum."""
    from monarch_muon_b200 import _lib, fp8_state
    pk = peaks()
    gen = torch.Generator(device=dev).manual_seed(99)
    n = n // 128 * 128
    expand_fmt = state_format == "fp8_expand"
    mode = _lib.DIV_NAMES[div]
    m0 = torch.empty(n, dtype=torch.float32, device=dev).normal_(0, 1e-3, generator=gen)
    st = {}
    fp8_state.quantize_(st, "momentum_buffer", m0, codec="expand" if expand_fmt else "absmax", div_mode=mode)
    codes = st["momentum_buffer"].view(torch.uint8)
    scales = st["scale_momentum_buffer"]
    side = dict(expand=st["expand_momentum_buffer"], sqrt_minmax=st["sqrt_minmax_momentum_buffer"]) if expand_fmt else {}
    del m0
    g = torch.empty(n, dtype=torch.bfloat16, device=dev).normal_(0, 1e-3, generator=gen)
    m16 = torch.empty(n, dtype=torch.bfloat16, device=dev)

    def fn():
        fp8_state.fp8_momentum_flat(codes, scales, g, 0.95, m_bf16=m16, div_mode=mode, **side)
    sampler = ClockSampler(dev.index or 0)
    sampler.start()
    ms, tb, te = _timed(fn, steps, warmup)
    per_elem = S.FP8_ABSMAX_BYTES_PER_ELEM + (2 * 2 * 4 / 128 if expand_fmt else 0.0)   # two more fp32 per group, in and out
    ach = n * per_elem / (ms * 1e-3) / 1e9
    name = "range-expansion" if expand_fmt else "absmax"
    out = {"value": ach, "unit": "GB/s", "ms": ms, "steps": steps, "elements": n, "division": div,
           "workload": f"isolated FP8 {name} momentum kernel, flat buffer of {n} elements, bf16 gradients N(0,1e-3), "
                       "groups of 128",
           "roofline": {"bound": "hbm", "achieved": ach, "peak": pk["hbm_gbs"], "unit": "GB/s",
                        "frac": ach / pk["hbm_gbs"], "peak_kind": f"{pk['source']}, copy bandwidth", "traffic": None},
           "clocks": sampler.stop(tb, te)}
    del codes, scales, g, m16, st, side
    torch.cuda.empty_cache()
    return out


def run_isolated(args, dev):
    """The two isolated kernels of the metric: batched Newton-Schulz (TFLOP/s
    against the bf16 tensor peak) and the FP8 momentum kernel (GB/s against HBM)."""
    from monarch_muon_b200 import _lib
    l0 = _lib.launch_count()
    if args.case == "ns":
        r = measure_isolated_ns(dev, args.nblocks, args.ns_blocks, args.steps, args.warmup, bool(args.ns_update))
        line = {"metric": "newton_schulz_tflops"}
    else:
        r = measure_isolated_fp8(dev, args.fp8_elems, args.state_format, args.fp8_div, args.steps, args.warmup)
        line = {"metric": "fp8_momentum_gbs"}
    line.update({"value": r["value"], "unit": r["unit"], "higher_is_better": True, "ms_per_step": r["ms"],
                 "config": {"workload": r["workload"], "cache": "inputs_larger_than_l2"}, "roofline": r["roofline"],
                 "n_gpus": 1, "steps": args.steps, "warmup": max(3, args.warmup), "dtype": "bf16",
                 "data": "synthetic", "scaling": "strong", "vs_baseline": None,
                 "gpu_launches": _lib.launch_count() - l0, "clocks": r["clocks"],
                 "device_status": _lib.read_status(dev)})
    print(json.dumps(line))
    return 0


def run_e2e(opt, muon, adamw, steps: int, dev):
    """optimizer.step() with all gradients arriving from pinned host memory inside
    the timed region, and the per-block momentum sums of squares read back."""
    params = muon + adamw
    host = [torch.empty(p.shape, dtype=p.dtype, pin_memory=True).copy_(p.grad) for p in params]
    h2d = sum(h.numel() * h.element_size() for h in host)
    ss = opt.block_sumsq()
    out_host = torch.empty(ss.shape, dtype=ss.dtype, pin_memory=True)
    d2h = out_host.numel() * out_host.element_size()

    def one():
        opt.step(host_grads=host)          # copies are pipelined slice by slice inside the step
        out_host.copy_(opt.block_sumsq(), non_blocking=True)

    for _ in range(2):
        one()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        one()
    e1.record()
    torch.cuda.synchronize()
    return {"value": e0.elapsed_time(e1) / steps, "unit": "ms", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
            "note": "optimizer.step(host_grads=...): every gradient copied from pinned host memory inside the step, slice by slice on a side stream, then block norms read back"}


if __name__ == "__main__":
    sys.exit(main())
