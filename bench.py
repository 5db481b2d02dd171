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

`--impl reference` times the CPU restatement of the reference step (oracle/,
torch CPU kernels on all host threads) on a bounded sample of blocks and scales
it to the full step by block and element counts.
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
def build_workload(device, nblocks: int, seed: int = 1234, shard=None):
    """Parameters and gradients of the 6.89B-reference model's optimizer step.
    `shard=(rank, world)` keeps every world-th tensor's blocks split evenly: each
    rank owns 1/world of the blocks of every tensor (used for N > 1)."""
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
def cpu_reference_step_ms(nblocks: int, steps: int, warmup: int, threads: int | None = None):
    """The oracle's restatement of the reference step (bf16 twin: bf16 state,
    bf16 Newton-Schulz) on host cores, on a sample of blocks, scaled to the full
    step.  Returns (ms per full step, description of the sample, threads)."""
    from oracle import muon_oracle
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
    groups = {}
    for (r, c), nb in sample.items():
        w = (0.02 * torch.randn(nb, r, c, generator=gen)).bfloat16()
        g = (1e-3 * torch.randn(nb, r, c, generator=gen)).bfloat16()
        groups[(r, c)] = (w, g, torch.zeros_like(w))
    _, _, adamw_elems = workload_counts(nblocks)
    a_n = 1 << 23
    ap = (0.02 * torch.randn(a_n, generator=gen)).bfloat16()
    ag = (1e-3 * torch.randn(a_n, generator=gen)).bfloat16()
    am, av = torch.zeros_like(ap), torch.zeros_like(ap)

    def one_pass(step_no: int) -> float:
        total = 0.0
        for (r, c), (w, g, buf) in groups.items():
            t0 = time.perf_counter()
            muon_oracle.muon_group_step([w], [g], [buf], lr=0.02, beta=0.95, ns_dtype=torch.bfloat16)
            total += (time.perf_counter() - t0) * full[(r, c)] / sample[(r, c)]
        t0 = time.perf_counter()
        muon_oracle.adamw_tensor_step(ap, ag, am, av, step_no, lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1, eps=1e-8)
        total += (time.perf_counter() - t0) * adamw_elems / a_n
        return total * 1e3

    with torch.no_grad():
        for i in range(warmup):
            one_pass(i + 1)
        times = [one_pass(warmup + i + 1) for i in range(steps)]
    desc = ("bf16 reference step (momentum, cat, Newton-Schulz, update) on "
            + ", ".join(f"{nb} of {full[k]} blocks {k[0]}x{k[1]}" for k, nb in sample.items())
            + f"; AdamW on {a_n} of {adamw_elems} elements; each part scaled linearly to the full count")
    return sum(times) / len(times), desc, threads


def gpu_reference_step(args, config) -> int:
    """The reference step's torch-op sequence (bf16 twin: _foreach momentum, cat, bmm-based
    Newton-Schulz, per-tensor add_, _foreach AdamW) on the full workload on cuda:0, timed with
    CUDA events.  It is the restatement used as the parity checker, here only timed: it shows
    what the reference's own GPU path (cuBLAS batched GEMMs + elementwise torch kernels) costs
    on the same box."""
    from oracle import muon_oracle
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    torch.backends.cuda.matmul.allow_tf32 = True     # as the reference's harness sets it
    muon, adamw = build_workload(dev, args.nblocks)
    ref = muon_oracle.OracleMonarchMuon([p.data for p in muon], [p.data for p in adamw], lr=0.02, momentum=0.95,
                                        adamw_betas=(0.9, 0.95), adamw_weight_decay=0.1, adamw_eps=1e-8,
                                        ns_dtype=torch.bfloat16, foreach_cpu=True)
    mg, ag = [p.grad for p in muon], [p.grad for p in adamw]
    sampler = ClockSampler(0)
    sampler.start()
    for _ in range(max(3, args.warmup)):
        ref.step(mg, ag)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_begin = time.time()
    e0.record()
    for _ in range(args.steps):
        ref.step(mg, ag)
    e1.record()
    torch.cuda.synchronize()
    t_end = time.time()
    ms = e0.elapsed_time(e1) / args.steps
    line = {"impl": "reference", "reference_device": "cuda", "metric": METRIC, "value": ms, "unit": "ms", "n_gpus": 1,
            "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms, "higher_is_better": False,
            "scaling": "strong", "vs_baseline": ms / H100_PUBLISHED_MS, "dtype": "bf16", "data": "synthetic",
            "config": dict(config, workload=config["workload"].replace("FP8 E4M3 absmax momentum state",
                                                                       "bf16 momentum state (the reference's)")),
            "note": "torch-op restatement of the reference's bf16 step on the GPU (cuBLAS bmm + elementwise kernels), "
                    "full workload, gradients resident",
            "peak_memory_gb": torch.cuda.max_memory_allocated(dev) / 1e9,
            "clocks": sampler.stop(t_begin, t_end), "gpu_launches": 0}
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
    ap.add_argument("--case", default="step", choices=["step", "ns", "fp8", "gemm", "adamw"],
                    help="step: the full optimizer step (headline); ns: isolated batched Newton-Schulz on the "
                         "128+64+64 block set; fp8: isolated FP8 momentum kernel on a flat buffer; gemm: the library's "
                         "batched GEMM beside cuBLAS (torch.bmm) on the Newton-Schulz shapes, each run back to "
                         "back for seconds so that the power cap is in force; adamw: the AdamW kernel alone on a flat bf16 "
                         "tensor of --fp8-elems elements (FP8 moments with --state-format coat)")
    ap.add_argument("--ns-blocks", type=int, default=128, help="square blocks in --case ns (tall/wide get half each)")
    ap.add_argument("--fp8-elems", type=int, default=1_600_000_000)
    ap.add_argument("--comm-sms", type=int, default=0, help="SMs left to NCCL during the sharded step")
    ap.add_argument("--chunks", type=int, default=4, help="pipeline chunks of the sharded (multi-GPU) step")
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
    ap.add_argument("--no-e2e", action="store_true")
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
        ms, desc, threads = cpu_reference_step_ms(args.nblocks, max(1, args.steps), max(0, args.warmup))
        line = {"impl": "reference", "metric": METRIC, "value": ms, "unit": "ms", "n_gpus": args.gpus,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": False,
                "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": config,
                "cpu_baseline": {"value": ms, "unit": "ms", "cores": threads, "kind": "port", "sample": desc},
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
    if args.case == "gemm":
        return run_gemm_comparison(args, dev)
    if args.case == "adamw":
        return run_adamw_isolated(args, dev)
    if args.case != "step":
        return run_isolated(args, dev)

    muon, adamw = build_workload(dev, args.nblocks)
    if args.state_format == "coat":
        from monarch_muon_b200 import CoatStateMonarchMuon
        opt = CoatStateMonarchMuon(muon, adamw, lr=0.02, momentum=0.95, adamw_betas=(0.9, 0.95),
                                   adamw_weight_decay=0.1, adamw_eps=1e-8, ns_max_batch=args.ns_max_batch,
                                   overlap=bool(args.overlap))
    else:
        opt = MonarchMuonOptimizer(muon, adamw, lr=0.02, momentum=0.95, adamw_betas=(0.9, 0.95),
                                   adamw_weight_decay=0.1, adamw_eps=1e-8, state_format=args.state_format,
                                   ns_max_batch=args.ns_max_batch, overlap=bool(args.overlap))
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
                "traffic": 1.0e11,
                "traffic_note": "DRAM bytes summed over the step's 120 GEMM launches, scaled by block count from the "
                                "ncu capture of the 32-block case in profiles/gemm_kernel_ns_32blocks.md"}
    mom_ms = phases.get("momentum", float("nan"))
    mom_gbs = muon_elems * S.FP8_ABSMAX_BYTES_PER_ELEM / (mom_ms * 1e-3) / 1e9
    roofline_fp8 = {"kernel": "momentum_kernel (FP8 absmax heavy-ball)", "bound": "hbm", "achieved": mom_gbs,
                    "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": mom_gbs / pk["hbm_gbs"],
                    "peak_kind": f"{pk['source']}, copy bandwidth", "traffic": 0.98 * muon_elems * S.FP8_ABSMAX_BYTES_PER_ELEM,
                    "traffic_note": "0.98 x algorithmic bytes, ncu capture of 4e8 elements in "
                                    "profiles/momentum_kernel_fp8_400M.md scaled by element count"}

    e2e = None
    if not args.no_e2e:
        e2e = run_e2e(opt, muon, adamw, args.steps, dev)
    cpu = None
    if not args.no_cpu_baseline:
        cms, desc, threads = cpu_reference_step_ms(args.nblocks, 1, 1)
        cpu = {"value": cms, "unit": "ms", "cores": threads, "kind": "port", "sample": desc}

    line = {"metric": METRIC, "value": ms, "unit": "ms", "n_gpus": 1, "steps": args.steps, "warmup": max(3, args.warmup),
            "ms_per_step": ms, "higher_is_better": False, "scaling": "strong",
            "vs_baseline": ms / H100_PUBLISHED_MS, "dtype": "bf16", "data": "synthetic", "config": config,
            "phases_ms": phases, "phases_note": "per-phase device time with everything on one stream (sum = the step "
            "without overlap)" if args.overlap else "per-phase device time", "phases_overlapped_ms": phases_timed if args.overlap else None,
            "roofline": roofline, "roofline_fp8_state": roofline_fp8,
            "ns_algorithmic_tflop_per_step": flops / 1e12, "cpu_baseline": cpu, "e2e": e2e,
            "gpu_launches": launches, "clocks": clocks, "device_status": status,
            "baseline_note": "vs_baseline divides by the reference's published 304.4 ms on one H100 (bf16 state)"}
    print(json.dumps(line))
    return 0


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


def run_isolated(args, dev):
    """The two isolated kernels of the metric: batched Newton-Schulz (TFLOP/s
    against the bf16 tensor peak) and the FP8 momentum kernel (GB/s against HBM)."""
    from monarch_muon_b200 import _lib, fp8_state, newton_schulz_batched
    pk = peaks()
    gen = torch.Generator(device=dev).manual_seed(99)
    sampler = ClockSampler(dev.index)
    sampler.start()
    l0 = _lib.launch_count()
    if args.case == "ns":
        nb = args.ns_blocks
        r = 1024 * 4 // args.nblocks
        t = 2752 * 4 // args.nblocks
        sets = [(nb, r, r), (max(1, nb // 2), t, r), (max(1, nb // 2), r, t)]
        xs = [torch.empty(s, dtype=torch.bfloat16, device=dev).normal_(0, 1, generator=gen) for s in sets]
        outs = [torch.empty_like(x) for x in xs]
        flops = sum(s[0] * S.ns_flops(s[1], s[2]) for s in sets)

        def fn():
            for x, o in zip(xs, outs):
                newton_schulz_batched(x, out=o, max_batch=256)
        ms, tb, te = _timed(fn, args.steps, args.warmup)
        ach = flops / (ms * 1e-3) / 1e12
        line = {"metric": "newton_schulz_tflops", "value": ach, "unit": "TFLOP/s", "higher_is_better": True,
                "ms_per_step": ms, "config": {"workload": "isolated batched Newton-Schulz, bf16, N(0,1) blocks: "
                                              + ", ".join(f"{s[0]}x{s[1]}x{s[2]}" for s in sets),
                                              "cache": "inputs_larger_than_l2"},
                "roofline": {"bound": "tensor", "achieved": ach, "peak": pk["bf16_tflops"], "unit": "TFLOP/s",
                             "frac": ach / pk["bf16_tflops"], "peak_kind": f"{pk['source']}, burst bf16 GEMM",
                             "traffic": None}}
    else:
        n = args.fp8_elems // 128 * 128
        expand_fmt = args.state_format == "fp8_expand"
        m0 = torch.empty(n, dtype=torch.float32, device=dev).normal_(0, 1e-3, generator=gen)
        st = {}
        fp8_state.quantize_(st, "momentum_buffer", m0, codec="expand" if expand_fmt else "absmax")
        codes = st["momentum_buffer"].view(torch.uint8)
        scales = st["scale_momentum_buffer"]
        side = dict(expand=st["expand_momentum_buffer"], sqrt_minmax=st["sqrt_minmax_momentum_buffer"]) if expand_fmt else {}
        del m0
        g = torch.empty(n, dtype=torch.bfloat16, device=dev).normal_(0, 1e-3, generator=gen)
        m16 = torch.empty(n, dtype=torch.bfloat16, device=dev)

        def fn():
            fp8_state.fp8_momentum_flat(codes, scales, g, 0.95, m_bf16=m16, **side)
        ms, tb, te = _timed(fn, args.steps, args.warmup)
        per_elem = S.FP8_ABSMAX_BYTES_PER_ELEM + (2 * 2 * 4 / 128 if expand_fmt else 0.0)   # two more fp32 per group, in and out
        ach = n * per_elem / (ms * 1e-3) / 1e9
        name = "range-expansion" if expand_fmt else "absmax"
        line = {"metric": "fp8_momentum_gbs", "value": ach, "unit": "GB/s", "higher_is_better": True,
                "ms_per_step": ms, "config": {"workload": f"isolated FP8 {name} momentum kernel, flat buffer of {n} "
                                              "elements, bf16 gradients N(0,1e-3), groups of 128",
                                              "cache": "inputs_larger_than_l2"},
                "roofline": {"bound": "hbm", "achieved": ach, "peak": pk["hbm_gbs"], "unit": "GB/s",
                             "frac": ach / pk["hbm_gbs"], "peak_kind": f"{pk['source']}, copy bandwidth",
                             "traffic": None}}
    line.update({"n_gpus": 1, "steps": args.steps, "warmup": max(3, args.warmup), "dtype": "bf16",
                 "data": "synthetic", "scaling": "strong", "vs_baseline": None,
                 "gpu_launches": _lib.launch_count() - l0, "clocks": sampler.stop(tb, te),
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
