"""Multi-GPU leg of bench.py: the owner-computes sharded optimizer step.

Launched by torchrun with one rank per GPU (bench.py dispatches here when
WORLD_SIZE > 1).  Total work is fixed (the whole 6.89B-reference model), so this
is strong scaling: `value` is device-timed milliseconds per step for the whole
job, max over ranks, covering gradient reduce-scatter, the local steps and the
weight all-gather.  Compute-only and communication-only passes are timed too so
that exposed communication can be read off.
"""
from __future__ import annotations

import json
import os
import time

import torch
import torch.distributed as dist


def _timed_max(fn, steps, warmup, dev):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.time()
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t1 = time.time()
    dist.barrier()
    ms = torch.tensor([e0.elapsed_time(e1) / steps], device=dev)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return float(ms.item()), t0, t1


def parity_check(dev, rank: int, world: int, comm: str) -> str:
    """A small sharded run against the serial step on the summed gradient, in this process group, before
    anything is timed: gradients are multiples of 2^-12, so their bf16 sums over the ranks are exact and the
    order of the reduction cannot matter; weights after two steps must be equal bit for bit ("ok")."""
    from monarch_muon_b200 import MonarchMuonOptimizer
    from monarch_muon_b200.sharded import ShardedMonarchMuon
    gen = torch.Generator().manual_seed(5)
    ms = [(2, 128, 128)] * 8 + [(1, 344, 128)] * 8 + [(1, 128, 344)] * 8
    asz = [(1000, 64), (64,), (64,)]
    w_m = [(0.02 * torch.randn(s, generator=gen)).bfloat16() for s in ms]
    w_a = [(0.02 * torch.randn(s, generator=gen)).bfloat16() for s in asz]

    def grads(r, step):
        g = torch.Generator().manual_seed(100 * step + r)
        return [(torch.randint(-8, 9, s, generator=g).float() * 2.0 ** -12).bfloat16() for s in ms + asz]
    muon = [torch.nn.Parameter(w.to(dev)) for w in w_m]
    adamw = [torch.nn.Parameter(w.to(dev)) for w in w_a]
    opt = ShardedMonarchMuon(muon, adamw, lr=0.02, n_chunks=2, average=False, state_format="fp8_absmax", comm=comm)
    smuon = [torch.nn.Parameter(w.to(dev)) for w in w_m]
    sadamw = [torch.nn.Parameter(w.to(dev)) for w in w_a]
    ser = MonarchMuonOptimizer(smuon, sadamw, lr=0.02, state_format="fp8_absmax")
    for step in range(2):
        for p, g in zip(muon + adamw, grads(rank, step)):
            p.grad.copy_(g.to(dev))
        opt.step()
        tot = [sum(gs) for gs in zip(*[[t.float() for t in grads(r, step)] for r in range(world)])]
        for p, g in zip(smuon + sadamw, tot):
            p.grad = g.bfloat16().to(dev)
        ser.step()
    torch.cuda.synchronize()
    ok = all(torch.equal(a.data, b.data) for a, b in zip(muon + adamw, smuon + sadamw))
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    used = opt.comm
    del opt, ser
    torch.cuda.empty_cache()
    return ("ok" if int(flag.item()) == 1 else "differs") + f" ({used})"


def run_sharded(args, rank, world, local_rank, config, metric):
    import bench
    from monarch_muon_b200 import _lib, shapes as S
    from monarch_muon_b200.sharded import ShardedMonarchMuon

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=dev)
    if not args.dependent_launch:
        _lib.set_gemm_dependent_launch(False)
    parity = parity_check(dev, rank, world, args.comm)
    muon, adamw = bench.build_workload(dev, args.nblocks, seed=1234)      # same weights on every rank
    grads = [p.grad for p in muon + adamw]
    for p in muon + adamw:
        p.grad = None
    opt = ShardedMonarchMuon(muon, adamw, lr=0.02, momentum=0.95, adamw_betas=(0.9, 0.95),
                             adamw_weight_decay=0.1, adamw_eps=1e-8, n_chunks=args.chunks,
                             comm_sms=None if args.comm_sms < 0 else args.comm_sms,
                             comm_ctas=None if args.comm_ctas < 0 else args.comm_ctas, chunk_edge=args.chunk_edge,
                             dynamic_schedule=args.dynamic_schedule != 0,
                             state_format="fp8_absmax", comm=args.comm, fp8_div=args.fp8_div)
    if parity.startswith("differs") and opt.comm in ("multimem", "p2p"):
        # never time a transport whose result is wrong: fall back to NCCL and say so
        del opt
        torch.cuda.empty_cache()
        for p in muon + adamw:
            p.grad = None
        opt = ShardedMonarchMuon(muon, adamw, lr=0.02, momentum=0.95, adamw_betas=(0.9, 0.95), adamw_weight_decay=0.1,
                                 adamw_eps=1e-8, n_chunks=args.chunks, dynamic_schedule=args.dynamic_schedule != 0,
                                 state_format="fp8_absmax", comm="nccl", fp8_div=args.fp8_div)
        parity += "; timed with nccl instead"
    gen = torch.Generator(device=dev).manual_seed(4321 + rank)           # each rank's own gradients
    opt.g_arena.normal_(0.0, 1e-3, generator=gen)
    del grads
    torch.cuda.empty_cache()
    flops, muon_elems, adamw_elems = bench.workload_counts(args.nblocks)
    pk = bench.peaks()
    warm = max(3, args.warmup)

    sampler = bench.ClockSampler(local_rank)
    sampler.start()
    l0 = None

    def full():
        opt.step()

    ms, t0, t1 = _timed_max(full, args.steps, warm, dev)
    clocks = sampler.stop(t0, t1)
    l0 = _lib.launch_count()
    opt.step()
    torch.cuda.synchronize()
    launches_per_step = _lib.launch_count() - l0

    # compute only: the local steps with the collectives left out
    def compute_only():
        scale = 1.0 / world
        for k, o in enumerate(opt.local):
            if o is not None:
                o.grad_scale = scale if opt.plan.chunks[k].kind == "muon" else 1.0
                o.step()

    ms_compute, _, _ = _timed_max(compute_only, args.steps, 1, dev)

    def comm_only_own_kernels():
        main = torch.cuda.current_stream()
        s_red, s_bc = opt._streams
        opt._fence()
        s_red.wait_stream(main)
        s_bc.wait_stream(main)
        lib = _lib.load()
        for k in range(len(opt.plan.chunks)):
            opt._launch_reduce(lib, k, s_red.cuda_stream)
            opt._launch_broadcast(lib, k, s_bc.cuda_stream)
        main.wait_stream(s_red)
        main.wait_stream(s_bc)
        opt._fence()

    def comm_only():
        if opt.comm in ("multimem", "p2p"):
            return comm_only_own_kernels()
        works = []
        for k in range(len(opt.plan.chunks)):
            g_whole, g_mine, w_whole, w_mine = opt.chunk_views(k)
            works.append(opt._reduce_scatter(g_whole, g_mine))
        for k in range(len(opt.plan.chunks)):
            works[k].wait()
            g_whole, g_mine, w_whole, w_mine = opt.chunk_views(k)
            works.append(opt._all_gather(w_whole, w_mine))
        for w in works:
            w.wait()

    ms_comm, _, _ = _timed_max(comm_only, args.steps, 1, dev)
    status = torch.tensor([_lib.read_status(dev)], device=dev)
    dist.all_reduce(status, op=dist.ReduceOp.MAX)

    e2e = None
    if not args.no_e2e:
        try:
            host = torch.empty(opt.g_arena.shape, dtype=opt.g_arena.dtype, pin_memory=True)
            host.copy_(opt.g_arena)
            small = next(o for o in opt.local if o is not None and o.block_sumsq() is not None).block_sumsq()
            out_host = torch.empty(small.shape, dtype=small.dtype, pin_memory=True)

            def one():
                opt.step(host_grad_arena=host)         # chunk copies pipelined under reduction and compute
                out_host.copy_(small, non_blocking=True)

            ems, _, _ = _timed_max(one, args.steps, 1, dev)
            e2e = {"value": ems, "unit": "ms", "h2d_bytes_per_step": host.numel() * host.element_size() * world,
                   "d2h_bytes_per_step": out_host.numel() * out_host.element_size() * world,
                   "note": "every rank feeds its full gradient arena from pinned host memory each step, chunk by chunk "
                           "inside step(host_grad_arena=...)"}
        except RuntimeError as exc:                                       # e.g. not enough pinnable host memory
            e2e = {"value": None, "unit": "ms", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                   "note": f"not measured: {str(exc)[:120]}"}

    if rank == 0:
        arena_bytes = opt.plan.total_elems * 2
        if opt.comm == "multimem":
            # reduce: the whole arena leaves each GPU once, one shard comes back; broadcast: the mirror image
            per_dir = arena_bytes * (1 + 1 / world)
            nvlink = {"transport": "multimem", "bytes_per_direction_per_gpu_per_step": per_dir,
                      "achieved_gbs_per_direction_per_gpu": per_dir / (ms_comm * 1e-3) / 1e9, "reference_gbs": 770.0,
                      "note": "reduce (outbound) and broadcast (inbound) of all chunks timed together, no compute"}
        elif opt.comm == "p2p":
            # reduce: (N-1)/N of the arena comes in (the peers' copies of the own shard) and as much goes out
            # (the peers reading theirs); broadcast: the same amounts the other way round
            per_dir = 2 * (world - 1) / world * arena_bytes
            nvlink = {"transport": "p2p", "bytes_per_direction_per_gpu_per_step": per_dir,
                      "achieved_gbs_per_direction_per_gpu": per_dir / (ms_comm * 1e-3) / 1e9, "reference_gbs": 770.0,
                      "note": "peer-load reduce and peer-store broadcast of all chunks timed together, no compute"}
        else:
            per_dir = 2 * (world - 1) / world * arena_bytes      # both ring collectives load both directions
            nvlink = {"transport": "nccl", "bytes_per_direction_per_gpu_per_step": per_dir,
                      "achieved_gbs_per_direction_per_gpu": per_dir / (ms_comm * 1e-3) / 1e9, "reference_gbs": 770.0,
                      "note": "reduce-scatter then all-gather of all chunks, no compute"}
        wire = 2 * (world - 1) / world * (muon_elems + adamw_elems) * 2
        line = {"metric": metric, "value": ms, "unit": "ms", "n_gpus": world, "steps": args.steps, "warmup": warm,
                "ms_per_step": ms, "higher_is_better": False, "scaling": "strong",
                "vs_baseline": ms / bench.H100_PUBLISHED_MS, "dtype": "bf16", "data": "synthetic",
                "config": dict(config, parallelism=f"owner-computes dp{world}: bf16 grad reduce-scatter, local "
                                                   "momentum/Newton-Schulz/update/AdamW, weight all-gather over "
                                                   f"{ {'multimem': 'NVSwitch multicast kernels of this library', 'p2p': 'peer load/store kernels of this library'}.get(opt.comm, 'NCCL') }; "
                                                   f"{args.chunks} chunks pipelined, {opt.comm_sms} SMs left to communication, "
                                                   f"{'dynamic' if args.dynamic_schedule != 0 else 'static'} GEMM tile schedule"),
                "phases_ms": {"step": ms, "compute_only": ms_compute, "communication_only": ms_comm,
                              "exposed_communication": max(0.0, ms - ms_compute)},
                "roofline": {"kernel": "gemm_kernel (tcgen05 Newton-Schulz GEMMs)", "bound": "tensor",
                             "achieved": flops / world / (ms_compute * 1e-3) / 1e12,
                             "peak": pk["bf16_tflops_sustained"], "unit": "TFLOP/s",
                             "frac": flops / world / (ms_compute * 1e-3) / 1e12 / pk["bf16_tflops_sustained"],
                             "peak_kind": f"{pk['source']}, sustained bf16 GEMM; per-GPU algorithmic FLOPs over the "
                                          "whole local step", "traffic": None},
                "parity_check": parity,
                "nvlink": nvlink,
                "cpu_baseline": None, "e2e": e2e, "gpu_launches": launches_per_step * args.steps * world,
                "clocks": clocks, "device_status": int(status.item())}
        print(json.dumps(line))
    # no rank leaves while another may still use the arenas it shares (symmetric memory mappings)
    torch.cuda.synchronize()
    dist.barrier()
    del opt
    torch.cuda.synchronize()
    dist.barrier()
    dist.destroy_process_group()
    return 0
