"""The sharded step on real GPUs (needs at least two; skipped otherwise)."""
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

WORKER = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["MMB_ROOT"]); sys.path.insert(0, os.path.join(os.environ["MMB_ROOT"], "tests"))
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dev = torch.device("cuda", rank)
dist.init_process_group("nccl", device_id=dev)
from monarch_muon_b200.sharded import ShardedMonarchMuon
from monarch_muon_b200 import MonarchMuonOptimizer
gen = torch.Generator().manual_seed(5)
ms = [(2, 128, 128)] * 6 + [(1, 344, 128)] * 4 + [(1, 128, 344)] * 2
asz = [(1000, 64), (64,), (64,)]
w_m = [(0.02 * torch.randn(s, generator=gen)).bfloat16() for s in ms]
w_a = [(0.02 * torch.randn(s, generator=gen)).bfloat16() for s in asz]
def grads(r, step):
    g = torch.Generator().manual_seed(100 * step + r)
    # multiples of 2^-12 keep the bf16 sums over ranks exact, so the reduction order cannot matter
    return [(torch.randint(-8, 9, s, generator=g).float() * 2.0 ** -12).bfloat16() for s in ms + asz]
muon = [torch.nn.Parameter(w.to(dev)) for w in w_m]; adamw = [torch.nn.Parameter(w.to(dev)) for w in w_a]
comm = os.environ.get("MMB_TEST_COMM", "nccl")
opt = ShardedMonarchMuon(muon, adamw, lr=0.02, n_chunks=2, average=False, state_format="fp8_absmax", comm=comm)
assert opt.comm == comm, (opt.comm, comm)
host = torch.empty(opt.g_arena.shape, dtype=opt.g_arena.dtype, pin_memory=True)
# serial twin on the summed gradient, same kernels
smuon = [torch.nn.Parameter(w.to(dev)) for w in w_m]; sadamw = [torch.nn.Parameter(w.to(dev)) for w in w_a]
ser = MonarchMuonOptimizer(smuon, sadamw, lr=0.02, state_format="fp8_absmax")
for step in range(3):
    for p, g in zip(muon + adamw, grads(rank, step)):
        p.grad.copy_(g.to(dev))
    if step == 2:                       # third step: gradients fed from pinned host memory, chunk by chunk
        host.copy_(opt.g_arena)
        torch.cuda.synchronize()
        opt.g_arena.zero_()
        opt.step(host_grad_arena=host)
    else:
        opt.step()
    tot = [sum(gs) for gs in zip(*[[t.float() for t in grads(r, step)] for r in range(world)])]
    for p, g in zip(smuon + sadamw, tot):
        p.grad = g.bfloat16().to(dev)
    ser.step()
torch.cuda.synchronize()
ok = all(torch.equal(a.data, b.data) for a, b in zip(muon + adamw, smuon + sadamw))
flag = torch.tensor([1 if ok else 0], device=dev); dist.all_reduce(flag, op=dist.ReduceOp.MIN)
if rank == 0: print("SHARDED_EQUALS_SERIAL" if int(flag) == 1 else "SHARDED_DIFFERS")
del opt, host                       # no rank leaves while another may still use the shared mappings
torch.cuda.synchronize(); dist.barrier(); torch.cuda.synchronize()
dist.destroy_process_group()
'''


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("comm", ["nccl", "multimem", "p2p"])
def test_sharded_step_is_bitwise_the_serial_step(tmp_path, comm):
    """Two GPUs, three steps (the last one fed from pinned host memory), gradients whose sums over the ranks
    are exact in bf16: the sharded weights must equal, bit for bit, those of the serial step on the summed
    gradient - with NCCL collectives, with this library's NVSwitch multicast kernels and with its peer
    load/store kernels.  Ranks live in
    child processes and leave only after their last step; NCCL's own in-switch algorithms are off here."""
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    env = dict(os.environ, MMB_ROOT=os.path.dirname(os.path.dirname(os.path.abspath(__file__))),
               NCCL_NVLS_ENABLE="0", MMB_TEST_COMM=comm)
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                          "--master-addr", "127.0.0.1", "--master-port", str(port), str(script)],
                         env=env, capture_output=True, text=True, timeout=600)
    assert "SHARDED_EQUALS_SERIAL" in out.stdout, out.stdout[-2000:] + out.stderr[-2000:]


ZERO_WORKER = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["MMB_ROOT"])
from torch.distributed.optim import ZeroRedundancyOptimizer
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dev = torch.device("cuda", rank)
dist.init_process_group("nccl", device_id=dev)
from monarch_muon_b200.sft import SFTOptimizer
ok = True
for algorithm in ("adamw", "muon"):
    gen = torch.Generator().manual_seed(29)
    shapes = [(64, 128), (128, 64), (2, 64, 128), (2, 128, 64)]
    params = [torch.nn.Parameter(torch.randn(s, generator=gen).bfloat16().to(dev)) for s in shapes]
    refs = [torch.nn.Parameter(p.detach().clone()) for p in params]
    zero = ZeroRedundancyOptimizer([{"params": params, "algorithm": algorithm}], optimizer_class=SFTOptimizer, lr=1e-3)
    serial = SFTOptimizer([{"params": refs, "algorithm": algorithm}], lr=1e-3)
    for step in range(4):
        for p, r in zip(params, refs):
            p.grad = torch.randn(p.shape, generator=gen).bfloat16().to(dev)
            r.grad = p.grad.clone()
        zero.step()
        serial.step()
        ok = ok and all(torch.equal(p.data, r.data) for p, r in zip(params, refs))
    owned = sum(p.numel() for g in zero.optim.param_groups for p in g["params"])
    ok = ok and owned < sum(p.numel() for p in params)
torch.cuda.synchronize()
flag = torch.tensor([1 if ok else 0], device=dev); dist.all_reduce(flag, op=dist.ReduceOp.MIN)
if rank == 0: print("ZERO_EQUALS_SERIAL" if int(flag) == 1 else "ZERO_DIFFERS")
dist.destroy_process_group()
'''


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_sft_optimizer_under_zero_redundancy_wrapper(tmp_path):
    """The reference shards its fine-tuning optimizer with torch's ZeroRedundancyOptimizer
    (finetune/train_sft.py:69-72; finetune/test_sft_distributed.py:15-36 checks it against the serial
    optimizer bit for bit).  Same check with this library's SFTOptimizer as the wrapped class."""
    script = tmp_path / "zero_worker.py"
    script.write_text(ZERO_WORKER)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    env = dict(os.environ, MMB_ROOT=os.path.dirname(os.path.dirname(os.path.abspath(__file__))),
               NCCL_NVLS_ENABLE="0")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                          "--master-addr", "127.0.0.1", "--master-port", str(port), str(script)],
                         env=env, capture_output=True, text=True, timeout=600)
    assert "ZERO_EQUALS_SERIAL" in out.stdout, out.stdout[-2000:] + out.stderr[-2000:]
