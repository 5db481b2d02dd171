"""The allocation-free momentum entry point, mmb_momentum_step_static.

Some callers of this library cannot allocate device memory (a plugin inside
another program's memory pool, a fixed device-memory budget, a latency-critical
loop where an allocation may stall or fail).  For them the momentum step exists
in a second form whose scratch is a fixed array inside the library.  This test
drives both forms through the C ABI on identical inputs, twice in a row, and
requires identical bits in every output: E4M3 codes, fp32 scales, the bf16
momentum and the per-block sums of squares; the same outputs are also held
against the CPU oracle.  It also checks the size limit.

The file name sorts last on purpose: a run that stops at the first failure has
then already executed every other test.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _segments(lib_mod, grads, codes, scales, m16, block):
    segs = (lib_mod.MomentumSeg * len(grads))()
    first = 0
    for k, g in enumerate(grads):
        s = segs[k]
        s.grad = g.data_ptr()
        s.state = codes[k].data_ptr()
        s.scale = scales[k].data_ptr()
        s.m_bf16 = m16[k].data_ptr()
        s.numel = g.numel()
        s.block_elems = block
        s.first_block = first
        first += g.numel() // block
    return segs, first


def test_static_scratch_entry_matches_allocating_entry():
    from monarch_muon_b200 import _lib
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    gen = torch.Generator().manual_seed(2024)
    block = 344 * 128
    sizes = [4 * block, 2 * block, 6 * block]

    def fresh():
        return ([torch.zeros(n, dtype=torch.uint8, device=dev) for n in sizes],
                [torch.zeros(n // 128, dtype=torch.float32, device=dev) for n in sizes],
                [torch.zeros(n, dtype=torch.bfloat16, device=dev) for n in sizes])

    codes_a, scales_a, m_a = fresh()
    codes_b, scales_b, m_b = fresh()
    nblocks = sum(sizes) // block
    ss_a = torch.zeros(nblocks, device=dev)
    ss_b = torch.zeros(nblocks, device=dev)
    stream = _lib.stream_ptr()
    oracle_state = [(torch.zeros(n, dtype=torch.uint8), torch.zeros(n // 128)) for n in sizes]
    for call in range(2):                                   # two calls in a row share the built-in array
        grads = [(1e-3 * torch.randn(n, generator=gen)).bfloat16().to(dev) for n in sizes]
        segs_a, _ = _segments(_lib, grads, codes_a, scales_a, m_a, block)
        segs_b, _ = _segments(_lib, grads, codes_b, scales_b, m_b, block)
        need = lib.mmb_momentum_scratch_floats(segs_a, len(sizes))
        scratch = torch.empty(need, dtype=torch.float32, device=dev)
        _lib.check(lib.mmb_momentum_step(segs_a, len(sizes), _lib.BF16, _lib.STATE_FP8_ABSMAX, _lib.DIV_IEEE,
                                         0.95, 1.0, 16, ss_a.data_ptr(), scratch.data_ptr(), need, stream))
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info(dev)[0] if call == 1 else None
        _lib.check(lib.mmb_momentum_step_static(segs_b, len(sizes), _lib.BF16, _lib.STATE_FP8_ABSMAX,
                                                _lib.DIV_IEEE, 0.95, 1.0, 16, ss_b.data_ptr(), stream))
        torch.cuda.synchronize()
        if free_before is not None:                         # after its first call it takes no device memory
            assert torch.cuda.mem_get_info(dev)[0] == free_before
        for a, b in zip(codes_a + scales_a + m_a + [ss_a], codes_b + scales_b + m_b + [ss_b]):
            av = a.view(torch.int16) if a.dtype == torch.bfloat16 else a
            bv = b.view(torch.int16) if b.dtype == torch.bfloat16 else b
            assert torch.equal(av, bv), f"outputs differ on call {call}"
        assert float(ss_b.min()) > 0.0
        # and against the CPU oracle directly (IEEE division on both sides): codes, scales, bf16 momentum
        from oracle import fp8_oracle
        for k, g in enumerate(grads):
            want = fp8_oracle.absmax_momentum_step(oracle_state[k][0], oracle_state[k][1], g.cpu(), 0.95)
            oracle_state[k] = (want[0], want[1])
            assert torch.equal(codes_b[k].cpu(), want[0]), f"codes differ from the oracle on call {call}"
            assert torch.equal(scales_b[k].cpu().view(torch.int32), want[1].view(torch.int32))
            assert torch.equal(m_b[k].cpu().view(torch.int16), want[3].view(torch.int16))


def test_static_scratch_entry_refuses_oversized_tables():
    from monarch_muon_b200 import _lib
    lib = _lib.load()
    limit = lib.mmb_momentum_static_max_floats()
    assert limit == 1 << 20
    dev = torch.device("cuda", 0)
    tiny = torch.zeros(128, dtype=torch.uint8, device=dev)          # never touched: the size check comes first
    seg = (_lib.MomentumSeg * 1)()
    seg[0].grad = tiny.data_ptr()
    seg[0].state = tiny.data_ptr()
    seg[0].scale = tiny.data_ptr()
    seg[0].numel = (limit + 1) * 4096
    seg[0].block_elems = seg[0].numel
    rc = lib.mmb_momentum_step_static(seg, 1, _lib.BF16, _lib.STATE_FP8_ABSMAX, _lib.DIV_IEEE, 0.95, 1.0, 16,
                                      tiny.data_ptr(), _lib.stream_ptr())
    assert rc != 0
    msg = lib.mmb_last_error().decode()
    assert "built-in scratch" in msg and str(limit) in msg
