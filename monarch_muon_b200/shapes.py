"""Shapes, counts and operation counts of the Monarch-Muon workload.

Factor shapes follow MonarchLinear (pretrain/src/models/monarch/
monarch_linear.py:73-83); the LLaMA layout (q,k,v,o,gate,up,down per layer,
lm_head left dense) follows apply_monarch (:108-154).
"""
from __future__ import annotations

NS_ITERS = 5
FP8_ABSMAX_BYTES_PER_ELEM = 1 + 2 + 1 + 2 + 2 * 4 / 128   # code in, bf16 grad, code out, bf16 m, scale in+out


def monarch_factor_shapes(in_features: int, out_features: int, nblocks: int):
    in_blk = -(-in_features // nblocks)
    out_blk = -(-out_features // nblocks)
    if in_blk < out_blk:
        return (nblocks, in_blk, in_blk), (nblocks, out_blk, in_blk)
    return (nblocks, out_blk, in_blk), (nblocks, out_blk, out_blk)


def llama_monarch_muon_shapes(d_model: int, n_layers: int, intermediate: int, nblocks: int):
    """(nblocks, rows, cols) of every Muon tensor, in model order."""
    shapes = []
    for _ in range(n_layers):
        for _ in range(4):
            shapes += list(monarch_factor_shapes(d_model, d_model, nblocks))
        for _ in range(2):
            shapes += list(monarch_factor_shapes(d_model, intermediate, nblocks))
        shapes += list(monarch_factor_shapes(intermediate, d_model, nblocks))
    return shapes


def llama_adamw_shapes(d_model: int, n_layers: int, vocab: int):
    """Embedding, LM head and the RMSNorm vectors (two per layer plus the final one)."""
    return [(vocab, d_model), (vocab, d_model)] + [(d_model,)] * (2 * n_layers + 1)


def ns_flops(rows: int, cols: int) -> float:
    """Algorithmic FLOPs of five quintic iterations on one block:
    Gram 2m^2n + square 2m^3 + apply 2m^2n, m = min(rows, cols), n = max."""
    m, n = min(rows, cols), max(rows, cols)
    return NS_ITERS * (4.0 * m * m * n + 2.0 * m ** 3)


MODEL_689B = dict(d_model=4096, n_layers=32, intermediate=11008, vocab=50257)
