"""A small LLaMA-style decoder with Monarch linear layers, in plain PyTorch.

Test infrastructure: it exists to produce realistic parameter lists and
gradients for the optimizer (the reference builds the same architecture with
pretrain/src/models/llama.py + models/monarch/monarch_linear.py; none of that
code is on the optimizer path, so it is not part of the product).  Shapes follow
the reference: every attention / MLP linear of out m x in n becomes two
block-diagonal factors, blkdiag1 (nb, min-side block, in block) and blkdiag2
(nb, out block, ...) exactly as monarch_linear.py:73-83 sizes them.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F


class MonarchLinear(nn.Module):
    def __init__(self, in_features: int, out_features: int, nblocks: int):
        super().__init__()
        in_blk = -(-in_features // nblocks)
        out_blk = -(-out_features // nblocks)
        self.nb, self.in_features, self.out_features = nblocks, in_features, out_features
        if in_blk < out_blk:
            s1, s2 = (nblocks, in_blk, in_blk), (nblocks, out_blk, in_blk)
        else:
            s1, s2 = (nblocks, out_blk, in_blk), (nblocks, out_blk, out_blk)
        self.blkdiag1 = nn.Parameter(torch.empty(s1))
        self.blkdiag2 = nn.Parameter(torch.empty(s2))

    def forward(self, x):
        lead = x.shape[:-1]
        k, q, p = self.blkdiag1.shape
        l, s, r = self.blkdiag2.shape
        h = x.reshape(-1, k, p)                                   # split features into k blocks
        h = torch.einsum("bkp,kqp->bkq", h, self.blkdiag1)        # first block-diagonal factor
        h = h.reshape(-1, r, l).permute(0, 2, 1)                  # riffle: (b, k*q) viewed as (r, l) -> (l, r)
        h = torch.einsum("blr,lsr->bls", h, self.blkdiag2)        # second factor
        return h.transpose(1, 2).reshape(*lead, s * l)[..., :self.out_features]


class RMSNorm(nn.Module):
    def __init__(self, dim, eps=1e-5):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps = eps

    def forward(self, x):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + self.eps) * self.weight


def _rope(x, base=10000.0):
    b, h, t, d = x.shape
    inv = 1.0 / (base ** (torch.arange(0, d, 2, device=x.device, dtype=torch.float32) / d))
    ang = torch.arange(t, device=x.device, dtype=torch.float32)[:, None] * inv[None, :]
    cos, sin = ang.cos()[None, None], ang.sin()[None, None]
    x1, x2 = x[..., 0::2], x[..., 1::2]
    return torch.stack([x1 * cos - x2 * sin, x1 * sin + x2 * cos], dim=-1).flatten(-2)


class Block(nn.Module):
    def __init__(self, d, heads, inter, nb):
        super().__init__()
        self.heads = heads
        self.attn_norm, self.mlp_norm = RMSNorm(d), RMSNorm(d)
        self.q, self.k, self.v, self.o = (MonarchLinear(d, d, nb) for _ in range(4))
        self.gate, self.up = MonarchLinear(d, inter, nb), MonarchLinear(d, inter, nb)
        self.down = MonarchLinear(inter, d, nb)

    def forward(self, x):
        b, t, d = x.shape
        h = self.attn_norm(x)
        shape = (b, t, self.heads, d // self.heads)
        q, k, v = (m(h).view(shape).transpose(1, 2) for m in (self.q, self.k, self.v))
        a = F.scaled_dot_product_attention(_rope(q), _rope(k), v, is_causal=True)
        x = x + self.o(a.transpose(1, 2).reshape(b, t, d))
        h = self.mlp_norm(x)
        return x + self.down(F.silu(self.gate(h)) * self.up(h))


class TinyMonarchLlama(nn.Module):
    def __init__(self, d_model=256, n_layers=4, heads=4, inter=688, vocab=50257, nblocks=2, seed=0):
        super().__init__()
        self.wte = nn.Embedding(vocab, d_model)
        self.layers = nn.ModuleList(Block(d_model, heads, inter, nblocks) for _ in range(n_layers))
        self.norm = RMSNorm(d_model)
        self.lm_head = nn.Linear(d_model, vocab, bias=False)
        gen = torch.Generator().manual_seed(seed)
        with torch.no_grad():
            for name, p in self.named_parameters():
                if p.dim() >= 2:
                    p.copy_(0.02 * torch.randn(p.shape, generator=gen))      # N(0, 0.02) as the config asks

    def forward(self, idx, targets):
        x = self.wte(idx)
        for layer in self.layers:
            x = layer(x)
        logits = self.lm_head(self.norm(x))
        return F.cross_entropy(logits.view(-1, logits.size(-1)), targets.reshape(-1))


def split_params(model):
    """The reference's grouping rule (pretrain/src/main.py:156-165): Muon takes
    every parameter with ndim >= 2 whose name has none of wte/wpe/lm_head/embed."""
    muon, adamw = [], []
    for name, p in model.named_parameters():
        if p.ndim >= 2 and not any(k in name for k in ("wte", "wpe", "lm_head", "embed")):
            muon.append(p)
        else:
            adamw.append(p)
    return muon, adamw
