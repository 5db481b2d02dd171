"""Ownership plan for the data-parallel (owner-computes) Monarch-Muon step.

Every Monarch block is an independent unit of the Muon update (momentum, FP8
groups, Newton-Schulz and the weight update touch only that block), and AdamW is
element-wise, so the step shards without any exchange inside it: one gradient
reduce-scatter before and one all-gather of updated values after.  This module
only computes *where things live*; it has no torch.distributed or CUDA in it so
it can be tested anywhere.

Layout.  The flat arenas (one for weights, one for gradients, same geometry) are
cut into `n_chunks` chunk arenas that are communicated and processed one after
the other so that communication of one chunk overlaps computation of another.
A chunk arena is `world` equal shards, shard r owned by rank r:

    arena = [chunk 0: shard(rank 0) | shard(rank 1) | ... ][chunk 1: ...] ... [AdamW chunk] ... [last chunk]

The first and the last Muon chunk are half as large as the inner ones and the AdamW chunk sits in the middle:
the first reduction and the last gather are the communication no computation can hide.

Inside a Muon shard the owned tensors lie back to back, grouped by block shape.
Whole tensors are owned (a parameter must stay one contiguous view).  Tensors of
one shape are dealt to ranks in contiguous runs of equal length - equal FLOPs and
equal bytes at once when the counts divide, as they do for the LLaMA shapes here -
and what does not divide goes, one tensor each, to the ranks with the least
Newton-Schulz work so far (longest-processing-time rule), heavy shapes first.
Shards are padded to the longest one.  The AdamW chunk is cut element-wise into equal slices, so a
tensor may straddle ranks.
"""
from __future__ import annotations

from dataclasses import dataclass, field


@dataclass
class TensorPlace:
    index: int          # position in the caller's parameter list
    chunk: int
    rank: int
    offset: int         # element offset inside the whole arena
    numel: int


@dataclass
class ChunkPlan:
    offset: int         # element offset of the chunk arena inside the whole arena
    shard_elems: int    # elements per rank (padded); chunk arena = world * shard_elems
    kind: str           # "muon" or "adamw"


@dataclass
class Plan:
    world: int
    chunks: list = field(default_factory=list)            # ChunkPlan
    muon: list = field(default_factory=list)              # TensorPlace per Muon tensor
    adamw: list = field(default_factory=list)             # (index, offset, numel) of AdamW tensors in the arena
    total_elems: int = 0

    def owned_muon(self, rank: int, chunk: int):
        return [t for t in self.muon if t.rank == rank and t.chunk == chunk]

    def adamw_slices(self, rank: int):
        """Intersections of AdamW tensors with the slice rank `rank` owns:
        (tensor index, start inside the tensor, length, arena offset)."""
        ch = next((c for c in self.chunks if c.kind == "adamw"), None)
        if ch is None:
            return []
        lo = ch.offset + rank * ch.shard_elems
        hi = lo + ch.shard_elems
        out = []
        for idx, off, n in self.adamw:
            a, b = max(lo, off), min(hi, off + n)
            if a < b:
                out.append((idx, a - off, b - a, a))
        return out


def _align(n: int, a: int) -> int:
    return -(-n // a) * a


def _tensor_flops(shape) -> float:
    """Newton-Schulz work of one (nblocks, rows, cols) tensor: 5 x (4 m^2 n + 2 m^3) per block."""
    nb, r, c = shape
    m, n = min(r, c), max(r, c)
    return nb * 5.0 * (4.0 * m * m * n + 2.0 * m ** 3)


def chunk_fractions(n_chunks: int, edge: float = 0.5):
    """Cumulative boundaries of the Muon chunks as fractions of each shape's tensors.  The first and the last
    chunk are `edge` times as large as the inner ones: the first reduce-scatter and the last all-gather are
    the part of the communication that no computation can hide, so they are made short, while the inner
    chunks stay large enough for efficient GEMM batches."""
    if n_chunks <= 2:
        w = [1.0] * n_chunks
    else:
        w = [edge] + [1.0] * (n_chunks - 2) + [edge]
    total = sum(w)
    out, acc = [0.0], 0.0
    for x in w:
        acc += x
        out.append(acc / total)
    out[-1] = 1.0
    return out


def make_plan(muon_shapes, adamw_numels, world: int, n_chunks: int = 4, align: int = 128, edge: float = 0.5) -> Plan:
    """muon_shapes: (nblocks, rows, cols) per Muon tensor; adamw_numels: element
    counts of the AdamW tensors.  `align` keeps every tensor and shard on a
    128-element (256-byte) boundary: FP8 groups and vector accesses stay aligned.
    `edge`: size of the first and last Muon chunk relative to the inner ones (see chunk_fractions)."""
    if world < 1 or n_chunks < 1:
        raise ValueError("world and n_chunks must be positive")
    bounds = chunk_fractions(n_chunks, edge)
    plan = Plan(world=world)
    by_shape: dict = {}
    for i, (nb, r, c) in enumerate(muon_shapes):
        by_shape.setdefault((r, c), []).append(i)
    places = {}
    cursor = 0
    load = [0.0] * world           # Newton-Schulz FLOPs dealt to each rank so far, over all chunks
    # heaviest tensors first, so that the remainders of the light shapes can even out those of the heavy ones
    order = sorted(by_shape.items(), key=lambda kv: -_tensor_flops(muon_shapes[kv[1][0]]))
    def place_adamw():
        nonlocal cursor
        total = sum(_align(n, align) for n in adamw_numels)
        shard = _align(-(-total // world), align)
        plan.chunks.append(ChunkPlan(offset=cursor, shard_elems=shard, kind="adamw"))
        at = cursor
        for i, n in enumerate(adamw_numels):
            plan.adamw.append((i, at, n))
            at += _align(n, align)
        cursor += world * shard

    # The AdamW chunk goes in the middle of the sequence: its (tiny) computation needs no position, and in the
    # middle both its reduction and its gather run under Newton-Schulz of the neighbouring Muon chunks.
    adamw_at = n_chunks // 2 if (adamw_numels and n_chunks >= 2) else None
    for ch in range(n_chunks):
        if adamw_at is not None and ch == adamw_at:
            place_adamw()
        per_rank = [[] for _ in range(world)]
        for (r, c), idxs in order:
            n = len(idxs)
            # this chunk's share of the shape, cut on multiples of the world size where the count allows, so
            # that every rank gets the same number of tensors of the shape in every chunk
            unit = world if n >= world * n_chunks else 1
            lo = int(round(bounds[ch] * n / unit)) * unit
            hi = n if ch == n_chunks - 1 else int(round(bounds[ch + 1] * n / unit)) * unit
            mine = idxs[lo:hi]
            k = len(mine)
            # every rank gets k // world tensors of the shape; the k % world left over go, one each, to the
            # ranks that carry the least work so far (longest-processing-time rule on the remainders)
            counts = [k // world] * world
            for rank in sorted(range(world), key=lambda q: (load[q], q))[:k % world]:
                counts[rank] += 1
            at = 0
            for rank in range(world):
                take = mine[at:at + counts[rank]]
                at += counts[rank]
                per_rank[rank] += take
                load[rank] += sum(_tensor_flops(muon_shapes[i]) for i in take)
        sizes = [sum(_align(muon_shapes[i][0] * muon_shapes[i][1] * muon_shapes[i][2], align) for i in lst)
                 for lst in per_rank]
        shard = _align(max(sizes) if sizes else 0, align)
        if shard == 0:
            continue
        chunk_index = len(plan.chunks)
        plan.chunks.append(ChunkPlan(offset=cursor, shard_elems=shard, kind="muon"))
        for rank, lst in enumerate(per_rank):
            at = cursor + rank * shard
            for i in lst:
                numel = muon_shapes[i][0] * muon_shapes[i][1] * muon_shapes[i][2]
                places[i] = TensorPlace(index=i, chunk=chunk_index, rank=rank, offset=at, numel=numel)
                at += _align(numel, align)
        cursor += world * shard
    plan.muon = [places[i] for i in range(len(muon_shapes))]
    if adamw_numels and adamw_at is None:
        place_adamw()
    plan.total_elems = cursor
    return plan


def flops_per_rank(plan: Plan, muon_shapes, ns_flops) -> list:
    """Newton-Schulz FLOPs each rank owns (for reporting balance)."""
    out = [0.0] * plan.world
    for t in plan.muon:
        nb, r, c = muon_shapes[t.index]
        out[t.rank] += nb * ns_flops(r, c)
    return out
