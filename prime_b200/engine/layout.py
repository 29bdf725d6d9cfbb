"""Flat parameter layout shared by the fused engine, the ZeRO-3 collectives, DiLoCo and checkpoints.

All parameters of the model live in ONE flat buffer, ordered by *group* (embedding, one group per
transformer block, head). Inside the flat buffer every parameter is contiguous in its natural
``[out, in]`` shape, so a kernel can address it directly (TMA tensor maps need no gather).

Sharding follows FSDP2's per-parameter dim-0 rule (``torch.chunk`` semantics, the layout the
reference gets from ``fully_shard``, src/zeroband/train.py:150-168): rank ``r`` of ``W`` owns rows
``[r*ceil(rows/W), (r+1)*ceil(rows/W))`` of every parameter. A rank's *shard buffer* is the
concatenation of its row-slices in parameter order; each (parameter, rank) pair is one contiguous
``Segment`` in both buffers. Because the slices are dim-0 chunks they can be exposed as
``DTensor(Shard(0))`` locals, which keeps distributed checkpoints interchangeable.
"""
from __future__ import annotations

from dataclasses import dataclass, field

ALIGN = 64  # elements; keeps every parameter / shard slice 128-byte aligned in bf16


def _align(n: int, a: int = ALIGN) -> int:
    return (n + a - 1) // a * a


@dataclass
class ParamSpec:
    name: str
    shape: tuple[int, ...]
    group: int
    offset: int = 0          # element offset in the full flat buffer
    numel: int = 0

    @property
    def rows(self) -> int:
        return self.shape[0]

    @property
    def row_numel(self) -> int:
        return self.numel // self.shape[0]


@dataclass
class Segment:
    """Rows of one parameter owned by one rank: contiguous in the full and in the shard buffer."""
    param: int               # index into ParamLayout.params
    full_offset: int
    shard_offset: int
    numel: int
    row_start: int
    row_end: int


@dataclass
class GroupInfo:
    name: str
    params: list[int] = field(default_factory=list)
    full_start: int = 0
    full_end: int = 0


class ParamLayout:
    def __init__(self, specs: list[tuple[str, tuple[int, ...], int]], group_names: list[str], world: int = 1):
        self.world = world
        self.params: list[ParamSpec] = []
        self.groups = [GroupInfo(n) for n in group_names]
        off = 0
        for name, shape, g in specs:
            n = 1
            for s in shape:
                n *= s
            p = ParamSpec(name, tuple(shape), g, off, n)
            if not self.groups[g].params:
                self.groups[g].full_start = off
            self.groups[g].params.append(len(self.params))
            self.params.append(p)
            off = _align(off + n)
            self.groups[g].full_end = off
        self.full_numel = off
        self.by_name = {p.name: i for i, p in enumerate(self.params)}
        # per-rank segments
        self.segments: list[list[Segment]] = []
        self.shard_numel: list[int] = []
        for r in range(world):
            segs, soff = [], 0
            for i, p in enumerate(self.params):
                per = -(-p.rows // world)
                r0, r1 = min(r * per, p.rows), min((r + 1) * per, p.rows)
                n = (r1 - r0) * p.row_numel
                segs.append(Segment(i, p.offset + r0 * p.row_numel, soff, n, r0, r1))
                soff = _align(soff + n)
            self.segments.append(segs)
            self.shard_numel.append(soff)
        self.max_shard_numel = max(self.shard_numel)

    def group_segments(self, rank: int, group: int) -> list[Segment]:
        return [self.segments[rank][i] for i in self.groups[group].params]

    def group_shard_range(self, rank: int, group: int) -> tuple[int, int]:
        segs = self.group_segments(rank, group)
        last = segs[-1]
        return segs[0].shard_offset, _align(last.shard_offset + last.numel)


def llama_layout(args, world: int = 1) -> ParamLayout:
    """Layout of a Llama model described by :class:`prime_b200.models.llama.ModelArgs`.

    Within a block wq/wk/wv are adjacent (one fused ``[(H+2KV)*hd, D]`` GEMM operand) and so are
    w1/w3 (one fused ``[2F, D]`` operand)."""
    D, F, hd = args.dim, args.hidden_dim, args.head_dim
    H, KV, V, L = args.n_heads, args.kv_heads, args.vocab_size, args.n_layers
    specs: list[tuple[str, tuple[int, ...], int]] = [("tok_embeddings.weight", (V, D), 0)]
    names = ["tok_embeddings"]
    for i in range(L):
        g = 1 + i
        names.append(f"layers.{i}")
        pre = f"layers.{i}."
        specs += [
            (pre + "attention_norm.weight", (D,), g),
            (pre + "attention.wq.weight", (H * hd, D), g),
            (pre + "attention.wk.weight", (KV * hd, D), g),
            (pre + "attention.wv.weight", (KV * hd, D), g),
            (pre + "attention.wo.weight", (D, H * hd), g),
            (pre + "ffn_norm.weight", (D,), g),
            (pre + "feed_forward.w1.weight", (F, D), g),
            (pre + "feed_forward.w3.weight", (F, D), g),
            (pre + "feed_forward.w2.weight", (D, F), g),
        ]
    names.append("head")
    specs += [("norm.weight", (D,), L + 1), ("output.weight", (V, D), L + 1)]
    return ParamLayout(specs, names, world)
