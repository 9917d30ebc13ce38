"""Request sharding over GPUs: which rank serves which sequence.

The path has no exchange step: sequences are independent and a sequence's KV records live on the GPU that serves
it. Sharding is therefore a host-side assignment and nothing else; the only collective is the caller's final
gather of outputs. The cost of a sequence is its number of KV units (committed blocks plus the fresh block) per
query block, which is proportional to the bytes the step streams for it.
"""
from __future__ import annotations

from typing import List, Sequence


def units(nblocks: int, nq: int = 1) -> int:
    """KV units one step touches for a sequence with `nblocks` committed blocks and nq query blocks (per kv head)."""
    return sum(nblocks + j + 1 for j in range(nq))


def shard_round_robin(nseq: int, world: int) -> List[List[int]]:
    """Equal-length batches: sequence i goes to rank i % world."""
    return [list(range(r, nseq, world)) for r in range(world)]


def shard_lpt(lengths: Sequence[int], world: int, nq: Sequence[int] | None = None) -> List[List[int]]:
    """Ragged batches: longest-processing-time greedy on KV units. Deterministic: ties go to the
    lower sequence index, then to the lower rank. Returns, per rank, the sequence indices it serves (ascending)."""
    n = len(lengths)
    nq = [1] * n if nq is None else list(nq)
    cost = [units(int(lengths[i]), nq[i]) for i in range(n)]
    order = sorted(range(n), key=lambda i: (-cost[i], i))
    load = [0] * world
    out: List[List[int]] = [[] for _ in range(world)]
    for i in order:
        r = min(range(world), key=lambda k: (load[k], k))
        out[r].append(i)
        load[r] += cost[i]
    return [sorted(x) for x in out]


def imbalance(lengths: Sequence[int], shards: List[List[int]], nq: Sequence[int] | None = None) -> float:
    """max / mean KV units per rank (1.0 = perfect)."""
    n = len(lengths)
    nq = [1] * n if nq is None else list(nq)
    loads = [sum(units(int(lengths[i]), nq[i]) for i in s) for s in shards]
    mean = sum(loads) / len(loads)
    return max(loads) / mean if mean else 1.0
