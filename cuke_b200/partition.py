"""Relation-aware partitioning of a triple list over workers / GPUs.

Same contracts as the partitioners of the reference's data layer (apps/kge/data/sampler.py:10-268:
SoftRelationPartition, BalancedRelationPartition, RandomPartition): the edge arrays are permuted IN PLACE so that
partition k owns one contiguous index range, and the per-partition relation lists say which relation matrices /
vectors a worker needs.  With a relation partition every triple of a (non-split) relation is scored by one worker, so
the large per-relation tables of TransR / RESCAL (108-131 MB in the benchmark configurations) need no gradient
all-reduce: `shard_relations` builds the per-worker tables and id maps for that.

The assignment rules are the reference's; the per-edge bookkeeping is done with array operations instead of a Python
loop over edges (rank of an edge among the edges of its relation -> owning part through the cumulative part sizes).
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple

import numpy as np


def _relations_by_size(rels: np.ndarray):
    uniq, cnts = np.unique(rels, return_counts=True)
    order = np.flip(np.argsort(cnts))              # largest relation first (ties as numpy's argsort leaves them)
    return uniq[order], cnts[order]


def _place_edges(rels: np.ndarray, plan: dict, n: int) -> List[np.ndarray]:
    """plan[r] = [(part, count), ...]: the k-th edge of relation r (in edge order) goes to the part whose cumulative
    count first exceeds k.  Returns the edge indices of every part, ascending."""
    order = np.argsort(rels, kind="stable")
    sorted_rels = rels[order]
    starts = np.flatnonzero(np.r_[True, sorted_rels[1:] != sorted_rels[:-1]])
    ends = np.r_[starts[1:], len(rels)]
    part_of = np.empty(len(rels), dtype=np.int64)
    for s, e in zip(starts, ends):
        r = sorted_rels[s]
        parts = np.array([p for p, c in plan[r] if c > 0], dtype=np.int64)
        sizes = np.array([c for p, c in plan[r] if c > 0], dtype=np.int64)
        k = np.arange(e - s)
        part_of[order[s:e]] = parts[np.searchsorted(np.cumsum(sizes), k, side="right")]
    return [np.flatnonzero(part_of == j).astype(np.int64) for j in range(n)]


def _apply(edges: Sequence[np.ndarray], parts: List[np.ndarray]) -> List[np.ndarray]:
    shuffle = np.concatenate(parts)
    for a in edges:
        a[:] = a[shuffle]
    out, off = [], 0
    for p in parts:
        out.append(np.arange(off, off + len(p)))
        off += len(p)
    return out


def soft_relation_partition(edges, n: int, has_importance: bool = False, threshold: float = 0.05):
    """Relations with more than `threshold` of all edges (or more than one partition's share) are spread evenly over all
    n partitions; every other relation goes whole to the partition that holds the fewest edges so far.
    Returns (parts, rel_parts, cross, cross_rels) like the reference's SoftRelationPartition."""
    rels = edges[1]
    uniq, cnts = _relations_by_size(rels)
    if not cnts[0] > cnts[-1]:
        raise AssertionError("relation sizes are all equal")      # the reference asserts the same
    edge_cnts = np.zeros(n, dtype=np.int64)
    rel_parts: List[list] = [[] for _ in range(n)]
    large = min(int(len(rels) * threshold), int(len(rels) / n))
    plan, cross = {}, []
    for r, cnt in zip(uniq, cnts):
        cnt = int(cnt)
        if cnt > large:
            share = cnt // n + 1
            alloc = []
            for j in range(n):
                take = share if cnt > share else cnt
                alloc.append((j, take))
                rel_parts[j].append(r)
                edge_cnts[j] += take
                cnt -= take
            plan[r] = alloc
            cross.append(r)
        else:
            j = int(np.argmin(edge_cnts))
            plan[r] = [(j, cnt)]
            rel_parts[j].append(r)
            edge_cnts[j] += cnt
    parts = _apply(edges[:4] if has_importance else edges[:3], _place_edges(rels.copy(), plan, n))
    return parts, [np.array(x) for x in rel_parts], len(cross) > 0, np.array(cross)


def balanced_relation_partition(edges, n: int, has_importance: bool = False):
    """Every partition is filled up to len(edges) // n + 1 edges: a relation goes to the emptiest partition, spilling
    into the next emptiest one when it does not fit.  Returns (parts, rel_parts, cross)."""
    rels = edges[1]
    uniq, cnts = _relations_by_size(rels)
    if not cnts[0] > cnts[-1]:
        raise AssertionError("relation sizes are all equal")
    edge_cnts = np.zeros(n, dtype=np.int64)
    rel_parts: List[list] = [[] for _ in range(n)]
    cap = len(rels) // n + 1
    plan, n_cross = {}, 0
    for r, cnt in zip(uniq, cnts):
        cnt = int(cnt)
        alloc = []
        while cnt > 0:
            j = int(np.argmin(edge_cnts))
            take = cnt if edge_cnts[j] + cnt <= cap else int(cap - edge_cnts[j])
            if take < cnt:
                n_cross += 1
            alloc.append((j, take))
            rel_parts[j].append(r)
            edge_cnts[j] += take
            cnt -= take
        plan[r] = alloc
    parts = _apply(edges[:4] if has_importance else edges[:3], _place_edges(rels.copy(), plan, n))
    return parts, [np.array(x) for x in rel_parts], n_cross > 0


def random_partition(edges, n: int, has_importance: bool = False, rng: Optional[np.random.Generator] = None):
    """Edges permuted at random (numpy's global generator unless `rng` is given), n contiguous parts of ceil(len / n)."""
    m = len(edges[0])
    idx = np.random.permutation(m) if rng is None else rng.permutation(m)
    for a in (edges[:4] if has_importance else edges[:3]):
        a[:] = a[idx]
    size = int(math.ceil(m / n))
    return [idx[size * i: min(size * (i + 1), m)] for i in range(n)]


def shard_relations(rel_parts: List[np.ndarray], tables: Sequence[np.ndarray]):
    """Per-partition copies of the relation tables: for partition k, (local tables holding only rel_parts[k]'s rows in
    that order, global -> local id map with -1 for relations the partition does not hold)."""
    n_rel = tables[0].shape[0]
    out = []
    for rp in rel_parts:
        rp = np.asarray(rp, dtype=np.int64)
        g2l = np.full(n_rel, -1, dtype=np.int64)
        g2l[rp] = np.arange(len(rp))
        out.append(([np.ascontiguousarray(t[rp]) for t in tables], g2l))
    return out
