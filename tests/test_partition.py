"""Relation-aware partitioning (cuke_b200.partition) against outputs of the reference's own partitioners
(tests/golden/partition.npz, produced by tests/golden/make_partition_golden.py from apps/kge/data/sampler.py:10-268)."""
import os

import numpy as np
import pytest

from cuke_b200 import partition

Z = np.load(os.path.join(os.path.dirname(__file__), "golden", "partition.npz"))


@pytest.mark.parametrize("case", [0, 1, 2])
def test_soft_relation_partition_matches_reference(case):
    h, r, t = (Z[f"in{case}"][k].copy() for k in range(3))
    n = int(Z[f"n{case}"])
    parts, rel_parts, cross, cross_rels = partition.soft_relation_partition((h, r, t), n)
    assert np.array_equal(np.stack([h, r, t]), Z[f"soft{case}_edges"])
    assert [len(p) for p in parts] == Z[f"soft{case}_sizes"].tolist()
    for k in range(n):
        assert np.array_equal(rel_parts[k], Z[f"soft{case}_rel{k}"])
    assert np.array_equal(cross_rels, Z[f"soft{case}_cross"]) and cross == (len(cross_rels) > 0)
    assert np.array_equal(np.concatenate(parts), np.arange(len(h)))          # contiguous index ranges


@pytest.mark.parametrize("case", [0, 1, 2])
def test_balanced_relation_partition_matches_reference(case):
    h, r, t = (Z[f"in{case}"][k].copy() for k in range(3))
    n = int(Z[f"n{case}"])
    parts, rel_parts, cross = partition.balanced_relation_partition((h, r, t), n)
    assert np.array_equal(np.stack([h, r, t]), Z[f"bal{case}_edges"])
    assert [len(p) for p in parts] == Z[f"bal{case}_sizes"].tolist()
    for k in range(n):
        assert np.array_equal(rel_parts[k], Z[f"bal{case}_rel{k}"])
    assert cross == bool(Z[f"bal{case}_crossflag"])
    assert max(len(p) for p in parts) <= len(h) // n + 1


def test_random_partition_and_relation_shards():
    g = np.random.default_rng(3)
    h, r, t = g.integers(0, 50, 1000), g.integers(0, 9, 1000), g.integers(0, 50, 1000)
    before = sorted(zip(h.tolist(), r.tolist(), t.tolist()))
    parts = partition.random_partition((h, r, t), 3, rng=np.random.default_rng(1))
    assert sorted(zip(h.tolist(), r.tolist(), t.tolist())) == before and [len(p) for p in parts] == [334, 334, 332]
    h2, r2, t2 = h.copy(), r.copy(), t.copy()
    w = np.arange(1, 10, dtype=np.float64) ** -1.5
    r2[:] = g.choice(9, size=1000, p=w / w.sum())
    parts, rel_parts, cross, cross_rels = partition.soft_relation_partition((h2, r2, t2), 3)
    P = g.standard_normal((9, 4, 4)).astype(np.float32)
    shards = partition.shard_relations(rel_parts, [P])
    for k, ((Pk,), g2l) in enumerate(shards):
        rk = r2[parts[k]]
        assert (g2l[rk] >= 0).all()                                  # every edge of the part finds its relation locally
        assert np.array_equal(Pk[g2l[rk]], P[rk])
    single = [rel for rel in range(9) if rel not in set(cross_rels.tolist())]
    for rel in single:                                               # an unsplit relation lives in exactly one partition
        assert sum(rel in set(rp.tolist()) for rp in rel_parts) == 1
