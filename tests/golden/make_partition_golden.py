"""Golden outputs of the reference's own partitioners (apps/kge/data/sampler.py:10-268), generated in the build
container where the reference checkout is present:

    CUKE_REFERENCE=<cuke checkout> python tests/golden/make_partition_golden.py

The module imports dgl at the top; only numpy is used by the three functions, so dgl is stubbed before the import.
Writes tests/golden/partition.npz (inputs, and the outputs of SoftRelationPartition / BalancedRelationPartition)."""
import contextlib
import io
import os
import sys
import types

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def main():
    ref = os.environ.get("CUKE_REFERENCE", os.path.join(HERE, "..", "..", "..", "reference"))
    for name in ("dgl", "dgl.backend", "dgl.base"):
        sys.modules.setdefault(name, types.ModuleType(name))
    sys.modules["dgl.base"].NID, sys.modules["dgl.base"].EID = "_ID", "_ID"
    sys.modules["dgl"].DGLGraph = object            # base class of a sampler wrapper defined further down the module
    sys.path.insert(0, os.path.join(ref, "apps", "kge", "data"))
    sys.dont_write_bytecode = True
    import sampler as ref_sampler
    out = {}
    for case, (n_edges, n_rel, n_parts, skew) in enumerate([(4000, 37, 4, 1.3), (2500, 11, 3, 0.7), (6000, 120, 8, 1.0)]):
        g = np.random.Generator(np.random.PCG64(90 + case))
        w = np.arange(1, n_rel + 1, dtype=np.float64) ** -skew
        rels = g.choice(n_rel, size=n_edges, p=w / w.sum()).astype(np.int64)
        heads, tails = g.integers(0, 500, n_edges), g.integers(0, 500, n_edges)
        out[f"in{case}"] = np.stack([heads, rels, tails])
        out[f"n{case}"] = np.array(n_parts)
        with contextlib.redirect_stdout(io.StringIO()):
            h, r, t = heads.copy(), rels.copy(), tails.copy()
            parts, rel_parts, cross, cross_rels = ref_sampler.SoftRelationPartition((h, r, t), n_parts)
            out[f"soft{case}_edges"] = np.stack([h, r, t])
            out[f"soft{case}_sizes"] = np.array([len(p) for p in parts])
            for k, rp in enumerate(rel_parts):
                out[f"soft{case}_rel{k}"] = np.asarray(rp)
            out[f"soft{case}_cross"] = np.asarray(cross_rels)
            h, r, t = heads.copy(), rels.copy(), tails.copy()
            parts, rel_parts, cross = ref_sampler.BalancedRelationPartition((h, r, t), n_parts)
            out[f"bal{case}_edges"] = np.stack([h, r, t])
            out[f"bal{case}_sizes"] = np.array([len(p) for p in parts])
            for k, rp in enumerate(rel_parts):
                out[f"bal{case}_rel{k}"] = np.asarray(rp)
            out[f"bal{case}_crossflag"] = np.array(cross)
    np.savez_compressed(os.path.join(HERE, "partition.npz"), **out)
    print("wrote partition.npz with", len(out), "arrays")


if __name__ == "__main__":
    main()
