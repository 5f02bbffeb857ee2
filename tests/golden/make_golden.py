"""Generates tests/golden/ref_<model>.npz by RUNNING THE REFERENCE's own generated C++.

Needs oracle/_ref/*.so (python oracle/build_ref.py, which needs the reference checkout); the fixtures it
writes are committed so that every other machine can pin the oracle without the reference.

For each of the seven scorers: small seeded tables and ids (duplicates included: ids are drawn from a space
much smaller than the batch), the reference module's output for the positive triples, and its output for
the flattened negative triples (the reference's own way of scoring negatives,
apps/kge/data/data_init.py:55-61).  Also stores the single-thread and OpenMP outputs' agreement.

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle  # noqa: E402

OUT = os.path.dirname(os.path.abspath(__file__))
SEED = 20240501

SHAPES = {  # model: (n_ent, n_rel, floats per row, batch, n_neg, n_neg_head)
    "TransE": (61, 7, 24, 48, 6, 0),
    "TransH": (53, 5, 20, 40, 8, 4),
    "TransR": (47, 6, 12, 36, 4, 2),
    "TransF": (59, 7, 28, 44, 5, 2),
    "DistMult": (61, 7, 24, 48, 6, 3),
    "RESCAL": (43, 4, 16, 32, 5, 0),
    "ComplEx": (57, 6, 32, 40, 6, 3),
}


def main():
    for mi, (model, (ne, nr, d, B, nn, nnh)) in enumerate(SHAPES.items()):
        g = np.random.Generator(np.random.PCG64(SEED + mi))
        sig = 1.0 / np.sqrt(d)
        E = (g.standard_normal((ne, d)) * sig).astype(np.float32)
        R = None if model == "RESCAL" else (g.standard_normal((nr, d)) * sig).astype(np.float32)
        P2 = None
        if model == "TransH":
            w = g.standard_normal((nr, d))
            P2 = (w / np.linalg.norm(w, axis=1, keepdims=True)).astype(np.float32)
        if model in ("TransR", "RESCAL"):
            P2 = (g.standard_normal((nr, d, d)) * sig).astype(np.float32)
        h = g.integers(0, ne, B); t = g.integers(0, ne, B); r = g.integers(0, nr, B)
        neg = g.integers(0, ne, (B, nn))
        fh, fr, ft = oracle.flatten(h, r, t, neg, "per_triple", nnh)
        tt = lambda a: None if a is None else torch.from_numpy(a)
        out_pos = oracle.ref_run(model, tt(E), tt(R), tt(P2), tt(h), tt(r), tt(t)).numpy()
        out_neg = oracle.ref_run(model, tt(E), tt(R), tt(P2), tt(fh), tt(fr), tt(ft)).numpy()
        omp_pos = oracle.ref_run(model, tt(E), tt(R), tt(P2), tt(h), tt(r), tt(t), omp=True).numpy()
        assert np.array_equal(out_pos, omp_pos), f"{model}: OpenMP variant differs from single-thread variant"
        arrs = dict(E=E, h=h, r=r, t=t, neg=neg, n_neg_head=np.int64(nnh), ref_pos=out_pos, ref_neg=out_neg)
        if R is not None:
            arrs["R"] = R
        if P2 is not None:
            arrs["P2"] = P2
        np.savez_compressed(os.path.join(OUT, f"ref_{model}.npz"), **arrs)
        print(model, "pos", out_pos.shape, "neg", out_neg.shape)


if __name__ == "__main__":
    main()
