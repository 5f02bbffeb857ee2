"""Shared helpers of the parity tests: seeded problems, the GPU pipeline through the C ABI, comparisons."""
import numpy as np
import torch

from oracle import oracle

MODELS = ["TransE", "TransH", "TransR", "TransF", "DistMult", "RESCAL", "ComplEx"]
FP32_TOL = 1e-4      # north-star tolerance for fp32 CUDA-core scores and gradients (relative)
BF16_TOL = 2e-2      # bf16 storage, fp32 accumulate


def rel_err(a, b):
    """max |a - b| / max |b| : error relative to the scale of the reference tensor."""
    a = np.asarray(a, dtype=np.float64); b = np.asarray(b, dtype=np.float64)
    if b.size == 0:
        return 0.0
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


def make_problem(model, seed=0, ne=300, nr=11, d=40, B=64, nn=8, neg_mode="per_triple", chunk=0, zipf=False):
    g = np.random.Generator(np.random.PCG64(1234 + seed))
    sig = 1.0 / np.sqrt(d)
    E = (g.standard_normal((ne, d)) * sig).astype(np.float32)
    R = None if model == "RESCAL" else (g.standard_normal((nr, d)) * sig).astype(np.float32)
    P2 = None
    if model == "TransH":
        w = g.standard_normal((nr, d)); P2 = (w / np.linalg.norm(w, axis=1, keepdims=True)).astype(np.float32)
    if model in ("TransR", "RESCAL"):
        P2 = (g.standard_normal((nr, d, d)) * sig).astype(np.float32)

    def ids(size):
        if zipf:
            w = np.arange(1, ne + 1, dtype=np.float64) ** -1.1
            return g.choice(ne, size=size, p=w / w.sum()).astype(np.int64)
        return g.integers(0, ne, size).astype(np.int64)

    h, t, r = ids(B), ids(B), g.integers(0, nr, B).astype(np.int64)
    neg = None
    if neg_mode == "per_triple":
        neg = ids((B, nn))
    elif neg_mode == "chunk_shared":
        neg = ids((B // chunk, nn))
    return dict(model=model, E=E, R=R, P2=P2, h=h, r=r, t=t, neg=neg, neg_mode=neg_mode, chunk=chunk, g=g)


def to_dev(a, dtype=None, bf16=False):
    if a is None:
        return None
    x = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    if bf16 and x.dtype == torch.float32:
        x = x.to(torch.bfloat16)
    if dtype is not None:
        x = x.to(dtype)
    return x.contiguous()


def bf16_round(a):
    return None if a is None else torch.from_numpy(a).to(torch.bfloat16).float().numpy()


def gpu_scorer(p, n_neg_head=0, bf16=False, precision="fp32"):
    from cuke_b200.scoring import Scorer
    return Scorer(p["model"], to_dev(p["E"], bf16=bf16), to_dev(p["R"], bf16=bf16), to_dev(p["P2"], bf16=bf16),
                  p["neg_mode"], n_neg_head, p["chunk"], precision)


def gpu_ids(p, id_dtype=torch.int64):
    return tuple(to_dev(p[k], id_dtype) for k in ("h", "r", "t", "neg"))


def dense_from_compact(uniq, n_unique, rows, n_rows_total):
    """Scatter one-row-per-distinct-id gradients into a dense table (test-side only)."""
    U = int(n_unique.item())
    out = np.zeros((n_rows_total,) + tuple(rows.shape[1:]), dtype=np.float64)
    out[uniq[:U].cpu().numpy()] = rows[:U].double().cpu().numpy()
    return out


def gpu_grads_dense(p, sc, h, r, t, neg, dpos, dneg):
    """forward -> backward -> inspector -> segmented reduction; returns dense (gE, gR, gP2) as float64 numpy."""
    from cuke_b200 import scoring
    pos, negs, rel_insp = sc.forward(h, r, t, neg)
    sg = sc.backward(h, r, t, neg, pos, negs, dpos, dneg, rel_insp)
    ids = scoring.entity_id_list(h, t, neg)
    insp = scoring.inspect(ids, p["E"].shape[0])
    ge = scoring.segment_reduce(sg.ent_slots, insp)
    gE = dense_from_compact(insp.uniq, insp.n_unique, ge, p["E"].shape[0])
    gR = gP = None
    nr = (p["R"] if p["R"] is not None else p["P2"]).shape[0]
    rinsp = sg.rel_insp if sg.rel_insp is not None else scoring.inspect(r, nr)
    if sg.rel_slots is not None:
        gr = scoring.segment_reduce(sg.rel_slots, rinsp)
        gR = dense_from_compact(rinsp.uniq, rinsp.n_unique, gr, nr)
    if sg.rel2_slots is not None:
        gw = scoring.segment_reduce(sg.rel2_slots, rinsp)
        gP = dense_from_compact(rinsp.uniq, rinsp.n_unique, gw, nr)
    if sg.rel2_groups is not None:
        gP = dense_from_compact(rinsp.uniq, rinsp.n_unique, sg.rel2_groups, nr)
    return pos, negs, gE, gR, gP
