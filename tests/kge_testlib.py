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


def elem_err(a, b):
    """Element-wise companion of rel_err: max |a - b| / (|b| + 1e-3 max |b|).  Small entries are judged (almost) on
    their own scale, so an error that the tensor-wide norm would hide behind one large entry shows up here."""
    a = np.asarray(a, dtype=np.float64); b = np.asarray(b, dtype=np.float64)
    if b.size == 0:
        return 0.0
    floor = 1e-3 * max(np.abs(b).max(), 1e-30)
    return float((np.abs(a - b) / (np.abs(b) + floor)).max())


def par_map(fn, items, workers=8):
    """The oracle is single-threaded C called through ctypes (the GIL is released): independent pieces run side by side."""
    from concurrent.futures import ThreadPoolExecutor
    oracle.lib()
    with ThreadPoolExecutor(max_workers=workers) as ex:
        return list(ex.map(fn, items))


def occurrence_problem(E, R, P2, h, r, t, neg):
    """The same triples over tables in which every entity-id OCCURRENCE has a row of its own (copies of the original rows,
    in the slot order [h | t | neg]) and relations are renumbered by first appearance in sorted order.  The oracle's dense
    entity gradient over these tables IS the per-slot gradient the backward kernels write, so a sample of triples out of
    a large batch can be checked without reducing the whole batch on the CPU.
    Returns (E', R', P2', h', r', t', neg', rel_uniq)."""
    h, r, t = (np.asarray(x, dtype=np.int64) for x in (h, r, t))
    B = h.shape[0]
    parts = [E[h], E[t]]
    neg2 = None
    if neg is not None:
        neg = np.asarray(neg, dtype=np.int64)
        parts.append(E[neg.reshape(-1)])
        neg2 = (2 * B + np.arange(neg.size, dtype=np.int64)).reshape(neg.shape)
    E2 = np.ascontiguousarray(np.concatenate(parts))
    ru, r2 = np.unique(r, return_inverse=True)
    R2 = None if R is None else np.ascontiguousarray(R[ru])
    P22 = None if P2 is None else np.ascontiguousarray(P2[ru])
    return E2, R2, P22, np.arange(B, dtype=np.int64), r2.astype(np.int64), B + np.arange(B, dtype=np.int64), neg2, ru


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
