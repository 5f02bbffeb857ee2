"""GPU parity on the benchmark configurations themselves (cuke_b200.synth.CONFIGS c1-c5, c4 also over bf16 tables).

c1 and c2 run at full size and every score is compared.  c3, c4 and c5 run at full batch, dim, chunk and negative
count (c5 with the entity table scaled down: only its row count shrinks); the CPU oracle cannot score 10^6..10^8
triples of those shapes in seconds, so it checks
  * all positives,
  * the negatives of a seeded sample: whole chunks (chunk-shared) or all triples of a few relations (per-triple),
  * the per-slot gradient rows of the same sample, by running the oracle over tables in which every id occurrence has a
    row of its own (kge_testlib.occurrence_problem), and the relation-side gradients of the sampled relations,
and the reduction of ALL slot rows into one row per distinct id is compared with a float64 index_add of the same rows.
c5 goes through KgeStep(precision="tensor") - the fused forward + loss + backward call the benchmark times - and its
loss and final gradients are compared with the oracle directly.

Tolerances: 1e-4 relative for fp32 tables (max |d| / max |ref| per tensor), 2e-2 for bf16 tables against the oracle on
the bf16-rounded tables.  An element-wise figure, max |d| / (|ref| + 1e-3 max |ref|), is computed beside each and bounded
for fp32 (1e-2: entries a thousand times smaller than the largest are still right to 1e-5 of the largest).
Set KGE_PARITY_REPORT=<file> to get every figure as JSON.
"""
import json
import os

import numpy as np
import pytest
import torch

from cuke_b200 import synth
from oracle import oracle
from tests.kge_testlib import BF16_TOL, FP32_TOL, bf16_round, elem_err, occurrence_problem, par_map, rel_err, to_dev

pytestmark = pytest.mark.gpu
REPORT = {}


def _check(name, got, ref, tol):
    got = got.detach().cpu().numpy() if isinstance(got, torch.Tensor) else np.asarray(got)
    r, e = rel_err(got, ref), elem_err(got, ref)
    REPORT[name] = {"rel_err": r, "elem_err": e, "tol": tol, "n": int(np.asarray(ref).size)}
    path = os.environ.get("KGE_PARITY_REPORT")
    if path:
        with open(path, "w") as f:
            json.dump(REPORT, f, indent=1)
    assert r < tol, f"{name}: rel_err {r:.3e} >= {tol}"
    if tol == FP32_TOL:
        assert e < 1e-2, f"{name}: element-wise error {e:.3e}"


def _tables(cfg, model):
    ent, rel, rel2 = synth.make_tables(cfg, model)
    if cfg.dtype == "bf16":
        ent, rel, rel2 = bf16_round(ent), bf16_round(rel), bf16_round(rel2)
    return ent, rel, rel2


def _scorer(cfg, model, tabs, precision, n_neg_head=None):
    from cuke_b200.scoring import Scorer
    bf = cfg.dtype == "bf16"
    nnh = cfg.n_neg_head if n_neg_head is None else n_neg_head
    return Scorer(model, to_dev(tabs[0], bf16=bf), to_dev(tabs[1], bf16=bf), to_dev(tabs[2], bf16=bf), cfg.neg_mode,
                  0 if model == "RESCAL" else nnh, cfg.chunk, precision)


def _reduce_all_slots(slots, ids, n_ent, name, tol):
    """kge_inspect + kge_segment_reduce over every slot row of the batch against a float64 index_add of the same rows."""
    from cuke_b200 import scoring
    insp = scoring.inspect(ids, n_ent)
    rows = scoring.segment_reduce(slots, insp)
    U = insp.count()
    uniq, inverse = torch.unique(ids, return_inverse=True)
    assert U == uniq.numel() and torch.equal(insp.uniq[:U], uniq) and torch.equal(insp.inverse.long(), inverse)
    ref = torch.zeros((U, slots.shape[1]), dtype=torch.float64, device=slots.device)
    ref.index_add_(0, inverse, slots.double())
    _check(name, rows[:U], ref.cpu().numpy(), tol)
    return insp, rows


def _softplus(x):
    return np.maximum(x, 0.0) + np.log1p(np.exp(-np.abs(x)))


def _sigmoid(x):
    return 1.0 / (1.0 + np.exp(-x))


# ---- c1: TransE forward, every score ---------------------------------------------------------------------------------
def test_c1_transe_forward_full_size():
    cfg = synth.CONFIGS["c1"]
    tabs = _tables(cfg, "TransE")
    h, r, t, neg = synth.make_batch(cfg)
    sc = _scorer(cfg, "TransE", tabs, "fp32")
    pos, negs, _ = sc.forward(*(to_dev(x) for x in (h, r, t, neg)))
    rpos, rneg = oracle.scores("TransE", tabs[0], tabs[1], None, h, r, t, neg, "per_triple", 0)
    _check("c1.pos", pos, rpos, FP32_TOL)
    _check("c1.neg", negs, rneg, FP32_TOL)
    # what the reference itself returns for this batch: the (B, dim) vectors of the flattened triples
    # (apps/kge/data/data_init.py:55-61), through the drop-in forward
    fh, fr, ft = oracle.flatten(h, r, t, neg, "per_triple", 0)
    vec = sc.ref_forward(to_dev(fh), to_dev(fr), to_dev(ft))
    _check("c1.ref_vectors", vec, oracle.ref_forward("TransE", tabs[0], tabs[1], None, fh, fr, ft), FP32_TOL)


# ---- c2: TransH forward + backward, every score, sampled slot gradients, full reduction -------------------------------
def test_c2_transh_full_size():
    from cuke_b200 import scoring
    cfg = synth.CONFIGS["c2"]
    E, R, W = _tables(cfg, "TransH")
    h, r, t, neg = synth.make_batch(cfg)
    B, nn, nnh = cfg.batch, cfg.n_neg, cfg.n_neg_head
    sc = _scorer(cfg, "TransH", (E, R, W), "fp32")
    dh, dr, dt, dn = (to_dev(x) for x in (h, r, t, neg))
    pos, negs, _ = sc.forward(dh, dr, dt, dn)
    step = B // 8
    parts = par_map(lambda k: oracle.scores("TransH", E, R, W, h[k:k + step], r[k:k + step], t[k:k + step], neg[k:k + step],
                                            "per_triple", nnh), range(0, B, step))
    _check("c2.pos", pos, np.concatenate([p[0] for p in parts]), FP32_TOL)
    _check("c2.neg", negs, np.concatenate([p[1] for p in parts]), FP32_TOL)

    loss, dpos, dneg = scoring.logistic_loss(pos, negs)
    sg = sc.backward(dh, dr, dt, dn, pos, negs, dpos, dneg)
    idx = np.sort(np.random.default_rng(2).choice(B, 128, replace=False))
    E2, R2, W2, h2, r2, t2, neg2, ru = occurrence_problem(E, R, W, h[idx], r[idx], t[idx], neg[idx])
    oE, oR, oW = oracle.grads("TransH", E2, R2, W2, h2, r2, t2, dpos[idx].cpu().numpy(), neg2, dneg[idx].cpu().numpy(), "per_triple", nnh)
    ti = torch.from_numpy(idx).cuda()
    nslots = (2 * B + ti[:, None] * nn + torch.arange(nn, device="cuda")[None, :]).reshape(-1)
    got = torch.cat([sg.ent_slots[ti], sg.ent_slots[B + ti], sg.ent_slots[nslots]])
    _check("c2.slot_grads", got, oE, FP32_TOL)
    for nm, rows, ref in (("c2.rel_grads", sg.rel_slots, oR), ("c2.normal_grads", sg.rel2_slots, oW)):
        acc = np.zeros_like(ref)
        np.add.at(acc, r2, rows[ti].double().cpu().numpy())
        _check(nm, acc, ref, FP32_TOL)
    _reduce_all_slots(sg.ent_slots, scoring.entity_id_list(dh, dt, dn), cfg.n_ent, "c2.reduced_entity_grads", 1e-5)


# ---- c3: TransR over bf16 tables, relation-grouped products on the tensor cores ----------------------------------------
def test_c3_transr_bf16_full_size():
    from cuke_b200 import scoring
    cfg = synth.CONFIGS["c3"]
    E, R, P = _tables(cfg, "TransR")
    h, r, t, neg = synth.make_batch(cfg)
    B, nn, nnh = cfg.batch, cfg.n_neg, cfg.n_neg_head
    sc = _scorer(cfg, "TransR", (E, R, P), "tensor")
    dh, dr, dt, dn = (to_dev(x) for x in (h, r, t, neg))
    pos, negs, rinsp = sc.forward(dh, dr, dt, dn)
    assert scoring.device_flags() == 0
    step = B // 8
    rpos = np.concatenate(par_map(lambda k: oracle.flat_scores("TransR", E, R, P, h[k:k + step], r[k:k + step], t[k:k + step]),
                                  range(0, B, step)))
    _check("c3.pos", pos, rpos, BF16_TOL)
    # sample: every triple of 16 seeded relations (their groups are whole, so the relation-matrix gradients are too)
    rels = np.sort(np.random.default_rng(3).choice(np.unique(r), 16, replace=False))
    idx = np.nonzero(np.isin(r, rels))[0]
    assert idx.size >= 32
    _, rneg = oracle.scores("TransR", E, R, P, h[idx], r[idx], t[idx], neg[idx], "per_triple", nnh)
    ti = torch.from_numpy(idx).cuda()
    _check("c3.neg_sample", negs[ti], rneg, BF16_TOL)

    loss, dpos, dneg = scoring.logistic_loss(pos, negs)
    sg = sc.backward(dh, dr, dt, dn, pos, negs, dpos, dneg, rinsp)
    assert scoring.device_flags() == 0
    E2, R2, P2, h2, r2, t2, neg2, ru = occurrence_problem(E, R, P, h[idx], r[idx], t[idx], neg[idx])
    assert np.array_equal(ru, rels)
    oE, oR, oP = oracle.grads("TransR", E2, R2, P2, h2, r2, t2, dpos[idx].cpu().numpy(), neg2, dneg[idx].cpu().numpy(), "per_triple", nnh)
    nslots = (2 * B + ti[:, None] * nn + torch.arange(nn, device="cuda")[None, :]).reshape(-1)
    got = torch.cat([sg.ent_slots[ti], sg.ent_slots[B + ti], sg.ent_slots[nslots]])
    _check("c3.slot_grads", got, oE, BF16_TOL)
    acc = np.zeros_like(oR)
    np.add.at(acc, r2, sg.rel_slots[ti].double().cpu().numpy())
    _check("c3.rel_grads", acc, oR, BF16_TOL)
    G = rinsp.count()
    groups = np.searchsorted(rinsp.uniq[:G].cpu().numpy(), rels)
    _check("c3.matrix_grads", sg.rel2_groups[torch.from_numpy(groups).cuda()], oP, BF16_TOL)
    _reduce_all_slots(sg.ent_slots, scoring.entity_id_list(dh, dt, dn), cfg.n_ent, "c3.reduced_entity_grads", 1e-5)


# ---- c4: RESCAL (dim 256) and ComplEx (2 x 256), chunk-shared negatives, fp32 and bf16 tables ---------------------------
def _chunk_sample_checks(tag, cfg, model, tabs, sc_by_prec, tol, n_score_chunks, n_grad_chunks, n_rel_sample):
    from cuke_b200 import scoring
    E, R, P = tabs
    h, r, t, neg = synth.make_batch(cfg)
    B, nn, chunk = cfg.batch, cfg.n_neg, cfg.chunk
    n_chunks = B // chunk
    dh, dr, dt, dn = (to_dev(x) for x in (h, r, t, neg))
    rng = np.random.default_rng(40 + len(model))
    chunks = np.sort(rng.choice(n_chunks, n_score_chunks, replace=False))
    step = B // 8
    rpos = np.concatenate(par_map(lambda k: oracle.flat_scores(model, E, R, P, h[k:k + step], r[k:k + step], t[k:k + step]),
                                  range(0, B, step)))

    def chunk_scores(c):
        s = slice(c * chunk, (c + 1) * chunk)
        return oracle.scores(model, E, R, P, h[s], r[s], t[s], neg[c:c + 1], "chunk_shared", 0, chunk)[1]
    rneg = np.stack(par_map(chunk_scores, chunks))                                  # (chunks, chunk, n_neg)

    for prec, sc in sc_by_prec.items():
        name = f"{tag}.{model}.{prec}"
        pos, negs, rinsp = sc.forward(dh, dr, dt, dn)
        assert scoring.device_flags() == 0
        _check(name + ".pos", pos, rpos, tol)
        _check(name + ".neg_chunks", negs[torch.from_numpy(chunks).cuda()], rneg, tol)
        loss, dpos, dneg = scoring.logistic_loss(pos, negs)
        sg = sc.backward(dh, dr, dt, dn, pos, negs, dpos, dneg, rinsp)
        assert scoring.device_flags() == 0
        dpos_np, dneg_np = dpos.cpu().numpy(), dneg.cpu().numpy()                  # dneg (n_chunks, chunk, n_neg)

        def chunk_grads(c):
            s = slice(c * chunk, (c + 1) * chunk)
            E2, R2, P2, h2, r2, t2, neg2, ru = occurrence_problem(E, R, P, h[s], r[s], t[s], neg[c:c + 1])
            oE, oR, _ = oracle.grads(model, E2, R2, P2, h2, r2, t2, dpos_np[s], neg2, dneg_np[c], "chunk_shared", 0, chunk)
            return oE, oR, r2
        for c, (oE, oR, r2) in zip(chunks[:n_grad_chunks], par_map(chunk_grads, chunks[:n_grad_chunks])):
            s = slice(c * chunk, (c + 1) * chunk)
            got = torch.cat([sg.ent_slots[s], sg.ent_slots[B + c * chunk: B + (c + 1) * chunk],
                             sg.ent_slots[2 * B + c * nn: 2 * B + (c + 1) * nn]])
            _check(f"{name}.slot_grads.chunk{c}", got, oE, tol)
            if oR is not None:
                acc = np.zeros_like(oR)
                np.add.at(acc, r2, sg.rel_slots[s].double().cpu().numpy())
                _check(f"{name}.rel_grads.chunk{c}", acc, oR, tol)
        if P is not None:
            # relation-matrix gradients: every triple of a few relations, each against its own chunk's negatives
            rels = np.sort(rng.choice(np.unique(r), n_rel_sample, replace=False))
            idx = np.nonzero(np.isin(r, rels))[0]
            negs_of = neg[idx // chunk]                                              # (n, n_neg)
            E2, R2, P2, h2, r2, t2, neg2, ru = occurrence_problem(E, R, P, h[idx], r[idx], t[idx], negs_of)
            dn_s = dneg_np[idx // chunk, idx % chunk]
            _, _, oP = oracle.grads(model, E2, R2, P2, h2, r2, t2, dpos_np[idx], neg2, dn_s, "per_triple", 0)
            G = rinsp.count()
            groups = np.searchsorted(rinsp.uniq[:G].cpu().numpy(), rels)
            _check(name + ".matrix_grads", sg.rel2_groups[torch.from_numpy(groups).cuda()], oP, tol)
        _reduce_all_slots(sg.ent_slots, scoring.entity_id_list(dh, dt, dn), cfg.n_ent, name + ".reduced_entity_grads", 1e-5)


@pytest.mark.parametrize("cname", ["c4", "c4_bf16"])
def test_c4_rescal_full_size(cname):
    cfg = synth.CONFIGS[cname]
    tabs = _tables(cfg, "RESCAL")
    tol = BF16_TOL if cfg.dtype == "bf16" else FP32_TOL
    scs = {"tensor": _scorer(cfg, "RESCAL", tabs, "tensor"), "fp32": _scorer(cfg, "RESCAL", tabs, "fp32")}
    _chunk_sample_checks(cname, cfg, "RESCAL", tabs, scs, tol, n_score_chunks=4, n_grad_chunks=1, n_rel_sample=2)


@pytest.mark.parametrize("cname", ["c4", "c4_bf16"])
def test_c4_complex_full_size(cname):
    cfg = synth.CONFIGS[cname]
    tabs = _tables(cfg, "ComplEx")
    tol = BF16_TOL if cfg.dtype == "bf16" else FP32_TOL
    scs = {"tensor": _scorer(cfg, "ComplEx", tabs, "tensor"), "fp32": _scorer(cfg, "ComplEx", tabs, "fp32")}
    _chunk_sample_checks(cname, cfg, "ComplEx", tabs, scs, tol, n_score_chunks=4, n_grad_chunks=4, n_rel_sample=0)


# ---- c5: TransE + DistMult through the step pipeline, tensor-core precision, fused forward + loss + backward -----------------
def _c5_setup(ent_scale, n_chunks):
    from cuke_b200.pipeline import KgeStep
    base = synth.CONFIGS["c5"]
    cfg = base.scaled(ent=ent_scale, batch=n_chunks * base.chunk / base.batch)
    assert cfg.dim == 400 and cfg.chunk == 1024 and cfg.n_neg == 1024 and cfg.batch == n_chunks * 1024
    models = ["TransE", "DistMult"]
    E = synth.make_tables(cfg, "TransE")[0]
    rel = {m: (np.random.default_rng(50 + i).standard_normal((cfg.n_rel, cfg.dim)) / np.sqrt(cfg.dim)).astype(np.float32)
           for i, m in enumerate(models)}
    stepper = KgeStep(models, to_dev(E), {m: to_dev(rel[m]) for m in models}, cfg.n_ent, cfg.neg_mode, 0, cfg.chunk,
                      precision="tensor")
    return cfg, models, E, rel, stepper


def test_c5_fused_step_four_chunks_against_oracle():
    """Four whole c5 chunks (1024 triples x 1024 shared negatives x dim 400 each) through KgeStep: loss, every entity
    gradient row and the relation gradients against the oracle."""
    from cuke_b200 import scoring
    cfg, models, E, rel, stepper = _c5_setup(0.01, 4)
    h, r, t, neg = synth.make_batch(cfg)
    out = stepper.step(*(to_dev(x) for x in (h, r, t, neg)))
    assert scoring.device_flags() == 0
    U = int(out.n_ent_rows.item())
    ids = out.ent_ids[:U].cpu().numpy()
    assert np.array_equal(ids, np.unique(np.concatenate([h, t, neg.reshape(-1)])))
    chunk, nn = cfg.chunk, cfg.n_neg
    for m in models:
        sc = scoring.Scorer(m, stepper.ent_local, stepper.rel[m], None, cfg.neg_mode, 0, chunk, "tensor")
        assert sc.supports_fused_step(nn), "the step must take the fused call for this scorer"

        def one(c):
            s = slice(c * chunk, (c + 1) * chunk)
            pos, negs = oracle.scores(m, E, rel[m], None, h[s], r[s], t[s], neg[c:c + 1], "chunk_shared", 0, chunk)
            p64, n64 = pos.astype(np.float64), negs.astype(np.float64)
            loss = _softplus(-p64).sum() + _softplus(n64).sum() / nn
            gE, gR, _ = oracle.grads(m, E, rel[m], None, h[s], r[s], t[s], (-_sigmoid(-p64)).astype(np.float32), neg[c:c + 1],
                                     (_sigmoid(n64) / nn).astype(np.float32), "chunk_shared", 0, chunk)
            return pos, loss, gE[ids], gR
        res = par_map(one, range(cfg.batch // chunk), workers=4)
        _check(f"c5.{m}.pos", out.pos[m], np.concatenate([x[0] for x in res]), FP32_TOL)
        ref_loss = sum(x[1] for x in res)
        lerr = abs(out.loss[m].item() - ref_loss) / abs(ref_loss)
        REPORT[f"c5.{m}.loss"] = {"rel_err": lerr, "tol": FP32_TOL}
        assert lerr < FP32_TOL
        _check(f"c5.{m}.entity_grads", out.ent_grad[m][:U], sum(x[2] for x in res), FP32_TOL)
        _check(f"c5.{m}.relation_grads", out.rel_grad[m], sum(x[3] for x in res), FP32_TOL)


def test_c5_full_batch_properties():
    """65,536 triples per step (64 chunks) at full dim / chunk / negative count: all positives and four whole chunks of
    negative scores against the oracle, and size-independent properties of the fused step's results."""
    from cuke_b200 import scoring
    cfg, models, E, rel, stepper = _c5_setup(0.05, 64)
    h, r, t, neg = synth.make_batch(cfg)
    dh, dr, dt, dn = (to_dev(x) for x in (h, r, t, neg))
    out = stepper.step(dh, dr, dt, dn)
    out2 = stepper.step(dh, dr, dt, dn)
    assert scoring.device_flags() == 0
    U = int(out.n_ent_rows.item())
    chunk, nn, B = cfg.chunk, cfg.n_neg, cfg.batch
    chunks = np.sort(np.random.default_rng(5).choice(B // chunk, 4, replace=False))
    step = B // 8
    for m in models:
        assert torch.equal(out.ent_grad[m][:U], out2.ent_grad[m][:U]) and torch.equal(out.loss[m], out2.loss[m])   # fixed order
        rpos = np.concatenate(par_map(lambda k: oracle.flat_scores(m, E, rel[m], None, h[k:k + step], r[k:k + step], t[k:k + step]),
                                      range(0, B, step)))
        _check(f"c5full.{m}.pos", out.pos[m], rpos, FP32_TOL)
        sc = scoring.Scorer(m, stepper.ent_local, stepper.rel[m], None, cfg.neg_mode, 0, chunk, "tensor")
        pos_u, negs_u, _ = sc.forward(dh, dr, dt, dn)
        rneg = np.stack(par_map(lambda c: oracle.scores(m, E, rel[m], None, h[c * chunk:(c + 1) * chunk], r[c * chunk:(c + 1) * chunk],
                                                        t[c * chunk:(c + 1) * chunk], neg[c:c + 1], "chunk_shared", 0, chunk)[1], chunks,
                                workers=4))
        _check(f"c5full.{m}.neg_chunks", negs_u[torch.from_numpy(chunks).cuda()], rneg, FP32_TOL)
        # the fused call and the three separate calls are the same function of the inputs
        loss_u, dpos, dneg = scoring.logistic_loss(pos_u, negs_u)
        assert abs(out.loss[m].item() - loss_u.item()) < FP32_TOL * abs(loss_u.item())
        sg = sc.backward(dh, dr, dt, dn, pos_u, negs_u, dpos, dneg)
        insp = scoring.inspect(scoring.entity_id_list(dh, dt, dn), cfg.n_ent)
        rows_u = scoring.segment_reduce(sg.ent_slots, insp)
        _check(f"c5full.{m}.fused_vs_separate_calls", out.ent_grad[m][:U], rows_u[:U].double().cpu().numpy(), FP32_TOL)
    # TransE: every gradient contribution enters one entity row with + and another with -, so the rows sum to zero
    ge = out.ent_grad["TransE"][:U].double()
    assert ge.sum(0).abs().max().item() < 1e-5 * ge.abs().sum(0).max().item()
