"""GPU parity: every entry of the C ABI against the CPU oracle on identical seeded inputs (bit-exact for the
inspector's integer outputs, relative 1e-4 for fp32 scores/gradients, 2e-2 for bf16 tables)."""
import os

import numpy as np
import pytest
import torch

from oracle import oracle
from tests.kge_testlib import (BF16_TOL, FP32_TOL, MODELS, bf16_round, gpu_grads_dense, gpu_ids, gpu_scorer,
                               make_problem, rel_err, to_dev)

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
TENSOR_PRECISIONS = ["tensor", "tensor_tf32"]      # fp32 operands as two bf16 terms (default) or two tf32 terms
CHUNK_MODELS = ["TransE", "DistMult", "ComplEx", "RESCAL"]
BWD_MODELS = ["TransE", "TransH", "TransR", "TransF", "DistMult", "RESCAL", "ComplEx"]


# ---- reference-compatible forward against the reference's own golden outputs ------------------------------
@pytest.mark.parametrize("model", MODELS)
def test_ref_forward_golden(model):
    from cuke_b200.scoring import Scorer
    z = np.load(os.path.join(GOLDEN, f"ref_{model}.npz"))
    g = {k: z[k] for k in z.files}
    sc = Scorer(model, to_dev(g["E"]), to_dev(g.get("R")), to_dev(g.get("P2")))
    out = sc.ref_forward(to_dev(g["h"]), to_dev(g["r"]), to_dev(g["t"])).cpu().numpy()
    assert out.shape == g["ref_pos"].shape
    assert rel_err(out, g["ref_pos"]) < FP32_TOL
    fh, fr, ft = oracle.flatten(g["h"], g["r"], g["t"], g["neg"], "per_triple", int(g["n_neg_head"]))
    outn = sc.ref_forward(to_dev(fh), to_dev(fr), to_dev(ft)).cpu().numpy()
    assert rel_err(outn, g["ref_neg"]) < FP32_TOL


@pytest.mark.parametrize("model", MODELS)
@pytest.mark.parametrize("d,B", [(4, 1), (37, 20), (128, 33), (200, 64), (520, 16)])
@pytest.mark.parametrize("idt", [torch.int64, torch.int32])
def test_ref_forward_shapes(model, d, B, idt):
    if model == "ComplEx" and d % 2:
        d += 1
    if model in ("TransR", "RESCAL") and d > 256:
        d = 264
    p = make_problem(model, seed=d, d=d, B=B, neg_mode="none")
    sc = gpu_scorer(p)
    h, r, t, _ = gpu_ids(p, idt)
    out = sc.ref_forward(h, r, t).cpu().numpy()
    ref = oracle.ref_forward(model, p["E"], p["R"], p["P2"], p["h"], p["r"], p["t"])
    assert rel_err(out, ref) < FP32_TOL


# ---- scores ---------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("model", MODELS)
@pytest.mark.parametrize("d,B,nn,nnh", [(40, 64, 8, 0), (40, 64, 8, 8), (37, 20, 5, 2), (200, 48, 70, 35), (512, 8, 33, 1)])
def test_score_forward_per_triple(model, d, B, nn, nnh):
    if model == "ComplEx" and d % 2:
        d += 1
    if model == "RESCAL":
        nnh = 0
    if model in ("TransR", "RESCAL") and d > 256:
        d = 264
    p = make_problem(model, seed=d + nn, d=d, B=B, nn=nn)
    sc = gpu_scorer(p, nnh)
    h, r, t, neg = gpu_ids(p)
    pos, negs, _ = sc.forward(h, r, t, neg)
    rpos, rneg = oracle.scores(model, p["E"], p["R"], p["P2"], p["h"], p["r"], p["t"], p["neg"], "per_triple", nnh)
    assert rel_err(pos.cpu().numpy(), rpos) < FP32_TOL
    assert rel_err(negs.cpu().numpy(), rneg) < FP32_TOL
    pos2, negs2, _ = sc.forward(h, r, t, neg)      # same launch twice: bit-identical (no races)
    assert torch.equal(pos, pos2) and torch.equal(negs, negs2)


@pytest.mark.parametrize("model", CHUNK_MODELS)
@pytest.mark.parametrize("d,chunk,nchunks,nn,head", [(40, 16, 3, 24, 0), (128, 128, 2, 128, 0), (200, 130, 2, 150, 1),
                                                     (38, 7, 3, 9, 0), (400, 256, 1, 300, 0)])
def test_score_forward_chunk_shared(model, d, chunk, nchunks, nn, head):
    if model == "RESCAL":
        head = 0
        d = min(d, 200)
    p = make_problem(model, seed=d + chunk, d=d, B=chunk * nchunks, nn=nn, neg_mode="chunk_shared", chunk=chunk, zipf=True)
    nnh = nn if head else 0
    sc = gpu_scorer(p, nnh)
    h, r, t, neg = gpu_ids(p, torch.int32 if d == 40 else torch.int64)
    pos, negs, _ = sc.forward(h, r, t, neg)
    rpos, rneg = oracle.scores(model, p["E"], p["R"], p["P2"], p["h"], p["r"], p["t"], p["neg"], "chunk_shared", nnh, chunk)
    assert rel_err(pos.cpu().numpy(), rpos) < FP32_TOL
    assert rel_err(negs.reshape(len(rpos), -1).cpu().numpy(), rneg) < FP32_TOL


@pytest.mark.parametrize("model", ["TransE", "DistMult", "ComplEx", "RESCAL"])
@pytest.mark.parametrize("d,chunk,nchunks,nn,head", [(32, 128, 1, 128, 0), (64, 128, 2, 256, 0), (400, 256, 2, 384, 0),
                                                     (200, 130, 2, 150, 1), (36, 7, 3, 9, 0), (512, 1024, 1, 1024, 0),
                                                     (100, 384, 2, 200, 0), (64, 520, 1, 1000, 1)])
@pytest.mark.parametrize("prec", TENSOR_PRECISIONS)
def test_score_forward_tensor_cores(model, d, chunk, nchunks, nn, head, prec):
    """tcgen05 path of the chunk-shared dot-product scorers (fp32 operands split in two bf16 or two tf32 terms, three MMAs
    per product): same 1e-4 tolerance as the fp32 CUDA-core path."""
    from cuke_b200 import scoring
    if model == "RESCAL":
        head = 0
        d = min(d, 200)
    p = make_problem(model, seed=7 * d + chunk, d=d, B=chunk * nchunks, nn=nn, neg_mode="chunk_shared", chunk=chunk, zipf=True)
    nnh = nn if head else 0
    sc = gpu_scorer(p, nnh, precision=prec)
    h, r, t, neg = gpu_ids(p)
    pos, negs, _ = sc.forward(h, r, t, neg)
    assert scoring.device_flags() == 0, "a bounded wait inside the tensor-core kernel ran out"
    rpos, rneg = oracle.scores(model, p["E"], p["R"], p["P2"], p["h"], p["r"], p["t"], p["neg"], "chunk_shared", nnh, chunk)
    assert rel_err(pos.cpu().numpy(), rpos) < FP32_TOL
    err = rel_err(negs.reshape(len(rpos), -1).cpu().numpy(), rneg)
    assert err < FP32_TOL, err
    pos2, negs2, _ = sc.forward(h, r, t, neg)
    assert torch.equal(negs, negs2)


@pytest.mark.parametrize("prec", TENSOR_PRECISIONS)
@pytest.mark.parametrize("frac,overflow", [(0.004, False), (0.05, False), (0.5, True)])
def test_transe_tensor_cores_cancellation(frac, overflow, prec):
    """TransE on the tensor cores uses |a|^2+|x|^2-2a.x; negatives that (nearly) coincide with the anchor cancel there
    and must come out exact through the fix-up list - or, when the list overflows, through the exact kernel."""
    from cuke_b200 import scoring
    d, chunk, nchunks, nn = 128, 256, 2, 512
    p = make_problem("TransE", seed=5, ne=4000, d=d, B=chunk * nchunks, nn=nn, neg_mode="chunk_shared", chunk=chunk)
    g = p["g"]
    E, R = p["E"], p["R"]
    # plant rows equal (or within 1e-3 relative) to anchors h + r of triples of the same chunk
    n_plant = int(frac * nn)
    for c in range(nchunks):
        for k in range(n_plant):
            i = c * chunk + int(g.integers(0, chunk))
            anchor = E[p["h"][i]] + R[p["r"][i]]
            row = 3000 + (c * n_plant + k) % 1000
            E[row] = anchor * (1.0 + (1e-3 * g.standard_normal(d)).astype(np.float32) * (k % 2))
            p["neg"][c, k] = row
    if overflow:          # every negative row within 1e-3 of every anchor: all pairs cancel, the fix-up list overflows
        anchor0 = E[p["h"][0]] + R[p["r"][0]]
        E[3000:4000] = anchor0[None, :] * (1.0 + 1e-3 * g.standard_normal((1000, d))).astype(np.float32)
        p["h"][:] = p["h"][0]; p["r"][:] = p["r"][0]
        p["neg"][:] = g.integers(3000, 4000, p["neg"].shape)
    sc = gpu_scorer(p, 0, precision=prec)
    pos, negs, _ = sc.forward(*gpu_ids(p))
    assert scoring.device_flags() == 0
    rpos, rneg = oracle.scores("TransE", E, R, None, p["h"], p["r"], p["t"], p["neg"], "chunk_shared", 0, chunk)
    got = negs.reshape(len(rpos), -1).cpu().numpy()
    assert rel_err(got, rneg) < FP32_TOL
    small = np.abs(rneg) < (2.0 if overflow else 0.05) * np.abs(rneg).max()   # the cancelling entries, on their own scale
    assert small.any()
    assert np.abs(got[small] - rneg[small]).max() <= 1e-4 * max(np.abs(rneg[small]).max(), 1e-6) + 1e-6


@pytest.mark.parametrize("model", ["TransE", "DistMult", "ComplEx", "RESCAL"])
@pytest.mark.parametrize("d,chunk,nchunks,nn,head", [(32, 128, 1, 128, 0), (400, 256, 2, 384, 0), (200, 130, 2, 152, 1),
                                                     (36, 7, 4, 12, 0), (512, 512, 1, 1024, 0), (100, 384, 2, 200, 0),
                                                     (72, 520, 1, 1000, 1), (40, 260, 2, 129, 0), (36, 7, 3, 9, 0)])
@pytest.mark.parametrize("prec", TENSOR_PRECISIONS)
def test_backward_tensor_cores(model, d, chunk, nchunks, nn, head, prec):
    from cuke_b200 import scoring
    if model == "RESCAL":
        head = 0
        d = min(d, 200)
    p = make_problem(model, seed=11 * d + chunk, ne=600, d=d, B=chunk * nchunks, nn=nn, neg_mode="chunk_shared", chunk=chunk, zipf=True)
    _check_grads(p, nn if head else 0, chunk, precision=prec)
    assert scoring.device_flags() == 0


def _softplus(x):
    return np.maximum(x, 0.0) + np.log1p(np.exp(-np.abs(x)))


@pytest.mark.parametrize("model", ["TransE", "DistMult", "ComplEx"])
@pytest.mark.parametrize("d,chunk,nchunks,nn,head", [(32, 128, 1, 128, 0), (400, 256, 2, 384, 0), (200, 130, 2, 152, 1),
                                                     (36, 7, 4, 12, 0), (100, 384, 2, 200, 0), (72, 520, 1, 1000, 1),
                                                     (40, 260, 2, 129, 0), (36, 7, 3, 9, 0)])
@pytest.mark.parametrize("prec", TENSOR_PRECISIONS)
def test_fused_loss_backward(model, d, chunk, nchunks, nn, head, prec):
    """kge_score_loss_backward = forward -> logistic loss -> backward without the score matrix: the loss against the
    oracle's scores (float64 softplus), positives and gradient rows against the unfused calls, all at the fp32 tolerance."""
    from cuke_b200 import scoring
    p = make_problem(model, seed=13 * d + chunk, ne=600, d=d, B=chunk * nchunks, nn=nn, neg_mode="chunk_shared", chunk=chunk, zipf=True)
    nnh = nn if head else 0
    sc = gpu_scorer(p, nnh, precision=prec)
    assert sc.supports_fused_step(nn)
    h, r, t, neg = gpu_ids(p)
    pos, loss, sg = sc.loss_backward(h, r, t, neg)
    assert scoring.device_flags() == 0
    rpos, rneg = oracle.scores(model, p["E"], p["R"], p["P2"], p["h"], p["r"], p["t"], p["neg"], "chunk_shared", nnh, chunk)
    ref_loss = _softplus(-rpos.astype(np.float64)).sum() + _softplus(rneg.astype(np.float64)).sum() / nn
    assert rel_err(pos.cpu().numpy(), rpos) < FP32_TOL
    assert abs(float(loss.item()) - ref_loss) < FP32_TOL * abs(ref_loss)
    pos_u, negs_u, _ = sc.forward(h, r, t, neg)
    loss_u, dpos, dneg = scoring.logistic_loss(pos_u, negs_u)
    sg_u = sc.backward(h, r, t, neg, pos_u, negs_u, dpos, dneg)
    assert abs(float(loss.item()) - float(loss_u.item())) < FP32_TOL * abs(float(loss_u.item()))
    assert rel_err(sg.ent_slots.cpu().numpy(), sg_u.ent_slots.cpu().numpy()) < FP32_TOL
    assert rel_err(sg.rel_slots.cpu().numpy(), sg_u.rel_slots.cpu().numpy()) < FP32_TOL
    pos2, loss2, sg2 = sc.loss_backward(h, r, t, neg)      # fixed summation orders: bit-identical on a second call
    assert torch.equal(loss, loss2) and torch.equal(sg.ent_slots, sg2.ent_slots) and torch.equal(sg.rel_slots, sg2.rel_slots)


@pytest.mark.parametrize("prec", TENSOR_PRECISIONS)
def test_fused_loss_backward_cancellation(prec):
    """TransE negatives that (nearly) coincide with their anchor: the fused epilogue recomputes those distances from the
    rows themselves, so loss and gradients still match the unfused exact path."""
    from cuke_b200 import scoring
    d, chunk, nchunks, nn = 128, 256, 2, 512
    p = make_problem("TransE", seed=5, ne=4000, d=d, B=chunk * nchunks, nn=nn, neg_mode="chunk_shared", chunk=chunk)
    g = p["g"]
    E, R = p["E"], p["R"]
    for c in range(nchunks):
        for k in range(24):
            i = c * chunk + int(g.integers(0, chunk))
            anchor = E[p["h"][i]] + R[p["r"][i]]
            row = 3000 + c * 24 + k
            E[row] = anchor * (1.0 + (1e-3 * g.standard_normal(d)).astype(np.float32) * (k % 2))
            p["neg"][c, k] = row
    sc = gpu_scorer(p, 0, precision=prec)
    sc_exact = gpu_scorer(p, 0)                      # CUDA-core fp32 path
    h, r, t, neg = gpu_ids(p)
    pos, loss, sg = sc.loss_backward(h, r, t, neg)
    assert scoring.device_flags() == 0
    pos_u, negs_u, _ = sc_exact.forward(h, r, t, neg)
    loss_u, dpos, dneg = scoring.logistic_loss(pos_u, negs_u)
    sg_u = sc_exact.backward(h, r, t, neg, pos_u, negs_u, dpos, dneg)
    assert abs(float(loss.item()) - float(loss_u.item())) < FP32_TOL * abs(float(loss_u.item()))
    assert rel_err(sg.ent_slots.cpu().numpy(), sg_u.ent_slots.cpu().numpy()) < FP32_TOL
    assert rel_err(sg.rel_slots.cpu().numpy(), sg_u.rel_slots.cpu().numpy()) < FP32_TOL


@pytest.mark.parametrize("d,B,nn,nnh,nr", [(200, 64, 16, 8, 11), (64, 300, 5, 0, 3), (256, 40, 33, 33, 40), (200, 500, 0, 0, 1),
                                           (200, 1024, 128, 64, 50)])
def test_transr_tensor_cores_bf16(d, B, nn, nnh, nr):
    """TransR over bf16 tables on the tensor cores (relation-grouped tiles, bf16 MMA, fp32 accumulate): 2e-2 relative
    against the oracle run on the bf16-rounded tables."""
    from cuke_b200 import scoring
    p = make_problem("TransR", seed=d + B, nr=nr, d=d, B=B, nn=max(nn, 1), neg_mode="per_triple" if nn else "none")
    sc = gpu_scorer(p, nnh, bf16=True, precision="tensor")
    h, r, t, neg = gpu_ids(p)
    pos, negs, _ = sc.forward(h, r, t, neg if nn else None)
    assert scoring.device_flags() == 0
    rpos, rneg = oracle.scores("TransR", bf16_round(p["E"]), bf16_round(p["R"]), bf16_round(p["P2"]), p["h"], p["r"], p["t"],
                               p["neg"] if nn else None, "per_triple" if nn else "none", nnh)
    assert rel_err(pos.cpu().numpy(), rpos) < BF16_TOL
    if nn:
        assert rel_err(negs.cpu().numpy(), rneg) < BF16_TOL
    pos2, negs2, _ = sc.forward(h, r, t, neg if nn else None)
    assert torch.equal(pos, pos2)


@pytest.mark.parametrize("model", ["TransE", "TransH", "DistMult", "ComplEx", "RESCAL", "TransR"])
def test_score_forward_bf16(model):
    d = 200 if model != "ComplEx" else 256
    p = make_problem(model, seed=77, d=d, B=64, nn=16)
    nnh = 0 if model == "RESCAL" else 8
    sc = gpu_scorer(p, nnh, bf16=True)
    h, r, t, neg = gpu_ids(p)
    pos, negs, _ = sc.forward(h, r, t, neg)
    # oracle on the bf16-rounded tables: isolates kernel error from storage rounding
    rpos, rneg = oracle.scores(model, bf16_round(p["E"]), bf16_round(p["R"]), bf16_round(p["P2"]), p["h"], p["r"], p["t"],
                               p["neg"], "per_triple", nnh)
    assert rel_err(pos.cpu().numpy(), rpos) < BF16_TOL
    assert rel_err(negs.cpu().numpy(), rneg) < BF16_TOL


# ---- gradients -------------------------------------------------------------------------------------------------
def _check_grads(p, nnh, chunk, bf16=False, tol=FP32_TOL, precision="fp32"):
    model = p["model"]
    sc = gpu_scorer(p, nnh, bf16=bf16, precision=precision)
    h, r, t, neg = gpu_ids(p)
    g = p["g"]
    B = len(p["h"])
    dpos_np = g.standard_normal(B).astype(np.float32)
    if p["neg"] is None:
        dneg_np, dneg = None, None
    else:
        nshape = (B, p["neg"].shape[1])
        dneg_np = g.standard_normal(nshape).astype(np.float32)
        dneg = to_dev(dneg_np if p["neg_mode"] == "per_triple" else dneg_np.reshape(B // chunk, chunk, -1))
    pos, negs, gE, gR, gP = gpu_grads_dense(p, sc, h, r, t, neg, to_dev(dpos_np), dneg)
    E, R, P2 = (bf16_round(p[k]) for k in ("E", "R", "P2")) if bf16 else (p["E"], p["R"], p["P2"])
    oE, oR, oP = oracle.grads(model, E, R, P2, p["h"], p["r"], p["t"], dpos_np, p["neg"], dneg_np, p["neg_mode"], nnh, chunk)
    assert rel_err(gE, oE) < tol, "entity gradient"
    if oR is not None:
        assert rel_err(gR, oR) < tol, "relation gradient"
    if oP is not None:
        assert rel_err(gP, oP) < tol, "relation-2 gradient"


@pytest.mark.parametrize("model", BWD_MODELS)
@pytest.mark.parametrize("d,B,nn,nnh", [(40, 64, 8, 0), (40, 64, 8, 8), (36, 20, 5, 2), (200, 48, 40, 20), (264, 8, 9, 1)])
def test_backward_per_triple(model, d, B, nn, nnh):
    if model == "RESCAL":
        nnh = 0
    p = make_problem(model, seed=3 * d + nn, ne=90, d=d, B=B, nn=nn, zipf=True)
    _check_grads(p, nnh, 0)


@pytest.mark.parametrize("model", CHUNK_MODELS)
@pytest.mark.parametrize("d,chunk,nchunks,nn,head", [(40, 16, 3, 24, 0), (128, 128, 2, 128, 0), (200, 130, 2, 150, 1),
                                                     (36, 7, 4, 9, 0), (400, 64, 1, 300, 0)])
def test_backward_chunk_shared(model, d, chunk, nchunks, nn, head):
    if model == "RESCAL":
        head = 0
        d = min(d, 200)
    p = make_problem(model, seed=5 * d + chunk, ne=150, d=d, B=chunk * nchunks, nn=nn, neg_mode="chunk_shared", chunk=chunk, zipf=True)
    _check_grads(p, nn if head else 0, chunk)


@pytest.mark.parametrize("d,B,nn,nnh,nr", [(200, 64, 16, 8, 11), (64, 300, 5, 0, 3), (256, 40, 33, 33, 40), (200, 96, 0, 0, 2)])
def test_transr_backward_tensor_cores_bf16(d, B, nn, nnh, nr):
    """TransR gradients over bf16 tables on the tensor cores (three relation-grouped bf16 products): 2e-2 relative."""
    from cuke_b200 import scoring
    p = make_problem("TransR", seed=2 * d + B, ne=120, nr=nr, d=d, B=B, nn=max(nn, 1), neg_mode="per_triple" if nn else "none", zipf=True)
    if not nn:
        p["neg"] = None
    _check_grads(p, nnh, 0, bf16=True, tol=BF16_TOL, precision="tensor")
    assert scoring.device_flags() == 0


@pytest.mark.parametrize("model", ["TransE", "DistMult", "ComplEx"])
def test_backward_bf16_tables(model):
    p = make_problem(model, seed=9, ne=90, d=64, B=32, nn=8, zipf=True)
    _check_grads(p, 4, 0, bf16=True, tol=BF16_TOL)


# ---- inspector ------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("n,space", [(1, 1), (1, 7), (16, 3), (255, 256), (2048, 5), (2049, 70000), (5000, 300),
                                     (100000, 4000000), (300000, 1 << 25), (70001, 1 << 31)])
@pytest.mark.parametrize("idt", [torch.int64, torch.int32])
def test_inspect_bit_exact(n, space, idt):
    from cuke_b200 import scoring
    if idt == torch.int32 and space > (1 << 31) - 1:
        space = (1 << 31) - 1
    g = np.random.Generator(np.random.PCG64(n + space % 1000))
    ids = g.integers(0, space, n)
    if n > 1000:   # make heavy duplicates as Zipf ids do
        ids[: n // 3] = ids[0]
    insp = scoring.inspect(to_dev(ids, idt), space)
    uniq, inv, perm, seg = oracle.inspect(ids)
    U = insp.count()
    assert U == len(uniq)
    assert np.array_equal(insp.uniq[:U].cpu().numpy(), uniq)
    assert np.array_equal(insp.inverse[:n].cpu().numpy(), inv)
    assert np.array_equal(insp.perm[:n].cpu().numpy(), perm)
    assert np.array_equal(insp.seg.cpu().numpy(), seg)


def test_inspect_empty():
    from cuke_b200 import scoring
    insp = scoring.inspect(torch.empty(0, dtype=torch.int64, device="cuda"), 10)
    assert insp.count() == 0 and insp.seg.cpu().tolist() == [0]


@pytest.mark.parametrize("n,space,d", [(1, 1, 4), (40, 3, 8), (1000, 7, 40), (5000, 900, 200), (3000, 3000, 37), (4096, 2, 400)])
def test_segment_reduce(n, space, d):
    from cuke_b200 import scoring
    g = np.random.Generator(np.random.PCG64(n + d))
    w = np.arange(1, space + 1, dtype=np.float64) ** -1.1
    ids = g.choice(space, size=n, p=w / w.sum())
    rows = g.standard_normal((n, d)).astype(np.float32)
    insp = scoring.inspect(to_dev(ids), space)
    out = scoring.segment_reduce(to_dev(rows), insp).cpu().numpy()
    uniq, inv, _, _ = oracle.inspect(ids)
    ref = np.zeros((n, d), dtype=np.float64)
    np.add.at(ref, inv, rows.astype(np.float64))
    assert rel_err(out, ref) < 1e-5
    assert np.all(out[len(uniq):] == 0)
    out2 = scoring.segment_reduce(to_dev(rows), insp).cpu().numpy()
    assert np.array_equal(out, out2)          # fixed summation order


@pytest.mark.parametrize("dtype,d", [(torch.float32, 200), (torch.bfloat16, 200), (torch.float32, 37), (torch.bfloat16, 3)])
def test_gather_rows(dtype, d):
    from cuke_b200 import scoring
    g = np.random.Generator(np.random.PCG64(d))
    table = torch.from_numpy(g.standard_normal((500, d)).astype(np.float32)).cuda().to(dtype).contiguous()
    ids = torch.from_numpy(g.integers(100, 400, 77)).cuda()
    out = scoring.gather_rows(table[100:].clone(), ids, first_row=100)
    assert torch.equal(out, table[ids])
    n_dev = torch.tensor([10], dtype=torch.int64, device="cuda")
    out = torch.zeros((77, d), dtype=dtype, device="cuda")
    scoring.gather_rows(table, ids, n_dev=n_dev, out=out)
    assert torch.equal(out[:10], table[ids[:10]]) and torch.all(out[10:] == 0)


def test_owner_counts():
    from cuke_b200 import scoring
    g = np.random.Generator(np.random.PCG64(8))
    ids = g.integers(0, 1000, 600)
    insp = scoring.inspect(to_dev(ids), 1000)
    for world in (1, 2, 4, 8):
        rpr = (1000 + world - 1) // world
        counts = scoring.owner_counts(insp, rpr, world).cpu().numpy()
        ref = np.bincount(np.minimum(np.unique(ids) // rpr, world - 1), minlength=world)
        assert np.array_equal(counts, ref)


def test_legacy_inspector_matches_reference_semantics():
    from cuke_b200 import scoring
    g = np.random.Generator(np.random.PCG64(21))
    for rel_num in (3, 9, 40, 1350):
        rel = np.sort(g.integers(0, rel_num, 16 * 300))
        rel[:16] = np.arange(16) % rel_num if rel_num >= 16 else rel[:16]
        if rel_num >= 16:
            rel[:16] = np.arange(16)          # a chunk of 16 distinct ids
        uniq, buf, cnt = scoring.legacy_inspector(to_dev(rel), rel_num)
        ou, ob, oc = oracle.legacy_inspect(rel, rel_num)
        assert np.array_equal(uniq.cpu().numpy(), ou)
        assert np.array_equal(buf.cpu().numpy(), ob)
        assert np.array_equal(cnt.cpu().numpy(), oc)


def test_logistic_loss():
    from cuke_b200 import scoring
    g = np.random.Generator(np.random.PCG64(4))
    pos = torch.from_numpy(g.standard_normal(1000).astype(np.float32) * 3).cuda()
    neg = torch.from_numpy(g.standard_normal((1000, 7)).astype(np.float32) * 3).cuda()
    loss, dpos, dneg = scoring.logistic_loss(pos, neg)
    p64, n64 = pos.double().requires_grad_(True), neg.double().requires_grad_(True)
    ref = torch.nn.functional.softplus(-p64).sum() + torch.nn.functional.softplus(n64).sum() / 7
    ref.backward()
    assert abs(loss.item() - ref.item()) / abs(ref.item()) < 1e-5
    assert rel_err(dpos.cpu().numpy(), p64.grad.cpu().numpy()) < 1e-5
    assert rel_err(dneg.cpu().numpy(), n64.grad.cpu().numpy()) < 1e-5


# ---- staged scoring: scoring a compact buffer through the inverse map equals scoring the table ------------------
@pytest.mark.parametrize("model", ["TransE", "DistMult"])
def test_staged_equals_direct(model):
    from cuke_b200 import scoring
    p = make_problem(model, seed=31, ne=5000, d=400, B=256, nn=128, neg_mode="chunk_shared", chunk=128, zipf=True)
    sc = gpu_scorer(p, 0)
    h, r, t, neg = gpu_ids(p)
    pos, negs, _ = sc.forward(h, r, t, neg)
    ids = scoring.entity_id_list(h, t, neg)
    insp = scoring.inspect(ids, 5000)
    staged = scoring.gather_rows(sc.ent, insp.uniq, n_dev=insp.n_unique)
    B = h.numel()
    sh, st, sneg = insp.inverse[:B], insp.inverse[B:2 * B], insp.inverse[2 * B:].reshape(neg.shape)
    pos2, negs2, _ = sc.with_entities(staged).forward(sh.contiguous(), r.to(torch.int32), st.contiguous(), sneg.contiguous())
    assert torch.equal(pos, pos2) and torch.equal(negs, negs2)


# ---- error behaviour ------------------------------------------------------------------------------------------------
def test_argument_errors():
    from cuke_b200._lib import KgeError
    p = make_problem("TransH", d=40, B=32, nn=8, neg_mode="chunk_shared", chunk=16)
    sc = gpu_scorer(p, 0)
    h, r, t, neg = gpu_ids(p)
    with pytest.raises(KgeError) as e:
        sc.forward(h, r, t, neg)
    assert e.value.code == -3 and "per-triple" in str(e.value)
    p = make_problem("TransE", d=40, B=30, nn=8, neg_mode="chunk_shared", chunk=16)
    p["neg"] = p["neg"][:1]
    sc = gpu_scorer(p, 0)
    with pytest.raises((KgeError, ValueError)):
        sc.forward(*gpu_ids(p))


# ---- opt-in safety checks -----------------------------------------------------------------------------------------------
def test_validate_ids_reports_and_sanitises():
    from cuke_b200 import _lib, scoring
    assert scoring.device_flags() == 0
    ids = torch.tensor([0, 5, 9, 10, -1, 3, 1 << 40], dtype=torch.int64, device="cuda")
    out = torch.full_like(ids, 77)
    scoring.validate_ids(ids, 10, out)
    assert scoring.device_flags() == _lib.ERR_ID_RANGE
    assert out.tolist() == [0, 5, 9, 0, 0, 3, 0]
    assert scoring.device_flags() == 0                       # reading clears the word
    good = torch.arange(10, dtype=torch.int32, device="cuda")
    scoring.validate_ids(good, 10)
    assert scoring.device_flags() == 0


@pytest.mark.parametrize("model,neg_mode", [("TransE", "per_triple"), ("DistMult", "chunk_shared"), ("TransR", "per_triple")])
def test_checked_scoring_skips_ids_outside_the_tables(model, neg_mode):
    """KGE_FLAG_CHECK_IDS: a call whose ids leave the tables reports it and reads row 0 instead; the other triples are
    scored as usual, and a clean batch gives the unchecked result bit for bit."""
    from cuke_b200 import _lib, scoring
    from cuke_b200.scoring import Scorer
    chunk = 16 if neg_mode == "chunk_shared" else 0
    p = make_problem(model, seed=31, ne=200, nr=7, d=40, B=32, nn=8, neg_mode=neg_mode, chunk=chunk)
    E, R, P2 = to_dev(p["E"]), to_dev(p["R"]), to_dev(p["P2"])
    plain = Scorer(model, E, R, P2, neg_mode, 0, chunk)
    checked = Scorer(model, E, R, P2, neg_mode, 0, chunk, check_ids=True)
    h, r, t, neg = gpu_ids(p)
    pos0, neg0, _ = plain.forward(h, r, t, neg)
    pos1, neg1, _ = checked.forward(h, r, t, neg)
    assert scoring.device_flags() == 0
    assert torch.equal(pos0, pos1) and torch.equal(neg0, neg1)
    hb, rb, nb = h.clone(), r.clone(), neg.clone()
    hb[3] = 200                      # one past the entity table
    rb[5] = -2                       # (TransR too: the scorer builds its relation grouping from the checked ids)
    nb.view(-1)[11] = 1 << 33
    pos2, neg2, rinsp = checked.forward(hb, rb, t, nb)
    assert scoring.device_flags() == _lib.ERR_ID_RANGE
    keep = torch.ones(32, dtype=torch.bool, device="cuda")
    keep[3] = keep[5] = False
    assert torch.equal(pos2[keep], pos0[keep])
    # backward with the same bad ids: reported again, finite rows everywhere
    loss, dpos, dneg = scoring.logistic_loss(pos2, neg2)
    sg = checked.backward(hb, rb, t, nb, pos2, neg2, dpos, dneg, rinsp)
    assert scoring.device_flags() == _lib.ERR_ID_RANGE
    assert torch.isfinite(sg.ent_slots).all()


def test_bounded_wait_runs_out_harmlessly():
    """The waits inside the tensor-core kernels are bounded polls; when one runs out the kernel records it and leaves.
    The library's self-test kernel waits on a barrier nothing completes: it must return and report, and the context
    must stay usable."""
    from cuke_b200 import _lib, scoring
    assert scoring.device_flags() == 0
    scoring.selftest_wait_timeout(2048)
    assert scoring.device_flags() == _lib.ERR_WAIT_TIMEOUT
    assert scoring.device_flags() == 0
    x = torch.arange(8, device="cuda").sum().item()          # the context still works
    assert x == 28
    from cuke_b200._lib import KgeError
    with pytest.raises(KgeError):
        scoring.selftest_wait_timeout(0)


def test_backward_with_rows_that_are_not_quads():
    """dim % 4 != 0 takes the element-wise row path: gradient slices then only need 4-byte alignment (B * dim * 4 is
    not a multiple of 16 here)."""
    for model, mode in (("TransE", "per_triple"), ("DistMult", "none"), ("TransH", "per_triple")):
        p = make_problem(model, seed=8, ne=60, d=37, B=21, nn=3, neg_mode=mode, zipf=True)
        if mode == "none":
            p["neg"] = None
        _check_grads(p, 1 if mode == "per_triple" else 0, 0)


@pytest.mark.parametrize("d,B,nn,nnh,nr", [(200, 64, 16, 8, 11), (64, 300, 5, 0, 3), (256, 40, 33, 33, 40), (200, 1024, 128, 64, 50)])
def test_transr_fused_step_matches_separate_calls(d, B, nn, nnh, nr):
    """kge_score_loss_backward for TransR over bf16 tables packs the relation-grouped difference rows once; loss, positives
    and every gradient must equal forward -> logistic loss -> backward (same kernels on the same packed rows: bit for bit)."""
    from cuke_b200 import scoring
    p = make_problem("TransR", seed=3 * d + B, ne=150, nr=nr, d=d, B=B, nn=nn, zipf=True)
    sc = gpu_scorer(p, nnh, bf16=True, precision="tensor")
    assert sc.supports_fused_step(nn)
    h, r, t, neg = gpu_ids(p)
    pos, loss, sg = sc.loss_backward(h, r, t, neg)
    assert scoring.device_flags() == 0
    pos_u, negs_u, rinsp = sc.forward(h, r, t, neg)
    loss_u, dpos, dneg = scoring.logistic_loss(pos_u, negs_u)
    sg_u = sc.backward(h, r, t, neg, pos_u, negs_u, dpos, dneg, rinsp)
    assert torch.equal(pos, pos_u) and torch.equal(loss, loss_u)
    assert torch.equal(sg.ent_slots, sg_u.ent_slots) and torch.equal(sg.rel_slots, sg_u.rel_slots)
    G = rinsp.count()
    assert torch.equal(sg.rel2_groups[:G], sg_u.rel2_groups[:G])
