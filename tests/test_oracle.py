"""Pins the CPU oracle: against golden vectors produced by the reference's own generated C++
(tests/golden/make_golden.py), against the live reference-built modules when present, and (gradients)
against torch autograd in float64."""
import glob
import os

import numpy as np
import pytest
import torch

from oracle import oracle

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
MODELS = ["TransE", "TransH", "TransR", "TransF", "DistMult", "RESCAL", "ComplEx"]


def load_golden(model):
    z = np.load(os.path.join(GOLDEN, f"ref_{model}.npz"))
    return {k: z[k] for k in z.files}


@pytest.mark.parametrize("model", MODELS)
def test_oracle_matches_reference_golden(model):
    g = load_golden(model)
    R, P2 = g.get("R"), g.get("P2")
    out = oracle.ref_forward(model, g["E"], R, P2, g["h"], g["r"], g["t"])
    # same loops, same float arithmetic: the restatement must reproduce the reference bit for bit
    assert out.shape == g["ref_pos"].shape
    np.testing.assert_array_equal(out, g["ref_pos"])
    fh, fr, ft = oracle.flatten(g["h"], g["r"], g["t"], g["neg"], "per_triple", int(g["n_neg_head"]))
    outn = oracle.ref_forward(model, g["E"], R, P2, fh, fr, ft)
    np.testing.assert_array_equal(outn, g["ref_neg"])


@pytest.mark.parametrize("model", MODELS)
def test_oracle_matches_live_reference_build(model):
    if not oracle.have_ref(model):
        pytest.skip("oracle/_ref not built (needs the reference checkout)")
    g = np.random.Generator(np.random.PCG64(99))
    ne, nr, d, B = 37, 5, 16, 64
    E = g.standard_normal((ne, d)).astype(np.float32)
    R = None if model == "RESCAL" else g.standard_normal((nr, d)).astype(np.float32)
    P2 = None
    if model == "TransH":
        P2 = g.standard_normal((nr, d)).astype(np.float32)
    if model in ("TransR", "RESCAL"):
        P2 = g.standard_normal((nr, d, d)).astype(np.float32)
    h, t, r = g.integers(0, ne, B), g.integers(0, ne, B), g.integers(0, nr, B)
    tt = lambda a: None if a is None else torch.from_numpy(np.ascontiguousarray(a))
    ref = oracle.ref_run(model, tt(E), tt(R), tt(P2), tt(h), tt(r), tt(t)).numpy()
    np.testing.assert_array_equal(oracle.ref_forward(model, E, R, P2, h, r, t), ref)


def torch_scores(model, E, R, P2, h, r, t):
    """Independent float64 statement of the scores (formulas of apps/kge/test_pytorch.py:21,40,58,74,91)."""
    eh, et = E[h], E[t]
    if model == "TransE":
        return -(eh - et + R[r]).norm(dim=1)
    if model == "TransH":
        u = eh - et
        return -(u + R[r] - torch.einsum("a,ab->ab", torch.einsum("ab,ab->a", P2[r], u), P2[r])).norm(dim=1)
    if model == "TransR":
        return -(torch.einsum("ab,abc->ac", eh - et, P2[r]) + R[r]).norm(dim=1)
    if model == "TransF":
        return torch.einsum("ab,ab->a", eh + R[r], et) + torch.einsum("ab,ab->a", et - R[r], eh)
    if model == "DistMult":
        return (eh * R[r] * et).sum(1)
    if model == "RESCAL":
        return torch.einsum("ab,ab->a", torch.einsum("ab,abc->ac", eh, P2[r]), et)
    if model == "ComplEx":
        hc = torch.complex(eh[:, 0::2], eh[:, 1::2]); tc = torch.complex(et[:, 0::2], et[:, 1::2])
        rc = torch.complex(R[r][:, 0::2], R[r][:, 1::2])
        return (hc * rc * tc.conj()).sum(1).real
    raise KeyError(model)


def small_problem(model, seed=5, ne=29, nr=4, d=12, B=40, nn=5):
    g = np.random.Generator(np.random.PCG64(seed))
    E = (g.standard_normal((ne, d)) / np.sqrt(d)).astype(np.float32)
    R = None if model == "RESCAL" else (g.standard_normal((nr, d)) / np.sqrt(d)).astype(np.float32)
    P2 = None
    if model == "TransH":
        w = g.standard_normal((nr, d)); P2 = (w / np.linalg.norm(w, axis=1, keepdims=True)).astype(np.float32)
    if model in ("TransR", "RESCAL"):
        P2 = (g.standard_normal((nr, d, d)) / np.sqrt(d)).astype(np.float32)
    h, t, r = g.integers(0, ne, B), g.integers(0, ne, B), g.integers(0, nr, B)
    neg = g.integers(0, ne, (B, nn))
    return E, R, P2, h, r, t, neg, g


@pytest.mark.parametrize("model", MODELS)
def test_scores_match_torch_formulas(model):
    E, R, P2, h, r, t, neg, _ = small_problem(model)
    pos, ns = oracle.scores(model, E, R, P2, h, r, t, neg, "per_triple", 2)
    T = lambda a: None if a is None else torch.from_numpy(a).double()
    ref = torch_scores(model, T(E), T(R), T(P2), torch.from_numpy(h), torch.from_numpy(r), torch.from_numpy(t)).numpy()
    np.testing.assert_allclose(pos, ref, rtol=2e-5, atol=2e-6)
    fh, fr, ft = oracle.flatten(h, r, t, neg, "per_triple", 2)
    refn = torch_scores(model, T(E), T(R), T(P2), torch.from_numpy(fh), torch.from_numpy(fr), torch.from_numpy(ft)).numpy()
    np.testing.assert_allclose(ns.reshape(-1), refn, rtol=2e-5, atol=2e-6)


@pytest.mark.parametrize("model", MODELS)
@pytest.mark.parametrize("neg_mode", ["per_triple", "chunk_shared"])
def test_grads_match_autograd(model, neg_mode):
    E, R, P2, h, r, t, neg, g = small_problem(model)
    B = len(h)
    chunk, nnh = 0, 2
    if neg_mode == "chunk_shared":
        chunk, nnh = 8, 0
        neg = neg[: B // chunk]
    dpos = g.standard_normal(B).astype(np.float32)
    dneg = g.standard_normal((B, neg.shape[1])).astype(np.float32)
    gE, gR, gP = oracle.grads(model, E, R, P2, h, r, t, dpos, neg, dneg, neg_mode, nnh, chunk)
    T = lambda a: None if a is None else torch.from_numpy(a).double().requires_grad_(True)
    tE, tR, tP = T(E), T(R), T(P2)
    fh, fr, ft = oracle.flatten(h, r, t, neg, neg_mode, nnh, chunk)
    L = lambda a: torch.from_numpy(np.asarray(a))
    loss = (torch_scores(model, tE, tR, tP, L(h), L(r), L(t)) * torch.from_numpy(dpos).double()).sum() + \
           (torch_scores(model, tE, tR, tP, L(fh), L(fr), L(ft)) * torch.from_numpy(dneg).double().reshape(-1)).sum()
    loss.backward()
    np.testing.assert_allclose(gE, tE.grad.numpy(), rtol=1e-6, atol=1e-7)
    if R is not None:
        np.testing.assert_allclose(gR, tR.grad.numpy(), rtol=1e-6, atol=1e-7)
    if P2 is not None:
        np.testing.assert_allclose(gP, tP.grad.numpy(), rtol=1e-6, atol=1e-7)


def test_chunk_shared_flatten_layout():
    # negative j of triple i is row j of chunk i // chunk  (apps/examples/examples.py:1434-1441)
    h = np.arange(6); r = np.zeros(6, dtype=int); t = np.arange(6) + 10
    neg = np.array([[100, 101], [200, 201]])
    fh, fr, ft = oracle.flatten(h, r, t, neg, "chunk_shared", 0, 3)
    assert ft.reshape(6, 2).tolist() == [[100, 101]] * 3 + [[200, 201]] * 3
    assert fh.reshape(6, 2)[:, 0].tolist() == list(range(6))
    fh, fr, ft = oracle.flatten(h, r, t, neg, "chunk_shared", 2, 3)
    assert fh.reshape(6, 2).tolist() == [[100, 101]] * 3 + [[200, 201]] * 3
    assert ft.reshape(6, 2)[:, 1].tolist() == list(range(10, 16))


def test_inspect_model_properties():
    g = np.random.Generator(np.random.PCG64(3))
    for n, space in [(1, 5), (17, 3), (1000, 50), (513, 100000)]:
        ids = g.integers(0, space, n)
        uniq, inv, perm, seg = oracle.inspect(ids)
        U = len(uniq)
        assert np.all(np.diff(uniq) > 0)
        assert np.array_equal(uniq[inv], ids)
        assert np.array_equal(ids[perm], np.sort(ids, kind="stable"))
        assert seg[0] == 0 and np.all(seg[U:] == n)
        for u in range(U):
            assert np.all(ids[perm[seg[u]:seg[u + 1]]] == uniq[u])
            assert np.all(np.diff(perm[seg[u]:seg[u + 1]]) > 0)   # stable


def test_legacy_inspect_known_cases():
    rel_num = 50
    rel = np.array([3] * 16 + list(range(16)) + [7, 7, 7, 9, 9, 1, 2, 3, 4, 5, 6, 8, 10, 11, 12, 13])
    uniq, buf, cnt = oracle.legacy_inspect(rel, rel_num)
    assert uniq[0].tolist() == [3] + [rel_num] * 15 and cnt[0] == 1 and buf[0].tolist() == [0] * 16
    assert uniq[1].tolist() == [rel_num] * 16 and cnt[1] == 0 and buf[1].tolist() == [i + 16 for i in range(16)]
    assert uniq[2][:2].tolist() == [7, 9] and cnt[2] == 2
    assert buf[2].tolist() == [0, 0, 0, 1, 1] + [x + 16 for x in [1, 2, 3, 4, 5, 6, 8, 10, 11, 12, 13]]


def test_legacy_inspect_random_invariants():
    g = np.random.Generator(np.random.PCG64(11))
    rel_num = 9
    rel = np.sort(g.integers(0, rel_num, 16 * 200))
    uniq, buf, cnt = oracle.legacy_inspect(rel, rel_num)
    rel2 = rel.reshape(-1, 16)
    for b in range(rel2.shape[0]):
        c = int(cnt[b])
        assert np.all(uniq[b, c:] == rel_num) and np.all(uniq[b, :c] < rel_num)
        for i in range(16):
            if buf[b, i] < 16:
                assert uniq[b, buf[b, i]] == rel2[b, i]          # cached slot holds this id
            else:
                assert buf[b, i] == rel2[b, i] + 16
        if c:
            vals, counts = np.unique(rel2[b], return_counts=True)
            assert counts.max() == np.sum(rel2[b] == uniq[b, 0])   # slot 0 = the most frequent id


@pytest.mark.parametrize("model", ["TransE", "TransH", "TransR", "DistMult", "RESCAL", "ComplEx"])
def test_occurrence_problem_gives_per_slot_gradients(model):
    """kge_testlib.occurrence_problem: the oracle's dense gradient over one-row-per-occurrence tables, summed back by id,
    is the dense gradient of the original problem (this is what lets the config tests check a sample of a large batch)."""
    from tests.kge_testlib import make_problem, occurrence_problem
    p = make_problem(model, seed=21, ne=40, nr=5, d=12, B=24, nn=6, zipf=True)
    nnh = 0 if model == "RESCAL" else 3
    g = p["g"]
    dpos, dneg = g.standard_normal(24).astype(np.float32), g.standard_normal((24, 6)).astype(np.float32)
    gE, gR, gP = oracle.grads(model, p["E"], p["R"], p["P2"], p["h"], p["r"], p["t"], dpos, p["neg"], dneg, "per_triple", nnh)
    E2, R2, P2, h2, r2, t2, neg2, ru = occurrence_problem(p["E"], p["R"], p["P2"], p["h"], p["r"], p["t"], p["neg"])
    oE, oR, oP = oracle.grads(model, E2, R2, P2, h2, r2, t2, dpos, neg2, dneg, "per_triple", nnh)
    ids = np.concatenate([p["h"], p["t"], p["neg"].reshape(-1)])
    back = np.zeros_like(gE)
    np.add.at(back, ids, oE)
    np.testing.assert_allclose(back, gE, rtol=1e-9, atol=1e-12)
    if gR is not None:
        np.testing.assert_allclose(oR, gR[ru], rtol=1e-9, atol=1e-12)
    if gP is not None:
        np.testing.assert_allclose(oP, gP[ru], rtol=1e-9, atol=1e-12)
