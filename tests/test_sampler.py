"""The device id sampler and the sparse optimizers: numpy models (CPU) and kernel-against-model parity (GPU)."""
import numpy as np
import pytest
import torch

from oracle import sampler_model as sm

# known-answer vectors of Philox4x32-10 (counter, key, output) as distributed with the Random123 library's kat_vectors
KATS = [((0, 0, 0, 0), (0, 0), (0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8)),
        ((0xffffffff,) * 4, (0xffffffff, 0xffffffff), (0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd)),
        ((0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344), (0xa4093822, 0x299f31d0), (0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1))]


def test_philox_model_known_answers():
    for c, k, exp in KATS:
        out = sm.philox4x32_10(*[np.array([x], dtype=np.uint64) for x in c], k[0], k[1])
        assert tuple(int(o[0]) for o in out) == exp


def test_mulhi_and_uniform_model():
    w = sm.words(1000, 0x1234567890ABCDEF, 5)
    for m in (1, 7, 1000, 4_000_000, (1 << 40) + 12345):
        assert [int(x) for x in sm.mulhi64(w, m)] == [(int(x) * m) >> 64 for x in w]
    ids = sm.sample_uniform(20000, 10, 9, 0)
    assert ids.min() == 0 and ids.max() == 9 and abs(np.bincount(ids, minlength=10) / 20000 - 0.1).max() < 0.01
    assert not np.array_equal(ids, sm.sample_uniform(20000, 10, 9, 1))         # another stream
    assert np.array_equal(ids[:100], sm.sample_uniform(100, 10, 9, 0))         # element i does not depend on n


def test_zipf_table_is_the_host_generators_table():
    from cuke_b200 import sampler, synth
    cdf, perm = sampler.zipf_table(5000, 1.1, perm_seed=4)
    synth.zipf_ids(np.random.default_rng(0), 5000, 10, perm_seed=4)
    cdf2, perm2 = synth._zipf_cache[(5000, 1.1, 4)]
    assert np.array_equal(cdf, cdf2) and np.array_equal(perm, perm2)
    ids = sm.sample_cdf(50000, cdf, perm, 3, 0)
    top = perm[0]
    share = (ids == top).mean()
    assert 0.8 * (cdf[0]) < share < 1.2 * cdf[0]                                # the hottest id carries cdf[0] of the draws


def test_load_triples_format(tmp_path):
    """entities.dict / relations.dict / train.txt as the reference's preprocessing reads them
    (apps/kge/data/preprocess.py:26-98): "<id>\\t<name>" lines and "<head>\\t<relation>\\t<tail>" name triples."""
    from cuke_b200 import sampler
    (tmp_path / "entities.dict").write_text("0\tparis\n1\tfrance\n2\tberlin\n3\tgermany\n")
    (tmp_path / "relations.dict").write_text("0\tcapital_of\n1\tborders\n")
    (tmp_path / "train.txt").write_text("paris\tcapital_of\tfrance\nberlin\tcapital_of\tgermany\nfrance\tborders\tgermany\n\n")
    triples, ne, nr = sampler.load_triples(str(tmp_path))
    assert (ne, nr) == (4, 2)
    assert triples.tolist() == [[0, 0, 1], [2, 0, 3], [1, 1, 3]]


# ---- GPU --------------------------------------------------------------------------------------------------------------
@pytest.mark.gpu
@pytest.mark.parametrize("idt", [torch.int64, torch.int32])
def test_device_sampler_bit_exact(idt):
    from cuke_b200 import sampler
    s = sampler.DeviceSampler(n_ent=100003, n_rel=517, batch=512, n_neg=96, neg_mode="chunk_shared", chunk=128, ent_dist="zipf",
                              seed=0xC0FFEE1234, rank=3, id_dtype=idt, perm_seed=2)
    cdf, perm = sampler.zipf_table(100003, 1.1, 2)
    for step in (0, 1, 70000):
        ids, h, r, t, neg = s.draw(step)
        sid = lambda k: s.stream_id(step, k)
        assert np.array_equal(h.cpu().numpy(), sm.sample_cdf(512, cdf, perm, s.seed, sid(0)))
        assert np.array_equal(t.cpu().numpy(), sm.sample_cdf(512, cdf, perm, s.seed, sid(1)))
        assert np.array_equal(r.cpu().numpy(), sm.sample_uniform(512, 517, s.seed, sid(2)))
        assert np.array_equal(neg.cpu().numpy().reshape(-1), sm.sample_cdf(4 * 96, cdf, perm, s.seed, sid(3)))
        assert ids.data_ptr() == h.data_ptr() and neg.shape == (4, 96)
    u = sampler.DeviceSampler(n_ent=(1 << 31) - 5 if idt == torch.int32 else (1 << 40) + 7, n_rel=3, batch=300, n_neg=7,
                              neg_mode="per_triple", seed=11, id_dtype=idt)
    ids, h, r, t, neg = u.draw(2)
    assert np.array_equal(h.cpu().numpy(), sm.sample_uniform(300, u.n_ent, 11, u.stream_id(2, 0)))
    assert np.array_equal(neg.cpu().numpy().reshape(-1), sm.sample_uniform(2100, u.n_ent, 11, u.stream_id(2, 3)))


@pytest.mark.gpu
def test_device_sampler_draws_stored_triples():
    from cuke_b200 import sampler
    g = np.random.default_rng(1)
    triples = np.stack([g.integers(0, 900, 5000), g.integers(0, 12, 5000), g.integers(0, 900, 5000)], 1).astype(np.int64)
    s = sampler.DeviceSampler(900, 12, 256, 16, "per_triple", seed=5, triples=torch.from_numpy(triples))
    ids, h, r, t, neg = s.draw(4)
    mh, mr, mt = sm.sample_triples(256, triples, 5, s.stream_id(4, 1))
    assert np.array_equal(h.cpu().numpy(), mh) and np.array_equal(r.cpu().numpy(), mr) and np.array_equal(t.cpu().numpy(), mt)


@pytest.mark.gpu
def test_sampled_batch_feeds_the_step():
    """ids drawn on the device go straight into the step (no host copy): same results as the same ids passed in."""
    from cuke_b200 import sampler
    from cuke_b200.pipeline import KgeStep
    g = np.random.default_rng(2)
    ne, nr, d, chunk = 4000, 9, 64, 128
    E = torch.from_numpy((g.standard_normal((ne, d)) / 8).astype(np.float32)).cuda()
    R = {"DistMult": torch.from_numpy((g.standard_normal((nr, d)) / 8).astype(np.float32)).cuda()}
    s = sampler.DeviceSampler(ne, nr, 2 * chunk, 64, "chunk_shared", chunk, "zipf", seed=3)
    step = KgeStep(["DistMult"], E, R, ne, "chunk_shared", 0, chunk, precision="tensor")
    ids, h, r, t, neg = s.draw(0)
    a = step.step(h, r, t, neg, ids=ids)
    b = step.step(h.clone(), r.clone(), t.clone(), neg.clone())
    U = int(a.n_ent_rows.item())
    assert torch.equal(a.loss["DistMult"], b.loss["DistMult"]) and torch.equal(a.ent_grad["DistMult"][:U], b.ent_grad["DistMult"][:U])


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("kind", ["sgd", "adagrad"])
def test_sparse_optimizers_three_steps(kind, dtype):
    """Three consecutive updates of the touched rows against a float64 numpy update (bf16 tables: the model rounds the
    stored value to bf16 after every step, as the kernel does)."""
    from cuke_b200 import scoring
    g = np.random.default_rng(7)
    rows, d, first = 300, 40, 1000
    table = torch.from_numpy(g.standard_normal((rows, d)).astype(np.float32)).to(dtype).cuda()
    ref = table.float().double().cpu().numpy()
    state = torch.zeros((rows, d), dtype=torch.float32, device="cuda")
    ref_state = np.zeros((rows, d))
    lr, eps = 0.05, 1e-6
    for it in range(3):
        U = 60 + it
        ids = np.sort(g.choice(rows, U, replace=False)) + first
        grad = g.standard_normal((80, d)).astype(np.float32)                   # more rows than valid ids: n_dev bounds them
        d_ids = torch.zeros(80, dtype=torch.int64, device="cuda"); d_ids[:U] = torch.from_numpy(ids).cuda()
        n_dev = torch.tensor([U], dtype=torch.int64, device="cuda")
        if kind == "sgd":
            scoring.apply_sgd(table, torch.from_numpy(grad).cuda(), lr, d_ids, n_dev, first)
            ref[ids - first] -= lr * grad[:U].astype(np.float64)
        else:
            scoring.apply_adagrad(table, state, torch.from_numpy(grad).cuda(), lr, eps, d_ids, n_dev, first)
            ref_state[ids - first] += grad[:U].astype(np.float64) ** 2
            ref[ids - first] -= lr * grad[:U] / (np.sqrt(ref_state[ids - first]) + eps)
        if dtype == torch.bfloat16:
            ref = torch.from_numpy(ref).float().to(torch.bfloat16).double().numpy()
        got = table.float().double().cpu().numpy()
        tol = 1e-6 if dtype == torch.float32 else 2 ** -8
        assert np.abs(got - ref).max() <= tol * np.abs(ref).max()
    if kind == "adagrad":
        assert np.abs(state.cpu().numpy() - ref_state).max() <= 1e-6 * ref_state.max()
    dense = torch.from_numpy(g.standard_normal((rows, d)).astype(np.float32)).cuda()      # ids = None: row i
    before = table.float().clone()
    scoring.apply_sgd(table, dense, 0.5)
    assert torch.allclose(table.float(), (before - 0.5 * dense).to(dtype).float(), atol=1e-6)
