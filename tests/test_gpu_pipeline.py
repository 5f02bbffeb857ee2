"""GPU tests of the whole step (inspector -> staging -> forward -> loss -> backward -> segmented reduction), of the
drop-in compile_and_run surface, and (with >= 2 GPUs) of the row-partitioned multi-GPU step."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from oracle import oracle
from tests.kge_testlib import FP32_TOL, make_problem, rel_err, to_dev

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def softplus(x):
    return np.maximum(x, 0) + np.log1p(np.exp(-np.abs(x)))


def sigmoid(x):
    return 1.0 / (1.0 + np.exp(-x))


@pytest.mark.parametrize("models,precision,chunk,nn", [(["TransE", "DistMult"], "tensor", 256, 160), (["ComplEx"], "tensor", 64, 96),
                                                       (["TransE", "DistMult"], "fp32", 64, 96)])
def test_step_matches_oracle(models, precision, chunk, nn):
    from cuke_b200.pipeline import KgeStep
    ne, d, B, nr = 3000, 64, 2 * chunk if chunk > 64 else 256, 17
    p = make_problem(models[0], seed=41, ne=ne, nr=nr, d=d, B=B, nn=nn, neg_mode="chunk_shared", chunk=chunk, zipf=True)
    g = p["g"]
    rel = {m: (g.standard_normal((nr, d)) / np.sqrt(d)).astype(np.float32) for m in models}
    step = KgeStep(models, to_dev(p["E"]), {m: to_dev(rel[m]) for m in models}, ne, "chunk_shared", 0, chunk, precision=precision)
    h, r, t, neg = (to_dev(p[k]) for k in ("h", "r", "t", "neg"))
    out = step.step(h, r, t, neg)
    out2 = step.step(h, r, t, neg)
    U = int(out.n_ent_rows.item())
    ids = out.ent_ids[:U].cpu().numpy()
    assert np.array_equal(ids, np.unique(np.concatenate([p["h"], p["t"], p["neg"].reshape(-1)])))
    for m in models:
        pos, negs = oracle.scores(m, p["E"], rel[m], None, p["h"], p["r"], p["t"], p["neg"], "chunk_shared", 0, chunk)
        w = 1.0 / nn
        loss = softplus(-pos.astype(np.float64)).sum() + w * softplus(negs.astype(np.float64)).sum()
        assert abs(out.loss[m].item() - loss) / abs(loss) < FP32_TOL
        dpos = (-sigmoid(-pos.astype(np.float64))).astype(np.float32)
        dneg = (w * sigmoid(negs.astype(np.float64))).astype(np.float32)
        gE, gR, _ = oracle.grads(m, p["E"], rel[m], None, p["h"], p["r"], p["t"], dpos, p["neg"], dneg, "chunk_shared", 0, chunk)
        dense = np.zeros_like(gE)
        dense[ids] = out.ent_grad[m][:U].double().cpu().numpy()
        assert rel_err(dense, gE) < FP32_TOL
        assert rel_err(out.rel_grad[m].double().cpu().numpy(), gR) < FP32_TOL
        assert torch.equal(out.ent_grad[m][:U], out2.ent_grad[m][:U])       # bit-reproducible step


@pytest.mark.parametrize("model,neg_mode,bf16,precision", [("TransH", "per_triple", False, "fp32"), ("TransF", "per_triple", False, "fp32"),
                                                           ("TransR", "per_triple", False, "fp32"), ("TransR", "per_triple", True, "tensor"),
                                                           ("RESCAL", "chunk_shared", False, "tensor"), ("RESCAL", "per_triple", False, "fp32")])
def test_step_covers_every_scorer(model, neg_mode, bf16, precision):
    """The step pipeline with relation-side tables of every kind: normals (TransH), matrices (TransR, RESCAL)."""
    from cuke_b200.pipeline import KgeStep
    from tests.kge_testlib import BF16_TOL, bf16_round
    ne, d, nr, nn = 1500, 64, 9, 24
    chunk = 64 if neg_mode == "chunk_shared" else 0
    B = 192
    p = make_problem(model, seed=17, ne=ne, nr=nr, d=d, B=B, nn=nn, neg_mode=neg_mode, chunk=chunk, zipf=True)
    E, R, P2 = (bf16_round(p[k]) for k in ("E", "R", "P2")) if bf16 else (p["E"], p["R"], p["P2"])
    nnh = 0 if model == "RESCAL" else nn // 2
    if neg_mode == "chunk_shared":
        nnh = 0
    rel = {} if R is None else {model: to_dev(R, bf16=bf16)}
    rel2 = {} if P2 is None else {model: to_dev(P2, bf16=bf16)}
    step = KgeStep([model], to_dev(E, bf16=bf16), rel, ne, neg_mode, nnh, chunk, precision=precision, rel2=rel2)
    out = step.step(*(to_dev(p[k]) for k in ("h", "r", "t", "neg")))
    tol = BF16_TOL if bf16 else FP32_TOL
    pos, negs = oracle.scores(model, E, R, P2, p["h"], p["r"], p["t"], p["neg"], neg_mode, nnh, chunk)
    n_per = negs.shape[1]
    loss = softplus(-pos.astype(np.float64)).sum() + softplus(negs.astype(np.float64)).sum() / n_per
    assert abs(out.loss[model].item() - loss) / abs(loss) < tol
    dpos = (-sigmoid(-pos.astype(np.float64))).astype(np.float32)
    dneg = (sigmoid(negs.astype(np.float64)) / n_per).astype(np.float32)
    gE, gR, gP = oracle.grads(model, E, R, P2, p["h"], p["r"], p["t"], dpos, p["neg"], dneg, neg_mode, nnh, chunk)
    U = int(out.n_ent_rows.item())
    dense = np.zeros_like(gE)
    dense[out.ent_ids[:U].cpu().numpy()] = out.ent_grad[model][:U].double().cpu().numpy()
    assert rel_err(dense, gE) < tol
    if gR is not None:
        assert rel_err(out.rel_grad[model].double().cpu().numpy(), gR) < tol
    if model == "TransH":
        assert rel_err(out.rel2_grad[model].double().cpu().numpy(), gP) < tol
    if model in ("TransR", "RESCAL"):
        G = int(out.n_rel2_groups.item())
        dP = np.zeros_like(gP)
        dP[out.rel2_ids[:G].cpu().numpy()] = out.rel2_grad[model][:G].double().cpu().numpy()
        assert rel_err(dP, gP) < tol


# Adagrad divides by sqrt(sum g^2) + eps: with a tiny eps the first update of an element is +-lr whatever the size of its
# gradient, which turns rounding noise in near-zero gradient entries into full-size steps; eps at the scale of the
# gradients keeps the comparison about the optimizer, not about the sign of noise
@pytest.mark.parametrize("opt", [("sgd", 0.5), ("adagrad", 0.1, 1e-3)])
@pytest.mark.parametrize("models,neg_mode,precision", [(["TransE", "DistMult"], "chunk_shared", "tensor"), (["RESCAL"], "chunk_shared", "fp32"),
                                                       (["TransH"], "per_triple", "fp32")])
def test_three_training_steps_match_float64_updates(opt, models, neg_mode, precision):
    """KgeStep with a sparse optimizer: three consecutive steps (inspector -> ... -> update of the touched rows) against
    float64 numpy updates driven by the oracle's gradients of the same tables."""
    from cuke_b200.pipeline import KgeStep
    ne, d, nr, nn, B = 800, 64, 7, 32, 128
    chunk = 64 if neg_mode == "chunk_shared" else 0
    p0 = make_problem(models[0], seed=23, ne=ne, nr=nr, d=d, B=B, nn=nn, neg_mode=neg_mode, chunk=chunk, zipf=True)
    g = p0["g"]
    T = {"E": p0["E"].astype(np.float64)}
    rel, rel2 = {}, {}
    for m in models:
        pm = make_problem(m, seed=29 + len(m), ne=8, nr=nr, d=d, B=8, nn=2)
        if pm["R"] is not None:
            T[("R", m)] = pm["R"].astype(np.float64); rel[m] = to_dev(pm["R"])
        if pm["P2"] is not None:
            T[("P", m)] = pm["P2"].astype(np.float64); rel2[m] = to_dev(pm["P2"])
    S = {k: np.zeros_like(v) for k, v in T.items()}
    step = KgeStep(models, to_dev(p0["E"]), rel, ne, neg_mode, 0, chunk, precision=precision, rel2=rel2, optimizer=opt)

    def upd(key, grad):
        if opt[0] == "sgd":
            T[key] -= opt[1] * grad
        else:
            S[key] += grad ** 2
            T[key] -= opt[1] * grad / (np.sqrt(S[key]) + opt[2])

    for it in range(3):
        pb = make_problem(models[0], seed=100 + it, ne=ne, nr=nr, d=d, B=B, nn=nn, neg_mode=neg_mode, chunk=chunk, zipf=True)
        h, r, t, neg = pb["h"], pb["r"], pb["t"], pb["neg"]
        step.step(to_dev(h), to_dev(r), to_dev(t), to_dev(neg))
        f32 = lambda k: None if k not in T else T[k].astype(np.float32)
        grads = []
        for m in models:                   # every scorer sees the tables as they were when the step began
            E, R, P2 = f32("E"), f32(("R", m)), f32(("P", m))
            pos, negs = oracle.scores(m, E, R, P2, h, r, t, neg, neg_mode, 0, chunk)
            dpos = (-sigmoid(-pos.astype(np.float64))).astype(np.float32)
            dneg = (sigmoid(negs.astype(np.float64)) / negs.shape[1]).astype(np.float32)
            grads.append((m, oracle.grads(m, E, R, P2, h, r, t, dpos, neg, dneg, neg_mode, 0, chunk)))
        for m, (gE, gR, gP) in grads:
            touched = np.unique(np.concatenate([h, t, neg.reshape(-1)]))
            mask = np.zeros((ne, 1)); mask[touched] = 1.0        # only touched rows move (Adagrad: untouched rows have g = 0 anyway)
            upd("E", gE * mask)
            if gR is not None:
                upd(("R", m), gR)
            if gP is not None:
                upd(("P", m), gP)
    assert rel_err(step.ent_local.double().cpu().numpy(), T["E"]) < FP32_TOL
    for m in models:
        if m in rel:
            assert rel_err(step.rel[m].double().cpu().numpy(), T[("R", m)]) < FP32_TOL
        if m in rel2:
            assert rel_err(step.rel2[m].double().cpu().numpy(), T[("P", m)]) < FP32_TOL


def test_prefetched_plan_gives_identical_steps():
    """step(..., prefetch=next_batch): the next batch's inspections run on a side stream; results are bit-identical."""
    from cuke_b200.pipeline import KgeStep
    ne, d, nr, nn, chunk, B = 3000, 64, 11, 96, 128, 256
    p = make_problem("TransE", seed=5, ne=ne, nr=nr, d=d, B=B, nn=nn, neg_mode="chunk_shared", chunk=chunk, zipf=True)
    rel = {m: to_dev((p["g"].standard_normal((nr, d)) / 8).astype(np.float32)) for m in ("TransE", "DistMult")}
    batches = []
    for it in range(3):
        pb = make_problem("TransE", seed=50 + it, ne=ne, nr=nr, d=d, B=B, nn=nn, neg_mode="chunk_shared", chunk=chunk, zipf=True)
        batches.append(tuple(to_dev(pb[k]) for k in ("h", "r", "t", "neg")))
    a = KgeStep(["TransE", "DistMult"], to_dev(p["E"]), rel, ne, "chunk_shared", 0, chunk, precision="tensor")
    plain = [a.step(*b) for b in batches]
    ahead = [a.step(*batches[i], prefetch=batches[i + 1] if i + 1 < 3 else None) for i in range(3)]
    for x, y in zip(plain, ahead):
        for m in ("TransE", "DistMult"):
            U = int(x.n_ent_rows.item())
            assert torch.equal(x.loss[m], y.loss[m]) and torch.equal(x.ent_grad[m][:U], y.ent_grad[m][:U])
            assert torch.equal(x.rel_grad[m], y.rel_grad[m])


@pytest.mark.parametrize("micro,precision", [(2, "tensor"), (3, "tensor"), (2, "fp32")])
def test_micro_batched_step_equals_whole_step(micro, precision):
    """A step cut into micro-batches (runs of whole chunks, each staged, scored and reduced on its own) gives the whole
    batch's loss, positives and gradients, and with SGD the same tables afterwards - prefetched plans included."""
    from cuke_b200.pipeline import KgeStep
    ne, d, nr, nn, chunk, n_chunks = 3000, 64, 11, 96, 64, 5
    B = chunk * n_chunks
    models = ["TransE", "DistMult"]
    p = make_problem("TransE", seed=8, ne=ne, nr=nr, d=d, B=B, nn=nn, neg_mode="chunk_shared", chunk=chunk, zipf=True)
    rel0 = {m: (p["g"].standard_normal((nr, d)) / 8).astype(np.float32) for m in models}
    batches = []
    for it in range(2):
        pb = make_problem("TransE", seed=70 + it, ne=ne, nr=nr, d=d, B=B, nn=nn, neg_mode="chunk_shared", chunk=chunk, zipf=True)
        batches.append(tuple(to_dev(pb[k]) for k in ("h", "r", "t", "neg")))

    def run(k, optimizer):
        E = to_dev(p["E"].copy())
        rel = {m: to_dev(rel0[m].copy()) for m in models}
        st = KgeStep(models, E, rel, ne, "chunk_shared", 0, chunk, precision=precision, optimizer=optimizer, micro=k)
        outs = [st.step(*batches[i], prefetch=batches[i + 1] if i + 1 < len(batches) else None) for i in range(len(batches))]
        torch.cuda.synchronize()
        return E, rel, outs

    _, _, whole = run(1, None)
    _, _, cut = run(micro, None)
    for x, y in zip(whole, cut):
        assert y.parts is not None and len(y.parts) == micro
        U = int(x.n_ent_rows.item())
        for m in models:
            assert abs(float(x.loss[m]) - float(y.loss[m])) <= 1e-5 * abs(float(x.loss[m]))
            assert rel_err(y.pos[m].cpu().numpy(), x.pos[m].cpu().numpy()) < 1e-6
            assert rel_err(y.rel_grad[m].cpu().numpy(), x.rel_grad[m].cpu().numpy()) < 1e-5
            ref = np.zeros((ne, d), dtype=np.float64)
            ref[x.ent_ids[:U].cpu().numpy()] = x.ent_grad[m][:U].double().cpu().numpy()
            got = np.zeros((ne, d), dtype=np.float64)
            for o in y.parts:
                u = int(o.n_ent_rows.item())
                got[o.ent_ids[:u].cpu().numpy()] += o.ent_grad[m][:u].double().cpu().numpy()
            assert rel_err(got, ref) < 1e-5
    Ea, ra, _ = run(1, ("sgd", 0.05))
    Eb, rb, _ = run(micro, ("sgd", 0.05))
    assert rel_err((Eb - to_dev(p["E"])).cpu().numpy(), (Ea - to_dev(p["E"])).cpu().numpy()) < 1e-4      # the updates themselves
    for m in models:
        assert rel_err((rb[m] - to_dev(rel0[m])).cpu().numpy(), (ra[m] - to_dev(rel0[m])).cpu().numpy()) < 1e-4


@pytest.mark.parametrize("model", ["TransE", "TransH", "TransR", "TransF", "RESCAL", "DistMult", "ComplEx"])
def test_compile_and_run_drop_in(model):
    """The reference's user code path: build the expression, print_cuda, compile_and_run(code, *args) with the
    reference's positional argument lists (apps/kge/test_cuke.py:54,104,153,198,244)."""
    from cuke_b200 import kge, run
    p = make_problem(model, seed=3, ne=200, nr=9, d=48, B=64, neg_mode="none")
    fn = {"TransE": kge.transE, "TransH": kge.transH, "TransR": kge.transR, "TransF": kge.transF, "RESCAL": kge.RESCAL,
          "DistMult": kge.distmult, "ComplEx": kge.complEx}[model]
    code = fn()
    order = np.argsort(p["r"], kind="stable")            # the reference sorts by relation first (test_cuke.py:93-96)
    hs, ts, rs = p["h"][order], p["t"][order], p["r"][order]
    E, R, P2 = to_dev(p["E"]), to_dev(p["R"]), to_dev(p["P2"])
    h, t, r = to_dev(hs), to_dev(ts), to_dev(rs)
    uniq, buf, cnt = kge.inspector(r, 9)
    B, d = 64, 48
    if model == "TransE":
        x = run.gpu.compile_and_run(code, B, d, 200, E, h, t, 9, R, r, uniq, buf, cnt)
    elif model == "TransH":
        x = run.gpu.compile_and_run(code, B, d, 200, E, h, t, 9, R, r, uniq, buf, cnt, P2)
    elif model == "TransR":
        x = run.gpu.compile_and_run(code, B, d, 0, E, h, t, 0, P2, r, uniq, buf, cnt, R)
    elif model in ("TransF", "DistMult"):
        x = run.gpu.compile_and_run(code, B, d, 200, E, h, 9, R, r, uniq, buf, cnt, t)
    elif model == "RESCAL":
        x = run.gpu.compile_and_run(code, B, d, 200, E, h, 9, P2, r, uniq, buf, cnt, t)
    else:
        Ere, Eim = E[:, 0::2].contiguous(), E[:, 1::2].contiguous()
        Rre, Rim = R[:, 0::2].contiguous(), R[:, 1::2].contiguous()
        x = run.gpu.compile_and_run(code, B, d // 2, 200, Ere, h, 9, Rre, r, uniq, buf, cnt, Eim, Rim, t)
    ref = oracle.ref_forward(model, p["E"], p["R"], p["P2"], hs, rs, ts)
    assert tuple(x.shape) == ref.shape
    assert rel_err(x.cpu().numpy(), ref) < FP32_TOL
    with pytest.raises(TypeError):
        run.gpu.compile_and_run(code, B, d)


def test_missing_library_fails_loudly(tmp_path):
    code = ("import sys; sys.path.insert(0, %r); import cuke_b200._lib as L; L.LIB_PATH = %r\n"
            "try:\n    L.lib()\nexcept RuntimeError as e:\n    print('LOUD', e)\n") % (ROOT, str(tmp_path / "nope.so"))
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True)
    assert "LOUD" in r.stdout and "no CPU or PyTorch fallback" in r.stdout


@pytest.mark.parametrize("world", [2])
def test_sharded_step_equals_single_gpu(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", "29711", os.path.join(ROOT, "tests", "mgpu_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "SHARDED_OK" in r.stdout
