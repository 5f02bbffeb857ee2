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
